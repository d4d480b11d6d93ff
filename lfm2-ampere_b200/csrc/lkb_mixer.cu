// lkb_mixer.cu - the sequence-mixer kernels of a batch-1 decode step for sm_100a: the short gated
// convolution step, per-head RMSNorm + NEOX RoPE + KV-cache append, and split-K decode attention over an
// fp16 KV cache (GQA 32 query / 8 KV heads, head_dim 64).
//
// Attention is HBM-bound at long context (256 B of K and V per token and KV head; 2.7 GB per token at
// 131072 positions) and latency-bound at short context.  Design: grid (8 KV heads x up to 18 slices) = at
// most 144 CTAs, one per SM; a CTA's eight warps each stream 32-token groups of K and V through a private
// 3-stage cp.async ring (two groups in flight while one is consumed: 128 KB in flight per SM), run their
// own online softmax (no CTA-wide barrier per tile) and merge once at the end.  The four query heads that
// share a KV head are evaluated together, so K and V cross HBM once.  The definition of correct is the
// float64 evaluation (ref: tests/test_attn.cu:46-75); the reference's own kernel is not bit-reproducible
// across its versions either (ref: src/kernels.cu:1383-1392) and gates on that float64 form.
#include "lkb_attn.cuh"

#define AT_STAGES  3
typedef AtSmem<AT_STAGES> AtSmem3;
static_assert(sizeof(AtSmem3) <= 232448, "attention staging exceeds the 227 KB a CTA may hold");
static_assert(sizeof(((AtWarp<2> *) 0)->k) >= AT_GQA * AT_D * sizeof(float), "the merge reuses a warp's K staging");

// ref: src/kernels.cu:1303-1560 (k_attn_split: same arguments, same partial layout [head][slice][2 + 64])
__global__ void __launch_bounds__(AT_WARPS * 32, 2) k_attn_split(const float * __restrict__ q, const __half * __restrict__ kc,
                                                                 const __half * __restrict__ vc, const int * __restrict__ d_pos,
                                                                 float * __restrict__ part) {
    extern __shared__ __align__(16) unsigned char at_raw[];
    AtSmem3 & S = *reinterpret_cast<AtSmem3 *>(at_raw);
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int seq_len = *d_pos + 1;
    const int kvh = blockIdx.x, sp = blockIdx.y;
    const int nsl = at_slices(seq_len);
    const int chunk = at_chunk(seq_len, nsl);
    const int t0 = sp * chunk;
    const int t1 = min(t0 + chunk, seq_len);
    if (t0 >= t1) return;                                   // CTA-uniform: dead slices write nothing
    const int tid = threadIdx.x;
    if (tid < AT_D) {
        const float * qh = q + (size_t) kvh * AT_GQA * AT_D + tid;
        S.q[tid] = make_float4(qh[0], qh[AT_D], qh[2 * AT_D], qh[3 * AT_D]);
    }
    __syncthreads();
    at_slice<AT_STAGES>(S, kc, vc, kvh, sp, t0, t1, part);
}

// ref: src/kernels.cu:1562-1599 (k_attn_combine: same arguments)
__global__ void __launch_bounds__(AT_D) k_attn_combine(const float * __restrict__ part, const int * __restrict__ d_pos,
                                                       float * __restrict__ out, lkb_q8blk * __restrict__ yq8) {
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int head = blockIdx.x, d = threadIdx.x;
    const float o = at_combine(part, head, d, *d_pos + 1);
    if (out) out[head * AT_D + d] = o;
    if (yq8) lkb_quant_store(o, yq8 + 2 * head + (d >> 5), d & 31);
}

// Per-head RMSNorm (weights qn / kn over 64 dims), NEOX half-split rotation at position *d_pos, and the
// append of the rotated K and of V to the fp16 cache.  One warp per head.  ref: src/kernels.cu:871-915
__global__ void __launch_bounds__(256) k_qk_norm_rope(float * __restrict__ qf, float * __restrict__ kf, const float * __restrict__ vf,
                                                      const float * __restrict__ qn, const float * __restrict__ kn,
                                                      const int * __restrict__ d_pos, __half * __restrict__ kc, __half * __restrict__ vc,
                                                      float theta) {
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int head_all = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (head_all >= AT_HEADS + AT_KVH) return;
    const bool is_q = head_all < AT_HEADS;
    const int head = is_q ? head_all : head_all - AT_HEADS;
    float * dst = (is_q ? qf : kf) + (size_t) head * AT_D;
    const int ipos = *d_pos;
    float y0, y1;
    at_norm_rope(dst[lane], dst[lane + 32], is_q ? qn : kn, (float) ipos, theta, lane, y0, y1);
    dst[lane] = y0; dst[lane + 32] = y1;
    if (!is_q) {
        const size_t off = ((size_t) ipos * AT_KVH + head) * AT_D;
        kc[off + lane] = __float2half(y0); kc[off + lane + 32] = __float2half(y1);
        vc[off + lane] = __float2half(vf[(size_t) head * AT_D + lane]);
        vc[off + lane + 32] = __float2half(vf[(size_t) head * AT_D + lane + 32]);
    }
}

// Short gated convolution, one decode step: bx = B*X; conv = h0*w0 + h1*w1 + bx*w2; y = C*conv; the
// two-tap history shifts.  bcx = [B | C | X] (3n floats), conv_w[ch*3 + tap], hist[ch*2 + {0,1}].
// ref: src/kernels.cu:521-545
__global__ void __launch_bounds__(256) k_shortconv(const float * __restrict__ bcx, const float * __restrict__ conv_w,
                                                   float * __restrict__ hist, float * __restrict__ y,
                                                   lkb_q8blk * __restrict__ yq8, int n) {
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;    // n % 32 == 0: whole warps are live or dead together
    if (ch >= n) return;
    const float bx = __fmul_rn(bcx[ch], bcx[2 * n + ch]);
    const float2 h = *reinterpret_cast<const float2 *>(hist + 2 * ch);
    const float conv = fmaf(bx, conv_w[3 * ch + 2], fmaf(h.y, conv_w[3 * ch + 1], __fmul_rn(h.x, conv_w[3 * ch])));
    *reinterpret_cast<float2 *>(hist + 2 * ch) = make_float2(h.y, bx);
    const float v = __fmul_rn(bcx[n + ch], conv);
    if (y) y[ch] = v;
    if (yq8) lkb_quant_store(v, yq8 + (ch >> 5), threadIdx.x & 31);
}

static int g_mixer_ready = 0;
int lkb_mixer_init() {
    const cudaError_t e = cudaFuncSetAttribute(k_attn_split, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(AtSmem3));
    if (e != cudaSuccess) return -(int) e;
    g_mixer_ready = 1;
    return LKB_OK;
}

extern "C" {

int lkb_attn_split(const float * q, const void * kc, const void * vc, const int * d_pos, float * part, lkb_stream_t st) {
    if (!lkb_context().inited || !g_mixer_ready) return LKB_ERR_NOT_INIT;
    if (!q || !kc || !vc || !d_pos || !part) return LKB_ERR_NULL;
    return lkb_launch(k_attn_split, dim3(AT_KVH, LKB_ATTN_SPLIT), dim3(AT_WARPS * 32), sizeof(AtSmem3), (cudaStream_t) st,
                      q, (const __half *) kc, (const __half *) vc, d_pos, part);
}

int lkb_attn_combine(const float * part, const int * d_pos, float * out, lkb_block_q8_1 * yq8, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!part || !d_pos || (!out && !yq8)) return LKB_ERR_NULL;
    return lkb_launch(k_attn_combine, dim3(AT_HEADS), dim3(AT_D), 0, (cudaStream_t) st, part, d_pos, out, (lkb_q8blk *) yq8);
}

int lkb_qk_norm_rope(float * qf, float * kf, const float * vf, const float * qn, const float * kn, const int * d_pos,
                     void * kc, void * vc, float theta, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!qf || !kf || !vf || !qn || !kn || !d_pos || !kc || !vc) return LKB_ERR_NULL;
    if (!(theta > 1.0f)) return LKB_ERR_SHAPE;
    return lkb_launch(k_qk_norm_rope, dim3((AT_HEADS + AT_KVH + 7) / 8), dim3(256), 0, (cudaStream_t) st,
                      qf, kf, vf, qn, kn, d_pos, (__half *) kc, (__half *) vc, theta);
}

int lkb_shortconv(const float * bcx, int t, const float * conv_w, float * hist, float * y, lkb_block_q8_1 * yq8, int n,
                  lkb_stream_t st) {
    (void) t;                                               // kept for the reference's argument list; unused there too
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!bcx || !conv_w || !hist || (!y && !yq8)) return LKB_ERR_NULL;
    if (n <= 0 || n % 32) return LKB_ERR_SHAPE;
    return lkb_launch(k_shortconv, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t) st, bcx, conv_w, hist, y, (lkb_q8blk *) yq8, n);
}

}  // extern "C"
