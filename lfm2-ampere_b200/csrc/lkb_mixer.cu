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
#include "lkb_device.cuh"

#define AT_HEADS   32
#define AT_KVH     8
#define AT_GQA     4
#define AT_D       64
#define AT_WARPS   8
#define AT_G       32                       // tokens per warp group
#define AT_STAGES  3
#define AT_ROW     72                       // halfs per staged row: 64 + 8 padding (144 B: conflict-free 16-B reads)
#define AT_SCALE   0.125f                   // 1/sqrt(64), exact.  ref: src/kernels.cuh:24

__host__ __device__ __forceinline__ int at_slices(int seq_len) {
    int s = (seq_len + 255) / 256;
    if (s < 1) s = 1;
    if (s > LKB_ATTN_SPLIT) s = LKB_ATTN_SPLIT;
    return s;
}

struct AtWarp {
    __half k[AT_STAGES][AT_G][AT_ROW];
    __half v[AT_STAGES][AT_G][AT_ROW];
    float4 p[AT_G];
};
struct AtSmem {
    AtWarp w[AT_WARPS];
    float4 q[AT_D];                         // q[d] = the four heads' values of dim d
    float  m[AT_WARPS][AT_GQA], l[AT_WARPS][AT_GQA];
};
static_assert(sizeof(AtSmem) <= 232448, "attention staging exceeds the 227 KB a CTA may hold");
static_assert(sizeof(((AtWarp *) 0)->k) >= AT_GQA * AT_D * sizeof(float), "the merge reuses a warp's K staging");

__device__ __forceinline__ void at_cp16(void * dst, const void * src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"((unsigned) __cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}

// ref: src/kernels.cu:1303-1560 (k_attn_split: same arguments, same partial layout [head][slice][2 + 64])
__global__ void __launch_bounds__(AT_WARPS * 32, 2) k_attn_split(const float * __restrict__ q, const __half * __restrict__ kc,
                                                                 const __half * __restrict__ vc, const int * __restrict__ d_pos,
                                                                 float * __restrict__ part) {
    extern __shared__ __align__(16) unsigned char at_raw[];
    AtSmem & S = *reinterpret_cast<AtSmem *>(at_raw);
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int seq_len = *d_pos + 1;
    const int kvh = blockIdx.x, sp = blockIdx.y;
    const int nsl = at_slices(seq_len);
    const int chunk = (((seq_len + nsl - 1) / nsl) + AT_G - 1) / AT_G * AT_G;      // whole groups per slice
    const int t0 = sp * chunk;
    const int t1 = min(t0 + chunk, seq_len);
    if (t0 >= t1) return;                                   // CTA-uniform: dead slices write nothing
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < AT_D) {
        const float * qh = q + (size_t) kvh * AT_GQA * AT_D + tid;
        S.q[tid] = make_float4(qh[0], qh[AT_D], qh[2 * AT_D], qh[3 * AT_D]);
    }
    __syncthreads();

    AtWarp & W = S.w[warp];
    const int ngrp = (t1 - t0 + AT_G - 1) / AT_G;           // groups of this slice; warp w owns w, w+8, ...
    const int mine = (ngrp - warp + AT_WARPS - 1) / AT_WARPS;
    const size_t tstride = (size_t) AT_KVH * AT_D;          // halfs between consecutive tokens
    const __half * kbase = kc + (size_t) kvh * AT_D, * vbase = vc + (size_t) kvh * AT_D;
    auto issue = [&](int i) {                               // group i of this warp -> stage i % AT_STAGES
        if (i < mine) {
            const int st = i % AT_STAGES, g0 = t0 + (warp + i * AT_WARPS) * AT_G;
            const size_t off0 = (size_t) (g0 + (lane >> 3)) * tstride + (lane & 7) * 8;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const int j = r * 4 + (lane >> 3);
                const bool live = g0 + j < t1;
                // dead rows are zero-filled (size 0) from an address that is always inside the cache
                const size_t off = live ? off0 + (size_t) r * 4 * tstride : (size_t) t0 * tstride;
                at_cp16(&W.k[st][j][(lane & 7) * 8], kbase + off, live ? 16 : 0);
                at_cp16(&W.v[st][j][(lane & 7) * 8], vbase + off, live ? 16 : 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    issue(0);
    issue(1);
    float m[AT_GQA], l[AT_GQA], acc[AT_GQA][2];
#pragma unroll
    for (int h = 0; h < AT_GQA; ++h) { m[h] = -1e30f; l[h] = 0.0f; acc[h][0] = acc[h][1] = 0.0f; }
    for (int i = 0; i < mine; ++i) {
        issue(i + 2);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        __syncwarp();
        const int st = i % AT_STAGES, g0 = t0 + (warp + i * AT_WARPS) * AT_G;
        const bool live = g0 + lane < t1;
        // scores of token g0 + lane against the four heads.  q is re-read from shared memory in every
        // iteration (the opaque zero stops the compiler from hoisting 64 float4 into registers).
        int zero;
        asm volatile("mov.u32 %0, 0;" : "=r"(zero));
        const float4 * Q = S.q + zero;
        float s[AT_GQA] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 2
        for (int c = 0; c < 8; ++c) {
            const uint4 kw = *reinterpret_cast<const uint4 *>(&W.k[st][lane][c * 8]);
            const __half2 * k2 = reinterpret_cast<const __half2 *>(&kw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 kf = __half22float2(k2[e]);
                const float4 qa = Q[c * 8 + 2 * e], qb = Q[c * 8 + 2 * e + 1];
                s[0] = fmaf(qa.x, kf.x, s[0]); s[1] = fmaf(qa.y, kf.x, s[1]); s[2] = fmaf(qa.z, kf.x, s[2]); s[3] = fmaf(qa.w, kf.x, s[3]);
                s[0] = fmaf(qb.x, kf.y, s[0]); s[1] = fmaf(qb.y, kf.y, s[1]); s[2] = fmaf(qb.z, kf.y, s[2]); s[3] = fmaf(qb.w, kf.y, s[3]);
            }
        }
        float sc[AT_GQA], pr[AT_GQA];
#pragma unroll
        for (int h = 0; h < AT_GQA; ++h) {
            s[h] = live ? s[h] * AT_SCALE : -1e30f;
            float mx = s[h];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(LKB_FULL, mx, o));
            const float mn = fmaxf(m[h], mx);
            sc[h] = __expf(m[h] - mn);
            pr[h] = live ? __expf(s[h] - mn) : 0.0f;
            l[h] = fmaf(l[h], sc[h], lkb_warp_sum(pr[h]));
            m[h] = mn;
        }
        W.p[lane] = make_float4(pr[0], pr[1], pr[2], pr[3]);
        __syncwarp();
        // acc[h][dims 2*lane, 2*lane+1] = acc * sc + sum_j p[j][h] * V[j][dims]
#pragma unroll
        for (int h = 0; h < AT_GQA; ++h) { acc[h][0] *= sc[h]; acc[h][1] *= sc[h]; }
#pragma unroll 8
        for (int j = 0; j < AT_G; ++j) {
            const float2 vf = __half22float2(*reinterpret_cast<const __half2 *>(&W.v[st][j][2 * lane]));
            const float4 p = W.p[j];
            acc[0][0] = fmaf(p.x, vf.x, acc[0][0]); acc[0][1] = fmaf(p.x, vf.y, acc[0][1]);
            acc[1][0] = fmaf(p.y, vf.x, acc[1][0]); acc[1][1] = fmaf(p.y, vf.y, acc[1][1]);
            acc[2][0] = fmaf(p.z, vf.x, acc[2][0]); acc[2][1] = fmaf(p.z, vf.y, acc[2][1]);
            acc[3][0] = fmaf(p.w, vf.x, acc[3][0]); acc[3][1] = fmaf(p.w, vf.y, acc[3][1]);
        }
        __syncwarp();
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // merge the eight warps' (m, l, acc); a warp parks its accumulators in its own, now idle, K staging
    __syncwarp();
    float * wacc = reinterpret_cast<float *>(&W.k[0][0][0]);
#pragma unroll
    for (int h = 0; h < AT_GQA; ++h) {
        if (lane == 0) { S.m[warp][h] = m[h]; S.l[warp][h] = l[h]; }
        wacc[h * AT_D + 2 * lane] = acc[h][0]; wacc[h * AT_D + 2 * lane + 1] = acc[h][1];
    }
    __syncthreads();
    {
        const int h = tid >> 6, d = tid & 63;
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) M = fmaxf(M, S.m[w][h]);
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) {
            const float e = __expf(S.m[w][h] - M);
            L = fmaf(S.l[w][h], e, L);
            A = fmaf(reinterpret_cast<const float *>(&S.w[w].k[0][0][0])[h * AT_D + d], e, A);
        }
        float * P = part + ((size_t) (kvh * AT_GQA + h) * LKB_ATTN_SPLIT + sp) * LKB_ATTN_PARTW;
        if (d == 0) { P[0] = M; P[1] = L; }
        P[2 + d] = A;
    }
}

// ref: src/kernels.cu:1562-1599 (k_attn_combine: same arguments)
__global__ void __launch_bounds__(AT_D) k_attn_combine(const float * __restrict__ part, const int * __restrict__ d_pos,
                                                       float * __restrict__ out, lkb_q8blk * __restrict__ yq8) {
    lkb_pdl_trigger();
    lkb_pdl_wait();
    const int head = blockIdx.x, d = threadIdx.x;
    const int seq_len = *d_pos + 1;
    const int nsl = at_slices(seq_len);
    const int chunk = (((seq_len + nsl - 1) / nsl) + AT_G - 1) / AT_G * AT_G;
    const float * P = part + (size_t) head * LKB_ATTN_SPLIT * LKB_ATTN_PARTW;
    float M = -1e30f;
    for (int s = 0; s < nsl && s * chunk < seq_len; ++s) M = fmaxf(M, P[s * LKB_ATTN_PARTW]);
    float L = 0.0f, A = 0.0f;
    for (int s = 0; s < nsl && s * chunk < seq_len; ++s) {
        const float e = __expf(P[s * LKB_ATTN_PARTW] - M);
        L = fmaf(P[s * LKB_ATTN_PARTW + 1], e, L);
        A = fmaf(P[s * LKB_ATTN_PARTW + 2 + d], e, A);
    }
    const float o = __fdiv_rn(A, L);
    if (out) out[head * AT_D + d] = o;
    if (yq8) lkb_quant_store(o, yq8 + 2 * head + (d >> 5), d & 31);
}

// Per-head RMSNorm (weights qn / kn over 64 dims), NEOX half-split rotation at position *d_pos, and the
// append of the rotated K and of V to the fp16 cache.  One warp per head: lane i holds dims i and i + 32,
// which are exactly the pair that rotates together.  The sum of squares follows the reference's halving
// tree (s[i] += s[i + o], o = 32..1), whose root is what lane 0 of an xor butterfly holds.
// ref: src/kernels.cu:871-915, src/kernels.cuh:35-54
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
    const float * nw = is_q ? qn : kn;
    const int ipos = *d_pos;
    const float pos = (float) ipos;
    const float a = dst[lane], b = dst[lane + 32];
    float ss = __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b));
    ss = __shfl_sync(LKB_FULL, lkb_warp_sum(ss), 0);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float) AT_D), 1e-5f));
    const float x0 = __fmul_rn(__fmul_rn(a, inv), nw[lane]), x1 = __fmul_rn(__fmul_rn(b, inv), nw[lane + 32]);
    const float invf = powf(theta, __fdiv_rn(__fmul_rn(-2.0f, (float) lane), (float) AT_D));
    float sn, cs;
    sincosf(__fmul_rn(pos, invf), &sn, &cs);                // precise form: large arguments (ref: src/kernels.cuh:45-48)
    const float y0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn)), y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
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
    const cudaError_t e = cudaFuncSetAttribute(k_attn_split, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(AtSmem));
    if (e != cudaSuccess) return -(int) e;
    g_mixer_ready = 1;
    return LKB_OK;
}

extern "C" {

int lkb_attn_split(const float * q, const void * kc, const void * vc, const int * d_pos, float * part, lkb_stream_t st) {
    if (!lkb_context().inited || !g_mixer_ready) return LKB_ERR_NOT_INIT;
    if (!q || !kc || !vc || !d_pos || !part) return LKB_ERR_NULL;
    return lkb_launch(k_attn_split, dim3(AT_KVH, LKB_ATTN_SPLIT), dim3(AT_WARPS * 32), sizeof(AtSmem), (cudaStream_t) st,
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
