// lkb_lmhead.cu - the Q6_K output projection (lm_head GEMV), the two-stage argmax and the Q6_K
// embedding row for sm_100a.  HBM-bound: 1680 bytes per vocabulary row (ql 1024 + qh 512 + scales 128 +
// d 16), 110 MB at vocab 65536, read exactly once.
//
// Streaming design: a persistent CTA per SM owns a contiguous range of rows and pulls it through a ring of
// shared-memory chunks (16 rows = 26,880 B each, 5 deep = 134 KB in flight per SM) with 1-D bulk async
// copies (TMA, non-multicast) issued by a dedicated producer warp; sixteen consumer warps take one row each
// per chunk.  The arithmetic is the reference's shipped dp4a form (ref: src/kernels.cu:426-478): lane L owns
// elements 8L..8L+7 of every super-block, integer group sums are exact, one fp32 term per lane and
// super-block accumulated in super-block order, then the xor butterfly -- bit-identical results.
#include "lkb_device.cuh"

#define LM_ROWS    16
#define LM_NBUF    5
#define LM_THREADS ((LM_ROWS + 1) * 32)
#define LM_SPIN    (1u << 22)

struct LmChunk {
    alignas(128) unsigned char ql[LM_ROWS * 1024];
    alignas(128) unsigned char qh[LM_ROWS * 512];
    alignas(16)  int8_t        sc[LM_ROWS * 128];
    alignas(16)  __half        d[LM_ROWS * 8];
};
struct LmSmem {
    LmChunk c[LM_NBUF];
    alignas(8) unsigned long long full[LM_NBUF], empty[LM_NBUF];
    int abort;
};

__device__ unsigned g_lm_status;

__device__ __forceinline__ unsigned lm_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ bool lm_try(unsigned long long * b, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(lm_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool lm_wait(LmSmem & S, unsigned long long * b, unsigned parity, unsigned code) {
    for (unsigned i = 0; i < LM_SPIN; ++i) {
        if (lm_try(b, parity)) return true;
        if ((i & 255u) == 255u && *(volatile int *) &S.abort) return false;
    }
    atomicCAS(&g_lm_status, 0u, code);
    *(volatile int *) &S.abort = 1;
    return false;
}
__device__ __forceinline__ void lm_bulk(void * dst, const void * src, unsigned bytes, unsigned long long * b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(lm_u32(dst)), "l"(src), "r"(bytes), "r"(lm_u32(b)) : "memory");
}

// One row's lane partial: 8 super-blocks, the lane's 8 elements of each.  ref: src/kernels.cu:452-475
struct LmLane { int ql_idx, qh_idx, qh_sh, hi_nib, sci; };
__device__ __forceinline__ LmLane lm_lane(int lane) {
    LmLane m;
    const int s = 8 * (lane & 15);
    m.hi_nib = (s >= 64);
    const int k = s >> 5;
    m.ql_idx = ((lane >= 16) ? 64 : 0) + (m.hi_nib ? s - 64 : s);
    m.qh_idx = ((lane >= 16) ? 32 : 0) + s - 32 * k;
    m.qh_sh = 2 * k;
    m.sci = lane >> 1;
    return m;
}
__device__ __forceinline__ int lm_group(const unsigned char * QL, const unsigned char * QH, const LmLane & m, int u0, int u1) {
    const uint2 qw = *reinterpret_cast<const uint2 *>(QL + m.ql_idx);
    const uint2 hw = *reinterpret_cast<const uint2 *>(QH + m.qh_idx);
    const unsigned l0 = m.hi_nib ? ((qw.x >> 4) & 0x0F0F0F0Fu) : (qw.x & 0x0F0F0F0Fu);
    const unsigned l1 = m.hi_nib ? ((qw.y >> 4) & 0x0F0F0F0Fu) : (qw.y & 0x0F0F0F0Fu);
    const unsigned h0 = ((hw.x >> m.qh_sh) & 0x03030303u) << 4, h1 = ((hw.y >> m.qh_sh) & 0x03030303u) << 4;
    int a = __dp4a((int) __vsubss4(l0 | h0, 0x20202020u), u0, 0);
    return __dp4a((int) __vsubss4(l1 | h1, 0x20202020u), u1, a);
}

__global__ void __launch_bounds__(LM_THREADS, 1) k_gemv_q6_K_stream(const unsigned char * __restrict__ ql, const unsigned char * __restrict__ qh,
                                                                    const int8_t * __restrict__ sc, const __half * __restrict__ d,
                                                                    const lkb_q8blk * __restrict__ xq, int out_rows, float * __restrict__ y,
                                                                    const float * __restrict__ ssq, float eps) {
    extern __shared__ __align__(128) unsigned char lm_raw[];
    LmSmem & S = *reinterpret_cast<LmSmem *>(lm_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = (int) (((long long) blockIdx.x * out_rows) / gridDim.x), r1 = (int) (((long long) (blockIdx.x + 1) * out_rows) / gridDim.x);
    const int nchunk = (r1 - r0 + LM_ROWS - 1) / LM_ROWS;
    if (tid == 0) {
        S.abort = 0;
        for (int i = 0; i < LM_NBUF; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(lm_u32(&S.full[i])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(lm_u32(&S.empty[i])), "r"(LM_ROWS));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == LM_ROWS) {                                   // producer
        if (lane == 0) {
            for (int c = 0; c < nchunk; ++c) {
                const int b = c % LM_NBUF;
                if (!lm_wait(S, &S.empty[b], ((c / LM_NBUF) & 1u) ^ 1u, 1u)) break;
                const int row = r0 + c * LM_ROWS, n = min(LM_ROWS, r1 - row);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(lm_u32(&S.full[b])), "r"((unsigned) n * 1680u) : "memory");
                lm_bulk(S.c[b].ql, ql + (size_t) row * 1024, (unsigned) n * 1024u, &S.full[b]);
                lm_bulk(S.c[b].qh, qh + (size_t) row * 512, (unsigned) n * 512u, &S.full[b]);
                lm_bulk(S.c[b].sc, sc + (size_t) row * 128, (unsigned) n * 128u, &S.full[b]);
                lm_bulk(S.c[b].d, d + (size_t) row * 8, (unsigned) n * 16u, &S.full[b]);
            }
        }
        return;
    }
    // consumers: the activation this lane needs (8 bytes and d8 of 8 Q8_1 blocks) stays in registers
    lkb_pdl_wait();
    const LmLane m = lm_lane(lane);
    int u0[8], u1[8]; float d8[8];
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        const int * p = reinterpret_cast<const int *>(xq + sb * 8 + (lane >> 2));
        const int ds = p[0];
        d8[sb] = __low2float(*reinterpret_cast<const __half2 *>(&ds));
        u0[sb] = p[1 + 2 * (lane & 3)]; u1[sb] = p[2 + 2 * (lane & 3)];
    }
    float ninv = 1.0f;
    if (ssq) ninv = lkb_norm_inv(ssq, lane, eps);
    for (int c = 0; c < nchunk; ++c) {
        const int b = c % LM_NBUF;
        if (!lm_wait(S, &S.full[b], (c / LM_NBUF) & 1u, 2u)) break;
        const int row = r0 + c * LM_ROWS + warp;
        if (row < r1) {
            const LmChunk & C = S.c[b];
            float acc = 0.0f;
#pragma unroll
            for (int sb = 0; sb < 8; ++sb) {
                const int a = lm_group(C.ql + warp * 1024 + sb * 128, C.qh + warp * 512 + sb * 64, m, u0[sb], u1[sb]);
                const int scv = (int) C.sc[warp * 128 + sb * 16 + m.sci];
                acc = fmaf(__half2float(C.d[warp * 8 + sb]), __fmul_rn(d8[sb], (float) (a * scv)), acc);
            }
            acc = lkb_warp_sum(acc);
            if (lane == 0) y[row] = __fmul_rn(acc, ninv);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(lm_u32(&S.empty[b])) : "memory");
    }
}

// Any shape / alignment: warp per row straight from global memory (same arithmetic).
__global__ void __launch_bounds__(256) k_gemv_q6_K_simple(const unsigned char * __restrict__ ql, const unsigned char * __restrict__ qh,
                                                          const int8_t * __restrict__ sc, const __half * __restrict__ d,
                                                          const lkb_q8blk * __restrict__ xq, int out_rows, int sbpr, float * __restrict__ y,
                                                          const float * __restrict__ ssq, float eps) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= out_rows) return;
    const LmLane m = lm_lane(lane);
    float ninv = 1.0f;
    if (ssq) ninv = lkb_norm_inv(ssq, lane, eps);
    float acc = 0.0f;
    for (int sb = 0; sb < sbpr; ++sb) {
        const size_t blk = (size_t) row * sbpr + sb;
        const int * p = reinterpret_cast<const int *>(xq + sb * 8 + (lane >> 2));
        const int ds = p[0];
        const float d8 = __low2float(*reinterpret_cast<const __half2 *>(&ds));
        const unsigned char * QL = ql + blk * 128 + m.ql_idx; const unsigned char * QH = qh + blk * 64 + m.qh_idx;
        // byte-wise assembly: no alignment assumed
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            w[i] = QL[4 * i] | (QL[4 * i + 1] << 8) | (QL[4 * i + 2] << 16) | ((unsigned) QL[4 * i + 3] << 24);
            w[2 + i] = QH[4 * i] | (QH[4 * i + 1] << 8) | (QH[4 * i + 2] << 16) | ((unsigned) QH[4 * i + 3] << 24);
        }
        int a = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const unsigned lo = m.hi_nib ? ((w[i] >> 4) & 0x0F0F0F0Fu) : (w[i] & 0x0F0F0F0Fu);
            const unsigned hi = ((w[2 + i] >> m.qh_sh) & 0x03030303u) << 4;
            a = __dp4a((int) __vsubss4(lo | hi, 0x20202020u), p[1 + 2 * (lane & 3) + i], a);
        }
        acc = fmaf(__half2float(d[blk]), __fmul_rn(d8, (float) (a * (int) sc[blk * 16 + m.sci])), acc);
    }
    acc = lkb_warp_sum(acc);
    if (lane == 0) y[row] = __fmul_rn(acc, ninv);
}

// Two-stage argmax, lowest index among equal maxima; values that do not exceed -1e30 (and NaN) never win.
// Each candidate becomes one 64-bit key -- the float's bits remapped so that unsigned order is numeric order,
// above the complemented index -- and a block reduces keys with warp shuffles: max key = largest value, and
// among equals the smallest index.  ref: src/kernels.cu:954-995 (fixed 1024 values per block there, any n here)
__device__ __forceinline__ unsigned long long lm_key(float v, int idx) {
    const unsigned u = __float_as_uint(__fadd_rn(v, 0.0f));       // -0 -> +0: equal values must tie
    const unsigned o = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long) o << 32) | (unsigned) (0x7fffffff - idx);
}
__device__ __forceinline__ unsigned long long lm_block_max(unsigned long long k, unsigned long long * sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(LKB_FULL, k, o);
        k = t > k ? t : k;
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = k;
    __syncthreads();
    k = sh[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) k = sh[w] > k ? sh[w] : k;
    return k;
}
__device__ __forceinline__ void lm_unkey(unsigned long long k, float & v, int & idx) {
    const unsigned o = (unsigned) (k >> 32);
    v = __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
    idx = 0x7fffffff - (int) (unsigned) k;
}
__global__ void __launch_bounds__(256) k_argmax_part(const float * __restrict__ v, int n, float * __restrict__ pv, int * __restrict__ pi) {
    lkb_pdl_wait();
    __shared__ unsigned long long sh[8];
    const int base = (blockIdx.x * 256 + threadIdx.x) * 4;
    unsigned long long k = lm_key(-1e30f, blockIdx.x * 1024);
    if (base + 3 < n && !((size_t) v & 15)) {
        const float4 t = *reinterpret_cast<const float4 *>(v + base);
        const float tv[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) if (tv[j] > -1e30f) { const unsigned long long c = lm_key(tv[j], base + j); k = c > k ? c : k; }
    } else {
        for (int j = 0; base + j < n; ++j) if (v[base + j] > -1e30f) { const unsigned long long c = lm_key(v[base + j], base + j); k = c > k ? c : k; }
    }
    k = lm_block_max(k, sh);
    if (threadIdx.x == 0) { float bv; int bi; lm_unkey(k, bv, bi); pv[blockIdx.x] = bv; pi[blockIdx.x] = bi; }
}
__global__ void __launch_bounds__(256) k_argmax_final(const float * __restrict__ pv, const int * __restrict__ pi, int n,
                                                      int * __restrict__ d_token, int * __restrict__ d_pos) {
    lkb_pdl_wait();
    __shared__ unsigned long long sh[8];
    unsigned long long k = lm_key(-1e30f, 0);
    for (int i = threadIdx.x; i < n; i += 256) if (pv[i] > -1e30f) { const unsigned long long c = lm_key(pv[i], pi[i]); k = c > k ? c : k; }
    k = lm_block_max(k, sh);
    if (threadIdx.x == 0) { float bv; int bi; lm_unkey(k, bv, bi); *d_token = bi; if (d_pos) atomicAdd(d_pos, 1); }
}

// One embedding row.  ref: src/kernels.cu:855-868
__global__ void __launch_bounds__(256) k_embed_q6_K(const unsigned char * __restrict__ ql, const unsigned char * __restrict__ qh,
                                                    const int8_t * __restrict__ sc, const __half * __restrict__ d,
                                                    const int * __restrict__ d_token, int n, float * __restrict__ x) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int token = *d_token, sbpr = n / 256;
    const size_t blk = (size_t) token * sbpr + i / 256;
    const int e = i % 256;
    const int nn = (e >= 128) ? 128 : 0, r = e - nn;
    const int qlb = ql[blk * 128 + (nn >> 1) + (r & 63)], qhb = qh[blk * 64 + (nn >> 2) + (r & 31)];
    const int q6 = ((r >= 64) ? (qlb >> 4) : (qlb & 15)) | (((qhb >> (2 * (r >> 5))) & 3) << 4);
    x[i] = __fmul_rn(__fmul_rn(__half2float(d[blk]), (float) sc[blk * 16 + e / 16]), (float) (q6 - 32));
}

static int g_lm_ready = 0;
int lkb_lmhead_init() {
    const cudaError_t e = cudaFuncSetAttribute(k_gemv_q6_K_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(LmSmem));
    if (e != cudaSuccess) return -(int) e;
    g_lm_ready = 1;
    return LKB_OK;
}

extern "C" {

int lkb_gemv_q6_K(const void * ql, const void * qh, const void * sc, const void * d, const lkb_block_q8_1 * xq,
                  int out_rows, int sbpr, float * y, const float * ssq, float eps, lkb_stream_t st) {
    if (!lkb_context().inited || !g_lm_ready) return LKB_ERR_NOT_INIT;
    if (!ql || !qh || !sc || !d || !xq || !y) return LKB_ERR_NULL;
    if (out_rows <= 0 || sbpr <= 0) return LKB_ERR_SHAPE;
    const bool aligned = !(((size_t) ql | (size_t) qh | (size_t) sc | (size_t) d) & 15);
    if (sbpr == 8 && aligned) {
        int grid = lkb_context().sm_count;
        if (grid > (out_rows + LM_ROWS - 1) / LM_ROWS) grid = (out_rows + LM_ROWS - 1) / LM_ROWS;
        k_gemv_q6_K_stream<<<grid, LM_THREADS, sizeof(LmSmem), (cudaStream_t) st>>>(
            (const unsigned char *) ql, (const unsigned char *) qh, (const int8_t *) sc, (const __half *) d,
            (const lkb_q8blk *) xq, out_rows, y, ssq, eps);
    } else {
        k_gemv_q6_K_simple<<<(out_rows + 7) / 8, 256, 0, (cudaStream_t) st>>>(
            (const unsigned char *) ql, (const unsigned char *) qh, (const int8_t *) sc, (const __half *) d,
            (const lkb_q8blk *) xq, out_rows, sbpr, y, ssq, eps);
    }
    return lkb_check_launch();
}

int lkb_argmax_part(const float * v, int n, float * pv, int * pi, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!v || !pv || !pi) return LKB_ERR_NULL;
    if (n <= 0) return LKB_ERR_SHAPE;
    k_argmax_part<<<(n + 1023) / 1024, 256, 0, (cudaStream_t) st>>>(v, n, pv, pi);
    return lkb_check_launch();
}

int lkb_argmax_final(const float * pv, const int * pi, int n, int * d_token, int * d_pos, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!pv || !pi || !d_token) return LKB_ERR_NULL;
    if (n <= 0) return LKB_ERR_SHAPE;
    k_argmax_final<<<1, 256, 0, (cudaStream_t) st>>>(pv, pi, n, d_token, d_pos);
    return lkb_check_launch();
}

int lkb_embed_q6_K(const void * ql, const void * qh, const void * sc, const void * d, const int * d_token, int n,
                   float * x, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!ql || !qh || !sc || !d || !d_token || !x) return LKB_ERR_NULL;
    if (n <= 0 || n % 256) return LKB_ERR_SHAPE;
    k_embed_q6_K<<<(n + 255) / 256, 256, 0, (cudaStream_t) st>>>((const unsigned char *) ql, (const unsigned char *) qh,
                                                                 (const int8_t *) sc, (const __half *) d, d_token, n, x);
    return lkb_check_launch();
}

int lkb_gemv_q6_K_status(void) {
    unsigned v = 0, z = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_lm_status, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_lm_status, &z, sizeof z);
    return (int) v;
}

}  // extern "C"
