// lkb_lmhead.cu - the Q6_K output projection (lm_head GEMV), the two-stage argmax and the Q6_K
// embedding row for sm_100a.  HBM-bound: 1680 bytes per vocabulary row (ql 1024 + qh 512 + scales 128 +
// d 16), 110 MB at vocab 65536, read exactly once.
//
// Streaming design: one persistent CTA per SM pulls chunks of 32 rows (53,760 B) through a 4-deep ring of
// shared memory (215 KB in flight per SM) with 1-D bulk async copies (TMA, non-multicast) issued by a
// dedicated producer warp; sixteen consumer warps take two rows each per chunk.  Most chunks are dealt out
// statically (a contiguous range per CTA), the last 3/16 through a device-side ticket counter so that all SMs
// finish together.  The kernel is issue-limited as much as HBM-limited (about 200 instructions per row and
// warp against 1680 bytes), which is why per-row overhead is amortised over two rows.
// The arithmetic is the reference's shipped dp4a form (ref: src/kernels.cu:426-478): lane L owns elements
// 8L..8L+7 of every super-block, integer group sums are exact, one fp32 term per lane and super-block
// accumulated in super-block order, then the xor butterfly -- bit-identical results.
#include "lkb_device.cuh"
#include <atomic>
#include <cstdlib>

#ifndef LM_RPW
#define LM_RPW     2                          // rows per consumer warp and chunk
#endif
#ifndef LM_NBUF
#define LM_NBUF    4
#endif
#ifndef LM_WARPS
#define LM_WARPS   16                         // consumer warps
#endif
#define LM_ROWS    (LM_WARPS * LM_RPW)        // rows per chunk
#define LM_THREADS ((LM_WARPS + 1) * 32)
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
    int row[LM_NBUF];                                  // first row of the chunk in each slot, -1 = no more work
    int abort;
};

// Chunks are handed out by a device-side ticket counter, so an SM whose memory requests are served faster
// simply takes more chunks and all SMs finish together.  Each launch uses one of LM_SLOTS counter pairs
// {next ticket, CTAs finished}; the last CTA to finish zeroes its pair, so no launch needs a memset.
#define LM_SLOTS 16
#ifndef LM_STATIC
#define LM_STATIC 13
#endif
__device__ unsigned g_lm_status;
__device__ unsigned g_lm_ticket[LM_SLOTS][2];

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
// The -32 offset of the 6-bit values is folded into the accumulator's start value: sum((q-32)*u) =
// sum(q*u) - 32*sum(u), and sum(u) over the lane's 8 activation bytes is known before the weights arrive.
struct LmLane { int ql_idx, qh_idx, qh_sh, nib_sh, sci; };
__device__ __forceinline__ LmLane lm_lane(int lane) {
    LmLane m;
    const int s = 8 * (lane & 15);
    const int hi = (s >= 64);
    const int k = s >> 5;
    m.nib_sh = hi ? 4 : 0;
    m.ql_idx = ((lane >= 16) ? 64 : 0) + (hi ? s - 64 : s);
    m.qh_idx = ((lane >= 16) ? 32 : 0) + s - 32 * k;
    m.qh_sh = 2 * k;
    m.sci = lane >> 1;
    return m;
}
__device__ __forceinline__ int lm_usum(int u0, int u1) { return __dp4a(0x01010101, u0, __dp4a(0x01010101, u1, 0)); }
__device__ __forceinline__ int lm_group(const unsigned char * QL, const unsigned char * QH, const LmLane & m, int u0, int u1, int start) {
    const uint2 qw = *reinterpret_cast<const uint2 *>(QL + m.ql_idx);
    const uint2 hw = *reinterpret_cast<const uint2 *>(QH + m.qh_idx);
    const unsigned q0 = ((qw.x >> m.nib_sh) & 0x0F0F0F0Fu) + 16u * ((hw.x >> m.qh_sh) & 0x03030303u);
    const unsigned q1 = ((qw.y >> m.nib_sh) & 0x0F0F0F0Fu) + 16u * ((hw.y >> m.qh_sh) & 0x03030303u);
    return __dp4a((int) q1, u1, __dp4a((int) q0, u0, start));
}

__global__ void __launch_bounds__(LM_THREADS, 1) k_gemv_q6_K_stream(const unsigned char * __restrict__ ql, const unsigned char * __restrict__ qh,
                                                                    const int8_t * __restrict__ sc, const __half * __restrict__ d,
                                                                    const lkb_q8blk * __restrict__ xq, int out_rows, float * __restrict__ y,
                                                                    const float * __restrict__ ssq, float eps, int slot, int stat16) {
    extern __shared__ __align__(128) unsigned char lm_raw[];
    LmSmem & S = *reinterpret_cast<LmSmem *>(lm_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned total = (unsigned) ((out_rows + LM_ROWS - 1) / LM_ROWS);
    lkb_pdl_trigger();                                       // the next kernel may be scheduled; it waits for our results itself
    if (tid == 0) {
        S.abort = 0;
        for (int i = 0; i < LM_NBUF; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(lm_u32(&S.full[i])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(lm_u32(&S.empty[i])), "r"(LM_WARPS));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == LM_WARPS) {                                  // producer: weights do not depend on the previous kernel
        if (lane == 0) {
            unsigned * ctr = g_lm_ticket[slot];
            // Four tickets in flight: one atomic round trip (~1 us) is longer than a chunk's share of the stream.
            // The loop is unrolled by hand so that each ticket lives in its own register and using one does not
            // wait for the younger ones.
            unsigned t0 = atomicAdd(&ctr[0], 1u), t1 = atomicAdd(&ctr[0], 1u), t2 = atomicAdd(&ctr[0], 1u), t3 = atomicAdd(&ctr[0], 1u);
            int c = 0;
            // The first LM_STATIC/16 of the chunks are dealt out statically (CTA c streams a contiguous range);
            // only the rest goes through the ticket counter, which evens out the finish times.
            const unsigned nstat = (unsigned) (((unsigned long long) total * stat16 / 16) / gridDim.x);
            const unsigned dyn0 = nstat * gridDim.x;
            auto issue = [&](unsigned id) -> bool {           // one ring slot: a chunk, or the end marker
                const int b = c % LM_NBUF;
                if (!lm_wait(S, &S.empty[b], ((c / LM_NBUF) & 1u) ^ 1u, 1u)) return false;
                if (id >= total) {
                    S.row[b] = -1;
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(lm_u32(&S.full[b])) : "memory");
                    return false;
                }
                const int row = (int) id * LM_ROWS, n = min(LM_ROWS, out_rows - row);
                S.row[b] = row;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(lm_u32(&S.full[b])), "r"((unsigned) n * 1680u) : "memory");
                lm_bulk(S.c[b].ql, ql + (size_t) row * 1024, (unsigned) n * 1024u, &S.full[b]);
                lm_bulk(S.c[b].qh, qh + (size_t) row * 512, (unsigned) n * 512u, &S.full[b]);
                lm_bulk(S.c[b].sc, sc + (size_t) row * 128, (unsigned) n * 128u, &S.full[b]);
                lm_bulk(S.c[b].d, d + (size_t) row * 8, (unsigned) n * 16u, &S.full[b]);
                ++c;
                return true;
            };
            // Tickets are used strictly in the order they were drawn (t0, t1, t2, t3, t0, ...): a CTA's tickets
            // ascend, so the first one past the end means every ticket it still holds is past the end too.
            auto ticketed = [&](unsigned & t) -> bool {
                const unsigned id = dyn0 + t;
                if (id < total) t = atomicAdd(&ctr[0], 1u);
                return issue(id);
            };
            bool ok = true;
            for (unsigned i = 0; ok && i < nstat; ++i) ok = issue(blockIdx.x * nstat + i);
            if (ok) while (ticketed(t0) && ticketed(t1) && ticketed(t2) && ticketed(t3)) { }
            __threadfence();
            if (atomicAdd(&ctr[1], 1u) == gridDim.x - 1) { ctr[0] = 0u; ctr[1] = 0u; __threadfence(); }
        }
        return;
    }
    // consumers: the activation this lane needs (8 bytes and d8 of 8 Q8_1 blocks) stays in registers
    lkb_pdl_wait();
    const LmLane m = lm_lane(lane);
    int u0[8], u1[8], st32[8]; float d8[8];
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
        const int * p = reinterpret_cast<const int *>(xq + sb * 8 + (lane >> 2));
        const int ds = p[0];
        d8[sb] = __low2float(*reinterpret_cast<const __half2 *>(&ds));
        u0[sb] = p[1 + 2 * (lane & 3)]; u1[sb] = p[2 + 2 * (lane & 3)];
        st32[sb] = -32 * lm_usum(u0[sb], u1[sb]);
    }
    float ninv = 1.0f;
    if (ssq) ninv = lkb_norm_inv(ssq, lane, eps);
    for (int b = 0, ph = 0;;) {
        if (!lm_wait(S, &S.full[b], (unsigned) ph, 2u)) break;
        const int base = *(volatile int *) &S.row[b];
        if (base < 0) break;
        const LmChunk & C = S.c[b];
        float acc[LM_RPW];
        unsigned dv[LM_RPW][4];
#pragma unroll
        for (int r = 0; r < LM_RPW; ++r) {
            const uint4 dw = *reinterpret_cast<const uint4 *>(C.d + (warp * LM_RPW + r) * 8);   // the row's 8 fp16 d
            dv[r][0] = dw.x; dv[r][1] = dw.y; dv[r][2] = dw.z; dv[r][3] = dw.w;
            acc[r] = 0.0f;
        }
#pragma unroll
        for (int sb = 0; sb < 8; ++sb) {
#pragma unroll
            for (int r = 0; r < LM_RPW; ++r) {
                const int lr = warp * LM_RPW + r;
                const int a = lm_group(C.ql + lr * 1024 + sb * 128, C.qh + lr * 512 + sb * 64, m, u0[sb], u1[sb], st32[sb]);
                const int scv = (int) C.sc[lr * 128 + sb * 16 + m.sci];
                const __half2 dp = *reinterpret_cast<const __half2 *>(&dv[r][sb >> 1]);
                acc[r] = fmaf((sb & 1) ? __high2float(dp) : __low2float(dp), __fmul_rn(d8[sb], (float) (a * scv)), acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < LM_RPW; ++r) {
            const float t = lkb_warp_sum(acc[r]);
            const int row = base + warp * LM_RPW + r;
            if (lane == 0 && row < out_rows) y[row] = __fmul_rn(t, ninv);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(lm_u32(&S.empty[b])) : "memory");
        if (++b == LM_NBUF) { b = 0; ph ^= 1; }
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
        int a = -32 * lm_usum(p[1 + 2 * (lane & 3)], p[2 + 2 * (lane & 3)]);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const unsigned q = ((w[i] >> m.nib_sh) & 0x0F0F0F0Fu) + 16u * ((w[2 + i] >> m.qh_sh) & 0x03030303u);
            a = __dp4a((int) q, p[1 + 2 * (lane & 3) + i], a);
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
    return ((unsigned long long) lkb_orderable(v) << 32) | (unsigned) (0x7fffffff - idx);
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
    lkb_pdl_trigger();
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
    lkb_pdl_trigger();
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
static int g_lm_static = LM_STATIC;      // sixteenths of the chunks dealt out statically (env LKB_LM_STATIC, tuning)
int lkb_lmhead_init() {
    const cudaError_t e = cudaFuncSetAttribute(k_gemv_q6_K_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(LmSmem));
    if (e != cudaSuccess) return -(int) e;
    if (const char * e = getenv("LKB_LM_STATIC")) { const int v = atoi(e); if (v >= 0 && v <= 16) g_lm_static = v; }
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
        static std::atomic<unsigned> seq{0};               // consecutive launches take different ticket counters
        return lkb_launch(k_gemv_q6_K_stream, dim3(grid), dim3(LM_THREADS), sizeof(LmSmem), (cudaStream_t) st,
                          (const unsigned char *) ql, (const unsigned char *) qh, (const int8_t *) sc, (const __half *) d,
                          (const lkb_q8blk *) xq, out_rows, y, ssq, eps, (int) (seq.fetch_add(1u) % LM_SLOTS), g_lm_static);
    }
    return lkb_launch(k_gemv_q6_K_simple, dim3((out_rows + 7) / 8), dim3(256), 0, (cudaStream_t) st,
                      (const unsigned char *) ql, (const unsigned char *) qh, (const int8_t *) sc, (const __half *) d,
                      (const lkb_q8blk *) xq, out_rows, sbpr, y, ssq, eps);
}

int lkb_argmax_part(const float * v, int n, float * pv, int * pi, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!v || !pv || !pi) return LKB_ERR_NULL;
    if (n <= 0) return LKB_ERR_SHAPE;
    return lkb_launch(k_argmax_part, dim3((n + 1023) / 1024), dim3(256), 0, (cudaStream_t) st, v, n, pv, pi);
}

int lkb_argmax_final(const float * pv, const int * pi, int n, int * d_token, int * d_pos, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!pv || !pi || !d_token) return LKB_ERR_NULL;
    if (n <= 0) return LKB_ERR_SHAPE;
    return lkb_launch(k_argmax_final, dim3(1), dim3(256), 0, (cudaStream_t) st, pv, pi, n, d_token, d_pos);
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
    if (v) {                                               // an aborted launch may leave its ticket counters mid-count
        static const unsigned zeros[LM_SLOTS][2] = {};
        cudaMemcpyToSymbol(g_lm_status, &z, sizeof z);
        cudaMemcpyToSymbol(g_lm_ticket, zeros, sizeof zeros);
    }
    return (int) v;
}

}  // extern "C"
