// lkb_fused.cu - one persistent cooperative kernel for the batch-1 MoE FFN stack.
//
// The reference runs five kernels per MoE layer (router dot, top-4, gate|up GEMV,
// SwiGLU quantiser, down GEMV + accumulate; ref: src/engine.cu:739-811).  On B200 a
// layer streams 21.8 MB in about 3.3 us of HBM time, so five launch boundaries cost
// more than the data.  Here ONE launch walks any number of layers:
//   * one CTA per SM, co-resident (cooperative launch), three grid barriers per layer
//     (after the router logits, after gate|up, after the residual update);
//   * as soon as the four experts are known, each CTA requests ALL the weight rows it
//     will need for the layer -- its slice of gate|up and of down -- with 1-D bulk
//     async copies (TMA, no multicast) into ~150 KB of shared memory, completion
//     tracked by mbarriers per 8-row chunk, so the whole 21 MB is in flight at once
//     and arithmetic starts as chunks land;
//   * the next layer's router row is requested while the down projection runs.
// Arithmetic per output is exactly that of the stand-alone kernels (lane-strided
// blocks, xor butterfly, fixed k = 0..3 order), so results are bit-identical to the
// five-kernel sequence.
//
// Every wait (grid barrier, mbarrier) is bounded: on expiry the CTA records a code in
// the status word and leaves; the other CTAs' waits then expire too.
#include <cooperative_groups.h>
#include "lkb_device.cuh"

#define FUSED_THREADS 512
#define FUSED_WARPS   (FUSED_THREADS / 32)
#define CH_ROWS       8                       // rows per mbarrier chunk
#define MAX_GU_ROWS   96                      // gate|up rows a CTA may own (12288 / #CTAs, rounded up; 84 on 148 SMs)
#define MAX_DN_ROWS   16                      // down rows a CTA may own (2048 / #CTAs, rounded up; 14 on 148 SMs)
#define GU_BPR        (LKB_HIDDEN / 32)       // 64
#define DN_BPR        (LKB_MOE_INTER / 32)    // 48
#define N_GU_CH       (MAX_GU_ROWS / CH_ROWS) // 12
#define N_DN_CH       (LKB_TOP_K * ((MAX_DN_ROWS + CH_ROWS - 1) / CH_ROWS))   // 8
#define SPIN_LIMIT    (1u << 22)

struct FusedSmem {
    alignas(128) unsigned char gu_q[MAX_GU_ROWS * GU_BPR * 16];          // 98304
    alignas(128) unsigned char dn_q[LKB_TOP_K * MAX_DN_ROWS * DN_BPR * 16]; // 49152
    alignas(16)  __half gu_d[MAX_GU_ROWS * GU_BPR];                       // 12288
    alignas(16)  __half dn_d[LKB_TOP_K * MAX_DN_ROWS * DN_BPR];           // 6144
    alignas(16)  float  router[LKB_HIDDEN];                               // 8192
    alignas(16)  float  h[LKB_HIDDEN];                                    // 8192 raw u = x*w
    alignas(16)  lkb_q8blk xq[LKB_HIDDEN / 32];                           // 2304
    alignas(16)  lkb_q8blk xq2[LKB_TOP_K * DN_BPR];                       // 6912
    float  ssq[LKB_HIDDEN / 32];
    float  sel[LKB_N_EXPERTS];
    float  sig[LKB_N_EXPERTS];
    float  dot[LKB_TOP_K][MAX_DN_ROWS];
    int    idx[LKB_TOP_K];
    float  wk[LKB_TOP_K];
    float  inv;
    int    abort;
    alignas(8) unsigned long long mbar_gu[N_GU_CH];
    alignas(8) unsigned long long mbar_dn[N_DN_CH];
    alignas(8) unsigned long long mbar_rt;
};

// ---- PTX wrappers -----------------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long * b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long * b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long * b, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait; returns false on expiry.
__device__ __forceinline__ bool mbar_wait(unsigned long long * b, unsigned parity) {
    for (unsigned i = 0; i < SPIN_LIMIT; ++i) if (mbar_try_wait(b, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void * dst, const void * src, unsigned bytes, unsigned long long * b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned * p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Grid barrier over gridDim.x CTAs on a monotonically increasing counter (zeroed by
// the launcher).  Returns false if the wait expired or another CTA reported a fault.
__device__ __forceinline__ bool grid_barrier(unsigned * bar, unsigned * status, FusedSmem & S, unsigned code) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned ticket = atomicAdd(bar, 1u);
        const unsigned target = (ticket / gridDim.x + 1u) * gridDim.x;
        bool ok = false;
        for (unsigned i = 0; i < SPIN_LIMIT; ++i) {
            if (ld_acquire(bar) >= target) { ok = true; break; }
            if ((i & 1023u) == 1023u && ld_acquire(status) != 0u) break;
            __nanosleep(20);
        }
        if (!ok) { atomicCAS(status, 0u, code); S.abort = 1; }
    }
    __syncthreads();
    return S.abort == 0;
}

// Rows [j0, j1) of a logical row space made of `nseg` equal segments of `seg_rows`
// rows; segment s lives at base_q[s]/base_d[s].  Issues the bulk copies of chunk c.
struct SegView {
    const uint4 *  q[8];
    const __half * d[8];
};

__device__ __forceinline__ void issue_rows(const SegView & v, int seg_rows, int bpr, int g_begin, int g_end,
                                           unsigned char * sq, __half * sd, unsigned long long * mb) {
    // [g_begin, g_end) may straddle one segment boundary
    unsigned bytes = (unsigned) (g_end - g_begin) * (unsigned) bpr * 18u;
    mbar_expect_tx(mb, bytes);
    int g = g_begin;
    while (g < g_end) {
        const int s = g / seg_rows, r = g - s * seg_rows;
        int n = g_end - g; if (n > seg_rows - r) n = seg_rows - r;
        bulk_g2s(sq, v.q[s] + (size_t) r * bpr, (unsigned) n * bpr * 16u, mb);
        bulk_g2s(sd, v.d[s] + (size_t) r * bpr, (unsigned) n * bpr * 2u, mb);
        sq += (size_t) n * bpr * 16; sd += (size_t) n * bpr; g += n;
    }
}

// One row's lane partial from shared memory (blocks lane, lane+32), reference order.
template <int NB>
__device__ __forceinline__ float smem_row_partial(const unsigned char * q, const __half * d, int bpr, int lane,
                                                  const int (&xq)[NB][8], const float (&d8)[NB], const float (&s8)[NB]) {
    float a = 0.0f;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int k = lane + 32 * j;
        if (k < bpr) {
            const uint4 w = *reinterpret_cast<const uint4 *>(q + (size_t) k * 16);
            a = lkb_block_acc(__half2float(d[k]), d8[j], lkb_sumi(w, xq[j]), s8[j], a);
        }
    }
    return a;
}

template <int NB>
__device__ __forceinline__ void load_xregs(const lkb_q8blk * xq, int bpr, int lane, int (&q)[NB][8], float (&d8)[NB], float (&s8)[NB]) {
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int k = lane + 32 * j;
        if (k < bpr) {
            const int * p = reinterpret_cast<const int *>(xq + k);
            const int ds = p[0];
            const __half2 h = *reinterpret_cast<const __half2 *>(&ds);
            d8[j] = __low2float(h); s8[j] = __fmul_rn(8.0f, __high2float(h));
#pragma unroll
            for (int i = 0; i < 8; ++i) q[j][i] = p[1 + i];
        } else {
            d8[j] = 0.0f; s8[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) q[j][i] = 0;
        }
    }
}

struct FusedArgs {
    lkb_moe_layer         one;         // used when layers == nullptr
    const lkb_moe_layer * layers;      // device array, or null
    int                   n_layers;
    float *               x;           // residual stream, updated in place
    const float *         final_norm_w;   // optional: produce (h32, yq8, ssq) of the final x
    float *               out_h32;
    lkb_q8blk *           out_yq8;
    float *               out_ssq;
    int *                 idx_out;     // optional [n_layers][4]
    float *               w_out;       // optional [n_layers][4]
    float *               logits;      // scratch [64]
    float *               gu;          // scratch [2*4*1536]
    unsigned *            bar;         // scratch [2]: {barrier counter, status}
    int                   softmax;
};

// Quantise u = x*w for all 2048 elements into S.xq / S.ssq / S.h (every CTA, redundantly).
__device__ __forceinline__ void fused_norm_prod(FusedSmem & S, const float * __restrict__ x, const float * __restrict__ nw) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < (LKB_HIDDEN / 32) / FUSED_WARPS; ++j) {
        const int b = warp + FUSED_WARPS * j;
        const int i = b * 32 + lane;
        const float xv = __ldcg(x + i);                    // written by other CTAs: bypass L1
        const float uv = __fmul_rn(xv, nw[i]);
        S.h[i] = uv;
        lkb_norm_prod_warp(xv, uv, lane, S.xq, S.ssq, b);
    }
    __syncthreads();
    if (warp == 0) {
        const float inv = lkb_norm_inv(S.ssq, lane, LKB_EPS);
        if (lane == 0) S.inv = inv;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(FUSED_THREADS, 1) k_moe_ffn_stack(const FusedArgs a) {
    extern __shared__ __align__(128) unsigned char fused_smem_raw[];
    FusedSmem & S = *reinterpret_cast<FusedSmem *>(fused_smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nct = gridDim.x, cta = blockIdx.x;
    unsigned * status = a.bar + 1;

    // static partition of the layer's rows over the CTAs (balanced, contiguous)
    const int GU_TOTAL = 2 * LKB_TOP_K * LKB_MOE_INTER;
    const int gu0 = (int) (((long long) cta * GU_TOTAL) / nct), gu1 = (int) (((long long) (cta + 1) * GU_TOTAL) / nct);
    const int dn0 = (int) (((long long) cta * LKB_HIDDEN) / nct), dn1 = (int) (((long long) (cta + 1) * LKB_HIDDEN) / nct);
    const int n_gu = gu1 - gu0, n_dn = dn1 - dn0;
    const int n_gu_ch = (n_gu + CH_ROWS - 1) / CH_ROWS;
    const int dn_ch_per_k = (n_dn + CH_ROWS - 1) / CH_ROWS;

    if (tid == 0) {
        S.abort = 0;
        for (int i = 0; i < N_GU_CH; ++i) mbar_init(&S.mbar_gu[i], 1);
        for (int i = 0; i < N_DN_CH; ++i) mbar_init(&S.mbar_dn[i], 1);
        mbar_init(&S.mbar_rt, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const lkb_moe_layer * L = a.layers ? a.layers : &a.one;
    // first layer's router row
    if (cta < LKB_N_EXPERTS && tid == 0) {
        mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
        bulk_g2s(S.router, L[0].router + (size_t) cta * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
    }

    for (int l = 0; l < a.n_layers; ++l) {
        const lkb_moe_layer & ly = L[l];
        const unsigned par = (unsigned) (l & 1);

        // ---- phase 0: u = x*w, Q8_1, ssq, inv (every CTA) ----------------------
        fused_norm_prod(S, a.x, ly.norm_w);

        // ---- phase 1: router logit of expert `cta` ------------------------------
        if (cta < LKB_N_EXPERTS && warp == 0) {
            if (!mbar_wait(&S.mbar_rt, par)) { if (lane == 0) { atomicCAS(status, 0u, 100u + l); S.abort = 1; } }
            else {
                float acc = 0.0f;
#pragma unroll 16
                for (int j = 0; j < LKB_HIDDEN / 32; ++j) acc = fmaf(S.router[j * 32 + lane], S.h[j * 32 + lane], acc);
                acc = lkb_warp_sum(acc);
                if (lane == 0) a.logits[cta] = __fmul_rn(acc, S.inv);
            }
        }
        if (!grid_barrier(a.bar, status, S, 1000u + 10u * l + 1u)) return;

        // ---- phase 2: selection (every CTA), then request every weight row ------
        if (tid < LKB_N_EXPERTS) {
            const float lg = __ldcg(a.logits + tid);
            if (!a.softmax) {
                const float g = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg)));
                S.sig[tid] = g;
                S.sel[tid] = __fadd_rn(g, ly.rbias ? ly.rbias[tid] : 0.0f);
            } else {
                S.sel[tid] = lg;
            }
        }
        __syncthreads();
        if (a.softmax) {
            float p = 0.0f;
            if (tid < LKB_N_EXPERTS) {
                float mx = S.sel[0];
                for (int e = 1; e < LKB_N_EXPERTS; ++e) mx = fmaxf(mx, S.sel[e]);
                p = expf(__fsub_rn(S.sel[tid], mx));
                S.sig[tid] = p;
            }
            __syncthreads();
            float pn = 0.0f;
            if (tid < LKB_N_EXPERTS) {
                float den = 0.0f;
                for (int e = 0; e < LKB_N_EXPERTS; ++e) den = __fadd_rn(den, S.sig[e]);
                pn = __fdiv_rn(p, den);
            }
            __syncthreads();
            if (tid < LKB_N_EXPERTS) { S.sig[tid] = pn; S.sel[tid] = __fadd_rn(pn, ly.rbias ? ly.rbias[tid] : 0.0f); }
            __syncthreads();
        }
        if (warp == 0) {
            int ord[LKB_TOP_K]; float wv[LKB_TOP_K];
            lkb_router_select(S.sel, S.sig, lane, ord, wv);
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < LKB_TOP_K; ++k) { S.idx[k] = ord[k]; S.wk[k] = wv[k]; }
                if (cta == 0) {
#pragma unroll
                    for (int k = 0; k < LKB_TOP_K; ++k) {
                        if (a.idx_out) a.idx_out[l * 4 + k] = ord[k];
                        if (a.w_out) a.w_out[l * 4 + k] = wv[k];
                    }
                }
            }
        }
        __syncthreads();
        if (tid == 0) {
            fence_proxy_async();
            SegView gv, dv;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) {
                const size_t eo = (size_t) S.idx[k] * LKB_MOE_INTER * GU_BPR;
                gv.q[k] = (const uint4 *) ly.gate_qs + eo;     gv.d[k] = (const __half *) ly.gate_d + eo;
                gv.q[4 + k] = (const uint4 *) ly.up_qs + eo;   gv.d[4 + k] = (const __half *) ly.up_d + eo;
                const size_t ed = (size_t) S.idx[k] * LKB_HIDDEN * DN_BPR;
                dv.q[k] = (const uint4 *) ly.down_qs + ed;     dv.d[k] = (const __half *) ly.down_d + ed;
            }
            for (int c = 0; c < n_gu_ch; ++c) {
                const int j0 = c * CH_ROWS, j1 = min(n_gu, j0 + CH_ROWS);
                issue_rows(gv, LKB_MOE_INTER, GU_BPR, gu0 + j0, gu0 + j1, S.gu_q + (size_t) j0 * GU_BPR * 16,
                           S.gu_d + (size_t) j0 * GU_BPR, &S.mbar_gu[c]);
            }
            for (int k = 0; k < LKB_TOP_K; ++k)
                for (int c = 0; c < dn_ch_per_k; ++c) {
                    const int j0 = c * CH_ROWS, j1 = min(n_dn, j0 + CH_ROWS);
                    // expert k's rows dn0+j0 .. dn0+j1 (one segment: no straddle)
                    SegView one; one.q[0] = dv.q[k]; one.d[0] = dv.d[k];
                    issue_rows(one, LKB_HIDDEN, DN_BPR, dn0 + j0, dn0 + j1,
                               S.dn_q + ((size_t) k * MAX_DN_ROWS + j0) * DN_BPR * 16,
                               S.dn_d + ((size_t) k * MAX_DN_ROWS + j0) * DN_BPR, &S.mbar_dn[k * dn_ch_per_k + c]);
                }
        }

        // ---- phase 3: gate|up rows of this CTA ----------------------------------
        {
            int xq[2][8]; float d8[2], s8[2];
            load_xregs<2>(S.xq, GU_BPR, lane, xq, d8, s8);
            const float ninv = S.inv;
            for (int j = warp; j < n_gu; j += FUSED_WARPS) {
                if (!mbar_wait(&S.mbar_gu[j / CH_ROWS], par)) {
                    if (lane == 0) { atomicCAS(status, 0u, 200u + l); S.abort = 1; }
                    break;
                }
                const float acc = lkb_warp_sum(smem_row_partial<2>(S.gu_q + (size_t) j * GU_BPR * 16, S.gu_d + (size_t) j * GU_BPR,
                                                                   GU_BPR, lane, xq, d8, s8));
                // logical row -> (half, k, row): the stand-alone kernel's y_a / y_b layout, gate first
                if (lane == 0) a.gu[gu0 + j] = __fmul_rn(acc, ninv);
            }
        }
        if (!grid_barrier(a.bar, status, S, 1000u + 10u * l + 2u)) return;

        // ---- phase 4: SwiGLU + Q8_1 (every CTA), down rows, residual ------------
        {
            const int GU = LKB_TOP_K * LKB_MOE_INTER;
            for (int b = warp; b < GU / 32; b += FUSED_WARPS) {
                const int i = b * 32 + lane;
                const float g = __ldcg(a.gu + i), u = __ldcg(a.gu + GU + i);
                const float v = __fmul_rn(lkb_silu(g), u);
                lkb_quant_store(v, S.xq2 + b, lane);
            }
        }
        __syncthreads();
        // next layer's router row can start now (S.router is no longer read in this layer)
        if (l + 1 < a.n_layers && cta < LKB_N_EXPERTS && tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
            bulk_g2s(S.router, L[l + 1].router + (size_t) cta * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
        }
        for (int t = warp; t < n_dn * LKB_TOP_K; t += FUSED_WARPS) {
            const int k = t % LKB_TOP_K, j = t / LKB_TOP_K;
            int xq[2][8]; float d8[2], s8[2];
            load_xregs<2>(S.xq2 + k * DN_BPR, DN_BPR, lane, xq, d8, s8);
            if (!mbar_wait(&S.mbar_dn[k * dn_ch_per_k + j / CH_ROWS], par)) {
                if (lane == 0) { atomicCAS(status, 0u, 300u + l); S.abort = 1; }
                break;
            }
            const float acc = lkb_warp_sum(smem_row_partial<2>(S.dn_q + ((size_t) k * MAX_DN_ROWS + j) * DN_BPR * 16,
                                                               S.dn_d + ((size_t) k * MAX_DN_ROWS + j) * DN_BPR,
                                                               DN_BPR, lane, xq, d8, s8));
            if (lane == 0) S.dot[k][j] = acc;
        }
        __syncthreads();
        if (tid < n_dn) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) acc = fmaf(S.wk[k], S.dot[k][tid], acc);
            a.x[dn0 + tid] = __fadd_rn(__ldcg(a.x + dn0 + tid), acc);
        }
        if (!grid_barrier(a.bar, status, S, 1000u + 10u * l + 3u)) return;
    }

    // optional: the quantised, un-normalised activation of the final x for the caller's next consumer
    if (a.final_norm_w && cta == 0) {
        fused_norm_prod(S, a.x, a.final_norm_w);
        for (int i = tid; i < LKB_HIDDEN; i += FUSED_THREADS) if (a.out_h32) a.out_h32[i] = S.h[i];
        for (int i = tid; i < LKB_HIDDEN / 32 * 9; i += FUSED_THREADS)
            reinterpret_cast<int *>(a.out_yq8)[i] = reinterpret_cast<const int *>(S.xq)[i];
        if (tid < LKB_HIDDEN / 32) a.out_ssq[tid] = S.ssq[tid];
    }
}

// ---------------------------------------------------------------------------
static int g_fused_ready = 0;

int lkb_fused_init() {
    const cudaError_t e = cudaFuncSetAttribute(k_moe_ffn_stack, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int) sizeof(FusedSmem));
    if (e != cudaSuccess) return -(int) e;
    g_fused_ready = 1;
    return LKB_OK;
}

static int fused_launch(FusedArgs & a, cudaStream_t st) {
    if (!lkb_context().inited || !g_fused_ready) return LKB_ERR_NOT_INIT;
    if (!a.x || !a.logits || !a.gu || !a.bar) return LKB_ERR_NULL;
    if (a.n_layers <= 0) return LKB_ERR_SHAPE;
    if (a.final_norm_w && (!a.out_yq8 || !a.out_ssq)) return LKB_ERR_NULL;
    int grid = lkb_context().sm_count;
    // every CTA's share must fit the shared-memory staging
    const int GU_TOTAL = 2 * LKB_TOP_K * LKB_MOE_INTER;
    if ((GU_TOTAL + grid - 1) / grid > MAX_GU_ROWS || (LKB_HIDDEN + grid - 1) / grid > MAX_DN_ROWS) return LKB_ERR_DEVICE;
    cudaError_t e = cudaMemsetAsync(a.bar, 0, 2 * sizeof(unsigned), st);
    if (e != cudaSuccess) return -(int) e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(FUSED_THREADS); cfg.dynamicSmemBytes = sizeof(FusedSmem); cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, k_moe_ffn_stack, a);
    if (e != cudaSuccess) { (void) cudaGetLastError(); return -(int) e; }
    return LKB_OK;
}

extern "C" {

int lkb_moe_ffn_decode(const lkb_moe_layer * layer, float * x, int * idx_out, float * w_out,
                       const lkb_norm_prod_t * next, const lkb_moe_scratch * scratch, lkb_stream_t st) {
    if (!layer || !scratch) return LKB_ERR_NULL;
    FusedArgs a = {};
    a.one = *layer; a.layers = nullptr; a.n_layers = 1; a.x = x; a.idx_out = idx_out; a.w_out = w_out;
    if (next && next->w) { a.final_norm_w = next->w; a.out_h32 = next->h32; a.out_yq8 = reinterpret_cast<lkb_q8blk *>(next->yq8); a.out_ssq = next->ssq; }
    a.logits = scratch->logits; a.gu = scratch->gu; a.bar = scratch->sync; a.softmax = layer->softmax;
    return fused_launch(a, (cudaStream_t) st);
}

int lkb_moe_ffn_decode_stack(const lkb_moe_layer * layers_dev, int n_layers, int softmax, float * x,
                             int * idx_out, float * w_out, const lkb_norm_prod_t * next,
                             const lkb_moe_scratch * scratch, lkb_stream_t st) {
    if (!layers_dev || !scratch) return LKB_ERR_NULL;
    FusedArgs a = {};
    a.layers = layers_dev; a.n_layers = n_layers; a.x = x; a.idx_out = idx_out; a.w_out = w_out;
    if (next && next->w) { a.final_norm_w = next->w; a.out_h32 = next->h32; a.out_yq8 = reinterpret_cast<lkb_q8blk *>(next->yq8); a.out_ssq = next->ssq; }
    a.logits = scratch->logits; a.gu = scratch->gu; a.bar = scratch->sync; a.softmax = softmax;
    return fused_launch(a, (cudaStream_t) st);
}

}  // extern "C"
