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
    alignas(16)  int8_t xq2_q[LKB_TOP_K * DN_BPR * 32];                   // 6144: quants of silu(g)*u, 32 B per block
    alignas(8)   float2 xq2_s[LKB_TOP_K * DN_BPR];                        // 1536: (float(fp16 d), 8*float(fp16 sum))
    float  ssq[LKB_HIDDEN / 32];
    float  sel[LKB_N_EXPERTS];
    float  sig[LKB_N_EXPERTS];
    float  dot[LKB_TOP_K][MAX_DN_ROWS];
    int    idx[LKB_TOP_K];
    float  wk[LKB_TOP_K];
    float  inv;
    int    abort;
    unsigned bar_target;
    alignas(8) lkb_moe_layer ly;          // this layer's descriptor (staged: a global read costs ~1 us of latency)
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
// the launcher), split into arrive and wait so that independent work can sit between
// them.  Both are called by every thread; thread 0 does the global traffic.
// wait returns false if it expired or another CTA reported a fault.
__device__ __forceinline__ void grid_arrive(unsigned * bar, FusedSmem & S) {
    __syncthreads();                                   // this CTA's global writes are issued
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned ticket = atomicAdd(bar, 1u);
        S.bar_target = (ticket / gridDim.x + 1u) * gridDim.x;
    }
}
__device__ __forceinline__ bool grid_wait(unsigned * bar, unsigned * status, FusedSmem & S, unsigned code,
                                          unsigned spin_limit = SPIN_LIMIT) {
    if (threadIdx.x == 0) {
        const unsigned target = S.bar_target;
        bool ok = false;
        for (unsigned i = 0; i < spin_limit; ++i) {
            if (ld_acquire(bar) >= target) { ok = true; break; }
            if ((i & 1023u) == 1023u && ld_acquire(status) != 0u) break;
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

// Gate|up logical rows g = (half*4 + k)*1536 + row; [g_begin, g_end) may straddle one segment boundary.
__device__ __forceinline__ void issue_gu_rows(const lkb_moe_layer & ly, const int * idx, int g_begin, int g_end,
                                              unsigned char * sq, __half * sd, unsigned long long * mb) {
    mbar_expect_tx(mb, (unsigned) (g_end - g_begin) * (unsigned) GU_BPR * 18u);
    int g = g_begin;
    while (g < g_end) {
        const int seg = g / LKB_MOE_INTER, r = g - seg * LKB_MOE_INTER;
        int n = g_end - g; if (n > LKB_MOE_INTER - r) n = LKB_MOE_INTER - r;
        const size_t blk = ((size_t) idx[seg & 3] * LKB_MOE_INTER + r) * GU_BPR;
        const uint4 * q = (const uint4 *) (seg < 4 ? ly.gate_qs : ly.up_qs) + blk;
        const __half * d = (const __half *) (seg < 4 ? ly.gate_d : ly.up_d) + blk;
        bulk_g2s(sq, q, (unsigned) n * GU_BPR * 16u, mb);
        bulk_g2s(sd, d, (unsigned) n * GU_BPR * 2u, mb);
        sq += (size_t) n * GU_BPR * 16; sd += (size_t) n * GU_BPR; g += n;
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

// Optional phase timestamps (clock64 of thread 0) for tuning: [cta][layer][16].
static unsigned long long * g_fused_timing = nullptr;
static int g_fused_absent_cta = -1;              // test hook, see lkb_debug_fused_absent_cta
static unsigned g_fused_spin_limit = 0;          // 0: default
#define FUSED_STAMP(slot) do { if (a.timing && tid == 0 && l < 4) a.timing[((size_t) cta * 4 + l) * 16 + (slot)] = clock64(); } while (0)


// Four independent 32-element blocks quantised together: the same operations per block
// as lkb_quant_lane, with the four dependency chains interleaved so their latencies
// overlap (the idea of the reference's quantize_q8_1_warp2, ref: src/quant.cuh:83-104).
template <int N>
__device__ __forceinline__ void quantN(const float (&v)[N], int (&q)[N], float (&d)[N], float (&sum)[N]) {
    unsigned am[N];
#pragma unroll
    for (int j = 0; j < N; ++j) { am[j] = __reduce_max_sync(LKB_FULL, __float_as_uint(fabsf(v[j]))); sum[j] = v[j]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int j = 0; j < N; ++j) sum[j] = __fadd_rn(sum[j], __shfl_xor_sync(LKB_FULL, sum[j], o));
#pragma unroll
    for (int j = 0; j < N; ++j) {
        d[j] = __fdiv_rn(__uint_as_float(am[j]), 127.0f);
        q[j] = (am[j] == 0u) ? 0 : (int) roundf(__fdiv_rn(v[j], d[j]));
    }
}
__device__ __forceinline__ void quant4(const float (&v)[4], int (&q)[4], float (&d)[4], float (&sum)[4]) { quantN<4>(v, q, d, sum); }
__device__ __forceinline__ void sumsq4(const float (&x)[4], float (&sq)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) sq[j] = __fmul_rn(x[j], x[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int j = 0; j < 4; ++j) sq[j] = __fadd_rn(sq[j], __shfl_xor_sync(LKB_FULL, sq[j], o));
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
    unsigned long long *  timing;
    int                   absent_cta;  // test hook: this CTA leaves at once and never arrives (-1: none)
    unsigned              spin_limit;  // iterations a grid-barrier wait may spin
};

// Blocks b = warp + 16 j (j = 0..3) of the 2048-vector belong to this warp, element `lane`.
// Loads x (written by other CTAs -> L2) and forms u = x*w into S.h.
__device__ __forceinline__ void fused_load_u(FusedSmem & S, const float * __restrict__ x, const float (&nw)[4],
                                             float (&xv)[4], float (&uv)[4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int j = 0; j < 4; ++j) xv[j] = __ldcg(x + (warp + FUSED_WARPS * j) * 32 + lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) { uv[j] = __fmul_rn(xv[j], nw[j]); S.h[(warp + FUSED_WARPS * j) * 32 + lane] = uv[j]; }
}
// Q8_1 of u, ssq of x, inv -> S.xq, S.ssq, S.inv (ends with a CTA barrier).
__device__ __forceinline__ void fused_quant_u(FusedSmem & S, const float (&xv)[4], const float (&uv)[4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int q[4]; float d[4], sm[4], sq[4];
    quant4(uv, q, d, sm);
    sumsq4(xv, sq);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int b = warp + FUSED_WARPS * j;
        S.xq[b].qs[lane] = (int8_t) q[j];
        if (lane == 0) { S.xq[b].ds = __floats2half2_rn(d[j], sm[j]); S.ssq[b] = sq[j]; }
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
    if ((int) blockIdx.x == a.absent_cta) return;          // host-requested: the others' bounded waits must expire

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
    // first layer's router row, first layer's norm weights
    if (cta < LKB_N_EXPERTS && tid == 0) {
        mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
        bulk_g2s(S.router, L[0].router + (size_t) cta * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
    }
    float nw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) nw[j] = L[0].norm_w[(warp + FUSED_WARPS * j) * 32 + lane];

    if (tid < (int) (sizeof(lkb_moe_layer) / 8))
        reinterpret_cast<unsigned long long *>(&S.ly)[tid] = reinterpret_cast<const unsigned long long *>(&L[0])[tid];
    __syncthreads();

    for (int l = 0; l < a.n_layers; ++l) {
        const lkb_moe_layer & ly = S.ly;
        const unsigned par = (unsigned) (l & 1);

        // ---- A: u = x*w; the 64 router CTAs produce their logit; arrive ----------
        FUSED_STAMP(0);
        float xv[4], uv[4];
        fused_load_u(S, a.x, nw, xv, uv);
        if (cta < LKB_N_EXPERTS) {
            __syncthreads();                                        // S.h complete
            if (warp == 0) {
                if (!mbar_wait(&S.mbar_rt, par)) { if (lane == 0) { atomicCAS(status, 0u, 100u + l); S.abort = 1; } }
                else {
                    float acc = 0.0f;
#pragma unroll 16
                    for (int j = 0; j < LKB_HIDDEN / 32; ++j) acc = fmaf(S.router[j * 32 + lane], S.h[j * 32 + lane], acc);
                    acc = lkb_warp_sum(acc);
                    if (lane == 0) S.sel[0] = acc;                   // multiplied by inv below, once inv exists
                }
            }
        }
        FUSED_STAMP(1);
        // ---- B: Q8_1 of u, ssq, inv (needed for the logit scale and for gate|up) --
        fused_quant_u(S, xv, uv);
        if (cta < LKB_N_EXPERTS && tid == 0) a.logits[cta] = __fmul_rn(S.sel[0], S.inv);
        FUSED_STAMP(2);
        grid_arrive(a.bar, S);
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 1u, a.spin_limit)) return;
        FUSED_STAMP(3);

        // ---- C: selection (every CTA, warp 0; the softmax gate takes the 64-thread path) ----
        if (!a.softmax) {
            if (warp == 0) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int e = lane + 32 * h;
                    const float lg = __ldcg(a.logits + e);
                    const float g = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg)));
                    S.sig[e] = g;
                    S.sel[e] = __fadd_rn(g, ly.rbias ? ly.rbias[e] : 0.0f);
                }
                __syncwarp();
            }
        } else {
            if (tid < LKB_N_EXPERTS) S.sel[tid] = __ldcg(a.logits + tid);
            __syncthreads();
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
        FUSED_STAMP(8);
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
        FUSED_STAMP(9);
        // ---- D: request every weight row of the layer, one issuing lane per chunk ---
        if (lane == 0) {
            fence_proxy_async();
            for (int c = warp; c < n_gu_ch + LKB_TOP_K * dn_ch_per_k; c += FUSED_WARPS) {
                if (c < n_gu_ch) {
                    const int j0 = c * CH_ROWS, j1 = min(n_gu, j0 + CH_ROWS);
                    issue_gu_rows(ly, S.idx, gu0 + j0, gu0 + j1, S.gu_q + (size_t) j0 * GU_BPR * 16,
                                  S.gu_d + (size_t) j0 * GU_BPR, &S.mbar_gu[c]);
                } else {
                    const int cc = c - n_gu_ch, k = cc / dn_ch_per_k, ch = cc % dn_ch_per_k;
                    const int j0 = ch * CH_ROWS, j1 = min(n_dn, j0 + CH_ROWS);
                    const size_t ed = (size_t) S.idx[k] * LKB_HIDDEN * DN_BPR;
                    unsigned long long * mb = &S.mbar_dn[k * dn_ch_per_k + ch];
                    mbar_expect_tx(mb, (unsigned) (j1 - j0) * DN_BPR * 18u);
                    bulk_g2s(S.dn_q + ((size_t) k * MAX_DN_ROWS + j0) * DN_BPR * 16,
                             (const uint4 *) ly.down_qs + ed + (size_t) (dn0 + j0) * DN_BPR, (unsigned) (j1 - j0) * DN_BPR * 16u, mb);
                    bulk_g2s(S.dn_d + ((size_t) k * MAX_DN_ROWS + j0) * DN_BPR,
                             (const __half *) ly.down_d + ed + (size_t) (dn0 + j0) * DN_BPR, (unsigned) (j1 - j0) * DN_BPR * 2u, mb);
                }
            }
        }
        __syncwarp();
        FUSED_STAMP(4);

        // ---- E: gate|up rows of this CTA ------------------------------------------
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
                // logical row g = (half*4 + k)*1536 + row: the stand-alone kernel's y_a | y_b layout
                if (lane == 0) a.gu[gu0 + j] = __fmul_rn(acc, ninv);
            }
        }
        FUSED_STAMP(5);
        grid_arrive(a.bar, S);
        // between arrive and wait: the next layer's router row and norm weights (static data)
        if (l + 1 < a.n_layers) {
            if (cta < LKB_N_EXPERTS && tid == 0) {
                fence_proxy_async();
                mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
                bulk_g2s(S.router, L[l + 1].router + (size_t) cta * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) nw[j] = L[l + 1].norm_w[(warp + FUSED_WARPS * j) * 32 + lane];
        }
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 2u, a.spin_limit)) return;
        FUSED_STAMP(6);

        // ---- F: SwiGLU + Q8_1 (every CTA), down rows, residual ---------------------
        {
            const int GU = LKB_TOP_K * LKB_MOE_INTER;             // 6144 = 192 blocks, 12 per warp
            float g[12], u[12], v[12], d[12], sm[12]; int q[12];
#pragma unroll
            for (int j = 0; j < 12; ++j) {
                const int i = (warp + FUSED_WARPS * j) * 32 + lane;
                g[j] = __ldcg(a.gu + i); u[j] = __ldcg(a.gu + GU + i);
            }
#pragma unroll
            for (int j = 0; j < 12; ++j) v[j] = __fmul_rn(lkb_silu(g[j]), u[j]);
            FUSED_STAMP(10);
            quantN<12>(v, q, d, sm);
#pragma unroll
            for (int j = 0; j < 12; ++j) {
                const int b = warp + FUSED_WARPS * j;
                S.xq2_q[b * 32 + lane] = (int8_t) q[j];
                if (lane == 0) {
                    const __half2 ds = __floats2half2_rn(d[j], sm[j]);
                    S.xq2_s[b] = make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
                }
            }
        }
        __syncthreads();
        FUSED_STAMP(11);
        // one output row per warp, its four expert dots interleaved
        for (int j = warp; j < n_dn; j += FUSED_WARPS) {
            bool ok = true;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) ok = ok && mbar_wait(&S.mbar_dn[k * dn_ch_per_k + j / CH_ROWS], par);
            if (!ok) { if (lane == 0) { atomicCAS(status, 0u, 300u + l); S.abort = 1; } break; }
            float acc[LKB_TOP_K];
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) {
                const unsigned char * wq = S.dn_q + ((size_t) k * MAX_DN_ROWS + j) * DN_BPR * 16;
                const __half * wd = S.dn_d + ((size_t) k * MAX_DN_ROWS + j) * DN_BPR;
                float acc_k = 0.0f;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int blk = lane + 32 * h;
                    if (blk < DN_BPR) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(wq + (size_t) blk * 16);
                        const int4 x0 = *reinterpret_cast<const int4 *>(S.xq2_q + (k * DN_BPR + blk) * 32);
                        const int4 x1 = *reinterpret_cast<const int4 *>(S.xq2_q + (k * DN_BPR + blk) * 32 + 16);
                        const int xv8[8] = { x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w };
                        const float2 sc = S.xq2_s[k * DN_BPR + blk];
                        acc_k = lkb_block_acc(__half2float(wd[blk]), sc.x, lkb_sumi(w, xv8), sc.y, acc_k);
                    }
                }
                acc[k] = acc_k;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int k = 0; k < LKB_TOP_K; ++k) acc[k] = __fadd_rn(acc[k], __shfl_xor_sync(LKB_FULL, acc[k], o));
            if (lane == 0) {
#pragma unroll
                for (int k = 0; k < LKB_TOP_K; ++k) S.dot[k][j] = acc[k];
            }
        }
        __syncthreads();
        FUSED_STAMP(12);
        if (tid < n_dn) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) acc = fmaf(S.wk[k], S.dot[k][tid], acc);
            a.x[dn0 + tid] = __fadd_rn(__ldcg(a.x + dn0 + tid), acc);
        }
        FUSED_STAMP(7);
        grid_arrive(a.bar, S);
        if (l + 1 < a.n_layers && tid < (int) (sizeof(lkb_moe_layer) / 8))
            reinterpret_cast<unsigned long long *>(&S.ly)[tid] = reinterpret_cast<const unsigned long long *>(&L[l + 1])[tid];
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 3u, a.spin_limit)) return;
    }

    // optional: the quantised, un-normalised activation of the final x for the caller's next consumer
    if (a.final_norm_w && cta == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) nw[j] = a.final_norm_w[(warp + FUSED_WARPS * j) * 32 + lane];
        float xv[4], uv[4];
        fused_load_u(S, a.x, nw, xv, uv);
        fused_quant_u(S, xv, uv);
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
    a.timing = g_fused_timing;
    a.absent_cta = g_fused_absent_cta;
    a.spin_limit = g_fused_spin_limit ? g_fused_spin_limit : SPIN_LIMIT;
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

// Tuning hook (not part of the public header): device buffer of [#CTAs][4 layers][16] clock64 stamps, or null.
__attribute__((visibility("default"))) int lkb_debug_fused_timing(unsigned long long * buf) { g_fused_timing = buf; return LKB_OK; }

// Test hook (not in the public header): the next launches run WITHOUT CTA `cta` (it returns at once), so every
// other CTA's first grid-barrier wait runs out after `spin_limit` polls and the kernel ends with a status code
// instead of hanging.  cta = -1 restores normal operation.  Nothing faults, traps or spins without a bound.
__attribute__((visibility("default"))) int lkb_debug_fused_absent_cta(int cta, unsigned spin_limit) {
    g_fused_absent_cta = cta; g_fused_spin_limit = spin_limit; return LKB_OK;
}

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

// ---------------------------------------------------------------------------
// The same stack kernel for callers that may not allocate device memory: its global scratch
// (router logits, gate|up outputs, barrier words) lives in a fixed array inside this library.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[LKB_STATIC_SCRATCH_BYTES];
static void * g_static_scratch_addr[LKB_STATIC_MAX_DEVICES] = {};     // device address of the array, per device

int lkb_moe_ffn_decode_stack_static(const lkb_moe_layer * layers_dev, int n_layers, int hidden, int inter,
                                    int n_experts, int top_k, int softmax, float * x, int * idx_out, float * w_out,
                                    const lkb_norm_prod_t * next, lkb_stream_t st) {
    if (!layers_dev) return LKB_ERR_NULL;
    if (hidden <= 0 || inter <= 0 || n_experts <= 0 || top_k <= 0) return LKB_ERR_SHAPE;
    // bytes of scratch this shape needs, laid out in 256-byte aligned pieces
    const size_t logits_b = (((size_t) n_experts * 4) + 255) & ~(size_t) 255;
    const size_t gu_b = (((size_t) 2 * top_k * inter * 4) + 255) & ~(size_t) 255;
    const size_t need = logits_b + gu_b + 256;
    if (need > (size_t) LKB_STATIC_SCRATCH_BYTES) return LKB_ERR_SCRATCH;      // larger than the built-in array
    if (hidden != LKB_HIDDEN || inter != LKB_MOE_INTER || n_experts != LKB_N_EXPERTS || top_k != LKB_TOP_K)
        return LKB_ERR_SHAPE;                                                  // the kernel is built for one shape
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return -(int) e;
    if (dev < 0 || dev >= LKB_STATIC_MAX_DEVICES) return LKB_ERR_DEVICE;
    if (!g_static_scratch_addr[dev]) {
        // First call on this device: the array's NAME is only a host-side handle; the kernel needs the
        // address the array has on the current device.
        void * p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return e != cudaSuccess ? -(int) e : LKB_ERR_DEVICE;
        g_static_scratch_addr[dev] = p;
    }
    unsigned char * base = static_cast<unsigned char *>(g_static_scratch_addr[dev]);
    FusedArgs a = {};
    a.layers = layers_dev; a.n_layers = n_layers; a.x = x; a.idx_out = idx_out; a.w_out = w_out;
    if (next && next->w) { a.final_norm_w = next->w; a.out_h32 = next->h32; a.out_yq8 = reinterpret_cast<lkb_q8blk *>(next->yq8); a.out_ssq = next->ssq; }
    a.logits = reinterpret_cast<float *>(base);
    a.gu = reinterpret_cast<float *>(base + logits_b);
    a.bar = reinterpret_cast<unsigned *>(base + logits_b + gu_b);              // zeroed by the launcher before every launch
    a.softmax = softmax;
    return fused_launch(a, (cudaStream_t) st);
}

}  // extern "C"
