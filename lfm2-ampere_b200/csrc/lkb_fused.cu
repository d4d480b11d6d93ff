// lkb_fused.cu - one persistent cooperative kernel for the batch-1 MoE FFN stack and, as its template
// variant with sequence mixers in front of every MoE layer, for all layers of a whole decode step.
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
//   * a CTA owns the gate row and the up row of the same intermediate elements, so it forms
//     silu(gate)*up itself and publishes one value per pair; every CTA then quantises the 6144
//     values it needs for its down rows;
//   * the next layer's router row is requested while the down projection runs;
//   * optional (template flag PF, lkb_decode_set_expert_prefetch; off by default): 64 otherwise idle CTAs evaluate the
//     NEXT layer's router on this layer's input, and every CTA asks for its slice of the four guessed experts to be
//     brought into L2 while the barrier after gate|up completes.  74-81% of the guesses are chosen (synthetic weights)
//     and the average CTA's gate|up wait drops by 0.4-1.0 us, but the slowest CTA's does not, and the burst of prefetch
//     requests delays the polls and loads behind it on every SM: measured 2-4% slower as a whole, hence off;
//   * whole-step variant (MIX): the mixers' weight rows are static, so they are requested a phase
//     ahead into staging the MoE phases have finished with; a conv mixer adds two grid barriers
//     per layer, an attention mixer four (see the M0..M3 phases in the kernel).
// Arithmetic per output is exactly that of the stand-alone kernels (lane-strided
// blocks, xor butterfly, fixed k = 0..3 order), so results are bit-identical to the
// five-kernel sequence.
//
// Every wait (grid barrier, mbarrier) is bounded: on expiry the CTA records a code in
// the status word and leaves; the other CTAs' waits then expire too.
#include <cooperative_groups.h>
#include "lkb_attn.cuh"

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
// Expert prefetch (optional, see the kernel): the unused second half of the `gu` scratch holds the 64 guessed logits of
// the next layer, then the guessed and the actual choices of every layer ([layer][4], integers) for the caller's hit count.
#define PF_LOGITS_OFF (LKB_TOP_K * LKB_MOE_INTER)
#define PF_MAXL       512
#define PF_GUESS_OFF  (PF_LOGITS_OFF + 128)
#define PF_REAL_OFF   (PF_GUESS_OFF + 4 * PF_MAXL)
static_assert(PF_REAL_OFF + 4 * PF_MAXL <= 2 * LKB_TOP_K * LKB_MOE_INTER, "prefetch records must fit the gu scratch");

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
    alignas(16) unsigned key[LKB_N_EXPERTS];      // order-preserving integer image of sel
    float  dot[LKB_TOP_K][MAX_DN_ROWS];
    int    idx[LKB_TOP_K];
    int    pidx[LKB_TOP_K];               // expert prefetch: the guessed choice of the next layer
    float  ppart[FUSED_WARPS];            // expert prefetch: per-warp partials of the guessed logit
    float  wk[LKB_TOP_K];
    float  inv;
    int    abort;
    unsigned bar_target;
    alignas(8) lkb_moe_layer ly;          // this layer's descriptor (staged: a global read costs ~1 us of latency)
    alignas(8) lkb_moe_layer ly_next;     // the next layer's (expert prefetch)
    alignas(8) lkb_mixer_layer mx;        // whole-step kernel: this layer's sequence-mixer descriptor
    alignas(8) unsigned long long mbar_mi, mbar_mo;   // whole-step kernel: mixer input rows / output rows staged
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
// Bring [src, src+bytes) into L2 without a destination (16-byte aligned address and size).
__device__ __forceinline__ void bulk_prefetch_l2(const void * src, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(src), "r"(bytes) : "memory");
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
// Every CTA executes the same sequence of barriers, so the k-th barrier completes when the
// counter reaches (k+1)*gridDim.x: the arrival is a fire-and-forget reduction (no returned
// ticket to wait for) and the waiter starts polling at once.
// wait returns false if it expired or another CTA reported a fault.
__device__ __forceinline__ void grid_arrive(unsigned * bar, FusedSmem & S) {
    __syncthreads();                                   // this CTA's global writes are issued
    if (threadIdx.x == 0) {
        S.bar_target += gridDim.x;
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar) : "memory");
    }
}
// One poll in flight per CTA.  (Keeping four relaxed polls in flight per CTA, a quarter of a round trip apart, was
// measured: every barrier got 0.4-0.7 us SLOWER -- 148 CTAs x 4 loads on the one L2 line delay the arriving
// reductions more than the finer sampling gains.  Sleeping 400 / 800 ns before the first poll cost 0.4 / 1.1 us
// per layer as well.)
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

// The same rows of the guessed experts of the next layer, into L2 only.
__device__ __forceinline__ void prefetch_gu_rows(const lkb_moe_layer & ly, const int * idx, int g_begin, int g_end) {
    int g = g_begin;
    while (g < g_end) {
        const int seg = g / LKB_MOE_INTER, r = g - seg * LKB_MOE_INTER;
        int n = g_end - g; if (n > LKB_MOE_INTER - r) n = LKB_MOE_INTER - r;
        const size_t blk = ((size_t) idx[seg & 3] * LKB_MOE_INTER + r) * GU_BPR;
        bulk_prefetch_l2((const uint4 *) (seg < 4 ? ly.gate_qs : ly.up_qs) + blk, (unsigned) n * GU_BPR * 16u);
        bulk_prefetch_l2((const __half *) (seg < 4 ? ly.gate_d : ly.up_d) + blk, (unsigned) n * GU_BPR * 2u);
        g += n;
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

// Tuning builds only (-DLKB_TUNING; the default build has none of it): phase timestamps (clock64 of thread 0),
// [cta][layer][32].
#ifdef LKB_TUNING
static unsigned long long * g_fused_timing = nullptr;
#endif
static int g_fused_absent_cta = -1;              // test hook, see lkb_debug_fused_absent_cta
static unsigned g_fused_spin_limit = 0;          // 0: default
static int g_fused_prefetch = 0;                 // bit 0: MoE stack, bit 1: whole-step kernel (lkb_decode_set_expert_prefetch)
#ifdef LKB_TUNING
#define FUSED_STAMP(slot) do { if (a.timing && tid == 0 && l < 4) a.timing[((size_t) cta * 4 + l) * 32 + (slot)] = clock64(); } while (0)
#define FUSED_STAMP1(slot) do { if (a.timing && tid == 32 && l < 4) a.timing[((size_t) cta * 4 + l) * 32 + (slot)] = clock64(); } while (0)
#else
#define FUSED_STAMP(slot) do { } while (0)
#define FUSED_STAMP1(slot) do { } while (0)
#endif


// Thread t holds elements 4t .. 4t+3 of a 2048-vector (one 128-bit access): a 32-element block lives in 8 adjacent
// lanes, a warp covers four blocks, the 16 warps the 64 blocks.  Quantisation and sums of squares go through
// lkb_quad_quant_ds / lkb_quad_sum, whose pairings are those of the one-element-per-lane butterfly (same bits), with
// 6 shuffles per block instead of 10 plus a redux, and a reciprocal with an exact fallback instead of 32 divisions.
__device__ __forceinline__ void load4(const float * __restrict__ p, float (&o)[4]) {
    const float4 t = reinterpret_cast<const float4 *>(p)[threadIdx.x];
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
}
// Q8_1 of the block this lane's group of 8 holds -> S.xq[tid >> 3]
__device__ __forceinline__ void quad_quant_to_xq(lkb_q8blk * xq, const float (&v)[4]) {
    const int b = threadIdx.x >> 3, l8 = threadIdx.x & 7;
    __half2 ds;
    const unsigned pk = lkb_quad_quant_ds(make_float4(v[0], v[1], v[2], v[3]), ds);
    reinterpret_cast<unsigned *>(xq[b].qs)[l8] = pk;
    if (l8 == 0) xq[b].ds = ds;
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
    float *               gu;          // scratch [2*4*1536]: silu(gate)*up of the 4*1536 pairs in its first half
    unsigned *            bar;         // scratch [2]: {barrier counter, status}
    int                   softmax;
    unsigned long long *  timing;
    int                   absent_cta;  // test hook: this CTA leaves at once and never arrives (-1: none)
    unsigned              spin_limit;  // iterations a grid-barrier wait may spin
    int                   prefetch;    // expert prefetch on
    // whole-step kernel only
    const lkb_mixer_layer * mixers;    // device array [n_layers]
    const lkb_q8blk *     xq_first;    // layer 0's normalised Q8_1 activation (lkb_rmsnorm_q8_1)
    const int *           d_pos;       // device-side position
    float                 theta;       // RoPE base
    float *               mxbuf;       // scratch [3072]: q | k | v of an attention layer, or the conv output
    float *               part;        // scratch [32][LKB_ATTN_SPLIT][LKB_ATTN_PARTW]
};

// Loads x (written by other CTAs -> L2), elements 4*tid .. +3, and forms u = x*w into S.h.
__device__ __forceinline__ void fused_load_u(FusedSmem & S, const float * __restrict__ x, const float (&nw)[4],
                                             float (&xv)[4], float (&uv)[4]) {
    const float4 t = __ldcg(reinterpret_cast<const float4 *>(x) + threadIdx.x);
    xv[0] = t.x; xv[1] = t.y; xv[2] = t.z; xv[3] = t.w;
#pragma unroll
    for (int j = 0; j < 4; ++j) uv[j] = __fmul_rn(xv[j], nw[j]);
    reinterpret_cast<float4 *>(S.h)[threadIdx.x] = make_float4(uv[0], uv[1], uv[2], uv[3]);
}
// Q8_1 of u, ssq of x, inv -> S.xq, S.ssq, S.inv (ends with a CTA barrier).
__device__ __forceinline__ void fused_quant_u(FusedSmem & S, const float (&xv)[4], const float (&uv)[4]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    quad_quant_to_xq(S.xq, uv);
    const float sq = lkb_quad_sum(__fmul_rn(xv[0], xv[0]), __fmul_rn(xv[1], xv[1]), __fmul_rn(xv[2], xv[2]), __fmul_rn(xv[3], xv[3]));
    if ((lane & 7) == 0) S.ssq[threadIdx.x >> 3] = sq;
    __syncthreads();
    if (warp == 0) {
        const float inv = lkb_norm_inv(S.ssq, lane, LKB_EPS);
        if (lane == 0) S.inv = inv;
    }
    __syncthreads();
}


// ---------------------------------------------------------------------------
// Whole-step kernel: the sequence mixers in front of every MoE FFN.
// Mixer weight rows are static, so they are requested a phase ahead of their use into staging that the
// MoE phases have finished with: input-projection rows into gu_q / gu_d, output-projection rows into
// dn_q / dn_d.  Attention staging (two cp.async stages per warp) also lives in the gu_q .. dn_d range.
// ---------------------------------------------------------------------------
typedef AtSmem<2> AtSmem2;
static_assert(sizeof(AtSmem2) <= offsetof(FusedSmem, router), "attention staging must end before the live per-layer state");
#define MIX_QKV_ROWS (LKB_HIDDEN + 2 * AT_KVH * AT_D)      // 3072 logical rows: q | k | v

// One thread: request this CTA's mixer input rows.  Conv: channels [dn0, dn0+n_dn) of B, C and X (rows ch,
// 2048+ch, 4096+ch of in_proj) -> staged rows s*n_dn + j.  Attention: logical rows [a0, a1) of q | k | v.
__device__ __forceinline__ void mix_issue_in(FusedSmem & S, const lkb_mixer_layer & mx, int dn0, int n_dn, int a0, int a1) {
    fence_proxy_async();
    if (!mx.is_attn) {
        mbar_expect_tx(&S.mbar_mi, 3u * (unsigned) n_dn * GU_BPR * 18u);
        for (int s = 0; s < 3; ++s) {
            const size_t blk = ((size_t) s * LKB_HIDDEN + dn0) * GU_BPR;
            bulk_g2s(S.gu_q + (size_t) s * n_dn * GU_BPR * 16, (const uint4 *) mx.in_qs + blk, (unsigned) n_dn * GU_BPR * 16u, &S.mbar_mi);
            bulk_g2s(S.gu_d + (size_t) s * n_dn * GU_BPR, (const __half *) mx.in_d + blk, (unsigned) n_dn * GU_BPR * 2u, &S.mbar_mi);
        }
    } else {
        mbar_expect_tx(&S.mbar_mi, (unsigned) (a1 - a0) * GU_BPR * 18u);
        unsigned char * sq = S.gu_q; __half * sd = S.gu_d;
        for (int g = a0; g < a1; ) {
            const int seg = g < LKB_HIDDEN ? 0 : (g < LKB_HIDDEN + AT_KVH * AT_D ? 1 : 2);
            const int base = seg == 0 ? 0 : (seg == 1 ? LKB_HIDDEN : LKB_HIDDEN + AT_KVH * AT_D);
            const int end = seg == 0 ? LKB_HIDDEN : (seg == 1 ? LKB_HIDDEN + AT_KVH * AT_D : MIX_QKV_ROWS);
            const int n = min(a1, end) - g;
            const void * q = seg == 0 ? mx.wq_qs : (seg == 1 ? mx.wk_qs : mx.wv_qs);
            const void * d = seg == 0 ? mx.wq_d : (seg == 1 ? mx.wk_d : mx.wv_d);
            const size_t blk = (size_t) (g - base) * GU_BPR;
            bulk_g2s(sq, (const uint4 *) q + blk, (unsigned) n * GU_BPR * 16u, &S.mbar_mi);
            bulk_g2s(sd, (const __half *) d + blk, (unsigned) n * GU_BPR * 2u, &S.mbar_mi);
            sq += (size_t) n * GU_BPR * 16; sd += (size_t) n * GU_BPR; g += n;
        }
    }
}
// One thread: request this CTA's rows [dn0, dn0+n_dn) of the mixer's output projection.
__device__ __forceinline__ void mix_issue_out(FusedSmem & S, const lkb_mixer_layer & mx, int dn0, int n_dn) {
    fence_proxy_async();
    mbar_expect_tx(&S.mbar_mo, (unsigned) n_dn * GU_BPR * 18u);
    bulk_g2s(S.dn_q, (const uint4 *) mx.out_qs + (size_t) dn0 * GU_BPR, (unsigned) n_dn * GU_BPR * 16u, &S.mbar_mo);
    bulk_g2s(S.dn_d, (const __half *) mx.out_d + (size_t) dn0 * GU_BPR, (unsigned) n_dn * GU_BPR * 2u, &S.mbar_mo);
}

template <bool MIX, bool PF>
__global__ void __launch_bounds__(FUSED_THREADS, 1) k_moe_ffn_stack(const FusedArgs a) {
    extern __shared__ __align__(128) unsigned char fused_smem_raw[];
    FusedSmem & S = *reinterpret_cast<FusedSmem *>(fused_smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nct = gridDim.x, cta = blockIdx.x;
    unsigned * status = a.bar + 1;
    if ((int) blockIdx.x == a.absent_cta) return;          // host-requested: the others' bounded waits must expire

    // static partition of the layer's rows over the CTAs (balanced, contiguous)
    // A CTA owns (expert slot k, intermediate row r) PAIRS p = k*1536 + r, i.e. the gate row and the up row of
    // the same intermediate element, so it can form silu(g)*u itself and publish one value instead of two.
    // Staging: gate rows of the pairs at [0, n_gu), their up rows at [gu_pad, gu_pad + n_gu).
    const int GU_PAIRS = LKB_TOP_K * LKB_MOE_INTER;
    const int gu0 = (int) (((long long) cta * GU_PAIRS) / nct), gu1 = (int) (((long long) (cta + 1) * GU_PAIRS) / nct);
    const int dn0 = (int) (((long long) cta * LKB_HIDDEN) / nct), dn1 = (int) (((long long) (cta + 1) * LKB_HIDDEN) / nct);
    const int n_gu = gu1 - gu0, n_dn = dn1 - dn0;
    const int gu_half_ch = (n_gu + CH_ROWS - 1) / CH_ROWS, gu_pad = gu_half_ch * CH_ROWS;
    const int n_gu_ch = 2 * gu_half_ch;
    const int dn_ch_per_k = (n_dn + CH_ROWS - 1) / CH_ROWS;

    if (tid == 0) {
        S.abort = 0;
        S.bar_target = 0u;
        for (int i = 0; i < N_GU_CH; ++i) mbar_init(&S.mbar_gu[i], 1);
        for (int i = 0; i < N_DN_CH; ++i) mbar_init(&S.mbar_dn[i], 1);
        mbar_init(&S.mbar_rt, 1);
        mbar_init(&S.mbar_mi, 1);
        mbar_init(&S.mbar_mo, 1);
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
    load4(L[0].norm_w, nw);

    if (tid < (int) (sizeof(lkb_moe_layer) / 8))
        reinterpret_cast<unsigned long long *>(&S.ly)[tid] = reinterpret_cast<const unsigned long long *>(&L[0])[tid];
    // Expert prefetch.  While layer l runs, CTAs 64..127 evaluate layer l+1's router on layer l's INPUT (the residual
    // before this layer's FFN is added: the exact input does not exist yet), every CTA ranks the 64 guesses, and once
    // its own rows of layer l have landed it asks the copy engine to bring its slice of the four guessed experts of
    // layer l+1 into L2 (no destination, nothing waits on it).  HBM is idle from there to the next selection; a right
    // guess turns the next layer's stream into L2 hits, a wrong one costs bandwidth nobody was using.  Results do
    // not depend on it: the exact selection decides what is computed.
    const bool pf = PF && a.layers != nullptr && !a.softmax && nct >= 2 * LKB_N_EXPERTS;      // PF = false: none of it is compiled in
    const bool pcta = pf && cta >= LKB_N_EXPERTS && cta < 2 * LKB_N_EXPERTS;
    float pnw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (pf && a.n_layers > 1) {
        if (tid < (int) (sizeof(lkb_moe_layer) / 8))
            reinterpret_cast<unsigned long long *>(&S.ly_next)[tid] = reinterpret_cast<const unsigned long long *>(&L[1])[tid];
        if (pcta) {
            if (tid == 0) {
                mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
                bulk_g2s(S.router, L[1].router + (size_t) (cta - LKB_N_EXPERTS) * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
            }
            load4(L[1].norm_w, pnw);
        }
    }
    if (tid < LKB_TOP_K) S.pidx[tid] = tid;
    // whole-step kernel: row ranges of the mixers, layer 0's descriptor and weight rows
    const int qa0 = (int) (((long long) cta * MIX_QKV_ROWS) / nct), qa1 = (int) (((long long) (cta + 1) * MIX_QKV_ROWS) / nct);
    int pos = 0;
    float anw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if constexpr (MIX) {
        pos = __ldg(a.d_pos);
        if (tid < (int) (sizeof(lkb_mixer_layer) / 8))
            reinterpret_cast<unsigned long long *>(&S.mx)[tid] = reinterpret_cast<const unsigned long long *>(&a.mixers[0])[tid];
    }
    __syncthreads();
    if constexpr (MIX) {
        // KV capacity: an attention layer whose descriptor states max_seq refuses a position past its cache.  Every CTA
        // evaluates the same test before anything is in flight, so all leave together (status 600 + layer).
        int over = -1;
        for (int l = tid; l < a.n_layers; l += blockDim.x)
            if (a.mixers[l].is_attn && a.mixers[l].max_seq > 0 && pos >= a.mixers[l].max_seq) over = l;
        if (__syncthreads_or(over >= 0)) {
            if (over >= 0) atomicCAS(status, 0u, 600u + (unsigned) over);
            return;
        }
        if (tid == 0) {
            mix_issue_in(S, S.mx, dn0, n_dn, qa0, qa1);
            if (!S.mx.is_attn) mix_issue_out(S, S.mx, dn0, n_dn);
        }
    }

    for (int l = 0; l < a.n_layers; ++l) {
        const lkb_moe_layer & ly = S.ly;
        const unsigned par = (unsigned) (l & 1);
        const bool pf_next = pf && l + 1 < a.n_layers;              // a next layer to guess for

        if constexpr (MIX) {
            const lkb_mixer_layer & mx = S.mx;
            const bool is_attn = mx.is_attn != 0;
            FUSED_STAMP(16);
            // conv state of this CTA's channels, requested before anything waits
            float2 cv_h = make_float2(0.0f, 0.0f); float cv_w0 = 0.0f, cv_w1 = 0.0f, cv_w2 = 0.0f;
            if (!is_attn && tid < n_dn) {
                const int ch = dn0 + tid;
                cv_h = *reinterpret_cast<const float2 *>(mx.hist + 2 * ch);
                cv_w0 = __ldg(mx.conv_w + 3 * ch); cv_w1 = __ldg(mx.conv_w + 3 * ch + 1); cv_w2 = __ldg(mx.conv_w + 3 * ch + 2);
            }
            // ---- M0: the mixer's input activation: layer 0 arrives normalised and quantised; later layers
            //          quantise raw u = x * attn_norm_w and carry 1/rms into the consumer (S.inv) ----
            if (l == 0) {
                for (int i = tid; i < LKB_HIDDEN / 32 * 9; i += FUSED_THREADS)
                    reinterpret_cast<int *>(S.xq)[i] = reinterpret_cast<const int *>(a.xq_first)[i];
                if (tid == 0) S.inv = 1.0f;
                __syncthreads();
            } else {
                float xv[4], uv[4];
                fused_load_u(S, a.x, anw, xv, uv);
                fused_quant_u(S, xv, uv);
            }
            FUSED_STAMP(17);
            // ---- M1: input projection rows of this CTA (staged a phase ago) ----
            {
                int xq[2][8]; float d8[2], s8[2];
                load_xregs<2>(S.xq, GU_BPR, lane, xq, d8, s8);
                const float ninv = S.inv;
                const int nrows = is_attn ? (qa1 - qa0) : 3 * n_dn;
                float * mixv = &S.dot[0][0];
                if (!mbar_wait(&S.mbar_mi, par)) { if (lane == 0) { atomicCAS(status, 0u, 400u + l); S.abort = 1; } }
                else {
                    for (int j = warp; j < nrows; j += FUSED_WARPS) {
                        const float acc = lkb_warp_sum(smem_row_partial<2>(S.gu_q + (size_t) j * GU_BPR * 16, S.gu_d + (size_t) j * GU_BPR,
                                                                           GU_BPR, lane, xq, d8, s8));
                        if (lane == 0) {
                            const float v = __fmul_rn(acc, ninv);
                            if (is_attn) a.mxbuf[qa0 + j] = v; else mixv[j] = v;
                        }
                    }
                }
                if (!is_attn) {
                    // short convolution on this CTA's channels: B, C, X of a channel are rows j, n_dn + j, 2 n_dn + j
                    __syncthreads();
                    if (tid < n_dn) {
                        const int ch = dn0 + tid;
                        const float bx = __fmul_rn(mixv[tid], mixv[2 * n_dn + tid]);
                        const float conv = fmaf(bx, cv_w2, fmaf(cv_h.y, cv_w1, __fmul_rn(cv_h.x, cv_w0)));
                        *reinterpret_cast<float2 *>(mx.hist + 2 * ch) = make_float2(cv_h.y, bx);
                        a.mxbuf[ch] = __fmul_rn(mixv[n_dn + tid], conv);
                    }
                }
            }
            FUSED_STAMP(18);
            grid_arrive(a.bar, S);
            if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 4u, a.spin_limit)) return;
            FUSED_STAMP(19);
            const int seq_len = pos + 1;
            if (is_attn) {
                // ---- M2: one slice of one KV head per CTA; the query heads' norm + rotation are redone by every
                //          slice, the new K / V row is written by the slice that contains it (the last one) ----
                const int nsl = at_slices(seq_len), chunk = at_chunk(seq_len, nsl);
                const int kvh = cta & (AT_KVH - 1), sp = cta >> 3;
                const int t0 = sp * chunk, t1 = min(t0 + chunk, seq_len);
                if (sp < nsl && t0 < t1) {                                  // CTA-uniform
                    AtSmem2 & A = *reinterpret_cast<AtSmem2 *>(fused_smem_raw);
                    __half * kc = reinterpret_cast<__half *>(mx.kc), * vc = reinterpret_cast<__half *>(mx.vc);
                    if (warp < AT_GQA) {
                        const float * qh = a.mxbuf + (size_t) (kvh * AT_GQA + warp) * AT_D;
                        float y0, y1;
                        at_norm_rope(__ldcg(qh + lane), __ldcg(qh + lane + 32), mx.qnorm, (float) pos, a.theta, lane, y0, y1);
                        reinterpret_cast<float *>(&A.q[lane])[warp] = y0;
                        reinterpret_cast<float *>(&A.q[lane + 32])[warp] = y1;
                    } else if (warp == AT_GQA && t1 == seq_len) {
                        const float * kh = a.mxbuf + LKB_HIDDEN + (size_t) kvh * AT_D;
                        const float * vh = a.mxbuf + LKB_HIDDEN + AT_KVH * AT_D + (size_t) kvh * AT_D;
                        float y0, y1;
                        at_norm_rope(__ldcg(kh + lane), __ldcg(kh + lane + 32), mx.knorm, (float) pos, a.theta, lane, y0, y1);
                        const size_t off = ((size_t) pos * AT_KVH + kvh) * AT_D;
                        kc[off + lane] = __float2half(y0); kc[off + lane + 32] = __float2half(y1);
                        vc[off + lane] = __float2half(__ldcg(vh + lane)); vc[off + lane + 32] = __float2half(__ldcg(vh + lane + 32));
                        __threadfence();
                    }
                    __syncthreads();
                    at_slice<2>(A, kc, vc, kvh, sp, t0, t1, a.part);
                }
                FUSED_STAMP(20);
                grid_arrive(a.bar, S);
                if (tid == 32) mix_issue_out(S, mx, dn0, n_dn);             // the attention staging is idle again
                if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 5u, a.spin_limit)) return;
                FUSED_STAMP(21);
                // merge of the slices: one head per CTA (every CTA reading every partial would cost 150 KB of
                // L2 sectors per CTA), published through mxbuf like a conv output
                if (cta < AT_HEADS && tid < AT_D) a.mxbuf[cta * AT_D + tid] = at_combine(a.part, cta, tid, seq_len);
                grid_arrive(a.bar, S);
                if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 7u, a.spin_limit)) return;
                FUSED_STAMP(25);
            }
            // ---- M3: the mixer's 2048 outputs, written by their owner CTAs, quantised by every CTA; then this CTA's output-projection rows, added to the residual ----
            {
                const float4 o4 = __ldcg(reinterpret_cast<const float4 *>(a.mxbuf) + tid);
                const float o[4] = {o4.x, o4.y, o4.z, o4.w};
                quad_quant_to_xq(S.xq, o);
                __syncthreads();
                FUSED_STAMP(22);
                int xq[2][8]; float d8[2], s8[2];
                load_xregs<2>(S.xq, GU_BPR, lane, xq, d8, s8);
                if (!mbar_wait(&S.mbar_mo, par)) { if (lane == 0) { atomicCAS(status, 0u, 500u + l); S.abort = 1; } }
                else {
                    for (int j = warp; j < n_dn; j += FUSED_WARPS) {
                        const float acc = lkb_warp_sum(smem_row_partial<2>(S.dn_q + (size_t) j * GU_BPR * 16, S.dn_d + (size_t) j * GU_BPR,
                                                                           GU_BPR, lane, xq, d8, s8));
                        if (lane == 0) a.x[dn0 + j] = __fadd_rn(__ldcg(a.x + dn0 + j), acc);
                    }
                }
            }
            FUSED_STAMP(23);
            grid_arrive(a.bar, S);
            if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 6u, a.spin_limit)) return;
            FUSED_STAMP(24);
        }

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
        } else if (pcta && pf_next) {
            // the next layer's router row (cta - 64) against this layer's input under the next layer's norm weights
            if (!mbar_wait(&S.mbar_rt, par)) { if (lane == 0) { atomicCAS(status, 0u, 100u + l); S.abort = 1; } }
            else {
                float acc = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    acc = fmaf(S.router[tid * 4 + j], __fmul_rn(xv[j], pnw[j]), acc);
                acc = lkb_warp_sum(acc);
                if (lane == 0) S.ppart[warp] = acc;
            }
        }
        FUSED_STAMP(1);
        // ---- B: Q8_1 of u, ssq, inv (needed for the logit scale and for gate|up) --
        fused_quant_u(S, xv, uv);
        if (cta < LKB_N_EXPERTS && tid == 0) a.logits[cta] = __fmul_rn(S.sel[0], S.inv);
        if (pcta && pf_next && tid == 0) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < FUSED_WARPS; ++w) acc += S.ppart[w];
            a.gu[PF_LOGITS_OFF + cta - LKB_N_EXPERTS] = acc * S.inv;
        }
        FUSED_STAMP(2);
        grid_arrive(a.bar, S);
        // static data of the selection, fetched while the barrier completes
        float rb0 = 0.0f, rb1 = 0.0f;
        if (warp == 0 && ly.rbias) { rb0 = __ldg(ly.rbias + lane); rb1 = __ldg(ly.rbias + lane + 32); }
        float prb0 = 0.0f, prb1 = 0.0f, plg0 = 0.0f, plg1 = 0.0f;
        if (pf_next && warp == 1 && S.ly_next.rbias) { prb0 = __ldg(S.ly_next.rbias + lane); prb1 = __ldg(S.ly_next.rbias + lane + 32); }
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 1u, a.spin_limit)) return;
        FUSED_STAMP(3);

        // the guessed logits of the next layer: requested here, used by warp 1 once the gate|up rows are done
        if (pf_next && warp == 1) { plg0 = __ldcg(a.gu + PF_LOGITS_OFF + lane); plg1 = __ldcg(a.gu + PF_LOGITS_OFF + lane + 32); }
        // ---- C: selection (every CTA, warp 0; the softmax gate takes the 64-thread path) ----
        if (!a.softmax) {
            if (warp == 0) {
                // both logits are requested before either is used: a shared-memory store between two global
                // loads would serialise them (the compiler cannot prove the pointers distinct)
                const float lg0 = __ldcg(a.logits + lane), lg1 = __ldcg(a.logits + lane + 32);
                const float g0 = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg0)));
                const float g1 = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-lg1)));
                S.sig[lane] = g0; S.sig[lane + 32] = g1;
                const float s0 = __fadd_rn(g0, rb0), s1 = __fadd_rn(g1, rb1);
                S.sel[lane] = s0; S.sel[lane + 32] = s1;
                S.key[lane] = lkb_orderable(s0); S.key[lane + 32] = lkb_orderable(s1);
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
            if (tid < LKB_N_EXPERTS) {
                const float sv = __fadd_rn(pn, ly.rbias ? ly.rbias[tid] : 0.0f);
                S.sig[tid] = pn; S.sel[tid] = sv; S.key[tid] = lkb_orderable(sv);
            }
        }
        FUSED_STAMP(8);
        // Top-4 by rank counting over the whole CTA: expert e's rank is the number of experts that beat it
        // ("greater value wins, equal value -> lower index", ref: src/kernels.cuh:515-541); the experts of rank
        // 0..3 are the selection, in rank order.  Thread t compares expert t>>3 with experts (t&7)*8 .. +7 and the
        // eight partial counts are summed by shuffles: no serial rounds.  Same winners as lkb_router_select.
        __syncthreads();                                            // keys of all 64 experts are in S.key
        {
            const int e = tid >> 3, j0 = (tid & 7) * 8;
            const unsigned ke = S.key[e];
            const uint4 ka = *reinterpret_cast<const uint4 *>(&S.key[j0]), kb = *reinterpret_cast<const uint4 *>(&S.key[j0 + 4]);
            const unsigned kj[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
            int cnt = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) cnt += (kj[i] > ke || (kj[i] == ke && j0 + i < e)) ? 1 : 0;
            cnt += __shfl_xor_sync(LKB_FULL, cnt, 1);
            cnt += __shfl_xor_sync(LKB_FULL, cnt, 2);
            cnt += __shfl_xor_sync(LKB_FULL, cnt, 4);
            if ((tid & 7) == 0 && cnt < LKB_TOP_K) S.idx[cnt] = e;
        }
        __syncthreads();
        FUSED_STAMP(13);
        if (warp == 0 && lane == 0) {
            // weights: unbiased gate values of the winners, renormalised (sum clamped), in rank order
            float wv[LKB_TOP_K], wsum = 0.0f;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) { wv[k] = S.sig[S.idx[k]]; wsum = __fadd_rn(wsum, wv[k]); }
            if (wsum < LKB_TOPK_GUARD) wsum = LKB_TOPK_GUARD;
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) { wv[k] = __fdiv_rn(wv[k], wsum); S.wk[k] = wv[k]; }
            if (cta == 0) {
#pragma unroll
                for (int k = 0; k < LKB_TOP_K; ++k) {
                    if (a.idx_out) a.idx_out[l * 4 + k] = S.idx[k];
                    if (a.w_out) a.w_out[l * 4 + k] = wv[k];
                    if (pf && l < PF_MAXL) a.gu[PF_REAL_OFF + l * 4 + k] = __int_as_float(S.idx[k]);
                }
            }
        }
        FUSED_STAMP(9);
        // ---- D: request every weight row of the layer, one issuing lane per chunk ---
        if (lane == 0) {
            fence_proxy_async();
            for (int c = warp; c < n_gu_ch + LKB_TOP_K * dn_ch_per_k; c += FUSED_WARPS) {
                if (c < n_gu_ch) {
                    const int up = c >= gu_half_ch, ch = up ? c - gu_half_ch : c;
                    const int j0 = ch * CH_ROWS, j1 = min(n_gu, j0 + CH_ROWS);
                    const int g0 = up * GU_PAIRS + gu0, s0 = up * gu_pad + j0;       // logical rows: gate 0..6143, up 6144..12287
                    issue_gu_rows(ly, S.idx, g0 + j0, g0 + j1, S.gu_q + (size_t) s0 * GU_BPR * 16,
                                  S.gu_d + (size_t) s0 * GU_BPR, &S.mbar_gu[c]);
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

        // ---- E: gate and up rows of this CTA's pairs, silu(gate)*up published -----
        {
            int xq[2][8]; float d8[2], s8[2];
            load_xregs<2>(S.xq, GU_BPR, lane, xq, d8, s8);
            const float ninv = S.inv;
            for (int j = warp; j < n_gu; j += FUSED_WARPS) {
                // both probes are issued before either answer is used (a probe takes ~0.1 us even when the rows are there)
                unsigned long long * const mg = &S.mbar_gu[j / CH_ROWS], * const mu = &S.mbar_gu[gu_half_ch + j / CH_ROWS];
                const bool hg = mbar_try_wait(mg, par), hu = mbar_try_wait(mu, par);
                if (__any_sync(LKB_FULL, (!hg && !mbar_wait(mg, par)) || (!hu && !mbar_wait(mu, par)))) {
                    if (lane == 0) { atomicCAS(status, 0u, 200u + l); S.abort = 1; }
                    break;
                }
                float pg = smem_row_partial<2>(S.gu_q + (size_t) j * GU_BPR * 16, S.gu_d + (size_t) j * GU_BPR, GU_BPR, lane, xq, d8, s8);
                float pu = smem_row_partial<2>(S.gu_q + (size_t) (gu_pad + j) * GU_BPR * 16, S.gu_d + (size_t) (gu_pad + j) * GU_BPR,
                                               GU_BPR, lane, xq, d8, s8);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    pg = __fadd_rn(pg, __shfl_xor_sync(LKB_FULL, pg, o));
                    pu = __fadd_rn(pu, __shfl_xor_sync(LKB_FULL, pu, o));
                }
                // v = silu(gate) * up of pair gu0 + j (the stand-alone k_swiglu's arithmetic on the two GEMV outputs)
                if (lane == 0) a.gu[gu0 + j] = __fmul_rn(lkb_silu(__fmul_rn(pg, ninv)), __fmul_rn(pu, ninv));
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
            load4(L[l + 1].norm_w, nw);
            if constexpr (MIX) {
                // gate|up staging is idle from here to the next layer's selection: the next mixer's input rows
                if (tid == 32) mix_issue_in(S, a.mixers[l + 1], dn0, n_dn, qa0, qa1);   // not thread 0: it polls the barrier
                load4(a.mixers[l + 1].attn_norm, anw);
            }
        }
        if (pf_next && warp > 0) {
            // Warps 1..15, inside this barrier's shadow (warp 0 polls).  First the router row of the layer after next.
            FUSED_STAMP1(26);
            if (pcta && l + 2 < a.n_layers && tid == 32) {
                fence_proxy_async();
                mbar_expect_tx(&S.mbar_rt, LKB_HIDDEN * 4);
                bulk_g2s(S.router, L[l + 2].router + (size_t) (cta - LKB_N_EXPERTS) * LKB_HIDDEN, LKB_HIDDEN * 4, &S.mbar_rt);
            }
            // rank the 64 guesses by the rule of the selection: warp 1 forms the keys, thread e counts who beats expert e
            if (warp <= 2) {
                if (warp == 1) {
                    S.key[lane] = lkb_orderable(__fadd_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-plg0))), prb0));
                    S.key[lane + 32] = lkb_orderable(__fadd_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-plg1))), prb1));
                }
                asm volatile("bar.sync 2, 64;" ::: "memory");
                const int e = tid - 32;
                const unsigned ke = S.key[e];
                int cnt = 0;
#pragma unroll 4
                for (int j = 0; j < LKB_N_EXPERTS; j += 4) {
                    const uint4 kk = *reinterpret_cast<const uint4 *>(&S.key[j]);
                    const unsigned kj[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) cnt += (kj[i] > ke || (kj[i] == ke && j + i < e)) ? 1 : 0;
                }
                if (cnt < LKB_TOP_K) S.pidx[cnt] = e;
            }
            FUSED_STAMP1(27);
            asm volatile("bar.sync 1, %0;" :: "r"(FUSED_THREADS - 32) : "memory");
            // this CTA's gate|up rows of layer l have landed: its slice of the guessed experts of layer l+1 goes to L2,
            // in the chunks of the real request, one or two per issuing lane
            if (lane == 0) {
                const lkb_moe_layer & nx = S.ly_next;
                for (int c = warp - 1; c < n_gu_ch + LKB_TOP_K * dn_ch_per_k; c += FUSED_WARPS - 1) {
                    if (c < n_gu_ch) {
                        const int up = c >= gu_half_ch, ch = up ? c - gu_half_ch : c;
                        const int j0 = ch * CH_ROWS, j1 = min(n_gu, j0 + CH_ROWS);
                        prefetch_gu_rows(nx, S.pidx, up * GU_PAIRS + gu0 + j0, up * GU_PAIRS + gu0 + j1);
                    } else {
                        const int cc = c - n_gu_ch, k = cc / dn_ch_per_k, ch = cc % dn_ch_per_k;
                        const int j0 = ch * CH_ROWS, j1 = min(n_dn, j0 + CH_ROWS);
                        const size_t blk = (size_t) S.pidx[k] * LKB_HIDDEN * DN_BPR + (size_t) (dn0 + j0) * DN_BPR;
                        bulk_prefetch_l2((const uint4 *) nx.down_qs + blk, (unsigned) (j1 - j0) * DN_BPR * 16u);
                        bulk_prefetch_l2((const __half *) nx.down_d + blk, (unsigned) (j1 - j0) * DN_BPR * 2u);
                    }
                }
            }
            if (cta == 0 && warp == 1 && lane < LKB_TOP_K && l + 1 < PF_MAXL)
                a.gu[PF_GUESS_OFF + (l + 1) * 4 + lane] = __int_as_float(S.pidx[lane]);
            FUSED_STAMP1(29);
        }
        if (pf_next && pcta && l + 2 < a.n_layers) {
            load4(L[l + 2].norm_w, pnw);
        }
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 2u, a.spin_limit)) return;
        FUSED_STAMP(6);

        // ---- F: Q8_1 of the 6144 published values (every CTA), down rows, residual --
        {
            // 192 blocks, four per warp step (lane l holds elements 4(l&7).. of block l>>3): three 128-bit loads per
            // lane; same quants, scale and raw sum as the one-element-per-lane form (lkb_quad_quant)
            float4 v[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) v[j] = __ldcg(reinterpret_cast<const float4 *>(a.gu) + (warp + FUSED_WARPS * j) * 32 + lane);
            FUSED_STAMP(10);
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                float2 sc;
                const unsigned pk = lkb_quad_quant(v[j], lane, sc);
                const int b = (warp + FUSED_WARPS * j) * 4 + (lane >> 3);
                reinterpret_cast<unsigned *>(S.xq2_q)[b * 8 + (lane & 7)] = pk;
                if ((lane & 7) == 0) S.xq2_s[b] = sc;
            }
        }
        __syncthreads();
        FUSED_STAMP(11);
        // one output row per warp, its four expert dots interleaved
        for (int j = warp; j < n_dn; j += FUSED_WARPS) {
            bool here[LKB_TOP_K], ok = true;                        // four probes in flight, then the bounded waits if needed
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) here[k] = mbar_try_wait(&S.mbar_dn[k * dn_ch_per_k + j / CH_ROWS], par);
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) ok = ok && (here[k] || mbar_wait(&S.mbar_dn[k * dn_ch_per_k + j / CH_ROWS], par));
            ok = __all_sync(LKB_FULL, ok);                          // the shuffles below need the whole warp
            if (!ok) { if (lane == 0) { atomicCAS(status, 0u, 300u + l); S.abort = 1; } break; }
            FUSED_STAMP(15);
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
            FUSED_STAMP(14);
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
        if (pf && l + 2 < a.n_layers && tid >= 32 && tid < 32 + (int) (sizeof(lkb_moe_layer) / 8))
            reinterpret_cast<unsigned long long *>(&S.ly_next)[tid - 32] = reinterpret_cast<const unsigned long long *>(&L[l + 2])[tid - 32];
        if constexpr (MIX) {
            if (l + 1 < a.n_layers) {
                if (tid < (int) (sizeof(lkb_mixer_layer) / 8))
                    reinterpret_cast<unsigned long long *>(&S.mx)[tid] = reinterpret_cast<const unsigned long long *>(&a.mixers[l + 1])[tid];
                // down staging is idle until the next layer's selection: a conv mixer's output rows
                if (tid == 32 && !a.mixers[l + 1].is_attn) mix_issue_out(S, a.mixers[l + 1], dn0, n_dn);
            }
        }
        if (!grid_wait(a.bar, status, S, 1000u + 10u * l + 3u, a.spin_limit)) return;
    }

    // optional: the quantised, un-normalised activation of the final x for the caller's next consumer
    if (a.final_norm_w && cta == 0) {
        load4(a.final_norm_w, nw);
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
    const void * kernels[4] = {(const void *) k_moe_ffn_stack<false, false>, (const void *) k_moe_ffn_stack<false, true>,
                               (const void *) k_moe_ffn_stack<true, false>, (const void *) k_moe_ffn_stack<true, true>};
    for (const void * k : kernels) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(FusedSmem));
        if (e != cudaSuccess) return -(int) e;
    }
    g_fused_ready = 1;
    return LKB_OK;
}

static int fused_launch(FusedArgs & a, cudaStream_t st) {
    if (!lkb_context().inited || !g_fused_ready) return LKB_ERR_NOT_INIT;
    if (!a.x || !a.logits || !a.gu || !a.bar) return LKB_ERR_NULL;
    if (a.n_layers <= 0) return LKB_ERR_SHAPE;
    if (a.final_norm_w && (!a.out_yq8 || !a.out_ssq)) return LKB_ERR_NULL;
    // the residual, the norm weights and the scratch vectors are read 128 bits at a time
    auto misaligned = [](const void * p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) != 0; };
    if (misaligned(a.x) || misaligned(a.gu) || misaligned(a.final_norm_w) || misaligned(a.mxbuf) ||
        (!a.layers && misaligned(a.one.norm_w))) return LKB_ERR_SHAPE;
    int grid = lkb_context().sm_count;
    // every CTA's share must fit the shared-memory staging
    const int pairs = (LKB_TOP_K * LKB_MOE_INTER + grid - 1) / grid;          // gate rows, then (chunk-aligned) as many up rows
    if ((pairs + CH_ROWS - 1) / CH_ROWS * CH_ROWS + pairs > MAX_GU_ROWS || 2 * ((pairs + CH_ROWS - 1) / CH_ROWS) > N_GU_CH ||
        (LKB_HIDDEN + grid - 1) / grid > MAX_DN_ROWS) return LKB_ERR_DEVICE;
    cudaError_t e = cudaMemsetAsync(a.bar, 0, 2 * sizeof(unsigned), st);
    if (e != cudaSuccess) return -(int) e;
#ifdef LKB_TUNING
    a.timing = g_fused_timing;
#else
    a.timing = nullptr;
#endif
    a.absent_cta = g_fused_absent_cta;
    a.spin_limit = g_fused_spin_limit ? g_fused_spin_limit : SPIN_LIMIT;
    a.prefetch = (g_fused_prefetch >> (a.mixers ? 1 : 0)) & 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(FUSED_THREADS); cfg.dynamicSmemBytes = sizeof(FusedSmem); cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (a.mixers) e = a.prefetch ? cudaLaunchKernelEx(&cfg, k_moe_ffn_stack<true, true>, a) : cudaLaunchKernelEx(&cfg, k_moe_ffn_stack<true, false>, a);
    else          e = a.prefetch ? cudaLaunchKernelEx(&cfg, k_moe_ffn_stack<false, true>, a) : cudaLaunchKernelEx(&cfg, k_moe_ffn_stack<false, false>, a);
    if (e != cudaSuccess) { (void) cudaGetLastError(); return -(int) e; }
    return LKB_OK;
}

extern "C" {

#ifdef LKB_TUNING
// Tuning hook (not part of the public header): device buffer of [#CTAs][4 layers][32] clock64 stamps, or null.
__attribute__((visibility("default"))) int lkb_debug_fused_timing(unsigned long long * buf) { g_fused_timing = buf; return LKB_OK; }
#endif

// Test hook (not in the public header): the next launches run WITHOUT CTA `cta` (it returns at once), so every
// other CTA's first grid-barrier wait runs out after `spin_limit` polls and the kernel ends with a status code
// instead of hanging.  cta = -1 restores normal operation.  Nothing faults, traps or spins without a bound.
__attribute__((visibility("default"))) int lkb_debug_fused_absent_cta(int cta, unsigned spin_limit) {
    g_fused_absent_cta = cta; g_fused_spin_limit = spin_limit; return LKB_OK;
}

int lkb_decode_set_expert_prefetch(int mode) {
    if (mode < 0 || mode > 3) return LKB_ERR_SHAPE;
    g_fused_prefetch = mode;
    return LKB_OK;
}

int lkb_decode_expert_prefetch_hits(const lkb_moe_scratch * scratch, int n_layers, int * hits, int * guesses, lkb_stream_t st) {
    if (!scratch || !scratch->gu || !hits || !guesses) return LKB_ERR_NULL;
    if (n_layers < 2) return LKB_ERR_SHAPE;
    const int nl = n_layers < PF_MAXL ? n_layers : PF_MAXL;
    static int rec[2][4 * PF_MAXL];
    cudaError_t e = cudaStreamSynchronize((cudaStream_t) st);
    if (e == cudaSuccess) e = cudaMemcpy(rec[0], scratch->gu + PF_GUESS_OFF, sizeof(int) * 4 * nl, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(rec[1], scratch->gu + PF_REAL_OFF, sizeof(int) * 4 * nl, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return -(int) e;
    int h = 0;
    for (int l = 1; l < nl; ++l)
        for (int i = 0; i < 4; ++i)
            for (int j = 0; j < 4; ++j) h += rec[0][l * 4 + i] == rec[1][l * 4 + j];
    *hits = h; *guesses = 4 * (nl - 1);
    return LKB_OK;
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

int lkb_decode_layers(const lkb_moe_layer * moe_dev, const lkb_mixer_layer * mixers_dev, int n_layers, float * x,
                      const lkb_block_q8_1 * xq_first, const int * d_pos, float theta, const lkb_norm_prod_t * next,
                      const lkb_moe_scratch * scratch, const lkb_step_scratch * step_scratch, lkb_stream_t st) {
    if (!moe_dev || !mixers_dev || !scratch || !step_scratch || !xq_first || !d_pos) return LKB_ERR_NULL;
    if (!step_scratch->mx || !step_scratch->part) return LKB_ERR_NULL;
    if (!(theta > 1.0f)) return LKB_ERR_SHAPE;
    FusedArgs a = {};
    a.layers = moe_dev; a.n_layers = n_layers; a.x = x;
    if (next && next->w) { a.final_norm_w = next->w; a.out_h32 = next->h32; a.out_yq8 = reinterpret_cast<lkb_q8blk *>(next->yq8); a.out_ssq = next->ssq; }
    a.logits = scratch->logits; a.gu = scratch->gu; a.bar = scratch->sync; a.softmax = 0;
    a.mixers = mixers_dev; a.xq_first = reinterpret_cast<const lkb_q8blk *>(xq_first); a.d_pos = d_pos; a.theta = theta;
    a.mxbuf = step_scratch->mx; a.part = step_scratch->part;
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

// The status word of the built-in scratch: what `scratch->sync[1]` is for the allocating entry point.  Copies four bytes
// out of the library's array with cudaMemcpyFromSymbol; allocates nothing.
int lkb_moe_ffn_decode_stack_static_status(void) {
    const size_t logits_b = (((size_t) LKB_N_EXPERTS * 4) + 255) & ~(size_t) 255;
    const size_t gu_b = (((size_t) 2 * LKB_TOP_K * LKB_MOE_INTER * 4) + 255) & ~(size_t) 255;
    unsigned v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_static_scratch, sizeof v, logits_b + gu_b + sizeof(unsigned)) != cudaSuccess) return -1;
    return (int) v;
}

}  // extern "C"
