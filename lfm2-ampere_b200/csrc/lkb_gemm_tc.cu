// lkb_gemm_tc.cu - tensor-core form of the Q4_0 x Q8_1 grouped GEMM for sm_100a:
// tcgen05.mma.kind::i8 with accumulators in tensor memory (TMEM).
//
//   out[slot][n] (+)= scale[arow] * sum_{b ascending} fma(d4[n][b], fma(d8[arow][b], float(S_b), -8sum[arow][b]), .)
//   S_b = sum_{i<32} nibble[n][b][i] * q8[arow][b][i]                     (int32, exact)
//
// One MMA per 32-element block: K = 32 int8 is exactly one Q4_0/Q8_1 block, and the
// per-block scales forbid accumulating across blocks inside the tensor core, so every
// block's 128x128 int32 result is read back from TMEM and folded into fp32 register
// accumulators by the CUDA cores (2 FMA + 1 convert per value).  That epilogue, not
// the MMA, bounds the kernel (MMA ~64 clk per block per SM, epilogue >= 256), so the
// design spends the SM on it:
//   * M (TMEM lanes) = 128 tokens, N (TMEM columns) = 128 weight rows.  A thread owns one
//     token: d8 / 8sum are per-thread scalars, the 32 intermediate rows of a Q8_1 output
//     block sit in 32 registers of one thread, so the SwiGLU epilogue quantises with no
//     shuffle at all (in the standard butterfly order: bit-identical to the unfused path);
//   * two loader warps (cp.async, two stages ahead): activations are gathered through `perm`
//     straight into the canonical K-major core-matrix layout (8 rows x 16 B), nibbles are staged
//     raw and expanded to int8 from shared memory; one thread of a warp of its own issues the MMAs;
//     sixteen epilogue warps (four per TMEM lane quadrant, 32 columns each);
//   * four TMEM buffers of 128 columns: MMAs run up to four blocks ahead of the epilogue;
//   * persistent: one CTA per SM walks (row tile, 128-token tile) work items built from
//     the device-side tile list, expert by expert, so an expert's weights stay in L2.
// Every wait is bounded; on expiry a status word is set and all roles drain and exit,
// freeing TMEM.
#include "lkb_device.cuh"

#ifndef TC_LW
#define TC_LW        2              // loader warps; each loader thread serves TC_RPT tokens and TC_RPT weight rows
#endif
#define TC_RPT       (128 / (32 * TC_LW))
#ifndef TC_SUSPEND_NS
#define TC_SUSPEND_NS 0             // > 0: suspend-time hint (ns) on every mbarrier wait; 2000 measured 4% slower (65.6 against 63.3 ms)
#endif
#ifndef TC_LAYOUT
#define TC_LAYOUT 1                   // measured: 65.1 ms per 40-layer 4k-token step with layout 0, 63.0 ms with layout 1
#endif
// Which warp plays which role.  A warp's scheduler is warp % 4, and that is also the TMEM lane quadrant an epilogue
// warp may read, so every scheduler carries four epilogue warps whatever the layout; the layouts differ in which
// schedulers ALSO carry a loader warp.  0: loaders are warps 0, 1 (schedulers 0, 1), epilogue 2..17, issuer 18.
// 1: epilogue 0..15, issuer 16, warp 17 idle, loaders 18, 19 (schedulers 2, 3: the quadrants that hold the
//    padding rows of a partly filled token tile, whose epilogue warps have the least to do).
#if TC_LAYOUT == 1
#define TC_THREADS   (20 * 32)
#define TC_LOADER_W0 (20 - TC_LW)
#define TC_EPI_W0    0
#define TC_MMA_WARP  16
#else
#define TC_THREADS   ((TC_LW + 16 + 1) * 32)   // loaders, 16 epilogue warps, 1 MMA-issuing warp
#define TC_LOADER_W0 0
#define TC_EPI_W0    TC_LW
#define TC_MMA_WARP  (TC_LW + 16)
#endif
#define TC_LOADERS   (32 * TC_LW)
#define TC_EPI_WARPS 16
#define TC_KB        4              // blocks per pipeline stage
#define TC_STAGES    3
#define TC_TBUF      4              // TMEM buffers (128 columns each)
#define TC_M         128            // tokens per tile
#define TC_N         128            // weight rows (columns of D) per MMA
#define TC_AHEAD     2              // stages of cp.async lookahead in the loaders
#define TC_SPIN      (1u << 24)
#define TC_MAX_TILES 1024           // 64-token plan tiles the work list can hold
// Epilogue shape switches (defaults = the fastest measured on B200; the others are kept for ablation):
#ifndef TC_LD8
#define TC_LD8 1                     // 1: TMEM is read 8 columns at a time (four reads per block); 0: 16 columns (two reads)
#endif
#ifndef TC_FFMA2
#define TC_FFMA2 1                   // 1: both FMAs of a value pair as fma.rn.f32x2 (same IEEE roundings, half the issue slots):
                                     //    72.0 -> 65.8 ms per 40-layer step; with TC_LD8 0: 67.4 ms
#endif
#ifndef TC_UNROLLJ
#define TC_UNROLLJ 1                 // 1: the four blocks of a stage unrolled, TMEM buffer index and parity static: 65.8 -> 65.1 ms
#endif
#ifndef TC_MAGIC
#define TC_MAGIC 0                   // 1: int32 -> fp32 by the 1.5*2^23 bit trick (integer add + fp add) instead of
                                     //    cvt.rn.f32.s32; measured 8% slower than the convert on B200, kept as a switch
#endif

struct TcStage {
    alignas(128) unsigned char A[TC_KB][TC_M * 32];      // activations, canonical layout, 4 KB per block
    alignas(128) unsigned char B[TC_KB][TC_N * 32];      // weights expanded to int8, 4 KB per block
    alignas(16)  float  d4[TC_KB][TC_N];                 // weight block scales as fp32
    alignas(16)  float2 sc[TC_M][TC_KB];                 // (d8, 8*sum) per token
    alignas(16)  unsigned char rawq[TC_N][TC_KB * 16 + 16];   // nibbles as they lie in the pack (+16: bank spread)
    alignas(8)   __half rawd[TC_N][TC_KB];
};

struct TcSmem {
    TcStage st[TC_STAGES];
    alignas(8) unsigned long long full[TC_STAGES], empty[TC_STAGES], tfull[TC_TBUF], tempty[TC_TBUF], qbar[4];
    unsigned tmem_base;
    int      abort;
    int      n_mtiles;
    // work list: M tiles of up to 128 slots: {expert, start in perm, count}
    int      mt_expert[TC_MAX_TILES], mt_start[TC_MAX_TILES], mt_count[TC_MAX_TILES];
    float    vbuf[TC_M][65];        // SwiGLU epilogue: v = silu(g)*u of 64 intermediate rows per token (+1: bank spread)
};

__device__ unsigned long long g_tc_prof[32];   // tuning: cycles spent per wait class (CTA 0)
#if TC_PROF
#define TC_TL_N 2048
__device__ long long g_tc_tl[8][TC_TL_N];   // tuning: per-block timestamps of CTA 0 (MMA thread: 0-2, epilogue warps: 3-5, 6-7)
#define TC_TL(row, b, v) do { if (blockIdx.x == 0 && (b) < TC_TL_N) g_tc_tl[row][b] = (v); } while (0)
#else
#define TC_TL(row, b, v) do { } while (0)
#endif
__device__ unsigned g_tc_status;     // 0, or the code of the first bounded wait that expired

// ---- PTX -------------------------------------------------------------------
__device__ __forceinline__ unsigned tc_smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(unsigned long long * b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(tc_smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_arrive(unsigned long long * b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(tc_smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(unsigned long long * b, unsigned parity) {
    unsigned ok;
#if TC_SUSPEND_NS
    // with a time hint the thread may stay suspended in hardware until the phase completes (or the hint runs out)
    // instead of coming back to spin through the issue slots its scheduler's epilogue warps need
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(tc_smem_u32(b)), "r"(parity), "r"((unsigned) TC_SUSPEND_NS) : "memory");
#else
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(tc_smem_u32(b)), "r"(parity) : "memory");
#endif
    return ok != 0;
}
// Bounded wait.  Returns false when it expired or another role already aborted.
__device__ __forceinline__ bool tc_wait(TcSmem & S, unsigned long long * b, unsigned parity, unsigned code) {
    for (unsigned i = 0; i < TC_SPIN; ++i) {
        if (tc_mbar_try(b, parity)) return true;
        if ((i & 255u) == 255u && *(volatile int *) &S.abort) return false;
    }
    atomicCAS(&g_tc_status, 0u, code);
    *(volatile int *) &S.abort = 1;
    return false;
}
#ifndef TC_PROF
#define TC_PROF 0                    // 1: accumulate cycles per wait class (tuning builds only)
#endif
#if TC_PROF
#define TC_TWAIT(acc, ...) ([&]() { const long long t0_ = TC_CLK(); const bool r_ = tc_wait(__VA_ARGS__); acc += TC_CLK() - t0_; return r_; })()
#define TC_CLK() clock64()
#else
#define TC_TWAIT(acc, ...) tc_wait(__VA_ARGS__)
#define TC_CLK() 0ll
#endif
__device__ __forceinline__ void tc_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long * b) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(tc_smem_u32(b)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, 0, 0;\n"          // enable_input_d = 0: D = A*B (no accumulate)
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
// K-major, no swizzle: core matrix = 8 rows x 16 B contiguous; K-adjacent core matrix at
// +128 B (leading byte offset), next 8-row group at +256 B (stride byte offset).
__device__ __forceinline__ unsigned long long tc_desc(const void * smem) {
    const unsigned a = tc_smem_u32(smem);
    return (unsigned long long) ((a >> 4) & 0x3FFFu) | ((unsigned long long) (128u >> 4) << 16)
         | ((unsigned long long) (256u >> 4) << 32) | (1ull << 46);
}
// s8 x s8 -> s32, M = 128, N = 128, both operands K-major.
#define TC_IDESC (0x20u | (1u << 7) | (1u << 10) | ((TC_N >> 3) << 17) | ((TC_M >> 4) << 24))

__device__ __forceinline__ void tc_ld32(unsigned taddr, int (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(unsigned taddr, int * r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld8(unsigned taddr, int * r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
// Two independent IEEE fused multiply-adds in one instruction (halves the issue slots of the epilogue).
__device__ __forceinline__ float2 tc_ffma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float tc_i2f(int s) {
#if TC_MAGIC
    return __fsub_rn(__int_as_float(s + 0x4B400000), 12582912.0f);      // exact for |s| < 2^22
#else
    return (float) s;
#endif
}
// Two int32 block sums -> fp32, exactly.  |s| <= 32*15*127 < 2^22, so the integer s + 0x4B400000 read as a
// float is 12582912 + s with no rounding, and subtracting 12582912 (one packed add) recovers float(s).
__device__ __forceinline__ float2 tc_i2f2(int a, int b) {
#if TC_MAGIC
    unsigned long long r, m, o;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a + 0x4B400000), "r"(b + 0x4B400000));
    asm("mov.b64 %0, {%1, %1};" : "=l"(m) : "f"(-12582912.0f));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(o) : "l"(r), "l"(m));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(o));
    return d;
#else
    return make_float2((float) a, (float) b);
#endif
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_cp16(void * dst, const void * src, bool valid) {
    const unsigned n = valid ? 16u : 0u;                       // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(tc_smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void tc_cp8(void * dst, const void * src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"(tc_smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tc_cp_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Offset of (row r, 16-byte K chunk kc) inside one 4 KB canonical operand block.
__device__ __forceinline__ int tc_canon(int r, int kc) { return (r >> 3) * 256 + kc * 128 + (r & 7) * 16; }

// ---------------------------------------------------------------------------
// EPI 0: out (+)= scale * acc           (N tile = 128 rows of one weight segment)
// EPI 1: SwiGLU + Q8_1                  (N tile = 64 gate rows | the same 64 up rows)
// ---------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(TC_THREADS, 1) k_pf_gemm_tc(const lkb_pf_gemm g, const int max_tiles) {
    extern __shared__ __align__(128) unsigned char tc_smem_raw[];
    TcSmem & S = *reinterpret_cast<TcSmem *>(tc_smem_raw);
    const int ptid = threadIdx.x, warp = ptid >> 5, lane = ptid & 31;
    const int tid = ptid - TC_LOADER_W0 * 32;          // index among the loader threads (meaningful in the loader warps only)

    // ---- set-up: barriers, TMEM, work list -------------------------------------
    if (ptid == 0) {
        S.abort = 0;
        for (int i = 0; i < TC_STAGES; ++i) { tc_mbar_init(&S.full[i], TC_LOADERS / 32); tc_mbar_init(&S.empty[i], 1 + TC_EPI_WARPS); }
        for (int i = 0; i < TC_TBUF; ++i) { tc_mbar_init(&S.tfull[i], 1); tc_mbar_init(&S.tempty[i], TC_EPI_WARPS); }
        for (int i = 0; i < 4; ++i) tc_mbar_init(&S.qbar[i], 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(tc_smem_u32(&S.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 1) {
        // Work list of M tiles (<= 128 slots of one expert) from the 64-slot plan tiles: consecutive
        // tiles of the same expert are merged pairwise.  Dense GEMM: ceil(ntok/128) plain ranges.
        int n = 0;
        if (g.perm) {
            int nt = *g.ntiles; if (nt > max_tiles) nt = max_tiles; if (nt > TC_MAX_TILES) nt = TC_MAX_TILES;
            // lane-strided scan; a tile opens an M tile when it is the first of its expert or an even
            // number of tiles after the first
            int run_first = 0;          // index of the first tile of the current expert (carried across chunks)
            for (int base = 0; base < nt; base += 32) {
                const int t = base + lane;
                int4 tl = make_int4(-1, 0, 0, 0), tp = make_int4(-2, 0, 0, 0), tn = make_int4(-3, 0, 0, 0);
                if (t < nt) tl = reinterpret_cast<const int4 *>(g.tiles)[t];
                if (t > 0 && t < nt) tp = reinterpret_cast<const int4 *>(g.tiles)[t - 1];
                if (t + 1 < nt) tn = reinterpret_cast<const int4 *>(g.tiles)[t + 1];
                const bool first = (t < nt) && (tl.x != tp.x);
                // index of the first tile of my expert: max over lanes <= mine of (first ? t : -1), seeded by run_first
                int f = first ? t : -1;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(LKB_FULL, f, o); if (lane >= o && v > f) f = v; }
                if (f < 0) f = run_first;
                const bool opens = (t < nt) && (((t - f) & 1) == 0);
                const unsigned m = __ballot_sync(LKB_FULL, opens);
                if (opens) {
                    const int k = n + __popc(m & ((1u << lane) - 1u));
                    S.mt_expert[k] = tl.x; S.mt_start[k] = tl.y;
                    S.mt_count[k] = tl.z + ((tn.x == tl.x) ? tn.z : 0);
                }
                n += __popc(m);
                run_first = __shfl_sync(LKB_FULL, f, 31);
            }
        } else {
            n = (g.ntok + TC_M - 1) / TC_M;
            for (int k = lane; k < n; k += 32) { S.mt_expert[k] = 0; S.mt_start[k] = k * TC_M; S.mt_count[k] = min(TC_M, g.ntok - k * TC_M); }
        }
        if (lane == 0) S.n_mtiles = n;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = S.tmem_base;
    const int n_mt = S.n_mtiles;
    const int n_rt = EPI ? g.N / 64 : g.N / TC_N;
    const int n_items = n_mt * n_rt;
    const int nstage_per_item = g.bpr / TC_KB;

    // ============================ loaders (warps 0-3) ============================
    // Thread tid owns token tid of the M tile and weight row tid of the N tile.  All global
    // traffic is cp.async (16 B), issued TC_AHEAD stages ahead: activations and their scales land
    // directly in the canonical operand layout, nibbles land in a raw staging row and are expanded
    // to int8 from shared memory when their stage comes up.
    if (warp >= TC_LOADER_W0 && warp < TC_LOADER_W0 + TC_LW) {
        struct Cur { int item, ks; int ar[TC_RPT]; const int8_t * aq[TC_RPT]; const float2 * as[TC_RPT];
                     const uint4 * wq[TC_RPT]; const __half * wd[TC_RPT]; };
        auto setup = [&](Cur & c) {
            if (c.item >= n_items) return;
            const int mt = c.item / n_rt, rt = c.item % n_rt;
            const int expert = S.mt_expert[mt], tstart = S.mt_start[mt], tcnt = S.mt_count[mt];
            const size_t eo = (size_t) expert * g.exp_stride;
#pragma unroll
            for (int q = 0; q < TC_RPT; ++q) {
                const int rr = tid + q * TC_LOADERS;                // token of the M tile == weight row of the N tile
                int slot = -1;
                if (rr < tcnt) slot = g.perm ? g.perm[tstart + rr] : tstart + rr;
                c.ar[q] = (slot >= 0) ? (slot >> g.a_shift) : -1;
                if (EPI) {
                    const int r = rt * 64 + (rr & 63);
                    const int sg = rr >> 6;                         // 0: gate, 1: up
                    c.wq[q] = (const uint4 *) g.qs[sg] + eo + (size_t) r * g.bpr;
                    c.wd[q] = (const __half *) g.d[sg] + eo + (size_t) r * g.bpr;
                } else {
                    const int r = rt * TC_N + rr;
                    const int seg = (r < g.seg_end[0]) ? 0 : (r < g.seg_end[1]) ? 1 : 2;
                    const int sbase = seg ? g.seg_end[seg - 1] : 0;
                    c.wq[q] = (const uint4 *) g.qs[seg] + eo + (size_t) (r - sbase) * g.bpr;
                    c.wd[q] = (const __half *) g.d[seg] + eo + (size_t) (r - sbase) * g.bpr;
                }
                c.aq[q] = g.aqs + (size_t) (c.ar[q] < 0 ? 0 : c.ar[q]) * g.bpr * 32;
                c.as[q] = reinterpret_cast<const float2 *>(g.asc) + (size_t) (c.ar[q] < 0 ? 0 : c.ar[q]) * g.bpr;
            }
        };
        auto advance = [&](Cur & c) { if (++c.ks == nstage_per_item) { c.ks = 0; c.item += gridDim.x; setup(c); } };
        int my_items = 0;
        if ((int) blockIdx.x < n_items) my_items = (n_items - 1 - (int) blockIdx.x) / (int) gridDim.x + 1;
        const unsigned total = (unsigned) my_items * (unsigned) nstage_per_item;
        Cur ci;
        ci.item = blockIdx.x; ci.ks = 0;
#pragma unroll
        for (int q = 0; q < TC_RPT; ++q) ci.ar[q] = -1;
        setup(ci);
        unsigned it_issue = 0;
        bool ok = true;
        long long pw_empty = 0, pw_cp = 0, pw_fence = 0, pw_unpack = 0; const long long pt0 = clock64();
        auto issue = [&]() {
            // stage it_issue: wait for its buffer, then fire the copies
            if (ok && it_issue < total) {
                const int stg = it_issue % TC_STAGES;
                if (!TC_TWAIT(pw_empty, S, &S.empty[stg], ((it_issue / TC_STAGES) & 1u) ^ 1u, 10u)) ok = false;
                else {
                    TcStage & T = S.st[stg];
                    const int kb0 = ci.ks * TC_KB;
#pragma unroll
                    for (int q = 0; q < TC_RPT; ++q) {
                        const int rr = tid + q * TC_LOADERS;
                        const bool live = ci.ar[q] >= 0;
#pragma unroll
                        for (int j = 0; j < TC_KB; ++j) {
                            tc_cp16(T.A[j] + tc_canon(rr, 0), ci.aq[q] + (size_t) (kb0 + j) * 32, live);
                            tc_cp16(T.A[j] + tc_canon(rr, 1), ci.aq[q] + (size_t) (kb0 + j) * 32 + 16, live);
                            tc_cp16(T.rawq[rr] + j * 16, ci.wq[q] + kb0 + j, true);
                        }
                        tc_cp16(&T.sc[rr][0], ci.as[q] + kb0, live);
                        tc_cp16(&T.sc[rr][2], ci.as[q] + kb0 + 2, live);
                        tc_cp8(T.rawd[rr], ci.wd[q] + kb0);
                    }
                    advance(ci);
                }
            }
            tc_cp_commit();                                         // one group per call, possibly empty
            ++it_issue;
        };
        // Expansion and publication of one landed stage.
        auto publish = [&](unsigned it) {
            TcStage & T = S.st[it % TC_STAGES];
            const long long tu0_ = TC_CLK();
            // every raw read of the stage first, then the expansion: a store between two loads would order them
            // (the compiler cannot tell the staging arrays apart through the computed offsets)
            uint4 wv[TC_RPT][TC_KB];
            uint2 dv[TC_RPT];
#pragma unroll
            for (int q = 0; q < TC_RPT; ++q) {
                const int rr = tid + q * TC_LOADERS;
#pragma unroll
                for (int j = 0; j < TC_KB; ++j) wv[q][j] = *reinterpret_cast<const uint4 *>(T.rawq[rr] + j * 16);
                dv[q] = *reinterpret_cast<const uint2 *>(T.rawd[rr]);               // the row's four fp16 block scales
            }
#pragma unroll
            for (int q = 0; q < TC_RPT; ++q) {
                const int rr = tid + q * TC_LOADERS;
                const __half2 d01 = *reinterpret_cast<const __half2 *>(&dv[q].x), d23 = *reinterpret_cast<const __half2 *>(&dv[q].y);
                const float df[4] = {__low2float(d01), __high2float(d01), __low2float(d23), __high2float(d23)};
#pragma unroll
                for (int j = 0; j < TC_KB; ++j) {
                    // byte i of the 16: element i (low nibble) | element i+16 (high nibble)
                    const uint4 w = wv[q][j];
                    *reinterpret_cast<uint4 *>(T.B[j] + tc_canon(rr, 0)) =
                        make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint4 *>(T.B[j] + tc_canon(rr, 1)) =
                        make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                    T.d4[j][rr] = df[j];
                }
            }
            const long long tf0_ = TC_CLK(); pw_unpack += tf0_ - tu0_;
            tc_fence_async();                                       // generic-proxy writes -> visible to the MMA
            pw_fence += TC_CLK() - tf0_;
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&S.full[it % TC_STAGES]);
        };
        // Publishing runs as far ahead as the copies: a stage is expanded and published as soon as its copies have
        // landed, BEFORE the loader blocks on the buffer of the next stage to request.  (Blocking first delayed the
        // publication of a stage that had landed long ago until the epilogue released an older buffer, and the MMA
        // issuer starved for the length of one expansion per stage.)
        for (int p = 0; p < TC_AHEAD; ++p) issue();                 // stages 0 .. TC_AHEAD-1 requested
        unsigned pub = 0;                                           // stages [0, pub) are published
        while (pub < total && ok) {
            // everything requested so far must land; then publish all of it, then request one more stage
            { const long long t0_ = TC_CLK(); tc_cp_wait<0>(); pw_cp += TC_CLK() - t0_; }
            const unsigned have = it_issue < total ? it_issue : total;
            for (; pub < have; ++pub) publish(pub);
            issue();                                                // blocks until the epilogue has released the buffer
        }
        tc_cp_wait<0>();
        if (blockIdx.x == 0 && tid == 0) { g_tc_prof[0] = pw_empty; g_tc_prof[1] = pw_cp; g_tc_prof[2] = clock64() - pt0; g_tc_prof[13] = pw_fence; g_tc_prof[14] = pw_unpack; }
    }
    // ============================ MMA issuer (last warp) =========================
    else if (warp == TC_MMA_WARP) {
        if (lane == 0) {
            unsigned it = 0, blk = 0;
            long long pw_full = 0, pw_te = 0; const long long pt0 = clock64();
            for (int item = blockIdx.x; item < n_items && !*(volatile int *) &S.abort; item += gridDim.x) {
                bool ok = true;
                for (int ks = 0; ks < nstage_per_item && ok; ++ks, ++it) {
                    const int stg = it % TC_STAGES;
                    if (!TC_TWAIT(pw_full, S, &S.full[stg], (it / TC_STAGES) & 1u, 20u)) { ok = false; break; }
                    tc_fence_after();
                    TcStage & T = S.st[stg];
#pragma unroll
                    for (int j = 0; j < TC_KB; ++j, ++blk) {
                        const int tb = blk % TC_TBUF;
                        TC_TL(0, blk, TC_CLK());
                        if (!TC_TWAIT(pw_te, S, &S.tempty[tb], ((blk / TC_TBUF) & 1u) ^ 1u, 21u)) { ok = false; break; }
                        TC_TL(1, blk, TC_CLK());
                        tc_fence_after();
                        tc_mma_i8(tmem + tb * TC_N, tc_desc(T.A[j]), tc_desc(T.B[j]), TC_IDESC);
                        tc_commit(&S.tfull[tb]);                    // this block's result is ready
                        TC_TL(2, blk, TC_CLK());
                    }
                    if (ok) tc_commit(&S.empty[stg]);               // the MMAs have finished reading the stage
                }
                if (!ok) break;
            }
            if (blockIdx.x == 0) { g_tc_prof[4] = pw_full; g_tc_prof[5] = pw_te; g_tc_prof[6] = clock64() - pt0; g_tc_prof[7] = blk; }
        }
    }
    // ============================ epilogue (sixteen warps) ========================
    // Four warps per TMEM lane quadrant, each folding 32 of the 128 columns: 32 accumulators
    // per thread, four warps per scheduler to hide the TMEM read latency.
    else if (warp >= TC_EPI_W0 && warp < TC_EPI_W0 + TC_EPI_WARPS) {
        const int ew = warp - TC_EPI_W0;             // 0..15
        const int quad = warp & 3;                  // TMEM lane quadrant this warp may access
        const int sub = ew >> 2;                    // which 32 columns
        const int tok = quad * 32 + lane;           // token (TMEM lane) of this thread
        const unsigned tlane = (unsigned) (quad * 32) << 16;
        // EPI 0: columns [32 sub, +32).  EPI 1: gate [16 sub, +16) -> acc[0..15], up [64 + 16 sub, +16) -> acc[16..31].
        const int c0 = EPI ? 16 * sub : 32 * sub;
        const int c1 = EPI ? 64 + 16 * sub : 32 * sub + 16;
        unsigned it = 0, blk = 0, nitem = 0;
        long long pw_full = 0, pw_tf = 0, pw_ld = 0, pw_tail = 0, pw_math = 0, pw_rel = 0; const long long pt0 = clock64();
        for (int item = blockIdx.x; item < n_items && !*(volatile int *) &S.abort; item += gridDim.x, ++nitem) {
            const int mt = item / n_rt, rt = item % n_rt;
            const int tstart = S.mt_start[mt], tcnt = S.mt_count[mt];
            const bool warp_live = quad * 32 < tcnt;          // padding-only warps skip the arithmetic
            int slot = -1;
            if (tok < tcnt) slot = g.perm ? g.perm[tstart + tok] : tstart + tok;
            const int ar = (slot >= 0) ? (slot >> g.a_shift) : -1;
            const float scl = (ar >= 0 && g.scale) ? g.scale[ar] : 1.0f;
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
            bool ok = true;
            for (int ks = 0; ks < nstage_per_item && ok; ++ks, ++it) {
                const int stg = it % TC_STAGES;
                if (!TC_TWAIT(pw_full, S, &S.full[stg], (it / TC_STAGES) & 1u, 30u)) { ok = false; break; }   // d4 / sc are in place
                TcStage & T = S.st[stg];
#if TC_UNROLLJ
                static_assert(TC_KB == TC_TBUF, "block j of a stage lands in TMEM buffer j");
                const unsigned tpar = it & 1u;                     // == (blk / TC_TBUF) & 1 for every block of the stage
#pragma unroll
#else
#pragma unroll 1
#endif
                for (int j = 0; j < TC_KB; ++j, ++blk) {
#if TC_UNROLLJ
                    const int tb = j;
#else
                    const int tb = blk % TC_TBUF;
                    const unsigned tpar = (blk / TC_TBUF) & 1u;
#endif
                    if (lane == 0 && warp == TC_LW) TC_TL(3, blk, TC_CLK());
                    if (lane == 0 && warp == TC_LW + 15) TC_TL(6, blk, TC_CLK());
                    if (!TC_TWAIT(pw_tf, S, &S.tfull[tb], tpar, 31u)) { ok = false; break; }
                    if (lane == 0 && warp == TC_LW) TC_TL(4, blk, TC_CLK());
                    if (lane == 0 && warp == TC_LW + 15) TC_TL(7, blk, TC_CLK());
                    tc_fence_after();
                    if (warp_live) {
                        const float2 sc = T.sc[tok][j];
                        const float d8 = sc.x, nc = -sc.y;
#if TC_LD8
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            // 8 columns at a time: few enough live registers that the three passes below stay
                            // separate (eight independent converts, then eight inner, then eight outer FMAs)
                            const int col = ((q & 2) ? c1 : c0) + 8 * (q & 1);
                            int sv[8];
                            const long long tl0_ = TC_CLK();
                            tc_ld8(tmem + tlane + tb * TC_N + col, sv);
                            const float4 da = *reinterpret_cast<const float4 *>(&T.d4[j][col]);
                            const float4 db = *reinterpret_cast<const float4 *>(&T.d4[j][col + 4]);
                            tc_wait_ld();
                            const long long tl1_ = TC_CLK(); pw_ld += tl1_ - tl0_;
                            if (q == 3) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) tc_mbar_arrive(&S.tempty[tb]);      // TMEM buffer is free again
                            }
                            const long long tl2_ = TC_CLK(); pw_rel += tl2_ - tl1_;
#if TC_FFMA2
                            // two IEEE FMAs per issue slot: same roundings, half the FMA instructions
                            const float2 d8p = make_float2(d8, d8), ncp = make_float2(nc, nc);
                            const float2 ddp[4] = {make_float2(da.x, da.y), make_float2(da.z, da.w), make_float2(db.x, db.y), make_float2(db.z, db.w)};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                float2 f = make_float2(tc_i2f(sv[2 * i]), tc_i2f(sv[2 * i + 1]));
                                f = tc_ffma2(d8p, f, ncp);
                                const float2 r = tc_ffma2(ddp[i], f, make_float2(acc[8 * q + 2 * i], acc[8 * q + 2 * i + 1]));
                                acc[8 * q + 2 * i] = r.x; acc[8 * q + 2 * i + 1] = r.y;
                            }
#if TC_PROF
                            pw_math += TC_CLK() - tl2_ + (__float_as_int(acc[8 * q]) == 0x7fc12345 ? 1 : 0);   // keeps the clock read after the math
#endif
#else
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = tc_i2f(sv[i]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = fmaf(d8, f[i], nc);
                            const float dd8[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[8 * q + i] = fmaf(dd8[i], f[i], acc[8 * q + i]);
#endif
                        }
#else
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            // 16 columns at a time keeps the live registers under the 96-register budget (no spills)
                            int sv[16];
                            tc_ld16(tmem + tlane + tb * TC_N + (h ? c1 : c0), sv);
                            // the weight scales of these 16 columns come from shared memory while the TMEM read is in flight
                            const float * dp = &T.d4[j][h ? c1 : c0];
                            float4 dd[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) dd[i] = *reinterpret_cast<const float4 *>(dp + 4 * i);
                            { const long long t0_ = TC_CLK(); tc_wait_ld(); pw_ld += TC_CLK() - t0_; }
                            if (h == 1) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) tc_mbar_arrive(&S.tempty[tb]);      // TMEM buffer is free again
                                if (lane == 0 && warp == TC_LW) TC_TL(5, blk, TC_CLK());
                            }
#ifdef TC_ABLATE_MATH
                            acc[h] += __int_as_float(sv[0] ^ sv[15]);
#else
#if TC_FFMA2
#pragma unroll
                            for (int i = 0; i < 16; i += 4) {
                                const int o = h * 16 + i;
                                const float2 d8p = make_float2(d8, d8), ncp = make_float2(nc, nc);
                                float2 f0 = tc_ffma2(d8p, make_float2(tc_i2f(sv[i + 0]), tc_i2f(sv[i + 1])), ncp);
                                float2 f1 = tc_ffma2(d8p, make_float2(tc_i2f(sv[i + 2]), tc_i2f(sv[i + 3])), ncp);
                                f0 = tc_ffma2(make_float2(dd[i / 4].x, dd[i / 4].y), f0, make_float2(acc[o + 0], acc[o + 1]));
                                f1 = tc_ffma2(make_float2(dd[i / 4].z, dd[i / 4].w), f1, make_float2(acc[o + 2], acc[o + 3]));
                                acc[o + 0] = f0.x; acc[o + 1] = f0.y; acc[o + 2] = f1.x; acc[o + 3] = f1.y;
                            }
#else
#pragma unroll
                            for (int i = 0; i < 16; i += 4) {
                                const int o = h * 16 + i;
                                acc[o + 0] = fmaf(dd[i / 4].x, fmaf(d8, tc_i2f(sv[i + 0]), nc), acc[o + 0]);
                                acc[o + 1] = fmaf(dd[i / 4].y, fmaf(d8, tc_i2f(sv[i + 1]), nc), acc[o + 1]);
                                acc[o + 2] = fmaf(dd[i / 4].z, fmaf(d8, tc_i2f(sv[i + 2]), nc), acc[o + 2]);
                                acc[o + 3] = fmaf(dd[i / 4].w, fmaf(d8, tc_i2f(sv[i + 3]), nc), acc[o + 3]);
                            }
#endif
#endif
                        }
#endif
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) tc_mbar_arrive(&S.tempty[tb]);
                    }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&S.empty[stg]);                   // done with the stage's d4 / sc
            }
            if (!ok) break;
            // ---- tile epilogue -----------------------------------------------------
            const long long tt0_ = TC_CLK();
            if (EPI) {
                // acc[0..7] = 16 gate rows, acc[8..15] = the same 16 up rows.  v goes through shared memory so
                // that one thread sees the 32 rows of a Q8_1 block: subs (0,1) form block 0, (2,3) block 1.
                if (slot >= 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float g0 = __fmul_rn(acc[2 * i], scl), g1 = __fmul_rn(acc[2 * i + 1], scl);
                        const float u0 = __fmul_rn(acc[16 + 2 * i], scl), u1 = __fmul_rn(acc[16 + 2 * i + 1], scl);
                        S.vbuf[tok][16 * sub + 2 * i]     = __fmul_rn(lkb_silu(g0), u0);
                        S.vbuf[tok][16 * sub + 2 * i + 1] = __fmul_rn(lkb_silu(g1), u1);
                    }
                }
                // the four warps of this quadrant meet (bounded, like every other wait)
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&S.qbar[quad]);
                if (!tc_wait(S, &S.qbar[quad], nitem & 1u, 32u)) break;
                if ((sub & 1) == 0 && slot >= 0) {
                    const int b = sub >> 1;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = S.vbuf[tok][32 * b + i];
                    float am = 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) am = fmaxf(am, fabsf(v[i]));
                    // the sum in xor-butterfly order (16, 8, 4, 2, 1), as the warp quantiser produces it
                    float t[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) t[i] = __fadd_rn(v[i], v[i + 16]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) t[i] = __fadd_rn(t[i], t[i + 8]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) t[i] = __fadd_rn(t[i], t[i + 4]);
                    const float sum = __fadd_rn(__fadd_rn(t[0], t[2]), __fadd_rn(t[1], t[3]));
                    const float d = __fdiv_rn(am, 127.0f);
                    unsigned pk[8];
#pragma unroll
                    for (int w = 0; w < 8; ++w) {
                        unsigned pp = 0;
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) {
                            const int q = (am == 0.0f) ? 0 : (int) roundf(__fdiv_rn(v[w * 4 + bb], d));
                            pp |= ((unsigned) q & 0xFFu) << (8 * bb);
                        }
                        pk[w] = pp;
                    }
                    const int orow0 = rt * 64 + 32 * b;                // first intermediate row of the block
                    int8_t * oq = g.oqs + (size_t) slot * (g.okb * 32) + orow0;
                    *reinterpret_cast<uint4 *>(oq) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4 *>(oq + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                    const __half2 ds = __floats2half2_rn(d, sum);
                    reinterpret_cast<float2 *>(g.osc)[(size_t) slot * g.okb + orow0 / 32] =
                        make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
                }
            } else if (slot >= 0) {
                float * p0 = g.out + (size_t) slot * g.out_ld + rt * TC_N + c0;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    float4 o0 = make_float4(__fmul_rn(acc[i], scl), __fmul_rn(acc[i + 1], scl),
                                            __fmul_rn(acc[i + 2], scl), __fmul_rn(acc[i + 3], scl));
                    if (g.add) {
                        const float4 a0 = *reinterpret_cast<const float4 *>(p0 + i);
                        o0 = make_float4(__fadd_rn(a0.x, o0.x), __fadd_rn(a0.y, o0.y), __fadd_rn(a0.z, o0.z), __fadd_rn(a0.w, o0.w));
                    }
                    *reinterpret_cast<float4 *>(p0 + i) = o0;
                }
            }
            pw_tail += TC_CLK() - tt0_;
        }
        if (blockIdx.x == 0 && ptid == (TC_EPI_W0 + 0) * 32) { g_tc_prof[8] = pw_full; g_tc_prof[9] = pw_tf; g_tc_prof[10] = clock64() - pt0; g_tc_prof[11] = pw_ld; g_tc_prof[12] = pw_tail; g_tc_prof[21] = pw_math; g_tc_prof[22] = pw_rel; }
        if (blockIdx.x == 0 && ptid == (TC_EPI_W0 + 2) * 32) { g_tc_prof[16] = pw_full; g_tc_prof[17] = pw_tf; g_tc_prof[18] = clock64() - pt0; g_tc_prof[19] = pw_ld; g_tc_prof[20] = pw_tail; g_tc_prof[23] = pw_math; g_tc_prof[24] = pw_rel; }
    }

    // ---- teardown: everyone meets, then the allocating warp frees TMEM ------------
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512) : "memory");
    }
}

// ---------------------------------------------------------------------------
static int g_tc_ready = 0;

int lkb_gemm_tc_init() {
    cudaError_t e = cudaFuncSetAttribute(k_pf_gemm_tc<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(TcSmem));
    if (e != cudaSuccess) return -(int) e;
    e = cudaFuncSetAttribute(k_pf_gemm_tc<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) sizeof(TcSmem));
    if (e != cudaSuccess) return -(int) e;
    g_tc_ready = 1;
    return LKB_OK;
}

// Shapes the tensor-core form covers; otherwise LKB_ERR_UNSUPPORTED (the caller falls back
// to the CUDA-core form): out_ld / okb rows must allow 16-byte vector stores.
int lkb_gemm_tc_launch(const lkb_pf_gemm * g, int epi, int max_tiles, cudaStream_t st) {
    if (!g_tc_ready) return LKB_ERR_NOT_INIT;
    if (g->bpr % TC_KB) return LKB_ERR_UNSUPPORTED;
    if (epi) { if (g->N % 64 || (g->okb * 32) % 16) return LKB_ERR_UNSUPPORTED; }
    else if (g->N % TC_N || g->out_ld % 4 || ((size_t) g->out & 15)) return LKB_ERR_UNSUPPORTED;
    if (g->perm && max_tiles > TC_MAX_TILES) return LKB_ERR_UNSUPPORTED;
    if (!g->perm && (g->ntok + TC_M - 1) / TC_M > TC_MAX_TILES) return LKB_ERR_UNSUPPORTED;
    if (((size_t) g->aqs & 15) || ((size_t) g->asc & 15)) return LKB_ERR_UNSUPPORTED;
    const int grid = lkb_context().sm_count;
    if (epi) k_pf_gemm_tc<1><<<grid, TC_THREADS, sizeof(TcSmem), st>>>(*g, max_tiles);
    else     k_pf_gemm_tc<0><<<grid, TC_THREADS, sizeof(TcSmem), st>>>(*g, max_tiles);
    return lkb_check_launch();
}

extern "C" {
// Tuning hook (not in the public header): copies the 16 profiling counters of the last launch.
__attribute__((visibility("default"))) int lkb_debug_gemm_prof(unsigned long long * out16) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpyFromSymbol(out16, g_tc_prof, 32 * sizeof(unsigned long long)) == cudaSuccess ? 0 : -1;
}
#if TC_PROF
__attribute__((visibility("default"))) int lkb_debug_gemm_timeline(long long * out) {      // [8][TC_TL_N]
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpyFromSymbol(out, g_tc_tl, sizeof(long long) * 8 * TC_TL_N) == cudaSuccess ? 0 : -1;
}
#endif
int lkb_pf_gemm_status(void) {
    unsigned v = 0, z = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tc_status, &z, sizeof z);
    return (int) v;
}
}
