// lkb_gemm_tc.cu - tensor-core form of the Q4_0 x Q8_1 grouped GEMM for sm_100a:
// tcgen05.mma.kind::i8 with accumulators in tensor memory (TMEM), every operand byte delivered by the
// tensor memory accelerator (cp.async.bulk.tensor: tiles of the activation planes -- gathered into token-tile
// order first when a workspace is registered, row-gathered through `perm` otherwise -- and tiles of the raw
// nibble plane of the weights).
//
//   out[slot][n] (+)= scale[arow] * sum_{b ascending} fma(d4[n][b], fma(d8[arow][b], F_b, -c[arow][b]), .)
//   S_b = sum_{i<32} nibble[n][b][i] * q8[arow][b][i]                     (int32, exact)
//   F_b = the fp32 whose bit pattern is 0x4B400000 + S_b  (= 12582912 + S_b, exact: |S_b| < 2^22)
//   c   = fma(d8, 12582912, 8sum)
// This (FOLD = 1) is the arithmetic of the reference's shipped GEMM (its accumulator is seeded with the
// bit pattern of 1.5 * 2^23 and the offset is folded into a per-(token, block) constant), so fp32
// results are bit-identical to that kernel's.  ref: src/prefill.cu:32-50,131-139,341-342,381-384
// FOLD = 0 spends one more packed add per value pair to recover float(S_b) = F_b - 12582912 exactly and
// evaluates the decode kernels' term fma(d4, fma(d8, float(S_b), -8sum), .) -- ref: src/quant.cuh:154-157,
// src/prefill.cu:391-399 (the reference's PF_EPI2 = 0 build) -- which stays within 1e-5 of float64.
//
// One MMA per 32-element block: K = 32 int8 is exactly one Q4_0/Q8_1 block, and the per-block scales forbid
// accumulating across blocks inside the tensor core, so every block's 128x128 int32 result is read back from
// TMEM and folded into fp32 register accumulators by the CUDA cores: two FMAs per value and no conversion --
// F_b is the loaded int32 plus 0x4B400000 as an INTEGER add, which rides on the move that pairs two columns for
// the packed FMA (no extra instruction).  That epilogue (256 FMA-pipe cycles per block and SM) bounds the
// kernel, not the MMA (64); measured costs on B200 that shaped it: a TMEM load occupies a scheduler's TMEM port
// ~26 cycles whether it moves 8 or 32 columns, a TMEM store ~1.2 cycles per column (presetting the buffers to
// the offset and letting the MMA accumulate onto it cost 789 / 402 us per layer against 721 / 383 us with the
// integer add); an integer-to-float conversion runs at a quarter of the FMA rate; a warp-uniform 16-byte
// shared-memory load costs two wavefronts.
//   * M (TMEM lanes) = 128 tokens, N (TMEM columns) = 128 weight rows.  A thread owns one token and 64 columns:
//     d8 / c are per-thread scalars, and in the SwiGLU form its columns are the gate AND up rows of one 32-row
//     Q8_1 output block, which it quantises alone, in the standard butterfly order (bit-identical to the
//     unfused path), with no exchange between threads;
//   * eight epilogue warps (two per TMEM lane quadrant), each a software pipeline over half blocks: the TMEM
//     load of the next 32 columns is in flight while the 32 just read are folded, so the TMEM port, the FMA pipe
//     and shared memory work at the same time inside one warp;
//   * one producer warp issuing only bulk tensor copies; two expansion warps turn the staged nibbles into the
//     int8 B operand (swizzled stores) and the fp16 block scales (read straight from global memory, one stage
//     ahead) into fp32; one thread issues the MMAs; four TMEM buffers of 128 columns: MMAs run up to four
//     blocks ahead;
//   * setmaxnreg moves registers from the producer / expansion / issuer warpgroup to the epilogue warpgroups;
//   * persistent: one CTA per SM walks (128-token tile, row tile) work items built from the device-side tile
//     list, expert by expert, so an expert's weights stay in L2.
// No copy in this file is a multicast one; every tensor map covers memory of the GPU the kernel runs on.
// Every wait is bounded; on expiry a status word is set and all roles drain and exit, freeing TMEM.
#include "lkb_device.cuh"
#include <cuda.h>

#define TC_M         128            // tokens per tile (TMEM lanes)
#define TC_N         128            // weight rows per tile (TMEM columns of one buffer)
#define TC_KB        4              // blocks per pipeline stage = 128 bytes of K per operand row
#define TC_TBUF      4              // TMEM buffers
#define TC_EPI_WARPS 8              // warps 0..7: quadrant = warp & 3, column half = warp >> 2
#define TC_MMA_WARP  8
#define TC_PROD_WARP 9
#define TC_EXP_W0    10             // expansion warps 10, 11: thread e serves staged weight rows e and e + 64
#define TC_EXP_WARPS 2
#define TC_TAIL_W0   12             // tail warps 12..15: finish a tile from shared memory while the next one is folded
#define TC_TAIL_WARPS 4
// The plain form (EPI 0) hands finished tiles to the tail warps through shared memory (3 pipeline stages + the staged
// tile); the SwiGLU form finishes its tiles in the epilogue threads themselves and runs without tail warps, 4 stages.
template <int EPI> struct TcCfg {
    static constexpr int NS = EPI ? 4 : 3;
    static constexpr int THREADS = (EPI ? TC_TAIL_W0 : TC_TAIL_W0 + TC_TAIL_WARPS) * 32;
    static constexpr int OUT_CHUNKS = EPI ? 1 : 32 * 129;
};
#define TC_OUT_PITCH 129            // 16-byte chunks per 4-column group of the staged tile (+1: bank spread)
#define TC_SPIN      (1u << 24)
#define TC_MAX_TILES 1024           // 64-token plan tiles the work list can hold
#define TC_MAGIC_I   0x4B400000
#define TC_MAGIC_F   12582912.0f

struct TcStage {
    alignas(1024) unsigned char A[TC_M * 128];          // activations: row r at r*128, 16-byte chunk c at c ^ (r & 7)
    alignas(1024) unsigned char B[TC_N * 128];          // weights as int8, same layout
    alignas(1024) unsigned char rawq[TC_N * 64];        // nibbles as in the pack: row r at r*64, chunk c at c ^ ((r >> 1) & 3)
    alignas(128)  float2 sc[TC_M][TC_KB];               // (d8, 8*sum) per token and block
    alignas(16)   float  d4[TC_KB][TC_N];               // weight block scales as fp32
};
static_assert(sizeof(TcStage) % 1024 == 0, "stages keep the 1024-byte alignment of the swizzled operands");

template <int EPI>
struct TcSmem {
    static constexpr int NS = TcCfg<EPI>::NS;
    TcStage st[NS];
    // a finished tile's 128 x 128 accumulators on their way to the tail warps: the 4 columns [4c, +4) of token t at
    // float4 index c * TC_OUT_PITCH + t (writers: consecutive tokens, readers: consecutive c, both conflict-free)
    alignas(16) float4 tile_out[TcCfg<EPI>::OUT_CHUNKS];
    alignas(8) unsigned long long rawfull[NS], full[NS], empty[NS], tfull[TC_TBUF], tempty[TC_TBUF], tailfull, tailempty;
    unsigned tmem_base;
    int      abort;
    int      n_mtiles;
    // work list: M tiles of up to 128 slots: {expert, start in perm, count}
    int      mt_expert[TC_MAX_TILES], mt_start[TC_MAX_TILES], mt_count[TC_MAX_TILES];
};

__device__ unsigned g_tc_status;     // 0, or the code of the first bounded wait that expired

#ifdef LKB_TUNING
// Tuning builds only (-DLKB_TUNING; the default build has none of this): clock64 stamps of CTA 0, one row per
// role, four stamps per block or stage.
#define TC_TL_N 1024
__device__ long long g_tc_tl[6][TC_TL_N][4];
#define TC_TL(row, i, k) do { if (blockIdx.x == 0 && (i) < TC_TL_N) g_tc_tl[row][i][k] = clock64(); } while (0)
#else
#define TC_TL(row, i, k) do { } while (0)
#endif

// ---- PTX -------------------------------------------------------------------
__device__ __forceinline__ unsigned tc_smem_u32(const void * p) { return (unsigned) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void tc_mbar_init(unsigned long long * b, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(tc_smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void tc_mbar_arrive(unsigned long long * b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(tc_smem_u32(b)) : "memory");
}
__device__ __forceinline__ void tc_mbar_arrive_tx(unsigned long long * b, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(tc_smem_u32(b)), "r"(bytes) : "memory");
}
// One poll of an mbarrier phase.  HINT_NS > 0: the thread may stay suspended in hardware until the phase completes or
// the hint runs out, instead of coming back at once to spin through the issue slots the epilogue warps need.
template <int HINT_NS>
__device__ __forceinline__ bool tc_mbar_try(unsigned long long * b, unsigned parity) {
    unsigned ok;
    if (HINT_NS > 0)
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(tc_smem_u32(b)), "r"(parity), "r"((unsigned) HINT_NS) : "memory");
    else
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(tc_smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when it expired or another role already aborted.  The roles with slack (producer,
// expansion, issuer) poll with a suspend hint; the epilogue warps, whose waits are almost always over already, spin.
template <int HINT_NS = 0, class SM>
__device__ __forceinline__ bool tc_wait(SM & S, unsigned long long * b, unsigned parity, unsigned code) {
    for (unsigned i = 0; i < (HINT_NS > 0 ? TC_SPIN >> 4 : TC_SPIN); ++i) {
        if (tc_mbar_try<HINT_NS>(b, parity)) return true;
        if ((i & (HINT_NS > 0 ? 15u : 255u)) == 0u && *(volatile int *) &S.abort) return false;
    }
    atomicCAS(&g_tc_status, 0u, code);
    *(volatile int *) &S.abort = 1;
    return false;
}
#ifndef TC_HINT_PROD
#define TC_HINT_PROD 2000           // ns
#endif
#ifndef TC_HINT_MMA
#define TC_HINT_MMA 500
#endif
__device__ __forceinline__ void tc_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long * b) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(tc_smem_u32(b)) : "memory");
}
// D = A*B (the TMEM buffer is overwritten: enable-input-d predicate false)
__device__ __forceinline__ void tc_mma_i8(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, 0, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
// K-major operand with the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
// (stride byte offset); a K step of 32 bytes inside the swizzle span moves the start address.
__device__ __forceinline__ unsigned long long tc_desc(unsigned smem_addr) {
    return (unsigned long long) ((smem_addr >> 4) & 0x3FFFu) | (1ull << 16)
         | ((unsigned long long) (1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// s8 x s8 -> s32, M = 128, N = 128, both operands K-major.
#define TC_IDESC (0x20u | (1u << 7) | (1u << 10) | ((TC_N >> 3) << 17) | ((TC_M >> 4) << 24))

// 32 columns of this warp's 32 lanes -> 32 registers
__device__ __forceinline__ void tc_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Two independent IEEE fused multiply-adds in one instruction (half the issue slots of the epilogue).
__device__ __forceinline__ unsigned long long tc_pack(float x, float y) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ unsigned long long tc_pack_u(unsigned x, unsigned y) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(x), "r"(y));
    return r;
}
__device__ __forceinline__ unsigned long long tc_ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long tc_fadd2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ void tc_unpack(unsigned long long v, float & x, float & y) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
// one tile of a 2-D tensor: box at (x, y) -> shared memory, bytes counted on the mbarrier
__device__ __forceinline__ void tc_tma_tile(void * dst, const CUtensorMap * map, int x, int y, unsigned long long * bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 :: "r"(tc_smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(tc_smem_u32(bar)) : "memory");
}
// four rows y0..y3 of a 2-D tensor, columns from x on, one box width each -> four consecutive rows in shared memory
__device__ __forceinline__ void tc_tma_gather4(void * dst, const CUtensorMap * map, int x, int y0, int y1, int y2, int y3,
                                               unsigned long long * bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 :: "r"(tc_smem_u32(dst)), "l"(map), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3), "r"(tc_smem_u32(bar)) : "memory");
}

// Fold 32 columns of one block into 16 accumulator pairs: acc = fma(d4, fma(d8, F, -c), acc), two columns per
// instruction.  d4c -> the 32 weight scales of these columns (shared memory, warp-uniform).
template <int FOLD, int OFF>
__device__ __forceinline__ void tc_fold32(unsigned long long (&acc)[32], const unsigned (&sv)[32], const float * d4c,
                                          unsigned long long d8p, unsigned long long ncp) {
    const unsigned long long nmag = tc_pack(-TC_MAGIC_F, -TC_MAGIC_F);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 dd = *reinterpret_cast<const float4 *>(d4c + 4 * i);
        unsigned long long f0 = tc_pack_u(sv[4 * i] + TC_MAGIC_I, sv[4 * i + 1] + TC_MAGIC_I);   // (F, F) of two columns
        unsigned long long f1 = tc_pack_u(sv[4 * i + 2] + TC_MAGIC_I, sv[4 * i + 3] + TC_MAGIC_I);
        if (!FOLD) { f0 = tc_fadd2(f0, nmag); f1 = tc_fadd2(f1, nmag); }       // float(S), exact
        f0 = tc_ffma2(d8p, f0, ncp);
        f1 = tc_ffma2(d8p, f1, ncp);
        acc[OFF + 2 * i] = tc_ffma2(tc_pack(dd.x, dd.y), f0, acc[OFF + 2 * i]);
        acc[OFF + 2 * i + 1] = tc_ffma2(tc_pack(dd.z, dd.w), f1, acc[OFF + 2 * i + 1]);
    }
}

// ---------------------------------------------------------------------------
// Gather of the activation rows of a grouped GEMM into token-tile order: row p of the workspace planes = the row
// of slot perm[p] (p < number of planned slots), so that the GEMM fetches a 128-token tile with one tile copy.
// One warp per row.
// ---------------------------------------------------------------------------
// a_pitch > 0: the activation rows are PACKED rows of a_pitch bytes (quants, then the (d8, 8sum) pairs), as the
// expert-parallel dispatch delivers them; g.aqs points at the first one and g.asc is not read.
__global__ void __launch_bounds__(256) k_pf_gather_rows(const lkb_pf_gemm g, const int max_tiles, int8_t * __restrict__ wq,
                                                        float2 * __restrict__ ws, const int cap_rows, const int a_pitch) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int nt = *g.ntiles; if (nt > max_tiles) nt = max_tiles;
    if (nt <= 0) return;
    const int4 tl = reinterpret_cast<const int4 *>(g.tiles)[nt - 1];
    int n_live = tl.y + tl.z; if (n_live > cap_rows) n_live = cap_rows;
    const int row_bytes = g.bpr * 32;
    for (int p = blockIdx.x * 8 + warp; p < n_live; p += gridDim.x * 8) {
        const int ar = g.perm[p] >> g.a_shift;
        const uint4 * src = reinterpret_cast<const uint4 *>(g.aqs + (size_t) ar * (a_pitch ? a_pitch : row_bytes));
        uint4 * dst = reinterpret_cast<uint4 *>(wq + (size_t) p * row_bytes);
        for (int i = lane; i < row_bytes / 16; i += 32) dst[i] = __ldg(src + i);
        const float4 * ss = a_pitch ? reinterpret_cast<const float4 *>(g.aqs + (size_t) ar * a_pitch + row_bytes)
                                    : reinterpret_cast<const float4 *>(reinterpret_cast<const float2 *>(g.asc) + (size_t) ar * g.bpr);
        float4 * sd = reinterpret_cast<float4 *>(ws + (size_t) p * g.bpr);
        for (int i = lane; i < g.bpr / 2; i += 32) sd[i] = __ldg(ss + i);
    }
}

// ---------------------------------------------------------------------------
// EPI 0: out (+)= scale * acc           (N tile = 128 rows of one weight segment)
// EPI 1: SwiGLU + Q8_1                  (N tile = 64 gate rows | the same 64 up rows)
// rpe = weight rows per expert (exp_stride / bpr).  tiled = 1: map_a / map_s cover planes whose row p is the
// activation row of token-tile position p (the dense form, or the gathered workspace), fetched as 128-row tiles;
// tiled = 0: they cover the caller's planes and rows are gathered through perm, four per copy.
// ---------------------------------------------------------------------------
template <int EPI, int FOLD>
__global__ void __launch_bounds__(TcCfg<EPI>::THREADS, 1) k_pf_gemm_tc(const lkb_pf_gemm g, const int max_tiles, const int rpe, const int tiled,
                                                              const __grid_constant__ CUtensorMap map_a,
                                                              const __grid_constant__ CUtensorMap map_s,
                                                              const __grid_constant__ CUtensorMap map_w0,
                                                              const __grid_constant__ CUtensorMap map_w1,
                                                              const __grid_constant__ CUtensorMap map_w2,
                                                              float * const * __restrict__ out_rows) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    extern __shared__ unsigned char tc_smem_raw[];
    // the swizzle patterns are functions of the shared-memory address: stages start on 1024-byte boundaries
    typedef TcSmem<EPI> Smem;
    constexpr int TC_NS = Smem::NS;
    Smem & S = *reinterpret_cast<Smem *>(tc_smem_raw + ((1024u - (tc_smem_u32(tc_smem_raw) & 1023u)) & 1023u));
    const int ptid = threadIdx.x, warp = ptid >> 5, lane = ptid & 31;

    // ---- set-up: barriers, TMEM, work list -------------------------------------
    if (ptid == 0) {
        S.abort = 0;
        for (int i = 0; i < TC_NS; ++i) {
            tc_mbar_init(&S.rawfull[i], 1);                           // the lane that posts the tile bytes
            tc_mbar_init(&S.full[i], 1 + TC_EXP_WARPS);               // the lane that posts the activation bytes + the expansion warps
            tc_mbar_init(&S.empty[i], 1 + TC_EPI_WARPS);              // MMA commit + epilogue warps
        }
        for (int i = 0; i < TC_TBUF; ++i) { tc_mbar_init(&S.tfull[i], 1); tc_mbar_init(&S.tempty[i], TC_EPI_WARPS); }
        tc_mbar_init(&S.tailfull, TC_EPI_WARPS); tc_mbar_init(&S.tailempty, TC_TAIL_WARPS);
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

    // Registers follow the work: the warpgroup of the issuer, producer and expansion warps gives most of its
    // allocation to the two epilogue warpgroups (64 accumulators and two 32-column block-sum sets per thread).
    // (setmaxnreg sits inside the branch it governs: after a join the compiler must assume the smaller limit.)
    if (warp >= TC_EPI_WARPS) {
    if (EPI) asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    else     asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    // ============================ tail (four warps) ==============================
    // A finished tile leaves the epilogue warps' registers through shared memory, and these warps turn it into the
    // output while the epilogue warps are already folding the next tile.  Plain form: one token row (128 floats) per
    // warp instruction, scaled (and added to the residual), stored as 512 contiguous bytes.  SwiGLU form: lane = one of
    // the 32 intermediate rows of a Q8_1 block, quantised by the standard warp quantiser (the unfused kernels' code).
    if (!EPI && warp >= TC_TAIL_W0) {
        const int tw = warp - TC_TAIL_W0;
        unsigned k = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++k) {
            const int mt = item / n_rt, rt = item % n_rt;
            const int tstart = S.mt_start[mt], tcnt = S.mt_count[mt];
            // lane i: the slot and row scale of token 32 tw + i
            const int tokl = 32 * tw + lane;
            int slot_l = -1;
            if (tokl < tcnt) slot_l = g.perm ? g.perm[tstart + tokl] : tstart + tokl;
            const float scl_l = (slot_l >= 0 && g.scale) ? g.scale[slot_l >> g.a_shift] : 1.0f;
            // where the slot's output row starts: the caller's matrix, or a row address of its own (the expert-parallel
            // form: the row goes straight into its home rank's buffer, a peer's memory included -- plain stores)
            unsigned long long rowp_l = 0ull;
            if (slot_l >= 0) rowp_l = (unsigned long long) (EPI == 0 && out_rows ? out_rows[slot_l] : g.out + (size_t) slot_l * g.out_ld);
            if (!tc_wait<TC_HINT_PROD>(S, &S.tailfull, k & 1u, 40u)) break;
            const int nrows = min(32, tcnt - 32 * tw);
            // four rows per iteration: their dependent chains (shuffles, divisions) interleave
            for (int i0 = 0; i0 < nrows; i0 += 4) {
                int slot[4]; float scl[4]; unsigned long long rowp[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    slot[u] = __shfl_sync(LKB_FULL, slot_l, (i0 + u) & 31);
                    scl[u] = __shfl_sync(LKB_FULL, scl_l, (i0 + u) & 31);
                    rowp[u] = __shfl_sync(LKB_FULL, rowp_l, (i0 + u) & 31);
                    if (i0 + u >= nrows) slot[u] = -1;
                }
                {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (slot[u] < 0) continue;
                        const int t = 32 * tw + i0 + u;
                        const float4 a = S.tile_out[lane * TC_OUT_PITCH + t];
                        float4 * p = reinterpret_cast<float4 *>(reinterpret_cast<float *>(rowp[u]) + rt * TC_N) + lane;
                        float4 o;
                        if (g.add) {
                            // the residual add as the reference's build evaluates it: one fused multiply-add
                            // (nvcc contracts its `*p + acc * scale`, src/prefill.cu:484-486)
                            const float4 r = *p;
                            o = make_float4(fmaf(a.x, scl[u], r.x), fmaf(a.y, scl[u], r.y), fmaf(a.z, scl[u], r.z), fmaf(a.w, scl[u], r.w));
                        } else {
                            o = make_float4(__fmul_rn(a.x, scl[u]), __fmul_rn(a.y, scl[u]), __fmul_rn(a.z, scl[u]), __fmul_rn(a.w, scl[u]));
                        }
                        *p = o;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) tc_mbar_arrive(&S.tailempty);            // the staged tile may be overwritten
        }
    }
    else
    // ============================ producer (one warp) ============================
    // Everything a stage needs from memory arrives by bulk tensor copies completing on mbarriers: lane 0 fetches the
    // two 64-row tiles of the nibble plane and, in the tiled form, the 128-token tiles of the quants and of the
    // (d8, 8sum) rows; in the gather form lane l fetches the rows of tokens 4l..4l+3 through perm.
    if (warp == TC_PROD_WARP) {
        unsigned it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const int mt = item / n_rt, rt = item % n_rt;
            const int expert = S.mt_expert[mt], tstart = S.mt_start[mt], tcnt = S.mt_count[mt];
            int crd[4] = {0, 0, 0, 0};        // gather form: activation rows (a dead token repeats a live one: never read back)
            if (!tiled) {
                int last = 0;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int rr = 4 * lane + q;
                    if (rr < tcnt) last = (g.perm ? g.perm[tstart + rr] : tstart + rr) >> g.a_shift;
                    crd[q] = last;
                }
            }
            const bool glive = !tiled && 4 * lane < tcnt;
            const unsigned a_bytes = tiled ? (unsigned) (TC_M * 128 + TC_M * TC_KB * 8) : (512u + 128u) * (unsigned) ((tcnt + 3) >> 2);
            const CUtensorMap * mw0 = &map_w0, * mw1 = &map_w1;
            int wrow0, wrow1;
            if (EPI) {
                wrow0 = wrow1 = expert * rpe + rt * 64;
            } else {
                const int r = rt * TC_N;
                const int seg = (r < g.seg_end[0]) ? 0 : (r < g.seg_end[1]) ? 1 : 2;
                const int sbase = seg ? g.seg_end[seg - 1] : 0;
                mw0 = mw1 = (seg == 0) ? &map_w0 : (seg == 1) ? &map_w1 : &map_w2;
                wrow0 = expert * rpe + (r - sbase); wrow1 = wrow0 + 64;
            }
            for (int ks = 0; ks < nstage_per_item; ++ks, ++it) {
                const int stg = it % TC_NS;
                if (lane == 0) TC_TL(0, it, 0);
                if (!tc_wait<TC_HINT_PROD>(S, &S.empty[stg], ((it / TC_NS) & 1u) ^ 1u, 10u)) { ok = false; break; }
                if (lane == 0) TC_TL(0, it, 1);
                TcStage & T = S.st[stg];
                const int kb0 = ks * TC_KB;
                if (lane == 0) {
                    tc_mbar_arrive_tx(&S.rawfull[stg], 2u * 64u * 64u);
                    tc_tma_tile(T.rawq, mw0, kb0 * 16, wrow0, &S.rawfull[stg]);
                    tc_tma_tile(T.rawq + 64 * 64, mw1, kb0 * 16, wrow1, &S.rawfull[stg]);
                    tc_mbar_arrive_tx(&S.full[stg], a_bytes);
                    if (tiled) {
                        tc_tma_tile(T.A, &map_a, kb0 * 32, tstart, &S.full[stg]);
                        tc_tma_tile(&T.sc[0][0], &map_s, kb0 * 8, tstart, &S.full[stg]);
                    }
                }
                __syncwarp();
                if (glive) {
                    tc_tma_gather4(T.A + lane * 512, &map_a, kb0 * 32, crd[0], crd[1], crd[2], crd[3], &S.full[stg]);
                    tc_tma_gather4(&T.sc[4 * lane][0], &map_s, kb0 * 8, crd[0], crd[1], crd[2], crd[3], &S.full[stg]);
                }
                if (lane == 0) TC_TL(0, it, 2);
            }
        }
    }
    // ============================ expansion (two warps) ==========================
    // Thread e turns the staged nibbles of weight rows e and e + 64 into int8 (byte i of a block's 16:
    // element i in the low nibble, element i + 16 in the high one) and their fp16 scales into fp32.  The scales
    // (8 bytes per row and stage: below the copy engine's 16-byte minimum) come straight from global memory, requested
    // one stage ahead.
    else if (warp >= TC_EXP_W0) {
        const int e = ptid - TC_EXP_W0 * 32;
        unsigned it = 0;
        bool ok = true;
        // scale rows of the two weight rows of item `item`
        auto scale_rows = [&](int item, const __half * (&dp)[2]) {
            const int mt = item / n_rt, rt = item % n_rt;
            const size_t eo = (size_t) S.mt_expert[mt] * g.exp_stride;
            if (EPI) {
                dp[0] = (const __half *) g.d[0] + eo + (size_t) (rt * 64 + e) * g.bpr;
                dp[1] = (const __half *) g.d[1] + eo + (size_t) (rt * 64 + e) * g.bpr;
            } else {
                const int r = rt * TC_N;
                const int seg = (r < g.seg_end[0]) ? 0 : (r < g.seg_end[1]) ? 1 : 2;
                const int sbase = seg ? g.seg_end[seg - 1] : 0;
                dp[0] = (const __half *) g.d[seg] + eo + (size_t) (r - sbase + e) * g.bpr;
                dp[1] = dp[0] + (size_t) 64 * g.bpr;
            }
        };
        const __half * dp[2] = {nullptr, nullptr};
        uint2 dnext[2] = {make_uint2(0, 0), make_uint2(0, 0)};
        if ((int) blockIdx.x < n_items) {
            scale_rows(blockIdx.x, dp);
            dnext[0] = __ldg(reinterpret_cast<const uint2 *>(dp[0]));
            dnext[1] = __ldg(reinterpret_cast<const uint2 *>(dp[1]));
        }
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            for (int ks = 0; ks < nstage_per_item; ++ks, ++it) {
                const uint2 dcur[2] = {dnext[0], dnext[1]};
                {   // request the next stage's scales before waiting for this stage's nibbles
                    int nks = ks + 1, nitem = item;
                    if (nks == nstage_per_item) { nks = 0; nitem += gridDim.x; if (nitem < n_items) scale_rows(nitem, dp); }
                    if (nitem < n_items) {
                        dnext[0] = __ldg(reinterpret_cast<const uint2 *>(dp[0] + nks * TC_KB));
                        dnext[1] = __ldg(reinterpret_cast<const uint2 *>(dp[1] + nks * TC_KB));
                    }
                }
                const int stg = it % TC_NS;
                if (e == 0) TC_TL(1, it, 0);
                if (!tc_wait<TC_HINT_PROD>(S, &S.rawfull[stg], (it / TC_NS) & 1u, 15u)) { ok = false; break; }
                if (e == 0) TC_TL(1, it, 1);
                TcStage & T = S.st[stg];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int rr = e + 64 * h;                         // staged row
                    const unsigned char * rq = T.rawq + rr * 64;
                    const int xs = (rr >> 1) & 3;
                    uint4 wv[TC_KB];
#pragma unroll
                    for (int j = 0; j < TC_KB; ++j) wv[j] = *reinterpret_cast<const uint4 *>(rq + ((j ^ xs) << 4));
                    // staged row -> operand row r (= TMEM column).  EPI 1: the staged rows are 64 gate rows then the
                    // same 64 up rows; 32 gate rows and their 32 up rows share a 64-column half (one epilogue thread
                    // holds a whole Q8_1 output block)
                    const int r = EPI ? 64 * (e >> 5) + 32 * h + (e & 31) : rr;
                    unsigned char * rb = T.B + (r >> 3) * 1024 + (r & 7) * 128;
                    const int x = r & 7;
                    const uint2 dv = dcur[h];
                    const __half2 d01 = *reinterpret_cast<const __half2 *>(&dv.x), d23 = *reinterpret_cast<const __half2 *>(&dv.y);
                    const float df[4] = {__low2float(d01), __high2float(d01), __low2float(d23), __high2float(d23)};
#pragma unroll
                    for (int j = 0; j < TC_KB; ++j) {
                        const uint4 w = wv[j];
                        *reinterpret_cast<uint4 *>(rb + (((2 * j) ^ x) << 4)) =
                            make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                        *reinterpret_cast<uint4 *>(rb + (((2 * j + 1) ^ x) << 4)) =
                            make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                        T.d4[j][r] = df[j];
                    }
                }
                tc_fence_async();                                       // generic-proxy writes -> visible to the MMA
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&S.full[stg]);
                if (e == 0) TC_TL(1, it, 2);
            }
        }
    }
    // ============================ MMA issuer =====================================
    else if (warp == TC_MMA_WARP) {
        if (lane == 0) {
            unsigned it = 0, blk = 0;
            for (int item = blockIdx.x; item < n_items && !*(volatile int *) &S.abort; item += gridDim.x) {
                bool ok = true;
                for (int ks = 0; ks < nstage_per_item && ok; ++ks, ++it) {
                    const int stg = it % TC_NS;
                    TC_TL(2, it, 0);
                    if (!tc_wait<TC_HINT_MMA>(S, &S.full[stg], (it / TC_NS) & 1u, 20u)) { ok = false; break; }
                    TC_TL(2, it, 1);
                    tc_fence_after();
                    const unsigned a0 = tc_smem_u32(S.st[stg].A), b0 = tc_smem_u32(S.st[stg].B);
#pragma unroll
                    for (int j = 0; j < TC_KB; ++j, ++blk) {
                        const int tb = blk % TC_TBUF;
                        // use k of a buffer waits for phase k: the epilogue releases every buffer once up front,
                        // then after every read
                        TC_TL(3, blk, 0);
                        if (!tc_wait<TC_HINT_MMA>(S, &S.tempty[tb], (blk / TC_TBUF) & 1u, 21u)) { ok = false; break; }
                        TC_TL(3, blk, 1);
                        tc_fence_after();
                        tc_mma_i8(tmem + tb * TC_N, tc_desc(a0 + j * 32), tc_desc(b0 + j * 32), TC_IDESC);
                        tc_commit(&S.tfull[tb]);                    // this block's result is ready
                        TC_TL(3, blk, 2);
                    }
                    if (ok) tc_commit(&S.empty[stg]);               // the MMAs have finished reading the stage
                }
                if (!ok) break;
            }
        }
    }
    }
    // ============================ epilogue (eight warps) =========================
    // Two warps per TMEM lane quadrant, each folding 64 of the 128 columns as two halves of 32.  The loop is a software
    // pipeline over half blocks: while one half's 32 block sums are folded into the accumulators (FMA pipe, shared-memory
    // scale reads) the TMEM load of the next half is in flight.
    else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int quad = warp & 3;                  // TMEM lane quadrant this warp may access
        const int half = warp >> 2;                 // which 64 columns
        const int tok = quad * 32 + lane;           // token (TMEM lane) of this thread
        const int c0 = 64 * half;
        // EPI 1: the expansion warps place gate rows [32 half, +32) of the item in columns [c0, +32) and the same up rows
        // in [c0 + 32, +32): acc[0..15] are gate pairs and acc[16..31] the matching up pairs.
        const unsigned tbase = tmem + ((unsigned) (quad * 32) << 16) + c0;
        // all four buffers start out free for the MMA issuer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
            for (int tb = 0; tb < TC_TBUF; ++tb) tc_mbar_arrive(&S.tempty[tb]);
        }
        unsigned it = 0, nitem = 0;
        unsigned svA[32], svB[32];
        bool ok = (int) blockIdx.x < n_items && !*(volatile int *) &S.abort;
        // prologue of the pipeline: the first half of the first block
        if (ok) {
            if (!tc_wait(S, &S.tfull[0], 0u, 31u)) ok = false;
            else { tc_fence_after(); tc_ld32(tbase, svA); }
        }
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const bool last_item = item + (int) gridDim.x >= n_items;
            unsigned long long acc[32];                        // 64 fp32 accumulators as 32 pairs
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0ull;
            for (int ks = 0; ks < nstage_per_item && ok; ++ks, ++it) {
                const int stg = it % TC_NS;
                if (!tc_wait(S, &S.full[stg], (it / TC_NS) & 1u, 30u)) { ok = false; break; }   // d4 / sc are in place
                TcStage & T = S.st[stg];
                static_assert(TC_KB == TC_TBUF, "block j of a stage lands in TMEM buffer j");
                const unsigned tpar = it & 1u;                     // phase parity of every TMEM buffer during this stage
#pragma unroll
                for (int j = 0; j < TC_KB; ++j) {
                    const unsigned ta = tbase + j * TC_N;
                    // a padding token reads whatever the stage held before: finite or not, the value stays in this
                    // thread's registers and is never stored
                    const float2 sc = T.sc[tok][j];
                    const float d8 = sc.x, nc = FOLD ? -fmaf(sc.x, TC_MAGIC_F, sc.y) : -sc.y;
                    const unsigned long long d8p = tc_pack(d8, d8), ncp = tc_pack(nc, nc);
                    if (ptid == 0) TC_TL(4, it * TC_KB + j, 0);
                    tc_wait_ld();                                   // first half of this block is in svA
                    if (ptid == 0) TC_TL(4, it * TC_KB + j, 1);
                    tc_ld32(ta + 32, svB);                          // second half in flight ...
                    tc_fold32<FOLD, 0>(acc, svA, &T.d4[j][c0], d8p, ncp);        // ... while the first is folded
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) tc_mbar_arrive(&S.tempty[j]);    // TMEM buffer is free again
                    if (ptid == 0) TC_TL(4, it * TC_KB + j, 2);
                    // first half of the next block (if any) in flight while the second half of this one is folded
                    const bool more = !(last_item && ks == nstage_per_item - 1 && j == TC_KB - 1);
                    if (more) {
                        const int nj = (j + 1) % TC_KB;
                        const unsigned npar = (j == TC_KB - 1) ? (tpar ^ 1u) : tpar;
                        if (!tc_wait(S, &S.tfull[nj], npar, 31u)) { ok = false; break; }
                        tc_fence_after();
                        tc_ld32(tbase + nj * TC_N, svA);
                    }
                    if (ptid == 0) TC_TL(4, it * TC_KB + j, 3);
                    tc_fold32<FOLD, 16>(acc, svB, &T.d4[j][c0 + 32], d8p, ncp);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&S.empty[stg]);                   // done with the stage's d4 / sc
            }
            if (!ok) break;
            if (EPI) {
                // ---- SwiGLU + Q8_1 of this thread's own Q8_1 block ---------------------
                const int mt = item / n_rt, rt = item % n_rt;
                const int tstart = S.mt_start[mt], tcnt = S.mt_count[mt];
                int slot = -1;
                if (tok < tcnt) slot = g.perm ? g.perm[tstart + tok] : tstart + tok;
                if (slot >= 0) {
                    const float scl = g.scale ? g.scale[slot >> g.a_shift] : 1.0f;
                    float a[64];
#pragma unroll
                    for (int i = 0; i < 32; ++i) tc_unpack(acc[i], a[2 * i], a[2 * i + 1]);
                    // a[0..31] = 32 gate rows, a[32..63] = the same 32 up rows: one Q8_1 block of the output row
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(lkb_silu(__fmul_rn(a[i], scl)), __fmul_rn(a[32 + i], scl));
                    float am = 0.0f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) am = fmaxf(am, fabsf(v[i]));
                    float sum;
                    if (FOLD) {
                        // shipped arithmetic: the block sum in the order of the reference's fused epilogue, where a lane adds
                        // rows (g, g+8) + (g+16, g+24) and the eight lanes then pair over g ^ 1, 2, 4 (src/prefill.cu:424-448)
                        float t[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) t[i] = __fadd_rn(__fadd_rn(v[i], v[i + 8]), __fadd_rn(v[i + 16], v[i + 24]));
                        sum = __fadd_rn(__fadd_rn(__fadd_rn(t[0], t[1]), __fadd_rn(t[2], t[3])),
                                        __fadd_rn(__fadd_rn(t[4], t[5]), __fadd_rn(t[6], t[7])));
                    } else {
                        // exact mode: xor-butterfly order (16, 8, 4, 2, 1), as the warp quantiser of the unfused path produces it
                        float t[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) t[i] = __fadd_rn(v[i], v[i + 16]);
#pragma unroll
                        for (int i = 0; i < 8; ++i) t[i] = __fadd_rn(t[i], t[i + 8]);
#pragma unroll
                        for (int i = 0; i < 4; ++i) t[i] = __fadd_rn(t[i], t[i + 4]);
                        sum = __fadd_rn(__fadd_rn(t[0], t[2]), __fadd_rn(t[1], t[3]));
                    }
                    const float d = __fdiv_rn(am, 127.0f);
                    // q = roundf(v / d), the quotient rounded as IEEE division rounds it.  The product with the
                    // reciprocal is within 2e-5 of that quotient (|q| <= 127), so unless it lies that close to a
                    // half-integer it rounds to the same integer; the rare close calls (and a reciprocal that
                    // overflowed: NaN fails the test) take the division itself.
                    const float rd = __frcp_rn(d);
                    unsigned pk[8];
#pragma unroll
                    for (int w = 0; w < 8; ++w) {
                        unsigned pp = 0;
#pragma unroll
                        for (int bb = 0; bb < 4; ++bb) {
                            const float x = v[w * 4 + bb];
                            const float tq = __fmul_rn(x, rd);
                            const float at = fabsf(tq);
                            int q;
                            if (fabsf((at - floorf(at)) - 0.5f) > 1e-4f) q = (int) roundf(tq);
                            else q = (int) roundf(__fdiv_rn(x, d));
                            if (am == 0.0f) q = 0;
                            pp |= ((unsigned) q & 0xFFu) << (8 * bb);
                        }
                        pk[w] = pp;
                    }
                    const int orow0 = rt * 64 + 32 * half;             // first intermediate row of the block
                    int8_t * oq = g.oqs + (size_t) slot * (g.okb * 32) + orow0;
                    *reinterpret_cast<uint4 *>(oq) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    *reinterpret_cast<uint4 *>(oq + 16) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                    const __half2 ds = __floats2half2_rn(d, sum);
                    reinterpret_cast<float2 *>(g.osc)[(size_t) slot * g.okb + orow0 / 32] =
                        make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
                }
            } else {
                // ---- hand the finished tile to the tail warps ----------------------------
                // (the previous tile must have left the staging area: phase nitem - 1 of tailempty; none before the first)
                if (!tc_wait(S, &S.tailempty, (nitem & 1u) ^ 1u, 32u)) { ok = false; break; }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float4 v;
                    tc_unpack(acc[2 * i], v.x, v.y);
                    tc_unpack(acc[2 * i + 1], v.z, v.w);
                    S.tile_out[(16 * half + i) * TC_OUT_PITCH + tok] = v;
                }
                __syncwarp();
                if (lane == 0) tc_mbar_arrive(&S.tailfull);
                ++nitem;
            }
        }
        tc_wait_ld();                                   // nothing of this thread is left in flight
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
typedef CUresult (*tc_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static tc_encode_fn g_tc_encode = nullptr;
static void * g_tc_ws = nullptr;            // caller-owned workspace for the gathered activation planes
static size_t g_tc_ws_bytes = 0;

int lkb_gemm_tc_init() {
    cudaError_t e = cudaSuccess;
    const int sm0 = (int) sizeof(TcSmem<0>) + 1024, sm1 = (int) sizeof(TcSmem<1>) + 1024;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_pf_gemm_tc<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm0);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_pf_gemm_tc<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm0);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_pf_gemm_tc<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm1);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_pf_gemm_tc<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm1);
    if (e != cudaSuccess) return -(int) e;
    // the tensor-map encoder is a driver entry point; it is looked up through the runtime so that the
    // library carries no link-time dependency on the driver
    void * fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr);
    if (e != cudaSuccess) return -(int) e;
    if (!fn || qr != cudaDriverEntryPointSuccess) return LKB_ERR_UNSUPPORTED;
    g_tc_encode = (tc_encode_fn) fn;
    g_tc_ready = 1;
    return LKB_OK;
}

// A byte matrix [rows][row_bytes] as a 2-D tensor; box = box_bytes x box_rows.  Rows past `rows` read as zero.
static int tc_make_map(CUtensorMap * m, const void * base, unsigned row_bytes, unsigned long long rows, unsigned box_bytes,
                       unsigned box_rows, CUtensorMapSwizzle sw) {
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = g_tc_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? LKB_OK : LKB_ERR_UNSUPPORTED;
}
#define TC_ANY_ROWS (1ull << 30)            // row bound of a plane whose extent the caller does not state: it only clips

// Shapes the tensor-core form covers; otherwise LKB_ERR_UNSUPPORTED (the caller falls back
// to the CUDA-core form): out_ld / okb rows must allow 16-byte vector stores, the planes the
// alignment the copy engine asks for.
int lkb_gemm_tc_launch(const lkb_pf_gemm * g, int epi, int fold, int max_tiles, cudaStream_t st, float * const * out_rows, int a_pitch) {
    if (a_pitch && (!g->perm || a_pitch % 16 || a_pitch < g->bpr * 40)) return LKB_ERR_SHAPE;     // packed rows: grouped form, 16-byte aligned
    if (out_rows && (epi || !g->perm || g->add)) return LKB_ERR_SHAPE;          // row targets: the plain grouped form, no residual add
    if (!g_tc_ready) return LKB_ERR_NOT_INIT;
    if (g->bpr % TC_KB) return LKB_ERR_UNSUPPORTED;
    if (epi) { if (g->N % 64 || (g->okb * 32) % 16) return LKB_ERR_UNSUPPORTED; }
    else if (g->N % TC_N || g->out_ld % 4 || ((size_t) g->out & 15)) return LKB_ERR_UNSUPPORTED;
    if (g->perm && max_tiles > TC_MAX_TILES) return LKB_ERR_UNSUPPORTED;
    if (!g->perm && (g->ntok + TC_M - 1) / TC_M > TC_MAX_TILES) return LKB_ERR_UNSUPPORTED;
    if (((size_t) g->aqs & 15) || (!a_pitch && ((size_t) g->asc & 15))) return LKB_ERR_UNSUPPORTED;
    if (g->exp_stride % g->bpr) return LKB_ERR_UNSUPPORTED;
    const int nseg = epi ? 2 : (g->seg_end[0] >= g->N ? 1 : g->seg_end[1] >= g->N ? 2 : 3);
    const unsigned qrow = (unsigned) g->bpr * 32u, srow = (unsigned) g->bpr * 8u;
    CUtensorMap ma, ms, mw[3];
    int r, tiled = 1;
    if (!g->perm) {
        // dense: token tile t = rows [128 t, +128) of the caller's planes
        r = tc_make_map(&ma, g->aqs, qrow, (unsigned long long) g->ntok, 128u, TC_M, CU_TENSOR_MAP_SWIZZLE_128B);
        if (r == LKB_OK) r = tc_make_map(&ms, g->asc, srow, (unsigned long long) g->ntok, 32u, TC_M, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        const size_t cap = (size_t) max_tiles * LKB_MOE_BN;                 // slots the plan can hold
        const size_t need = cap * ((size_t) qrow + srow);
        if (g_tc_ws && g_tc_ws_bytes >= need) {
            // grouped, workspace registered: gather the rows into token-tile order, then fetch tiles
            int8_t * wq = (int8_t *) g_tc_ws;
            float2 * ws = (float2 *) ((char *) g_tc_ws + cap * qrow);
            const int grid = lkb_context().sm_count * 4;
            LKB_PF_LAUNCH(k_pf_gather_rows, dim3(grid), dim3(256), 0, st, *g, max_tiles, wq, ws, (int) cap, a_pitch);
            r = lkb_check_launch();
            if (r != LKB_OK) return r;
            r = tc_make_map(&ma, wq, qrow, cap, 128u, TC_M, CU_TENSOR_MAP_SWIZZLE_128B);
            if (r == LKB_OK) r = tc_make_map(&ms, ws, srow, cap, 32u, TC_M, CU_TENSOR_MAP_SWIZZLE_NONE);
        } else {
            // grouped, no workspace: rows gathered through perm inside the kernel, four per copy
            if (a_pitch) return LKB_ERR_UNSUPPORTED;                        // packed rows need the gather pass
            tiled = 0;
            r = tc_make_map(&ma, g->aqs, qrow, TC_ANY_ROWS, 128u, 1u, CU_TENSOR_MAP_SWIZZLE_128B);
            if (r == LKB_OK) r = tc_make_map(&ms, g->asc, srow, TC_ANY_ROWS, 32u, 1u, CU_TENSOR_MAP_SWIZZLE_NONE);
        }
    }
    if (r != LKB_OK) return r;
    for (int s = 0; s < 3; ++s) {
        const int src = s < nseg ? s : 0;
        if (((size_t) g->qs[src] & 15) || ((size_t) g->d[src] & 7)) return LKB_ERR_UNSUPPORTED;
        r = tc_make_map(&mw[s], g->qs[src], (unsigned) g->bpr * 16u, TC_ANY_ROWS, 64u, 64u, CU_TENSOR_MAP_SWIZZLE_64B);
        if (r != LKB_OK) return r;
    }
    const int rpe = (int) (g->exp_stride / g->bpr);
    const int grid = lkb_context().sm_count;
    const size_t sm0 = sizeof(TcSmem<0>) + 1024, sm1 = sizeof(TcSmem<1>) + 1024;
    if (epi && fold)       LKB_PF_LAUNCH((k_pf_gemm_tc<1, 1>), dim3(grid), dim3(TcCfg<1>::THREADS), sm1, st, *g, max_tiles, rpe, tiled, ma, ms, mw[0], mw[1], mw[2], out_rows);
    else if (epi)          LKB_PF_LAUNCH((k_pf_gemm_tc<1, 0>), dim3(grid), dim3(TcCfg<1>::THREADS), sm1, st, *g, max_tiles, rpe, tiled, ma, ms, mw[0], mw[1], mw[2], out_rows);
    else if (fold)         LKB_PF_LAUNCH((k_pf_gemm_tc<0, 1>), dim3(grid), dim3(TcCfg<0>::THREADS), sm0, st, *g, max_tiles, rpe, tiled, ma, ms, mw[0], mw[1], mw[2], out_rows);
    else                   LKB_PF_LAUNCH((k_pf_gemm_tc<0, 0>), dim3(grid), dim3(TcCfg<0>::THREADS), sm0, st, *g, max_tiles, rpe, tiled, ma, ms, mw[0], mw[1], mw[2], out_rows);
    return lkb_check_launch();
}

extern "C" {
#ifdef LKB_TUNING
__attribute__((visibility("default"))) int lkb_debug_gemm_timeline(long long * out) {      // [6][TC_TL_N][4]
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    return cudaMemcpyFromSymbol(out, g_tc_tl, sizeof(long long) * 6 * TC_TL_N * 4) == cudaSuccess ? 0 : -1;
}
#endif
int lkb_pf_gemm_workspace_bytes(int max_tiles, int k_max, size_t * bytes_out) {
    if (!bytes_out) return LKB_ERR_NULL;
    if (max_tiles <= 0 || k_max <= 0 || k_max % 32) return LKB_ERR_SHAPE;
    *bytes_out = (size_t) max_tiles * LKB_MOE_BN * ((size_t) k_max + (size_t) k_max / 4);      // quants + (d8, 8sum) per 32
    return LKB_OK;
}
int lkb_pf_gemm_set_workspace(void * ptr, size_t bytes) {
    if (ptr && ((size_t) ptr & 255)) return LKB_ERR_SHAPE;
    g_tc_ws = ptr; g_tc_ws_bytes = ptr ? bytes : 0;
    return LKB_OK;
}
int lkb_pf_gemm_status(void) {
    unsigned v = 0, z = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof v) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tc_status, &z, sizeof z);
    return (int) v;
}
}
