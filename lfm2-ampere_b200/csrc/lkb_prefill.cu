// lkb_prefill.cu - batched-prefill kernels around the grouped GEMM (sm_100a):
// per-token RMSNorm -> planar Q8_1, row quantiser, SwiGLU quantiser, the batched
// router, top-4 selection, the deterministic expert count / tile plan / scatter,
// the rank-order combine, and a CUDA-core (dp4a) form of the Q4_0 x Q8_1 GEMM that
// serves as the always-available configuration (the tensor-core form lives in
// lkb_gemm_tc.cu).  Each kernel evaluates the per-token formula of its decode
// twin, so per-token results are bit-identical to the decode kernels.
#include "lkb_device.cuh"
#include <cstdlib>

#define LKB_REQUIRE_INIT() do { if (!lkb_context().inited) return LKB_ERR_NOT_INIT; } while (0)

// ---------------------------------------------------------------------------
// Per-token kernels.  Warps own contiguous 512-byte runs: four elements per lane through 128-bit loads, four
// 32-element blocks per step (lkb_quad_quant), several tokens per CTA and no CTA-wide barrier.  The arithmetic per
// element, per block and per token is that of the decode kernels (reference semantics: src/prefill.cu:871-932 norm,
// :1574-1594 row quantisers), so outputs compare byte for byte.
// ---------------------------------------------------------------------------
#ifndef PF_TOK_SPLIT
#define PF_TOK_SPLIT 4                   // warps sharing one token in k_pf_token_norm
#endif
#define PF_TOK_WARPS (PF_TOK_SPLIT > 4 ? PF_TOK_SPLIT : 4)        // warps per CTA of the per-token kernels
#define PF_TOK_PER_CTA (PF_TOK_WARPS / PF_TOK_SPLIT)

// MODE 0: norm of X.  MODE 1: X += sum_k w[4t+k] * D[4t+k] first (rank-order chain), then the norm.
// MODE 2: as 1 with the row of slot 4t+k found through pos[].  PF_TOK_SPLIT warps share a token (consecutive runs of blocks): each quantises u = x * nw per block and leaves each block's sum of squares of x in shared memory;
// after a named barrier over the token's warps the first warp of the token ends with 1/rms from the 64 partials in the decode
// kernels' order ((ssq[l] + ssq[l+32]) butterflied over l).
template <int MODE>
__global__ void __launch_bounds__(PF_TOK_WARPS * 32) k_pf_token_norm(float * __restrict__ X, const float * __restrict__ D,
                                                                      const int * __restrict__ pos, const float * __restrict__ wts,
                                                                      const float * __restrict__ nw, int8_t * __restrict__ aqs,
                                                                      float2 * __restrict__ asc, float * __restrict__ inv_out,
                                                                      float * __restrict__ h32, int m) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ float s_sq[PF_TOK_PER_CTA][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tl = warp / PF_TOK_SPLIT, part = warp % PF_TOK_SPLIT;
    const int t = blockIdx.x * PF_TOK_PER_CTA + tl;
    if (t >= m) return;                                   // all warps of the token leave together
    float4 * x4 = reinterpret_cast<float4 *>(X + (size_t) t * LKB_HIDDEN);
    const float4 * w4 = reinterpret_cast<const float4 *>(nw);
    unsigned * q4 = reinterpret_cast<unsigned *>(aqs + (size_t) t * LKB_HIDDEN);
    float2 * sc = asc + (size_t) t * (LKB_HIDDEN / 32);
    float4 * h4 = (MODE == 0 && h32) ? reinterpret_cast<float4 *>(h32 + (size_t) t * LKB_HIDDEN) : nullptr;
    const float4 * d4[LKB_TOP_K]; float wk[LKB_TOP_K];
    if (MODE) {
#pragma unroll
        for (int k = 0; k < LKB_TOP_K; ++k) {
            wk[k] = wts[t * 4 + k];
            const int row = (MODE == 2) ? pos[t * 4 + k] : t * 4 + k;
            d4[k] = reinterpret_cast<const float4 *>(D + (size_t) row * LKB_HIDDEN);
        }
    }
    constexpr int STEPS = LKB_HIDDEN / 128 / PF_TOK_SPLIT;
#pragma unroll
    for (int s = part * STEPS; s < part * STEPS + STEPS; ++s) {
        const int i4 = s * 32 + lane;
        float4 xv = x4[i4];
        if (MODE) {
            float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int k = 0; k < LKB_TOP_K; ++k) {
                const float4 dv = d4[k][i4];
                a.x = fmaf(wk[k], dv.x, a.x); a.y = fmaf(wk[k], dv.y, a.y);
                a.z = fmaf(wk[k], dv.z, a.z); a.w = fmaf(wk[k], dv.w, a.w);
            }
            xv = make_float4(__fadd_rn(xv.x, a.x), __fadd_rn(xv.y, a.y), __fadd_rn(xv.z, a.z), __fadd_rn(xv.w, a.w));
            x4[i4] = xv;
        }
        const float4 wv = __ldg(w4 + i4);
        const float4 u = make_float4(__fmul_rn(xv.x, wv.x), __fmul_rn(xv.y, wv.y), __fmul_rn(xv.z, wv.z), __fmul_rn(xv.w, wv.w));
        if (h4) h4[i4] = u;
        float2 s2;
        q4[i4] = lkb_quad_quant(u, lane, s2);
        const float sq = lkb_quad_sum(__fmul_rn(xv.x, xv.x), __fmul_rn(xv.y, xv.y), __fmul_rn(xv.z, xv.z), __fmul_rn(xv.w, xv.w));
        if ((lane & 7) == 0) { sc[s * 4 + (lane >> 3)] = s2; s_sq[tl][s * 4 + (lane >> 3)] = sq; }
    }
    asm volatile("bar.sync %0, %1;" :: "r"(1 + tl), "n"(32 * PF_TOK_SPLIT) : "memory");
    if (part == 0) {
        const float sv = lkb_warp_sum(__fadd_rn(s_sq[tl][lane], s_sq[tl][lane + 32]));
        if (lane == 0) inv_out[t] = rsqrtf(fmaf(sv, 1.0f / (float) LKB_HIDDEN, LKB_EPS));
    }
}

// Layer-0 form: normalise first (x * inv) * w, quantise that, report scale 1.  The sum of squares keeps the
// order of a 256-wide reduction (element i in chain i mod 256, chains folded 128 / 64 / 32 apart, then the
// butterfly): lane l runs the eight chains l + 32g and folds them in registers.
__global__ void __launch_bounds__(PF_TOK_WARPS * 32) k_pf_token_norm_plain(const float * __restrict__ X, const float * __restrict__ nw,
                                                                            int8_t * __restrict__ aqs, float2 * __restrict__ asc,
                                                                            float * __restrict__ inv_out, int m) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * PF_TOK_WARPS + (threadIdx.x >> 5);
    if (t >= m) return;
    const float * x = X + (size_t) t * LKB_HIDDEN;
    float S[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        S[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float xv = x[lane + 32 * g + 256 * j]; S[g] = fmaf(xv, xv, S[g]); }
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) S[g] = __fadd_rn(S[g], S[g + 4]);
    S[0] = __fadd_rn(S[0], S[2]); S[1] = __fadd_rn(S[1], S[3]);
    const float ss = lkb_warp_sum(__fadd_rn(S[0], S[1]));
    const float inv = rsqrtf(fmaf(ss, 1.0f / (float) LKB_HIDDEN, LKB_EPS));
    const float4 * x4 = reinterpret_cast<const float4 *>(x);
    const float4 * w4 = reinterpret_cast<const float4 *>(nw);
    unsigned * q4 = reinterpret_cast<unsigned *>(aqs + (size_t) t * LKB_HIDDEN);
    float2 * sc = asc + (size_t) t * (LKB_HIDDEN / 32);
#pragma unroll 4
    for (int s = 0; s < LKB_HIDDEN / 128; ++s) {
        const int i4 = s * 32 + lane;
        const float4 xv = x4[i4], wv = __ldg(w4 + i4);
        const float4 u = make_float4(__fmul_rn(__fmul_rn(xv.x, inv), wv.x), __fmul_rn(__fmul_rn(xv.y, inv), wv.y),
                                     __fmul_rn(__fmul_rn(xv.z, inv), wv.z), __fmul_rn(__fmul_rn(xv.w, inv), wv.w));
        float2 s2;
        q4[i4] = lkb_quad_quant(u, lane, s2);
        if ((lane & 7) == 0) sc[s * 4 + (lane >> 3)] = s2;
    }
    if (lane == 0) inv_out[t] = 1.0f;
}

// Row quantisers: a warp takes four adjacent blocks of one row (SWIGLU: of silu(gate) * up, the two halves of a
// row up_off apart).  Rows x ceil(kb / 4) warps, 8 per CTA.
template <int SWIGLU>
__global__ void __launch_bounds__(256) k_pf_rows_q8(const float * __restrict__ Y, int ld, int up_off, int kb, int rows,
                                                    int8_t * __restrict__ aqs, float2 * __restrict__ asc) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x & 31;
    const int gpr = (kb + 3) >> 2;
    const long long wid = (long long) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (wid >= (long long) rows * gpr) return;
    const int r = (int) (wid / gpr), g = (int) (wid - (long long) r * gpr);
    const int b = g * 4 + (lane >> 3);
    const bool live = b < kb;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (live) {
        const float * y = Y + (size_t) r * ld + b * 32 + (lane & 7) * 4;
        v = *reinterpret_cast<const float4 *>(y);
        if (SWIGLU) {
            const float4 up = *reinterpret_cast<const float4 *>(y + up_off);
            v = make_float4(__fmul_rn(lkb_silu(v.x), up.x), __fmul_rn(lkb_silu(v.y), up.y),
                            __fmul_rn(lkb_silu(v.z), up.z), __fmul_rn(lkb_silu(v.w), up.w));
        }
    }
    float2 s2;
    const unsigned pk = lkb_quad_quant(v, lane, s2);
    if (live) {
        reinterpret_cast<unsigned *>(aqs + (size_t) r * kb * 32 + b * 32)[lane & 7] = pk;
        if ((lane & 7) == 0) asc[(size_t) r * kb + b] = s2;
    }
}

// ---------------------------------------------------------------------------
// Router.  Short form for a few tokens: a CTA per token keeps the token's activation in registers (64 per lane)
// and each warp walks eight expert rows over it; a logit is the decode router's sum (lane l chains elements
// l, l+32, ... ascending, then the butterfly), so it is bit-identical to it.  ref semantics: src/prefill.cu:1668-1693
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_pf_router_token(const float * __restrict__ H, const float * __restrict__ Wr,
                                                         const float * __restrict__ bias, const float * __restrict__ inv,
                                                         float * __restrict__ sel, float * __restrict__ sig,
                                                         int4 * __restrict__ idx, float4 * __restrict__ wout) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ float s_sel[LKB_N_EXPERTS], s_sig[LKB_N_EXPERTS];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float * h = H + (size_t) t * LKB_HIDDEN;
    float hv[LKB_HIDDEN / 32];
#pragma unroll
    for (int j = 0; j < LKB_HIDDEN / 32; ++j) hv[j] = h[j * 32 + lane];
    float mine = 0.0f;
    for (int q = 0; q < 8; ++q) {
        const float * row = Wr + (size_t) (warp * 8 + q) * LKB_HIDDEN;
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < LKB_HIDDEN / 32; ++j) acc = fmaf(__ldg(row + j * 32 + lane), hv[j], acc);
        acc = lkb_warp_sum(acc);
        if (lane == q) mine = acc;
    }
    if (lane < 8) {
        const int e = warp * 8 + lane;
        const float l = __fmul_rn(mine, inv[t]);
        const float gv = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-l)));
        const float sv = __fadd_rn(gv, bias[e]);
        sig[(size_t) t * 64 + e] = gv;
        sel[(size_t) t * 64 + e] = sv;
        s_sig[e] = gv; s_sel[e] = sv;
    }
    if (idx) {                                             // the selection in the same launch (lkb_pf_select's result)
        __syncthreads();
        if (warp == 0) {
            int ord[LKB_TOP_K]; float wv[LKB_TOP_K];
            lkb_router_select(s_sel, s_sig, lane, ord, wv);
            if (lane == 0) { idx[t] = make_int4(ord[0], ord[1], ord[2], ord[3]); wout[t] = make_float4(wv[0], wv[1], wv[2], wv[3]); }
        }
    }
}

// Tiled form.  Each (token, expert) logit is one FMA chain over k = 0..2047 ascending (reference semantics:
// src/prefill.cu:1606-1666, same per-logit order), so a CTA runs a long sequential k loop and the kernel is bound by
// (a) how well the loads of the next k-tiles hide behind the FMAs of the current one and (b) how many FMAs each
// shared-memory wavefront feeds.  CTA = NW warps = 2 NW token groups x 16 expert lanes; a thread owns TPT tokens x the
// four experts (lane, lane + 16, + 32, + 48): 4 * TPT independent chains.  Tiles of RT_KT k-values of the CTA's token
// rows and of all 64 router rows travel global -> shared by 16-byte asynchronous copies through a ring of RT_STAGES
// buffers (rows keep their [row][k] layout, pitch RT_KT + 4 floats: nothing is transposed and 128-bit loads of 16 different
// rows are conflict-free); the multiply loop reads four k-values per load.  With TPT = 4 a warp spends 16 wavefronts
// (4 loads of router rows, 4 of token rows shared by half a warp) on 64 FMA instructions: the ratio at which the FMA
// pipes rather than shared memory set the pace.  One CTA barrier per tile.
#ifndef RT_KT
#define RT_KT     64                          // measured on B200, 4096 tokens: 32 -> 66 us, 64 -> 55 us, 128 (4 stages) -> 72 us
#endif
#define RT_PITCH  (RT_KT + 4)
#define RT_CPR    (RT_KT / 4)                 // 16-byte copies per staged row
#ifndef RT_STAGES
#define RT_STAGES 6
#endif
#ifndef RT_L_TPT
#define RT_L_TPT 4          // long form: 4 warps, 32 tokens per CTA (measured on B200 at 4096 tokens, 32-wide k-tiles: 66 us; 8 warps x 2 tokens 74 us,
#define RT_L_NW  4          // 8 warps x 4 tokens 94 us, 4 warps x 2 tokens 76 us; the k loop of one CTA is the critical path)
#endif
#ifndef RT_S_TPT
#define RT_S_TPT 2          // middle form: 4 warps, 16 tokens per CTA
#define RT_S_NW  4
#endif
__device__ __forceinline__ void rt_cp16(float * dst, const float * src, bool live) {
    const unsigned d = (unsigned) __cvta_generic_to_shared(dst);
    const int n = live ? 16 : 0;                          // 0: the 16 bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(d), "l"(src), "r"(n) : "memory");
}
template <int TPT, int NW>
__global__ void __launch_bounds__(32 * NW) k_pf_router_pipe(const float * __restrict__ H, int m, const float * __restrict__ Wr,
                                                        const float * __restrict__ bias, const float * __restrict__ inv,
                                                        float * __restrict__ sel, float * __restrict__ sig,
                                                        int4 * __restrict__ idx, float4 * __restrict__ wout) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    constexpr int TT = 2 * NW * TPT, ROWS = TT + LKB_N_EXPERTS, NTILES = LKB_HIDDEN / RT_KT;
    extern __shared__ __align__(16) float rt_ring[];                   // [RT_STAGES][ROWS][RT_PITCH]
    const int tid = threadIdx.x, te = tid & 15, tg = tid >> 4;
    const int t0 = blockIdx.x * TT;
    // a thread copies the same (row, 16-byte part) set of every tile: sources and ring offsets are computed once
    constexpr int NCP = (ROWS * RT_CPR + 32 * NW - 1) / (32 * NW);
    const float * src[NCP]; int dst[NCP]; bool live[NCP];
#pragma unroll
    for (int j = 0; j < NCP; ++j) {
        const int ch = tid + j * 32 * NW;
        const int row = ch / RT_CPR, part = (ch % RT_CPR) * 4;
        dst[j] = (ch < ROWS * RT_CPR) ? row * RT_PITCH + part : -1;
        if (row < TT) { const int tk = t0 + row; live[j] = tk < m; src[j] = H + (size_t) (tk < m ? tk : 0) * LKB_HIDDEN + part; }
        else          { live[j] = true; src[j] = Wr + (size_t) (row < ROWS ? row - TT : 0) * LKB_HIDDEN + part; }
    }
    auto issue = [&](int tile) {
        if (tile < NTILES) {
            float * st = rt_ring + (size_t) (tile % RT_STAGES) * ROWS * RT_PITCH;
            const int k0 = tile * RT_KT;
#pragma unroll
            for (int j = 0; j < NCP; ++j)
                if (dst[j] >= 0) rt_cp16(st + dst[j], src[j] + k0, live[j]);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");      // (an empty group keeps the count uniform)
    };
    float acc[TPT][4];
#pragma unroll
    for (int i = 0; i < TPT; ++i)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[i][q] = 0.0f;
#pragma unroll
    for (int s = 0; s < RT_STAGES - 1; ++s) issue(s);
    for (int tile = 0; tile < NTILES; ++tile) {
        asm volatile("cp.async.wait_group %0;" :: "n"(RT_STAGES - 2) : "memory");
        __syncthreads();                   // this tile has landed for everyone; the stage refilled below is no longer read
        issue(tile + RT_STAGES - 1);
        const float * st = rt_ring + (size_t) (tile % RT_STAGES) * ROWS * RT_PITCH;
        const float * sh = st + (tg * TPT) * RT_PITCH, * sw = st + (TT + te) * RT_PITCH;
#pragma unroll
        for (int c = 0; c < RT_KT; c += 4) {
            float4 w[4], h[TPT];
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = *reinterpret_cast<const float4 *>(sw + 16 * q * RT_PITCH + c);
#pragma unroll
            for (int i = 0; i < TPT; ++i) h[i] = *reinterpret_cast<const float4 *>(sh + i * RT_PITCH + c);
            // k-major order: consecutive FMAs belong to different chains, so none waits for its predecessor
#pragma unroll
            for (int i = 0; i < TPT; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(h[i].x, w[q].x, acc[i][q]);
#pragma unroll
            for (int i = 0; i < TPT; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(h[i].y, w[q].y, acc[i][q]);
#pragma unroll
            for (int i = 0; i < TPT; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(h[i].z, w[q].z, acc[i][q]);
#pragma unroll
            for (int i = 0; i < TPT; ++i)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][q] = fmaf(h[i].w, w[q].w, acc[i][q]);
        }
    }
    // the ring is free after the last tile: the CTA's sel / sig rows pass through it to the selection warps
    float * s_sel = rt_ring, * s_sig = rt_ring + TT * LKB_N_EXPERTS;
    if (idx) __syncthreads();
#pragma unroll
    for (int i = 0; i < TPT; ++i) {
        const int tl = tg * TPT + i, tk = t0 + tl;
        if (tk >= m) continue;
        const float iv = inv[tk];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = te + 16 * q;
            const float l = __fmul_rn(acc[i][q], iv);
            const float gv = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-l)));
            const float sv = __fadd_rn(gv, bias[e]);
            sig[(size_t) tk * 64 + e] = gv;
            sel[(size_t) tk * 64 + e] = sv;
            if (idx) { s_sig[tl * LKB_N_EXPERTS + e] = gv; s_sel[tl * LKB_N_EXPERTS + e] = sv; }
        }
    }
    if (idx) {                                             // the selection in the same launch (lkb_pf_select's result)
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        for (int tl = warp; tl < TT; tl += NW) {
            const int tk = t0 + tl;
            if (tk >= m) break;
            int ord[LKB_TOP_K]; float wv[LKB_TOP_K];
            lkb_router_select(s_sel + tl * LKB_N_EXPERTS, s_sig + tl * LKB_N_EXPERTS, lane, ord, wv);
            if (lane == 0) { idx[tk] = make_int4(ord[0], ord[1], ord[2], ord[3]); wout[tk] = make_float4(wv[0], wv[1], wv[2], wv[3]); }
        }
    }
}
template <int TPT, int NW>
static int rt_launch(const float * H, int m, const float * Wr, const float * bias, const float * inv, float * sel, float * sig,
                     int * idx, float * w, cudaStream_t st) {
    constexpr int TT = 2 * NW * TPT;
    constexpr size_t smem = (size_t) RT_STAGES * (TT + LKB_N_EXPERTS) * RT_PITCH * sizeof(float);
    static int ready[LKB_STATIC_MAX_DEVICES] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < LKB_STATIC_MAX_DEVICES && !ready[dev]) {
        if (cudaFuncSetAttribute(k_pf_router_pipe<TPT, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem) != cudaSuccess) return -(int) cudaGetLastError();
        ready[dev] = 1;
    }
    LKB_PF_LAUNCH((k_pf_router_pipe<TPT, NW>), dim3((m + TT - 1) / TT), dim3(32 * NW), smem, st, H, m, Wr, bias, inv, sel, sig,
                  reinterpret_cast<int4 *>(idx), reinterpret_cast<float4 *>(w));
    return lkb_check_launch();
}

// Top-4 of 64 per token: warps stride over the tokens (any grid); the selection itself is the redux-based
// lkb_router_select shared with the decode router.  ref semantics: src/prefill.cu:1696-1708
__global__ void __launch_bounds__(256) k_pf_select(const float * __restrict__ sel, const float * __restrict__ sig, int m,
                                                   int4 * __restrict__ idx, float4 * __restrict__ w) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x & 31;
    const int nw = gridDim.x * (blockDim.x >> 5);
    for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < m; t += nw) {
        int ord[LKB_TOP_K]; float wv[LKB_TOP_K];
        lkb_router_select(sel + (size_t) t * 64, sig + (size_t) t * 64, lane, ord, wv);
        if (lane == 0) {
            idx[t] = make_int4(ord[0], ord[1], ord[2], ord[3]);
            w[t] = make_float4(wv[0], wv[1], wv[2], wv[3]);
        }
    }
}

// ---------------------------------------------------------------------------
// count / plan / scatter.  ref: src/prefill.cu:1710-1756
// ---------------------------------------------------------------------------
// Per-CTA shared histogram, then 64 global atomics per CTA (integer: order-free).
__global__ void __launch_bounds__(256) k_pf_moe_count(const int * __restrict__ idx, int n, int * __restrict__ cnt) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ int s_c[LKB_N_EXPERTS];
    if (threadIdx.x < LKB_N_EXPERTS) s_c[threadIdx.x] = 0;
    __syncthreads();
    for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < n; s += gridDim.x * blockDim.x) atomicAdd(&s_c[idx[s]], 1);
    __syncthreads();
    if (threadIdx.x < LKB_N_EXPERTS && s_c[threadIdx.x]) atomicAdd(&cnt[threadIdx.x], s_c[threadIdx.x]);
}

// One warp: exclusive scan over the 64 counts, then tiles in expert order.
__global__ void __launch_bounds__(32) k_pf_moe_plan(const int * __restrict__ cnt, int * __restrict__ off,
                                                    int4 * __restrict__ tiles, int * __restrict__ ntiles) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x;
    const int c0 = cnt[lane], c1 = cnt[lane + 32];
    const int n0 = (c0 + LKB_MOE_BN - 1) / LKB_MOE_BN, n1 = (c1 + LKB_MOE_BN - 1) / LKB_MOE_BN;
    // inclusive scans over lanes for experts 0..31, then offset experts 32..63
    int so = c0, st = n0, so1 = c1, st1 = n1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int a = __shfl_up_sync(LKB_FULL, so, o), b = __shfl_up_sync(LKB_FULL, st, o);
        const int c = __shfl_up_sync(LKB_FULL, so1, o), d = __shfl_up_sync(LKB_FULL, st1, o);
        if (lane >= o) { so += a; st += b; so1 += c; st1 += d; }
    }
    const int tot_o = __shfl_sync(LKB_FULL, so, 31), tot_t = __shfl_sync(LKB_FULL, st, 31);
    const int off0 = so - c0, off1 = tot_o + so1 - c1;
    const int tb0 = st - n0, tb1 = tot_t + st1 - n1;
    off[lane] = off0; off[lane + 32] = off1;
    for (int i = 0; i < n0; ++i)
        tiles[tb0 + i] = make_int4(lane, off0 + i * LKB_MOE_BN, min(LKB_MOE_BN, c0 - i * LKB_MOE_BN), 0);
    for (int i = 0; i < n1; ++i)
        tiles[tb1 + i] = make_int4(lane + 32, off1 + i * LKB_MOE_BN, min(LKB_MOE_BN, c1 - i * LKB_MOE_BN), 0);
    if (lane == 31) *ntiles = tot_t + st1;
}

// Stable scatter.  CTA c owns slots [1024c, 1024c+1024): it histograms every
// earlier slot (L2-resident reads) to learn how many slots of each expert precede
// its chunk, ranks its own slots with match_any, and writes perm.  Result:
// expert-major, slot-ascending within an expert -- identical to the reference's
// per-expert compaction (ref: src/prefill.cu:1733-1756) without re-reading idx 64x.
__global__ void __launch_bounds__(1024) k_pf_moe_scatter(const int * __restrict__ idx, int n, const int * __restrict__ off,
                                                         int * __restrict__ perm) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    if ((int) blockIdx.x * 1024 >= n) return;              // CTA-uniform: nothing of this chunk is live
    __shared__ int s_prior[LKB_N_EXPERTS];
    __shared__ int s_wc[32][LKB_N_EXPERTS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int c0 = blockIdx.x * 1024;
    if (tid < LKB_N_EXPERTS) s_prior[tid] = off[tid];
    for (int i = tid; i < 32 * LKB_N_EXPERTS; i += 1024) (&s_wc[0][0])[i] = 0;
    __syncthreads();
    for (int s = tid; s < c0; s += 1024) atomicAdd(&s_prior[idx[s]], 1);
    const int s = c0 + tid;
    const bool live = s < n;
    const int e = live ? idx[s] : -1 - lane;               // dead lanes match nobody
    const unsigned same = __match_any_sync(LKB_FULL, e);
    const int rank_w = __popc(same & ((1u << lane) - 1u));
    if (live && rank_w == 0) s_wc[warp][e] = __popc(same);
    __syncthreads();
    // exclusive scan over warps, per expert (64 threads x 32 steps)
    if (tid < LKB_N_EXPERTS) {
        int run = s_prior[tid];
        for (int wv = 0; wv < 32; ++wv) { const int c = s_wc[wv][tid]; s_wc[wv][tid] = run; run += c; }
    }
    __syncthreads();
    if (live) perm[s_wc[warp][e] + rank_w] = s;
}

// ---------------------------------------------------------------------------
// combine: x[t] += sum over the token's four slots in rank order (one fused multiply-add chain from zero, then
// one add), four channels per thread.  The combine that feeds the next layer's norm is k_pf_token_norm<1>.
// ref semantics: src/prefill.cu:1804-1814 and 1764-1800
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_pf_moe_combine(float4 * __restrict__ X, const float4 * __restrict__ D,
                                                        const float * __restrict__ w, int m) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int i = blockIdx.x * blockDim.x + threadIdx.x;          // float4 index into X
    if (i >= m * (LKB_HIDDEN / 4)) return;
    const int t = i / (LKB_HIDDEN / 4), c = i - t * (LKB_HIDDEN / 4);
    const float4 wk = *reinterpret_cast<const float4 *>(w + t * 4);
    const float wv[4] = {wk.x, wk.y, wk.z, wk.w};
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < LKB_TOP_K; ++k) {
        const float4 dv = D[(size_t) (t * 4 + k) * (LKB_HIDDEN / 4) + c];
        a.x = fmaf(wv[k], dv.x, a.x); a.y = fmaf(wv[k], dv.y, a.y); a.z = fmaf(wv[k], dv.z, a.z); a.w = fmaf(wv[k], dv.w, a.w);
    }
    const float4 xv = X[i];
    X[i] = make_float4(__fadd_rn(xv.x, a.x), __fadd_rn(xv.y, a.y), __fadd_rn(xv.z, a.z), __fadd_rn(xv.w, a.w));
}

// planar row -> 36-byte blocks (exact: 8 sum is a power-of-two multiple).  Eight lanes per block, one word each.
// ref semantics: src/prefill.cu:1819-1828
__global__ void __launch_bounds__(512) k_pf_pack_q8_1(const int8_t * __restrict__ aqs, const float2 * __restrict__ asc, int t,
                                                      lkb_q8blk * __restrict__ y) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int b = threadIdx.x >> 3, wd = threadIdx.x & 7;
    reinterpret_cast<int *>(y[b].qs)[wd] = reinterpret_cast<const int *>(aqs + (size_t) t * LKB_HIDDEN + b * 32)[wd];
    if (wd == 0) {
        const float2 s = asc[(size_t) t * 64 + b];
        y[b].ds = __floats2half2_rn(s.x, __fmul_rn(s.y, 0.125f));
    }
}

// ---------------------------------------------------------------------------
// Expert-parallel dispatch helpers (no counterpart in the reference, which is single-GPU).
// A slot travels as ONE 2576-byte row: 2048 B of quants | 512 B of (d8, 8sum) pairs | 1/rms | expert id on the
// owner | 8 B pad, so that a layer's dispatch is a single all-to-all.
// ---------------------------------------------------------------------------
#define EP_ROW_BYTES (LKB_HIDDEN + (LKB_HIDDEN / 32) * 8 + 16)        // 2576, a multiple of 16

// Row p of `out` = the activation of slot send_order[p] (token = slot >> 2); pos[slot] = p.
__global__ void __launch_bounds__(192) k_ep_pack(const int8_t * __restrict__ aqs, const float2 * __restrict__ asc,
                                                 const float * __restrict__ inv, const int * __restrict__ idx,
                                                 const int * __restrict__ send_order, int experts_per_rank,
                                                 unsigned char * __restrict__ out, int * __restrict__ pos) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int p = blockIdx.x, i = threadIdx.x;
    const int slot = send_order[p], t = slot >> 2;
    uint4 * row = reinterpret_cast<uint4 *>(out + (size_t) p * EP_ROW_BYTES);
    if (i < 128) row[i] = reinterpret_cast<const uint4 *>(aqs + (size_t) t * LKB_HIDDEN)[i];
    else if (i < 160) row[i] = reinterpret_cast<const uint4 *>(asc + (size_t) t * (LKB_HIDDEN / 32))[i - 128];
    else if (i == 160) {
        const int e = idx[slot];
        row[160] = make_uint4(__float_as_uint(inv[t]), (unsigned) (e % experts_per_rank), 0u, 0u);
        pos[slot] = p;
    }
}

__global__ void __launch_bounds__(192) k_ep_unpack(const unsigned char * __restrict__ in, int8_t * __restrict__ qs,
                                                   float2 * __restrict__ sc, float * __restrict__ inv, int * __restrict__ le) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int p = blockIdx.x, i = threadIdx.x;
    const uint4 * row = reinterpret_cast<const uint4 *>(in + (size_t) p * EP_ROW_BYTES);
    if (i < 128) reinterpret_cast<uint4 *>(qs + (size_t) p * LKB_HIDDEN)[i] = row[i];
    else if (i < 160) reinterpret_cast<uint4 *>(sc + (size_t) p * (LKB_HIDDEN / 32))[i - 128] = row[i];
    else if (i == 160) { const uint4 v = row[160]; inv[p] = __uint_as_float(v.x); le[p] = (int) v.y; }
}


// ---------------------------------------------------------------------------
// CUDA-core form of the Q4_0 x Q8_1 GEMM (dense, grouped, SwiGLU epilogue).
// CTA = 64 weight rows (EPI 1: 32 gate + the same 32 up rows) x one 64-token
// tile; thread = rows (lane, lane+32) x 8 tokens, so a warp holds 32 consecutive
// rows of a token and the SwiGLU epilogue quantises with the standard warp
// quantiser: fused output == unfused output bit for bit.
// Per (row, token), b ascending: fold = 1: acc = fma(d4, fma(d8, F_b, -c), acc) with F_b = 12582912 + S_b and
// c = fma(d8, 12582912, 8sum) (the reference's shipped form, src/prefill.cu:131-139,341-342,381-384);
// fold = 0: acc = fma(d4, fma(d8, float(S_b), -8sum), acc) (src/prefill.cu:391-399); then * scale, then (+ out).
// ref: src/prefill.cu:172-491 (semantics)
// ---------------------------------------------------------------------------
#define SG_KB 8
#define SG_WP (SG_KB * 16 + 16)        // weight row pitch in smem (bytes), +16 against bank conflicts

template <int EPI>
__global__ void __launch_bounds__(256) k_pf_gemm_simple(const lkb_pf_gemm g, const int fold) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ __align__(16) unsigned char s_w[64 * SG_WP];
    __shared__ __align__(16) __half        s_d[64 * SG_KB];
    __shared__ __align__(16) int8_t        s_a[64 * SG_KB * 32];
    __shared__ __align__(16) float2        s_s[64 * SG_KB];
    __shared__ int   s_arow[64];
    __shared__ int   s_orow[64];
    __shared__ float s_scl[64];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int rt, tstart, tcnt, expert = 0;
    if (g.perm) {
        if ((int) blockIdx.y >= *g.ntiles) return;
        const int4 tl = reinterpret_cast<const int4 *>(g.tiles)[blockIdx.y];
        expert = tl.x; tstart = tl.y; tcnt = tl.z; rt = blockIdx.x;
    } else {
        rt = blockIdx.x; tstart = blockIdx.y * 64;
        tcnt = g.ntok - tstart; if (tcnt > 64) tcnt = 64;
    }
    if (tid < 64) {
        int slot = -1;
        if (tid < tcnt) slot = g.perm ? g.perm[tstart + tid] : tstart + tid;
        const int ar = (slot >= 0) ? (slot >> g.a_shift) : -1;
        s_arow[tid] = ar; s_orow[tid] = slot;
        s_scl[tid] = (ar >= 0 && g.scale) ? g.scale[ar] : 1.0f;
    }
    // weight rows of this CTA: local row r in [0,64)
    const int row0 = EPI ? rt * 32 : rt * 64;
    const size_t eo = (size_t) expert * g.exp_stride;
    const uint4 * wq[2]; const __half * wd[2];
    if (EPI) {
        wq[0] = (const uint4 *) g.qs[0] + eo + (size_t) row0 * g.bpr; wd[0] = (const __half *) g.d[0] + eo + (size_t) row0 * g.bpr;
        wq[1] = (const uint4 *) g.qs[1] + eo + (size_t) row0 * g.bpr; wd[1] = (const __half *) g.d[1] + eo + (size_t) row0 * g.bpr;
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = row0 + 32 * h;
            const int seg = (r < g.seg_end[0]) ? 0 : (r < g.seg_end[1]) ? 1 : 2;
            const int sbase = seg ? g.seg_end[seg - 1] : 0;
            wq[h] = (const uint4 *) g.qs[seg] + eo + (size_t) (r - sbase) * g.bpr;
            wd[h] = (const __half *) g.d[seg] + eo + (size_t) (r - sbase) * g.bpr;
        }
    }
    __syncthreads();

    float acc[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.0f;

    for (int kb0 = 0; kb0 < g.bpr; kb0 += SG_KB) {
        // stage: 64 rows x 8 blocks of weights, 64 tokens x 8 blocks of activations
        for (int c = tid; c < 64 * SG_KB; c += 256) {
            const int r = c / SG_KB, kk = c % SG_KB;
            const int h = r >> 5, rr = r & 31;
            *reinterpret_cast<uint4 *>(s_w + r * SG_WP + kk * 16) = wq[h][(size_t) rr * g.bpr + kb0 + kk];
            s_d[r * SG_KB + kk] = wd[h][(size_t) rr * g.bpr + kb0 + kk];
            const int ar = s_arow[r];
            s_s[r * SG_KB + kk] = (ar >= 0) ? reinterpret_cast<const float2 *>(g.asc)[(size_t) ar * g.bpr + kb0 + kk]
                                            : make_float2(0.0f, 0.0f);
        }
        for (int c = tid; c < 64 * SG_KB * 2; c += 256) {
            const int r = c / (SG_KB * 2), kk = c % (SG_KB * 2);
            const int ar = s_arow[r];
            int4 v = make_int4(0, 0, 0, 0);
            if (ar >= 0) v = *reinterpret_cast<const int4 *>(g.aqs + (size_t) ar * g.bpr * 32 + (size_t) kb0 * 32 + kk * 16);
            *reinterpret_cast<int4 *>(s_a + r * SG_KB * 32 + kk * 16) = v;
        }
        __syncthreads();
#pragma unroll 2
        for (int kk = 0; kk < SG_KB; ++kk) {
            uint4 wv[2]; float d4[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                wv[h] = *reinterpret_cast<const uint4 *>(s_w + (lane + 32 * h) * SG_WP + kk * 16);
                d4[h] = __half2float(s_d[(lane + 32 * h) * SG_KB + kk]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int tk = warp * 8 + j;
                const int4 a0 = *reinterpret_cast<const int4 *>(s_a + tk * SG_KB * 32 + kk * 32);
                const int4 a1 = *reinterpret_cast<const int4 *>(s_a + tk * SG_KB * 32 + kk * 32 + 16);
                const int xv[8] = { a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w };
                const float2 sc = s_s[tk * SG_KB + kk];
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    {
                        const int si = lkb_sumi(wv[h], xv);
                        acc[h][j] = fold ? lkb_block_acc_pf(d4[h], sc.x, si, sc.y, acc[h][j]) : lkb_block_acc(d4[h], sc.x, si, sc.y, acc[h][j]);
                    }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int tk = warp * 8 + j;
        const int orow = s_orow[tk];            // warp-uniform
        if (orow < 0) continue;
        const float scl = s_scl[tk];
        if (EPI) {
            const float gt = __fmul_rn(acc[0][j], scl);
            const float up = __fmul_rn(acc[1][j], scl);
            const float v = __fmul_rn(lkb_silu(gt), up);
            // shipped arithmetic: the block sum in the reference's fused-epilogue order; exact mode: the quantiser's butterfly
            if (fold) lkb_quant_store_planar_fused_epilogue(v, g.oqs + (size_t) orow * (g.okb * 32) + row0,
                                                            reinterpret_cast<float2 *>(g.osc) + (size_t) orow * g.okb + row0 / 32, lane);
            else      lkb_quant_store_planar(v, g.oqs + (size_t) orow * (g.okb * 32) + row0,
                                             reinterpret_cast<float2 *>(g.osc) + (size_t) orow * g.okb + row0 / 32, lane);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // the residual add is one fused multiply-add, as the reference's build contracts it (src/prefill.cu:484-486)
                float * p = g.out + (size_t) orow * g.out_ld + row0 + 32 * h + lane;
                *p = g.add ? fmaf(acc[h][j], scl, *p) : __fmul_rn(acc[h][j], scl);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
int lkb_gemm_tc_init();                                      // lkb_gemm_tc.cu
int lkb_gemm_tc_launch(const lkb_pf_gemm * g, int epi, int fold, int max_tiles, cudaStream_t st, float * const * out_rows, int a_pitch);   // LKB_ERR_UNSUPPORTED if shape not covered

static int g_gemm_cfg = -1;        // -1: tensor-core form when it covers the shape; 0: CUDA-core form
static int g_gemm_fold = 1;        // 1: the reference's shipped per-block term (folded offset); 0: the exact term

int lkb_prefill_init() {
    const char * v = getenv("LKB_PF_CFG");
    if (v) g_gemm_cfg = atoi(v);
    v = getenv("LKB_PF_ARITH");
    if (v) g_gemm_fold = atoi(v) ? 1 : 0;
    return lkb_gemm_tc_init();
}

static int gemm_check(const lkb_pf_gemm * g, int epi) {
    if (!g) return LKB_ERR_NULL;
    if (!g->qs[0] || !g->d[0] || !g->aqs || !g->asc) return LKB_ERR_NULL;
    if (epi) { if (!g->qs[1] || !g->d[1] || !g->oqs || !g->osc) return LKB_ERR_NULL; }
    else if (!g->out) return LKB_ERR_NULL;
    if (g->bpr <= 0 || g->bpr % 8) return LKB_ERR_SHAPE;
    if (epi ? (g->N % 64) : (g->N % 128)) return LKB_ERR_SHAPE;
    if (!epi && (g->seg_end[0] % 128 || g->seg_end[1] % 128)) return LKB_ERR_SHAPE;
    if (g->perm && (!g->tiles || !g->ntiles)) return LKB_ERR_NULL;
    return LKB_OK;
}

static int gemm_dispatch(const lkb_pf_gemm * g, int epi, int max_tiles, cudaStream_t st, float * const * out_rows = nullptr, int a_pitch = 0) {
    LKB_REQUIRE_INIT();
    const int r = gemm_check(g, epi);
    if (r != LKB_OK) return r;
    const int ty = g->perm ? max_tiles : (g->ntok + 63) / 64;
    if (ty <= 0) return g->perm ? LKB_ERR_SHAPE : LKB_OK;
    if (g_gemm_cfg != 0) {
        const int t = lkb_gemm_tc_launch(g, epi, g_gemm_fold, max_tiles, st, out_rows, a_pitch);
        if (t != LKB_ERR_UNSUPPORTED) return t;
        if (g_gemm_cfg > 0) return t;
    }
    if (out_rows || a_pitch) return LKB_ERR_UNSUPPORTED;   // row targets and packed rows exist in the tensor-core form only
    if (epi) LKB_PF_LAUNCH((k_pf_gemm_simple<1>), dim3(dim3(g->N / 32, ty)), dim3(256), 0, st, *g, g_gemm_fold);
    else     LKB_PF_LAUNCH((k_pf_gemm_simple<0>), dim3(dim3(g->N / 64, ty)), dim3(256), 0, st, *g, g_gemm_fold);
    return lkb_check_launch();
}

extern "C" {

int lkb_pf_gemm_config(int cfg) { g_gemm_cfg = cfg; return LKB_OK; }
int lkb_pf_gemm_arith(int fold) { g_gemm_fold = fold ? 1 : 0; return LKB_OK; }

int lkb_pf_norm(const float * X, const float * w, int plain, lkb_pf_act a, float * inv_out, float * h32,
                int m, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!X || !w || !a.qs || !a.sc || !inv_out) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    if (plain) LKB_PF_LAUNCH(k_pf_token_norm_plain, dim3((m + PF_TOK_WARPS - 1) / PF_TOK_WARPS), dim3(PF_TOK_WARPS * 32), 0, (cudaStream_t) st, X, w, a.qs, reinterpret_cast<float2 *>(a.sc), inv_out, m);
    else       LKB_PF_LAUNCH((k_pf_token_norm<0>), dim3((m + PF_TOK_PER_CTA - 1) / PF_TOK_PER_CTA), dim3(PF_TOK_WARPS * 32), 0, (cudaStream_t) st, const_cast<float *>(X), nullptr, nullptr, nullptr, w, a.qs,
                                                                                  reinterpret_cast<float2 *>(a.sc), inv_out, h32, m);
    return lkb_check_launch();
}

int lkb_pf_quant_rows(const float * X, int ld, int kb, lkb_pf_act a, int rows, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!X || !a.qs || !a.sc) return LKB_ERR_NULL;
    if (rows <= 0 || kb <= 0) return (rows == 0) ? LKB_OK : LKB_ERR_SHAPE;
    if ((ld & 3) || (reinterpret_cast<uintptr_t>(X) & 15)) return LKB_ERR_SHAPE;      // 128-bit loads
    const long long warps = (long long) rows * ((kb + 3) / 4);
    LKB_PF_LAUNCH((k_pf_rows_q8<0>), dim3((unsigned) ((warps + 7) / 8)), dim3(256), 0, (cudaStream_t) st, X, ld, 0, kb, rows, a.qs, reinterpret_cast<float2 *>(a.sc));
    return lkb_check_launch();
}

int lkb_pf_swiglu(const float * Y, int ld, int up_off, int kb, lkb_pf_act a, int rows, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!Y || !a.qs || !a.sc) return LKB_ERR_NULL;
    if (rows <= 0 || kb <= 0) return (rows == 0) ? LKB_OK : LKB_ERR_SHAPE;
    if ((ld & 3) || (up_off & 3) || (reinterpret_cast<uintptr_t>(Y) & 15)) return LKB_ERR_SHAPE;
    const long long warps = (long long) rows * ((kb + 3) / 4);
    LKB_PF_LAUNCH((k_pf_rows_q8<1>), dim3((unsigned) ((warps + 7) / 8)), dim3(256), 0, (cudaStream_t) st, Y, ld, up_off, kb, rows, a.qs, reinterpret_cast<float2 *>(a.sc));
    return lkb_check_launch();
}

static int router_small(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, int * idx, float * w, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!H || !Wr || !bias || !inv || !sel || !sig) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    if (m > 65535) return LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_pf_router_token, dim3(m), dim3(256), 0, (cudaStream_t) st, H, Wr, bias, inv, sel, sig,
                  reinterpret_cast<int4 *>(idx), reinterpret_cast<float4 *>(w));
    return lkb_check_launch();
}

static int router_tiled(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, int * idx, float * w, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!H || !Wr || !bias || !inv || !sel || !sig) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    // The k loop of one CTA is the critical path and its length grows with the tokens per thread, so a token range takes
    // the smallest CTA shape that still fits one wave (measured on B200, us: 8-token CTAs 36 up to 1184 tokens, 66 at 2048;
    // 16-token CTAs 43 up to 2368, 68-78 at 4096; 32-token CTAs 55 at any size up to 4736).  A rank's share of an
    // expert-parallel chunk lands in the first two.  LKB_ROUTER_FORM = 8 / 16 / 32 forces a shape (tuning).
    static const int form = [] { const char * e = getenv("LKB_ROUTER_FORM"); return e ? atoi(e) : 0; }();
    const int sms = lkb_context().sm_count;
    if (form == 8 || (form == 0 && m <= 8 * sms)) return rt_launch<1, 4>(H, m, Wr, bias, inv, sel, sig, idx, w, (cudaStream_t) st);
    if (form == 16 || (form == 0 && m <= 16 * sms)) return rt_launch<RT_S_TPT, RT_S_NW>(H, m, Wr, bias, inv, sel, sig, idx, w, (cudaStream_t) st);
    return rt_launch<RT_L_TPT, RT_L_NW>(H, m, Wr, bias, inv, sel, sig, idx, w, (cudaStream_t) st);
}

int lkb_pf_router_small(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, lkb_stream_t st) {
    return router_small(H, m, Wr, bias, inv, sel, sig, nullptr, nullptr, st);
}
int lkb_pf_router_tiled(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                        float * sel, float * sig, lkb_stream_t st) {
    return router_tiled(H, m, Wr, bias, inv, sel, sig, nullptr, nullptr, st);
}
int lkb_pf_router(const float * H, int m, const float * Wr, const float * bias, const float * inv,
                  float * sel, float * sig, lkb_stream_t st) {
    if (m > 0 && m <= 256) return lkb_pf_router_small(H, m, Wr, bias, inv, sel, sig, st);
    return lkb_pf_router_tiled(H, m, Wr, bias, inv, sel, sig, st);
}
int lkb_pf_router_select(const float * H, int m, int small_form, const float * Wr, const float * bias, const float * inv,
                         float * sel, float * sig, int * idx, float * w, lkb_stream_t st) {
    if (!idx || !w) return LKB_ERR_NULL;
    return small_form ? router_small(H, m, Wr, bias, inv, sel, sig, idx, w, st) : router_tiled(H, m, Wr, bias, inv, sel, sig, idx, w, st);
}

int lkb_pf_select(const float * sel, const float * sig, int m, int * idx, float * w, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!sel || !sig || !idx || !w) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_pf_select, dim3(min((m + 7) / 8, 148 * 8)), dim3(256), 0, (cudaStream_t) st, sel, sig, m, reinterpret_cast<int4 *>(idx), reinterpret_cast<float4 *>(w));
    return lkb_check_launch();
}

int lkb_pf_moe_count(const int * idx, int n, int * cnt, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!idx || !cnt) return LKB_ERR_NULL;
    if (n <= 0) return n == 0 ? LKB_OK : LKB_ERR_SHAPE;
    int grid = (n + 255) / 256; if (grid > 64) grid = 64;
    LKB_PF_LAUNCH(k_pf_moe_count, dim3(grid), dim3(256), 0, (cudaStream_t) st, idx, n, cnt);
    return lkb_check_launch();
}

int lkb_zero_i32(int * p, int n, lkb_stream_t st) {
    if (!p) return LKB_ERR_NULL;
    if (n < 0) return LKB_ERR_SHAPE;
    const cudaError_t e = cudaMemsetAsync(p, 0, (size_t) n * 4, (cudaStream_t) st);
    return e == cudaSuccess ? LKB_OK : -(int) e;
}

int lkb_pf_moe_plan(const int * cnt, int * off, int * tiles, int * ntiles, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!cnt || !off || !tiles || !ntiles) return LKB_ERR_NULL;
    LKB_PF_LAUNCH(k_pf_moe_plan, dim3(1), dim3(32), 0, (cudaStream_t) st, cnt, off, reinterpret_cast<int4 *>(tiles), ntiles);
    return lkb_check_launch();
}

int lkb_pf_moe_scatter(const int * idx, int n, const int * off, int * perm, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!idx || !off || !perm) return LKB_ERR_NULL;
    if (n <= 0) return n == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_pf_moe_scatter, dim3((n + 1023) / 1024), dim3(1024), 0, (cudaStream_t) st, idx, n, off, perm);
    return lkb_check_launch();
}

int lkb_pf_gemm_dense(const lkb_pf_gemm * g, lkb_stream_t st) {
    if (g && g->perm) return LKB_ERR_SHAPE;
    return gemm_dispatch(g, 0, 0, (cudaStream_t) st);
}
int lkb_pf_gemm_moe(const lkb_pf_gemm * g, int max_tiles, lkb_stream_t st) {
    if (g && !g->perm) return LKB_ERR_NULL;
    return gemm_dispatch(g, 0, max_tiles, (cudaStream_t) st);
}
int lkb_pf_gemm_moe_rows(const lkb_pf_gemm * g, int max_tiles, float * const * out_rows, lkb_stream_t st) {
    if (!out_rows) return LKB_ERR_NULL;
    return gemm_dispatch(g, 0, max_tiles, (cudaStream_t) st, out_rows);
}
int lkb_pf_gemm_swiglu_packed(const lkb_pf_gemm * g, int max_tiles, int row_pitch, lkb_stream_t st) {
    if (row_pitch <= 0) return LKB_ERR_SHAPE;
    return gemm_dispatch(g, 1, max_tiles, (cudaStream_t) st, nullptr, row_pitch);
}
int lkb_pf_gemm_swiglu(const lkb_pf_gemm * g, int max_tiles, lkb_stream_t st) {
    return gemm_dispatch(g, 1, max_tiles, (cudaStream_t) st);
}

int lkb_pf_moe_combine(float * X, const float * D, const float * w, int m, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!X || !D || !w) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_pf_moe_combine, dim3(m * (LKB_HIDDEN / 4 / 256)), dim3(256), 0, (cudaStream_t) st, reinterpret_cast<float4 *>(X), reinterpret_cast<const float4 *>(D), w, m);
    return lkb_check_launch();
}

int lkb_pf_moe_combine_norm(float * X, const float * D, const float * w, const float * nw, lkb_pf_act a,
                            float * inv_out, int m, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!X || !D || !w || !nw || !a.qs || !a.sc || !inv_out) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH((k_pf_token_norm<1>), dim3((m + PF_TOK_PER_CTA - 1) / PF_TOK_PER_CTA), dim3(PF_TOK_WARPS * 32), 0, (cudaStream_t) st, X, D, nullptr, w, nw, a.qs, reinterpret_cast<float2 *>(a.sc), inv_out, nullptr, m);
    return lkb_check_launch();
}

int lkb_ep_pack_rows(lkb_pf_act a, const float * inv, const int * idx, const int * send_order, int n,
                     int experts_per_rank, void * out, int * pos, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!a.qs || !a.sc || !inv || !idx || !send_order || !out || !pos) return LKB_ERR_NULL;
    if (n <= 0 || experts_per_rank <= 0) return n == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_ep_pack, dim3(n), dim3(192), 0, (cudaStream_t) st, a.qs, reinterpret_cast<const float2 *>(a.sc), inv, idx, send_order,
                                                experts_per_rank, static_cast<unsigned char *>(out), pos);
    return lkb_check_launch();
}

int lkb_ep_unpack_rows(const void * in, int n, lkb_pf_act a, float * inv, int * local_expert, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!in || !a.qs || !a.sc || !inv || !local_expert) return LKB_ERR_NULL;
    if (n <= 0) return n == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_ep_unpack, dim3(n), dim3(192), 0, (cudaStream_t) st, static_cast<const unsigned char *>(in), a.qs,
                                                  reinterpret_cast<float2 *>(a.sc), inv, local_expert);
    return lkb_check_launch();
}

int lkb_pf_moe_combine_norm_gather(float * X, const float * D, const int * pos, const float * w, const float * nw,
                                   lkb_pf_act a, float * inv_out, int m, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!X || !D || !pos || !w || !nw || !a.qs || !a.sc || !inv_out) return LKB_ERR_NULL;
    if (m <= 0) return m == 0 ? LKB_OK : LKB_ERR_SHAPE;
    LKB_PF_LAUNCH((k_pf_token_norm<2>), dim3((m + PF_TOK_PER_CTA - 1) / PF_TOK_PER_CTA), dim3(PF_TOK_WARPS * 32), 0, (cudaStream_t) st, X, D, pos, w, nw, a.qs, reinterpret_cast<float2 *>(a.sc), inv_out, nullptr, m);
    return lkb_check_launch();
}

int lkb_pf_pack_q8_1(lkb_pf_act a, int t, lkb_block_q8_1 * y, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!a.qs || !a.sc || !y) return LKB_ERR_NULL;
    if (t < 0) return LKB_ERR_SHAPE;
    LKB_PF_LAUNCH(k_pf_pack_q8_1, dim3(1), dim3(512), 0, (cudaStream_t) st, a.qs, reinterpret_cast<const float2 *>(a.sc), t, reinterpret_cast<lkb_q8blk *>(y));
    return lkb_check_launch();
}

}  // extern "C"
