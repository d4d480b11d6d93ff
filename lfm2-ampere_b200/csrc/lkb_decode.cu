// lkb_decode.cu - batch-1 decode kernels of the Q4_0 x Q8_1 MoE hot path (sm_100a).
//
// All of these are HBM-bound byte/integer work.  Design rules followed here:
//   * weights are streamed with 128-bit no-allocate loads, a whole warp reading
//     512 contiguous bytes per request; every warp keeps R rows (2R requests per
//     lane) in flight before it touches the first one;
//   * the Q8_1 activation a lane needs (blocks lane, lane+32) lives in registers
//     for the whole kernel, so the inner loop is loads + dp4a + two FMAs;
//   * grids are sized from the SM count (one CTA per SM for the large streams;
//     2-CTA clusters where a 32-row Q8_1 output block would otherwise pin the
//     grid to 64 CTAs);
//   * every kernel can run under programmatic dependent launch: weight rows whose
//     address does not depend on the predecessor are requested BEFORE
//     griddepcontrol.wait, activations after it.
// The summation order of every row (lane-strided blocks, then the xor butterfly)
// is the reference's, so outputs are bit-identical to its kernels.
#include <cooperative_groups.h>
#include "lkb_device.cuh"

namespace cg = cooperative_groups;

// ---------------------------------------------------------------------------
// host context
// ---------------------------------------------------------------------------
lkb_ctx & lkb_context() {
    static lkb_ctx c = {0, -1, 0, 0};
    return c;
}
int lkb_check_launch() {
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? LKB_OK : -(int) e;
}

#define LKB_REQUIRE_INIT() do { if (!lkb_context().inited) return LKB_ERR_NOT_INIT; } while (0)

// ---------------------------------------------------------------------------
// Activation registers: the Q8_1 blocks lane, lane+32, ... of one vector.
// ---------------------------------------------------------------------------
template <int NB>
struct XReg {
    int   q[NB][8];
    float d8[NB];
    float s8[NB];        // 8 * raw sum
};

template <int NB>
__device__ __forceinline__ void load_x(const lkb_q8blk * __restrict__ xq, int bpr, int lane, XReg<NB> & x) {
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int k = lane + 32 * j;
        if (k < bpr) {
            const int * p = reinterpret_cast<const int *>(xq + k);     // 36-byte blocks are 4-byte aligned
            const int ds = p[0];
            const __half2 h = *reinterpret_cast<const __half2 *>(&ds);
            x.d8[j] = __low2float(h);
            x.s8[j] = __fmul_rn(8.0f, __high2float(h));
#pragma unroll
            for (int i = 0; i < 8; ++i) x.q[j][i] = p[1 + i];
        } else {
            x.d8[j] = 0.0f; x.s8[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) x.q[j][i] = 0;
        }
    }
}

// R rows at once: request every weight block first, then do the arithmetic.
// Returns per-lane partial sums (before the butterfly).
template <int NB, int R>
__device__ __forceinline__ void rows_partial(const uint4 * const (&qrow)[R], const __half * const (&drow)[R],
                                             int bpr, int lane, const XReg<NB> & x, float (&acc)[R]) {
    uint4 q[R][NB];
    unsigned short d[R][NB];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int k = lane + 32 * j;
            if (k < bpr) { q[r][j] = lkb_ldg_stream(qrow[r] + k); d[r][j] = lkb_ldg_stream_u16(drow[r] + k); }
            else { q[r][j] = make_uint4(0, 0, 0, 0); d[r][j] = 0; }
        }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        float a = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (lane + 32 * j < bpr)
                a = lkb_block_acc(lkb_h2f(d[r][j]), x.d8[j], lkb_sumi(q[r][j], x.q[j]), x.s8[j], a);
        acc[r] = a;
    }
}

// Any bpr: activation read from global/L2 per block (used only for shapes with
// more than 64 blocks per row, e.g. a dense FFN's down projection).
__device__ __forceinline__ float row_partial_generic(const uint4 * __restrict__ qrow, const __half * __restrict__ drow,
                                                     int bpr, int lane, const lkb_q8blk * __restrict__ xq) {
    float a = 0.0f;
    for (int k = lane; k < bpr; k += 32) {
        const uint4 q = lkb_ldg_stream(qrow + k);
        const float d4 = lkb_h2f(lkb_ldg_stream_u16(drow + k));
        const int * p = reinterpret_cast<const int *>(xq + k);
        const int ds = p[0];
        const __half2 h = *reinterpret_cast<const __half2 *>(&ds);
        int xv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = p[1 + i];
        a = lkb_block_acc(d4, __low2float(h), lkb_sumi(q, xv), __fmul_rn(8.0f, __high2float(h)), a);
    }
    return a;
}

// ---------------------------------------------------------------------------
// Multi-segment GEMV: serves k_gemv_q4_0, k_gemv_q4_0_3, k_gemv_q4_0_exp and
// k_gemv_q4_0_exp2.  Logical rows [0, total) are the segments laid end to end;
// each warp owns a contiguous, balanced range of them.
// ref: src/kernels.cu:190-241, 1019-1047, 1049-1124, 1126-1145
// ---------------------------------------------------------------------------
#define LKB_MAX_SEG 8
struct GemvSeg {
    const uint4 *  qs;
    const __half * d;
    float *        y;
    int            rows;
    int            kslot;     // >= 0: weights offset by d_idx[kslot]*rows_per_expert rows, x by kslot*xq_stride
};
struct GemvArgs {
    GemvSeg          seg[LKB_MAX_SEG];
    int              nseg;
    int              total;
    int              bpr;
    const lkb_q8blk * xq;
    int              xq_stride;
    const int *      d_idx;
    int              rows_per_expert;
    int              add_residual;
    int              apply_inv;       // multiply by ninv (1 when ssq == null)
    const float *    ssq;
    float            eps;
    int              idx_from_pred;   // d_idx is written by the immediately preceding kernel
};

template <int NB, int R>
__global__ void __launch_bounds__(512) k_gemv_multi(const GemvArgs a) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long long gw = (long long) blockIdx.x * wpb + (threadIdx.x >> 5);
    const long long nw = (long long) gridDim.x * wpb;
    const int g0 = (int) ((gw * a.total) / nw);
    const int g1 = (int) (((gw + 1) * a.total) / nw);

    lkb_pdl_wait();
    lkb_pdl_trigger();
    if (g0 >= g1) return;

    float ninv = 1.0f;
    if (a.ssq) ninv = lkb_norm_inv(a.ssq, lane, a.eps);

    XReg<NB> x;
    int cur_xoff = -1;
    for (int g = g0; g < g1; ) {
        // A batch is up to R consecutive logical rows that share one activation
        // slice; slots past the batch repeat row 0 (computed, never stored).
        const uint4 * qrow[R]; const __half * drow[R]; float * yp[R];
        int xoff = 0, nvalid = 0;
        bool open = true;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int gg = (g + r < g1) ? g + r : g;
            int s = 0, base = 0;
            while (s + 1 < a.nseg && gg >= base + a.seg[s].rows) { base += a.seg[s].rows; ++s; }
            const int row = gg - base;
            size_t blk = (size_t) row * a.bpr;
            int xo = 0;
            if (a.seg[s].kslot >= 0) {
                blk += (size_t) a.d_idx[a.seg[s].kslot] * a.rows_per_expert * a.bpr;
                xo = a.seg[s].kslot * a.xq_stride;
            }
            if (r == 0) xoff = xo;
            open = open && (g + r < g1) && (xo == xoff);
            if (open) { qrow[r] = a.seg[s].qs + blk; drow[r] = a.seg[s].d + blk; yp[r] = a.seg[s].y + row; ++nvalid; }
            else      { qrow[r] = qrow[0];           drow[r] = drow[0];          yp[r] = nullptr; }
        }
        if (xoff != cur_xoff) { load_x<NB>(a.xq + xoff, a.bpr, lane, x); cur_xoff = xoff; }
        float acc[R];
        rows_partial<NB, R>(qrow, drow, a.bpr, lane, x, acc);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float v = lkb_warp_sum(acc[r]);
            if (r < nvalid) {
                const float o = a.apply_inv ? __fmul_rn(v, ninv) : v;
                if (lane == 0) *yp[r] = a.add_residual ? __fadd_rn(*yp[r], o) : o;
            }
        }
        g += nvalid;
    }
}

__global__ void __launch_bounds__(256) k_gemv_multi_generic(const GemvArgs a) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long long gw = (long long) blockIdx.x * wpb + (threadIdx.x >> 5);
    const long long nw = (long long) gridDim.x * wpb;
    const int g0 = (int) ((gw * a.total) / nw);
    const int g1 = (int) (((gw + 1) * a.total) / nw);
    lkb_pdl_wait();
    lkb_pdl_trigger();
    float ninv = 1.0f;
    if (a.ssq) ninv = lkb_norm_inv(a.ssq, lane, a.eps);
    for (int g = g0; g < g1; ++g) {
        int s = 0, base = 0;
        while (s + 1 < a.nseg && g >= base + a.seg[s].rows) { base += a.seg[s].rows; ++s; }
        const int row = g - base;
        size_t blk = (size_t) row * a.bpr;
        int xo = 0;
        if (a.seg[s].kslot >= 0) {
            blk += (size_t) a.d_idx[a.seg[s].kslot] * a.rows_per_expert * a.bpr;
            xo = a.seg[s].kslot * a.xq_stride;
        }
        const float v = lkb_warp_sum(row_partial_generic(a.seg[s].qs + blk, a.seg[s].d + blk, a.bpr, lane, a.xq + xo));
        const float o = a.apply_inv ? __fmul_rn(v, ninv) : v;
        float * yp = a.seg[s].y + row;
        if (lane == 0) *yp = a.add_residual ? __fadd_rn(*yp, o) : o;
    }
}

static int launch_gemv(GemvArgs & a, cudaStream_t st) {
    LKB_REQUIRE_INIT();
    if (a.bpr <= 0 || a.total <= 0) return LKB_ERR_SHAPE;
    const int sms = lkb_context().sm_count;
    if (a.bpr > 64) {
        const int wpb = 8;
        int grid = (a.total + wpb - 1) / wpb; if (grid > sms * 8) grid = sms * 8;
        return lkb_launch(k_gemv_multi_generic, dim3(grid), dim3(wpb * 32), 0, st, a);
    }
    // one CTA per SM, 16 warps; fewer CTAs when there are fewer rows than warps
    const int wpb = 16;
    int grid = sms;
    const int need = (a.total + wpb - 1) / wpb;
    if (need < grid) grid = need;
    const int rows_per_warp = (a.total + grid * wpb - 1) / (grid * wpb);
    if (a.bpr <= 32) {
        if (rows_per_warp >= 4) return lkb_launch(k_gemv_multi<1, 8>, dim3(grid), dim3(wpb * 32), 0, st, a);
        return lkb_launch(k_gemv_multi<1, 2>, dim3(grid), dim3(wpb * 32), 0, st, a);
    }
    if (rows_per_warp >= 5) return lkb_launch(k_gemv_multi<2, 6>, dim3(grid), dim3(wpb * 32), 0, st, a);
    if (rows_per_warp >= 3) return lkb_launch(k_gemv_multi<2, 4>, dim3(grid), dim3(wpb * 32), 0, st, a);
    if (rows_per_warp >= 2) return lkb_launch(k_gemv_multi<2, 2>, dim3(grid), dim3(wpb * 32), 0, st, a);
    return lkb_launch(k_gemv_multi<2, 1>, dim3(grid), dim3(wpb * 32), 0, st, a);
}

// ---------------------------------------------------------------------------
// Producer GEMVs: a 2-CTA cluster owns 32 consecutive output rows (16 per CTA),
// so 2048 rows spread over 128 CTAs; the second CTA hands its 16 (x, u) values to
// the first through distributed shared memory and one warp there quantises the
// 32-row block.
// ---------------------------------------------------------------------------
struct ProdArgs {
    const uint4 *  qs;
    const __half * d;
    const lkb_q8blk * xq;
    int            out_rows, bpr;
    int            rows_per_expert, xq_stride;
    const int *    d_idx;          // null: plain producer GEMV; else the four experts of a MoE down projection
    const float *  d_w;
    float *        y;              // residual stream / output
    int            add_residual;
    const float *  nw;             // norm weights or null
    float *        h32;
    lkb_q8blk *    yq8;
    float *        ssq;
};

// MoE down projection + weighted sum + residual (+ producer).
// ref: src/kernels.cu:1194-1236.  512 threads: warp w -> expert slot k = w & 3,
// rows (w >> 2)*4 .. +3 of the CTA's 16.
template <int NB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512) k_moe_down_accum(const ProdArgs a) {
    __shared__ float s_dot[4][16];
    __shared__ float s_x[32];
    __shared__ float s_u[32];
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned crank = cluster.block_rank();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int k = w & 3, rg = w >> 2;
    const int row0 = blockIdx.x * 16;

    // The expert ids were written two or more kernels upstream; the weight rows
    // can be requested before the predecessor (the SwiGLU quantiser) finishes.
    const size_t base = (size_t) a.d_idx[k] * a.rows_per_expert * a.bpr;
    const uint4 * qrow[4]; const __half * drow[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const size_t blk = base + (size_t) (row0 + rg * 4 + r) * a.bpr;
        qrow[r] = a.qs + blk; drow[r] = a.d + blk;
    }
    uint4 q[4][NB]; unsigned short d[4][NB];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int kb = lane + 32 * j;
            if (kb < a.bpr) { q[r][j] = lkb_ldg_stream(qrow[r] + kb); d[r][j] = lkb_ldg_stream_u16(drow[r] + kb); }
            else { q[r][j] = make_uint4(0, 0, 0, 0); d[r][j] = 0; }
        }
    lkb_pdl_wait();
    lkb_pdl_trigger();
    XReg<NB> x;
    load_x<NB>(a.xq + (size_t) k * a.xq_stride, a.bpr, lane, x);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (lane + 32 * j < a.bpr)
                acc = lkb_block_acc(lkb_h2f(d[r][j]), x.d8[j], lkb_sumi(q[r][j], x.q[j]), x.s8[j], acc);
        acc = lkb_warp_sum(acc);
        if (lane == 0) s_dot[k][rg * 4 + r] = acc;
    }
    __syncthreads();
    float xv = 0.0f, uv = 0.0f;
    if (threadIdx.x < 16) {
        const int row = row0 + threadIdx.x;
        float acc = 0.0f;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) acc = fmaf(a.d_w[kk], s_dot[kk][threadIdx.x], acc);
        xv = __fadd_rn(a.y[row], acc);
        a.y[row] = xv;
        if (a.nw) {
            uv = __fmul_rn(xv, a.nw[row]);
            if (a.h32) a.h32[row] = uv;
        }
    }
    if (a.nw == nullptr) return;            // uniform over the cluster
    if (threadIdx.x < 16) {
        float * dx = cluster.map_shared_rank(s_x, 0);
        float * du = cluster.map_shared_rank(s_u, 0);
        dx[crank * 16 + threadIdx.x] = xv;
        du[crank * 16 + threadIdx.x] = uv;
    }
    cluster.sync();
    if (crank == 0 && w == 0) lkb_norm_prod_warp(s_x[lane], s_u[lane], lane, a.yq8, a.ssq, blockIdx.x >> 1);
}

// Plain producer GEMV.  ref: src/kernels.cu:318-349.  512 threads, warp w -> row w.
template <int NB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(512) k_gemv_prod(const ProdArgs a) {
    __shared__ float s_x[32];
    __shared__ float s_u[32];
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned crank = cluster.block_rank();
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int row = blockIdx.x * 16 + w;
    const uint4 * qrow = a.qs + (size_t) row * a.bpr;
    const __half * drow = a.d + (size_t) row * a.bpr;
    float acc = 0.0f;
    if constexpr (NB > 0) {
        uint4 q[NB > 0 ? NB : 1]; unsigned short d[NB > 0 ? NB : 1];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int kb = lane + 32 * j;
            if (kb < a.bpr) { q[j] = lkb_ldg_stream(qrow + kb); d[j] = lkb_ldg_stream_u16(drow + kb); }
            else { q[j] = make_uint4(0, 0, 0, 0); d[j] = 0; }
        }
        lkb_pdl_wait();
        lkb_pdl_trigger();
        XReg<(NB > 0 ? NB : 1)> x;
        load_x<(NB > 0 ? NB : 1)>(a.xq, a.bpr, lane, x);
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (lane + 32 * j < a.bpr)
                acc = lkb_block_acc(lkb_h2f(d[j]), x.d8[j], lkb_sumi(q[j], x.q[j]), x.s8[j], acc);
    } else {
        lkb_pdl_wait();
        lkb_pdl_trigger();
        acc = row_partial_generic(qrow, drow, a.bpr, lane, a.xq);
    }
    acc = lkb_warp_sum(acc);
    float xv = 0.0f, uv = 0.0f;
    if (lane == 0) {
        xv = a.add_residual ? __fadd_rn(a.y[row], acc) : acc;
        a.y[row] = xv;
        uv = a.nw ? __fmul_rn(xv, a.nw[row]) : 0.0f;
        if (a.nw && a.h32) a.h32[row] = uv;
    }
    if (a.nw == nullptr) return;
    if (lane == 0) {
        cluster.map_shared_rank(s_x, 0)[crank * 16 + w] = xv;
        cluster.map_shared_rank(s_u, 0)[crank * 16 + w] = uv;
    }
    cluster.sync();
    if (crank == 0 && w == 0) lkb_norm_prod_warp(s_x[lane], s_u[lane], lane, a.yq8, a.ssq, blockIdx.x >> 1);
}

// x += sum_k w_k * down4[k] (+ producer).  ref: src/kernels.cu:1147-1166
__global__ void __launch_bounds__(256) k_moe_accum4(float * __restrict__ dst, const float * __restrict__ down4,
                                                    const float * __restrict__ d_w, int n, const lkb_norm_prod_t np) {
    lkb_pdl_wait();
    lkb_pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;                                   // n % 32 == 0: warp-uniform
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < LKB_TOP_K; ++k) acc = fmaf(d_w[k], down4[(size_t) k * n + i], acc);
    const float xv = __fadd_rn(dst[i], acc);
    dst[i] = xv;
    if (np.w) {
        const float uv = __fmul_rn(xv, np.w[i]);
        if (np.h32) np.h32[i] = uv;
        lkb_norm_prod_warp(xv, uv, lane, reinterpret_cast<lkb_q8blk *>(np.yq8), np.ssq, i >> 5);
    }
}

// ---------------------------------------------------------------------------
// Quantisers / norms
// ---------------------------------------------------------------------------
// ref: src/kernels.cu:165-171
__global__ void __launch_bounds__(256) k_quantize_q8_1(const float * __restrict__ x, lkb_q8blk * __restrict__ y, int nblocks) {
    lkb_pdl_wait();
    lkb_pdl_trigger();
    const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= nblocks) return;
    lkb_quant_store(x[(size_t) b * 32 + lane], y + b, lane);
}

// Fused RMSNorm + Q8_1, n == 2048, one CTA of 256 threads.  ref: src/kernels.cu:68-105
__global__ void __launch_bounds__(256) k_rmsnorm_q8_1(const float * __restrict__ x, const float * __restrict__ w, float eps,
                                                      float * __restrict__ y32, __half * __restrict__ y16,
                                                      lkb_q8blk * __restrict__ yq8) {
    __shared__ float s_sq[256];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float wv[8], xv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = w[tid + j * 256];
    lkb_pdl_wait();
    lkb_pdl_trigger();
#pragma unroll
    for (int j = 0; j < 8; ++j) xv[j] = x[tid + j * 256];
    float sq = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sq = fmaf(xv[j], xv[j], sq);
    s_sq[tid] = sq;
    __syncthreads();
#pragma unroll
    for (int o = 128; o > 16; o >>= 1) {
        if (tid < o) s_sq[tid] = __fadd_rn(s_sq[tid], s_sq[tid + o]);
        __syncthreads();
    }
    if (tid < 32) {
        const float v = lkb_warp_sum(s_sq[tid]);
        if (tid == 0) s_sq[0] = v;
    }
    __syncthreads();
    const float inv = rsqrtf(fmaf(s_sq[0], 1.0f / 2048.0f, eps));
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = tid + j * 256;
        const float t = __fmul_rn(__fmul_rn(xv[j], inv), wv[j]);
        if (y32) y32[i] = t;
        if (y16) y16[i] = __float2half(t);
        if (yq8) lkb_quant_store(t, yq8 + warp + 8 * j, lane);
    }
}

// Stand-alone producer: quantise x*w, emit ssq per 32.  ref: src/kernels.cuh:421-431
__global__ void __launch_bounds__(256) k_norm_prod(const float * __restrict__ x, int n, const lkb_norm_prod_t np) {
    lkb_pdl_wait();
    lkb_pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float xv = x[i];
    const float uv = __fmul_rn(xv, np.w[i]);
    if (np.h32) np.h32[i] = uv;
    lkb_norm_prod_warp(xv, uv, threadIdx.x & 31, reinterpret_cast<lkb_q8blk *>(np.yq8), np.ssq, i >> 5);
}

// silu(gate)*up + Q8_1, with L2 prefetch hints for the down-projection weights.
// ref: src/kernels.cu:488-518
__global__ void __launch_bounds__(256) k_swiglu(const float * __restrict__ gate, const float * __restrict__ up, int n,
                                                float * __restrict__ out, lkb_q8blk * __restrict__ yq8,
                                                const uint4 * __restrict__ pf_qs, const int * __restrict__ pf_idx,
                                                int pf_rows_per_expert, int pf_bpr, long pf_bytes) {
    if (pf_qs && pf_bytes > 0) {
        // pf_idx was written at least two kernels upstream of this one.
        const long expert_bytes = (long) pf_rows_per_expert * pf_bpr * 16;
        const long per = pf_bytes / LKB_TOP_K;
        const long lines = ((per < expert_bytes ? per : expert_bytes) >> 7);
        const long tid = (long) blockIdx.x * blockDim.x + threadIdx.x;
        const long nthr = (long) gridDim.x * blockDim.x;
        for (int k = 0; k < LKB_TOP_K; ++k) {
            const char * base = (const char *) (pf_qs + (size_t) pf_idx[k] * pf_rows_per_expert * pf_bpr);
            for (long i = tid; i < lines; i += nthr) asm volatile("prefetch.global.L2 [%0];" :: "l"(base + (i << 7)));
        }
    }
    lkb_pdl_wait();
    lkb_pdl_trigger();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float g = gate[i];
        const float v = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, __expf(-g))), up[i]);
        if (out) out[i] = v;
        if (yq8) lkb_quant_store(v, yq8 + (i >> 5), threadIdx.x & 31);
    }
}

// ---------------------------------------------------------------------------
// Router
// ---------------------------------------------------------------------------
// 64 CTAs x one warp; the whole 8 KB gate row of an expert is requested before
// the predecessor's output (h) is touched.  ref: src/kernels.cu:583-624
__global__ void __launch_bounds__(32) k_router_dot(const float * __restrict__ h, const float * __restrict__ gate_inp,
                                                   float * __restrict__ logits, const float * __restrict__ bias,
                                                   float * __restrict__ sel, float * __restrict__ sig,
                                                   const float * __restrict__ ssq, float eps) {
    const int e = blockIdx.x, lane = threadIdx.x;
    const float * row = gate_inp + (size_t) e * LKB_HIDDEN;
    float v[LKB_HIDDEN / 32];
#pragma unroll
    for (int j = 0; j < LKB_HIDDEN / 32; ++j) v[j] = __ldg(row + j * 32 + lane);
    lkb_pdl_wait();
    lkb_pdl_trigger();
    float ninv = 1.0f;
    if (ssq) ninv = lkb_norm_inv(ssq, lane, eps);
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < LKB_HIDDEN / 32; ++j) acc = fmaf(v[j], h[j * 32 + lane], acc);
    acc = lkb_warp_sum(acc);
    if (lane == 0) {
        const float l = __fmul_rn(acc, ninv);
        logits[e] = l;
        if (sel) {
            const float g = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-l)));
            sig[e] = g;
            sel[e] = __fadd_rn(g, bias[e]);
        }
    }
}

// ref: src/kernels.cu:629-681 (softmax = 0); softmax = 1 is the synthetic-config gate.
__global__ void __launch_bounds__(64) k_router_top4(const float * __restrict__ logits, const float * __restrict__ bias,
                                                    int * __restrict__ idx_out, float * __restrict__ w_out, int softmax) {
    __shared__ float s_sel[LKB_N_EXPERTS];
    __shared__ float s_sig[LKB_N_EXPERTS];
    lkb_pdl_wait();
    lkb_pdl_trigger();
    const int t = threadIdx.x;
    if (!softmax) {
        const float g = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-logits[t])));
        s_sig[t] = g;
        s_sel[t] = __fadd_rn(g, bias ? bias[t] : 0.0f);
    } else {
        // p = exp(l - max) / sum, the sum taken serially e = 0..63 (one fixed order)
        s_sel[t] = logits[t];
        __syncthreads();
        float mx = s_sel[0];
        for (int e = 1; e < LKB_N_EXPERTS; ++e) mx = fmaxf(mx, s_sel[e]);
        const float p = expf(__fsub_rn(logits[t], mx));
        s_sig[t] = p;
        __syncthreads();
        float den = 0.0f;
        for (int e = 0; e < LKB_N_EXPERTS; ++e) den = __fadd_rn(den, s_sig[e]);
        __syncthreads();
        const float pn = __fdiv_rn(p, den);
        s_sig[t] = pn;
        s_sel[t] = __fadd_rn(pn, bias ? bias[t] : 0.0f);
    }
    __syncthreads();
    if (t >= 32) return;
    int ord[LKB_TOP_K]; float wv[LKB_TOP_K];
    lkb_router_select(s_sel, s_sig, t, ord, wv);
    if (t != 0) return;
#pragma unroll
    for (int k = 0; k < LKB_TOP_K; ++k) { idx_out[k] = ord[k]; w_out[k] = wv[k]; }
}

// Debug tap: S[row][blk].  Warp per row.
__global__ void __launch_bounds__(256) k_block_sumi(const uint4 * __restrict__ qs, const lkb_q8blk * __restrict__ xq,
                                                    int rows, int bpr, int32_t * __restrict__ out) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    for (int k = lane; k < bpr; k += 32) {
        const uint4 q = qs[(size_t) row * bpr + k];
        const int * p = reinterpret_cast<const int *>(xq + k);
        int xv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = p[1 + i];
        out[(size_t) row * bpr + k] = lkb_sumi(q, xv);
    }
}

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
extern "C" {

int lkb_init(int device) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return -(int) e;
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, device);
    if (e != cudaSuccess) return -(int) e;
    if (p.major != 10) return LKB_ERR_DEVICE;
    lkb_ctx & c = lkb_context();
    c.device = device;
    c.sm_count = p.multiProcessorCount;
    int r = lkb_prefill_init();
    if (r != LKB_OK) return r;
    r = lkb_fused_init();
    if (r != LKB_OK) return r;
    r = lkb_lmhead_init();
    if (r != LKB_OK) return r;
    r = lkb_mixer_init();
    if (r != LKB_OK) return r;
    c.inited = 1;
    return LKB_OK;
}

int lkb_sm_count(void) { return lkb_context().sm_count; }
int lkb_set_pdl(int enable) { lkb_context().pdl = enable ? 1 : 0; return LKB_OK; }

const char * lkb_error_string(int s) {
    switch (s) {
    case LKB_OK: return "ok";
    case LKB_ERR_SHAPE: return "shape precondition violated";
    case LKB_ERR_NULL: return "required pointer is null";
    case LKB_ERR_UNSUPPORTED: return "mode not built";
    case LKB_ERR_NOT_INIT: return "lkb_init() has not run";
    case LKB_ERR_DEVICE: return "not an sm_100 device";
    case LKB_ERR_TIMEOUT: return "bounded device wait gave up";
    case LKB_ERR_SCRATCH: return "shape needs more scratch than the built-in array (LKB_STATIC_SCRATCH_BYTES) holds";
    default: return s < 0 ? cudaGetErrorString((cudaError_t) (-s)) : "unknown";
    }
}

int lkb_quantize_q8_1(const float * x, lkb_block_q8_1 * y, int nblocks, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!x || !y) return LKB_ERR_NULL;
    if (nblocks <= 0) return nblocks == 0 ? LKB_OK : LKB_ERR_SHAPE;
    return lkb_launch(k_quantize_q8_1, dim3((nblocks + 7) / 8), dim3(256), 0, (cudaStream_t) st,
                      x, reinterpret_cast<lkb_q8blk *>(y), nblocks);
}

int lkb_rmsnorm_q8_1(const float * x, const float * w, int n, float eps, float * y32, void * y16,
                     lkb_block_q8_1 * yq8, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!x || !w) return LKB_ERR_NULL;
    if (n != LKB_HIDDEN) return LKB_ERR_SHAPE;
    return lkb_launch(k_rmsnorm_q8_1, dim3(1), dim3(256), 0, (cudaStream_t) st, x, w, eps, y32,
                      reinterpret_cast<__half *>(y16), reinterpret_cast<lkb_q8blk *>(yq8));
}

int lkb_norm_produce(const float * x, int n, const lkb_norm_prod_t * np, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!x || !np || !np->w || !np->yq8 || !np->ssq) return LKB_ERR_NULL;
    if (n <= 0 || n % 32) return LKB_ERR_SHAPE;
    return lkb_launch(k_norm_prod, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t) st, x, n, *np);
}

int lkb_gemv_q4_0(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                  float * y, int add_residual, const float * ssq, float eps, lkb_stream_t st) {
    if (!qs || !d || !xq || !y) return LKB_ERR_NULL;
    GemvArgs a = {};
    a.seg[0] = { (const uint4 *) qs, (const __half *) d, y, out_rows, -1 };
    a.nseg = 1; a.total = out_rows; a.bpr = bpr; a.xq = (const lkb_q8blk *) xq;
    a.add_residual = add_residual; a.apply_inv = 1; a.ssq = ssq; a.eps = eps;
    return launch_gemv(a, (cudaStream_t) st);
}

int lkb_gemv_q4_0_3(const void * qs0, const void * d0, int rows0, float * y0,
                    const void * qs1, const void * d1, int rows1, float * y1,
                    const void * qs2, const void * d2, int rows2, float * y2,
                    const lkb_block_q8_1 * xq, int bpr, const float * ssq, float eps, lkb_stream_t st) {
    if (!qs0 || !qs1 || !qs2 || !d0 || !d1 || !d2 || !y0 || !y1 || !y2 || !xq) return LKB_ERR_NULL;
    if (rows0 <= 0 || rows1 <= 0 || rows2 <= 0) return LKB_ERR_SHAPE;
    GemvArgs a = {};
    a.seg[0] = { (const uint4 *) qs0, (const __half *) d0, y0, rows0, -1 };
    a.seg[1] = { (const uint4 *) qs1, (const __half *) d1, y1, rows1, -1 };
    a.seg[2] = { (const uint4 *) qs2, (const __half *) d2, y2, rows2, -1 };
    a.nseg = 3; a.total = rows0 + rows1 + rows2; a.bpr = bpr; a.xq = (const lkb_q8blk *) xq;
    a.apply_inv = 1; a.ssq = ssq; a.eps = eps;
    return launch_gemv(a, (cudaStream_t) st);
}

int lkb_gemv_q4_0_exp2(const void * qs_a, const void * d_a, const void * qs_b, const void * d_b,
                       const lkb_block_q8_1 * xq, int out_rows, int bpr, int rows_per_expert, int xq_stride,
                       const int * d_idx, const float * sel, const float * sig, int * idx_out, float * w_out,
                       float * y_a, float * y_b, const float * ssq, float eps, lkb_stream_t st) {
    if (sel || sig || idx_out || w_out) return LKB_ERR_UNSUPPORTED;
    if (!qs_a || !d_a || !qs_b || !d_b || !xq || !d_idx || !y_a || !y_b) return LKB_ERR_NULL;
    GemvArgs a = {};
    for (int half = 0; half < 2; ++half)
        for (int k = 0; k < LKB_TOP_K; ++k)
            a.seg[half * 4 + k] = { (const uint4 *) (half ? qs_b : qs_a), (const __half *) (half ? d_b : d_a),
                                    (half ? y_b : y_a) + (size_t) k * out_rows, out_rows, k };
    a.nseg = 8; a.total = 8 * out_rows; a.bpr = bpr; a.xq = (const lkb_q8blk *) xq; a.xq_stride = xq_stride;
    a.d_idx = d_idx; a.rows_per_expert = rows_per_expert; a.apply_inv = 1; a.ssq = ssq; a.eps = eps;
    return launch_gemv(a, (cudaStream_t) st);
}

int lkb_gemv_q4_0_exp(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                      int rows_per_expert, int xq_stride, const int * d_idx, float * y, lkb_stream_t st) {
    if (!qs || !d || !xq || !d_idx || !y) return LKB_ERR_NULL;
    GemvArgs a = {};
    for (int k = 0; k < LKB_TOP_K; ++k)
        a.seg[k] = { (const uint4 *) qs, (const __half *) d, y + (size_t) k * out_rows, out_rows, k };
    a.nseg = 4; a.total = 4 * out_rows; a.bpr = bpr; a.xq = (const lkb_q8blk *) xq; a.xq_stride = xq_stride;
    a.d_idx = d_idx; a.rows_per_expert = rows_per_expert; a.apply_inv = 0;
    return launch_gemv(a, (cudaStream_t) st);
}

static int prod_common(ProdArgs & a, const lkb_norm_prod_t * np) {
    if (np && np->w) {
        if (!np->yq8 || !np->ssq) return LKB_ERR_NULL;
        a.nw = np->w; a.h32 = np->h32; a.yq8 = reinterpret_cast<lkb_q8blk *>(np->yq8); a.ssq = np->ssq;
    }
    if (a.out_rows <= 0 || a.out_rows % 32 || a.bpr <= 0) return LKB_ERR_SHAPE;
    return LKB_OK;
}

int lkb_gemv_q4_0_prod(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                       float * y, int add_residual, const lkb_norm_prod_t * np, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!qs || !d || !xq || !y) return LKB_ERR_NULL;
    ProdArgs a = {};
    a.qs = (const uint4 *) qs; a.d = (const __half *) d; a.xq = (const lkb_q8blk *) xq;
    a.out_rows = out_rows; a.bpr = bpr; a.y = y; a.add_residual = add_residual;
    const int r = prod_common(a, np);
    if (r != LKB_OK) return r;
    const dim3 grid(out_rows / 16), block(512);
    if (bpr <= 32) return lkb_launch(k_gemv_prod<1>, grid, block, 0, (cudaStream_t) st, a);
    if (bpr <= 64) return lkb_launch(k_gemv_prod<2>, grid, block, 0, (cudaStream_t) st, a);
    return lkb_launch(k_gemv_prod<0>, grid, block, 0, (cudaStream_t) st, a);
}

int lkb_moe_down_accum(const void * qs, const void * d, const lkb_block_q8_1 * xq, int out_rows, int bpr,
                       int rows_per_expert, int xq_stride, const int * d_idx, const float * d_w,
                       float * dst, const lkb_norm_prod_t * np, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!qs || !d || !xq || !d_idx || !d_w || !dst) return LKB_ERR_NULL;
    if (bpr > 64) return LKB_ERR_SHAPE;
    ProdArgs a = {};
    a.qs = (const uint4 *) qs; a.d = (const __half *) d; a.xq = (const lkb_q8blk *) xq;
    a.out_rows = out_rows; a.bpr = bpr; a.rows_per_expert = rows_per_expert; a.xq_stride = xq_stride;
    a.d_idx = d_idx; a.d_w = d_w; a.y = dst; a.add_residual = 1;
    const int r = prod_common(a, np);
    if (r != LKB_OK) return r;
    const dim3 grid(out_rows / 16), block(512);
    if (bpr <= 32) return lkb_launch(k_moe_down_accum<1>, grid, block, 0, (cudaStream_t) st, a);
    return lkb_launch(k_moe_down_accum<2>, grid, block, 0, (cudaStream_t) st, a);
}

int lkb_moe_accum4(float * dst, const float * down4, const float * d_w, int n, const lkb_norm_prod_t * np,
                   lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!dst || !down4 || !d_w) return LKB_ERR_NULL;
    if (n <= 0 || n % 32) return LKB_ERR_SHAPE;
    lkb_norm_prod_t p = {};
    if (np) p = *np;
    if (p.w && (!p.yq8 || !p.ssq)) return LKB_ERR_NULL;
    return lkb_launch(k_moe_accum4, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t) st, dst, down4, d_w, n, p);
}

int lkb_swiglu(const float * gate, const float * up, int n, float * out, lkb_block_q8_1 * yq8,
               const void * pf_qs, const int * pf_idx, int pf_rows_per_expert, int pf_bpr, long pf_bytes,
               lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!gate || !up) return LKB_ERR_NULL;
    if (n <= 0 || n % 32) return LKB_ERR_SHAPE;
    if (pf_qs && pf_bytes > 0 && !pf_idx) return LKB_ERR_NULL;
    return lkb_launch(k_swiglu, dim3((n + 255) / 256), dim3(256), 0, (cudaStream_t) st, gate, up, n, out,
                      reinterpret_cast<lkb_q8blk *>(yq8), (const uint4 *) pf_qs, pf_idx, pf_rows_per_expert, pf_bpr, pf_bytes);
}

int lkb_router_dot(const float * h, const float * gate_inp, float * logits, const float * bias,
                   float * sel, float * sig, const float * ssq, float eps, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!h || !gate_inp || !logits) return LKB_ERR_NULL;
    if ((sel != nullptr) != (sig != nullptr)) return LKB_ERR_NULL;
    if (sel && !bias) return LKB_ERR_NULL;
    return lkb_launch(k_router_dot, dim3(LKB_N_EXPERTS), dim3(32), 0, (cudaStream_t) st, h, gate_inp, logits, bias,
                      sel, sig, ssq, eps);
}

int lkb_router_top4(const float * logits, const float * bias, int * idx_out, float * w_out, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!logits || !bias || !idx_out || !w_out) return LKB_ERR_NULL;
    return lkb_launch(k_router_top4, dim3(1), dim3(LKB_N_EXPERTS), 0, (cudaStream_t) st, logits, bias, idx_out, w_out, 0);
}

int lkb_router_top4_softmax(const float * logits, const float * bias, int * idx_out, float * w_out, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!logits || !idx_out || !w_out) return LKB_ERR_NULL;
    return lkb_launch(k_router_top4, dim3(1), dim3(LKB_N_EXPERTS), 0, (cudaStream_t) st, logits, bias, idx_out, w_out, 1);
}

int lkb_block_sumi(const void * qs, const lkb_block_q8_1 * xq, int rows, int bpr, int32_t * out, lkb_stream_t st) {
    LKB_REQUIRE_INIT();
    if (!qs || !xq || !out) return LKB_ERR_NULL;
    if (rows <= 0 || bpr <= 0) return LKB_ERR_SHAPE;
    k_block_sumi<<<(rows + 7) / 8, 256, 0, (cudaStream_t) st>>>((const uint4 *) qs, (const lkb_q8blk *) xq, rows, bpr, out);
    return lkb_check_launch();
}

}  // extern "C"
