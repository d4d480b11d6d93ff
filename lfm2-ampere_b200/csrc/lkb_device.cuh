// lkb_device.cuh - device primitives shared by the decode and prefill kernels.
//
// Arithmetic contract.  Every fused multiply-add is spelled fmaf() and every
// unfused product / sum uses __fmul_rn / __fadd_rn, so the rounding sequence is
// the one written here whatever the compiler's contraction setting.  The
// sequences are the ones the reference engine evaluates (file:line cited per
// function, relative to the reference repository), so integer results, fp16
// scale fields and -- wherever no approximate intrinsic is involved -- the fp32
// results are bit-identical to the reference's kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/lkb.h"

#define LKB_FULL 0xffffffffu

struct __align__(4) lkb_q8blk {            // == lkb_block_q8_1, device view
    __half2 ds;                            // .x = d, .y = raw sum
    int8_t  qs[32];
};
static_assert(sizeof(lkb_q8blk) == 36, "block_q8_1 is 36 bytes");
static_assert(sizeof(lkb_block_q8_1) == 36, "block_q8_1 is 36 bytes");

// xor-butterfly sum; every lane ends with the same value.  ref: src/kernels.cuh:28-32
__device__ __forceinline__ float lkb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, o));
    return v;
}

// silu with the fast exponential, as the reference.  ref: src/kernels.cuh:33
// (fast __expf, IEEE add and divide).
__device__ __forceinline__ float lkb_silu(float v) { return __fdiv_rn(v, __fadd_rn(1.0f, __expf(-v))); }

// Q8_1 quantiser, one warp per 32-element block, one element per lane.
// ref: src/quant.cuh:106-121.  Returns q for this lane; lane 0 gets (d, sum).
__device__ __forceinline__ int lkb_quant_lane(float xi, float & d_out, float & sum_out) {
    const unsigned am = __reduce_max_sync(LKB_FULL, __float_as_uint(fabsf(xi)));
    sum_out = lkb_warp_sum(xi);
    const float d = __fdiv_rn(__uint_as_float(am), 127.0f);
    d_out = d;
    return (am == 0u) ? 0 : (int) roundf(__fdiv_rn(xi, d));
}

__device__ __forceinline__ void lkb_quant_store(float xi, lkb_q8blk * __restrict__ y, int lane) {
    float d, s;
    const int q = lkb_quant_lane(xi, d, s);
    y->qs[lane] = (int8_t) q;
    if (lane == 0) y->ds = __floats2half2_rn(d, s);
}

// Planar twin.  ref: src/prefill.cu:90-103
__device__ __forceinline__ void lkb_quant_store_planar(float xi, int8_t * __restrict__ qs,
                                                       float2 * __restrict__ sc, int lane) {
    float d, s;
    const int q = lkb_quant_lane(xi, d, s);
    qs[lane] = (int8_t) q;
    if (lane == 0) {
        const __half2 ds = __floats2half2_rn(d, s);
        *sc = make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
    }
}

// The planar quantiser with the block sum in the order of the reference's FUSED SwiGLU epilogue, where a lane holds
// rows g, g+8, g+16, g+24 of the block, adds (v0 + v1) + (v2 + v3) and then exchanges over g ^ 1, 2, 4: in row terms
// the pairing order 8, 16, 1, 2, 4 (ref: src/prefill.cu:424-448).  Same quants and d as the butterfly form; the sum
// differs in its last bits, which the fp16 rounding of the field exposes for about one block in a few thousand.
__device__ __forceinline__ void lkb_quant_store_planar_fused_epilogue(float xi, int8_t * __restrict__ qs,
                                                                      float2 * __restrict__ sc, int lane) {
    float d, s;
    const int q = lkb_quant_lane(xi, d, s);
    qs[lane] = (int8_t) q;
    float v = xi;
    v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, 8));
    v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, 16));
    v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, 1));
    v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(LKB_FULL, v, 4));
    if (lane == 0) {
        const __half2 ds = __floats2half2_rn(d, v);
        *sc = make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
    }
}

// ---------------------------------------------------------------------------
// Four elements per lane.  A 32-element block lives in 8 adjacent lanes, lane l holding elements 4(l&7) .. +3
// (one 128-bit load), so a warp covers four blocks = 512 contiguous bytes per step.  The xor-butterfly of the
// one-element-per-lane form pairs element i with i^16, i^8, i^4, i^2, i^1: here the first three levels are lane
// exchanges (xor 4, 2, 1, one per held element) and the last two are adds inside the thread, so every partial
// sum is the same pair of operands as there (fp32 addition is commutative) and the result has the same bits.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float lkb_quad_sum(float a0, float a1, float a2, float a3) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        a0 = __fadd_rn(a0, __shfl_xor_sync(LKB_FULL, a0, o));
        a1 = __fadd_rn(a1, __shfl_xor_sync(LKB_FULL, a1, o));
        a2 = __fadd_rn(a2, __shfl_xor_sync(LKB_FULL, a2, o));
        a3 = __fadd_rn(a3, __shfl_xor_sync(LKB_FULL, a3, o));
    }
    return __fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a1, a3));
}

// Q8_1 of the block this lane's group of 8 holds: returns the lane's four quants packed low byte first;
// (d, 8 * sum) after the fp16 round trip of the planar layout in sc_out (same in all 8 lanes).
// q = roundf(v / d) without the four IEEE divisions: t = v * rcp(d) is within 3e-5 of the true quotient
// (|q| <= 127, two ulps of relative error), so wherever t is farther than 1e-4 from a half-integer the nearest
// integer of t IS roundf of the IEEE quotient; only the rare element inside that band (and any NaN) takes the
// division (one branch for the lane's four).  The nearest integer comes from the 1.5 * 2^23 trick, whose low mantissa
// byte is q's two's complement.
// lkb_quad_quant_ds hands back the block's (d, raw sum) as the fp16 pair of block_q8_1 instead.
__device__ __forceinline__ unsigned lkb_quad_quant_ds(const float4 v, __half2 & ds_out) {
    const unsigned m01 = max(__float_as_uint(fabsf(v.x)), __float_as_uint(fabsf(v.y)));
    const unsigned m23 = max(__float_as_uint(fabsf(v.z)), __float_as_uint(fabsf(v.w)));
    unsigned am = max(m01, m23);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) am = max(am, __shfl_xor_sync(LKB_FULL, am, o));      // exact, order-free
    const float sum = lkb_quad_sum(v.x, v.y, v.z, v.w);
    const float d = __fdiv_rn(__uint_as_float(am), 127.0f);
    ds_out = __floats2half2_rn(d, sum);
    float rd;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rd) : "f"(d));
    const float MAGIC = 12582912.0f;                     // 1.5 * 2^23: adding it rounds to the nearest (even) integer
    const float vv[4] = {v.x, v.y, v.z, v.w};
    float sft[4];
    bool sure = true;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        sft[k] = fmaf(vv[k], rd, MAGIC);                                  // nearest integer of v * rd, offset by MAGIC
        const float diff = fmaf(vv[k], rd, -__fadd_rn(sft[k], -MAGIC));   // v * rd - that integer
        sure = sure && (fabsf(diff) < 0.4999f);
    }
    if (!sure) {                                         // rare: some element within 1e-4 of a tie, a NaN, or an all-zero block
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float r = roundf(__fdiv_rn(vv[k], d));
            sft[k] = (am != 0u && r == r) ? __fadd_rn(r, MAGIC) : MAGIC;  // (int) NaN is 0; an all-zero block quantises to 0
        }
    }
    return __byte_perm(__byte_perm(__float_as_uint(sft[0]), __float_as_uint(sft[1]), 0x0040),
                       __byte_perm(__float_as_uint(sft[2]), __float_as_uint(sft[3]), 0x0040), 0x5410);
}
__device__ __forceinline__ unsigned lkb_quad_quant(const float4 v, int lane, float2 & sc_out) {
    (void) lane;
    __half2 ds;
    const unsigned pk = lkb_quad_quant_ds(v, ds);
    sc_out = make_float2(__low2float(ds), __fmul_rn(8.0f, __high2float(ds)));
    return pk;
}

// Producer of the scale-carrying norm split: quantise RAW u = x*w, emit the
// block's sum of squares of x.  ref: src/kernels.cuh:421-431
__device__ __forceinline__ void lkb_norm_prod_warp(float xv, float uv, int lane,
                                                   lkb_q8blk * __restrict__ yq8,
                                                   float * __restrict__ ssq, int b) {
    lkb_quant_store(uv, yq8 + b, lane);
    const float sq = lkb_warp_sum(__fmul_rn(xv, xv));
    if (lane == 0) ssq[b] = sq;
}

// Consumer: inv = rsqrt(sum(ssq)/2048 + eps) from 64 partials.  ref: src/kernels.cuh:441-447
__device__ __forceinline__ float lkb_norm_inv(const float * __restrict__ ssq, int lane, float eps) {
    const float s = lkb_warp_sum(__fadd_rn(ssq[lane], ssq[lane + 32]));
    return rsqrtf(fmaf(s, 1.0f / (float) LKB_HIDDEN, eps));
}

// Integer block sum: 16 weight bytes (unsigned nibbles) against 32 int8.
// ref: src/quant.cuh:141-151
__device__ __forceinline__ int lkb_sumi(const uint4 q, const int (&x)[8]) {
    // four independent integer chains (integer addition is exact in any order)
    int s0 = __dp4a((int) (q.x & 0x0F0F0F0Fu), x[0], 0), s1 = __dp4a((int) (q.y & 0x0F0F0F0Fu), x[1], 0);
    int s2 = __dp4a((int) (q.z & 0x0F0F0F0Fu), x[2], 0), s3 = __dp4a((int) (q.w & 0x0F0F0F0Fu), x[3], 0);
    s0 = __dp4a((int) ((q.x >> 4) & 0x0F0F0F0Fu), x[4], s0); s1 = __dp4a((int) ((q.y >> 4) & 0x0F0F0F0Fu), x[5], s1);
    s2 = __dp4a((int) ((q.z >> 4) & 0x0F0F0F0Fu), x[6], s2); s3 = __dp4a((int) ((q.w >> 4) & 0x0F0F0F0Fu), x[7], s3);
    return (s0 + s1) + (s2 + s3);
}

// acc + d4*(d8*sumi - 8*sum): inner = fma(d8, float(sumi), -8sum), acc' = fma(d4, inner, acc).
// ref: src/quant.cuh:154-157; src/prefill.cu:391-399
__device__ __forceinline__ float lkb_block_acc(float d4, float d8, int sumi, float sum8, float acc) {
    return fmaf(d4, fmaf(d8, (float) sumi, -sum8), acc);
}

// The batched-prefill GEMM's form of the same term, as the reference ships it: the integer block sum
// arrives as the fp32 F whose bit pattern is 0x4B400000 + sumi (= 12582912 + sumi, exact for |sumi| < 2^22)
// and the offset is folded into c = fma(d8, 12582912, 8sum): acc' = fma(d4, fma(d8, F, -c), acc).
// ref: src/prefill.cu:32-39,131-139,341-342,381-384
__device__ __forceinline__ float lkb_block_acc_pf(float d4, float d8, int sumi, float sum8, float acc) {
    const float c = fmaf(d8, 12582912.0f, sum8);
    return fmaf(d4, fmaf(d8, __int_as_float(0x4B400000 + sumi), -c), acc);
}

// Streaming 128-bit load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 lkb_ldg_stream(const uint4 * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned short lkb_ldg_stream_u16(const __half * p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float lkb_h2f(unsigned short bits) {
    return __half2float(__ushort_as_half(bits));
}

// Programmatic dependent launch hooks (no-ops when the launch carries no
// programmatic dependency).
__device__ __forceinline__ void lkb_pdl_wait()    { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void lkb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Top-4 of 64 with the reference's tie rule (greater value wins, equal value ->
// lower index), then w_k = sig[idx_k] / max(sum_k, guard).  One warp; every lane
// ends with the full result.  ref: src/kernels.cuh:515-541
__device__ __forceinline__ unsigned lkb_orderable(float f) {       // monotone float -> uint map
    const unsigned u = __float_as_uint(__fadd_rn(f, 0.0f));       // -0 -> +0: equal floats get equal keys
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ void lkb_router_select(const float * __restrict__ sel,
                                                  const float * __restrict__ sig,
                                                  int lane, int * ord, float * wv) {
    // Lane l holds experts l and l+32.  Each round: the maximum over all 64 values by one
    // hardware reduction on order-preserving keys, then the LOWEST expert index holding it
    // (ballot over the low half first) -- the same winner as the reference's butterfly with
    // "greater wins, equal -> lower index", in 3 warp-wide instructions instead of 10 shuffles.
    unsigned k0 = lkb_orderable(sel[lane]), k1 = lkb_orderable(sel[lane + 32]);
    const unsigned gone = lkb_orderable(-1e30f);
#pragma unroll
    for (int r = 0; r < LKB_TOP_K; ++r) {
        const unsigned m = __reduce_max_sync(LKB_FULL, k0 > k1 ? k0 : k1);
        const unsigned lo = __ballot_sync(LKB_FULL, k0 == m);
        const unsigned hi = __ballot_sync(LKB_FULL, k1 == m);
        const int mi = lo ? (__ffs(lo) - 1) : (32 + __ffs(hi) - 1);
        ord[r] = mi;
        if (mi == lane) k0 = gone;
        if (mi == lane + 32) k1 = gone;
    }
    float wsum = 0.0f;
#pragma unroll
    for (int k = 0; k < LKB_TOP_K; ++k) { wv[k] = sig[ord[k]]; wsum = __fadd_rn(wsum, wv[k]); }
    if (wsum < LKB_TOPK_GUARD) wsum = LKB_TOPK_GUARD;
#pragma unroll
    for (int k = 0; k < LKB_TOP_K; ++k) wv[k] = __fdiv_rn(wv[k], wsum);
}

// ---- host-side plumbing shared by the translation units ---------------------
struct lkb_ctx {
    int  inited;
    int  device;
    int  sm_count;
    int  pdl;
};
lkb_ctx & lkb_context();
int lkb_check_launch();        // cudaGetLastError -> status
int lkb_prefill_init();        // per-device attributes of the prefill kernels
int lkb_fused_init();          // ... of the fused decode kernel
int lkb_lmhead_init();         // ... of the Q6_K streaming GEMV
int lkb_mixer_init();          // ... of the decode attention kernel

// Launch helper: optional programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
static int lkb_launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (lkb_context().pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr; cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { (void) cudaGetLastError(); return -(int) e; }
    return LKB_OK;
}
// The prefill chain's launches: programmatic dependent launch when enabled (lkb_set_pdl), so that a kernel's launch
// latency hides behind its predecessor; every kernel launched this way starts with lkb_pdl_wait().
#define LKB_PF_LAUNCH(kern, grid, block, smem, st, ...) \
    do { const int lkb_r_ = lkb_launch(kern, grid, block, smem, st, __VA_ARGS__); if (lkb_r_ != LKB_OK) return lkb_r_; } while (0)

