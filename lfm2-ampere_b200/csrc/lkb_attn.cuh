// lkb_attn.cuh - device code of the decode attention shared by the stand-alone kernels (lkb_mixer.cu) and the
// whole-step persistent kernel (lkb_fused.cu): slice rule, per-head RMSNorm + NEOX RoPE, one slice's partial
// (m, l, acc[64]) for the four query heads of a KV head, and the merge of the slices.  Both users evaluate the
// same operations in the same order, so their results are bit-identical.
#pragma once
#include "lkb_device.cuh"

#define AT_HEADS   32
#define AT_KVH     8
#define AT_GQA     4
#define AT_D       64
#define AT_WARPS   8                        // warps that work on a slice
#define AT_G       32                       // tokens per warp group
#define AT_ROW     72                       // halfs per staged row: 64 + 8 padding (144 B: conflict-free 16-B reads)
#define AT_SCALE   0.125f                   // 1/sqrt(64), exact.  ref: src/kernels.cuh:24
#define AT_QKV     (LKB_HIDDEN + 2 * AT_KVH * AT_D)   // 3072: one token's q | k | v

__host__ __device__ __forceinline__ int at_slices(int seq_len) {
    int s = (seq_len + 255) / 256;
    if (s < 1) s = 1;
    if (s > LKB_ATTN_SPLIT) s = LKB_ATTN_SPLIT;
    return s;
}
// tokens per slice: whole 32-token groups
__host__ __device__ __forceinline__ int at_chunk(int seq_len, int nsl) { return (((seq_len + nsl - 1) / nsl) + AT_G - 1) / AT_G * AT_G; }

template <int STAGES>
struct AtWarp {
    __half k[STAGES][AT_G][AT_ROW];
    __half v[STAGES][AT_G][AT_ROW];
    float4 p[AT_G];
};
template <int STAGES>
struct AtSmem {
    AtWarp<STAGES> w[AT_WARPS];
    float4 q[AT_D];                         // q[d] = the four heads' values of dim d
    float  m[AT_WARPS][AT_GQA], l[AT_WARPS][AT_GQA];
};

__device__ __forceinline__ void at_cp16(void * dst, const void * src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"((unsigned) __cvta_generic_to_shared(dst)), "l"(src), "r"(bytes) : "memory");
}
template <int N> __device__ __forceinline__ void at_wait_group() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// RMSNorm over the 64 dims of one head with weights nw, then the NEOX half-split rotation at position pos.
// One warp; lane i holds dims i (a) and i + 32 (b), the pair that rotates together; returns the rotated pair.
// The sum of squares follows the halving tree s[i] += s[i + o] (o = 32..1), whose root is what lane 0 of an
// xor butterfly holds.  ref: src/kernels.cu:871-915, src/kernels.cuh:35-54
__device__ __forceinline__ void at_norm_rope(float a, float b, const float * __restrict__ nw, float pos, float theta, int lane,
                                             float & y0, float & y1) {
    float ss = __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b));
    ss = __shfl_sync(LKB_FULL, lkb_warp_sum(ss), 0);
    const float inv = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float) AT_D), 1e-5f));
    const float x0 = __fmul_rn(__fmul_rn(a, inv), nw[lane]), x1 = __fmul_rn(__fmul_rn(b, inv), nw[lane + 32]);
    const float invf = powf(theta, __fdiv_rn(__fmul_rn(-2.0f, (float) lane), (float) AT_D));
    float sn, cs;
    sincosf(__fmul_rn(pos, invf), &sn, &cs);                // precise form: large arguments (ref: src/kernels.cuh:45-48)
    y0 = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
    y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
}

// One slice [t0, t1) of one KV head: warps 0..7 of the CTA stream their 32-token groups of K and V through
// private cp.async rings, keep their own online softmax and are merged at the end into
// part[(kvh*4 + h)][sp] = {max, sum, acc[64]}.  Every thread of the CTA must call this (it contains CTA
// barriers); S.q must be filled and visible (a CTA barrier after the fill) before the call.
template <int STAGES>
__device__ __forceinline__ void at_slice(AtSmem<STAGES> & S, const __half * __restrict__ kc, const __half * __restrict__ vc,
                                         int kvh, int sp, int t0, int t1, float * __restrict__ part) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool worker = warp < AT_WARPS;
    float m[AT_GQA], l[AT_GQA], acc[AT_GQA][2];
#pragma unroll
    for (int h = 0; h < AT_GQA; ++h) { m[h] = -1e30f; l[h] = 0.0f; acc[h][0] = acc[h][1] = 0.0f; }
    if (worker) {
        AtWarp<STAGES> & W = S.w[warp];
        const int ngrp = (t1 - t0 + AT_G - 1) / AT_G;       // groups of this slice; warp w owns w, w+8, ...
        const int mine = (ngrp - warp + AT_WARPS - 1) / AT_WARPS;
        const size_t tstride = (size_t) AT_KVH * AT_D;      // halfs between consecutive tokens
        const __half * kbase = kc + (size_t) kvh * AT_D, * vbase = vc + (size_t) kvh * AT_D;
        auto issue = [&](int i) {                           // group i of this warp -> stage i % STAGES
            if (i < mine) {
                const int st = i % STAGES, g0 = t0 + (warp + i * AT_WARPS) * AT_G;
                const size_t off0 = (size_t) (g0 + (lane >> 3)) * tstride + (lane & 7) * 8;
#pragma unroll
                for (int r = 0; r < 8; ++r) {
                    const int j = r * 4 + (lane >> 3);
                    const bool live = g0 + j < t1;
                    // dead rows are zero-filled (size 0) from an address that is always inside the cache
                    const size_t off = live ? off0 + (size_t) r * 4 * tstride : (size_t) t0 * tstride;
                    at_cp16(&W.k[st][j][(lane & 7) * 8], kbase + off, live ? 16 : 0);
                    at_cp16(&W.v[st][j][(lane & 7) * 8], vbase + off, live ? 16 : 0);
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
#pragma unroll
        for (int i = 0; i < STAGES - 1; ++i) issue(i);
        for (int i = 0; i < mine; ++i) {
            issue(i + STAGES - 1);
            at_wait_group<STAGES - 1>();
            __syncwarp();
            const int st = i % STAGES, g0 = t0 + (warp + i * AT_WARPS) * AT_G;
            const bool live = g0 + lane < t1;
            // scores of token g0 + lane against the four heads.  q is re-read from shared memory in every
            // iteration (the opaque zero stops the compiler from hoisting 64 float4 into registers).
            int zero;
            asm volatile("mov.u32 %0, 0;" : "=r"(zero));
            const float4 * Q = S.q + zero;
            float s[AT_GQA] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 2
            for (int c = 0; c < 8; ++c) {
                const uint4 kw = *reinterpret_cast<const uint4 *>(&W.k[st][lane][c * 8]);
                const __half2 * k2 = reinterpret_cast<const __half2 *>(&kw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 kf = __half22float2(k2[e]);
                    const float4 qa = Q[c * 8 + 2 * e], qb = Q[c * 8 + 2 * e + 1];
                    s[0] = fmaf(qa.x, kf.x, s[0]); s[1] = fmaf(qa.y, kf.x, s[1]); s[2] = fmaf(qa.z, kf.x, s[2]); s[3] = fmaf(qa.w, kf.x, s[3]);
                    s[0] = fmaf(qb.x, kf.y, s[0]); s[1] = fmaf(qb.y, kf.y, s[1]); s[2] = fmaf(qb.z, kf.y, s[2]); s[3] = fmaf(qb.w, kf.y, s[3]);
                }
            }
            float sc[AT_GQA], pr[AT_GQA];
#pragma unroll
            for (int h = 0; h < AT_GQA; ++h) {
                s[h] = live ? __fmul_rn(s[h], AT_SCALE) : -1e30f;
                float mx = s[h];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(LKB_FULL, mx, o));
                const float mn = fmaxf(m[h], mx);
                sc[h] = __expf(__fsub_rn(m[h], mn));
                pr[h] = live ? __expf(__fsub_rn(s[h], mn)) : 0.0f;
                l[h] = fmaf(l[h], sc[h], lkb_warp_sum(pr[h]));
                m[h] = mn;
            }
            W.p[lane] = make_float4(pr[0], pr[1], pr[2], pr[3]);
            __syncwarp();
            // acc[h][dims 2*lane, 2*lane+1] = acc * sc + sum_j p[j][h] * V[j][dims]
#pragma unroll
            for (int h = 0; h < AT_GQA; ++h) { acc[h][0] = __fmul_rn(acc[h][0], sc[h]); acc[h][1] = __fmul_rn(acc[h][1], sc[h]); }
#pragma unroll 8
            for (int j = 0; j < AT_G; ++j) {
                const float2 vf = __half22float2(*reinterpret_cast<const __half2 *>(&W.v[st][j][2 * lane]));
                const float4 p = W.p[j];
                acc[0][0] = fmaf(p.x, vf.x, acc[0][0]); acc[0][1] = fmaf(p.x, vf.y, acc[0][1]);
                acc[1][0] = fmaf(p.y, vf.x, acc[1][0]); acc[1][1] = fmaf(p.y, vf.y, acc[1][1]);
                acc[2][0] = fmaf(p.z, vf.x, acc[2][0]); acc[2][1] = fmaf(p.z, vf.y, acc[2][1]);
                acc[3][0] = fmaf(p.w, vf.x, acc[3][0]); acc[3][1] = fmaf(p.w, vf.y, acc[3][1]);
            }
            __syncwarp();
        }
        at_wait_group<0>();
        // a warp parks its accumulators in its own, now idle, K staging
        __syncwarp();
        float * wacc = reinterpret_cast<float *>(&W.k[0][0][0]);
#pragma unroll
        for (int h = 0; h < AT_GQA; ++h) {
            if (lane == 0) { S.m[warp][h] = m[h]; S.l[warp][h] = l[h]; }
            wacc[h * AT_D + 2 * lane] = acc[h][0]; wacc[h * AT_D + 2 * lane + 1] = acc[h][1];
        }
    }
    __syncthreads();
    if (worker) {                                           // merge the eight warps: thread = (head h, dim d)
        const int h = tid >> 6, d = tid & 63;
        float M = -1e30f;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) M = fmaxf(M, S.m[w][h]);
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < AT_WARPS; ++w) {
            const float e = __expf(__fsub_rn(S.m[w][h], M));
            L = fmaf(S.l[w][h], e, L);
            A = fmaf(reinterpret_cast<const float *>(&S.w[w].k[0][0][0])[h * AT_D + d], e, A);
        }
        float * P = part + ((size_t) (kvh * AT_GQA + h) * LKB_ATTN_SPLIT + sp) * LKB_ATTN_PARTW;
        if (d == 0) { P[0] = M; P[1] = L; }
        P[2 + d] = A;
    }
}

// Output (head, d) from the live slices' partials: M = max m_s; L = sum l_s e_s; A = sum a_s e_s with
// e_s = exp(m_s - M), both sums as fma chains over ascending s; result A / L.  All loads of a pass are issued
// before the first is used (fixed trip count, predicated), so the merge costs two memory round trips.
// ref: src/kernels.cu:1562-1599
__device__ __forceinline__ float at_combine(const float * __restrict__ part, int head, int d, int seq_len) {
    const int nsl = at_slices(seq_len);
    const int chunk = at_chunk(seq_len, nsl);
    const int nlive = min(nsl, (seq_len + chunk - 1) / chunk);
    const float * P = part + (size_t) head * LKB_ATTN_SPLIT * LKB_ATTN_PARTW;
    float mv[LKB_ATTN_SPLIT], lv[LKB_ATTN_SPLIT], av[LKB_ATTN_SPLIT];
#pragma unroll
    for (int s = 0; s < LKB_ATTN_SPLIT; ++s) {
        const bool live = s < nlive;
        mv[s] = live ? __ldcg(P + s * LKB_ATTN_PARTW) : -1e30f;
        lv[s] = live ? __ldcg(P + s * LKB_ATTN_PARTW + 1) : 0.0f;
        av[s] = live ? __ldcg(P + s * LKB_ATTN_PARTW + 2 + d) : 0.0f;
    }
    float M = -1e30f;
#pragma unroll
    for (int s = 0; s < LKB_ATTN_SPLIT; ++s) M = fmaxf(M, mv[s]);
    float L = 0.0f, A = 0.0f;
#pragma unroll
    for (int s = 0; s < LKB_ATTN_SPLIT; ++s) {
        if (s < nlive) {
            const float e = __expf(__fsub_rn(mv[s], M));
            L = fmaf(lv[s], e, L);
            A = fmaf(av[s], e, A);
        }
    }
    return __fdiv_rn(A, L);
}
