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

// Warp-level tensor-core step: D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col).
__device__ __forceinline__ void at_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// x = hi + lo with hi, lo fp16: the pair carries x to ~2^-22 relative, so fp16 tensor-core operands lose nothing
// that fp32 arithmetic would have kept.
__device__ __forceinline__ void at_split(float x0, float x1, unsigned & hi, unsigned & lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(__fsub_rn(x0, hf.x), __fsub_rn(x1, hf.y));
    hi = *reinterpret_cast<const unsigned *>(&h);
    lo = *reinterpret_cast<const unsigned *>(&l);
}

// One slice [t0, t1) of one KV head: warps 0..7 of the CTA stream their 32-token groups of K and V through
// private cp.async rings, keep their own online softmax and are merged at the end into
// part[(kvh*4 + h)][sp] = {max, sum, acc[64]}.
// The four query heads of the KV head are the rows of a 16-row tensor-core tile (rows 4..15 are zero): per group
// S = Q K^T is 4 token tiles x 4 dim steps of m16n8k16, O += P V is 2 token steps x 8 dim tiles, with Q and P each
// carried as an fp16 (hi, lo) pair so the products are those of fp32 operands.  Lane (g = lane / 4, t4 = lane % 4)
// with g < 4 owns head g: scores of tokens 8 nt + 2 t4 + {0, 1} and output dims 8 nd + 2 t4 + {0, 1}.  This form needs
// ~300 instructions per group and warp where the scalar form needed ~1000, which is what makes the slice
// HBM-bound instead of issue-bound at long context.
// Every thread of the CTA must call this (it contains CTA barriers); S.q must be filled and visible (a CTA
// barrier after the fill) before the call.
template <int STAGES>
__device__ __forceinline__ void at_slice(AtSmem<STAGES> & S, const __half * __restrict__ kc, const __half * __restrict__ vc,
                                         int kvh, int sp, int t0, int t1, float * __restrict__ part) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const bool worker = warp < AT_WARPS;
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
        // Q fragments (rows 0..3 = heads, scaled by the exact 1/8): register pair kk holds dims 16 kk + 2 t4 + {0,1}
        // (a0) and + 8 (a2) of head g, as hi and lo parts; rows 8..15 (a1, a3) and heads g >= 4 are zero
        unsigned qh0[4], qh2[4], ql0[4], ql2[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const int d0 = kk * 16 + 2 * t4;
            float v0 = 0.0f, v1 = 0.0f, v2 = 0.0f, v3 = 0.0f;
            if (g < AT_GQA) {
                v0 = __fmul_rn(reinterpret_cast<const float *>(&S.q[d0])[g], AT_SCALE);
                v1 = __fmul_rn(reinterpret_cast<const float *>(&S.q[d0 + 1])[g], AT_SCALE);
                v2 = __fmul_rn(reinterpret_cast<const float *>(&S.q[d0 + 8])[g], AT_SCALE);
                v3 = __fmul_rn(reinterpret_cast<const float *>(&S.q[d0 + 9])[g], AT_SCALE);
            }
            at_split(v0, v1, qh0[kk], ql0[kk]);
            at_split(v2, v3, qh2[kk], ql2[kk]);
        }
        float m = -1e30f, l = 0.0f;                         // running max and (per-lane partial) sum of head g
        float o[8][4];
#pragma unroll
        for (int nd = 0; nd < 8; ++nd) { o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.0f; }
        for (int i = 0; i < mine; ++i) {
            issue(i + STAGES - 1);
            at_wait_group<STAGES - 1>();
            __syncwarp();
            const int st = i % STAGES, g0 = t0 + (warp + i * AT_WARPS) * AT_G;
            // S = Q K^T: s[nt][0..1] = scores of head g against tokens g0 + 8 nt + 2 t4 + {0, 1}
            float s[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const __half * kp = &W.k[st][nt * 8 + g][kk * 16 + 2 * t4];
                    const unsigned b0 = *reinterpret_cast<const unsigned *>(kp), b1 = *reinterpret_cast<const unsigned *>(kp + 8);
                    at_mma(s[nt], qh0[kk], 0u, qh2[kk], 0u, b0, b1);
                    at_mma(s[nt], ql0[kk], 0u, ql2[kk], 0u, b0, b1);
                }
            }
            float mx = -1e30f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (g0 + nt * 8 + 2 * t4 + e >= t1) s[nt][e] = -1e30f;      // past the slice
                    mx = fmaxf(mx, s[nt][e]);
                }
            mx = fmaxf(mx, __shfl_xor_sync(LKB_FULL, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(LKB_FULL, mx, 2));
            const float mn = fmaxf(m, mx);
            const float alpha = __expf(__fsub_rn(m, mn));
            m = mn;
            float ls = 0.0f;
            unsigned ph[4], pl[4];                          // P of tokens 8 nt + 2 t4 + {0,1} as fp16 hi / lo pairs
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float p0 = (s[nt][0] <= -1e30f) ? 0.0f : __expf(__fsub_rn(s[nt][0], mn));
                const float p1 = (s[nt][1] <= -1e30f) ? 0.0f : __expf(__fsub_rn(s[nt][1], mn));
                ls = __fadd_rn(ls, __fadd_rn(p0, p1));
                at_split(p0, p1, ph[nt], pl[nt]);
            }
            l = fmaf(l, alpha, ls);
#pragma unroll
            for (int nd = 0; nd < 8; ++nd) { o[nd][0] = __fmul_rn(o[nd][0], alpha); o[nd][1] = __fmul_rn(o[nd][1], alpha); }
            // O += P V: token step ks uses P tiles 2 ks (a0) and 2 ks + 1 (a2); V tiles come transposed from shared memory
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
                for (int nd = 0; nd < 8; nd += 2) {
                    const int mat = lane >> 3, rr = lane & 7;
                    const __half * vp = &W.v[st][ks * 16 + (mat & 1) * 8 + rr][(nd + (mat >> 1)) * 8];
                    unsigned b0, b1, b2, b3;
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"((unsigned) __cvta_generic_to_shared(vp)));
                    at_mma(o[nd], ph[2 * ks], 0u, ph[2 * ks + 1], 0u, b0, b1);
                    at_mma(o[nd], pl[2 * ks], 0u, pl[2 * ks + 1], 0u, b0, b1);
                    at_mma(o[nd + 1], ph[2 * ks], 0u, ph[2 * ks + 1], 0u, b2, b3);
                    at_mma(o[nd + 1], pl[2 * ks], 0u, pl[2 * ks + 1], 0u, b2, b3);
                }
            }
            __syncwarp();
        }
        at_wait_group<0>();
        l = __fadd_rn(l, __shfl_xor_sync(LKB_FULL, l, 1));
        l = __fadd_rn(l, __shfl_xor_sync(LKB_FULL, l, 2));
        // a warp parks its accumulators in its own, now idle, K staging
        __syncwarp();
        float * wacc = reinterpret_cast<float *>(&W.k[0][0][0]);
        if (g < AT_GQA) {
            if (t4 == 0) { S.m[warp][g] = m; S.l[warp][g] = l; }
#pragma unroll
            for (int nd = 0; nd < 8; ++nd) {
                wacc[g * AT_D + nd * 8 + 2 * t4] = o[nd][0];
                wacc[g * AT_D + nd * 8 + 2 * t4 + 1] = o[nd][1];
            }
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
