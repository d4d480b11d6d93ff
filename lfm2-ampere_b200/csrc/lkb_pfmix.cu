// lkb_pfmix.cu - the sequence-mixer kernels of batched prefill for sm_100a: embedding rows, the short gated
// convolution over a chunk, per-head RMSNorm + RoPE + KV append for a chunk, and causal GQA flash attention.
// Together with the dense form of the grouped GEMM (lkb_pf_gemm_dense) they complete a full-model prefill chunk.
//
// The per-token kernels evaluate their decode twins' arithmetic (same helper functions), so a chunk of m tokens
// leaves the same conv history, KV rows and activations as m decode steps would.
// The attention kernel is a first version on the legacy warp-level tensor path (mma.sync m16n8k16, fp16 in,
// fp32 accumulate): 6% of a prefill chunk's multiply-accumulates; a tcgen05 version is future work.
#include "lkb_attn.cuh"

// ref: src/prefill.cu:856-868 (k_pf_embed); grid (n/256, m)
__global__ void __launch_bounds__(256) k_pf_embed(const unsigned char * __restrict__ ql, const unsigned char * __restrict__ qh,
                                                  const int8_t * __restrict__ sc, const __half * __restrict__ d,
                                                  const int * __restrict__ toks, float * __restrict__ x, int n) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int token = toks[t], sbpr = n / 256;
    const size_t blk = (size_t) token * sbpr + i / 256;
    const int e = i % 256;
    const int nn = (e >= 128) ? 128 : 0, r = e - nn;
    const int qlb = ql[blk * 128 + (nn >> 1) + (r & 63)], qhb = qh[blk * 64 + (nn >> 2) + (r & 31)];
    const int q6 = ((r >= 64) ? (qlb >> 4) : (qlb & 15)) | (((qhb >> (2 * (r >> 5))) & 3) << 4);
    x[(size_t) t * n + i] = __fmul_rn(__fmul_rn(__half2float(d[blk]), (float) sc[blk * 16 + e / 16]), (float) (q6 - 32));
}

// Short gated convolution over a chunk.  Y = in_proj output [m][6144] = B | C | X; token t sees bx = B * X of
// tokens t-2 and t-1 (from the chunk, or from the two-tap history for the first two tokens); the output is the
// planar Q8_1 row of v = C * conv.  A warp owns 128 channels (four per lane, 128-bit loads) over a run of
// PF_CONV_RUN consecutive tokens and slides bx of the previous two tokens through registers, so Y is read once
// instead of three times; taps and the fused multiply-add nesting are the decode kernel's, per channel.
// ref semantics: src/prefill.cu:937-957
#ifndef PF_CONV_RUN
#define PF_CONV_RUN 4
#endif
__device__ __forceinline__ float4 pf_mul4(const float4 a, const float4 b) {
    return make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z), __fmul_rn(a.w, b.w));
}
__global__ void __launch_bounds__(128) k_pf_conv_run(const float * __restrict__ Y, const float * __restrict__ cw,
                                                     const float * __restrict__ hist, lkb_pf_act a, int m) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int lane = threadIdx.x & 31;
    const int wid = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int cg = wid & 15, t0 = (wid >> 4) * PF_CONV_RUN;
    if (t0 >= m) return;                                   // warp-uniform
    const int ch = cg * 128 + lane * 4;
    const float4 * c4 = reinterpret_cast<const float4 *>(cw + 3 * ch);
    const float4 f0 = __ldg(c4), f1 = __ldg(c4 + 1), f2 = __ldg(c4 + 2);
    const float tap[12] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w, f2.x, f2.y, f2.z, f2.w};    // [channel][3]
    float4 h0, h1;
    if (t0 == 0) {
        const float4 g0 = *reinterpret_cast<const float4 *>(hist + 2 * ch), g1 = *reinterpret_cast<const float4 *>(hist + 2 * ch + 4);
        h0 = make_float4(g0.x, g0.z, g1.x, g1.z);
        h1 = make_float4(g0.y, g0.w, g1.y, g1.w);
    } else {
        const float * y2 = Y + (size_t) (t0 - 2) * (3 * LKB_HIDDEN) + ch;
        h0 = pf_mul4(*reinterpret_cast<const float4 *>(y2), *reinterpret_cast<const float4 *>(y2 + 2 * LKB_HIDDEN));
        h1 = pf_mul4(*reinterpret_cast<const float4 *>(y2 + 3 * LKB_HIDDEN), *reinterpret_cast<const float4 *>(y2 + 5 * LKB_HIDDEN));
    }
#pragma unroll
    for (int j = 0; j < PF_CONV_RUN; ++j) {
        const int t = t0 + j;
        if (t >= m) break;
        const float * yt = Y + (size_t) t * (3 * LKB_HIDDEN) + ch;
        const float4 bx = pf_mul4(*reinterpret_cast<const float4 *>(yt), *reinterpret_cast<const float4 *>(yt + 2 * LKB_HIDDEN));
        const float4 cv = *reinterpret_cast<const float4 *>(yt + LKB_HIDDEN);
        float4 v;
        v.x = __fmul_rn(cv.x, fmaf(bx.x, tap[2],  fmaf(h1.x, tap[1],  __fmul_rn(h0.x, tap[0]))));
        v.y = __fmul_rn(cv.y, fmaf(bx.y, tap[5],  fmaf(h1.y, tap[4],  __fmul_rn(h0.y, tap[3]))));
        v.z = __fmul_rn(cv.z, fmaf(bx.z, tap[8],  fmaf(h1.z, tap[7],  __fmul_rn(h0.z, tap[6]))));
        v.w = __fmul_rn(cv.w, fmaf(bx.w, tap[11], fmaf(h1.w, tap[10], __fmul_rn(h0.w, tap[9]))));
        float2 s2;
        const unsigned pk = lkb_quad_quant(v, lane, s2);
        reinterpret_cast<unsigned *>(reinterpret_cast<int8_t *>(a.qs) + (size_t) t * LKB_HIDDEN + ch)[0] = pk;
        if ((lane & 7) == 0) reinterpret_cast<float2 *>(a.sc)[(size_t) t * (LKB_HIDDEN / 32) + (ch >> 5)] = s2;
        h0 = h1; h1 = bx;
    }
}

// The history after the chunk: bx of its last two tokens (of the last one and the old second tap when m = 1).
// Runs after the convolution, which reads the old history.  Four channels per thread.
// ref semantics: src/prefill.cu:960-970
__global__ void __launch_bounds__(256) k_pf_conv_hist(const float * __restrict__ Y, int m, float * __restrict__ hist) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int ch = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (ch >= LKB_HIDDEN) return;
    const float * yl = Y + (size_t) (m - 1) * (3 * LKB_HIDDEN) + ch;
    const float4 b1 = pf_mul4(*reinterpret_cast<const float4 *>(yl), *reinterpret_cast<const float4 *>(yl + 2 * LKB_HIDDEN));
    float4 * hp = reinterpret_cast<float4 *>(hist + 2 * ch);
    float4 b0;
    if (m >= 2) {
        const float * yp = yl - 3 * LKB_HIDDEN;
        b0 = pf_mul4(*reinterpret_cast<const float4 *>(yp), *reinterpret_cast<const float4 *>(yp + 2 * LKB_HIDDEN));
    } else {
        const float4 g0 = hp[0], g1 = hp[1];
        b0 = make_float4(g0.y, g0.w, g1.y, g1.w);
    }
    hp[0] = make_float4(b0.x, b1.x, b0.y, b1.y);
    hp[1] = make_float4(b0.z, b1.z, b0.w, b1.w);
}

// Per-head RMSNorm + RoPE of token t at position P + t.  Y = q|k|v GEMM output [m][3072].  Q leaves as fp16
// pre-scaled by 1/8 (exact) for the tensor-core attention; K and V enter the cache exactly as the decode kernel
// writes them.  grid (m, 5) x 256: one warp per head.  ref: src/prefill.cu:975-1016
__global__ void __launch_bounds__(256) k_pf_qknr(const float * __restrict__ Y, const float * __restrict__ qn, const float * __restrict__ kn,
                                                 int P, __half * __restrict__ qh, __half * __restrict__ kc, __half * __restrict__ vc,
                                                 float theta) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    const int t = blockIdx.x, blk = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const bool is_q = blk < AT_HEADS;
    const int head = is_q ? blk : blk - AT_HEADS;
    const float * src = Y + (size_t) t * AT_QKV + (is_q ? head * AT_D : LKB_HIDDEN + head * AT_D);
    float y0, y1;
    at_norm_rope(src[lane], src[lane + 32], is_q ? qn : kn, (float) (P + t), theta, lane, y0, y1);
    if (is_q) {
        __half * q = qh + (size_t) t * LKB_HIDDEN + head * AT_D;
        q[lane] = __float2half(__fmul_rn(y0, AT_SCALE)); q[lane + 32] = __float2half(__fmul_rn(y1, AT_SCALE));
    } else {
        const size_t off = ((size_t) (P + t) * AT_KVH + head) * AT_D;
        const float * v = Y + (size_t) t * AT_QKV + LKB_HIDDEN + AT_KVH * AT_D + head * AT_D;
        kc[off + lane] = __float2half(y0); kc[off + lane + 32] = __float2half(y1);
        vc[off + lane] = __float2half(v[lane]); vc[off + lane + 32] = __float2half(v[lane + 32]);
    }
}

// ---------------------------------------------------------------------------
// Causal GQA flash attention for a chunk of m queries at positions P .. P+m-1 over keys 0 .. P+m-1.
// grid (ceil(m/32), 8 KV heads) x 256.  A CTA owns 32 query positions of one KV head and its four query heads:
// warp w computes head kvh*4 + (w&3), positions q0 + (w>>2)*16 .. +15 (one m16 tile).  K / V tiles of 64 keys are
// double-buffered with cp.async and shared by all eight warps (128 query rows per tile).  Scores live in the
// log2 domain (Q carries the exact 1/8; log2 e is applied in fp32); online softmax; P is rounded to fp16 for
// the P V product (the reference's own choice and error bound, ref: src/prefill.cu:1018-1028).
// ---------------------------------------------------------------------------
#define FA_BQ  32
#define FA_BK  64
#define FA_ROW 72                           // halfs per staged row (144 B: conflict-free fragment reads)

__device__ __forceinline__ void fa_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned fa_pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned *>(&h);
}

__global__ void __launch_bounds__(256, 2) k_pf_attn(const __half * __restrict__ qh, int m, int P, const __half * __restrict__ kc,
                                                    const __half * __restrict__ vc, float * __restrict__ o) {
    lkb_pdl_wait(); lkb_pdl_trigger();           // programmatic dependent launch: inputs complete from here on
    __shared__ __align__(16) __half sK[2][FA_BK][FA_ROW];
    __shared__ __align__(16) __half sV[2][FA_BK][FA_ROW];
    const int qt = gridDim.x - 1 - blockIdx.x;              // longest rows first
    const int kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int head = kvh * AT_GQA + (warp & 3);
    const int q0 = qt * FA_BQ + (warp >> 2) * 16;
    const int qlast = min(qt * FA_BQ + FA_BQ, m);
    const int kend = P + qlast;                             // keys 0 .. kend-1 matter to this CTA
    const int nkt = (kend + FA_BK - 1) / FA_BK;

    // A fragments of the warp's 16 x 64 Q tile: register j of k-step kk holds two consecutive dims of row
    // g + 8 (j & 1) starting at dim 16 kk + 2 t4 + 8 (j >> 1); rows past the chunk read as zero
    unsigned qa[4][4];
    auto q_pair = [&](int row, int dim) -> unsigned {
        return row < m ? *reinterpret_cast<const unsigned *>(qh + (size_t) row * LKB_HIDDEN + head * AT_D + dim) : 0u;
    };
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int j = 0; j < 4; ++j) qa[kk][j] = q_pair(q0 + g + 8 * (j & 1), 16 * kk + 2 * t4 + 8 * (j >> 1));
    auto load = [&](int st, int kt) {                       // 64 keys x 128 B of K and of V: two 16-byte pieces per thread each
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int piece = tid + 256 * i, r = piece >> 3, c = (piece & 7) * 8;
            const int key = kt * FA_BK + r;
            const bool live = key < kend;
            const size_t off = ((size_t) (live ? key : 0) * AT_KVH + kvh) * AT_D + c;
            at_cp16(&sK[st][r][c], kc + off, live ? 16 : 0);    // keys past the end are zero-filled
            at_cp16(&sV[st][r][c], vc + off, live ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float oacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f; }
    float mrow[2] = {-1e30f, -1e30f}, lrow[2] = {0.0f, 0.0f};
    const float LOG2E = 1.4426950408889634f;
    const int row0 = P + q0 + g, row1 = row0 + 8;           // last key each of this lane's two rows may see

    load(0, 0);
    for (int kt = 0; kt < nkt; ++kt) {
        const int st = kt & 1;
        if (kt + 1 < nkt) load(st ^ 1, kt + 1); else asm volatile("cp.async.commit_group;" ::: "memory");
        at_wait_group<1>();
        __syncthreads();
        // S = Q K^T for 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const __half * kp = &sK[st][nt * 8 + g][kk * 16 + 2 * t4];
                fa_mma(s[nt], qa[kk], *reinterpret_cast<const unsigned *>(kp), *reinterpret_cast<const unsigned *>(kp + 8));
            }
        }
        // log2 domain, causal mask (only tiles that reach past the first row's position need it)
        const bool need_mask = kt * FA_BK + FA_BK - 1 > P + q0;
        float mx[2] = {-1e30f, -1e30f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int key = kt * FA_BK + nt * 8 + 2 * t4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * LOG2E;
                if (need_mask && key + (e & 1) > ((e & 2) ? row1 : row0)) v = -1e30f;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(LKB_FULL, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(LKB_FULL, mx[r], 2));
            const float mn = fmaxf(mrow[r], mx[r]);
            alpha[r] = exp2f(mrow[r] - mn);
            mrow[r] = mn;
        }
        float ls[2] = {0.0f, 0.0f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = (s[nt][e] <= -1e30f) ? 0.0f : exp2f(s[nt][e] - mrow[e >> 1]);
                s[nt][e] = p;
                ls[e >> 1] += p;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * alpha[r] + ls[r];
#pragma unroll
        for (int nd = 0; nd < 8; ++nd) { oacc[nd][0] *= alpha[0]; oacc[nd][1] *= alpha[0]; oacc[nd][2] *= alpha[1]; oacc[nd][3] *= alpha[1]; }
        // O += P V: P from the score registers (C layout of two n-tiles == A layout of one k16 step)
#pragma unroll
        for (int k2 = 0; k2 < 4; ++k2) {
            unsigned pa[4];
            pa[0] = fa_pack(s[2 * k2][0], s[2 * k2][1]);
            pa[1] = fa_pack(s[2 * k2][2], s[2 * k2][3]);
            pa[2] = fa_pack(s[2 * k2 + 1][0], s[2 * k2 + 1][1]);
            pa[3] = fa_pack(s[2 * k2 + 1][2], s[2 * k2 + 1][3]);
#pragma unroll
            for (int nd = 0; nd < 8; nd += 2) {
                // four transposed 8x8 pieces of V: keys 16 k2 + {0..7, 8..15} x dims 8 nd + {0..7, 8..15}
                const int mat = lane >> 3, rr = lane & 7;
                const __half * vp = &sV[st][k2 * 16 + (mat & 1) * 8 + rr][(nd + (mat >> 1)) * 8];
                unsigned b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"((unsigned) __cvta_generic_to_shared(vp)));
                fa_mma(oacc[nd], pa, b0, b1);
                fa_mma(oacc[nd + 1], pa, b2, b3);
            }
        }
        __syncthreads();                                    // the tile may be overwritten by the load of kt + 2
    }
    at_wait_group<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        lrow[r] += __shfl_xor_sync(LKB_FULL, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(LKB_FULL, lrow[r], 2);
    }
    const int r0 = q0 + g, r1 = q0 + g + 8;
    const float i0 = 1.0f / lrow[0], i1 = 1.0f / lrow[1];
#pragma unroll
    for (int nd = 0; nd < 8; ++nd) {
        const int c = head * AT_D + nd * 8 + 2 * t4;
        if (r0 < m) *reinterpret_cast<float2 *>(o + (size_t) r0 * LKB_HIDDEN + c) = make_float2(oacc[nd][0] * i0, oacc[nd][1] * i0);
        if (r1 < m) *reinterpret_cast<float2 *>(o + (size_t) r1 * LKB_HIDDEN + c) = make_float2(oacc[nd][2] * i1, oacc[nd][3] * i1);
    }
}

extern "C" {

int lkb_pf_embed(const void * ql, const void * qh, const void * sc, const void * d, const int * toks, float * x, int n, int m,
                 lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!ql || !qh || !sc || !d || !toks || !x) return LKB_ERR_NULL;
    if (n <= 0 || n % 256 || m <= 0) return LKB_ERR_SHAPE;
    return lkb_launch(k_pf_embed, dim3(n / 256, m), dim3(256), 0, (cudaStream_t) st, (const unsigned char *) ql,
                      (const unsigned char *) qh, (const int8_t *) sc, (const __half *) d, toks, x, n);
}

int lkb_pf_conv(const float * Y, const float * cw, const float * hist, lkb_pf_act a, int m, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!Y || !cw || !hist || !a.qs || !a.sc) return LKB_ERR_NULL;
    if (m <= 0) return LKB_ERR_SHAPE;
    const int runs = (m + PF_CONV_RUN - 1) / PF_CONV_RUN;      // 16 warps (channel groups) per run, 4 warps per CTA
    return lkb_launch(k_pf_conv_run, dim3(runs * 4), dim3(128), 0, (cudaStream_t) st, Y, cw, hist, a, m);
}

int lkb_pf_conv_hist(const float * Y, int m, float * hist, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!Y || !hist) return LKB_ERR_NULL;
    if (m <= 0) return LKB_ERR_SHAPE;
    return lkb_launch(k_pf_conv_hist, dim3(LKB_HIDDEN / 1024), dim3(256), 0, (cudaStream_t) st, Y, m, hist);
}

int lkb_pf_qknr(const float * Y, const float * qn, const float * kn, int P, void * qh, void * kc, void * vc, int m, float theta,
                lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!Y || !qn || !kn || !qh || !kc || !vc) return LKB_ERR_NULL;
    if (m <= 0 || P < 0 || !(theta > 1.0f)) return LKB_ERR_SHAPE;
    return lkb_launch(k_pf_qknr, dim3(m, (AT_HEADS + AT_KVH) / 8), dim3(256), 0, (cudaStream_t) st, Y, qn, kn, P,
                      (__half *) qh, (__half *) kc, (__half *) vc, theta);
}

int lkb_pf_attn(const void * qh, int m, int P, const void * kc, const void * vc, float * o, lkb_stream_t st) {
    if (!lkb_context().inited) return LKB_ERR_NOT_INIT;
    if (!qh || !kc || !vc || !o) return LKB_ERR_NULL;
    if (m <= 0 || P < 0) return LKB_ERR_SHAPE;
    return lkb_launch(k_pf_attn, dim3((m + FA_BQ - 1) / FA_BQ, AT_KVH), dim3(256), 0, (cudaStream_t) st,
                      (const __half *) qh, m, P, (const __half *) kc, (const __half *) vc, o);
}

}  // extern "C"
