/*
 * lkb_oracle.c - CPU restatement of the Q4_0 x Q8_1 MoE hot path of lfm2-ampere.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It exists so that the CUDA
 * kernels can be checked against an independent statement of the reference's
 * arithmetic.  Only the test-suite, the smoke check and the benchmark's
 * cpu-baseline leg may load it; the shipped library never links or calls it.
 *
 * Parity status: PINNED.  The functions below reproduce (i) the four Q4_0
 * known-answer cases of the reference's ref/quant_fixture.bin, (ii) the router
 * decision on the reference's real 64x2048 gate matrix + bias
 * (ref/kernel_fixture.bin with the input stream of tests/test_kernels.cu:19-24),
 * and (iii) vectors produced by executing the reference's own numpy helpers
 * (tools/ref_forward.py q8_1 / q4_mv_q8).  The pins are checked by
 * tests/test_oracle_golden.py from fixtures committed under tests/golden/.
 *
 * Floating-point contract.  Compile with -ffp-contract=off: every fused
 * multiply-add below is written as fmaf() and every unfused product/sum is a
 * separate statement, so the rounding sequence is exactly what is written.  The
 * sequence is the one the reference's kernels evaluate on the GPU (nvcc fuses
 * `a += b*c` into one FMA; the prefill GEMM spells its FMAs out).  Three device
 * functions are approximations on the GPU (rsqrtf, expf, __expf); wherever one
 * of them feeds a result, the function takes the GPU's value as an optional
 * override so that everything downstream can still be compared bit for bit.
 *
 * Each function cites the reference source it restates as <file>:<lines>,
 * paths relative to the reference repository root.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32, round-to-nearest-even, subnormals kept (what                */
/* __floats2half2_rn / __half2float do; src/quant.cuh:120,154-155).           */
/* ------------------------------------------------------------------------- */
ORC_API uint16_t orc_f32_to_f16(float f) {
    _Float16 h = (_Float16) f;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
ORC_API float orc_f16_to_f32(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float) h;
}

/* xor-butterfly over 32 lanes (offsets 16,8,4,2,1): src/kernels.cuh:28-32.
 * After the five steps every lane holds the same value; lane 0 is returned. */
static float butterfly32(const float v_in[32]) {
    float v[32], t[32];
    memcpy(v, v_in, sizeof v);
    for (int o = 16; o > 0; o >>= 1) {
        for (int i = 0; i < 32; ++i) t[i] = v[i] + v[i ^ o];
        memcpy(v, t, sizeof v);
    }
    return v[0];
}

/* The block sum as the reference's FUSED SwiGLU epilogue takes it (src/prefill.cu:424-448): a lane holds rows
 * g, g+8, g+16, g+24 of the block and adds (v0 + v1) + (v2 + v3), then xor-shuffles over 4, 8, 16 (g ^ 1, 2, 4):
 * in row terms the pairing order is 8, 16, 1, 2, 4.  Differs from butterfly32 in the last bits only, which the
 * fp16 rounding of the sum field exposes for about one block in a few thousand. */
static float butterfly32_fused_epilogue(const float v_in[32]) {
    static const int order[5] = {8, 16, 1, 2, 4};
    float v[32], t[32];
    memcpy(v, v_in, sizeof v);
    for (int k = 0; k < 5; ++k) {
        for (int i = 0; i < 32; ++i) t[i] = v[i] + v[i ^ order[k]];
        memcpy(v, t, sizeof v);
    }
    return v[0];
}

/* ------------------------------------------------------------------------- */
/* a1. Q8_1 quantiser for one 32-element block.                               */
/* src/quant.cuh:106-121 (quantize_q8_1_warp), src/prefill.cu:90-103.         */
/*   amax exact; sum = butterfly; d = amax/127.0f; q = roundf(x/d) (half away */
/*   from zero), 0 when amax == 0; d and sum stored as fp16 (RN).             */
/* ------------------------------------------------------------------------- */
static void quant_block(const float x[32], int8_t q[32], uint16_t * d16, uint16_t * s16) {
    float am = 0.0f;
    for (int i = 0; i < 32; ++i) { const float a = fabsf(x[i]); if (a > am) am = a; }
    const float sum = butterfly32(x);
    const float d = am / 127.0f;
    for (int i = 0; i < 32; ++i) q[i] = (am == 0.0f) ? (int8_t) 0 : (int8_t) roundf(x[i] / d);
    *d16 = orc_f32_to_f16(d);
    *s16 = orc_f32_to_f16(sum);
}

/* x[nblk*32] -> q[nblk*32], d16[nblk], s16[nblk].  src/kernels.cu:165-171. */
ORC_API void orc_quantize_q8_1(const float * x, int nblk, int8_t * q, uint16_t * d16, uint16_t * s16) {
#pragma omp parallel for if (nblk > 4096)
    for (int b = 0; b < nblk; ++b) quant_block(x + (size_t) b * 32, q + (size_t) b * 32, d16 + b, s16 + b);
}

/* Planar prefill form: sc[b] = (float(fp16 d), 8*float(fp16 sum)).
 * src/prefill.cu:90-103, src/prefill.cuh:27-36. */
static void quant_block_planar(const float x[32], int8_t q[32], float sc[2]) {
    uint16_t d16, s16;
    quant_block(x, q, &d16, &s16);
    sc[0] = orc_f16_to_f32(d16);
    sc[1] = 8.0f * orc_f16_to_f32(s16);
}
/* the same with the sum in the fused epilogue's order */
static void quant_block_planar_fused_epilogue(const float x[32], int8_t q[32], float sc[2]) {
    quant_block_planar(x, q, sc);
    sc[1] = 8.0f * orc_f16_to_f32(orc_f32_to_f16(butterfly32_fused_epilogue(x)));
}

/* 8 * fp16(sum) of each 32-element block of v in the fused epilogue's order: the second field of the planar
 * (d, 8 sum) pair the reference's fused SwiGLU GEMM writes. */
ORC_API void orc_fused_epilogue_sums(const float * v, long long nblocks, float * out) {
    for (long long b = 0; b < nblocks; ++b)
        out[b] = 8.0f * orc_f16_to_f32(orc_f32_to_f16(butterfly32_fused_epilogue(v + b * 32)));
}

/* ------------------------------------------------------------------------- */
/* a4. Integer block dot.  src/quant.cuh:131-158.                             */
/* byte j of the 16-byte qs = element j (low nibble) | element j+16 (high);   */
/* nibbles stay unsigned 0..15.                                               */
/* ------------------------------------------------------------------------- */
static inline int32_t block_sumi(const uint8_t qs[16], const int8_t q[32]) {
    int32_t s = 0;
    for (int j = 0; j < 16; ++j) {
        s += (int32_t) (qs[j] & 15) * (int32_t) q[j];
        s += (int32_t) (qs[j] >> 4) * (int32_t) q[j + 16];
    }
    return s;
}

/* All block sums of a [rows][bpr] Q4_0 matrix against one activation row. */
ORC_API void orc_block_sumi(const uint8_t * qs, const int8_t * aq, int rows, int bpr, int32_t * out) {
#pragma omp parallel for if (rows > 256)
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < bpr; ++b)
            out[(size_t) r * bpr + b] = block_sumi(qs + ((size_t) r * bpr + b) * 16, aq + (size_t) b * 32);
}

/* One block term accumulated:  acc + d4*(d8*sumi - 8*sum)  as the GPU rounds it:
 * inner = fma(d8, (float)sumi, -(8*sum)) [8*sum exact], acc' = fma(d4, inner, acc).
 * src/quant.cuh:154-157 (contracted by nvcc), src/prefill.cu:391-399 (explicit). */
static inline float block_term_acc(float d4, float d8, int32_t sumi, float sum8, float acc) {
    return fmaf(d4, fmaf(d8, (float) sumi, -sum8), acc);
}
/* The batched-prefill GEMM's form of the same term, as the reference ships it (PF_EPI2 = 1,
 * src/prefill.cu:32-39,131-139,341-342,381-384): the tensor-core accumulator is seeded with the bit
 * pattern of 1.5 * 2^23, so the block sum arrives as the float 12582912 + sumi (exact), and the offset
 * is folded into the per-(token, block) constant c = fma(d8, 12582912, 8sum). */
static inline float block_term_acc_pf(float d4, float d8, int32_t sumi, float sum8, float acc) {
    const float c = fmaf(d8, 12582912.0f, sum8);
    const float F = (float) (12582912 + sumi);          /* exact: |sumi| < 2^22 */
    return fmaf(d4, fmaf(d8, F, -c), acc);
}

/* One GEMV row in the reference's order: lane l accumulates blocks l, l+32, ...
 * then the butterfly.  src/kernels.cu:214-223 + warp_sum. */
static float gemv_row(const uint8_t * qs_row, const uint16_t * d_row, int bpr,
                      const int8_t * aq, const uint16_t * ad16, const uint16_t * as16) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int k = l; k < bpr; k += 32) {
            const int32_t s = block_sumi(qs_row + (size_t) k * 16, aq + (size_t) k * 32);
            acc = block_term_acc(orc_f16_to_f32(d_row[k]), orc_f16_to_f32(ad16[k]), s,
                                 8.0f * orc_f16_to_f32(as16[k]), acc);
        }
        lane[l] = acc;
    }
    return butterfly32(lane);
}

/* a5. y[row] = (add ? y[row] : 0) + gemv_row * ninv.
 * src/kernels.cu:190-241 (k_gemv_q4_0_t<false>); ninv = 1 when no ssq is given. */
ORC_API void orc_gemv_q4_0(const uint8_t * qs, const uint16_t * d, const int8_t * aq,
                           const uint16_t * ad16, const uint16_t * as16, int rows, int bpr,
                           float * y, int add_residual, float ninv) {
#pragma omp parallel for if (rows > 64)
    for (int r = 0; r < rows; ++r) {
        const float a = gemv_row(qs + (size_t) r * bpr * 16, d + (size_t) r * bpr, bpr, aq, ad16, as16) * ninv;
        y[r] = add_residual ? (y[r] + a) : a;
    }
}

/* float64 statement of the same sum (order-free) with the magnitude
 * sum|term| used as the tolerance yardstick: tests/test_prefill.cu:61-83. */
ORC_API void orc_gemv_q4_0_f64(const uint8_t * qs, const uint16_t * d, const int8_t * aq,
                               const uint16_t * ad16, const uint16_t * as16, int rows, int bpr,
                               double * y, double * mag) {
#pragma omp parallel for if (rows > 64)
    for (int r = 0; r < rows; ++r) {
        double acc = 0.0, am = 0.0;
        for (int k = 0; k < bpr; ++k) {
            const int32_t s = block_sumi(qs + ((size_t) r * bpr + k) * 16, aq + (size_t) k * 32);
            const double t = (double) orc_f16_to_f32(d[(size_t) r * bpr + k]) *
                             ((double) orc_f16_to_f32(ad16[k]) * (double) s - 8.0 * (double) orc_f16_to_f32(as16[k]));
            acc += t; am += fabs(t);
        }
        y[r] = acc;
        if (mag) mag[r] = am;
    }
}

/* ------------------------------------------------------------------------- */
/* a2. Plain fused RMSNorm -> Q8_1, n == 2048.  src/kernels.cu:68-105.        */
/* 256 "threads": thread t sums x[t+256j]^2, j = 0..7, as an FMA chain; tree  */
/* strides 128, 64, 32; then the 32-lane butterfly.  inv = rsqrt(ss/2048+eps) */
/* t = (x*inv)*w.  Q8_1 block of element t+256j is 8j + (t>>5).               */
/* inv_override > 0 substitutes the GPU's rsqrtf value.                       */
/* ------------------------------------------------------------------------- */
ORC_API float orc_rmsnorm_ss2048(const float * x) {
    float s[256];
    for (int t = 0; t < 256; ++t) {
        float sq = 0.0f;
        for (int j = 0; j < 8; ++j) sq = fmaf(x[t + 256 * j], x[t + 256 * j], sq);
        s[t] = sq;
    }
    for (int o = 128; o > 16; o >>= 1)
        for (int t = 0; t < o; ++t) s[t] = s[t] + s[t + o];
    return butterfly32(s);
}

ORC_API void orc_rmsnorm_q8_1(const float * x, const float * w, float eps, float inv_override,
                              float * y32, int8_t * q, uint16_t * d16, uint16_t * s16, float * inv_out) {
    const float ss = orc_rmsnorm_ss2048(x);
    float inv = 1.0f / sqrtf(fmaf(ss, 1.0f / 2048.0f, eps));
    if (inv_override > 0.0f) inv = inv_override;
    if (inv_out) *inv_out = inv;
    float t[2048];
    for (int i = 0; i < 2048; ++i) { const float a = x[i] * inv; t[i] = a * w[i]; }
    if (y32) memcpy(y32, t, sizeof t);
    if (q) orc_quantize_q8_1(t, 64, q, d16, s16);
}

/* ------------------------------------------------------------------------- */
/* a3. Scale-carrying norm split.  Producer: src/kernels.cuh:421-431          */
/* (quantise the RAW u = x*w, emit ssq[b] = butterfly of x^2 over block b).   */
/* Consumer: src/kernels.cuh:441-447 (s = ssq[l]+ssq[l+32], butterfly,        */
/* inv = rsqrt(s/2048 + eps)).                                                */
/* ------------------------------------------------------------------------- */
ORC_API void orc_norm_prod(const float * x, const float * w, int n, float * h32,
                           int8_t * q, uint16_t * d16, uint16_t * s16, float * ssq) {
    for (int b = 0; b < n / 32; ++b) {
        float u[32], sq[32];
        for (int i = 0; i < 32; ++i) {
            const float xv = x[b * 32 + i];
            u[i] = xv * w[b * 32 + i];
            sq[i] = xv * xv;
        }
        if (h32) memcpy(h32 + b * 32, u, sizeof u);
        quant_block(u, q + b * 32, d16 + b, s16 + b);
        ssq[b] = butterfly32(sq);
    }
}

/* Sum feeding the consumer's rsqrt, in the consumer's order (64 partials). */
ORC_API float orc_norm_ssq_total(const float * ssq) {
    float s[32];
    for (int l = 0; l < 32; ++l) s[l] = ssq[l] + ssq[l + 32];
    return butterfly32(s);
}
ORC_API float orc_norm_inv(const float * ssq, float eps) {
    return 1.0f / sqrtf(fmaf(orc_norm_ssq_total(ssq), 1.0f / 2048.0f, eps));
}

/* ------------------------------------------------------------------------- */
/* a6. Producer GEMV: y = (add ? y : 0) + dot (no ninv), then the a3 producer */
/* over each group of 32 rows.  src/kernels.cu:318-349.                       */
/* ------------------------------------------------------------------------- */
ORC_API void orc_gemv_q4_0_prod(const uint8_t * qs, const uint16_t * d, const int8_t * aq,
                                const uint16_t * ad16, const uint16_t * as16, int rows, int bpr,
                                float * y, int add_residual, const float * nw, float * h32,
                                int8_t * oq, uint16_t * od16, uint16_t * os16, float * ssq) {
    orc_gemv_q4_0(qs, d, aq, ad16, as16, rows, bpr, y, add_residual, 1.0f);
    if (nw) orc_norm_prod(y, nw, rows, h32, oq, od16, os16, ssq);
}

/* ------------------------------------------------------------------------- */
/* a8. Router logits.  src/kernels.cu:583-624: per expert, lane l accumulates */
/* W[e][i]*h[i] for i = l, l+32, ... ascending as an FMA chain; butterfly;    */
/* logit = acc * ninv.                                                        */
/* ------------------------------------------------------------------------- */
ORC_API void orc_router_dot(const float * h, const float * W, int n_exp, int hidden, float ninv,
                            float * logits) {
    for (int e = 0; e < n_exp; ++e) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int i = l; i < hidden; i += 32) acc = fmaf(W[(size_t) e * hidden + i], h[i], acc);
            lane[l] = acc;
        }
        logits[e] = butterfly32(lane) * ninv;
    }
}

/* sigmoid + bias.  src/kernels.cu:615-622, 646-650.  expf is the libm one here
 * (<= 1 ulp); the GPU's expf may differ in the last place. */
ORC_API void orc_router_gate(const float * logits, const float * bias, int n_exp, int softmax_mode,
                             float * sel, float * sig) {
    if (!softmax_mode) {
        for (int e = 0; e < n_exp; ++e) {
            const float g = 1.0f / (1.0f + expf(-logits[e]));
            sig[e] = g;
            sel[e] = g + (bias ? bias[e] : 0.0f);
        }
        return;
    }
    /* Softmax variant of the synthetic configs: rank by softmax probability
     * (monotone in the logit); the top-4 renormalisation is done by the
     * selector exactly as for the sigmoid gate. */
    float mx = logits[0];
    for (int e = 1; e < n_exp; ++e) if (logits[e] > mx) mx = logits[e];
    float den = 0.0f;
    for (int e = 0; e < n_exp; ++e) { sig[e] = expf(logits[e] - mx); den += sig[e]; }
    for (int e = 0; e < n_exp; ++e) { sig[e] = sig[e] / den; sel[e] = sig[e] + (bias ? bias[e] : 0.0f); }
}

/* a9. Top-4 of 64.  src/kernels.cuh:515-541: four rounds of arg-max with
 * "greater value wins, equal value -> lower index wins"; the winner is set to
 * -1e30; w_k = sig[idx_k]; wsum accumulated k = 0..3, clamped at 2^-14; divide. */
ORC_API void orc_router_select(const float * sel_in, const float * sig, int n_exp, int * idx, float * w) {
    float sel[256];
    for (int e = 0; e < n_exp; ++e) sel[e] = sel_in[e];
    for (int r = 0; r < 4; ++r) {
        int mi = 0; float mv = sel[0];
        for (int e = 1; e < n_exp; ++e) if (sel[e] > mv) { mv = sel[e]; mi = e; }
        idx[r] = mi;
        sel[mi] = -1e30f;
    }
    float ws = 0.0f;
    for (int k = 0; k < 4; ++k) { w[k] = sig[idx[k]]; ws += w[k]; }
    if (ws < 6.103515625e-5f) ws = 6.103515625e-5f;
    for (int k = 0; k < 4; ++k) w[k] = w[k] / ws;
}

/* Smallest gap between the 4th and 5th ranking value: lets a test attribute an
 * id mismatch to a near-tie rather than to a bug. */
ORC_API float orc_router_margin(const float * sel_in, int n_exp) {
    float sel[256];
    for (int e = 0; e < n_exp; ++e) sel[e] = sel_in[e];
    float v[5];
    for (int r = 0; r < 5; ++r) {
        int mi = 0; float mv = sel[0];
        for (int e = 1; e < n_exp; ++e) if (sel[e] > mv) { mv = sel[e]; mi = e; }
        v[r] = mv; sel[mi] = -1e30f;
    }
    return v[3] - v[4];
}

/* ------------------------------------------------------------------------- */
/* a11. SwiGLU.  src/kernels.cu:513-516, src/kernels.cuh:33:                  */
/* silu(g) = g / (1 + exp(-g)), v = silu(g)*u.  (The GPU uses the fast        */
/* __expf, so v is a tolerance item; its quantisation is checked on the GPU's */
/* own v.)                                                                    */
/* ------------------------------------------------------------------------- */
ORC_API void orc_swiglu(const float * gate, const float * up, int n, float * out) {
    for (int i = 0; i < n; ++i) {
        const float g = gate[i];
        const float s = g / (1.0f + expf(-g));
        out[i] = s * up[i];
    }
}

/* ------------------------------------------------------------------------- */
/* a10. Gate and up GEMVs of the four chosen experts.  src/kernels.cu:1049-   */
/* 1124: expert base = idx[k]*rows_per_expert*bpr blocks; y[k*rows + r].      */
/* ------------------------------------------------------------------------- */
ORC_API void orc_gemv_q4_0_exp(const uint8_t * qs, const uint16_t * d, const int8_t * aq,
                               const uint16_t * ad16, const uint16_t * as16, int out_rows, int bpr,
                               int rows_per_expert, int xq_stride, const int * idx, float ninv, float * y) {
    for (int k = 0; k < 4; ++k) {
        const size_t base = (size_t) idx[k] * rows_per_expert * bpr;
        orc_gemv_q4_0(qs + base * 16, d + base, aq + (size_t) k * xq_stride * 32,
                      ad16 + (size_t) k * xq_stride, as16 + (size_t) k * xq_stride,
                      out_rows, bpr, y + (size_t) k * out_rows, 0, ninv);
    }
}

/* ------------------------------------------------------------------------- */
/* a12. Down projection of the four experts + weighted sum + residual.        */
/* src/kernels.cu:1194-1236: a = 0; for k: a = fma(w[k], row_dot_k, a);       */
/* x[row] = x[row] + a; optional a3 producer over the new x.                  */
/* ------------------------------------------------------------------------- */
ORC_API void orc_moe_down_accum(const uint8_t * qs, const uint16_t * d, const int8_t * aq,
                                const uint16_t * ad16, const uint16_t * as16, int out_rows, int bpr,
                                int rows_per_expert, int xq_stride, const int * idx, const float * wk,
                                float * x, const float * nw, float * h32,
                                int8_t * oq, uint16_t * od16, uint16_t * os16, float * ssq) {
#pragma omp parallel for if (out_rows > 64)
    for (int r = 0; r < out_rows; ++r) {
        float a = 0.0f;
        for (int k = 0; k < 4; ++k) {
            const size_t base = ((size_t) idx[k] * rows_per_expert + r) * bpr;
            const float dot = gemv_row(qs + base * 16, d + base, bpr, aq + (size_t) k * xq_stride * 32,
                                       ad16 + (size_t) k * xq_stride, as16 + (size_t) k * xq_stride);
            a = fmaf(wk[k], dot, a);
        }
        x[r] = x[r] + a;
    }
    if (nw) orc_norm_prod(x, nw, out_rows, h32, oq, od16, os16, ssq);
}

/* ========================================================================= */
/* Batched prefill                                                           */
/* ========================================================================= */

/* a17. rows fp32 -> planar Q8_1.  src/prefill.cu:1574-1581. */
ORC_API void orc_pf_quant_rows(const float * X, int rows, int ld, int kb, int8_t * qs, float * sc) {
#pragma omp parallel for if (rows > 16)
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < kb; ++b)
            quant_block_planar(X + (size_t) r * ld + b * 32, qs + ((size_t) r * kb + b) * 32,
                               sc + ((size_t) r * kb + b) * 2);
}

/* a17. unfused SwiGLU over rows [gate | up] -> planar Q8_1.  src/prefill.cu:1584-1594.
 * vbuf (optional, rows*kb*32) receives / provides the fp32 v: when use_v != 0 the
 * given v is quantised instead of being recomputed (GPU __expf override). */
ORC_API void orc_pf_swiglu(const float * Y, int rows, int ld, int up_off, int kb, int8_t * qs, float * sc,
                           float * vbuf, int use_v) {
#pragma omp parallel for if (rows > 16)
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < kb; ++b) {
            float v[32];
            for (int i = 0; i < 32; ++i) {
                const size_t o = (size_t) r * kb * 32 + b * 32 + i;
                if (use_v) v[i] = vbuf[o];
                else {
                    const float g = Y[(size_t) r * ld + b * 32 + i];
                    v[i] = (g / (1.0f + expf(-g))) * Y[(size_t) r * ld + up_off + b * 32 + i];
                    if (vbuf) vbuf[o] = v[i];
                }
            }
            quant_block_planar(v, qs + ((size_t) r * kb + b) * 32, sc + ((size_t) r * kb + b) * 2);
        }
}

/* a2/a3 per token.  src/prefill.cu:871-932.  plain = 1: (x*inv)*w quantised,
 * inv_out = 1.  plain = 0: u = x*w quantised, inv_out = rsqrt(ssq/2048 + eps),
 * optional h32 = u.  inv_override (per token, may be null) replaces rsqrt. */
ORC_API void orc_pf_norm(const float * X, const float * w, int m, int plain, const float * inv_override,
                         int8_t * qs, float * sc, float * inv_out, float * h32) {
#pragma omp parallel for if (m > 8)
    for (int t = 0; t < m; ++t) {
        const float * x = X + (size_t) t * 2048;
        float v[2048];
        if (plain) {
            const float ss = orc_rmsnorm_ss2048(x);
            float inv = 1.0f / sqrtf(fmaf(ss, 1.0f / 2048.0f, 1e-5f));
            if (inv_override) inv = inv_override[t];
            for (int i = 0; i < 2048; ++i) { const float a = x[i] * inv; v[i] = a * w[i]; }
            inv_out[t] = 1.0f;
        } else {
            float ssq[64];
            for (int b = 0; b < 64; ++b) {
                float sq[32];
                for (int i = 0; i < 32; ++i) { const float xv = x[b * 32 + i]; v[b * 32 + i] = xv * w[b * 32 + i]; sq[i] = xv * xv; }
                ssq[b] = butterfly32(sq);
            }
            if (h32) memcpy(h32 + (size_t) t * 2048, v, sizeof v);
            inv_out[t] = inv_override ? inv_override[t] : orc_norm_inv(ssq, 1e-5f);
        }
        for (int b = 0; b < 64; ++b)
            quant_block_planar(v + b * 32, qs + ((size_t) t * 64 + b) * 32, sc + ((size_t) t * 64 + b) * 2);
    }
}

/* a14. Batched router logits * inv[t].
 * order = 0: the decode order (src/prefill.cu:1668-1693, bit-identical to a8).
 * order = 1: k ascending FMA chain per (token, expert) (src/prefill.cu:1636-1647). */
ORC_API void orc_pf_router_logits(const float * H, int m, const float * W, const float * inv, int order,
                                  float * logits) {
#pragma omp parallel for if (m > 4)
    for (int t = 0; t < m; ++t) {
        const float * h = H + (size_t) t * 2048;
        if (order == 0) {
            orc_router_dot(h, W, 64, 2048, inv[t], logits + (size_t) t * 64);
        } else {
            for (int e = 0; e < 64; ++e) {
                float acc = 0.0f;
                for (int k = 0; k < 2048; ++k) acc = fmaf(h[k], W[(size_t) e * 2048 + k], acc);
                logits[(size_t) t * 64 + e] = acc * inv[t];
            }
        }
    }
}

/* a9 per token.  src/prefill.cu:1696-1708. */
ORC_API void orc_pf_select(const float * sel, const float * sig, int m, int * idx, float * w) {
    for (int t = 0; t < m; ++t) orc_router_select(sel + (size_t) t * 64, sig + (size_t) t * 64, 64, idx + t * 4, w + t * 4);
}

/* a15. count / plan / scatter.  src/prefill.cu:1710-1756.
 * tiles[i] = {expert, start in perm, count <= 64, 0}; experts with no slot
 * emit no tile; perm is expert-major, slot-ascending within an expert. */
ORC_API void orc_moe_count(const int * idx, int n, int n_exp, int * cnt) {
    for (int e = 0; e < n_exp; ++e) cnt[e] = 0;
    for (int s = 0; s < n; ++s) cnt[idx[s]]++;
}
ORC_API void orc_moe_plan(const int * cnt, int n_exp, int * off, int * tiles, int * ntiles) {
    int o = 0, nt = 0;
    for (int e = 0; e < n_exp; ++e) {
        const int c = cnt[e];
        off[e] = o;
        for (int s = 0; s < c; s += 64) {
            tiles[nt * 4 + 0] = e; tiles[nt * 4 + 1] = o + s;
            tiles[nt * 4 + 2] = (c - s < 64) ? (c - s) : 64; tiles[nt * 4 + 3] = 0;
            ++nt;
        }
        o += c;
    }
    *ntiles = nt;
}
ORC_API void orc_moe_scatter(const int * idx, int n, int n_exp, const int * off, int * perm) {
    int * cur = (int *) malloc(sizeof(int) * (size_t) n_exp);
    for (int e = 0; e < n_exp; ++e) cur[e] = off[e];
    for (int s = 0; s < n; ++s) perm[cur[idx[s]]++] = s;
    free(cur);
}

/* a13. The grouped / dense Q4_0 x Q8_1 GEMM.  src/prefill.cuh:45-66,
 * src/prefill.cu:186-233, 391-399, 474-490.
 *   out[orow][n] = (add ? out : 0) + scale[arow] * sum_{b ascending} fma(d4, fma(d8, 12582912 + S_b, -c), .)
 *   with c = fma(d8, 12582912, 8sum), the reference's shipped form (block_term_acc_pf above)
 * Weight row n of the stacked tensor lives in segment seg (rows [seg_end[seg-1],
 * seg_end[seg])) at qs[seg] + expert*exp_stride + (n - seg_start)*bpr.
 * Tokens: dense rows [0, ntok) or, with perm != NULL, every slot perm[i]
 * (expert = idx_of_slot from the tile that covers i), arow = slot >> a_shift.
 * out64/mag/slack (optional) receive the float64 value before scale/add, sum|terms| and the folded
 * form's allowed rounding.
 */
typedef struct {
    const uint8_t *  qs[3];
    const uint16_t * d[3];
    int              seg_end[3];
    int              N, bpr;
    long long        exp_stride;     /* blocks */
    const int8_t *   aqs;
    const float *    asc;            /* [rows][bpr][2] */
    int              ntok;
    const int *      perm;
    const int *      tiles;          /* [ntiles][4] */
    int              ntiles;
    int              a_shift;
    const float *    scale;
    float *          out;
    int              out_ld;
    int              add;
} orc_gemm_t;

static void gemm_locate(const orc_gemm_t * g, int n, int expert, const uint8_t ** q, const uint16_t ** d) {
    const int seg = (n < g->seg_end[0]) ? 0 : (n < g->seg_end[1]) ? 1 : 2;
    const int sbase = seg ? g->seg_end[seg - 1] : 0;
    const size_t blk = (size_t) expert * (size_t) g->exp_stride + (size_t) (n - sbase) * g->bpr;
    *q = g->qs[seg] + blk * 16;
    *d = g->d[seg] + blk;
}

static int g_gemm_fold = 1;      /* 1: the reference's shipped (folded) term; 0: the exact term */
ORC_API void orc_set_gemm_fold(int fold) { g_gemm_fold = fold ? 1 : 0; }

static float gemm_dot32(const orc_gemm_t * g, const uint8_t * q, const uint16_t * d, int arow) {
    const int8_t * aq = g->aqs + (size_t) arow * g->bpr * 32;
    const float * as = g->asc + (size_t) arow * g->bpr * 2;
    float acc = 0.0f;
    for (int b = 0; b < g->bpr; ++b)
        acc = g_gemm_fold ? block_term_acc_pf(orc_f16_to_f32(d[b]), as[2 * b], block_sumi(q + (size_t) b * 16, aq + b * 32), as[2 * b + 1], acc)
                          : block_term_acc(orc_f16_to_f32(d[b]), as[2 * b], block_sumi(q + (size_t) b * 16, aq + b * 32), as[2 * b + 1], acc);
    return acc;
}

ORC_API void orc_pf_gemm(const orc_gemm_t * g, double * out64, double * mag, double * slack) {
    const int nrows = g->perm ? 0 : g->ntok;
    /* flatten (slot, expert) pairs */
    int total = nrows;
    if (g->perm) { total = 0; for (int t = 0; t < g->ntiles; ++t) total += g->tiles[t * 4 + 2]; }
    int * slot = (int *) malloc(sizeof(int) * (size_t) (total > 0 ? total : 1));
    int * expt = (int *) malloc(sizeof(int) * (size_t) (total > 0 ? total : 1));
    if (g->perm) {
        int c = 0;
        for (int t = 0; t < g->ntiles; ++t)
            for (int i = 0; i < g->tiles[t * 4 + 2]; ++i) { slot[c] = g->perm[g->tiles[t * 4 + 1] + i]; expt[c] = g->tiles[t * 4]; ++c; }
    } else {
        for (int i = 0; i < total; ++i) { slot[i] = i; expt[i] = 0; }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int i = 0; i < total; ++i) {
        const int orow = slot[i];
        const int arow = orow >> g->a_shift;
        const float scl = g->scale ? g->scale[arow] : 1.0f;
        for (int n = 0; n < g->N; ++n) {
            const uint8_t * q; const uint16_t * d;
            gemm_locate(g, n, expt[i], &q, &d);
            /* the residual add is ONE fused multiply-add: nvcc contracts the reference's `*p + acc * scale`
             * (src/prefill.cu:484-486), confirmed by byte comparison with the reference's kernel on a B200 */
            const float acc = gemm_dot32(g, q, d, arow);
            float * p = g->out + (size_t) orow * g->out_ld + n;
            *p = g->add ? fmaf(acc, scl, *p) : acc * scl;
            if (out64) {
                const int8_t * aq = g->aqs + (size_t) arow * g->bpr * 32;
                const float * as = g->asc + (size_t) arow * g->bpr * 2;
                double acc = 0.0, am = 0.0, sl = 0.0;
                for (int b = 0; b < g->bpr; ++b) {
                    const double d4 = (double) orc_f16_to_f32(d[b]);
                    const double t = d4 * ((double) as[2 * b] * (double) block_sumi(q + (size_t) b * 16, aq + b * 32) - (double) as[2 * b + 1]);
                    acc += t; am += fabs(t);
                    /* the rounding the folded form is allowed: |d4| * half an ulp of c (tests/test_prefill.cu:78-79) */
                    const float c = fabsf(fmaf(as[2 * b], 12582912.0f, as[2 * b + 1]));
                    sl += fabs(d4) * 0.5 * (double) (nextafterf(c, INFINITY) - c);
                }
                out64[(size_t) orow * g->out_ld + n] = acc;
                if (mag) mag[(size_t) orow * g->out_ld + n] = am;
                if (slack) slack[(size_t) orow * g->out_ld + n] = sl;
            }
        }
    }
    free(slot); free(expt);
}

/* a13 with the fused SwiGLU epilogue.  src/prefill.cu:424-469: g.qs[0] = gate,
 * g.qs[1] = up, N = intermediate width; gate and up values are multiplied by
 * scale[arow], v = silu(g)*u, then Q8_1 over 32 consecutive intermediate rows
 * of one slot -> oqs[orow][okb*32], osc[orow][okb][2].  The block sum follows the
 * arithmetic mode (orc_set_gemm_fold): the fused epilogue's own order, or the butterfly.
 * vbuf (optional) [nslots][N]: receives v, or when use_v != 0 supplies it. */
ORC_API void orc_pf_gemm_swiglu(const orc_gemm_t * g, int8_t * oqs, float * osc, int okb,
                                float * vbuf, int use_v) {
    int total = g->ntok;
    if (g->perm) { total = 0; for (int t = 0; t < g->ntiles; ++t) total += g->tiles[t * 4 + 2]; }
    int * slot = (int *) malloc(sizeof(int) * (size_t) (total > 0 ? total : 1));
    int * expt = (int *) malloc(sizeof(int) * (size_t) (total > 0 ? total : 1));
    if (g->perm) {
        int c = 0;
        for (int t = 0; t < g->ntiles; ++t)
            for (int i = 0; i < g->tiles[t * 4 + 2]; ++i) { slot[c] = g->perm[g->tiles[t * 4 + 1] + i]; expt[c] = g->tiles[t * 4]; ++c; }
    } else {
        for (int i = 0; i < total; ++i) { slot[i] = i; expt[i] = 0; }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int i = 0; i < total; ++i) {
        const int orow = slot[i];
        const int arow = orow >> g->a_shift;
        const float scl = g->scale ? g->scale[arow] : 1.0f;
        const size_t eo = (size_t) expt[i] * (size_t) g->exp_stride;
        for (int b0 = 0; b0 < g->N / 32; ++b0) {
            float v[32];
            for (int r = 0; r < 32; ++r) {
                const int n = b0 * 32 + r;
                if (use_v) { v[r] = vbuf[(size_t) orow * g->N + n]; continue; }
                const size_t blk = eo + (size_t) n * g->bpr;
                const float gt = gemm_dot32(g, g->qs[0] + blk * 16, g->d[0] + blk, arow) * scl;
                const float up = gemm_dot32(g, g->qs[1] + blk * 16, g->d[1] + blk, arow) * scl;
                v[r] = (gt / (1.0f + expf(-gt))) * up;
                if (vbuf) vbuf[(size_t) orow * g->N + n] = v[r];
            }
            /* shipped arithmetic: the fused epilogue's own sum order; exact mode: the quantiser's butterfly (fused == unfused) */
            if (g_gemm_fold) quant_block_planar_fused_epilogue(v, oqs + (size_t) orow * okb * 32 + b0 * 32, osc + ((size_t) orow * okb + b0) * 2);
            else quant_block_planar(v, oqs + (size_t) orow * okb * 32 + b0 * 32, osc + ((size_t) orow * okb + b0) * 2);
        }
    }
    free(slot); free(expt);
}

/* a16. x[t][n] += sum_{k=0..3} w[t*4+k] * D[t*4+k][n], FMA chain from 0.
 * src/prefill.cu:1804-1814. */
ORC_API void orc_pf_combine(float * X, const float * D, const float * w, int m, int hidden) {
#pragma omp parallel for if (m > 8)
    for (int t = 0; t < m; ++t)
        for (int n = 0; n < hidden; ++n) {
            float a = 0.0f;
            for (int k = 0; k < 4; ++k) a = fmaf(w[t * 4 + k], D[((size_t) t * 4 + k) * hidden + n], a);
            X[(size_t) t * hidden + n] = X[(size_t) t * hidden + n] + a;
        }
}

/* a16 + the next layer's a3 producer.  src/prefill.cu:1764-1800. */
ORC_API void orc_pf_combine_norm(float * X, const float * D, const float * w, const float * nw, int m,
                                 const float * inv_override, int8_t * qs, float * sc, float * inv_out) {
    orc_pf_combine(X, D, w, m, 2048);
    orc_pf_norm(X, nw, m, 0, inv_override, qs, sc, inv_out, NULL);
}

/* a17. planar row -> 36-byte blocks {fp16 d, fp16 sum, int8 q[32]}.
 * src/prefill.cu:1819-1828 (exact: both scale fields are fp16 values). */
ORC_API void orc_pf_pack_q8_1(const int8_t * qs, const float * sc, int t, int kb, uint8_t * blocks) {
    for (int b = 0; b < kb; ++b) {
        const uint16_t d = orc_f32_to_f16(sc[((size_t) t * kb + b) * 2]);
        const uint16_t s = orc_f32_to_f16(sc[((size_t) t * kb + b) * 2 + 1] * 0.125f);
        memcpy(blocks + (size_t) b * 36, &d, 2);
        memcpy(blocks + (size_t) b * 36 + 2, &s, 2);
        memcpy(blocks + (size_t) b * 36 + 4, qs + ((size_t) t * kb + b) * 32, 32);
    }
}

/* ------------------------------------------------------------------------- */
/* Throughput helper for the CPU-baseline leg of the benchmark: the integer   */
/* contraction of a block of GEMM work, all host threads.  Returns the number */
/* of (row, token) dot products evaluated.                                    */
/* ------------------------------------------------------------------------- */
/* Pin the OpenMP team size (the benchmark sets it from the process's CPU affinity, so that a launcher's
 * OMP_NUM_THREADS=1 does not decide the baseline). */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void) n;
#endif
}

ORC_API int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}

/* ========================================================================= */
/* Q6_K lm_head (the row the path feeds next): src/quant.cuh:171-250,          */
/* src/kernels.cu:426-478 (k_gemv_q6_K_dp4a), 855-868 (k_embed_q6_K).          */
/* Planar super-block of 256 weights: ql[128], qh[64], int8 scales[16], fp16 d. */
/* ========================================================================= */

/* 6-bit value of element idx: src/quant.cuh:171-195 (== tools/gguf.py:179-204). */
static inline int q6_at(const uint8_t * QL, const uint8_t * QH, int idx) {
    const int n = (idx >= 128) ? 128 : 0, r = idx - n;
    const int ql = QL[(n >> 1) + (r & 63)], qh = QH[(n >> 2) + (r & 31)];
    const int lo = (r >= 64) ? (ql >> 4) : (ql & 15);
    return lo | (((qh >> (2 * (r >> 5))) & 3) << 4);
}
ORC_API int orc_q6_at(const uint8_t * QL, const uint8_t * QH, int idx) { return q6_at(QL, QH, idx); }

/* Integer group sums a[row][sb][lane] = sum_{t<8} (q6(8*lane+t) - 32) * xq[sb*256 + 8*lane + t] (exact). */
ORC_API void orc_q6_group_sums(const uint8_t * ql, const uint8_t * qh, const int8_t * aq, int rows, int sbpr, int32_t * out) {
#pragma omp parallel for if (rows > 64)
    for (int r = 0; r < rows; ++r)
        for (int sb = 0; sb < sbpr; ++sb) {
            const size_t blk = (size_t) r * sbpr + sb;
            for (int L = 0; L < 32; ++L) {
                int32_t a = 0;
                for (int t = 0; t < 8; ++t) a += (q6_at(ql + blk * 128, qh + blk * 64, 8 * L + t) - 32) * (int32_t) aq[sb * 256 + 8 * L + t];
                out[(blk * 32) + L] = a;
            }
        }
}

/* lm_head GEMV in the shipped (dp4a) order: lane L owns elements 8L..8L+7 of every super-block;
 * acc = fma(d, d8 * float(a * scale), acc) over super-blocks ascending; butterfly; * ninv.
 * src/kernels.cu:426-478. */
ORC_API void orc_gemv_q6_K(const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const uint16_t * d,
                           const int8_t * aq, const uint16_t * ad16, int rows, int sbpr, float ninv, float * y) {
#pragma omp parallel for if (rows > 64)
    for (int r = 0; r < rows; ++r) {
        float lane[32];
        for (int L = 0; L < 32; ++L) {
            float acc = 0.0f;
            for (int sb = 0; sb < sbpr; ++sb) {
                const size_t blk = (size_t) r * sbpr + sb;
                int32_t a = 0;
                for (int t = 0; t < 8; ++t) a += (q6_at(ql + blk * 128, qh + blk * 64, 8 * L + t) - 32) * (int32_t) aq[sb * 256 + 8 * L + t];
                const float d8 = orc_f16_to_f32(ad16[sb * 8 + (L >> 2)]);
                const float t2 = d8 * (float) (a * (int32_t) sc[blk * 16 + (L >> 1)]);
                acc = fmaf(orc_f16_to_f32(d[blk]), t2, acc);
            }
            lane[L] = acc;
        }
        y[r] = butterfly32(lane) * ninv;
    }
}

/* float64 statement + sum|terms| per row (terms at 16-element scale-group granularity). */
ORC_API void orc_gemv_q6_K_f64(const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const uint16_t * d,
                               const int8_t * aq, const float * ad32, int rows, int sbpr, double * y, double * mag) {
#pragma omp parallel for if (rows > 64)
    for (int r = 0; r < rows; ++r) {
        double acc = 0.0, am = 0.0;
        for (int sb = 0; sb < sbpr; ++sb) {
            const size_t blk = (size_t) r * sbpr + sb;
            for (int g = 0; g < 16; ++g) {
                long a = 0;
                for (int t = 0; t < 16; ++t) a += (long) (q6_at(ql + blk * 128, qh + blk * 64, 16 * g + t) - 32) * aq[sb * 256 + 16 * g + t];
                const double term = (double) orc_f16_to_f32(d[blk]) * (double) ad32[sb * 8 + (g >> 1)] * (double) sc[blk * 16 + g] * (double) a;
                acc += term; am += fabs(term);
            }
        }
        y[r] = acc;
        if (mag) mag[r] = am;
    }
}

/* One embedding row: x[i] = (d * float(scale)) * float(q6 - 32).  src/kernels.cu:855-868. */
ORC_API void orc_embed_q6_K(const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const uint16_t * d,
                            int token, int sbpr, float * x) {
    for (int i = 0; i < sbpr * 256; ++i) {
        const size_t blk = (size_t) token * sbpr + i / 256;
        const int e = i % 256;
        const float t = orc_f16_to_f32(d[blk]) * (float) sc[blk * 16 + e / 16];
        x[i] = t * (float) (q6_at(ql + blk * 128, qh + blk * 64, e) - 32);
    }
}

/* ---- sequence mixers of a decode step ------------------------------------------------------------------- */

/* Short gated convolution, one step (src/kernels.cu:521-545): bx = B*X, conv = fma(bx, w2, fma(h1, w1, h0*w0)),
 * y = C*conv, history shifts.  The association of the three-term sum is fixed here; the reference leaves it to
 * the compiler's contraction and gates at 1e-5 against float64 (tests/test_kernels.cu:131-163). */
ORC_API void orc_shortconv(const float * bcx, const float * conv_w, float * hist, float * y, int n) {
    for (int ch = 0; ch < n; ++ch) {
        const float bx = bcx[ch] * bcx[2 * n + ch];
        const float h0 = hist[2 * ch], h1 = hist[2 * ch + 1];
        const float conv = fmaf(bx, conv_w[3 * ch + 2], fmaf(h1, conv_w[3 * ch + 1], h0 * conv_w[3 * ch]));
        hist[2 * ch] = h1;
        hist[2 * ch + 1] = bx;
        y[ch] = bcx[n + ch] * conv;
    }
}

/* Per-head RMSNorm + NEOX RoPE, float32 in the kernel's order (src/kernels.cu:871-915): sum of squares by the
 * halving tree over 64 (s[i] += s[i+o], o = 32..1), inv = 1/sqrt(ss/64 + eps), x = (v*inv)*w, angle =
 * pos * powf(theta, -2i/64), out[i] = x0*c - x1*s, out[i+32] = x0*s + x1*c.  inv_override (may be NULL) takes
 * the device's rsqrtf values, one per head, so that everything downstream can be compared exactly. */
ORC_API void orc_norm_rope_heads(float * x, const float * w, int n_heads, float pos, float theta,
                                 const float * inv_override, float * inv_out) {
    for (int h = 0; h < n_heads; ++h) {
        float * v = x + (size_t) h * 64;
        float s[64];
        for (int i = 0; i < 64; ++i) s[i] = v[i] * v[i];
        for (int o = 32; o > 0; o >>= 1)
            for (int i = 0; i < o; ++i) s[i] = s[i] + s[i + o];
        float inv = 1.0f / sqrtf(s[0] / 64.0f + 1e-5f);
        if (inv_out) inv_out[h] = inv;
        if (inv_override) inv = inv_override[h];
        for (int i = 0; i < 32; ++i) {
            const float x0 = (v[i] * inv) * w[i], x1 = (v[i + 32] * inv) * w[i + 32];
            const float invf = powf(theta, (-2.0f * (float) i) / 64.0f);
            const float ang = pos * invf;
            const float sn = sinf(ang), cs = cosf(ang);
            v[i] = x0 * cs - x1 * sn;
            v[i + 32] = x0 * sn + x1 * cs;
        }
    }
}

/* fp32 -> fp16 bits, round to nearest even (the device's __float2half). */
ORC_API void orc_f32_to_f16_array(const float * x, int n, uint16_t * out) {
    for (int i = 0; i < n; ++i) {
        const _Float16 hv = (_Float16) x[i];
        memcpy(&out[i], &hv, 2);
    }
}

/* Decode attention in float64: the definition both the reference's kernels and ours are roundings of
 * (tests/test_attn.cu:46-75).  q[32*64] fp32, kc / vc fp16 bits [seq][8][64], out[32*64]. */
ORC_API void orc_attn_decode_f64(const float * q, const uint16_t * kc, const uint16_t * vc, int seq, double * out) {
#pragma omp parallel for schedule(static)
    for (int head = 0; head < 32; ++head) {
        const int kv = head / 4;
        double * s = (double *) malloc((size_t) seq * sizeof(double));
        double m = -1e300;
        for (int t = 0; t < seq; ++t) {
            const uint16_t * k = kc + ((size_t) t * 8 + kv) * 64;
            double a = 0.0;
            for (int d = 0; d < 64; ++d) a += (double) q[head * 64 + d] * (double) orc_f16_to_f32(k[d]);
            a *= 0.125;
            s[t] = a;
            if (a > m) m = a;
        }
        double l = 0.0;
        for (int t = 0; t < seq; ++t) { s[t] = exp(s[t] - m); l += s[t]; }
        double acc[64];
        for (int d = 0; d < 64; ++d) acc[d] = 0.0;
        for (int t = 0; t < seq; ++t) {
            const uint16_t * v = vc + ((size_t) t * 8 + kv) * 64;
            for (int d = 0; d < 64; ++d) acc[d] += s[t] * (double) orc_f16_to_f32(v[d]);
        }
        for (int d = 0; d < 64; ++d) out[head * 64 + d] = acc[d] / l;
        free(s);
    }
}

/* Causal GQA attention of a chunk in float64 over the fp16 inputs (tests/test_prefill.cu:259-286): query t
 * (fp16 bits, [m][2048], already carrying the 1/8 scale) at position P + t sees keys 0 .. P + t. */
ORC_API void orc_pf_attn_f64(const uint16_t * qh, int m, int P, const uint16_t * kc, const uint16_t * vc, double * out) {
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int t = 0; t < m; ++t)
        for (int h = 0; h < 32; ++h) {
            const int kv = h / 4, qp = P + t;
            double * sc = (double *) malloc((size_t) (qp + 1) * sizeof(double));
            double q[64];
            for (int d = 0; d < 64; ++d) q[d] = (double) orc_f16_to_f32(qh[(size_t) t * 2048 + h * 64 + d]);
            double mx = -1e300;
            for (int j = 0; j <= qp; ++j) {
                const uint16_t * k = kc + ((size_t) j * 8 + kv) * 64;
                double s = 0.0;
                for (int d = 0; d < 64; ++d) s += q[d] * (double) orc_f16_to_f32(k[d]);
                sc[j] = s;
                if (s > mx) mx = s;
            }
            double l = 0.0, acc[64];
            for (int d = 0; d < 64; ++d) acc[d] = 0.0;
            for (int j = 0; j <= qp; ++j) {
                const double p = exp(sc[j] - mx);
                l += p;
                const uint16_t * v = vc + ((size_t) j * 8 + kv) * 64;
                for (int d = 0; d < 64; ++d) acc[d] += p * (double) orc_f16_to_f32(v[d]);
            }
            for (int d = 0; d < 64; ++d) out[(size_t) t * 2048 + h * 64 + d] = acc[d] / l;
            free(sc);
        }
}
