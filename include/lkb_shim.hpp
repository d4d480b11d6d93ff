// lkb_shim.hpp - the reference engine's kernel names as host-callable C++ wrappers over the C ABI.
//
// The reference launches its kernels with <<<grid, block, smem, stream>>> from src/engine.cu.  A caller
// written in that style switches to this library by replacing each launch
//     k_name<<<grid, block, smem, st>>>(args...);        with        lk::k_name(st, args...);
// (grid and block are chosen inside the library).  The wrappers keep the reference's argument order and
// types (ref: src/kernels.cuh:60-78,449-486,543-558,692-745; src/prefill.cuh:69-127) and its error policy
// (print and exit, ref: src/engine.cu:21-22, src/prefill.cu:7-8) unless LKB_SHIM_NO_EXIT is defined, in
// which case they return the status.
#pragma once
#include <cstdio>
#include <cstdlib>
#include "lkb.h"

namespace lk {

using block_q8_1 = lkb_block_q8_1;                       // ref: src/quant.cuh:27-31
struct QT4 { const void * qs; const void * d; };         // ref: src/kernels.cuh:6 (planar Q4_0 view)
using LKNormProd = lkb_norm_prod_t;                      // ref: src/kernels.cuh:413-418
using PfAct = lkb_pf_act;                                // ref: src/prefill.cuh:33-36
using PfGemm = lkb_pf_gemm;                              // ref: src/prefill.cuh:45-66
using stream_t = lkb_stream_t;                           // cudaStream_t

inline int check(int status, const char * what) {
#ifndef LKB_SHIM_NO_EXIT
    if (status != LKB_OK) { std::fprintf(stderr, "%s failed: %d (%s)\n", what, status, lkb_error_string(status)); std::exit(1); }
#endif
    (void) what;
    return status;
}

// ---- decode ------------------------------------------------------------------
inline int k_quantize_q8_1(stream_t st, const float * x, block_q8_1 * y, int nblocks) {
    return check(lkb_quantize_q8_1(x, y, nblocks, st), "k_quantize_q8_1"); }
inline int k_rmsnorm_q8_1(stream_t st, const float * x, const float * w, int n, float eps, float * y32, void * y16, block_q8_1 * yq8) {
    return check(lkb_rmsnorm_q8_1(x, w, n, eps, y32, y16, yq8, st), "k_rmsnorm_q8_1"); }
inline int k_gemv_q4_0(stream_t st, const void * qs, const void * d, const block_q8_1 * xq, int out_rows, int bpr,
                       float * y, int add_residual, const float * ssq, float eps) {
    return check(lkb_gemv_q4_0(qs, d, xq, out_rows, bpr, y, add_residual, ssq, eps, st), "k_gemv_q4_0"); }
inline int k_gemv_q4_0_prod(stream_t st, const void * qs, const void * d, const block_q8_1 * xq, int out_rows, int bpr,
                            float * y, int add_residual, LKNormProd np) {
    return check(lkb_gemv_q4_0_prod(qs, d, xq, out_rows, bpr, y, add_residual, &np, st), "k_gemv_q4_0_prod"); }
inline int k_gemv_q4_0_3(stream_t st, const void * qs0, const void * d0, int rows0, float * y0,
                         const void * qs1, const void * d1, int rows1, float * y1,
                         const void * qs2, const void * d2, int rows2, float * y2,
                         const block_q8_1 * xq, int bpr, const float * ssq, float eps) {
    return check(lkb_gemv_q4_0_3(qs0, d0, rows0, y0, qs1, d1, rows1, y1, qs2, d2, rows2, y2, xq, bpr, ssq, eps, st), "k_gemv_q4_0_3"); }
inline int k_gemv_q4_0_exp2(stream_t st, const void * qs_a, const void * d_a, const void * qs_b, const void * d_b,
                            const block_q8_1 * xq, int out_rows, int bpr, int rows_per_expert, int xq_stride,
                            const int * d_idx, const float * sel, const float * sig, int * idx_out, float * w_out,
                            float * y_a, float * y_b, const float * ssq, float eps) {
    return check(lkb_gemv_q4_0_exp2(qs_a, d_a, qs_b, d_b, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, sel, sig,
                                    idx_out, w_out, y_a, y_b, ssq, eps, st), "k_gemv_q4_0_exp2"); }
inline int k_gemv_q4_0_exp(stream_t st, const void * qs, const void * d, const block_q8_1 * xq, int out_rows, int bpr,
                           int rows_per_expert, int xq_stride, const int * d_idx, float * y) {
    return check(lkb_gemv_q4_0_exp(qs, d, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, y, st), "k_gemv_q4_0_exp"); }
inline int k_swiglu(stream_t st, const float * gate, const float * up, int n, float * out, block_q8_1 * yq8,
                    const void * pf_qs = nullptr, const int * pf_idx = nullptr, int pf_rows_per_expert = 0, int pf_bpr = 0,
                    long pf_bytes = 0) {
    return check(lkb_swiglu(gate, up, n, out, yq8, pf_qs, pf_idx, pf_rows_per_expert, pf_bpr, pf_bytes, st), "k_swiglu"); }
inline int k_moe_accum4(stream_t st, float * dst, const float * down4, const float * d_w, int n, LKNormProd np) {
    return check(lkb_moe_accum4(dst, down4, d_w, n, &np, st), "k_moe_accum4"); }
inline int k_moe_down_accum(stream_t st, const void * qs, const void * d, const block_q8_1 * xq, int out_rows, int bpr,
                            int rows_per_expert, int xq_stride, const int * d_idx, const float * d_w, float * dst, LKNormProd np) {
    return check(lkb_moe_down_accum(qs, d, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, d_w, dst, &np, st), "k_moe_down_accum"); }
inline int k_router_dot(stream_t st, const float * h, const float * gate_inp, float * logits, const float * bias,
                        float * sel, float * sig, const float * ssq, float eps) {
    return check(lkb_router_dot(h, gate_inp, logits, bias, sel, sig, ssq, eps, st), "k_router_dot"); }
inline int k_router_top4(stream_t st, const float * logits, const float * bias, int * idx_out, float * w_out) {
    return check(lkb_router_top4(logits, bias, idx_out, w_out, st), "k_router_top4"); }

// ---- prefill (the launch grid carried m / rows in the reference; here it is the trailing argument) ------
inline int k_pf_norm(stream_t st, int m, const float * X, const float * w, int plain, PfAct a, float * inv_out, float * h32) {
    return check(lkb_pf_norm(X, w, plain, a, inv_out, h32, m, st), "k_pf_norm"); }
inline int k_pf_quant_rows(stream_t st, int rows, const float * X, int ld, int kb, PfAct a) {
    return check(lkb_pf_quant_rows(X, ld, kb, a, rows, st), "k_pf_quant_rows"); }
inline int k_pf_swiglu(stream_t st, int rows, const float * Y, int ld, int up_off, int kb, PfAct a) {
    return check(lkb_pf_swiglu(Y, ld, up_off, kb, a, rows, st), "k_pf_swiglu"); }
inline int k_pf_router(stream_t st, const float * H, int m, const float * Wr, const float * bias, const float * inv, float * sel, float * sig) {
    return check(lkb_pf_router_tiled(H, m, Wr, bias, inv, sel, sig, st), "k_pf_router"); }
inline int k_pf_router_small(stream_t st, int m, const float * H, const float * Wr, const float * bias, const float * inv, float * sel, float * sig) {
    return check(lkb_pf_router_small(H, m, Wr, bias, inv, sel, sig, st), "k_pf_router_small"); }
inline int k_pf_select(stream_t st, const float * sel, const float * sig, int m, int * idx, float * w) {
    return check(lkb_pf_select(sel, sig, m, idx, w, st), "k_pf_select"); }
inline int k_pf_moe_count(stream_t st, const int * idx, int n, int * cnt) { return check(lkb_pf_moe_count(idx, n, cnt, st), "k_pf_moe_count"); }
inline int k_pf_moe_plan(stream_t st, const int * cnt, int * off, int * tiles, int * ntiles) {
    return check(lkb_pf_moe_plan(cnt, off, tiles, ntiles, st), "k_pf_moe_plan"); }
inline int k_pf_moe_scatter(stream_t st, const int * idx, int n, const int * off, int * perm) {
    return check(lkb_pf_moe_scatter(idx, n, off, perm, st), "k_pf_moe_scatter"); }
inline int k_pf_moe_combine(stream_t st, int m, float * X, const float * D, const float * w) {
    return check(lkb_pf_moe_combine(X, D, w, m, st), "k_pf_moe_combine"); }
inline int k_pf_moe_combine_norm(stream_t st, int m, float * X, const float * D, const float * w, const float * nw, PfAct a, float * inv_out) {
    return check(lkb_pf_moe_combine_norm(X, D, w, nw, a, inv_out, m, st), "k_pf_moe_combine_norm"); }
inline int k_pf_pack_q8_1(stream_t st, PfAct a, int t, block_q8_1 * y) { return check(lkb_pf_pack_q8_1(a, t, y, st), "k_pf_pack_q8_1"); }

// ---- output projection, argmax, embedding row (ref: src/kernels.cu:359, 426, 855, 954-995) ----------------
inline int k_gemv_q6_K(stream_t st, const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const void * d, const block_q8_1 * xq,
                       int out_rows, int sbpr, float * y, const float * ssq, float eps) {
    return check(lkb_gemv_q6_K(ql, qh, sc, d, xq, out_rows, sbpr, y, ssq, eps, st), "k_gemv_q6_K"); }
inline int k_gemv_q6_K_dp4a(stream_t st, const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const void * d, const block_q8_1 * xq,
                            int out_rows, int sbpr, float * y, const float * ssq, float eps) {
    return check(lkb_gemv_q6_K(ql, qh, sc, d, xq, out_rows, sbpr, y, ssq, eps, st), "k_gemv_q6_K_dp4a"); }
inline int k_argmax_part(stream_t st, const float * v, int n, float * pv, int * pi) { return check(lkb_argmax_part(v, n, pv, pi, st), "k_argmax_part"); }
inline int k_argmax_final(stream_t st, const float * pv, const int * pi, int n, int * d_token, int * d_pos) {
    return check(lkb_argmax_final(pv, pi, n, d_token, d_pos, st), "k_argmax_final"); }
inline int k_embed_q6_K(stream_t st, const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const void * d, const int * d_token, int n, float * x) {
    return check(lkb_embed_q6_K(ql, qh, sc, d, d_token, n, x, st), "k_embed_q6_K"); }

// ---- sequence mixers (ref: src/kernels.cu:521, 871, 1303, 1562) ------------------------------------------------
inline int k_shortconv(stream_t st, const float * bcx, int t, const float * conv_w, float * hist, float * y, block_q8_1 * yq8) {
    return check(lkb_shortconv(bcx, t, conv_w, hist, y, yq8, LKB_HIDDEN, st), "k_shortconv"); }
inline int k_qk_norm_rope(stream_t st, float * qf, float * kf, const float * vf, const float * qn, const float * kn, const int * d_pos,
                          void * kc, void * vc) {
    return check(lkb_qk_norm_rope(qf, kf, vf, qn, kn, d_pos, kc, vc, 10000000.0f, st), "k_qk_norm_rope"); }   // src/kernels.cuh:23
inline int k_attn_split(stream_t st, const float * q, const void * kc, const void * vc, const int * d_pos, float * part) {
    return check(lkb_attn_split(q, kc, vc, d_pos, part, st), "k_attn_split"); }
inline int k_attn_combine(stream_t st, const float * part, const int * d_pos, float * out, block_q8_1 * yq8) {
    return check(lkb_attn_combine(part, d_pos, out, yq8, st), "k_attn_combine"); }

// ---- prefill mixers (ref: src/prefill.cu:856, 937, 960, 975, 1029) -----------------------------------------------
inline int k_pf_embed(stream_t st, int m, const uint8_t * ql, const uint8_t * qh, const int8_t * sc, const void * d, const int * toks, float * x) {
    return check(lkb_pf_embed(ql, qh, sc, d, toks, x, LKB_HIDDEN, m, st), "k_pf_embed"); }
inline int k_pf_conv(stream_t st, int m, const float * Y, const float * cw, const float * hist, PfAct a) {
    return check(lkb_pf_conv(Y, cw, hist, a, m, st), "k_pf_conv"); }
inline int k_pf_conv_hist(stream_t st, const float * Y, int m, float * hist) { return check(lkb_pf_conv_hist(Y, m, hist, st), "k_pf_conv_hist"); }
inline int k_pf_qknr(stream_t st, int m, const float * Y, const float * qn, const float * kn, int P, void * qh, void * kc, void * vc) {
    return check(lkb_pf_qknr(Y, qn, kn, P, qh, kc, vc, m, 10000000.0f, st), "k_pf_qknr"); }
inline int k_pf_attn(stream_t st, const void * qh, int m, int P, const void * kc, const void * vc, float * o) {
    return check(lkb_pf_attn(qh, m, P, kc, vc, o, st), "k_pf_attn"); }

// ---- host launchers, same signatures as the reference's (ref: src/prefill.cuh:69-71) ---------------------
inline void pf_gemm_dense(const PfGemm & g, stream_t st) { check(lkb_pf_gemm_dense(&g, st), "pf_gemm_dense"); }
inline void pf_gemm_moe(const PfGemm & g, int max_tiles, stream_t st) { check(lkb_pf_gemm_moe(&g, max_tiles, st), "pf_gemm_moe"); }
inline void pf_gemm_swiglu(const PfGemm & g, int max_tiles, stream_t st) { check(lkb_pf_gemm_swiglu(&g, max_tiles, st), "pf_gemm_swiglu"); }

}  // namespace lk
