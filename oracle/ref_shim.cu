/* ref_shim.cu - TEST INFRASTRUCTURE, not product code.
 *
 * extern "C" launchers around the reference engine's OWN hot-path kernels, so that the parity tests
 * and the benchmark's A/B leg can run them on the same B200 next to this repository's kernels.  The
 * reference sources (src/kernels.cu, src/prefill.cu of Nathan-T-Ray/lfm2-ampere) are compiled where
 * they lie, unchanged, for sm_100a by oracle/Makefile (target ref_kernels) together with this file
 * into oracle/_ref/libref_kernels.so; nothing of the reference is copied into this tree.  Only tests/,
 * the smoke check and bench.py's reference-kernel leg load that library; lfm2-ampere_b200/ never does.
 *
 * Each launcher uses the grid and block shape of the reference's own call site (cited per function,
 * <file>:<line> relative to the reference repository) with the shipped build flags
 * (Makefile:9-73: BIGBLOCK=1, NORM_ACCUM=1, NORM_GEMV=1, SPLIT=128, ...).
 * Return value: 0, or the cudaError_t of the launch.  The GEMM launchers of the reference exit() the
 * process on a bad shape; callers pass only shapes the reference accepts.
 */
#include "kernels.cuh"
#include "prefill.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))
static int ref_rc() { return (int) cudaGetLastError(); }
static cudaStream_t S(void * st) { return (cudaStream_t) st; }

/* ---- decode ------------------------------------------------------------------------------- */
/* tests/test_prefill.cu:143 */
REF_API int ref_quantize_q8_1(const float * x, void * y, int nblocks, void * st) {
    k_quantize_q8_1<<<nblocks, 32, 0, S(st)>>>(x, (block_q8_1 *) y, nblocks);
    return ref_rc();
}
/* src/engine.cu:515 */
REF_API int ref_rmsnorm_q8_1(const float * x, const float * w, int n, float eps, float * y32, void * y16, void * yq8, void * st) {
    k_rmsnorm_q8_1<<<1, 256, LK_HIDDEN * 4, S(st)>>>(x, w, n, eps, y32, (__half *) y16, (block_q8_1 *) yq8);
    return ref_rc();
}
/* src/engine.cu:524 (256-thread shape) and :580 (the 2048-row call sites use the 1024-thread shape) */
REF_API int ref_gemv_q4_0(const void * qs, const void * d, const void * xq, int out_rows, int bpr, float * y,
                          int add_residual, const float * ssq, float eps, int wide, void * st) {
    if (wide) k_gemv_q4_0<<<LK_GEMV_WBLOCKS(out_rows), LK_GEMV_WTHREADS, 0, S(st)>>>((const uint4 *) qs, (const __half *) d, (const block_q8_1 *) xq, out_rows, bpr, y, add_residual, ssq, eps);
    else      k_gemv_q4_0<<<LK_GEMV_BLOCKS(out_rows), 256, 0, S(st)>>>((const uint4 *) qs, (const __half *) d, (const block_q8_1 *) xq, out_rows, bpr, y, add_residual, ssq, eps);
    return ref_rc();
}
/* src/engine.cu:570 */
REF_API int ref_gemv_q4_0_prod(const void * qs, const void * d, const void * xq, int out_rows, int bpr, float * y,
                               int add_residual, const float * np_w, float * np_h32, void * np_yq8, float * np_ssq, void * st) {
    LKNormProd np; np.w = np_w; np.h32 = np_h32; np.yq8 = (block_q8_1 *) np_yq8; np.ssq = np_ssq;
    k_gemv_q4_0_prod<<<LK_GEMV_WBLOCKS(out_rows), LK_GEMV_WTHREADS, 0, S(st)>>>((const uint4 *) qs, (const __half *) d, (const block_q8_1 *) xq, out_rows, bpr, y, add_residual, np);
    return ref_rc();
}
/* src/engine.cu:739-758 */
REF_API int ref_router_dot(const float * h, const float * gate_inp, float * logits, const float * bias,
                           float * sel, float * sig, const float * ssq, float eps, void * st) {
    k_router_dot<<<LK_N_EXPERTS, 32, 0, S(st)>>>(h, gate_inp, logits, bias, sel, sig, ssq, eps);
    return ref_rc();
}
REF_API int ref_router_top4(const float * logits, const float * bias, int * idx, float * w, void * st) {
    k_router_top4<<<1, LK_N_EXPERTS, 0, S(st)>>>(logits, bias, idx, w);
    return ref_rc();
}
/* src/engine.cu:766-777 (d_idx group live, router-in-prologue group null) */
REF_API int ref_gemv_q4_0_exp2(const void * qs_a, const void * d_a, const void * qs_b, const void * d_b, const void * xq,
                               int out_rows, int bpr, int rows_per_expert, int xq_stride, const int * d_idx,
                               float * y_a, float * y_b, const float * ssq, float eps, void * st) {
    k_gemv_q4_0_exp2<<<dim3((out_rows + 7) / 8, 2 * LK_TOP_K), 256, 0, S(st)>>>(
        (const uint4 *) qs_a, (const __half *) d_a, (const uint4 *) qs_b, (const __half *) d_b, (const block_q8_1 *) xq,
        out_rows, bpr, rows_per_expert, xq_stride, d_idx, nullptr, nullptr, nullptr, nullptr, y_a, y_b, ssq, eps);
    return ref_rc();
}
/* src/engine.cu:789-791, without the speculative prefetch (it changes no result) */
REF_API int ref_swiglu(const float * gate, const float * up, int n, float * out, void * yq8, void * st) {
    k_swiglu<<<(n + 127) / 128, 256, 0, S(st)>>>(gate, up, n, out, (block_q8_1 *) yq8);
    return ref_rc();
}
/* the same with the prefetch of the selected experts' down rows, as the engine launches it */
REF_API int ref_swiglu_prefetch(const float * gate, const float * up, int n, float * out, void * yq8, const void * pf_qs,
                                const int * pf_idx, int pf_rows_per_expert, int pf_bpr, long pf_bytes, void * st) {
    k_swiglu<<<(n + 127) / 128, 256, 0, S(st)>>>(gate, up, n, out, (block_q8_1 *) yq8, (const uint4 *) pf_qs, pf_idx,
                                                  pf_rows_per_expert, pf_bpr, pf_bytes);
    return ref_rc();
}
/* src/engine.cu:806-809 */
REF_API int ref_moe_down_accum(const void * qs, const void * d, const void * xq, int out_rows, int bpr, int rows_per_expert,
                               int xq_stride, const int * d_idx, const float * d_w, float * dst,
                               const float * np_w, float * np_h32, void * np_yq8, float * np_ssq, void * st) {
    LKNormProd np; np.w = np_w; np.h32 = np_h32; np.yq8 = (block_q8_1 *) np_yq8; np.ssq = np_ssq;
    k_moe_down_accum<<<out_rows / 32, 1024, 0, S(st)>>>((const uint4 *) qs, (const __half *) d, (const block_q8_1 *) xq,
                                                       out_rows, bpr, rows_per_expert, xq_stride, d_idx, d_w, dst, np);
    return ref_rc();
}

/* ---- batched prefill ------------------------------------------------------------------------ */
static PfAct act(void * qs, void * sc) { PfAct a; a.qs = (int8_t *) qs; a.sc = (float2 *) sc; return a; }
/* src/engine.cu:1031,1135 */
REF_API int ref_pf_norm(const float * X, const float * w, int plain, void * aqs, void * asc, float * inv, float * h32, int m, void * st) {
    k_pf_norm<<<m, 256, 0, S(st)>>>(X, w, plain, act(aqs, asc), inv, h32);
    return ref_rc();
}
/* tests/test_prefill.cu:96 */
REF_API int ref_pf_quant_rows(const float * X, int ld, int kb, void * aqs, void * asc, int rows, void * st) {
    k_pf_quant_rows<<<dim3(rows, (kb + 7) / 8), 256, 0, S(st)>>>(X, ld, kb, act(aqs, asc));
    return ref_rc();
}
/* src/engine.cu:1210 */
REF_API int ref_pf_swiglu(const float * Y, int ld, int up_off, int kb, void * aqs, void * asc, int rows, void * st) {
    k_pf_swiglu<<<dim3(rows, (kb + 7) / 8), 256, 0, S(st)>>>(Y, ld, up_off, kb, act(aqs, asc));
    return ref_rc();
}
/* src/engine.cu:1171-1176: the small form up to 256 tokens, the tiled form beyond (force: 1 small, 2 tiled) */
REF_API int ref_pf_router(const float * H, int m, const float * Wr, const float * bias, const float * inv, float * sel,
                          float * sig, int force, void * st) {
    const bool small_form = force ? force == 1 : m <= 256;
    if (small_form) k_pf_router_small<<<dim3(LK_N_EXPERTS, m), 32, 0, S(st)>>>(H, Wr, bias, inv, sel, sig);
    else            k_pf_router<<<(m + 63) / 64, 256, 0, S(st)>>>(H, m, Wr, bias, inv, sel, sig);
    return ref_rc();
}
/* src/engine.cu:1179 */
REF_API int ref_pf_select(const float * sel, const float * sig, int m, int * idx, float * w, void * st) {
    k_pf_select<<<(m + 7) / 8, 256, 0, S(st)>>>(sel, sig, m, idx, w);
    return ref_rc();
}
/* src/engine.cu:1186-1196: memset, count, plan, scatter */
REF_API int ref_pf_moe_plan(const int * idx, int ns, int * cnt, int * off, void * tiles, int * ntiles, int * perm, void * st) {
    cudaError_t e = cudaMemsetAsync(cnt, 0, LK_N_EXPERTS * 4, S(st));
    if (e != cudaSuccess) return (int) e;
    k_pf_moe_count<<<(ns + 255) / 256, 256, 0, S(st)>>>(idx, ns, cnt);
    k_pf_moe_plan<<<1, 32, 0, S(st)>>>(cnt, off, (int4 *) tiles, ntiles);
    k_pf_moe_scatter<<<LK_N_EXPERTS, 1024, 0, S(st)>>>(idx, ns, off, perm);
    return ref_rc();
}
/* src/prefill.cuh:69-71.  g points at a PfGemm (same layout as lkb_pf_gemm). */
REF_API int ref_pf_gemm_dense(const void * g, void * st) { pf_gemm_dense(*(const PfGemm *) g, S(st)); return ref_rc(); }
REF_API int ref_pf_gemm_moe(const void * g, int max_tiles, void * st) { pf_gemm_moe(*(const PfGemm *) g, max_tiles, S(st)); return ref_rc(); }
REF_API int ref_pf_gemm_swiglu(const void * g, int max_tiles, void * st) { pf_gemm_swiglu(*(const PfGemm *) g, max_tiles, S(st)); return ref_rc(); }
/* src/engine.cu:1229-1238 */
REF_API int ref_pf_moe_combine(float * X, const float * D, const float * w, int m, void * st) {
    k_pf_moe_combine<<<dim3(m, LK_HIDDEN / 256), 256, 0, S(st)>>>(X, D, w);
    return ref_rc();
}
REF_API int ref_pf_moe_combine_norm(float * X, const float * D, const float * w, const float * nw, void * aqs, void * asc,
                                    float * inv, int m, void * st) {
    k_pf_moe_combine_norm<<<m, 256, 0, S(st)>>>(X, D, w, nw, act(aqs, asc), inv);
    return ref_rc();
}
/* src/engine.cu:1546 */
REF_API int ref_pf_pack_q8_1(void * aqs, void * asc, int t, void * y, void * st) {
    k_pf_pack_q8_1<<<1, 64, 0, S(st)>>>(act(aqs, asc), t, (block_q8_1 *) y);
    return ref_rc();
}
REF_API int ref_sizeof_pf_gemm(void) { return (int) sizeof(PfGemm); }
