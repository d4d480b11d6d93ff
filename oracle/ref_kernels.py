"""ctypes view of oracle/_ref/libref_kernels.so: the REFERENCE's own CUDA kernels (src/kernels.cu, src/prefill.cu,
compiled unchanged for sm_100a by `make -C oracle ref_kernels`) behind the extern "C" launchers of ref_shim.cu.

TEST INFRASTRUCTURE ONLY.  It is the GPU-side checker of the parity tests and the "kernel to beat" of the
benchmark's A/B leg; nothing under lfm2-ampere_b200/ loads it.  Every wrapper takes torch CUDA tensors and launches on
torch's current stream.
"""
from __future__ import annotations

import ctypes as C
import pathlib

_SO = pathlib.Path(__file__).resolve().parent / "_ref" / "libref_kernels.so"


def available() -> bool:
    return _SO.exists()


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not _SO.exists():
            raise RuntimeError(f"{_SO} is missing: build it with `make -C oracle ref_kernels` where the reference checkout is present")
        _lib = C.CDLL(str(_SO))
    return _lib


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _st():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ck(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference kernel {what}: cudaError {rc}")


def quantize_q8_1(x, y, nblocks):
    _ck(lib().ref_quantize_q8_1(_p(x), _p(y), nblocks, _st()), "k_quantize_q8_1")


def rmsnorm_q8_1(x, w, n, eps, y32, y16, yq8):
    _ck(lib().ref_rmsnorm_q8_1(_p(x), _p(w), n, C.c_float(eps), _p(y32), _p(y16), _p(yq8), _st()), "k_rmsnorm_q8_1")


def gemv_q4_0(qs, d, xq, out_rows, bpr, y, add_residual=0, ssq=None, eps=1e-5, wide=0):
    _ck(lib().ref_gemv_q4_0(_p(qs), _p(d), _p(xq), out_rows, bpr, _p(y), add_residual, _p(ssq), C.c_float(eps), wide, _st()),
        "k_gemv_q4_0")


def gemv_q4_0_prod(qs, d, xq, out_rows, bpr, y, add_residual, w=None, h32=None, yq8=None, ssq=None):
    _ck(lib().ref_gemv_q4_0_prod(_p(qs), _p(d), _p(xq), out_rows, bpr, _p(y), add_residual, _p(w), _p(h32), _p(yq8), _p(ssq),
                                 _st()), "k_gemv_q4_0_prod")


def router_dot(h, gate_inp, logits, bias=None, sel=None, sig=None, ssq=None, eps=1e-5):
    _ck(lib().ref_router_dot(_p(h), _p(gate_inp), _p(logits), _p(bias), _p(sel), _p(sig), _p(ssq), C.c_float(eps), _st()),
        "k_router_dot")


def router_top4(logits, bias, idx, w):
    _ck(lib().ref_router_top4(_p(logits), _p(bias), _p(idx), _p(w), _st()), "k_router_top4")


def gemv_q4_0_exp2(qs_a, d_a, qs_b, d_b, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, y_a, y_b, ssq=None, eps=1e-5):
    _ck(lib().ref_gemv_q4_0_exp2(_p(qs_a), _p(d_a), _p(qs_b), _p(d_b), _p(xq), out_rows, bpr, rows_per_expert, xq_stride,
                                 _p(d_idx), _p(y_a), _p(y_b), _p(ssq), C.c_float(eps), _st()), "k_gemv_q4_0_exp2")


def swiglu(gate, up, n, out, yq8):
    _ck(lib().ref_swiglu(_p(gate), _p(up), n, _p(out), _p(yq8), _st()), "k_swiglu")


def swiglu_prefetch(gate, up, n, out, yq8, pf_qs, pf_idx, pf_rows_per_expert, pf_bpr, pf_bytes):
    _ck(lib().ref_swiglu_prefetch(_p(gate), _p(up), n, _p(out), _p(yq8), _p(pf_qs), _p(pf_idx), pf_rows_per_expert, pf_bpr,
                                  C.c_long(pf_bytes), _st()), "k_swiglu")


def moe_down_accum(qs, d, xq, out_rows, bpr, rows_per_expert, xq_stride, d_idx, d_w, dst, w=None, h32=None, yq8=None, ssq=None):
    _ck(lib().ref_moe_down_accum(_p(qs), _p(d), _p(xq), out_rows, bpr, rows_per_expert, xq_stride, _p(d_idx), _p(d_w), _p(dst),
                                 _p(w), _p(h32), _p(yq8), _p(ssq), _st()), "k_moe_down_accum")


def pf_norm(X, w, plain, aqs, asc, inv, h32, m):
    _ck(lib().ref_pf_norm(_p(X), _p(w), plain, _p(aqs), _p(asc), _p(inv), _p(h32), m, _st()), "k_pf_norm")


def pf_quant_rows(X, ld, kb, aqs, asc, rows):
    _ck(lib().ref_pf_quant_rows(_p(X), ld, kb, _p(aqs), _p(asc), rows, _st()), "k_pf_quant_rows")


def pf_swiglu(Y, ld, up_off, kb, aqs, asc, rows):
    _ck(lib().ref_pf_swiglu(_p(Y), ld, up_off, kb, _p(aqs), _p(asc), rows, _st()), "k_pf_swiglu")


def pf_router(H, m, Wr, bias, inv, sel, sig, force=0):
    _ck(lib().ref_pf_router(_p(H), m, _p(Wr), _p(bias), _p(inv), _p(sel), _p(sig), force, _st()), "k_pf_router")


def pf_select(sel, sig, m, idx, w):
    _ck(lib().ref_pf_select(_p(sel), _p(sig), m, _p(idx), _p(w), _st()), "k_pf_select")


def pf_moe_plan(idx, ns, cnt, off, tiles, ntiles, perm):
    _ck(lib().ref_pf_moe_plan(_p(idx), ns, _p(cnt), _p(off), _p(tiles), _p(ntiles), _p(perm), _st()), "k_pf_moe_count/plan/scatter")


def pf_gemm_dense(g):
    """g: the product's PfGemm ctypes structure (same layout as the reference's PfGemm)."""
    assert lib().ref_sizeof_pf_gemm() == C.sizeof(g), "PfGemm layouts differ"
    _ck(lib().ref_pf_gemm_dense(C.byref(g), _st()), "pf_gemm_dense")


def pf_gemm_moe(g, max_tiles):
    assert lib().ref_sizeof_pf_gemm() == C.sizeof(g), "PfGemm layouts differ"
    _ck(lib().ref_pf_gemm_moe(C.byref(g), max_tiles, _st()), "pf_gemm_moe")


def pf_gemm_swiglu(g, max_tiles):
    assert lib().ref_sizeof_pf_gemm() == C.sizeof(g), "PfGemm layouts differ"
    _ck(lib().ref_pf_gemm_swiglu(C.byref(g), max_tiles, _st()), "pf_gemm_swiglu")


def pf_moe_combine(X, D, w, m):
    _ck(lib().ref_pf_moe_combine(_p(X), _p(D), _p(w), m, _st()), "k_pf_moe_combine")


def pf_moe_combine_norm(X, D, w, nw, aqs, asc, inv, m):
    _ck(lib().ref_pf_moe_combine_norm(_p(X), _p(D), _p(w), _p(nw), _p(aqs), _p(asc), _p(inv), m, _st()), "k_pf_moe_combine_norm")


def pf_pack_q8_1(aqs, asc, t, y):
    _ck(lib().ref_pf_pack_q8_1(_p(aqs), _p(asc), t, _p(y), _st()), "k_pf_pack_q8_1")
