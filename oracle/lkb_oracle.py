"""ctypes view of the CPU checker (oracle/lkb_oracle.c).

TEST INFRASTRUCTURE ONLY.  Import this from tests/, from the smoke check and from
the benchmark's cpu-baseline leg -- never from the product package.  The arrays
are numpy; every function returns new arrays and leaves its inputs untouched
unless its name says "inplace".
"""
from __future__ import annotations

import ctypes as C
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_SO = _HERE / "_ref" / "liblkb_oracle.so"


def build(force: bool = False) -> pathlib.Path:
    """Compile the C restatement with the Makefile beside it (gcc, a second or two)."""
    src = _HERE / "lkb_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _SO


def _load():
    if not _SO.exists():
        build()
    return C.CDLL(str(_SO))


_lib = _load()

_u8p, _i8p = C.POINTER(C.c_uint8), C.POINTER(C.c_int8)
_u16p, _i32p = C.POINTER(C.c_uint16), C.POINTER(C.c_int32)
_f32p, _f64p = C.POINTER(C.c_float), C.POINTER(C.c_double)


def _p(a, ct):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be contiguous"
    return a.ctypes.data_as(ct)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


_lib.orc_f32_to_f16.restype = C.c_uint16
_lib.orc_f32_to_f16.argtypes = [C.c_float]
_lib.orc_f16_to_f32.restype = C.c_float
_lib.orc_f16_to_f32.argtypes = [C.c_uint16]
_lib.orc_rmsnorm_ss2048.restype = C.c_float
_lib.orc_norm_ssq_total.restype = C.c_float
_lib.orc_norm_inv.restype = C.c_float
_lib.orc_norm_inv.argtypes = [_f32p, C.c_float]
_lib.orc_router_margin.restype = C.c_float
_lib.orc_num_threads.restype = C.c_int

# block_q8_1 as the decode kernels see it: 36 bytes {fp16 d, fp16 sum, int8 qs[32]}
# (src/quant.cuh:27-31 of the reference).
BLOCK_Q8_1 = np.dtype([("d", "<u2"), ("s", "<u2"), ("qs", "i1", (32,))])
assert BLOCK_Q8_1.itemsize == 36


def pack_blocks(q, d16, s16):
    """(q[nblk*32], d16[nblk], s16[nblk]) -> structured array of 36-byte blocks."""
    n = d16.shape[0]
    out = np.zeros(n, dtype=BLOCK_Q8_1)
    out["d"] = d16
    out["s"] = s16
    out["qs"] = q.reshape(n, 32)
    return out


def unpack_blocks(blocks):
    b = np.asarray(blocks).view(BLOCK_Q8_1).reshape(-1)
    return np.ascontiguousarray(b["qs"]).reshape(-1), np.ascontiguousarray(b["d"]), np.ascontiguousarray(b["s"])


def f16_bits_to_f32(u16):
    return np.asarray(u16, dtype=np.uint16).view(np.float16).astype(np.float32)


def quantize_q8_1(x):
    x = _c(x, np.float32).reshape(-1)
    nblk = x.size // 32
    q = np.empty(nblk * 32, np.int8)
    d16 = np.empty(nblk, np.uint16)
    s16 = np.empty(nblk, np.uint16)
    _lib.orc_quantize_q8_1(_p(x, _f32p), nblk, _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p))
    return q, d16, s16


def block_sumi(qs, aq, rows, bpr):
    qs = _c(qs, np.uint8).reshape(-1)
    aq = _c(aq, np.int8).reshape(-1)
    out = np.empty((rows, bpr), np.int32)
    _lib.orc_block_sumi(_p(qs, _u8p), _p(aq, _i8p), rows, bpr, _p(out, _i32p))
    return out


def gemv_q4_0(qs, d, act, rows, bpr, y_in=None, ninv=1.0):
    """act = (q, d16, s16).  Returns y (fp32, reference summation order)."""
    qs = _c(qs, np.uint8).reshape(-1)
    d = _c(d, np.uint16).reshape(-1)
    q, d16, s16 = (_c(act[0], np.int8), _c(act[1], np.uint16), _c(act[2], np.uint16))
    y = np.zeros(rows, np.float32) if y_in is None else _c(y_in, np.float32).copy()
    _lib.orc_gemv_q4_0(_p(qs, _u8p), _p(d, _u16p), _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p),
                       rows, bpr, _p(y, _f32p), 0 if y_in is None else 1, C.c_float(ninv))
    return y


def gemv_q4_0_f64(qs, d, act, rows, bpr):
    qs = _c(qs, np.uint8).reshape(-1)
    d = _c(d, np.uint16).reshape(-1)
    q, d16, s16 = (_c(act[0], np.int8), _c(act[1], np.uint16), _c(act[2], np.uint16))
    y = np.empty(rows, np.float64)
    mag = np.empty(rows, np.float64)
    _lib.orc_gemv_q4_0_f64(_p(qs, _u8p), _p(d, _u16p), _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p),
                           rows, bpr, _p(y, _f64p), _p(mag, _f64p))
    return y, mag


def rmsnorm_q8_1(x, w, eps=1e-5, inv_override=0.0):
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    assert x.size == 2048
    y32 = np.empty(2048, np.float32)
    q = np.empty(2048, np.int8)
    d16 = np.empty(64, np.uint16)
    s16 = np.empty(64, np.uint16)
    inv = C.c_float(0)
    _lib.orc_rmsnorm_q8_1(_p(x, _f32p), _p(w, _f32p), C.c_float(eps), C.c_float(inv_override),
                          _p(y32, _f32p), _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p), C.byref(inv))
    return y32, (q, d16, s16), inv.value


def rmsnorm_ss2048(x):
    x = _c(x, np.float32)
    return float(_lib.orc_rmsnorm_ss2048(_p(x, _f32p)))


def norm_prod(x, w):
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    n = x.size
    h32 = np.empty(n, np.float32)
    q = np.empty(n, np.int8)
    d16 = np.empty(n // 32, np.uint16)
    s16 = np.empty(n // 32, np.uint16)
    ssq = np.empty(n // 32, np.float32)
    _lib.orc_norm_prod(_p(x, _f32p), _p(w, _f32p), n, _p(h32, _f32p), _p(q, _i8p), _p(d16, _u16p),
                       _p(s16, _u16p), _p(ssq, _f32p))
    return h32, (q, d16, s16), ssq


def norm_inv(ssq, eps=1e-5):
    ssq = _c(ssq, np.float32)
    return float(_lib.orc_norm_inv(_p(ssq, _f32p), C.c_float(eps)))


def norm_ssq_total(ssq):
    ssq = _c(ssq, np.float32)
    return float(_lib.orc_norm_ssq_total(_p(ssq, _f32p)))


def router_dot(h, W, ninv=1.0):
    h = _c(h, np.float32)
    W = _c(W, np.float32)
    n_exp, hidden = W.shape
    logits = np.empty(n_exp, np.float32)
    _lib.orc_router_dot(_p(h, _f32p), _p(W, _f32p), n_exp, hidden, C.c_float(ninv), _p(logits, _f32p))
    return logits


def router_gate(logits, bias=None, softmax=False):
    logits = _c(logits, np.float32)
    n = logits.size
    b = None if bias is None else _c(bias, np.float32)
    sel = np.empty(n, np.float32)
    sig = np.empty(n, np.float32)
    _lib.orc_router_gate(_p(logits, _f32p), _p(b, _f32p), n, 1 if softmax else 0, _p(sel, _f32p), _p(sig, _f32p))
    return sel, sig


def router_select(sel, sig):
    sel = _c(sel, np.float32)
    sig = _c(sig, np.float32)
    idx = np.empty(4, np.int32)
    w = np.empty(4, np.float32)
    _lib.orc_router_select(_p(sel, _f32p), _p(sig, _f32p), sel.size, _p(idx, _i32p), _p(w, _f32p))
    return idx, w


def router_margin(sel):
    sel = _c(sel, np.float32)
    return float(_lib.orc_router_margin(_p(sel, _f32p), sel.size))


def swiglu(gate, up):
    gate = _c(gate, np.float32).reshape(-1)
    up = _c(up, np.float32).reshape(-1)
    out = np.empty_like(gate)
    _lib.orc_swiglu(_p(gate, _f32p), _p(up, _f32p), gate.size, _p(out, _f32p))
    return out


def gemv_q4_0_exp(qs, d, act, out_rows, bpr, rows_per_expert, xq_stride, idx, ninv=1.0):
    qs = _c(qs, np.uint8).reshape(-1)
    d = _c(d, np.uint16).reshape(-1)
    q, d16, s16 = (_c(act[0], np.int8), _c(act[1], np.uint16), _c(act[2], np.uint16))
    idx = _c(idx, np.int32)
    y = np.empty(4 * out_rows, np.float32)
    _lib.orc_gemv_q4_0_exp(_p(qs, _u8p), _p(d, _u16p), _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p), out_rows, bpr,
                           rows_per_expert, xq_stride, _p(idx, _i32p), C.c_float(ninv), _p(y, _f32p))
    return y


def moe_down_accum(qs, d, act, out_rows, bpr, rows_per_expert, xq_stride, idx, wk, x, nw=None):
    """Returns (x_new, h32, (q, d16, s16), ssq); the last three are None when nw is None."""
    qs = _c(qs, np.uint8).reshape(-1)
    d = _c(d, np.uint16).reshape(-1)
    q, d16, s16 = (_c(act[0], np.int8), _c(act[1], np.uint16), _c(act[2], np.uint16))
    idx = _c(idx, np.int32)
    wk = _c(wk, np.float32)
    x = _c(x, np.float32).copy()
    if nw is not None:
        nw = _c(nw, np.float32)
        h32 = np.empty(out_rows, np.float32)
        oq = np.empty(out_rows, np.int8)
        od = np.empty(out_rows // 32, np.uint16)
        os_ = np.empty(out_rows // 32, np.uint16)
        ssq = np.empty(out_rows // 32, np.float32)
    else:
        h32 = oq = od = os_ = ssq = None
    _lib.orc_moe_down_accum(_p(qs, _u8p), _p(d, _u16p), _p(q, _i8p), _p(d16, _u16p), _p(s16, _u16p), out_rows, bpr,
                            rows_per_expert, xq_stride, _p(idx, _i32p), _p(wk, _f32p), _p(x, _f32p),
                            _p(nw, _f32p), _p(h32, _f32p), _p(oq, _i8p), _p(od, _u16p), _p(os_, _u16p), _p(ssq, _f32p))
    return x, h32, (None if nw is None else (oq, od, os_)), ssq


# ---------------------------------------------------------------- prefill ---
def pf_quant_rows(X, kb):
    X = _c(X, np.float32)
    rows, ld = X.shape
    qs = np.empty((rows, kb * 32), np.int8)
    sc = np.empty((rows, kb, 2), np.float32)
    _lib.orc_pf_quant_rows(_p(X, _f32p), rows, ld, kb, _p(qs, _i8p), _p(sc, _f32p))
    return qs, sc


def pf_swiglu(Y, up_off, kb, v=None):
    """Y rows hold [gate | up].  v (optional, [rows][kb*32]) overrides the computed silu(g)*u."""
    Y = _c(Y, np.float32)
    rows, ld = Y.shape
    qs = np.empty((rows, kb * 32), np.int8)
    sc = np.empty((rows, kb, 2), np.float32)
    vb = np.empty((rows, kb * 32), np.float32) if v is None else _c(v, np.float32).copy()
    _lib.orc_pf_swiglu(_p(Y, _f32p), rows, ld, up_off, kb, _p(qs, _i8p), _p(sc, _f32p), _p(vb, _f32p),
                       0 if v is None else 1)
    return qs, sc, vb


def pf_norm(X, w, plain, inv_override=None, want_h32=False):
    X = _c(X, np.float32)
    w = _c(w, np.float32)
    m = X.shape[0]
    qs = np.empty((m, 2048), np.int8)
    sc = np.empty((m, 64, 2), np.float32)
    inv = np.empty(m, np.float32)
    h32 = np.empty((m, 2048), np.float32) if want_h32 else None
    io = None if inv_override is None else _c(inv_override, np.float32)
    _lib.orc_pf_norm(_p(X, _f32p), _p(w, _f32p), m, 1 if plain else 0, _p(io, _f32p), _p(qs, _i8p), _p(sc, _f32p),
                     _p(inv, _f32p), _p(h32, _f32p))
    return qs, sc, inv, h32


def pf_router_logits(H, W, inv, order):
    H = _c(H, np.float32)
    W = _c(W, np.float32)
    inv = _c(inv, np.float32)
    m = H.shape[0]
    logits = np.empty((m, 64), np.float32)
    _lib.orc_pf_router_logits(_p(H, _f32p), m, _p(W, _f32p), _p(inv, _f32p), order, _p(logits, _f32p))
    return logits


def pf_gate(logits, bias=None, softmax=False):
    sel = np.empty_like(logits)
    sig = np.empty_like(logits)
    for t in range(logits.shape[0]):
        sel[t], sig[t] = router_gate(logits[t], bias, softmax)
    return sel, sig


def pf_select(sel, sig):
    sel = _c(sel, np.float32)
    sig = _c(sig, np.float32)
    m = sel.shape[0]
    idx = np.empty((m, 4), np.int32)
    w = np.empty((m, 4), np.float32)
    _lib.orc_pf_select(_p(sel, _f32p), _p(sig, _f32p), m, _p(idx, _i32p), _p(w, _f32p))
    return idx, w


def moe_plan(idx, n_exp=64):
    """idx: flat slot->expert.  Returns cnt, off, tiles[ntiles][4], perm."""
    idx = _c(idx, np.int32).reshape(-1)
    n = idx.size
    cnt = np.empty(n_exp, np.int32)
    off = np.empty(n_exp, np.int32)
    tiles = np.zeros((n // 64 + n_exp, 4), np.int32)
    nt = C.c_int(0)
    perm = np.empty(n, np.int32)
    _lib.orc_moe_count(_p(idx, _i32p), n, n_exp, _p(cnt, _i32p))
    _lib.orc_moe_plan(_p(cnt, _i32p), n_exp, _p(off, _i32p), _p(tiles, _i32p), C.byref(nt))
    _lib.orc_moe_scatter(_p(idx, _i32p), n, n_exp, _p(off, _i32p), _p(perm, _i32p))
    return cnt, off, tiles[: nt.value].copy(), perm


class _Gemm(C.Structure):
    _fields_ = [("qs", _u8p * 3), ("d", _u16p * 3), ("seg_end", C.c_int * 3), ("N", C.c_int), ("bpr", C.c_int),
                ("exp_stride", C.c_longlong), ("aqs", _i8p), ("asc", _f32p), ("ntok", C.c_int),
                ("perm", _i32p), ("tiles", _i32p), ("ntiles", C.c_int), ("a_shift", C.c_int),
                ("scale", _f32p), ("out", _f32p), ("out_ld", C.c_int), ("add", C.c_int)]


def _mk_gemm(segs, seg_end, N, bpr, exp_stride, aqs, asc, ntok, perm, tiles, a_shift, scale, out, out_ld, add, keep):
    g = _Gemm()
    for i in range(3):
        q, d = segs[min(i, len(segs) - 1)]
        q = _c(q, np.uint8).reshape(-1)
        d = _c(d, np.uint16).reshape(-1)
        keep += [q, d]
        g.qs[i] = _p(q, _u8p)
        g.d[i] = _p(d, _u16p)
        g.seg_end[i] = seg_end[min(i, len(seg_end) - 1)]
    g.N, g.bpr, g.exp_stride = N, bpr, exp_stride
    aqs = _c(aqs, np.int8)
    asc = _c(asc, np.float32)
    keep += [aqs, asc]
    g.aqs, g.asc, g.ntok = _p(aqs, _i8p), _p(asc, _f32p), ntok
    if perm is not None:
        perm = _c(perm, np.int32)
        tiles = _c(tiles, np.int32)
        keep += [perm, tiles]
        g.perm, g.tiles, g.ntiles = _p(perm, _i32p), _p(tiles, _i32p), tiles.shape[0]
    g.a_shift = a_shift
    if scale is not None:
        scale = _c(scale, np.float32)
        keep.append(scale)
        g.scale = _p(scale, _f32p)
    g.out = _p(out, _f32p) if out is not None else None
    g.out_ld, g.add = out_ld, add
    return g


def set_gemm_fold(fold):
    """Per-block term of pf_gemm / pf_gemm_swiglu: True (default) the reference's shipped folded form,
    False the exact term of the decode kernels."""
    _lib.orc_set_gemm_fold(1 if fold else 0)


def pf_gemm(segs, seg_end, N, bpr, aqs, asc, *, ntok=0, exp_stride=0, perm=None, tiles=None, a_shift=0,
            scale=None, out_rows=None, out_init=None, add=0, want_f64=False, want_slack=False):
    """The grouped / dense GEMM.  segs = [(qs, d), ...] up to three stacked tensors.
    Returns out (fp32, block-order accumulation) and, with want_f64, (out, out64, mag[, slack])."""
    rows = out_rows if out_rows is not None else ntok
    out = np.full((rows, N), np.nan, np.float32) if out_init is None else _c(out_init, np.float32).copy()
    keep = []
    g = _mk_gemm(segs, seg_end, N, bpr, exp_stride, aqs, asc, ntok, perm, tiles, a_shift, scale, out, N, add, keep)
    o64 = np.zeros((rows, N), np.float64) if want_f64 else None
    mag = np.zeros((rows, N), np.float64) if want_f64 else None
    slack = np.zeros((rows, N), np.float64) if (want_f64 and want_slack) else None
    _lib.orc_pf_gemm(C.byref(g), _p(o64, _f64p), _p(mag, _f64p), _p(slack, _f64p))
    if want_f64 and want_slack:
        return out, o64, mag, slack
    return (out, o64, mag) if want_f64 else out


def pf_gemm_swiglu(gate, up, N, bpr, aqs, asc, *, ntok=0, exp_stride=0, perm=None, tiles=None, a_shift=0,
                   scale=None, out_rows=None, v=None):
    rows = out_rows if out_rows is not None else ntok
    okb = N // 32
    oqs = np.zeros((rows, okb * 32), np.int8)
    osc = np.zeros((rows, okb, 2), np.float32)
    vb = np.zeros((rows, N), np.float32) if v is None else _c(v, np.float32).copy()
    keep = []
    g = _mk_gemm([gate, up], [N, N], N, bpr, exp_stride, aqs, asc, ntok, perm, tiles, a_shift, scale, None, N, 0, keep)
    _lib.orc_pf_gemm_swiglu(C.byref(g), _p(oqs, _i8p), _p(osc, _f32p), okb, _p(vb, _f32p), 0 if v is None else 1)
    return oqs, osc, vb


def fused_epilogue_sums(v):
    """8 * fp16(block sum) per 32-element block of v, summed in the order of the reference's fused SwiGLU epilogue."""
    v = _c(v, np.float32)
    out = np.empty(v.size // 32, np.float32)
    _lib.orc_fused_epilogue_sums(_p(v, _f32p), C.c_longlong(v.size // 32), _p(out, _f32p))
    return out.reshape(v.shape[:-1] + (v.shape[-1] // 32,))


def pf_combine(X, D, w):
    X = _c(X, np.float32).copy()
    D = _c(D, np.float32)
    w = _c(w, np.float32)
    m, hidden = X.shape
    _lib.orc_pf_combine(_p(X, _f32p), _p(D, _f32p), _p(w, _f32p), m, hidden)
    return X


def pf_combine_norm(X, D, w, nw, inv_override=None):
    X = _c(X, np.float32).copy()
    D = _c(D, np.float32)
    w = _c(w, np.float32)
    nw = _c(nw, np.float32)
    m = X.shape[0]
    qs = np.empty((m, 2048), np.int8)
    sc = np.empty((m, 64, 2), np.float32)
    inv = np.empty(m, np.float32)
    io = None if inv_override is None else _c(inv_override, np.float32)
    _lib.orc_pf_combine_norm(_p(X, _f32p), _p(D, _f32p), _p(w, _f32p), _p(nw, _f32p), m, _p(io, _f32p),
                             _p(qs, _i8p), _p(sc, _f32p), _p(inv, _f32p))
    return X, qs, sc, inv


def pf_pack_q8_1(qs, sc, t):
    qs = _c(qs, np.int8)
    sc = _c(sc, np.float32)
    kb = sc.shape[1]
    out = np.zeros(kb * 36, np.uint8)
    _lib.orc_pf_pack_q8_1(_p(qs, _i8p), _p(sc, _f32p), t, kb, _p(out, _u8p))
    return out.view(BLOCK_Q8_1)


def num_threads():
    return int(_lib.orc_num_threads())


def set_num_threads(n):
    _lib.orc_set_num_threads(int(n))


# ------------------------------------------------------------ Q6_K lm_head --
def gemv_q6_K(ql, qh, sc, d, act, rows, sbpr=8, ninv=1.0):
    """act = (q, d16, s16) of the activation; shipped (dp4a) summation order."""
    ql, qh = _c(ql, np.uint8).reshape(-1), _c(qh, np.uint8).reshape(-1)
    sc, d = _c(sc, np.int8).reshape(-1), _c(d, np.uint16).reshape(-1)
    q, d16 = _c(act[0], np.int8), _c(act[1], np.uint16)
    y = np.empty(rows, np.float32)
    _lib.orc_gemv_q6_K(_p(ql, _u8p), _p(qh, _u8p), _p(sc, _i8p), _p(d, _u16p), _p(q, _i8p), _p(d16, _u16p),
                       rows, sbpr, C.c_float(ninv), _p(y, _f32p))
    return y


def gemv_q6_K_f64(ql, qh, sc, d, q, d8_f32, rows, sbpr=8):
    ql, qh = _c(ql, np.uint8).reshape(-1), _c(qh, np.uint8).reshape(-1)
    sc, d = _c(sc, np.int8).reshape(-1), _c(d, np.uint16).reshape(-1)
    q, d8 = _c(q, np.int8), _c(d8_f32, np.float32)
    y, mag = np.empty(rows, np.float64), np.empty(rows, np.float64)
    _lib.orc_gemv_q6_K_f64(_p(ql, _u8p), _p(qh, _u8p), _p(sc, _i8p), _p(d, _u16p), _p(q, _i8p), _p(d8, _f32p),
                           rows, sbpr, _p(y, _f64p), _p(mag, _f64p))
    return y, mag


def q6_group_sums(ql, qh, aq, rows, sbpr=8):
    ql, qh, aq = _c(ql, np.uint8).reshape(-1), _c(qh, np.uint8).reshape(-1), _c(aq, np.int8)
    out = np.empty((rows, sbpr, 32), np.int32)
    _lib.orc_q6_group_sums(_p(ql, _u8p), _p(qh, _u8p), _p(aq, _i8p), rows, sbpr, _p(out, _i32p))
    return out


def embed_q6_K(ql, qh, sc, d, token, sbpr=8):
    ql, qh = _c(ql, np.uint8).reshape(-1), _c(qh, np.uint8).reshape(-1)
    sc, d = _c(sc, np.int8).reshape(-1), _c(d, np.uint16).reshape(-1)
    x = np.empty(sbpr * 256, np.float32)
    _lib.orc_embed_q6_K(_p(ql, _u8p), _p(qh, _u8p), _p(sc, _i8p), _p(d, _u16p), token, sbpr, _p(x, _f32p))
    return x


def dequant_q6_K(ql, qh, sc, d, nblk):
    """All weights of nblk super-blocks as float32 (via the embed formula)."""
    return embed_q6_K(ql, qh, sc, d, 0, sbpr=nblk)


# ---- sequence mixers of a decode step --------------------------------------------------------------
def shortconv(bcx, conv_w, hist):
    """One conv step; returns (y, new_hist).  hist is not modified."""
    bcx, conv_w = _c(bcx, np.float32).reshape(-1), _c(conv_w, np.float32).reshape(-1)
    n = bcx.size // 3
    h = _c(hist, np.float32).reshape(-1).copy()
    y = np.empty(n, np.float32)
    _lib.orc_shortconv(_p(bcx, _f32p), _p(conv_w, _f32p), _p(h, _f32p), _p(y, _f32p), n)
    return y, h


def norm_rope_heads(x, w, pos, theta, inv_override=None):
    """x [n_heads*64] -> (rotated copy, inv per head) in the kernel's float32 order."""
    v = _c(x, np.float32).reshape(-1).copy()
    w = _c(w, np.float32).reshape(-1)
    nh = v.size // 64
    inv = np.empty(nh, np.float32)
    ov = None if inv_override is None else _c(inv_override, np.float32)
    _lib.orc_norm_rope_heads(_p(v, _f32p), _p(w, _f32p), nh, C.c_float(pos), C.c_float(theta),
                             None if ov is None else _p(ov, _f32p), _p(inv, _f32p))
    return v, inv


def norm_rope_heads_f64(x, w, pos, theta):
    """float64 form (tests/test_kernels.cu:91-110 for the rotation)."""
    v = np.asarray(x, np.float64).reshape(-1, 64)
    inv = 1.0 / np.sqrt((v * v).mean(axis=1, keepdims=True) + 1e-5)
    u = v * inv * np.asarray(w, np.float64)[None, :]
    i = np.arange(32)
    ang = float(pos) * np.power(float(theta), -2.0 * i / 64.0)
    c, s = np.cos(ang), np.sin(ang)
    out = np.empty_like(u)
    out[:, :32] = u[:, :32] * c - u[:, 32:] * s
    out[:, 32:] = u[:, :32] * s + u[:, 32:] * c
    return out.reshape(-1)


def f32_to_f16_bits(x):
    x = _c(x, np.float32).reshape(-1)
    out = np.empty(x.size, np.uint16)
    _lib.orc_f32_to_f16_array(_p(x, _f32p), x.size, _p(out, _u16p))
    return out


def attn_decode_f64(q, kc, vc, seq):
    q = _c(q, np.float32).reshape(-1)
    kc, vc = _c(kc, np.uint16).reshape(-1), _c(vc, np.uint16).reshape(-1)
    out = np.empty(32 * 64, np.float64)
    _lib.orc_attn_decode_f64(_p(q, _f32p), _p(kc, _u16p), _p(vc, _u16p), seq, _p(out, _f64p))
    return out


def pf_attn_f64(qh, m, P, kc, vc):
    """Causal chunk attention in float64 over fp16 bit patterns; returns [m, 2048]."""
    qh, kc, vc = (_c(a, np.uint16).reshape(-1) for a in (qh, kc, vc))
    out = np.empty((m, 2048), np.float64)
    _lib.orc_pf_attn_f64(_p(qh, _u16p), m, P, _p(kc, _u16p), _p(vc, _u16p), _p(out, _f64p))
    return out


def pf_conv(Y, conv_w, hist):
    """Chunk convolution = the decode step applied token by token.  Y [m, 6144]; returns (v [m, 2048], hist')."""
    Y = _c(Y, np.float32)
    h = _c(hist, np.float32).reshape(-1).copy()
    out = np.empty((Y.shape[0], 2048), np.float32)
    for t in range(Y.shape[0]):
        out[t], h = shortconv(Y[t], conv_w, h)
    return out, h
