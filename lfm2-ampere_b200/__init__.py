"""lfm2-ampere_b200 - B200 (sm_100a) hot path of lfm2-ampere behind a C ABI.

The product is ``liblkb.so`` (CUDA kernels + ``extern "C"`` entry points declared
in ``include/lkb.h``).  This package is the Python-side plumbing used by the
tests and the benchmark: it loads the library with ctypes, gives every entry
point its argument types straight from the header, and offers thin wrappers
that take torch tensors (torch is used for device memory and streams only).

There is no CPU fallback: importing works anywhere (so that the symbol table can
be checked without a GPU), but every compute call needs the CUDA library and a
B200, and raises otherwise.
"""
from __future__ import annotations

import ctypes as C
import pathlib
import re

_HERE = pathlib.Path(__file__).resolve().parent
ROOT = _HERE.parent
HEADER = ROOT / "include" / "lkb.h"
LIB_PATH = _HERE / "liblkb.so"


class LkbError(RuntimeError):
    pass


class PfAct(C.Structure):
    """lkb_pf_act (passed by value)."""
    _fields_ = [("qs", C.c_void_p), ("sc", C.c_void_p)]


class NormProd(C.Structure):
    """lkb_norm_prod_t"""
    _fields_ = [("w", C.c_void_p), ("h32", C.c_void_p), ("yq8", C.c_void_p), ("ssq", C.c_void_p)]


class MoeLayer(C.Structure):
    """lkb_moe_layer"""
    _fields_ = [("gate_qs", C.c_void_p), ("gate_d", C.c_void_p), ("up_qs", C.c_void_p), ("up_d", C.c_void_p),
                ("down_qs", C.c_void_p), ("down_d", C.c_void_p), ("router", C.c_void_p), ("rbias", C.c_void_p),
                ("norm_w", C.c_void_p), ("softmax", C.c_int)]


class MoeScratch(C.Structure):
    """lkb_moe_scratch"""
    _fields_ = [("logits", C.c_void_p), ("gu", C.c_void_p), ("sync", C.c_void_p)]


class MixerLayer(C.Structure):
    """lkb_mixer_layer"""
    _fields_ = [("is_attn", C.c_int), ("max_seq", C.c_int), ("attn_norm", C.c_void_p),
                ("in_qs", C.c_void_p), ("in_d", C.c_void_p), ("conv_w", C.c_void_p), ("hist", C.c_void_p),
                ("wq_qs", C.c_void_p), ("wq_d", C.c_void_p), ("wk_qs", C.c_void_p), ("wk_d", C.c_void_p),
                ("wv_qs", C.c_void_p), ("wv_d", C.c_void_p), ("qnorm", C.c_void_p), ("knorm", C.c_void_p),
                ("kc", C.c_void_p), ("vc", C.c_void_p), ("out_qs", C.c_void_p), ("out_d", C.c_void_p)]


class StepScratch(C.Structure):
    """lkb_step_scratch"""
    _fields_ = [("mx", C.c_void_p), ("part", C.c_void_p)]


class EpPeers(C.Structure):
    """lkb_ep_peers"""
    _fields_ = [("cmat", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("recv", C.c_void_p * 8), ("dback", C.c_void_p * 8)]


class PfGemm(C.Structure):
    """lkb_pf_gemm"""
    _fields_ = [("qs", C.c_void_p * 3), ("d", C.c_void_p * 3), ("seg_end", C.c_int * 3), ("N", C.c_int),
                ("bpr", C.c_int), ("exp_stride", C.c_longlong), ("aqs", C.c_void_p), ("asc", C.c_void_p),
                ("ntok", C.c_int), ("perm", C.c_void_p), ("tiles", C.c_void_p), ("ntiles", C.c_void_p),
                ("a_shift", C.c_int), ("scale", C.c_void_p), ("out", C.c_void_p), ("out_ld", C.c_int),
                ("add", C.c_int), ("oqs", C.c_void_p), ("osc", C.c_void_p), ("okb", C.c_int)]


_SCALARS = {"int": C.c_int, "float": C.c_float, "long": C.c_long, "long long": C.c_longlong,
            "size_t": C.c_size_t, "lkb_stream_t": C.c_void_p, "lkb_pf_act": PfAct, "unsigned": C.c_uint,
            "unsigned long long": C.c_ulonglong}


def declared_entry_points():
    """[(name, restype, [argtypes])] parsed from include/lkb.h."""
    text = re.sub(r"/\*.*?\*/", " ", HEADER.read_text(), flags=re.S)
    out = []
    for m in re.finditer(r"\b(int|const char \*)\s*(lkb_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), " ".join(m.group(3).split())
        argtypes = []
        if args not in ("", "void"):
            for a in args.split(","):
                a = a.strip()
                if "*" in a:
                    argtypes.append(C.c_void_p)
                    continue
                ty = " ".join(a.replace("const ", "").split()[:-1])
                argtypes.append(_SCALARS[ty])
        out.append((name, C.c_char_p if "char" in ret else C.c_int, argtypes))
    return out


def load_library():
    if not LIB_PATH.exists():
        raise LkbError(f"{LIB_PATH} is missing: build it with `python lfm2-ampere_b200/build.py` "
                       "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, restype, argtypes in declared_entry_points():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = load_library()
_inited = set()


def check(status: int, what: str = ""):
    if status != 0:
        msg = lib.lkb_error_string(status).decode()
        raise LkbError(f"{what or 'lkb call'} failed: {status} ({msg})")


def init(device: int = 0):
    """lkb_init for `device` (once per process and device).  Needs a B200."""
    if device not in _inited:
        check(lib.lkb_init(device), "lkb_init")
        _inited.add(device)


from .api import *          # noqa: E402,F401,F403
