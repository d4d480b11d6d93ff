"""The C-ABI library loads and exports every entry point include/lkb.h declares (no GPU needed)."""
import ctypes
import re

import numpy as np


def test_every_declared_symbol_is_exported(lkb):
    names = [n for n, _, _ in lkb.declared_entry_points()]
    assert len(names) >= 35 and len(set(names)) == len(names)
    raw = ctypes.CDLL(str(lkb.LIB_PATH))
    for n in names:
        assert hasattr(raw, n), f"liblkb.so lacks {n}"
    # every declaration carries a citation of the reference interface it replaces (or says it has none)
    text = lkb.HEADER.read_text()
    for n in names:
        if n in ("lkb_error_string", "lkb_sm_count", "lkb_set_pdl"):
            continue
        pos = re.search(r"\bint\s+%s\(" % n, text).start()
        assert re.search(r"ref: src/\w+\.cuh?:\d+|[Nn]o\s+counterpart|Not part of the reference",
                         text[max(0, pos - 1500):pos]), n


def test_struct_layouts_match_header(lkb, tmp_path):
    """ctypes mirrors vs the C compiler's layout of include/lkb.h."""
    import subprocess
    src = tmp_path / "layout.c"
    src.write_text('''#include <stdio.h>
#include <stddef.h>
#include "lkb.h"
int main(void) {
    printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(lkb_pf_act), sizeof(lkb_norm_prod_t), sizeof(lkb_pf_gemm),
           offsetof(lkb_pf_gemm, exp_stride), offsetof(lkb_pf_gemm, aqs), offsetof(lkb_pf_gemm, a_shift),
           offsetof(lkb_pf_gemm, okb), sizeof(lkb_block_q8_1));
    printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(lkb_moe_layer), offsetof(lkb_moe_layer, softmax), sizeof(lkb_moe_scratch),
           sizeof(lkb_mixer_layer), offsetof(lkb_mixer_layer, attn_norm), offsetof(lkb_mixer_layer, kc),
           offsetof(lkb_mixer_layer, out_d), sizeof(lkb_step_scratch));
    return 0;
}''')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(lkb.ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    G = lkb.PfGemm
    X = lkb.MixerLayer
    assert got == [ctypes.sizeof(lkb.PfAct), ctypes.sizeof(lkb.NormProd), ctypes.sizeof(G), G.exp_stride.offset,
                   G.aqs.offset, G.a_shift.offset, G.okb.offset, 36,
                   ctypes.sizeof(lkb.MoeLayer), lkb.MoeLayer.softmax.offset, ctypes.sizeof(lkb.MoeScratch),
                   ctypes.sizeof(X), X.attn_norm.offset, X.kc.offset, X.out_d.offset, ctypes.sizeof(lkb.StepScratch)]


def test_compute_calls_fail_loudly_without_init(lkb):
    """No CPU fallback: before lkb_init (or without a GPU) every compute entry point refuses."""
    import torch
    if torch.cuda.is_available():
        return                      # on a GPU box another test may already have initialised the library
    assert lkb.lib.lkb_init(0) != 0
    buf = np.zeros(64, np.float32)
    p = buf.ctypes.data
    assert lkb.lib.lkb_quantize_q8_1(p, p, 1, None) == -10004
    assert lkb.lib.lkb_router_dot(p, p, p, None, None, None, None, 0.0, None) == -10004
    assert lkb.lib.lkb_pf_moe_plan(p, p, p, p, None) == -10004
    assert b"lkb_init" in lkb.lib.lkb_error_string(-10004)


def test_cpp_shim_compiles_and_links(lkb, tmp_path):
    """An engine-style C++ caller written against include/lkb_shim.hpp (the reference's kernel names)
    compiles and links against liblkb.so (no device needed for that)."""
    import subprocess
    src = tmp_path / "caller.cpp"
    src.write_text('''#include "lkb_shim.hpp"
int moe_layer(lk::stream_t st, const float * h, const float * router, const float * rbias, float * logits, int * idx, float * w,
              const void * gq, const void * gd, const void * uq, const void * ud, const void * dq, const void * dd,
              lk::block_q8_1 * xq, lk::block_q8_1 * xq2, float * gu, float * x, const float * ssq, lk::LKNormProd np) {
    lk::k_router_dot(st, h, router, logits, rbias, nullptr, nullptr, ssq, LKB_EPS);
    lk::k_router_top4(st, logits, rbias, idx, w);
    lk::k_gemv_q4_0_exp2(st, gq, gd, uq, ud, xq, 1536, 64, 1536, 0, idx, nullptr, nullptr, nullptr, nullptr, gu, gu + 6144, ssq, LKB_EPS);
    lk::k_swiglu(st, gu, gu + 6144, 6144, nullptr, xq2, dq, idx, 2048, 48, 2 << 20);
    return lk::k_moe_down_accum(st, dq, dd, xq2, 2048, 48, 2048, 48, idx, w, x, np);
}
int main() { return lkb_sm_count() < 0; }
''')
    exe = tmp_path / "caller"
    subprocess.run(["g++", "-std=c++17", "-I", str(lkb.ROOT / "include"), str(src), "-o", str(exe),
                    str(lkb.LIB_PATH), f"-Wl,-rpath,{lkb.LIB_PATH.parent}"], check=True)
    assert subprocess.run([str(exe)]).returncode == 0
