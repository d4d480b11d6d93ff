#!/usr/bin/env python3
"""Regenerate the golden fixtures under tests/golden/ from the reference checkout.

Run once, in a container that has the reference repository mounted:

    python tests/golden/make_golden.py /path/to/reference

It writes four small .npz files.  Nothing at test time reads the reference
checkout; the tests read only these files.

  quant_q4_cases.npz   The four Q4_0 known-answer cases of the reference's
                       ref/quant_fixture.bin (real weight blocks of
                       blk.2.attn_q.weight, x ~ N(0,1), format written by
                       tests/make_quant_fixture.py:105-116), with the stored
                       expected values, plus the per-block integer sums and
                       quants obtained by EXECUTING the reference's own
                       q8_1_quantize (tests/make_quant_fixture.py:27-40).
  router_fixture.npz   The reference's real router matrix blk.2.ffn_gate_inp
                       (64 x 2048 fp32) and selection bias blk.2.exp_probs_b
                       from ref/kernel_fixture.bin (tests/make_kernel_fixture.py:39-47),
                       the input vector of the reference's router test
                       (xorshift64 stream of tests/test_kernels.cu:19-24,170-171) and
                       the expected top-4 / weights from that test's float64
                       recipe (tests/test_kernels.cu:172-182).
  conv_taps.npz        The reference's real ShortConv tap weights (2048 x 3 fp32) from the same
                       kernel_fixture.bin.
  ref_numpy_vectors.npz  Seeded synthetic Q4_0 matrices and activations pushed
                       through the reference's numpy helpers q8_1() and
                       q4_mv_q8() (tools/ref_forward.py:60-100), whose source is
                       executed from the checkout (function bodies only; the
                       module's import-time pack loading is skipped).
"""
import ast
import pathlib
import struct
import sys

import numpy as np

OUT = pathlib.Path(__file__).resolve().parent


def _functions(path, names, ns):
    """Compile the named top-level functions of a reference .py file into ns."""
    tree = ast.parse(pathlib.Path(path).read_text())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in body} == set(names), (path, names)
    exec(compile(ast.Module(body=body, type_ignores=[]), str(path), "exec"), ns)
    return ns


def quant_cases(ref):
    raw = (ref / "ref" / "quant_fixture.bin").read_bytes()
    assert raw[:4] == b"LKQF"
    (ncase,) = struct.unpack_from("<I", raw, 4)
    pos = 8
    ns = _functions(ref / "tests" / "make_quant_fixture.py", ["q8_1_quantize"], {"np": np})
    out = {}
    k = 0
    k6 = 0
    for _ in range(ncase):
        kind, nblk, nplanes, _pad = struct.unpack_from("<IIIf", raw, pos)
        pos += 16
        planes = []
        for _p in range(nplanes):
            (sz,) = struct.unpack_from("<I", raw, pos)
            pos += 4
            planes.append(raw[pos:pos + sz])
            pos += sz
        (nx,) = struct.unpack_from("<I", raw, pos)
        pos += 4
        x = np.frombuffer(raw, np.float32, nx, pos).copy()
        pos += 4 * nx
        exact, fp32 = struct.unpack_from("<ff", raw, pos)
        pos += 8
        if kind != 0:            # Q6_K cases (token_embd / lm_head rows): stored under their own keys
            qi, d8, rawsum = ns["q8_1_quantize"](x, nblk * 8)
            out[f"k{k6}_ql"] = np.frombuffer(planes[0], np.uint8).copy()
            out[f"k{k6}_qh"] = np.frombuffer(planes[1], np.uint8).copy()
            out[f"k{k6}_sc"] = np.frombuffer(planes[2], np.int8).copy()
            out[f"k{k6}_d"] = np.frombuffer(planes[3], np.uint16).copy()
            out[f"k{k6}_x"] = x
            out[f"k{k6}_expected_exact"] = np.float32(exact)
            out[f"k{k6}_expected_fp32"] = np.float32(fp32)
            out[f"k{k6}_ref_q"] = qi.astype(np.int8)
            out[f"k{k6}_ref_d8"] = d8.astype(np.float32)
            k6 += 1
            continue
        qs = np.frombuffer(planes[0], np.uint8).reshape(nblk, 16).copy()
        d = np.frombuffer(planes[1], np.uint16).copy()
        qi, d8, rawsum = ns["q8_1_quantize"](x, nblk)
        nib = np.concatenate([(qs & 0x0F), (qs >> 4)], axis=1).astype(np.int32)
        sumi = (nib * qi.reshape(nblk, 32).astype(np.int32)).sum(axis=1).astype(np.int32)
        out[f"c{k}_qs"] = qs
        out[f"c{k}_d"] = d
        out[f"c{k}_x"] = x
        out[f"c{k}_expected_exact"] = np.float32(exact)
        out[f"c{k}_expected_fp32"] = np.float32(fp32)
        out[f"c{k}_ref_q"] = qi.astype(np.int8)
        out[f"c{k}_ref_d8"] = d8.astype(np.float32)
        out[f"c{k}_ref_rawsum"] = rawsum.astype(np.float32)
        out[f"c{k}_ref_sumi"] = sumi
        k += 1
    out["ncases"] = np.int32(k)
    out["ncases_q6k"] = np.int32(k6)
    np.savez_compressed(OUT / "quant_q4_cases.npz", **out)
    print("quant_q4_cases.npz:", k, "cases")


def router_fixture(ref):
    raw = (ref / "ref" / "kernel_fixture.bin").read_bytes()
    assert raw[:4] == b"LKKF"
    pos = 4
    arrs = []
    for _ in range(3):
        (n,) = struct.unpack_from("<I", raw, pos)
        pos += 4
        arrs.append(np.frombuffer(raw, np.float32, n, pos).copy())
        pos += 4 * n
    _conv_w, gate, bias = arrs
    gate = gate.reshape(64, 2048)

    # xorshift64 stream of the reference's kernel test; the router input is drawn
    # after 2*2048 (RMSNorm) + 256 (RoPE) + 5*2048 (ShortConv) earlier draws.
    seed = 88172645463325252
    M = (1 << 64) - 1

    def nrand():
        nonlocal seed
        seed ^= (seed << 13) & M
        seed ^= seed >> 7
        seed ^= (seed << 17) & M
        u = ((seed >> 11) & ((1 << 53) - 1)) / float(1 << 53)
        return u * 2.0 - 1.0

    for _ in range(2 * 2048 + 256 + 5 * 2048):
        nrand()
    h = np.array([np.float32(nrand()) for _ in range(2048)], np.float32)

    lg = gate.astype(np.float64) @ h.astype(np.float64)
    pr = 1.0 / (1.0 + np.exp(-lg))
    sel = pr + bias.astype(np.float64)
    order = np.argsort(-sel, kind="stable")
    ws = max(pr[order[:4]].sum(), 6.103515625e-5)
    # the reference's real ShortConv taps (2048 channels x 3), used by its conv test (tests/test_kernels.cu:131-163)
    np.savez_compressed(OUT / "conv_taps.npz", conv_w=_conv_w.astype(np.float32))
    np.savez_compressed(OUT / "router_fixture.npz", gate=gate, bias=bias, h=h,
                        expected_idx=order[:4].astype(np.int32),
                        expected_w=(pr[order[:4]] / ws).astype(np.float64),
                        expected_sel_sorted=sel[order[:6]].astype(np.float64))
    print("router_fixture.npz: idx", order[:4], "sel", sel[order[:5]])


def numpy_vectors(ref):
    rng = np.random.default_rng(20261125)
    store = {}
    planes = {}
    ent = {}
    ns = {"np": np, "_ent": ent, "plane": lambda name, p: planes[(name, p)]}
    _functions(ref / "tools" / "ref_forward.py", ["q8_1", "q4_mv_q8"], ns)
    for tag, rows, K in (("a", 96, 2048), ("b", 64, 1536), ("c", 32, 256)):
        bpr = K // 32
        qs = rng.integers(0, 256, size=(rows, bpr, 16), dtype=np.uint8)
        d = np.abs(rng.normal(0.0, 0.02, size=(rows, bpr))).astype(np.float16)
        x = rng.standard_normal(K).astype(np.float32)
        if tag == "c":
            x[:32] = 0.0                                 # an all-zero block
            x[32:64] *= 1e-6                             # a block whose d is fp16-subnormal
        ent[tag] = {"blocks_per_row": bpr, "rows": rows}
        planes[(tag, "qs")] = qs.tobytes()
        planes[(tag, "d")] = d.view(np.uint16).tobytes()
        q, d16, s16 = ns["q8_1"](x)
        y = ns["q4_mv_q8"](tag, x)
        store[f"{tag}_qs"] = qs
        store[f"{tag}_d"] = d.view(np.uint16)
        store[f"{tag}_x"] = x
        store[f"{tag}_ref_q"] = q.astype(np.int8)
        store[f"{tag}_ref_d8"] = d16.astype(np.float32)
        store[f"{tag}_ref_sum"] = s16.astype(np.float32)
        store[f"{tag}_ref_y"] = y.astype(np.float32)
    np.savez_compressed(OUT / "ref_numpy_vectors.npz", **store)
    print("ref_numpy_vectors.npz written")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    ref = pathlib.Path(sys.argv[1])
    quant_cases(ref)
    router_fixture(ref)
    numpy_vectors(ref)
