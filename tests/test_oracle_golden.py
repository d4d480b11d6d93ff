"""Pins the CPU checker against the reference's own golden vectors (CPU only)."""
import numpy as np


def _f16(u16):
    return np.asarray(u16, np.uint16).view(np.float16).astype(np.float32)


def test_quant_fixture_known_answers(orc, golden_dir):
    """ref/quant_fixture.bin: four Q4_0 cases on real weight blocks.

    The stored expected_exact uses fp32 (unrounded) d8 and sum
    (tests/make_quant_fixture.py:27-40,73-81), so it pins the formula and the
    integer block sums; the reference's own gate is 5e-3 relative
    (tests/test_quant.cu:162).  Feeding the checker's integer sums into that
    fp32-scale formula must reproduce the stored value to float32 resolution.
    """
    g = np.load(golden_dir / "quant_q4_cases.npz")
    assert int(g["ncases"]) == 4
    for k in range(4):
        qs, d, x = g[f"c{k}_qs"], g[f"c{k}_d"], g[f"c{k}_x"]
        nblk = d.size
        q, d16, s16 = orc.quantize_q8_1(x)
        # quants: C roundf vs numpy round differ only on exact .5 ties
        ref_q = g[f"c{k}_ref_q"]
        diff = np.nonzero(q != ref_q)[0]
        for i in diff:
            dd = np.float32(np.max(np.abs(x[i // 32 * 32:i // 32 * 32 + 32]))) / np.float32(127.0)
            r = np.float32(x[i]) / dd
            assert abs(abs(float(r)) % 1.0 - 0.5) < 1e-6, "quant mismatch that is not a rounding tie"
        sumi = orc.block_sumi(qs, q, 1, nblk)[0] if nblk <= 64 else None
        if diff.size == 0:
            assert np.array_equal(sumi, g[f"c{k}_ref_sumi"]), "integer block sums differ from the reference recipe"
        # fp32-scale convention of the fixture, float64 combine
        d4 = _f16(d).astype(np.float64)
        d8 = g[f"c{k}_ref_d8"].astype(np.float64)
        rs = g[f"c{k}_ref_rawsum"].astype(np.float64)
        val = float(np.sum(d4 * (d8 * sumi.astype(np.float64) - 8.0 * rs)))
        exp = float(g[f"c{k}_expected_exact"])
        assert abs(val - exp) <= 2e-7 * max(1.0, abs(exp)), (k, val, exp)
        # engine convention (fp16-rounded d8 / sum) through the checker's GEMV:
        y = orc.gemv_q4_0(qs, d, (q, d16, s16), 1, nblk)[0]
        y64, mag = orc.gemv_q4_0_f64(qs, d, (q, d16, s16), 1, nblk)
        assert abs(y - y64[0]) <= 1e-5 * mag[0]
        assert abs(y - exp) <= 5e-3 * abs(exp)          # the reference's own gate
        assert abs(y - float(g[f"c{k}_expected_fp32"])) <= 5e-2 * abs(exp) + 5e-2
    # the single-block case: known integer sum
    q, _, _ = orc.quantize_q8_1(g["c3_x"])
    assert int(orc.block_sumi(g["c3_qs"], q, 1, 1)[0, 0]) == -1720


def test_router_on_real_gate_matrix(orc, golden_dir):
    """ref/kernel_fixture.bin router: ids exact, weights 1e-5 (tests/test_kernels.cu:212-219)."""
    g = np.load(golden_dir / "router_fixture.npz")
    logits = orc.router_dot(g["h"], g["gate"])
    l64 = g["gate"].astype(np.float64) @ g["h"].astype(np.float64)
    assert np.max(np.abs(logits - l64)) < 1e-5
    sel, sig = orc.router_gate(logits, g["bias"])
    idx, w = orc.router_select(sel, sig)
    assert idx.tolist() == g["expected_idx"].tolist() == [59, 45, 58, 40]
    assert np.max(np.abs(w.astype(np.float64) - g["expected_w"])) < 1e-5
    assert abs(float(w.sum()) - 1.0) < 1e-6
    assert orc.router_margin(sel) > 1e-3                 # not a near-tie


def test_against_reference_numpy_helpers(orc, golden_dir):
    """tools/ref_forward.py q8_1() and q4_mv_q8() executed from the reference."""
    g = np.load(golden_dir / "ref_numpy_vectors.npz")
    for tag, rows, K in (("a", 96, 2048), ("b", 64, 1536), ("c", 32, 256)):
        bpr = K // 32
        x = g[f"{tag}_x"]
        q, d16, s16 = orc.quantize_q8_1(x)
        assert np.array_equal(_f16(d16), g[f"{tag}_ref_d8"])
        # the raw sum is order-dependent in fp32: ours is the GPU's butterfly, numpy's is pairwise
        assert np.all(np.abs(_f16(s16) - g[f"{tag}_ref_sum"]) <= np.maximum(np.abs(g[f"{tag}_ref_sum"]) * 2.0 ** -10, 1e-6))
        mism = np.nonzero(q != g[f"{tag}_ref_q"].reshape(-1))[0]
        assert mism.size <= 2                              # only rounding ties may differ
        y = orc.gemv_q4_0(g[f"{tag}_qs"], g[f"{tag}_d"], (q, d16, s16), rows, bpr)
        y64, mag = orc.gemv_q4_0_f64(g[f"{tag}_qs"], g[f"{tag}_d"], (q, d16, s16), rows, bpr)
        assert np.all(np.abs(y - y64) <= 1e-5 * mag)
        # numpy's answer used its own sum rounding: allow the fp16 step of 8*sum per block
        slack = 8.0 * np.sum(np.abs(_f16(s16)) * 2.0 ** -10) * np.max(_f16(g[f"{tag}_d"]))
        assert np.all(np.abs(y - g[f"{tag}_ref_y"]) <= 1e-5 * mag + slack)


def test_zero_and_subnormal_blocks(orc):
    x = np.zeros(64, np.float32)
    x[32:] = np.linspace(-3e-4, 3e-4, 32, dtype=np.float32)
    q, d16, s16 = orc.quantize_q8_1(x)
    assert np.all(q[:32] == 0) and d16[0] == 0 and s16[0] == 0
    assert np.max(np.abs(q[32:])) == 127 and q.min() >= -127
    assert 0 < d16[1] < 0x0400                               # fp16 subnormal scale kept, not flushed


def test_q6k_fixture_known_answers(orc, golden_dir):
    """ref/quant_fixture.bin: the four Q6_K cases (token_embd / lm_head rows).

    Decode + per-sub-block scale order are pinned by feeding the fixture's own quants and fp32 d8
    through the checker's float64 GEMV: it must reproduce expected_exact to float32 resolution
    (tests/make_quant_fixture.py:60-70,90-102).  The shipped fp32 form with fp16 d8 must stay inside the
    reference's own Q6_K gate of 5e-2 relative (tests/test_quant.cu:162-163) and far tighter against
    float64 over the same fp16 scales.
    """
    g = np.load(golden_dir / "quant_q4_cases.npz")
    assert int(g["ncases_q6k"]) == 4
    for k in range(4):
        ql, qh, sc, d, x = (g[f"k{k}_{n}"] for n in ("ql", "qh", "sc", "d", "x"))
        sb = d.size
        y64, _ = orc.gemv_q6_K_f64(ql, qh, sc, d, g[f"k{k}_ref_q"], g[f"k{k}_ref_d8"], 1, sb)
        exp = float(g[f"k{k}_expected_exact"])
        assert abs(y64[0] - exp) <= 1e-6 * max(1.0, abs(exp)), (k, y64[0], exp)
        # dequantised row . x in float64 == the fixture's fp32-path value to fp32 accumulation error
        w = orc.dequant_q6_K(ql, qh, sc, d, sb)
        exp32 = float(g[f"k{k}_expected_fp32"])
        assert abs(float(w.astype(np.float64) @ x.astype(np.float64)) - exp32) <= 1e-3 * max(1.0, abs(exp32))
        if sb == 8:
            # shipped order on the checker's own fp16-scale quantisation
            act = orc.quantize_q8_1(x)
            y = orc.gemv_q6_K(ql, qh, sc, d, act, 1, sb)
            assert abs(float(y[0]) - exp) <= 5e-2 * max(1.0, abs(exp))
            y64b, mag = orc.gemv_q6_K_f64(ql, qh, sc, d, act[0], _f16(act[1]), 1, sb)
            assert abs(float(y[0]) - y64b[0]) <= 1e-5 * mag[0]


def test_q6k_group_sums_and_embed(orc):
    """Integer group sums against a plain numpy decode; embed row == dequant row."""
    rng = np.random.default_rng(61)
    rows, sb = 24, 8
    ql = rng.integers(0, 256, (rows, sb, 128), dtype=np.uint8)
    qh = rng.integers(0, 256, (rows, sb, 64), dtype=np.uint8)
    sc = rng.integers(-128, 128, (rows, sb, 16), dtype=np.int8)
    d = np.abs(rng.normal(0, 1e-3, (rows, sb))).astype(np.float16).view(np.uint16)
    aq = rng.integers(-127, 128, sb * 256, dtype=np.int8)
    # numpy decode of element e of a super-block (src/quant.cuh:171-190 layout)
    e = np.arange(256)
    n, r = (e >= 128) * 128, e % 128
    qlb = ql[:, :, (n >> 1) + (r & 63)].astype(np.int32)
    qhb = qh[:, :, (n >> 2) + (r & 31)].astype(np.int32)
    q6 = np.where(r >= 64, qlb >> 4, qlb & 15) | (((qhb >> (2 * (r >> 5))) & 3) << 4)
    w = q6 - 32
    gs = (w * aq.reshape(sb, 256)[None].astype(np.int32)).reshape(rows, sb, 32, 8).sum(-1)
    assert np.array_equal(orc.q6_group_sums(ql, qh, aq, rows, sb), gs)
    deq = (_f16(d).reshape(rows, sb, 1) * np.repeat(sc, 16, axis=2).astype(np.float32)) * w.astype(np.float32)
    for t in (0, 7, rows - 1):
        assert np.array_equal(orc.embed_q6_K(ql, qh, sc, d, t, sb), deq[t].reshape(-1))


def test_shortconv_on_real_taps(orc, golden_dir):
    """The reference's conv test (tests/test_kernels.cu:131-163) on its real taps: y within 1e-5 of float64,
    history shifted exactly."""
    cw = np.load(golden_dir / "conv_taps.npz")["conv_w"]
    n = cw.size // 3
    assert n == 2048
    rng = np.random.default_rng(11)
    bcx = rng.uniform(-1, 1, 3 * n).astype(np.float32)
    hist = (0.5 * rng.uniform(-1, 1, 2 * n)).astype(np.float32)
    y, h2 = orc.shortconv(bcx, cw, hist)
    B, Cg, X = (bcx[i * n:(i + 1) * n].astype(np.float64) for i in range(3))
    w = cw.astype(np.float64).reshape(n, 3)
    hh = hist.astype(np.float64).reshape(n, 2)
    ref = Cg * (hh[:, 0] * w[:, 0] + hh[:, 1] * w[:, 1] + (B * X) * w[:, 2])
    assert np.max(np.abs(y - ref)) <= 1e-5
    assert np.array_equal(h2.reshape(n, 2)[:, 0], hist.reshape(n, 2)[:, 1])
    assert np.array_equal(h2.reshape(n, 2)[:, 1], (bcx[:n] * bcx[2 * n:]).astype(np.float32))


def test_norm_rope_and_attention_references(orc):
    """float32 restatement vs float64 within the reference's gates: RoPE 2e-3 absolute at pos 12345
    (tests/test_kernels.cu:91-129); the float64 attention equals a direct numpy softmax."""
    rng = np.random.default_rng(12)
    x = rng.uniform(-1, 1, 4 * 64).astype(np.float32)
    one = np.ones(64, np.float32)
    a, inv = orc.norm_rope_heads(x, one, 12345.0, 1e7)
    assert np.max(np.abs(a - orc.norm_rope_heads_f64(x, one, 12345.0, 1e7))) <= 2e-3
    a0, _ = orc.norm_rope_heads(x, one, 0.0, 1e7)                      # position 0: rotation is the identity
    assert np.max(np.abs(a0 - orc.norm_rope_heads_f64(x, one, 0.0, 1e7))) <= 1e-6
    seq = 77
    q = rng.uniform(-1.5, 1.5, 2048).astype(np.float32)
    kc = rng.uniform(-1, 1, (seq, 8, 64)).astype(np.float16)
    vc = rng.uniform(-1, 1, (seq, 8, 64)).astype(np.float16)
    o = orc.attn_decode_f64(q, kc.view(np.uint16), vc.view(np.uint16), seq).reshape(32, 64)
    for h in (0, 13, 31):
        s = (kc[:, h // 4, :].astype(np.float64) @ q[h * 64:(h + 1) * 64].astype(np.float64)) * 0.125
        p = np.exp(s - s.max())
        assert np.max(np.abs(o[h] - (p @ vc[:, h // 4, :].astype(np.float64)) / p.sum())) <= 1e-14


def test_chunk_references(orc, golden_dir):
    """The float64 causal attention equals a direct numpy softmax; the chunk convolution is the decode step applied
    token by token (history carried)."""
    rng = np.random.default_rng(21)
    m, P = 9, 5
    S = m + P
    K = rng.standard_normal((S, 8, 64)).astype(np.float16)
    V = rng.standard_normal((S, 8, 64)).astype(np.float16)
    Q = (rng.standard_normal((m, 2048)) * 0.2).astype(np.float16)
    o = orc.pf_attn_f64(Q.view(np.uint16), m, P, K.view(np.uint16), V.view(np.uint16))
    for t, h in ((0, 0), (4, 13), (8, 31)):
        q = Q[t, h * 64:(h + 1) * 64].astype(np.float64)
        s = K[:P + t + 1, h // 4].astype(np.float64) @ q
        p = np.exp(s - s.max())
        assert np.max(np.abs(o[t, h * 64:(h + 1) * 64] - (p @ V[:P + t + 1, h // 4].astype(np.float64)) / p.sum())) < 1e-13
    cw = np.load(golden_dir / "conv_taps.npz")["conv_w"]
    Y = rng.uniform(-1, 1, (4, 6144)).astype(np.float32)
    hist = rng.uniform(-0.5, 0.5, 4096).astype(np.float32)
    v, h2 = orc.pf_conv(Y, cw, hist)
    bx = Y[:, :2048] * Y[:, 4096:]
    assert np.array_equal(h2.reshape(2048, 2)[:, 1], bx[3]) and np.array_equal(h2.reshape(2048, 2)[:, 0], bx[2])
    w = cw.astype(np.float64).reshape(2048, 3)
    ref3 = Y[3, 2048:4096].astype(np.float64) * (bx[1] * w[:, 0] + bx[2] * w[:, 1] + bx[3].astype(np.float64) * w[:, 2])
    assert np.max(np.abs(v[3] - ref3)) < 1e-5
