"""GPU parity of the output projection (Q6_K GEMV), the two-stage argmax and the Q6_K embedding row
against the CPU checker, through the C ABI.  Float results are compared bit for bit: the kernels and
the checker evaluate the same rounding sequence (integer group sums, one fp32 term per lane and
super-block, xor butterfly)."""
import numpy as np
import pytest

from helpers import act_floats, dev, host, nan_f32

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L(lkb):
    lkb.init(0)
    return lkb


def rand_q6(rng, rows, sb):
    ql = rng.integers(0, 256, (rows, sb, 128), dtype=np.uint8)
    qh = rng.integers(0, 256, (rows, sb, 64), dtype=np.uint8)
    sc = rng.integers(-128, 128, (rows, sb, 16), dtype=np.int8)
    d = np.abs(rng.normal(0, 2e-4, (rows, sb))).astype(np.float16).view(np.uint16)
    return ql, qh, sc, d


@pytest.mark.parametrize("rows,sb", [(65536, 8), (16, 8), (1, 8), (33, 8), (2381, 8), (148 * 32 + 5, 8), (20000, 8), (148 * 32 * 4 - 1, 8), (300, 3), (64, 1)])
def test_gemv_q6_K_bit_exact(L, orc, rows, sb):
    rng = np.random.default_rng(rows * 10 + sb)
    ql, qh, sc, d = rand_q6(rng, rows, sb)
    act = orc.quantize_q8_1(act_floats(rng, sb * 256))
    xq = dev(orc.pack_blocks(*act))
    planes = [dev(a) for a in (ql, qh, sc, d)]
    y = nan_f32(rows)
    L.k_gemv_q6_K(*planes, xq, rows, sb, y, None, 0.0)
    assert L.gemv_q6_K_status() == 0
    y_ref = orc.gemv_q6_K(ql, qh, sc, d, act, rows, sb)
    assert np.array_equal(host(y), y_ref)
    n64 = min(rows, 512)
    y64, mag = orc.gemv_q6_K_f64(ql[:n64], qh[:n64], sc[:n64], d[:n64], act[0],
                                 np.asarray(act[1]).view(np.float16).astype(np.float32), n64, sb)
    assert np.all(np.abs(host(y)[:n64] - y64) <= 1e-5 * mag)        # the 1e-5 contract against float64
    # consumer-side 1/rms (rsqrtf on the device: 2 ulp on inv)
    ssq = (rng.random(64).astype(np.float32) + 0.5) * 32.0
    y2 = nan_f32(rows)
    L.k_gemv_q6_K(*planes, xq, rows, sb, y2, dev(ssq), 1e-5)
    ref2 = y_ref * np.float32(orc.norm_inv(ssq))
    assert np.all(np.abs(host(y2) - ref2) <= 4e-7 * np.abs(ref2) + 1e-30)


def test_gemv_q6_K_golden_rows(L, orc, golden_dir):
    """The reference fixture's real lm_head / token_embd rows (8 super-blocks) through the device path."""
    g = np.load(golden_dir / "quant_q4_cases.npz")
    for k in range(int(g["ncases_q6k"])):
        ql, qh, sc, d, x = (g[f"k{k}_{n}"] for n in ("ql", "qh", "sc", "d", "x"))
        sb = d.size
        act = orc.quantize_q8_1(x)
        y = nan_f32(1)
        L.k_gemv_q6_K(dev(ql), dev(qh), dev(sc), dev(d), dev(orc.pack_blocks(*act)), 1, sb, y, None, 0.0)
        assert np.array_equal(host(y), orc.gemv_q6_K(ql, qh, sc, d, act, 1, sb))
        exp = float(g[f"k{k}_expected_exact"])
        assert abs(float(host(y)[0]) - exp) <= 5e-2 * max(1.0, abs(exp))    # tests/test_quant.cu:162-163 gate


def test_gemv_q6_K_unaligned_planes_take_the_plain_kernel(L, orc):
    rng = np.random.default_rng(5)
    rows, sb = 100, 8
    ql, qh, sc, d = rand_q6(rng, rows, sb)
    act = orc.quantize_q8_1(act_floats(rng, sb * 256))
    buf = torch.zeros(ql.size + 64, dtype=torch.uint8, device="cuda")
    off = buf[4:4 + ql.size]
    off.copy_(dev(ql).reshape(-1))
    y = nan_f32(rows)
    L.k_gemv_q6_K(off, dev(qh), dev(sc), dev(d), dev(orc.pack_blocks(*act)), rows, sb, y, None, 0.0)
    assert np.array_equal(host(y), orc.gemv_q6_K(ql, qh, sc, d, act, rows, sb))


@pytest.mark.parametrize("n", [65536, 1024, 1000, 5, 262144 + 3])
def test_argmax_first_maximum(L, n):
    rng = np.random.default_rng(n)
    v = rng.standard_normal(n).astype(np.float32)
    hi = float(v.max()) + 1.0
    for pos in ([n - 1, n // 2], [0], [n // 3, n // 3 + 1]):
        w = v.copy()
        w[pos] = hi                                   # equal maxima: the lowest index wins
        nb = (n + 1023) // 1024
        pv, pi = nan_f32(nb), torch.full((nb,), -1, dtype=torch.int32, device="cuda")
        tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        cnt = torch.full((1,), 41, dtype=torch.int32, device="cuda")
        L.k_argmax_part(dev(w), n, pv, pi)
        L.k_argmax_final(pv, pi, nb, tok, cnt)
        assert int(tok.item()) == min(pos) == int(np.argmax(w))
        assert int(cnt.item()) == 42
        # stage-1 partials: per-1024 first maxima
        for b in (0, nb - 1):
            seg = w[b * 1024:(b + 1) * 1024]
            assert int(pi[b].item()) == b * 1024 + int(np.argmax(seg)) and float(pv[b].item()) == float(seg.max())
    # signed zeros tie; NaN and values <= -1e30 never win
    z = np.full(2048, -1.0, np.float32)
    z[100], z[50], z[7] = 0.0, -0.0, np.nan
    pv, pi = nan_f32(2), torch.zeros(2, dtype=torch.int32, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.k_argmax_part(dev(z), 2048, pv, pi)
    L.k_argmax_final(pv, pi, 2, tok, None)
    assert int(tok.item()) == 50
    L.k_argmax_part(dev(np.full(2048, -3e30, np.float32)), 2048, pv, pi)
    L.k_argmax_final(pv, pi, 2, tok, None)
    assert int(tok.item()) == 0 and host(pi).tolist() == [0, 1024]


def test_embed_q6_K_row(L, orc):
    rng = np.random.default_rng(77)
    rows, sb = 512, 8
    ql, qh, sc, d = rand_q6(rng, rows, sb)
    planes = [dev(a) for a in (ql, qh, sc, d)]
    for t in (0, 31, rows - 1):
        x = nan_f32(sb * 256)
        L.k_embed_q6_K(*planes, dev(np.array([t], np.int32)), sb * 256, x)
        assert np.array_equal(host(x), orc.embed_q6_K(ql, qh, sc, d, t, sb))


def test_lm_head_then_argmax_matches_checker_token(L, orc):
    """The decode tail as the engine runs it: norm producer -> Q6_K GEMV (1/rms folded in) -> argmax."""
    rng = np.random.default_rng(2048)
    rows, sb = 65536, 8
    ql, qh, sc, d = rand_q6(rng, rows, sb)
    act = orc.quantize_q8_1(act_floats(rng, 2048))
    y = nan_f32(rows)
    L.k_gemv_q6_K(*[dev(a) for a in (ql, qh, sc, d)], dev(orc.pack_blocks(*act)), rows, sb, y, None, 0.0)
    pv, pi = nan_f32(64), torch.zeros(64, dtype=torch.int32, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.k_argmax_part(y, rows, pv, pi)
    L.k_argmax_final(pv, pi, 64, tok, None)
    assert int(tok.item()) == int(np.argmax(orc.gemv_q6_K(ql, qh, sc, d, act, rows, sb)))
