"""GPU parity of the decode-step sequence mixers (short convolution, qk-norm + RoPE + KV append,
split-K attention) against the CPU checker, through the C ABI.

The convolution is compared bit for bit.  RoPE and attention are roundings of a float64 definition (as in
the reference, whose own gates are 2e-3 and 1e-3 absolute: tests/test_kernels.cu:129, tests/test_attn.cu:170);
the tolerances below are far tighter and stated per case."""
import numpy as np
import pytest

from helpers import dev, empty_blocks, host, nan_f32

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

SPLIT, PARTW = 18, 66


@pytest.fixture(scope="module")
def L(lkb):
    lkb.init(0)
    assert (lkb.ATTN_SPLIT, lkb.ATTN_PARTW) == (SPLIT, PARTW)
    return lkb


def _blocks(orc, t):
    return orc.unpack_blocks(host(t, orc.BLOCK_Q8_1))


def test_shortconv_bit_exact_and_state(L, orc, golden_dir):
    cw = np.load(golden_dir / "conv_taps.npz")["conv_w"]
    n = 2048
    rng = np.random.default_rng(3)
    hist = (0.5 * rng.uniform(-1, 1, 2 * n)).astype(np.float32)
    d_hist, d_cw = dev(hist), dev(cw)
    for step in range(3):                                   # three steps: the history really shifts
        bcx = rng.uniform(-1, 1, 3 * n).astype(np.float32)
        y, yq8 = nan_f32(n), empty_blocks(n // 32)
        L.k_shortconv(dev(bcx), d_cw, d_hist, y, yq8, n)
        y_ref, hist = orc.shortconv(bcx, cw, hist)
        assert np.array_equal(host(y), y_ref)
        assert np.array_equal(host(d_hist), hist)
        q, d16, s16 = _blocks(orc, yq8)
        rq, rd, rs = orc.quantize_q8_1(y_ref)
        assert np.array_equal(q, rq) and np.array_equal(d16, rd) and np.array_equal(s16, rs)
    # outputs are optional one at a time
    L.k_shortconv(dev(bcx), d_cw, d_hist, None, yq8, n)
    L.k_shortconv(dev(bcx), d_cw, d_hist, y, None, n)
    with pytest.raises(L.LkbError):
        L.k_shortconv(dev(bcx), d_cw, d_hist, y, None, 2040)


@pytest.mark.parametrize("pos,theta", [(0, 1e7), (1, 1e7), (4095, 1e7), (12345, 1e7), (131071, 1e7), (4095, 1e6)])
def test_qk_norm_rope_and_cache_append(L, orc, pos, theta):
    rng = np.random.default_rng(pos + 1)
    q = rng.standard_normal(32 * 64).astype(np.float32)
    k = rng.standard_normal(8 * 64).astype(np.float32)
    v = rng.standard_normal(8 * 64).astype(np.float32)
    qn = (1 + 0.05 * rng.standard_normal(64)).astype(np.float32)
    kn = (1 + 0.05 * rng.standard_normal(64)).astype(np.float32)
    rows = pos + 2
    kc = torch.full((rows, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    vc = torch.full((rows, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    dq, dk = dev(q), dev(k)
    L.k_qk_norm_rope(dq, dk, dev(v), dev(qn), dev(kn), dev(np.array([pos], np.int32)), kc, vc, theta)
    gq, gk = host(dq), host(dk)
    # float64 definition: the angle pos * theta^(-2i/64) is formed in fp32 by the kernel (and by the reference),
    # so the error grows with the position: a few fp32 ulp of the angle times |x| (up to ~4 after the norm),
    # plus 4e-6 of arithmetic.  The reference gates |x| <= 1 at position 12345 with 2e-3.
    tol = 4e-6 + 6e-7 * pos
    assert np.max(np.abs(gq - orc.norm_rope_heads_f64(q, qn, pos, theta))) <= tol
    assert np.max(np.abs(gk - orc.norm_rope_heads_f64(k, kn, pos, theta))) <= tol
    # float32 restatement in the kernel's order: agrees to a few ulp of the angle as well
    fq, _ = orc.norm_rope_heads(q, qn, float(pos), theta)
    assert np.max(np.abs(gq - fq)) <= tol
    # cache row pos = fp16 of what was written back; other rows untouched
    hk, hv = host(kc).view(np.uint16), host(vc).view(np.uint16)
    assert np.array_equal(hk[pos].reshape(-1), orc.f32_to_f16_bits(gk))
    assert np.array_equal(hv[pos].reshape(-1), orc.f32_to_f16_bits(v))
    seven = np.float16(7.0).view(np.uint16)
    assert np.all(hk[pos + 1] == seven) and np.all(hv[pos + 1] == seven) and (pos == 0 or np.all(hk[pos - 1] == seven))


@pytest.mark.parametrize("seq", [1, 5, 31, 32, 33, 100, 255, 256, 257, 512, 513, 4096, 4608, 4609, 8192, 16384, 100003, 131072])
def test_attention_split_combine_vs_float64(L, orc, seq):
    """The reference's cases (tests/test_attn.cu:190-222) plus the group / slice boundaries of this kernel."""
    rng = np.random.default_rng(seq)
    q = (rng.uniform(-1, 1, 32 * 64) * 1.5).astype(np.float32)
    kc = torch.empty(seq + 3, 8, 64, dtype=torch.float16, device="cuda").uniform_(-1, 1)
    vc = torch.empty(seq + 3, 8, 64, dtype=torch.float16, device="cuda").uniform_(-1, 1)
    kc[seq:] = float("nan")                                # rows past the position must never be read into a result
    vc[seq:] = float("nan")
    part = nan_f32(32 * SPLIT * PARTW)
    out, yq8 = nan_f32(32 * 64), empty_blocks(64)
    d_pos = dev(np.array([seq - 1], np.int32))
    L.k_attn_split(dev(q), kc, vc, d_pos, part)
    L.k_attn_combine(part, d_pos, out, yq8)
    ref = orc.attn_decode_f64(q, host(kc[:seq]).view(np.uint16), host(vc[:seq]).view(np.uint16), seq)
    got = host(out)
    assert np.all(np.isfinite(got))
    err = float(np.max(np.abs(got - ref)))
    assert err <= 2e-6, err                                # reference gate: 1e-3 (its kernel measures ~1e-8..1e-7)
    bq, bd, bs = _blocks(orc, yq8)
    rq, rd, rs = orc.quantize_q8_1(got)
    assert np.array_equal(bq, rq) and np.array_equal(bd, rd) and np.array_equal(bs, rs)
    # out is optional
    L.k_attn_combine(part, d_pos, None, yq8)


def test_attention_peaked_scores_and_graph_replay(L, orc):
    """One dominant key per head (softmax ~ one-hot) and large score ranges; then the same launches replayed
    from a CUDA graph at a new position read the new *d_pos."""
    rng = np.random.default_rng(99)
    seq = 3000
    q = (rng.standard_normal(32 * 64) * 4).astype(np.float32)
    k = rng.standard_normal((seq, 8, 64)).astype(np.float16)
    v = rng.standard_normal((seq, 8, 64)).astype(np.float16)
    k[1234] *= 4
    kc, vc = dev(k.view(np.int16)).view(torch.float16), dev(v.view(np.int16)).view(torch.float16)
    part, out = nan_f32(32 * SPLIT * PARTW), nan_f32(32 * 64)
    d_pos = dev(np.array([seq - 1], np.int32))
    dq = dev(q)
    L.k_attn_split(dq, kc, vc, d_pos, part)
    L.k_attn_combine(part, d_pos, out, None)
    ref = orc.attn_decode_f64(q, k.view(np.uint16), v.view(np.uint16), seq)
    assert np.max(np.abs(host(out) - ref)) <= 1e-5
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        L.k_attn_split(dq, kc, vc, d_pos, part)
        L.k_attn_combine(part, d_pos, out, None)
    for s2 in (700, 2999, 17):
        d_pos.fill_(s2 - 1)
        g.replay()
        torch.cuda.synchronize()
        ref = orc.attn_decode_f64(q, k.view(np.uint16), v.view(np.uint16), s2)
        assert np.max(np.abs(host(out) - ref)) <= 1e-5
