"""GPU parity of the batched-prefill sequence mixers through the C ABI.

Per-token kernels (embedding rows, chunk convolution, qk-norm + RoPE + KV append) must equal their decode twins
token by token, bit for bit.  The causal flash attention is compared with the float64 softmax over the same fp16
inputs (the reference's definition and gate: tests/test_prefill.cu:244-289, 4e-3 absolute), and with the decode
attention kernel of this library position by position."""
import numpy as np
import pytest

from helpers import dev, empty_blocks, host, nan_f32

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
H = 2048


@pytest.fixture(scope="module")
def L(lkb):
    lkb.init(0)
    return lkb


def test_pf_embed_rows(L, orc):
    rng = np.random.default_rng(1)
    rows, sb = 300, 8
    ql = rng.integers(0, 256, (rows, sb, 128), dtype=np.uint8)
    qh = rng.integers(0, 256, (rows, sb, 64), dtype=np.uint8)
    sc = rng.integers(-128, 128, (rows, sb, 16), dtype=np.int8)
    d = np.abs(rng.normal(0, 2e-4, (rows, sb))).astype(np.float16).view(np.uint16)
    toks = np.array([0, 299, 17, 17, 250], np.int32)
    x = nan_f32(len(toks), H)
    L.k_pf_embed(dev(ql), dev(qh), dev(sc), dev(d), dev(toks), x, H, len(toks))
    for i, t in enumerate(toks):
        assert np.array_equal(host(x)[i], orc.embed_q6_K(ql, qh, sc, d, int(t), sb))


@pytest.mark.parametrize("m", [1, 2, 3, 37])
def test_pf_conv_equals_decode_steps(L, orc, golden_dir, m):
    cw = np.load(golden_dir / "conv_taps.npz")["conv_w"]
    rng = np.random.default_rng(m)
    Y = rng.uniform(-1, 1, (m, 3 * H)).astype(np.float32)
    hist = (0.5 * rng.uniform(-1, 1, 2 * H)).astype(np.float32)
    a_qs = torch.full((m, H), 0x55, dtype=torch.int8, device="cuda")
    a_sc = nan_f32(m, H // 32, 2)
    d_hist = dev(hist)
    L.k_pf_conv(dev(Y), dev(cw), d_hist, L.pf_act(a_qs, a_sc), m)
    L.k_pf_conv_hist(dev(Y), m, d_hist)
    v_ref, h_ref = orc.pf_conv(Y, cw, hist)
    assert np.array_equal(host(d_hist), h_ref)
    for t in range(m):
        q, d16, s16 = orc.quantize_q8_1(v_ref[t])
        assert np.array_equal(host(a_qs)[t], q)
        sc = host(a_sc)[t]
        assert np.array_equal(sc[:, 0], np.asarray(d16).view(np.float16).astype(np.float32))
        assert np.array_equal(sc[:, 1], np.float32(8.0) * np.asarray(s16).view(np.float16).astype(np.float32))
    # and against the decode kernel itself, token by token
    d_hist2 = dev(hist)
    for t in range(m):
        yq8 = empty_blocks(H // 32)
        L.k_shortconv(dev(Y[t]), dev(cw), d_hist2, None, yq8, H)
        q, _, _ = orc.unpack_blocks(host(yq8, orc.BLOCK_Q8_1))
        assert np.array_equal(q, host(a_qs)[t])
    assert np.array_equal(host(d_hist2), host(d_hist))


@pytest.mark.parametrize("m,P", [(1, 0), (5, 0), (33, 100), (8, 4000)])
def test_pf_qknr_equals_decode_kernel(L, orc, m, P):
    rng = np.random.default_rng(m * 7 + P)
    Y = rng.standard_normal((m, 3072)).astype(np.float32)
    qn = (1 + 0.05 * rng.standard_normal(64)).astype(np.float32)
    kn = (1 + 0.05 * rng.standard_normal(64)).astype(np.float32)
    S = P + m + 1
    kc = torch.full((S, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    vc = torch.full((S, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    qh = torch.full((m, H), 9.0, dtype=torch.float16, device="cuda")
    L.k_pf_qknr(dev(Y), dev(qn), dev(kn), P, qh, kc, vc, m, 1e6)
    kc2 = torch.full((S, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    vc2 = torch.full((S, 8, 64), 7.0, dtype=torch.float16, device="cuda")
    for t in range(m):
        q, k, v = dev(Y[t, :2048].copy()), dev(Y[t, 2048:2560].copy()), dev(Y[t, 2560:].copy())
        L.k_qk_norm_rope(q, k, v, dev(qn), dev(kn), dev(np.array([P + t], np.int32)), kc2, vc2, 1e6)
        want = (host(q) * np.float32(0.125)).astype(np.float16)
        assert np.array_equal(host(qh)[t].view(np.uint16), want.view(np.uint16))
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    assert float(kc[P + m].float().min().item()) == 7.0 and (P == 0 or float(kc[P - 1].float().min().item()) == 7.0)


@pytest.mark.parametrize("m,P", [(64, 0), (100, 150), (37, 1000), (1, 0), (33, 31), (512, 0), (256, 3840),
                                 (64, 32704), (32, 131040)])
def test_pf_attn_vs_float64(L, orc, m, P):
    """The reference's three cases plus tile-boundary and long-prefix cases, and the last chunk rows of the long-context
    configuration's 32768- and 131072-token prompts (every query attends over the whole cache)."""
    rng = np.random.default_rng(m + P)
    S = P + m
    K = (rng.standard_normal((S + 2, 8, 64)) * 1.5).astype(np.float16)
    V = rng.standard_normal((S + 2, 8, 64)).astype(np.float16)
    Q = (rng.standard_normal((m, H)) * 1.5 * 0.125).astype(np.float16)
    K[S:] = np.nan                                        # never visible to any query
    V[S:] = np.nan
    o = nan_f32(m, H)
    f16 = lambda a: dev(a.view(np.int16)).view(torch.float16)
    L.k_pf_attn(f16(Q), m, P, f16(K), f16(V), o)
    ref = orc.pf_attn_f64(Q.view(np.uint16), m, P, K.view(np.uint16), V.view(np.uint16))
    got = host(o)
    assert np.all(np.isfinite(got))
    err = float(np.max(np.abs(got - ref)))
    assert err < 2e-3, err                                # reference gate: 4e-3


def test_pf_attn_last_row_matches_decode_attention(L, orc):
    """Same cache, same query: the chunk kernel's row for position p and the decode kernels at *d_pos = p agree
    to the fp16 rounding of Q and P (the decode path keeps both in fp32)."""
    rng = np.random.default_rng(5)
    m, P = 40, 700
    S = P + m
    K = (rng.standard_normal((S, 8, 64))).astype(np.float16)
    V = rng.standard_normal((S, 8, 64)).astype(np.float16)
    q32 = (rng.standard_normal((m, H)) * 1.5).astype(np.float32)
    Q = (q32 * np.float32(0.125)).astype(np.float16)
    f16 = lambda a: dev(a.view(np.int16)).view(torch.float16)
    kc, vc = f16(K), f16(V)
    o = nan_f32(m, H)
    L.k_pf_attn(f16(Q), m, P, kc, vc, o)
    part, out = nan_f32(32 * L.ATTN_SPLIT * L.ATTN_PARTW), nan_f32(H)
    for t in (0, 17, m - 1):
        d_pos = dev(np.array([P + t], np.int32))
        L.k_attn_split(dev(q32[t]), kc, vc, d_pos, part)
        L.k_attn_combine(part, d_pos, out, None)
        assert float(np.max(np.abs(host(out) - host(o)[t]))) < 3e-3
