"""Full decode step (embedding -> mixers + MoE FFN -> lm_head -> argmax) on a small synthetic model:
the call sequence itself.  Every kernel has its own parity test; here the chain is checked stage by stage
against the CPU checker on one conv layer, and the orchestration variants (eager / CUDA graph, fused MoE /
five-kernel MoE) are required to produce identical tokens and residuals."""
import importlib

import numpy as np
import pytest

from helpers import host

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

H = 2048


@pytest.fixture(scope="module")
def M(lkb):
    lkb.init(0)
    return importlib.import_module("lfm2-ampere_b200.model")


def _np(t, dtype=None):
    a = t.detach().cpu().numpy()
    return a if dtype is None else a.view(np.uint8).reshape(-1).view(dtype)


def test_conv_layer_chain_matches_checker(M, lkb, orc):
    """embed -> rmsnorm_q8_1 -> in_proj GEMV -> shortconv -> out_proj GEMV (+residual, producer) on layer 0."""
    model = M.make_full_model(n_layers=1, seed=77, vocab=2048)
    ds = M.DecodeStep(model, max_seq=64, moe_impl="kernels")
    mx = model.mixers[0]
    tok = 1234
    ds.d_token.fill_(tok)
    hist0 = torch.randn(2 * H, device="cuda") * 0.5
    ds.hist[0].copy_(hist0)
    api = lkb
    api.k_embed_q6_K(*model.emb, ds.d_token, H, ds.x)
    x0 = host(ds.x).copy()
    emb = [_np(t) for t in model.emb[:3]] + [_np(model.emb[3], np.uint16)]
    assert np.array_equal(x0, orc.embed_q6_K(*emb, tok, 8))
    api.k_rmsnorm_q8_1(ds.x, mx.attn_norm, H, 1e-5, None, None, ds.xq)
    dq, dd, dsum = orc.unpack_blocks(host(ds.xq, orc.BLOCK_Q8_1))
    act = None
    _, _, inv0 = orc.rmsnorm_q8_1(x0, host(mx.attn_norm))
    for k in (0, 1, -1, 2, -2):                           # the device's rsqrtf is within 2 ulp of 1/sqrt
        inv = np.float32(inv0)
        for _ in range(abs(k)):
            inv = np.nextafter(inv, np.float32(np.inf if k > 0 else 0), dtype=np.float32)
        _, a, _ = orc.rmsnorm_q8_1(x0, host(mx.attn_norm), inv_override=float(inv))
        if np.array_equal(a[0], dq) and np.array_equal(a[1], dd) and np.array_equal(a[2], dsum):
            act = a
            break
    assert act is not None
    api.k_gemv_q4_0(mx.in_qs, mx.in_d, ds.xq, 3 * H, 64, ds.y, 0, None, 1e-5)
    y_ref = orc.gemv_q4_0(_np(mx.in_qs), _np(mx.in_d, np.uint16), act, 3 * H, 64)
    assert np.array_equal(host(ds.y), y_ref)
    api.k_shortconv(ds.y, mx.conv_w, ds.hist[0], None, ds.xq, H)
    c_ref, h_ref = orc.shortconv(y_ref, host(mx.conv_w), host(hist0))
    assert np.array_equal(host(ds.hist[0]), h_ref)
    act2 = orc.quantize_q8_1(c_ref)
    q2, d2, s2 = orc.unpack_blocks(host(ds.xq, orc.BLOCK_Q8_1))
    assert np.array_equal(q2, act2[0]) and np.array_equal(d2, act2[1]) and np.array_equal(s2, act2[2])
    api.k_gemv_q4_0_prod(mx.out_qs, mx.out_d, ds.xq, H, 64, ds.x, 1, ds._np_ffn[0])
    x1 = orc.gemv_q4_0(_np(mx.out_qs), _np(mx.out_d, np.uint16), act2, H, 64, y_in=x0)
    assert np.array_equal(host(ds.x), x1)
    oh, oact, ossq = orc.norm_prod(x1, host(model.moe[0].norm_w))
    qf, df, sf = orc.unpack_blocks(host(ds.xqf, orc.BLOCK_Q8_1))
    assert np.array_equal(host(ds.h32), oh) and np.array_equal(host(ds.ssq), ossq)
    assert np.array_equal(qf, oact[0]) and np.array_equal(df, oact[1]) and np.array_equal(sf, oact[2])


def _run(M, model, impl, graph, steps, pos0):
    ds = M.DecodeStep(model, max_seq=pos0 + steps + 8, moe_impl=impl)
    ds.fill_kv(pos0)
    ds.d_token.fill_(17)
    toks, xs = [], []
    if graph:
        ds.step()                                          # warm the launch path, then rewind the state
        torch.cuda.synchronize()
        ds.hist.zero_()
        ds.fill_kv(pos0)
        ds.d_token.fill_(17)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            ds.step()
        # capture does not execute: state is still at the start
    for _ in range(steps):
        g.replay() if graph else ds.step()
        torch.cuda.synchronize()
        toks.append(int(ds.d_token.item()))
        xs.append(host(ds.x).copy())
    assert int(ds.d_pos.item()) == pos0 + steps
    assert ds.status() == 0
    return toks, xs, ds


def test_step_variants_agree_and_advance(M, lkb):
    """4 layers (conv, conv, attention, conv): eager == graph replay, fused MoE == five-kernel MoE, bit for bit;
    the position advances, the KV cache grows by one row per step, tokens stay inside the vocabulary."""
    model = M.make_full_model(n_layers=4, seed=5, vocab=4096)
    pos0, steps = 300, 4
    ref_t, ref_x, ds = _run(M, model, "kernels", False, steps, pos0)
    assert all(0 <= t < 4096 for t in ref_t)
    assert all(np.all(np.isfinite(x)) for x in ref_x)
    k_rows = host(ds.kc[0, pos0:pos0 + steps]).astype(np.float32)
    assert np.all(np.abs(k_rows).sum(axis=(1, 2)) > 0)     # every step appended a K row
    assert float(ds.kc[0, pos0 + steps].abs().sum().item()) == 0.0
    for impl, graph in (("kernels", True), ("fused", False), ("fused", True), ("mega", False), ("mega", True)):
        t, x, _ = _run(M, model, impl, graph, steps, pos0)
        assert t == ref_t, (impl, graph, t, ref_t)
        for a, b in zip(x, ref_x):
            assert np.array_equal(a, b), (impl, graph)
    lkb.set_pdl(True)
    try:
        t, x, _ = _run(M, model, "kernels", True, steps, pos0)
    finally:
        lkb.set_pdl(False)
    assert t == ref_t and all(np.array_equal(a, b) for a, b in zip(x, ref_x))
    # expert prefetch in the whole-step kernel: same tokens, same residuals
    lkb.decode_set_expert_prefetch(3)
    try:
        for graph in (False, True):
            t, x, _ = _run(M, model, "mega", graph, steps, pos0)
            assert t == ref_t and all(np.array_equal(a, b) for a, b in zip(x, ref_x)), graph
    finally:
        lkb.decode_set_expert_prefetch(0)


def test_new_entry_points_reject_bad_arguments(M, lkb):
    """Null pointers and shape preconditions come back as LkbError (status codes), never as a fault."""
    f = torch.zeros(4096, device="cuda")
    i = torch.zeros(4, dtype=torch.int32, device="cuda")
    u8 = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    with pytest.raises(lkb.LkbError):
        lkb.k_gemv_q6_K(None, u8, u8, u8, u8, 16, 8, f)
    with pytest.raises(lkb.LkbError):
        lkb.k_gemv_q6_K(u8, u8, u8, u8, u8, 0, 8, f)
    with pytest.raises(lkb.LkbError):
        lkb.k_argmax_part(f, 0, f, i)
    with pytest.raises(lkb.LkbError):
        lkb.k_embed_q6_K(u8, u8, u8, u8, i, 100, f)            # n % 256 != 0
    with pytest.raises(lkb.LkbError):
        lkb.k_attn_split(None, u8, u8, i, f)
    with pytest.raises(lkb.LkbError):
        lkb.k_attn_combine(f, i, None, None)                   # nothing to write
    with pytest.raises(lkb.LkbError):
        lkb.k_qk_norm_rope(f, f, f, f, f, i, u8, u8, theta=0.5)
    model = M.make_full_model(n_layers=1, seed=1, vocab=2048)
    ds = M.DecodeStep(model, max_seq=16, moe_impl="mega")
    with pytest.raises(lkb.LkbError):
        lkb.decode_layers(ds.moe_dev, None, 1, ds.x, ds.xq, ds.d_pos, 1e6, None, ds._scratch, ds._sscratch)
    with pytest.raises(lkb.LkbError):
        lkb.decode_layers(ds.moe_dev, ds.mixers_dev, 0, ds.x, ds.xq, ds.d_pos, 1e6, None, ds._scratch, ds._sscratch)
    torch.cuda.synchronize()


def _prefill_and_decode(M, n_layers, m, seed):
    model = M.make_full_model(n_layers=n_layers, seed=seed, vocab=4096)
    toks = torch.randint(0, 4096, (m,), dtype=torch.int32, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    ds = M.DecodeStep(model, max_seq=m + 8, moe_impl="kernels")
    xs = []
    for t in range(m):
        ds.d_token.copy_(toks[t:t + 1])
        ds.step()
        xs.append(ds.x.clone())
    st = M.DecodeStep(model, max_seq=m + 8, moe_impl="mega")
    pc = M.PrefillChunk(model, m, st)
    pc.toks.copy_(toks)
    pc.step(P=0)
    torch.cuda.synchronize()
    return ds, torch.stack(xs), st, pc


def test_prefill_chunk_agrees_with_token_by_token_decode(M, lkb):
    """Prefill of m tokens against m decode steps fed the same tokens.  The two paths round differently (GEMM block
    order vs GEMV lane order; fp16 Q / P in the chunk attention, as in the reference), and top-4 routing amplifies a
    1e-3 difference into a different expert for some tokens, so beyond the first layer the comparison is
    statistical: medians over tokens.  One conv + MoE layer must agree to rounding for every token."""
    rows = lambda a, b: ((a.float() - b.float()).flatten(1).norm(dim=1) / b.float().flatten(1).norm(dim=1))
    m = 48
    # the GEMM's exact per-block arithmetic is the decode GEMV's; the reference's shipped folded form rounds each block's
    # offset term (3e-4 of sum|terms|) and so differs from its own decode path by more than this comparison allows
    lkb.pf_gemm_arith(0)
    ds, xs, st, pc = _prefill_and_decode(M, 1, m, 9)
    assert lkb.lib.lkb_pf_gemm_status() == 0 and int(st.d_pos.item()) == m
    e1 = rows(pc.X, xs)                                                 # chunk conv (history across tokens) + MoE vs decode:
    assert float(e1.median()) < 1e-6 and float(e1.max()) < 2e-2         # fp32 rounding, except where a Q8_1 rounding flips
    assert float(rows(st.hist[:1], ds.hist[:1]).max()) < 1e-5
    ds, xs, st, pc = _prefill_and_decode(M, 3, m, 9)                    # conv, conv, attention
    assert torch.isfinite(pc.X).all()
    assert float(rows(pc.X, xs).median()) < 5e-2                        # Q8_1 rounding flips accumulate over layers
    assert float(rows(st.kc[0, :m], ds.kc[0, :m]).median()) < 5e-2 and float(rows(st.vc[0, :m], ds.vc[0, :m]).median()) < 5e-2
    assert float(rows(st.kc[0, :1], ds.kc[0, :1]).max()) < 1e-3          # the first token has no history: rounding only
    assert float(st.kc[0, m:].abs().sum().item()) == 0.0                # nothing written past the chunk
    # decoding continues from the prefilled state
    st.d_token.fill_(7)
    st.step()
    torch.cuda.synchronize()
    assert int(st.d_pos.item()) == m + 1 and 0 <= int(st.d_token.item()) < 4096 and st.status() == 0
    lkb.pf_gemm_arith(1)


def test_kv_capacity_is_checked(M, lkb):
    """A decode step at a position past the KV cache writes nothing and reports it (status 600 + layer); a prefill chunk
    that does not fit is refused on the host."""
    model = M.make_full_model(n_layers=3, seed=2, vocab=2048)
    ds = M.DecodeStep(model, max_seq=4, moe_impl="mega")
    ds.d_pos.fill_(3)
    ds.step()                                                      # position 3: the last one that fits
    torch.cuda.synchronize()
    assert ds.status() == 0 and int(ds.d_pos.item()) == 4
    kc, vc = ds.kc.clone(), ds.vc.clone()
    ds.step()                                                      # position 4: past the cache
    torch.cuda.synchronize()
    assert ds.status() == 602                                      # layer 2 is the attention layer
    assert torch.equal(kc, ds.kc) and torch.equal(vc, ds.vc)
    ds.sync.zero_()
    pc = M.PrefillChunk(model, 8, M.DecodeStep(model, max_seq=8, moe_impl="mega"))
    with pytest.raises(ValueError):
        pc.step(P=1)
