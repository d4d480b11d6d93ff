"""Parity of the decode kernels (through the C ABI) with the CPU checker.  Needs a B200.

Bar: bit-exact for quants, fp16 scale fields, int32 block sums, expert ids; fp32
outputs bit-exact wherever no approximate device function (rsqrtf, expf, __expf) is
involved, else within 1e-5 relative (tolerances are written at each check).
"""
import numpy as np
import pytest

from helpers import act_floats, dev, empty_blocks, host, nan_f32, rand_q4, ulp_diff

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L(lkb):
    lkb.init(0)
    return lkb


def _blocks(orc, t):
    return orc.unpack_blocks(host(t, orc.BLOCK_Q8_1))


def _f16(u16):
    return np.asarray(u16, np.uint16).view(np.float16).astype(np.float32)


def test_quantize_q8_1_bit_exact(L, orc):
    rng = np.random.default_rng(1)
    x = act_floats(rng, 64 * 32)
    x[0:32] = 0.0                                    # all-zero block
    x[32:64] = np.linspace(-3e-4, 3e-4, 32)          # fp16-subnormal d
    x[64:96] = np.arange(32, dtype=np.float32) - 15.5   # exact .5 ties after scaling by 127/amax
    x[96:128] = 1e4 * rng.standard_normal(32)        # large sum
    y = empty_blocks(64)
    L.k_quantize_q8_1(dev(x), y, 64)
    q, d16, s16 = _blocks(orc, y)
    oq, od, os_ = orc.quantize_q8_1(x)
    assert np.array_equal(q, oq) and np.array_equal(d16, od) and np.array_equal(s16, os_)
    assert q.min() >= -127


@pytest.mark.parametrize("rows,bpr", [(2048, 64), (2048, 48), (100, 8), (37, 33), (64, 368)])
def test_gemv_and_block_sums(L, orc, rows, bpr):
    rng = np.random.default_rng(rows * 1000 + bpr)
    qs, d = rand_q4(rng, rows, bpr)
    x = act_floats(rng, bpr * 32)
    act = orc.quantize_q8_1(x)
    xq = dev(orc.pack_blocks(*act))
    dqs, dd = dev(qs), dev(d)
    # int32 block sums: exact
    s_dev = torch.full((rows, bpr), -(1 << 30), dtype=torch.int32, device="cuda")
    L.block_sumi(dqs, xq, rows, bpr, s_dev)
    assert np.array_equal(host(s_dev), orc.block_sumi(qs, act[0], rows, bpr))
    # fp32 GEMV: same summation order as the checker -> bit-exact
    y = nan_f32(rows)
    L.k_gemv_q4_0(dqs, dd, xq, rows, bpr, y, 0, None, 0.0)
    y_ref = orc.gemv_q4_0(qs, d, act, rows, bpr)
    assert np.array_equal(host(y), y_ref)
    y64, mag = orc.gemv_q4_0_f64(qs, d, act, rows, bpr)
    assert np.all(np.abs(host(y) - y64) <= 1e-5 * mag)        # the 1e-5 contract against float64
    # residual add
    y0 = rng.standard_normal(rows).astype(np.float32)
    yr = dev(y0)
    L.k_gemv_q4_0(dqs, dd, xq, rows, bpr, yr, 1, None, 0.0)
    assert np.array_equal(host(yr), orc.gemv_q4_0(qs, d, act, rows, bpr, y_in=y0))
    # consumer-side norm scale (rsqrtf on the device: 2-ulp tolerance on inv)
    ssq = (rng.random(64).astype(np.float32) + 0.5) * 32.0
    y2 = nan_f32(rows)
    L.k_gemv_q4_0(dqs, dd, xq, rows, bpr, y2, 0, dev(ssq), 1e-5)
    inv = orc.norm_inv(ssq)
    ref2 = y_ref * np.float32(inv)
    assert np.all(np.abs(host(y2) - ref2) <= 4e-7 * np.abs(ref2) + 1e-30)


def test_rmsnorm_q8_1(L, orc):
    rng = np.random.default_rng(7)
    for trial in range(3):
        x = act_floats(rng, 2048) * (1.0 + trial)
        w = (1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32)
        if trial == 2:
            x[:] = 0.0
        y32, yq8 = nan_f32(2048), empty_blocks(64)
        y16 = torch.zeros(2048, dtype=torch.float16, device="cuda")
        L.k_rmsnorm_q8_1(dev(x), dev(w), 2048, 1e-5, y32, y16, yq8)
        g32 = host(y32)
        # rsqrtf is approximate on the device: find the inv (within 2 ulp of the
        # checker's) that reproduces the device's y32 bit for bit, then demand the
        # quantised blocks match exactly under that inv.
        _, _, inv0 = orc.rmsnorm_q8_1(x, w)
        found = False
        for k in (0, 1, -1, 2, -2):
            inv = np.float32(inv0)
            for _ in range(abs(k)):
                inv = np.nextafter(inv, np.float32(np.inf if k > 0 else 0), dtype=np.float32)
            o32, oact, _ = orc.rmsnorm_q8_1(x, w, inv_override=float(inv))
            if np.array_equal(o32, g32):
                found = True
                break
        assert found, "device inv is further than 2 ulp from 1/sqrt(ss/2048+eps)"
        q, d16, s16 = _blocks(orc, yq8)
        assert np.array_equal(q, oact[0]) and np.array_equal(d16, oact[1]) and np.array_equal(s16, oact[2])
        assert np.array_equal(host(y16).view(np.uint16), o32.astype(np.float16).view(np.uint16))


def test_norm_split_producer_consumer(L, orc):
    """Scale-carrying norm: quantise raw x*w + ssq (producer), inv applied by the consumer."""
    rng = np.random.default_rng(8)
    x = act_floats(rng, 2048)
    w = (1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32)
    h32, yq8, ssq = nan_f32(2048), empty_blocks(64), nan_f32(64)
    L.norm_produce(dev(x), 2048, L.norm_prod(dev(w), h32, yq8, ssq))
    oh, oact, ossq = orc.norm_prod(x, w)
    q, d16, s16 = _blocks(orc, yq8)
    assert np.array_equal(host(h32), oh) and np.array_equal(host(ssq), ossq)
    assert np.array_equal(q, oact[0]) and np.array_equal(d16, oact[1]) and np.array_equal(s16, oact[2])
    # scale invariance: GEMV(raw) * inv  vs  GEMV(plain-normed), <= 2.5 fp16 ulp (reference gate)
    qs, d = rand_q4(rng, 256, 64)
    y_split = nan_f32(256)
    L.k_gemv_q4_0(dev(qs), dev(d), yq8, 256, 64, y_split, 0, ssq, 1e-5)
    _, pact, _ = orc.rmsnorm_q8_1(x, w)
    y_plain = orc.gemv_q4_0(qs, d, pact, 256, 64)
    rel = np.linalg.norm(host(y_split) - y_plain) / np.linalg.norm(y_plain)
    assert rel <= 2.5 / 2048.0
    y_noscale = orc.gemv_q4_0(qs, d, oact, 256, 64)          # negative control: must be visibly wrong
    assert np.linalg.norm(y_noscale - y_plain) / np.linalg.norm(y_plain) > 0.05


def test_gemv_prod_and_three(L, orc):
    rng = np.random.default_rng(9)
    rows, bpr = 2048, 64
    qs, d = rand_q4(rng, rows, bpr)
    act = orc.quantize_q8_1(act_floats(rng, bpr * 32))
    xq = dev(orc.pack_blocks(*act))
    w = (1.0 + 0.05 * rng.standard_normal(rows)).astype(np.float32)
    for add in (0, 1):
        y0 = rng.standard_normal(rows).astype(np.float32)
        y = dev(y0)
        h32, yq8, ssq = nan_f32(rows), empty_blocks(rows // 32), nan_f32(rows // 32)
        L.k_gemv_q4_0_prod(dev(qs), dev(d), xq, rows, bpr, y, add, L.norm_prod(dev(w), h32, yq8, ssq))
        y_ref = orc.gemv_q4_0(qs, d, act, rows, bpr, y_in=y0 if add else None)
        assert np.array_equal(host(y), y_ref)
        oh, oact, ossq = orc.norm_prod(y_ref, w)
        q, d16, s16 = _blocks(orc, yq8)
        assert np.array_equal(host(h32), oh) and np.array_equal(host(ssq), ossq)
        assert np.array_equal(q, oact[0]) and np.array_equal(d16, oact[1]) and np.array_equal(s16, oact[2])
    # no producer (np.w null): outputs only
    y = nan_f32(rows)
    L.k_gemv_q4_0_prod(dev(qs), dev(d), xq, rows, bpr, y, 0, None)
    assert np.array_equal(host(y), orc.gemv_q4_0(qs, d, act, rows, bpr))
    # q/k/v in one launch
    r = (2048, 512, 512)
    ws = [rand_q4(rng, n, bpr) for n in r]
    ys = [nan_f32(n) for n in r]
    L.k_gemv_q4_0_3(dev(ws[0][0]), dev(ws[0][1]), r[0], ys[0], dev(ws[1][0]), dev(ws[1][1]), r[1], ys[1],
                    dev(ws[2][0]), dev(ws[2][1]), r[2], ys[2], xq, bpr, None, 0.0)
    for (q_, d_), n, yv in zip(ws, r, ys):
        assert np.array_equal(host(yv), orc.gemv_q4_0(q_, d_, act, n, bpr))


def test_router_golden_fixture(L, orc, golden_dir):
    """The reference's real gate matrix + bias: ids exact, weights 1e-5."""
    g = np.load(golden_dir / "router_fixture.npz")
    h, W, b = dev(g["h"]), dev(g["gate"]), dev(g["bias"])
    logits, sel, sig = nan_f32(64), nan_f32(64), nan_f32(64)
    L.k_router_dot(h, W, logits, b, sel, sig, None, 0.0)
    assert np.array_equal(host(logits), orc.router_dot(g["h"], g["gate"]))      # same FMA chain: bit-exact
    osel, osig = orc.router_gate(host(logits), g["bias"])
    assert np.max(ulp_diff(host(sig), osig)) <= 4 and np.max(np.abs(host(sel) - osel)) <= 1e-6
    idx = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    w = nan_f32(4)
    L.k_router_top4(logits, b, idx, w)
    assert host(idx).tolist() == [59, 45, 58, 40]
    assert np.max(np.abs(host(w).astype(np.float64) - g["expected_w"])) < 1e-5
    assert abs(float(host(w).sum()) - 1.0) < 1e-6
    # selection given the device's own sel/sig is exact
    oi, ow = orc.router_select(host(sel), host(sig))
    assert oi.tolist() == host(idx).tolist() and np.max(ulp_diff(ow, host(w))) <= 1


def test_router_ties_and_softmax(L, orc):
    logits = np.zeros(64, np.float32)            # all equal: lowest indices win
    bias = np.zeros(64, np.float32)
    idx = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    w = nan_f32(4)
    L.k_router_top4(dev(logits), dev(bias), idx, w)
    assert host(idx).tolist() == [0, 1, 2, 3] and np.allclose(host(w), 0.25)
    logits[:] = -200.0                           # sigmoid underflows: the 2^-14 guard on the weight sum
    L.k_router_top4(dev(logits), dev(bias), idx, w)
    assert host(idx).tolist() == [0, 1, 2, 3] and np.all(np.isfinite(host(w)))
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(64).astype(np.float32)
    L.router_top4_softmax(dev(logits), None, idx, w)
    sel, sig = orc.router_gate(logits, None, softmax=True)
    oi, ow = orc.router_select(sel, sig)
    assert host(idx).tolist() == oi.tolist() and np.max(np.abs(host(w) - ow)) < 1e-6
    e = np.exp(logits[oi].astype(np.float64))
    assert np.max(np.abs(host(w) - e / e.sum())) < 1e-6     # == exp(l_k)/sum_top4 exp(l)


def _moe_layer(rng, n_exp=64):
    H, I = 2048, 1536
    gate = rand_q4(rng, n_exp * I, H // 32)
    up = rand_q4(rng, n_exp * I, H // 32)
    down = rand_q4(rng, n_exp * H, I // 32)
    Wr = (0.02 * rng.standard_normal((n_exp, H))).astype(np.float32)
    return gate, up, down, Wr


def test_moe_ffn_layer_config1(L, orc):
    """One MoE FFN layer at batch 1 (benchmark configuration 1), kernel by kernel and end to end."""
    rng = np.random.default_rng(11)
    H, I = 2048, 1536
    gate, up, down, Wr = _moe_layer(rng)
    x = act_floats(rng, H, outliers=False)
    nw = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    bias = (0.05 * rng.standard_normal(64)).astype(np.float32)
    nw_next = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)

    d_x = dev(x)
    h32, xq, ssq = nan_f32(H), empty_blocks(64), nan_f32(64)
    L.norm_produce(d_x, H, L.norm_prod(dev(nw), h32, xq, ssq))
    logits = nan_f32(64)
    L.k_router_dot(h32, dev(Wr), logits, dev(bias), None, None, ssq, 1e-5)
    idx = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    wk = nan_f32(4)
    L.k_router_top4(logits, dev(bias), idx, wk)
    gu = nan_f32(2 * 4 * I)
    dg, du, dd_ = [dev(a) for a in gate], [dev(a) for a in up], [dev(a) for a in down]
    L.k_gemv_q4_0_exp2(dg[0], dg[1], du[0], du[1], xq, I, 64, I, 0, idx, gu[:4 * I], gu[4 * I:], ssq, 1e-5)
    v, xq2 = nan_f32(4 * I), empty_blocks(4 * 48)
    L.k_swiglu(gu[:4 * I], gu[4 * I:], 4 * I, v, xq2, dd_[0], idx, H, 48, 2 << 20)
    h32n, xqn, ssqn = nan_f32(H), empty_blocks(64), nan_f32(64)
    L.k_moe_down_accum(dd_[0], dd_[1], xq2, H, 48, H, 48, idx, wk, d_x, L.norm_prod(dev(nw_next), h32n, xqn, ssqn))
    torch.cuda.synchronize()

    # ---- the checker, stage by stage on the device's own upstream values ----
    oh, oact, ossq = orc.norm_prod(x, nw)
    assert np.array_equal(host(h32), oh) and np.array_equal(host(ssq), ossq)
    inv = orc.norm_inv(ossq)
    ol = orc.router_dot(oh, Wr, ninv=1.0) * np.float32(inv)
    assert np.all(np.abs(host(logits) - ol) <= 4e-7 * np.abs(ol) + 1e-12)
    sel, sig = orc.router_gate(host(logits), bias)
    oi, ow = orc.router_select(sel, sig)
    assert orc.router_margin(sel) > 1e-5
    assert host(idx).tolist() == oi.tolist()                              # expert ids: exact
    assert np.max(np.abs(host(wk) - ow)) <= 1e-6
    ogu_g = orc.gemv_q4_0_exp(gate[0], gate[1], oact, I, 64, I, 0, oi)
    ogu_u = orc.gemv_q4_0_exp(up[0], up[1], oact, I, 64, I, 0, oi)
    g_gu = host(gu)
    ref_gu = np.concatenate([ogu_g, ogu_u]) * np.float32(inv)
    assert np.all(np.abs(g_gu - ref_gu) <= 4e-7 * np.abs(ref_gu) + 1e-12)
    ov = orc.swiglu(g_gu[:4 * I], g_gu[4 * I:])
    assert np.all(np.abs(host(v) - ov) <= 2e-6 * np.abs(ov) + 1e-9)       # __expf on the device
    oact2 = orc.quantize_q8_1(host(v))                                    # quantisation of the device's v: exact
    q, d16, s16 = _blocks(orc, xq2)
    assert np.array_equal(q, oact2[0]) and np.array_equal(d16, oact2[1]) and np.array_equal(s16, oact2[2])
    xo, oh2, oact3, ossq3 = orc.moe_down_accum(down[0], down[1], oact2, H, 48, H, 48, oi, host(wk), x, nw_next)
    assert np.array_equal(host(d_x), xo)                                   # bit-exact given identical inputs
    q, d16, s16 = _blocks(orc, xqn)
    assert np.array_equal(q, oact3[0]) and np.array_equal(d16, oact3[1]) and np.array_equal(s16, oact3[2])
    assert np.array_equal(host(ssqn), ossq3) and np.array_equal(host(h32n), oh2)

    # ---- end to end against an all-CPU run (libm exp, 1/sqrt): 1e-5 relative ----
    cl = orc.router_dot(oh, Wr, ninv=inv)
    csel, csig = orc.router_gate(cl, bias)
    ci, cw = orc.router_select(csel, csig)
    assert ci.tolist() == oi.tolist()
    cg = orc.gemv_q4_0_exp(gate[0], gate[1], oact, I, 64, I, 0, ci, ninv=inv)
    cu = orc.gemv_q4_0_exp(up[0], up[1], oact, I, 64, I, 0, ci, ninv=inv)
    cact2 = orc.quantize_q8_1(orc.swiglu(cg, cu))
    cx, _, _, _ = orc.moe_down_accum(down[0], down[1], cact2, H, 48, H, 48, ci, cw, x, None)
    delta = host(d_x) - cx
    upd = cx - x
    assert np.linalg.norm(delta) <= 2e-3 * np.linalg.norm(upd)            # quantiser flips from 1-ulp v differences
    assert np.max(np.abs(delta)) <= 1e-5 * np.max(np.abs(cx)) + 2e-3 * np.max(np.abs(upd))


def test_moe_accum4_and_exp(L, orc):
    rng = np.random.default_rng(12)
    H = 2048
    down4 = rng.standard_normal(4 * H).astype(np.float32)
    wk = rng.random(4).astype(np.float32)
    x = rng.standard_normal(H).astype(np.float32)
    nw = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    dx = dev(x)
    h32, yq8, ssq = nan_f32(H), empty_blocks(64), nan_f32(64)
    L.k_moe_accum4(dx, dev(down4), dev(wk), H, L.norm_prod(dev(nw), h32, yq8, ssq))
    a = np.zeros(H, np.float32)          # float64 emulation of the fp32 FMA chain (<= 1 ulp from double rounding)
    for k in range(4):
        a = (np.float64(wk[k]) * down4[k * H:(k + 1) * H].astype(np.float64) + a.astype(np.float64)).astype(np.float32)
    xo = x + a
    assert np.max(ulp_diff(host(dx), xo)) <= 1
    oh, oact, ossq = orc.norm_prod(host(dx), nw)
    q, d16, s16 = _blocks(orc, yq8)
    assert np.array_equal(q, oact[0]) and np.array_equal(host(ssq), ossq) and np.array_equal(host(h32), oh)
    # per-expert activations (xq_stride != 0), no inv
    rows, bpr = 256, 48
    qs, d = rand_q4(rng, 8 * rows, bpr)
    act = orc.quantize_q8_1(act_floats(rng, 4 * bpr * 32))
    idx = np.array([5, 0, 7, 2], np.int32)
    y = nan_f32(4 * rows)
    L.k_gemv_q4_0_exp(dev(qs), dev(d), dev(orc.pack_blocks(*act)), rows, bpr, rows, bpr, dev(idx), y)
    assert np.array_equal(host(y), orc.gemv_q4_0_exp(qs, d, act, rows, bpr, rows, bpr, idx))


def test_error_statuses(L):
    x = torch.zeros(64, device="cuda")
    assert L.lib.lkb_gemv_q4_0(None, None, None, 1, 1, None, 0, None, 0.0, None) == -10002
    assert L.lib.lkb_rmsnorm_q8_1(x.data_ptr(), x.data_ptr(), 100, 1e-5, None, None, None, None) == -10001
    assert L.lib.lkb_moe_accum4(x.data_ptr(), x.data_ptr(), x.data_ptr(), 33, None, None) == -10001


def test_decode_stack_pdl_and_graph_are_bit_identical(L):
    """Programmatic dependent launch and CUDA-graph replay must not change a single bit."""
    import importlib
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    layers = synth.make_model(3, seed=77)
    st = decode.DecodeStack(layers)
    x0 = torch.randn(2048, device="cuda", generator=torch.Generator("cuda").manual_seed(5))
    outs = []
    for pdl in (False, True, True, False):
        L.set_pdl(pdl)
        st.x.copy_(x0)
        st.step()
        torch.cuda.synchronize()
        outs.append(st.x.clone())
    L.set_pdl(True)
    g = torch.cuda.CUDAGraph()
    st.x.copy_(x0)
    with torch.cuda.graph(g):
        st.step()
    for _ in range(3):
        st.x.copy_(x0)
        g.replay()
        torch.cuda.synchronize()
        outs.append(st.x.clone())
    L.set_pdl(False)
    assert torch.isfinite(outs[0]).all()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def test_fused_stack_is_bit_identical_to_kernel_sequence(L):
    """lkb_moe_ffn_decode(_stack): one persistent launch == the five-kernel sequence, bit for bit."""
    import importlib
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    layers = synth.make_model(4, seed=91, zipf_s=1.1)
    st = decode.DecodeStack(layers)
    gen = torch.Generator("cuda").manual_seed(6)
    for trial in range(3):
        x0 = torch.randn(2048, device="cuda", generator=gen) * (1.0 + trial)
        st.x.copy_(x0)
        st.step()
        ref = st.x.clone()
        st.x.copy_(x0)
        st.step_fused()
        torch.cuda.synchronize()
        assert st.status() == 0
        assert torch.isfinite(ref).all() and torch.equal(st.x, ref)
        idx_stack = st.sel_idx.clone()
        st.x.copy_(x0)
        st.step_fused(per_layer_launch=True)
        torch.cuda.synchronize()
        assert st.status() == 0 and torch.equal(st.x, ref) and torch.equal(st.sel_idx, idx_stack)
        assert torch.equal(st.sel_idx[-1], st.idx)            # the last layer's experts match the unfused router
    # the optional producer output for the caller's next consumer
    nw = layers[0].norm_w
    h32, yq8, ssq = nan_f32(2048), empty_blocks(64), nan_f32(64)
    st.x.copy_(x0)
    L.moe_ffn_decode(st._descs[0], st.x, st.sel_idx[0], st.sel_w[0], L.norm_prod(nw, h32, yq8, ssq), st._scratch)
    h2, y2, s2 = nan_f32(2048), empty_blocks(64), nan_f32(64)
    L.norm_produce(st.x, 2048, L.norm_prod(nw, h2, y2, s2))
    assert torch.equal(h32, h2) and torch.equal(yq8, y2) and torch.equal(ssq, s2)


def test_bounded_wait_reports_status_and_context_survives(L):
    """A CTA that never arrives (requested from the host) makes the other CTAs' bounded grid-barrier wait run out:
    the kernel ends with a status code, nothing hangs or faults, and the next launch is correct again."""
    import ctypes
    import importlib
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    layers = synth.make_model(2, seed=55)
    st = decode.DecodeStack(layers)
    x0 = torch.randn(2048, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    st.x.copy_(x0)
    st.step_fused()
    torch.cuda.synchronize()
    good = st.x.clone()
    assert st.status() == 0
    L.lib.lkb_debug_fused_absent_cta.argtypes = [ctypes.c_int, ctypes.c_uint]
    L.lib.lkb_debug_fused_absent_cta(5, 1 << 14)             # CTA 5 stays away; waits give up after 16384 polls
    try:
        st.x.copy_(x0)
        st.step_fused()
        torch.cuda.synchronize()                              # returns: the wait is bounded
        assert st.status() == 1001                            # grid barrier 1 of layer 0 expired
    finally:
        L.lib.lkb_debug_fused_absent_cta(-1, 0)
    st.x.copy_(x0)
    st.step_fused()
    torch.cuda.synchronize()
    assert st.status() == 0 and torch.equal(st.x, good)


def test_expert_prefetch_leaves_results_unchanged(L):
    """lkb_decode_set_expert_prefetch: the guessed experts of the next layer only warm L2.  The residual, the selection
    and the weights of every layer are those of the kernel sequence bit for bit, the status word stays 0, and the
    hit counter reports 4 guesses per layer after the first, each guess a valid expert."""
    import importlib
    synth = importlib.import_module("lfm2-ampere_b200.synth")
    decode = importlib.import_module("lfm2-ampere_b200.decode")
    n_layers = 6
    layers = synth.make_model(n_layers, seed=17, zipf_s=0.0)
    st = decode.DecodeStack(layers)
    gen = torch.Generator("cuda").manual_seed(8)
    try:
        for trial in range(3):
            x0 = torch.randn(2048, device="cuda", generator=gen) * (1.0 + 3 * trial)
            st.x.copy_(x0); st.step(); ref = st.x.clone()
            L.decode_set_expert_prefetch(0)
            st.x.copy_(x0); st.step_fused(); torch.cuda.synchronize()
            off_x, off_idx, off_w = st.x.clone(), st.sel_idx.clone(), st.sel_w.clone()
            L.decode_set_expert_prefetch(1)
            st.x.copy_(x0); st.step_fused(); torch.cuda.synchronize()
            assert st.status() == 0
            assert torch.isfinite(ref).all() and torch.equal(off_x, ref) and torch.equal(st.x, ref)
            assert torch.equal(st.sel_idx, off_idx) and torch.equal(st.sel_w, off_w)
            hits, guesses = L.decode_expert_prefetch_hits(st._scratch, n_layers)
            assert guesses == 4 * (n_layers - 1) and 0 <= hits <= guesses
            rec = st.gu[4 * 1536 + 128:].view(torch.int32)
            guess, real = rec[:4 * n_layers].view(n_layers, 4), rec[4 * 512:4 * 512 + 4 * n_layers].view(n_layers, 4)
            assert torch.equal(real, st.sel_idx)
            assert int(guess[1:].min()) >= 0 and int(guess[1:].max()) < 64
            for l in range(1, n_layers):
                assert len(set(guess[l].tolist())) == 4
        # a single layer has nothing to guess for
        L.moe_ffn_decode(st._descs[0], st.x, st.sel_idx[0], st.sel_w[0], None, st._scratch)
        torch.cuda.synchronize()
        assert st.status() == 0
    finally:
        L.decode_set_expert_prefetch(0)
