"""Parity of the batched-prefill kernels (through the C ABI) with the CPU checker.  Needs a B200.

Integer work (quants, block sums inside the GEMM, expert ids, count/plan/scatter)
is compared bit for bit; fp32 GEMM outputs are compared bit for bit with the
checker's block-order fp32 statement in both per-block arithmetic modes, AND against
float64: the exact mode (fold = 0) within 1e-5 of sum|terms|, the reference's shipped
folded mode (fold = 1) within the reference's own gate -- beyond the rounding that form
is allowed (half an ulp of c per block), 2e-6 * max(1, bpr/16) of sum|terms|
(tests/test_prefill.cu:61-83,129-134 of the reference).
"""
import numpy as np
import pytest

from helpers import act_floats, dev, empty_blocks, host, nan_f32, rand_q4, ulp_diff, zipf_bias

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L(lkb):
    lkb.init(0)
    return lkb


@pytest.fixture(params=[0, 1], ids=["exact", "fold"])
def fold(request, L, orc):
    """Both per-block arithmetic modes of the GEMM, in the library and in the checker."""
    L.pf_gemm_arith(request.param)
    orc.set_gemm_fold(request.param)
    yield request.param
    L.pf_gemm_arith(1)
    orc.set_gemm_fold(1)


@pytest.fixture(params=["gather", "tiles"])
def ws(request, L):
    """Both activation paths of the grouped tensor-core GEMM: rows gathered through perm inside the kernel (no
    workspace), or copied into token-tile order first (caller-owned workspace registered)."""
    buf = None
    if request.param == "tiles":
        buf = torch.full((L.pf_gemm_workspace_bytes(4 * 700 // 64 + 64, 2048),), 0x5A, dtype=torch.uint8, device="cuda")
    L.pf_gemm_set_workspace(buf)
    yield request.param
    L.pf_gemm_set_workspace(None)


def _f64_gate(got, full, mag, slack, s, bpr, fold):
    """fp32 result against float64 (see the module docstring)."""
    if fold:
        return np.all(np.maximum(0.0, np.abs(got - full) - slack * s) <= 2e-6 * max(1, bpr // 16) * mag * s + 1e-6 * np.abs(full))
    return np.all(np.abs(got - full) <= 1e-5 * mag * s + 1e-6 * np.abs(full))


def _sums_agree_to_fp16_rounding(fused8, unfused8, d):
    """The sum field (8 * fp16 sum) of the fused SwiGLU epilogue in shipped arithmetic against the unfused quantiser's:
    the same 32 values added in two orders (the reference's fused epilogue pairs rows 8, 16, 1, 2, 4 apart, its warp
    quantiser 16, 8, 4, 2, 1).  The fp32 sums differ by rounding only -- at most 32 roundings of partial sums no
    larger than 32 amax, amax = 127 d -- and the fp16 fields by that plus one fp16 step; most are equal."""
    a, b = fused8.astype(np.float32) / 8.0, unfused8.astype(np.float32) / 8.0
    step = np.spacing(np.maximum(np.abs(a), np.abs(b)).astype(np.float16)).astype(np.float32)
    assert np.all(np.abs(a - b) <= step + 32.0 * 32.0 * 127.0 * d.astype(np.float32) * 2.0 ** -24)
    assert np.count_nonzero(a != b) <= 2e-3 * a.size


def _act_bufs(rows, kb):
    qs = torch.full((rows, kb * 32), 0x5A, dtype=torch.int8, device="cuda")
    sc = nan_f32(rows, kb, 2)
    return qs, sc


def _plan_dev(L, idx_flat):
    ns = idx_flat.size
    d_idx = dev(idx_flat.astype(np.int32))
    cnt = torch.zeros(64, dtype=torch.int32, device="cuda")
    off = torch.full((64,), -1, dtype=torch.int32, device="cuda")
    max_tiles = ns // 64 + 64
    tiles = torch.full((max_tiles, 4), -1, dtype=torch.int32, device="cuda")
    ntiles = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    perm = torch.full((ns,), -1, dtype=torch.int32, device="cuda")
    L.k_pf_moe_count(d_idx, ns, cnt)
    L.k_pf_moe_plan(cnt, off, tiles, ntiles)
    L.k_pf_moe_scatter(d_idx, ns, off, perm)
    return cnt, off, tiles, ntiles, perm, max_tiles


@pytest.mark.parametrize("m,skew", [(1, 0), (70, 1), (700, 1), (4096, 2), (257, 3)])
def test_count_plan_scatter(L, orc, m, skew):
    rng = np.random.default_rng(100 + m)
    if skew == 0:
        idx = np.array([[3, 9, 63, 0]], np.int32)
    elif skew == 3:                       # everything on four experts: long runs, most experts empty
        idx = np.tile(np.array([7, 8, 40, 63], np.int32), (m, 1))
    else:
        p = np.ones(64) if skew == 1 else 1.0 / (rng.permutation(64) + 1.0) ** 1.1
        p /= p.sum()
        idx = np.stack([rng.choice(64, size=4, replace=False, p=p) for _ in range(m)]).astype(np.int32)
    cnt, off, tiles, ntiles, perm, _ = _plan_dev(L, idx.reshape(-1))
    ocnt, ooff, otiles, operm = orc.moe_plan(idx.reshape(-1))
    assert np.array_equal(host(cnt), ocnt) and np.array_equal(host(off), ooff)
    nt = int(host(ntiles)[0])
    assert nt == otiles.shape[0] and np.array_equal(host(tiles)[:nt], otiles)
    pv = host(perm)
    assert np.array_equal(pv, operm)
    # the reference's properties (tests/test_prefill.cu:217-223)
    assert np.array_equal(np.sort(pv), np.arange(m * 4))
    e = idx.reshape(-1)[pv]
    assert np.all((e[1:] > e[:-1]) | ((e[1:] == e[:-1]) & (pv[1:] > pv[:-1])))


def test_quant_rows_and_pack(L, orc):
    rng = np.random.default_rng(21)
    rows, kb = 37, 48
    X = act_floats(rng, rows * kb * 32).reshape(rows, kb * 32)
    X[3, :64] = 0.0
    qs, sc = _act_bufs(rows, kb)
    L.k_pf_quant_rows(dev(X), kb * 32, kb, L.pf_act(qs, sc), rows)
    oq, osc = orc.pf_quant_rows(X, kb)
    assert np.array_equal(host(qs), oq) and np.array_equal(host(sc), osc)
    rows, kb = 5, 64
    X = act_floats(rng, rows * kb * 32).reshape(rows, kb * 32)
    qs, sc = _act_bufs(rows, kb)
    L.k_pf_quant_rows(dev(X), kb * 32, kb, L.pf_act(qs, sc), rows)
    y = empty_blocks(64)
    L.k_pf_pack_q8_1(L.pf_act(qs, sc), 3, y)
    ob = orc.pf_pack_q8_1(host(qs), host(sc), 3)
    assert host(y, orc.BLOCK_Q8_1).tobytes() == ob.tobytes()
    q, d16, s16 = orc.quantize_q8_1(X[3])             # == the decode quantiser's blocks
    assert ob.tobytes() == orc.pack_blocks(q, d16, s16).tobytes()


def test_pf_norm_matches_decode_kernels(L, orc):
    """Per-token kernels are memcmp-identical to their decode twins (tests/test_prefill.cu:382-432)."""
    rng = np.random.default_rng(22)
    m = 9
    X = act_floats(rng, m * 2048).reshape(m, 2048)
    X[4] = 0.0
    w = (1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32)
    dX, dw = dev(X), dev(w)
    # split form (plain = 0)
    qs, sc = _act_bufs(m, 64)
    inv, h32 = nan_f32(m), nan_f32(m, 2048)
    L.k_pf_norm(dX, dw, 0, L.pf_act(qs, sc), inv, h32, m)
    oq, osc, oinv, oh = orc.pf_norm(X, w, plain=False, want_h32=True)
    assert np.array_equal(host(qs), oq) and np.array_equal(host(sc), osc) and np.array_equal(host(h32), oh)
    assert np.max(ulp_diff(host(inv), oinv)) <= 2                         # rsqrtf
    # plain form vs the decode kernel, token by token
    qs1, sc1 = _act_bufs(m, 64)
    inv1 = nan_f32(m)
    L.k_pf_norm(dX, dw, 1, L.pf_act(qs1, sc1), inv1, None, m)
    assert np.all(host(inv1) == 1.0)
    for t in range(m):
        yq8, y = empty_blocks(64), empty_blocks(64)
        L.k_rmsnorm_q8_1(dX[t], dw, 2048, 1e-5, None, None, yq8)
        L.k_pf_pack_q8_1(L.pf_act(qs1, sc1), t, y)
        assert torch.equal(yq8, y)


def test_pf_swiglu_matches_decode(L, orc):
    rng = np.random.default_rng(23)
    rows, I = 12, 1536
    Y = (2.0 * rng.standard_normal((rows, 2 * I))).astype(np.float32)
    qs, sc = _act_bufs(rows, I // 32)
    dY = dev(Y)
    L.k_pf_swiglu(dY, 2 * I, I, I // 32, L.pf_act(qs, sc), rows)
    for r in (0, 5, 11):
        v, yq8, y = nan_f32(I), empty_blocks(I // 32), empty_blocks(I // 32)
        L.k_swiglu(dY[r, :I], dY[r, I:], I, v, yq8)
        ov = orc.swiglu(Y[r, :I], Y[r, I:])
        assert np.all(np.abs(host(v) - ov) <= 2e-6 * np.abs(ov) + 1e-9)
        oq, od, os_ = orc.quantize_q8_1(host(v))
        assert host(yq8, orc.BLOCK_Q8_1).tobytes() == orc.pack_blocks(oq, od, os_).tobytes()
        # planar row r == decode blocks
        assert np.array_equal(host(qs)[r], oq)
        assert np.array_equal(host(sc)[r, :, 0], orc.f16_bits_to_f32(od))
        assert np.array_equal(host(sc)[r, :, 1], 8.0 * orc.f16_bits_to_f32(os_))


def test_router_token_tile_forms_agree(L):
    """The tiled router has an 8-token and a 32-token form (picked by how many CTAs the chunk gives); both evaluate
    the same ascending-k chains, so a long chunk (32-token form) equals its pieces (8-token form) bit for bit."""
    rng = np.random.default_rng(77)
    m = 32 * L.lib.lkb_sm_count() + 40
    H = dev(rng.uniform(-1, 1, size=(m, 2048)).astype(np.float32))
    W = dev(rng.normal(0, 0.05, size=(64, 2048)).astype(np.float32))
    bias = dev(rng.normal(0, 0.1, size=64).astype(np.float32))
    inv = dev(rng.uniform(0.5, 2.0, size=m).astype(np.float32))
    sel, sig = nan_f32(m, 64), nan_f32(m, 64)
    L.k_pf_router_tiled(H, m, W, bias, inv, sel, sig)
    sel2, sig2 = nan_f32(m, 64), nan_f32(m, 64)
    step = 8 * L.lib.lkb_sm_count() - 5                       # ragged pieces, each within one 8-token CTA per SM
    for a in range(0, m, step):
        n = min(step, m - a)
        L.k_pf_router_tiled(H[a:a + n], n, W, bias, inv[a:a + n], sel2[a:a + n], sig2[a:a + n])
    assert torch.equal(sel, sel2) and torch.equal(sig, sig2) and bool(torch.isfinite(sel).all())


@pytest.mark.parametrize("m", [70, 300])
def test_router_and_select(L, orc, golden_dir, m):
    g = np.load(golden_dir / "router_fixture.npz")
    rng = np.random.default_rng(24 + m)
    H = rng.uniform(-1, 1, size=(m, 2048)).astype(np.float32)
    H[0] = g["h"]
    inv = rng.uniform(0.5, 2.0, size=m).astype(np.float32)
    inv[0] = 1.0
    W, bias = g["gate"], g["bias"]
    sel, sig = nan_f32(m, 64), nan_f32(m, 64)
    L.k_pf_router(dev(H), m, dev(W), dev(bias), dev(inv), sel, sig)       # small form for m <= 256, tiled above
    order = 0 if m <= 256 else 1
    ol = orc.pf_router_logits(H, W, inv, order)
    osel, osig = orc.pf_gate(ol, bias)
    assert np.max(ulp_diff(host(sig), osig)) <= 4                          # expf
    assert np.max(np.abs(host(sel) - osel)) <= 1e-6
    idx = torch.full((m, 4), -1, dtype=torch.int32, device="cuda")
    w = nan_f32(m, 4)
    L.k_pf_select(sel, sig, m, idx, w)
    oi, ow = orc.pf_select(host(sel), host(sig))                           # selection on the device's sel/sig: exact
    assert np.array_equal(host(idx), oi) and np.max(ulp_diff(host(w), ow)) <= 1
    assert host(idx)[0].tolist() == [59, 45, 58, 40]                       # the reference's fixture answer
    if m <= 256:
        # small form is bit-identical to the decode router (tests/test_prefill.cu:549-568)
        for t in (0, 1, m - 1):
            lg, s1, g1 = nan_f32(64), nan_f32(64), nan_f32(64)
            ssq = None
            L.k_router_dot(dev(H[t]), dev(W), lg, dev(bias), s1, g1, ssq, 0.0)
            if inv[t] == 1.0:
                assert np.array_equal(host(s1), host(sel)[t]) and np.array_equal(host(g1), host(sig)[t])
    # ids against an all-CPU run, allowing flips only at near-ties
    ci, _ = orc.pf_select(osel, osig)
    bad = np.nonzero(np.any(ci != host(idx), axis=1))[0]
    for t in bad:
        assert orc.router_margin(osel[t]) < 1e-5


SHAPES_DENSE = [(256, 64, 130, False, False, False), (384, 48, 200, True, True, False),
                (512, 8, 64, False, True, True), (256, 368, 70, True, False, False)]


@pytest.mark.parametrize("cfg", [0, 1])
@pytest.mark.parametrize("N,bpr,M,add,scale,three", SHAPES_DENSE)
def test_gemm_dense(L, orc, fold, cfg, N, bpr, M, add, scale, three):
    L.pf_gemm_config(cfg)
    rng = np.random.default_rng(N + bpr + M)
    qs, d = rand_q4(rng, N, bpr, "ref")
    X = act_floats(rng, M * bpr * 32).reshape(M, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    sc = rng.uniform(0.5, 2.0, size=M).astype(np.float32) if scale else None
    o0 = rng.uniform(-1, 1, size=(M, N)).astype(np.float32) if add else None
    if three:
        s0 = N // 3 // 128 * 128
        s1 = s0 + 128
        segs = [(qs[:s0], d[:s0]), (qs[s0:s1], d[s0:s1]), (qs[s1:], d[s1:])]
        seg_end = [s0, s1, N]
    else:
        segs, seg_end = [(qs, d)], [N, N, N]
    dsegs = [(dev(q_), dev(d_)) for q_, d_ in segs]
    out = dev(o0) if add else nan_f32(M, N)
    g = L.make_pf_gemm(dsegs, seg_end, N, bpr, dev(aq), dev(asc), ntok=M, scale=None if sc is None else dev(sc),
                       out=out, out_ld=N, add=int(add))
    L.pf_gemm_dense(g)
    ref, r64, mag, slack = orc.pf_gemm(segs, seg_end, N, bpr, aq, asc, ntok=M, scale=sc, out_init=o0, add=int(add),
                                       want_f64=True, want_slack=True)
    got = host(out)
    assert not np.any(np.isnan(got))
    assert np.array_equal(got, ref)                                   # block-order fp32: bit-exact
    s = np.ones((M, 1)) if sc is None else sc[:, None].astype(np.float64)
    full = r64 * s + (o0 if add else 0.0)
    assert _f64_gate(got, full, mag, slack, s, bpr, fold)
    assert L.lib.lkb_pf_gemm_status() == 0                  # no bounded wait of the tensor-core form expired
    L.pf_gemm_config(-1)


@pytest.mark.parametrize("cfg", [0, 1])
@pytest.mark.parametrize("E,rows,bpr,M,a_shift", [(8, 256, 64, 130, 2), (8, 384, 48, 257, 0), (64, 128, 8, 700, 2)])
def test_gemm_moe(L, orc, fold, ws, cfg, E, rows, bpr, M, a_shift):
    L.pf_gemm_config(cfg)
    rng = np.random.default_rng(E * rows + bpr + M)
    NS = M * 4
    arows = M if a_shift else NS
    qs, d = rand_q4(rng, E * rows, bpr, "ref")
    X = act_floats(rng, arows * bpr * 32).reshape(arows, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    idx = np.empty((M, 4), np.int32)                                    # skewed: some experts get many slots
    for t in range(M):
        got = []
        while len(got) < 4:
            e = int(rng.integers(E)) if rng.integers(3) == 0 else int(rng.integers(max(1, E // 4)))
            if e not in got:
                got.append(e)
        idx[t] = got
    cnt, off, tiles, ntiles, perm, max_tiles = _plan_dev(L, idx.reshape(-1))
    ocnt, ooff, otiles, operm = orc.moe_plan(idx.reshape(-1))
    sc = rng.uniform(0.5, 2.0, size=M).astype(np.float32) if a_shift else None
    out = nan_f32(NS, rows)                                             # NaN: every slot must be written
    dq, dd = dev(qs), dev(d)
    g = L.make_pf_gemm([(dq, dd)], [rows, rows, rows], rows, bpr, dev(aq), dev(asc), exp_stride=rows * bpr,
                       perm=perm, tiles=tiles, ntiles=ntiles, a_shift=a_shift,
                       scale=None if sc is None else dev(sc), out=out, out_ld=rows)
    L.pf_gemm_moe(g, max_tiles)
    ref, r64, mag, slack = orc.pf_gemm([(qs, d)], [rows, rows, rows], rows, bpr, aq, asc, exp_stride=rows * bpr,
                                       perm=operm, tiles=otiles, a_shift=a_shift, scale=sc, out_rows=NS, want_f64=True,
                                       want_slack=True)
    got = host(out)
    assert not np.any(np.isnan(got))
    assert np.array_equal(got, ref)
    s = np.ones((NS, 1)) if sc is None else np.repeat(sc, 4)[:, None].astype(np.float64)
    assert _f64_gate(got, r64 * s, mag, slack, s, bpr, fold)
    assert L.lib.lkb_pf_gemm_status() == 0                  # no bounded wait of the tensor-core form expired
    L.pf_gemm_config(-1)


@pytest.mark.parametrize("cfg", [0, 1])
def test_gemm_swiglu_fused_equals_unfused(L, orc, fold, ws, cfg):
    L.pf_gemm_config(cfg)
    rng = np.random.default_rng(31)
    E, I, bpr, M = 8, 256, 64, 150
    NS = M * 4
    gq, gd = rand_q4(rng, E * I, bpr, "ref")
    uq, ud = rand_q4(rng, E * I, bpr, "ref")
    X = act_floats(rng, M * bpr * 32).reshape(M, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    idx = np.stack([rng.choice(E, size=4, replace=False) for _ in range(M)]).astype(np.int32)
    cnt, off, tiles, ntiles, perm, max_tiles = _plan_dev(L, idx.reshape(-1))
    inv = rng.uniform(0.5, 2.0, size=M).astype(np.float32)
    dgq, dgd, duq, dud, daq, dasc, dinv = dev(gq), dev(gd), dev(uq), dev(ud), dev(aq), dev(asc), dev(inv)
    oqs, osc = _act_bufs(NS, I // 32)
    g = L.make_pf_gemm([(dgq, dgd), (duq, dud)], [I, I, I], I, bpr, daq, dasc, exp_stride=I * bpr, perm=perm,
                       tiles=tiles, ntiles=ntiles, a_shift=2, scale=dinv, oqs=oqs, osc=osc, okb=I // 32)
    L.pf_gemm_swiglu(g, max_tiles)
    # unfused: gate|up GEMM into fp32, then the SwiGLU quantiser
    Y = nan_f32(NS, 2 * I)
    g2 = L.make_pf_gemm([(dgq, dgd), (duq, dud)], [I, 2 * I, 2 * I], 2 * I, bpr, daq, dasc, exp_stride=I * bpr,
                        perm=perm, tiles=tiles, ntiles=ntiles, a_shift=2, scale=dinv, out=Y, out_ld=2 * I)
    L.pf_gemm_moe(g2, max_tiles)
    uqs, usc = _act_bufs(NS, I // 32)
    L.k_pf_swiglu(Y, 2 * I, I, I // 32, L.pf_act(uqs, usc), NS)
    Yh = host(Y)
    _, _, v = orc.pf_swiglu(Yh, I, I // 32)
    if fold:
        # shipped arithmetic: quants and d as the unfused path; the block sum in the reference's fused-epilogue order,
        # bit-exact against the checker's statement of that order on the device's own v
        assert torch.equal(oqs, uqs) and torch.equal(osc[..., 0], usc[..., 0])
        _sums_agree_to_fp16_rounding(host(osc)[..., 1], host(usc)[..., 1], host(usc)[..., 0])
    else:
        assert torch.equal(oqs, uqs) and torch.equal(osc, usc)             # quants, d AND sum identical
    # and against the checker on the device's own v (fast exp on the device)
    tq, tsc, _ = orc.pf_swiglu(Yh, I, I // 32, v=v)
    flips = np.count_nonzero(host(oqs) != tq)
    assert flips <= 1e-4 * tq.size and np.max(np.abs(host(oqs).astype(np.int32) - tq)) <= 1
    assert L.lib.lkb_pf_gemm_status() == 0                  # no bounded wait of the tensor-core form expired
    L.pf_gemm_config(-1)


def test_combine_and_combine_norm(L, orc):
    rng = np.random.default_rng(41)
    m = 33
    X = rng.standard_normal((m, 2048)).astype(np.float32)
    D = rng.standard_normal((m * 4, 2048)).astype(np.float32)
    w = rng.random((m, 4)).astype(np.float32)
    nw = (1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32)
    dX = dev(X)
    L.k_pf_moe_combine(dX, dev(D), dev(w), m)
    oX = orc.pf_combine(X, D, w)
    assert np.array_equal(host(dX), oX)
    dX2 = dev(X)
    qs, sc = _act_bufs(m, 64)
    inv = nan_f32(m)
    L.k_pf_moe_combine_norm(dX2, dev(D), dev(w), dev(nw), L.pf_act(qs, sc), inv, m)
    oX2, oq, osc, oinv = orc.pf_combine_norm(X, D, w, nw)
    assert np.array_equal(host(dX2), oX2) and np.array_equal(host(qs), oq) and np.array_equal(host(sc), osc)
    assert np.max(ulp_diff(host(inv), oinv)) <= 2
    # == combine followed by the split-form norm (tests/test_prefill.cu:808-830)
    qs3, sc3 = _act_bufs(m, 64)
    inv3 = nan_f32(m)
    L.k_pf_norm(dX, dev(nw), 0, L.pf_act(qs3, sc3), inv3, None, m)
    assert torch.equal(qs, qs3) and torch.equal(sc, sc3) and torch.equal(inv, inv3)


def test_prefill_moe_layer_small_config3(L, orc):
    """A 256-token slice of the 4096-token prefill configuration (Zipf-skewed routing), end to end."""
    rng = np.random.default_rng(51)
    m, H, I, E = 256, 2048, 1536, 64
    gq, gd = rand_q4(rng, E * I, 64)
    uq, ud = rand_q4(rng, E * I, 64)
    dq_, dd_ = rand_q4(rng, E * H, 48)
    Wr = (0.02 * rng.standard_normal((E, H))).astype(np.float32)
    bias = zipf_bias(rng, E, 1.1, 0.05)
    X = rng.standard_normal((m, H)).astype(np.float32)
    nw = (1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32)
    dX = dev(X)
    aqs, asc = _act_bufs(m, 64)
    inv, h32 = nan_f32(m), nan_f32(m, H)
    L.k_pf_norm(dX, dev(nw), 0, L.pf_act(aqs, asc), inv, h32, m)
    sel, sig = nan_f32(m, 64), nan_f32(m, 64)
    L.k_pf_router(h32, m, dev(Wr), dev(bias), inv, sel, sig)
    idx = torch.full((m, 4), -1, dtype=torch.int32, device="cuda")
    w = nan_f32(m, 4)
    L.k_pf_select(sel, sig, m, idx, w)
    cnt, off, tiles, ntiles, perm, max_tiles = _plan_dev(L, host(idx).reshape(-1))
    a2q, a2s = _act_bufs(m * 4, I // 32)
    dg = [dev(a) for a in (gq, gd, uq, ud, dq_, dd_)]
    g = L.make_pf_gemm([(dg[0], dg[1]), (dg[2], dg[3])], [I, I, I], I, 64, aqs, asc, exp_stride=I * 64, perm=perm,
                       tiles=tiles, ntiles=ntiles, a_shift=2, scale=inv, oqs=a2q, osc=a2s, okb=I // 32)
    L.pf_gemm_swiglu(g, max_tiles)
    D = nan_f32(m * 4, H)
    gd_ = L.make_pf_gemm([(dg[4], dg[5])], [H, H, H], H, 48, a2q, a2s, exp_stride=H * 48, perm=perm, tiles=tiles,
                         ntiles=ntiles, a_shift=0, out=D, out_ld=H)
    L.pf_gemm_moe(gd_, max_tiles)
    L.k_pf_moe_combine(dX, D, w, m)
    torch.cuda.synchronize()

    # checker on the device's routing + second-stage activations
    oi = host(idx)
    ocnt, ooff, otiles, operm = orc.moe_plan(oi.reshape(-1))
    assert np.array_equal(host(perm), operm)
    oD = orc.pf_gemm([(dq_, dd_)], [H, H, H], H, 48, host(a2q), host(a2s), exp_stride=H * 48, perm=operm,
                     tiles=otiles, a_shift=0, out_rows=m * 4)
    assert np.array_equal(host(D), oD)
    assert np.array_equal(host(dX), orc.pf_combine(X, oD, host(w)))
    # first stage against the checker with the device's inv
    oq, osc_, oinv, oh = orc.pf_norm(X, nw, plain=False, want_h32=True)
    assert np.array_equal(host(aqs), oq) and np.array_equal(host(asc), osc_)
    _, _, v = orc.pf_gemm_swiglu((gq, gd), (uq, ud), I, 64, oq, osc_, exp_stride=I * 64, perm=operm, tiles=otiles,
                                 a_shift=2, scale=host(inv), out_rows=m * 4)
    tq, _, _ = orc.pf_gemm_swiglu((gq, gd), (uq, ud), I, 64, oq, osc_, exp_stride=I * 64, perm=operm, tiles=otiles,
                                  a_shift=2, scale=host(inv), out_rows=m * 4, v=v)
    dq8 = host(a2q).astype(np.int32) - tq
    assert np.max(np.abs(dq8)) <= 1 and np.count_nonzero(dq8) <= 2e-4 * tq.size   # __expf vs libm exp near ties


def _sub_plan(operm, otiles, rng, per_tile=9):
    """A sub-plan for the checker: from every tile of the device's plan its first and last rows (the ragged tails) plus a
    few random ones, regrouped into tiles of the same experts.  A slot's GEMM row depends only on its own activation row
    and its expert's weights, so the checker's rows on the sub-plan must equal the device's rows on the full plan."""
    perm_sub, tiles_sub = [], []
    for e, start, count, _ in otiles:
        pick = {0, count - 1, count // 2}
        pick.update(int(v) for v in rng.integers(0, count, size=per_tile))
        rows = sorted(pick)
        tiles_sub.append((e, len(perm_sub), len(rows), 0))
        perm_sub.extend(int(operm[start + r]) for r in rows)
    return np.asarray(perm_sub, np.int32), np.asarray(tiles_sub, np.int32).reshape(-1, 4)


def test_gemm_moe_full_size_4096_tokens_zipf(L, orc):
    """The benchmark's configuration at full size: 4096 tokens x top-4 = 16384 slots over 64 experts with Zipf(1.1)-skewed
    routing, real layer shapes (gate|up 2 x 1536 x 2048 with the fused SwiGLU quantiser, down 2048 x 1536), through the
    tensor-core kernel on its workspace path.  Every slot row is checked on the device against the unfused form; more than
    2048 slots (first / middle / last row of every tile and random ones) bit for bit against the CPU checker."""
    rng = np.random.default_rng(4096)
    m, H, I, E = 4096, 2048, 1536, 64
    NS = m * 4
    gq, gd = rand_q4(rng, E * I, 64)
    uq, ud = rand_q4(rng, E * I, 64)
    dq_, dd_ = rand_q4(rng, E * H, 48)
    # routing: Zipf(1.1) load over the experts, four distinct experts per token
    p = 1.0 / (rng.permutation(E) + 1.0) ** 1.1
    p /= p.sum()
    idx = np.stack([rng.choice(E, size=4, replace=False, p=p) for _ in range(m)]).astype(np.int32)
    X = act_floats(rng, m * H).reshape(m, H)
    aq, asc = orc.pf_quant_rows(X, 64)
    inv = rng.uniform(0.5, 2.0, size=m).astype(np.float32)
    cnt, off, tiles, ntiles, perm, max_tiles = _plan_dev(L, idx.reshape(-1))
    ocnt, ooff, otiles, operm = orc.moe_plan(idx.reshape(-1))
    assert np.array_equal(host(perm), operm) and np.array_equal(host(cnt), ocnt)
    assert ocnt.max() > 4 * ocnt[ocnt > 0].min()                         # the load really is skewed
    wsb = torch.zeros(L.pf_gemm_workspace_bytes(max_tiles, H), dtype=torch.uint8, device="cuda")
    L.pf_gemm_set_workspace(wsb)
    L.pf_gemm_config(1)
    dg = [dev(a) for a in (gq, gd, uq, ud, dq_, dd_)]
    daq, dasc, dinv = dev(aq), dev(asc), dev(inv)
    a2q, a2s = _act_bufs(NS, I // 32)
    g = L.make_pf_gemm([(dg[0], dg[1]), (dg[2], dg[3])], [I, I, I], I, 64, daq, dasc, exp_stride=I * 64, perm=perm,
                       tiles=tiles, ntiles=ntiles, a_shift=2, scale=dinv, oqs=a2q, osc=a2s, okb=I // 32)
    L.pf_gemm_swiglu(g, max_tiles)
    Y = nan_f32(NS, 2 * I)
    g2 = L.make_pf_gemm([(dg[0], dg[1]), (dg[2], dg[3])], [I, 2 * I, 2 * I], 2 * I, 64, daq, dasc, exp_stride=I * 64,
                        perm=perm, tiles=tiles, ntiles=ntiles, a_shift=2, scale=dinv, out=Y, out_ld=2 * I)
    L.pf_gemm_moe(g2, max_tiles)
    uqs, usc = _act_bufs(NS, I // 32)
    L.k_pf_swiglu(Y, 2 * I, I, I // 32, L.pf_act(uqs, usc), NS)
    # all 16384 slots: fused == unfused in quants and d; the block sums in the shipped fused-epilogue order, against the checker
    assert torch.equal(a2q, uqs) and torch.equal(a2s[..., 0], usc[..., 0])
    _sums_agree_to_fp16_rounding(host(a2s)[..., 1], host(usc)[..., 1], host(usc)[..., 0])
    D = nan_f32(NS, H)
    gd_ = L.make_pf_gemm([(dg[4], dg[5])], [H, H, H], H, 48, a2q, a2s, exp_stride=H * 48, perm=perm, tiles=tiles,
                         ntiles=ntiles, a_shift=0, out=D, out_ld=H)
    L.pf_gemm_moe(gd_, max_tiles)
    torch.cuda.synchronize()
    assert L.lib.lkb_pf_gemm_status() == 0
    gotY, gotD = host(Y), host(D)
    assert not np.any(np.isnan(gotY)) and not np.any(np.isnan(gotD))

    sperm, stiles = _sub_plan(operm, otiles, rng)
    assert sperm.size >= 2048 and np.unique(sperm).size == sperm.size
    oY = orc.pf_gemm([(gq, gd), (uq, ud)], [I, 2 * I, 2 * I], 2 * I, 64, aq, asc, exp_stride=I * 64, perm=sperm, tiles=stiles,
                     a_shift=2, scale=inv, out_rows=NS)
    assert np.array_equal(gotY[sperm], oY[sperm])                        # gate|up rows, bit for bit
    oD = orc.pf_gemm([(dq_, dd_)], [H, H, H], H, 48, host(a2q), host(a2s), exp_stride=H * 48, perm=sperm, tiles=stiles,
                     a_shift=0, out_rows=NS)
    assert np.array_equal(gotD[sperm], oD[sperm])                        # down rows, bit for bit
    L.pf_gemm_set_workspace(None)
    L.pf_gemm_config(-1)


@pytest.mark.parametrize("m", [1, 70, 256, 300, 1500, 2500, 4096])
def test_router_and_selection_in_one_launch(L, m):
    """lkb_pf_router_select == lkb_pf_router followed by lkb_pf_select, every CTA shape of the tiled form and the short form."""
    rng = np.random.default_rng(900 + m)
    H = dev(rng.standard_normal((m, 2048)).astype(np.float32))
    W = dev((0.02 * rng.standard_normal((64, 2048))).astype(np.float32))
    bias = dev(zipf_bias(rng, 64, 1.1, 0.05))
    inv = dev(rng.uniform(0.5, 2.0, size=m).astype(np.float32))
    for small in ((True, False) if m <= 256 else (False,)):
        sel, sig = nan_f32(m, 64), nan_f32(m, 64)
        idx, w = torch.full((m, 4), -1, dtype=torch.int32, device="cuda"), nan_f32(m, 4)
        (L.k_pf_router_small if small else L.k_pf_router_tiled)(H, m, W, bias, inv, sel, sig)
        L.k_pf_select(sel, sig, m, idx, w)
        sel2, sig2 = nan_f32(m, 64), nan_f32(m, 64)
        idx2, w2 = torch.full((m, 4), -1, dtype=torch.int32, device="cuda"), nan_f32(m, 4)
        L.k_pf_router_select(H, m, small, W, bias, inv, sel2, sig2, idx2, w2)
        torch.cuda.synchronize()
        assert torch.equal(sel, sel2) and torch.equal(sig, sig2) and torch.equal(idx, idx2) and torch.equal(w, w2)
