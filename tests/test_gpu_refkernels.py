"""Parity of this library's kernels with the REFERENCE's own CUDA kernels, run side by side on the same B200.

oracle/_ref/libref_kernels.so holds the reference's src/kernels.cu and src/prefill.cu compiled unchanged for
sm_100a (oracle/Makefile, target ref_kernels; launch shapes of the reference's own call sites, oracle/ref_shim.cu).
Both libraries get the same device buffers; outputs are compared byte for byte wherever the reference fixes the
arithmetic sequence, and within the reference's own gates where it leaves it to the compiler (FMA contraction in
dot_q4_0_q8_1, src/quant.cuh:154-157) or where this library picked a different, documented summation order.
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


@pytest.fixture(scope="module")
def R():
    import importlib
    rk = importlib.import_module("oracle.ref_kernels")
    if not rk.available():
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference checkout at build time)")
    return rk


def _act_bufs(rows, kb):
    return (torch.full((rows, kb * 32), 0x5A, dtype=torch.int8, device="cuda"), nan_f32(rows, kb, 2))


def _same(a, b):
    return torch.equal(a.view(torch.uint8).reshape(-1), b.view(torch.uint8).reshape(-1))


def test_quantiser_and_norms_memcmp(L, R, orc):
    rng = np.random.default_rng(301)
    x = act_floats(rng, 64 * 32)
    x[0:32] = 0.0
    x[32:64] = np.linspace(-3e-4, 3e-4, 32)
    x[64:96] = np.arange(32, dtype=np.float32) - 15.5
    dx = dev(x)
    y0, y1 = empty_blocks(64), empty_blocks(64)
    L.k_quantize_q8_1(dx, y0, 64)
    R.quantize_q8_1(dx, y1, 64)
    assert _same(y0, y1)
    w = dev((1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32))
    a32, b32 = nan_f32(2048), nan_f32(2048)
    a16, b16 = torch.zeros(2048, dtype=torch.float16, device="cuda"), torch.zeros(2048, dtype=torch.float16, device="cuda")
    aq, bq = empty_blocks(64), empty_blocks(64)
    L.k_rmsnorm_q8_1(dx, w, 2048, 1e-5, a32, a16, aq)
    R.rmsnorm_q8_1(dx, w, 2048, 1e-5, b32, b16, bq)
    assert _same(a32, b32) and _same(a16, b16) and _same(aq, bq)
    # per-token prefill norm, both forms, against the reference's k_pf_norm
    m = 37
    X = dev(act_floats(rng, m * 2048).reshape(m, 2048))
    for plain in (1, 0):
        q0, s0 = _act_bufs(m, 64)
        q1, s1 = _act_bufs(m, 64)
        i0, i1, h0, h1 = nan_f32(m), nan_f32(m), nan_f32(m, 2048), nan_f32(m, 2048)
        L.k_pf_norm(X, w, plain, L.pf_act(q0, s0), i0, None if plain else h0, m)
        R.pf_norm(X, w, plain, q1, s1, i1, None if plain else h1, m)
        assert _same(q0, q1) and _same(s0, s1) and _same(i0, i1)
        if not plain:
            assert _same(h0, h1)


@pytest.mark.parametrize("rows,bpr,wide", [(2048, 64, 1), (6144, 64, 0), (2048, 48, 1), (512, 368, 0)])
def test_gemv_against_reference_kernel(L, R, orc, rows, bpr, wide):
    """Configuration 0 and the other decode GEMV shapes.  Same lane-strided block order and butterfly; the reference
    leaves the per-block term's contraction to nvcc, so equality of bits is recorded, not demanded: the bar is
    1e-5 of sum|terms| (and both sides against float64)."""
    rng = np.random.default_rng(rows + bpr)
    qs, d = rand_q4(rng, rows, bpr)
    act = orc.quantize_q8_1(act_floats(rng, bpr * 32))
    xq, dq, dd = dev(orc.pack_blocks(*act)), dev(qs), dev(d)
    y0, y1 = nan_f32(rows), nan_f32(rows)
    L.k_gemv_q4_0(dq, dd, xq, rows, bpr, y0, 0, None, 0.0)
    R.gemv_q4_0(dq, dd, xq, rows, bpr, y1, 0, None, 0.0, wide)
    y64, mag = orc.gemv_q4_0_f64(qs, d, act, rows, bpr)
    a, b = host(y0), host(y1)
    assert np.all(np.abs(a - b) <= 1e-5 * mag) and np.all(np.abs(b - y64) <= 1e-5 * mag)
    print(f"gemv {rows}x{bpr * 32}: bit-identical to the reference kernel: {np.array_equal(a, b)}; max ulp {int(ulp_diff(a, b).max())}")


def test_router_against_reference_kernel(L, R, golden_dir):
    g = np.load(golden_dir / "router_fixture.npz")
    h, W, bias = dev(g["h"]), dev(g["gate"]), dev(g["bias"])
    l0, l1 = nan_f32(64), nan_f32(64)
    L.k_router_dot(h, W, l0, bias, None, None, None, 0.0)
    R.router_dot(h, W, l1, bias, None, None, None, 0.0)
    assert _same(l0, l1)
    i0 = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    i1 = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    w0, w1 = nan_f32(4), nan_f32(4)
    L.k_router_top4(l0, bias, i0, w0)
    R.router_top4(l1, bias, i1, w1)
    assert host(i0).tolist() == [59, 45, 58, 40] and _same(i0, i1)
    assert np.max(ulp_diff(host(w0), host(w1))) <= 1
    # many random inputs, including exact ties of the ranking value: ids identical
    rng = np.random.default_rng(302)
    for t in range(24):
        hv = rng.uniform(-1, 1, 2048).astype(np.float32)
        if t % 4 == 0:
            hv[:] = 0.0                                   # all logits equal: the tie rule decides everything
        l0.fill_(float("nan")); l1.fill_(float("nan"))
        bz = torch.zeros(64, device="cuda") if t % 4 == 0 else bias
        L.k_router_dot(dev(hv), W, l0, bz, None, None, None, 0.0)
        R.router_dot(dev(hv), W, l1, bz, None, None, None, 0.0)
        L.k_router_top4(l0, bz, i0, w0)
        R.router_top4(l1, bz, i1, w1)
        assert _same(l0, l1) and _same(i0, i1) and np.max(ulp_diff(host(w0), host(w1))) <= 1


def test_moe_decode_layer_against_reference_kernels(L, R, orc):
    """Configuration 1 through both kernel sets: gate|up GEMV of the four selected experts, SwiGLU + Q8_1, down
    projection + weighted sum + residual + the next layer's quantised activation."""
    rng = np.random.default_rng(303)
    E, I, H = 64, 1536, 2048
    gq, gd = rand_q4(rng, E * I, 64)
    uq, ud = rand_q4(rng, E * I, 64)
    wq, wd = rand_q4(rng, E * H, 48)
    act = orc.quantize_q8_1(act_floats(rng, H))
    xq = dev(orc.pack_blocks(*act))
    idx = dev(np.array([59, 3, 17, 40], np.int32))
    wk = dev(np.array([0.3, 0.28, 0.22, 0.2], np.float32))
    dg = [dev(a) for a in (gq, gd, uq, ud, wq, wd)]
    ya0, yb0, ya1, yb1 = nan_f32(4 * I), nan_f32(4 * I), nan_f32(4 * I), nan_f32(4 * I)
    L.k_gemv_q4_0_exp2(dg[0], dg[1], dg[2], dg[3], xq, I, 64, I, 0, idx, ya0, yb0, None, 0.0)
    R.gemv_q4_0_exp2(dg[0], dg[1], dg[2], dg[3], xq, I, 64, I, 0, idx, ya1, yb1, None, 0.0)
    scale = float(np.abs(host(ya1)).mean()) * 64
    assert np.all(np.abs(host(ya0) - host(ya1)) <= 1e-5 * scale) and np.all(np.abs(host(yb0) - host(yb1)) <= 1e-5 * scale)
    print("gate|up bit-identical to the reference kernel:", _same(ya0, ya1) and _same(yb0, yb1))
    # SwiGLU + Q8_1 on identical inputs (the reference's gate|up output): __expf and the quantiser must agree bit for bit
    q0, q1 = empty_blocks(4 * I // 32), empty_blocks(4 * I // 32)
    L.k_swiglu(ya1, yb1, 4 * I, None, q0)
    R.swiglu(ya1, yb1, 4 * I, None, q1)
    assert _same(q0, q1)
    # down + accumulate + producer on identical inputs
    x0 = rng.standard_normal(H).astype(np.float32)
    nw = dev((1.0 + 0.05 * rng.standard_normal(H)).astype(np.float32))
    xa, xb = dev(x0), dev(x0)
    na, nb = empty_blocks(64), empty_blocks(64)
    sa, sb = nan_f32(64), nan_f32(64)
    L.k_moe_down_accum(dg[4], dg[5], q1, H, 48, H, 48, idx, wk, xa, L.norm_prod(nw, None, na, sa))
    R.moe_down_accum(dg[4], dg[5], q1, H, 48, H, 48, idx, wk, xb, nw, None, nb, sb)
    a, b = host(xa), host(xb)
    assert np.all(np.abs(a - b) <= 1e-5 * np.maximum(1.0, np.abs(b)))
    same = _same(xa, xb)
    print("down+accumulate bit-identical to the reference kernel:", same)
    if same:
        assert _same(na, nb) and _same(sa, sb)


@pytest.mark.parametrize("m,skew", [(70, 1), (700, 1), (4096, 2), (257, 3)])
def test_plan_against_reference_kernels(L, R, m, skew):
    rng = np.random.default_rng(304 + m)
    if skew == 3:
        idx = np.tile(np.array([7, 8, 40, 63], np.int32), (m, 1))
    else:
        p = np.ones(64) if skew == 1 else 1.0 / (rng.permutation(64) + 1.0) ** 1.1
        p /= p.sum()
        idx = np.stack([rng.choice(64, size=4, replace=False, p=p) for _ in range(m)]).astype(np.int32)
    ns = m * 4
    d_idx = dev(idx.reshape(-1))
    max_tiles = ns // 64 + 64

    def bufs():
        return (torch.zeros(64, dtype=torch.int32, device="cuda"), torch.full((64,), -1, dtype=torch.int32, device="cuda"),
                torch.full((max_tiles, 4), -1, dtype=torch.int32, device="cuda"), torch.full((1,), -1, dtype=torch.int32, device="cuda"),
                torch.full((ns,), -1, dtype=torch.int32, device="cuda"))
    c0, o0, t0, n0, p0 = bufs()
    c1, o1, t1, n1, p1 = bufs()
    L.k_pf_moe_count(d_idx, ns, c0)
    L.k_pf_moe_plan(c0, o0, t0, n0)
    L.k_pf_moe_scatter(d_idx, ns, o0, p0)
    R.pf_moe_plan(d_idx, ns, c1, o1, t1, n1, p1)
    nt = int(host(n1)[0])
    assert _same(c0, c1) and _same(o0, o1) and _same(n0, n1) and _same(p0, p1)
    assert np.array_equal(host(t0)[:nt], host(t1)[:nt])


def _routing(rng, M, E):
    idx = np.empty((M, 4), np.int32)
    for t in range(M):
        got = []
        while len(got) < 4:
            e = int(rng.integers(E)) if rng.integers(3) == 0 else int(rng.integers(max(1, E // 4)))
            if e not in got:
                got.append(e)
        idx[t] = got
    return idx


@pytest.mark.parametrize("cfg", [0, 1, 2])
@pytest.mark.parametrize("E,rows,bpr,M,a_shift", [(8, 256, 64, 130, 2), (8, 384, 48, 257, 0), (64, 128, 8, 700, 2)])
def test_gemm_moe_memcmp_reference_kernel(L, R, orc, cfg, E, rows, bpr, M, a_shift):
    """pf_gemm_moe: the default (folded) per-block term is the reference kernel's own arithmetic -> identical bytes.
    cfg 0: CUDA-core form; 1: tensor-core form, rows gathered in the kernel; 2: tensor-core form with a workspace."""
    wsbuf = None
    if cfg == 2:
        wsbuf = torch.zeros(L.pf_gemm_workspace_bytes(M * 4 // 64 + 64, bpr * 32), dtype=torch.uint8, device="cuda")
        cfg = 1
    L.pf_gemm_set_workspace(wsbuf)
    L.pf_gemm_config(cfg)
    L.pf_gemm_arith(1)
    rng = np.random.default_rng(E * rows + bpr + M + 7)
    NS = M * 4
    arows = M if a_shift else NS
    qs, d = rand_q4(rng, E * rows, bpr, "ref")
    X = act_floats(rng, arows * bpr * 32).reshape(arows, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    idx = _routing(rng, M, E)
    d_idx = dev(idx.reshape(-1))
    max_tiles = NS // 64 + 64
    cnt = torch.zeros(64, dtype=torch.int32, device="cuda")
    off = torch.full((64,), -1, dtype=torch.int32, device="cuda")
    tiles = torch.full((max_tiles, 4), -1, dtype=torch.int32, device="cuda")
    ntiles = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    perm = torch.full((NS,), -1, dtype=torch.int32, device="cuda")
    R.pf_moe_plan(d_idx, NS, cnt, off, tiles, ntiles, perm)
    sc = dev(rng.uniform(0.5, 2.0, size=M).astype(np.float32)) if a_shift else None
    dq, dd, daq, dasc = dev(qs), dev(d), dev(aq), dev(asc)
    o0, o1 = nan_f32(NS, rows), nan_f32(NS, rows)
    g0 = L.make_pf_gemm([(dq, dd)], [rows, rows, rows], rows, bpr, daq, dasc, exp_stride=rows * bpr, perm=perm, tiles=tiles,
                        ntiles=ntiles, a_shift=a_shift, scale=sc, out=o0, out_ld=rows)
    g1 = L.make_pf_gemm([(dq, dd)], [rows, rows, rows], rows, bpr, daq, dasc, exp_stride=rows * bpr, perm=perm, tiles=tiles,
                        ntiles=ntiles, a_shift=a_shift, scale=sc, out=o1, out_ld=rows)
    L.pf_gemm_moe(g0, max_tiles)
    R.pf_gemm_moe(g1, max_tiles)
    torch.cuda.synchronize()
    assert not bool(torch.isnan(o1).any())
    assert _same(o0, o1)
    assert L.lib.lkb_pf_gemm_status() == 0
    L.pf_gemm_config(-1)
    L.pf_gemm_set_workspace(None)


@pytest.mark.parametrize("cfg", [0, 1])
def test_gemm_dense_and_swiglu_against_reference_kernel(L, R, orc, cfg):
    L.pf_gemm_config(cfg)
    L.pf_gemm_arith(1)
    rng = np.random.default_rng(305)
    # dense, three segments, residual add, row scale
    N, bpr, M = 384, 64, 200
    qs, d = rand_q4(rng, N, bpr, "ref")
    aq, asc = orc.pf_quant_rows(act_floats(rng, M * bpr * 32).reshape(M, bpr * 32), bpr)
    segs = [(dev(qs[:128]), dev(d[:128])), (dev(qs[128:256]), dev(d[128:256])), (dev(qs[256:]), dev(d[256:]))]
    sc = dev(rng.uniform(0.5, 2.0, size=M).astype(np.float32))
    init = rng.uniform(-1, 1, size=(M, N)).astype(np.float32)
    o0, o1 = dev(init), dev(init)
    daq, dasc = dev(aq), dev(asc)
    L.pf_gemm_dense(L.make_pf_gemm(segs, [128, 256, 384], N, bpr, daq, dasc, ntok=M, scale=sc, out=o0, out_ld=N, add=1))
    R.pf_gemm_dense(L.make_pf_gemm(segs, [128, 256, 384], N, bpr, daq, dasc, ntok=M, scale=sc, out=o1, out_ld=N, add=1))
    torch.cuda.synchronize()
    assert _same(o0, o1)
    # fused SwiGLU epilogue: quants, d AND the block sum identical -- the reference sums the 32 values of a block in
    # another order there than in its stand-alone quantiser (rows paired 8, 16, 1, 2, 4 apart; it gates the two against
    # each other within fp16 steps, tests/test_prefill.cu:788-800), and shipped arithmetic follows the fused order.
    # 38400 blocks: an order mismatch would show in about twenty of them
    E, I, M = 8, 512, 600
    NS = M * 4
    gq, gd = rand_q4(rng, E * I, bpr, "ref")
    uq, ud = rand_q4(rng, E * I, bpr, "ref")
    aq, asc = orc.pf_quant_rows(act_floats(rng, M * bpr * 32).reshape(M, bpr * 32), bpr)
    idx = np.stack([rng.choice(E, size=4, replace=False) for _ in range(M)]).astype(np.int32)
    d_idx = dev(idx.reshape(-1))
    max_tiles = NS // 64 + 64
    cnt = torch.zeros(64, dtype=torch.int32, device="cuda")
    off = torch.full((64,), -1, dtype=torch.int32, device="cuda")
    tiles = torch.full((max_tiles, 4), -1, dtype=torch.int32, device="cuda")
    ntiles = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    perm = torch.full((NS,), -1, dtype=torch.int32, device="cuda")
    R.pf_moe_plan(d_idx, NS, cnt, off, tiles, ntiles, perm)
    inv = dev(rng.uniform(0.5, 2.0, size=M).astype(np.float32))
    dw = [(dev(gq), dev(gd)), (dev(uq), dev(ud))]
    daq, dasc = dev(aq), dev(asc)
    q0, s0 = _act_bufs(NS, I // 32)
    q1, s1 = _act_bufs(NS, I // 32)
    L.pf_gemm_swiglu(L.make_pf_gemm(dw, [I, I, I], I, bpr, daq, dasc, exp_stride=I * bpr, perm=perm, tiles=tiles, ntiles=ntiles,
                                    a_shift=2, scale=inv, oqs=q0, osc=s0, okb=I // 32), max_tiles)
    R.pf_gemm_swiglu(L.make_pf_gemm(dw, [I, I, I], I, bpr, daq, dasc, exp_stride=I * bpr, perm=perm, tiles=tiles, ntiles=ntiles,
                                    a_shift=2, scale=inv, oqs=q1, osc=s1, okb=I // 32), max_tiles)
    torch.cuda.synchronize()
    assert _same(q0, q1) and _same(s0, s1)
    assert L.lib.lkb_pf_gemm_status() == 0
    L.pf_gemm_config(-1)


def test_batched_router_select_combine_against_reference_kernels(L, R, golden_dir):
    g = np.load(golden_dir / "router_fixture.npz")
    rng = np.random.default_rng(306)
    W, bias = dev(g["gate"]), dev(g["bias"])
    for m in (70, 300):
        H = dev(rng.uniform(-1, 1, size=(m, 2048)).astype(np.float32))
        inv = dev(rng.uniform(0.5, 2.0, size=m).astype(np.float32))
        s0, g0, s1, g1 = nan_f32(m, 64), nan_f32(m, 64), nan_f32(m, 64), nan_f32(m, 64)
        L.k_pf_router(H, m, W, bias, inv, s0, g0)
        R.pf_router(H, m, W, bias, inv, s1, g1)
        if m <= 256:
            assert _same(s0, s1) and _same(g0, g1)            # the small form is the decode router's arithmetic
        else:
            assert np.max(np.abs(host(s0) - host(s1))) <= 1e-5    # the tiled forms order the 2048 terms differently
        i0 = torch.full((m, 4), -1, dtype=torch.int32, device="cuda")
        i1 = torch.full((m, 4), -1, dtype=torch.int32, device="cuda")
        w0, w1 = nan_f32(m, 4), nan_f32(m, 4)
        L.k_pf_select(s1, g1, m, i0, w0)                      # the same sel / sig into both selections
        R.pf_select(s1, g1, m, i1, w1)
        assert _same(i0, i1) and np.max(ulp_diff(host(w0), host(w1))) <= 1
        # combine and combine + norm
        X = rng.standard_normal((m, 2048)).astype(np.float32)
        D = dev(rng.standard_normal((m * 4, 2048)).astype(np.float32))
        nw = dev((1.0 + 0.05 * rng.standard_normal(2048)).astype(np.float32))
        xa, xb = dev(X), dev(X)
        L.k_pf_moe_combine(xa, D, w1, m)
        R.pf_moe_combine(xb, D, w1, m)
        assert _same(xa, xb)
        xa, xb = dev(X), dev(X)
        qa, sa = _act_bufs(m, 64)
        qb, sb = _act_bufs(m, 64)
        ia, ib = nan_f32(m), nan_f32(m)
        L.k_pf_moe_combine_norm(xa, D, w1, nw, L.pf_act(qa, sa), ia, m)
        R.pf_moe_combine_norm(xb, D, w1, nw, qb, sb, ib, m)
        assert _same(xa, xb) and _same(qa, qb) and _same(sa, sb) and _same(ia, ib)
