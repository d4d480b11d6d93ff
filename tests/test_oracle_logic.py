"""Host-side logic of the checker: plan/scatter properties, GEMM vs GEMV consistency (CPU only)."""
import numpy as np

from helpers import act_floats, rand_q4


def test_plan_scatter_properties(orc):
    rng = np.random.default_rng(5)
    for m in (1, 63, 64, 65, 700):
        idx = np.stack([rng.choice(64, size=4, replace=False) for _ in range(m)]).astype(np.int32).reshape(-1)
        cnt, off, tiles, perm = orc.moe_plan(idx)
        assert cnt.sum() == m * 4 and np.array_equal(off, np.concatenate([[0], np.cumsum(cnt)[:-1]]))
        assert np.array_equal(np.sort(perm), np.arange(m * 4))
        e = idx[perm]
        assert np.all((e[1:] > e[:-1]) | ((e[1:] == e[:-1]) & (perm[1:] > perm[:-1])))
        assert np.all(tiles[:, 2] > 0) and np.all(tiles[:, 2] <= 64) and tiles[:, 2].sum() == m * 4
        assert np.all(np.diff(tiles[:, 0]) >= 0)                  # expert order
        for ex, st, c, _ in tiles:
            assert np.all(idx[perm[st:st + c]] == ex)


def test_gemm_rows_equal_gemv_terms(orc):
    """Block-order GEMM and lane-order GEMV agree to fp32 reassociation.  Exact per-block term: both within 1e-5
    of float64.  The reference's shipped (folded) term: within the reference's own gate -- beyond the rounding
    that form is allowed (half an ulp of c per block), 2e-6 * max(1, bpr/16) of the summed magnitudes
    (tests/test_prefill.cu:61-83,129-134 of the reference)."""
    rng = np.random.default_rng(6)
    N, bpr, M = 128, 64, 5
    qs, d = rand_q4(rng, N, bpr)
    X = act_floats(rng, M * bpr * 32).reshape(M, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    try:
        orc.set_gemm_fold(False)
        out, o64, mag = orc.pf_gemm([(qs, d)], [N, N, N], N, bpr, aq, asc, ntok=M, want_f64=True)
        orc.set_gemm_fold(True)
        outf, o64f, magf, slack = orc.pf_gemm([(qs, d)], [N, N, N], N, bpr, aq, asc, ntok=M, want_f64=True, want_slack=True)
    finally:
        orc.set_gemm_fold(True)
    assert np.array_equal(o64, o64f) and not np.array_equal(out, outf)
    assert np.all(np.maximum(0.0, np.abs(outf - o64) - slack) <= 2e-6 * max(1, bpr // 16) * mag)
    for t in range(M):
        act = orc.quantize_q8_1(X[t])
        y = orc.gemv_q4_0(qs, d, act, N, bpr)
        y64, m2 = orc.gemv_q4_0_f64(qs, d, act, N, bpr)
        assert np.allclose(o64[t], y64, rtol=0, atol=1e-12) and np.allclose(mag[t], m2)
        assert np.all(np.abs(out[t] - y64) <= 1e-5 * m2) and np.all(np.abs(y - y64) <= 1e-5 * m2)


def test_fused_swiglu_equals_unfused_in_checker(orc):
    rng = np.random.default_rng(7)
    I, bpr, M = 64, 8, 6
    gq, gd = rand_q4(rng, I, bpr)
    uq, ud = rand_q4(rng, I, bpr)
    X = act_floats(rng, M * bpr * 32).reshape(M, bpr * 32)
    aq, asc = orc.pf_quant_rows(X, bpr)
    oqs, osc, v = orc.pf_gemm_swiglu((gq, gd), (uq, ud), I, bpr, aq, asc, ntok=M)
    Y = orc.pf_gemm([(gq, gd), (uq, ud)], [I, 2 * I, 2 * I], 2 * I, bpr, aq, asc, ntok=M)
    uqs, usc, _ = orc.pf_swiglu(Y, I, I // 32)
    assert np.array_equal(oqs, uqs) and np.array_equal(osc, usc)
