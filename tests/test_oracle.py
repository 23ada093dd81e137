"""CPU-only checks of the oracle: against the reference's own known-answer
pruning cases, against an independent float64 numpy rendering, and against the
fixtures recorded from the reference engine."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as O
from helpers import rel_fro, make_problem, oracle_preprocess, baseline_scale

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _csr_from_dense(d):
    d = np.asarray(d, dtype=np.float32)
    rp, ci, va = [0], [], []
    for row in d:
        nz = np.nonzero(row)[0]
        ci += list(nz)
        va += list(row[nz])
        rp.append(len(ci))
    return np.array(va, np.float32), np.array(ci, np.int32), np.array(rp, np.int64)


# The four cases of cc/cuda_lrm_npeff/src/preprocess/column_pruning_test.cc:12-105
# (same pruning scheme as cc/cuda_d_npeff/src/util/sparse_util.h:79-159).
_M1 = [[1, 0, 0, -4, 0], [0, 2, 0, -.5, 0], [0, 4, 0, -.5, 0]]
_M2 = [[1, 0, 0, -4, 0], [0, 0, 1, 0, .5], [0, 4, 0, -.5, 0]]
PRUNE_KAT = [
    (_M1, 1, [[1, 0, -4], [0, 2, -.5], [0, 4, -.5]], [0, 1, 3]),
    (_M1, 2, [[0, -4], [2, -.5], [4, -.5]], [1, 3]),
    (_M1, 3, [[-4], [-.5], [-.5]], [3]),
    (_M2, 2, [[-4], [0], [-.5]], [3]),  # a row emptied by pruning stays as an empty row
]


@pytest.mark.parametrize("dense,min_count,expected,new_to_old", PRUNE_KAT)
def test_prune_known_answers(dense, min_count, expected, new_to_old):
    va, ci, rp = _csr_from_dense(dense)
    v2, c2, rp2, n2o = O.prune_columns(va, ci, rp, 5, min_count)
    ev, ec, erp = _csr_from_dense(expected)
    assert np.array_equal(n2o, np.array(new_to_old, np.int32))
    assert np.array_equal(rp2, erp)
    assert np.array_equal(c2, ec)
    assert np.array_equal(v2, ev)


def test_split_ranges_match_reference_rule():
    # getSizeOfSplit: floor(total/n) each, the last takes the remainder
    assert [O.split_range(10, 3, i) for i in range(3)] == [(0, 3), (3, 3), (6, 4)]
    assert [O.split_range(8, 4, i) for i in range(4)] == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert O.split_range(5, 1, 0) == (0, 5)


def test_split_columns_partitions_matrix():
    vals, idx, norms = make_problem(20, 97, 13, seed=3)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, 97)
    m = len(n2o)
    total = 0
    for s in range(3):
        c0, w = O.split_range(m, 3, s)
        sv, sc, srp = O.split_columns(v, c, rp, c0, w)
        total += len(sv)
        assert sc.min(initial=0) >= 0 and sc.max(initial=0) < w
        # within-row order preserved
        for i in range(20):
            row = c[rp[i]:rp[i + 1]]
            keep = (row >= c0) & (row < c0 + w)
            assert np.array_equal(sc[srp[i]:srp[i + 1]], row[keep] - c0)
    assert total == len(v)


def test_csc_is_stable_transpose():
    vals, idx, norms = make_problem(30, 64, 9, seed=5)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, 64)
    m = len(n2o)
    cv, cr, cp = O.csr_to_csc(v, c, rp, m)
    rows = np.repeat(np.arange(30), np.diff(rp))
    order = np.lexsort((rows, c))
    assert np.array_equal(cr, rows[order])
    assert np.array_equal(cv, v[order])
    assert np.array_equal(np.diff(cp), np.bincount(c, minlength=m))


def test_init_uniform_range_and_shard_invariance():
    full = O.init_uniform(0, 1000, 42, 1, 0.5)
    assert full.min() > 0 and full.max() <= 0.5
    part = O.init_uniform(300, 200, 42, 1, 0.5)
    assert np.array_equal(part, full[300:500])
    assert not np.array_equal(O.init_uniform(0, 1000, 42, 0, 0.5), full)


@pytest.mark.parametrize("n,m,k,r,eps", [(48, 300, 24, 6, 1e-12), (64, 512, 64, 8, 1e-8)])
def test_oracle_matches_numpy_float64(n, m, k, r, eps):
    vals, idx, norms = make_problem(n, m, k, seed=n)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, 0, baseline_scale(v, n, mk, r))
    Wn, Hn, ln = O.numpy_run(v, c, rp, mk, W0, H0, 30, eps)
    W1, H1, l1 = O.run(v, c, rp, mk, W0, H0, 30, eps, acc64=True, losses=True)
    # float32 storage against float64 everywhere: 1e-5 is ample, 1e-4 is the target
    assert rel_fro(W1, Wn) < 1e-5 and rel_fro(H1, Hn) < 1e-5
    assert np.max(np.abs(l1 - ln) / ln) < 1e-6
    W2, H2, l2 = O.run(v, c, rp, mk, W0, H0, 30, eps, acc64=False, losses=True)
    assert rel_fro(W2, Wn) < 1e-4 and rel_fro(H2, Hn) < 1e-4
    assert np.max(np.abs(l2 - ln) / ln) < 1e-5
    assert abs(O.loss(v, c, rp, mk, W1, H1) - l1[-1]) < 1e-9 * l1[-1]


def test_fit_w_only_matches_numpy():
    n, m, k, r = 40, 200, 16, 5
    vals, idx, norms = make_problem(n, m, k, seed=9)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, 3, 1.0)
    rng = np.random.default_rng(0)
    H0 = (H0 * (rng.random(H0.shape) > 0.9)).astype(np.float32)
    A = np.zeros((n, mk))
    np.add.at(A, (np.repeat(np.arange(n), np.diff(rp)), c), v.astype(np.float64))
    W = W0.astype(np.float64)
    AH, HH = A @ H0.T.astype(np.float64), H0.astype(np.float64) @ H0.T.astype(np.float64)
    for _ in range(25):
        W *= AH / (W @ HH + 1e-7)
    Wo, lo = O.fit_w_only(v, c, rp, mk, W0, H0, 25, 1e-7)
    assert rel_fro(Wo, W) < 1e-5
    assert abs(lo - np.linalg.norm(A - W @ H0)) < 1e-5 * lo


def test_sharded_update_equals_unsharded():
    """Summing per-shard A_d*H_d^T and H_d*H_d^T partials reproduces the unsharded W update."""
    n, m, k, r = 32, 240, 20, 4
    vals, idx, norms = make_problem(n, m, k, seed=21)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, 1, 0.1)
    AH = np.zeros((n, r))
    HH = np.zeros((r, r))
    for s in range(3):
        c0, w = O.split_range(mk, 3, s)
        sv, sc, srp = O.split_columns(v, c, rp, c0, w)
        Hs = H0[:, c0:c0 + w]
        AH += O.spmm(sv, sc, srp, np.ascontiguousarray(Hs.T)).astype(np.float64)
        HH += O.gram(np.ascontiguousarray(Hs.T)).astype(np.float64)
    Wsh = O.mu_update(W0, AH.astype(np.float32), HH.astype(np.float32), 1e-8)
    Wun = O.step_w(v, c, rp, mk, W0, H0, 1e-8)
    assert rel_fro(Wsh, Wun) < 1e-6


# ---- fixtures recorded from the reference engine itself ---------------------
_REF_CASES = sorted(glob.glob(os.path.join(GOLDEN, "ref_case_*.npz")))


@pytest.mark.skipif(not _REF_CASES, reason="no reference-engine fixtures recorded yet")
@pytest.mark.parametrize("path", _REF_CASES, ids=[os.path.basename(p) for p in _REF_CASES])
def test_oracle_matches_reference_engine(path):
    g = np.load(path)
    n, m, k, r = int(g["n"]), int(g["m"]), int(g["k"]), int(g["rank"])
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    v, c, rp, n2o = O.prune_columns(g["in_vals"], g["in_col"], rowptr, m, int(g["min_count"]))
    # integer work: bit-exact against removeSmallestL0NormColumns_inPlace
    assert np.array_equal(n2o, g["new_to_og"])
    assert np.array_equal(rp, g["p_rowptr"].astype(np.int64))
    assert np.array_equal(c, g["p_col"])
    assert np.array_equal(v, g["p_vals"])
    mk = len(n2o)
    # float work from the reference's own initial factors.  The reference sums
    # in cuSPARSE/cuBLAS order in fp32; 1e-4 relative Frobenius is the stated bar.
    W, H, ls = O.run(v, c, rp, mk, g["W0"], g["H0"], int(g["iters"]), float(g["eps"]),
                     acc64=True, losses=True)
    assert rel_fro(W, g["W"]) < 1e-4
    assert rel_fro(H, g["H"]) < 1e-4
    # the reference adds its three loss terms in fp32, so its printed loss
    # carries ~1e-4 of cancellation noise; compare at 1e-3.
    assert abs(ls[-1] - float(g["loss"])) < 1e-3 * ls[-1]
    assert abs(O.loss(v, c, rp, mk, g["W0"], g["H0"]) - float(g["loss0"])) < 1e-3 * float(g["loss0"])


def test_retain_columns_known_answer_and_properties():
    """RetainColumns_InPlace (src/cuda/host/sparse_matrix.h:141-170) worked by hand:
    new index = position in the list, other entries dropped, row order kept."""
    #      col: 0    1    2    3    4
    # row 0:   1.        2.        3.
    # row 1:        4.
    # row 2:   5.   6.        7.
    vals = np.array([1, 2, 3, 4, 5, 6, 7], np.float32)
    col = np.array([0, 2, 4, 1, 0, 1, 3], np.int32)
    rp = np.array([0, 3, 4, 7], np.int64)
    v, c, p = O.retain_columns(vals, col, rp, 5, [4, 0, 3])
    assert v.tolist() == [1, 3, 5, 7] and c.tolist() == [1, 0, 1, 2] and p.tolist() == [0, 2, 2, 4]
    # a repeated id keeps its last position; an id with no entries is simply an empty column
    v, c, p = O.retain_columns(vals, col, rp, 5, [1, 2, 1])
    assert v.tolist() == [2, 4, 6] and c.tolist() == [1, 2, 2] and p.tolist() == [0, 1, 2, 3]
    # retaining the pruning's own kept list reproduces the pruning
    vals2, idx2, norms2 = make_problem(40, 500, 30, seed=4)
    pv, pc, prp, n2o = oracle_preprocess(vals2, idx2, norms2, 500, 2)
    rowptr = np.arange(41, dtype=np.int64) * 30
    nv = O.normalize_rows(vals2.ravel(), rowptr, norms2)
    rv, rc, rrp = O.retain_columns(nv, idx2.ravel(), rowptr, 500, n2o)
    assert np.array_equal(rv, pv) and np.array_equal(rc, pc) and np.array_equal(rrp, prp)


def test_dense_to_csr_thresholding():
    A = np.array([[0.5, 0.0, 0.2], [0.0, 0.0, 0.0], [0.1, 0.3, 0.3]], np.float32)
    v, rp, c = O.dense_to_csr(A, 0.2)
    assert v.tolist() == pytest.approx([0.5, 0.2, 0.3, 0.3]) and rp.tolist() == [0, 2, 2, 4] and c.tolist() == [0, 2, 1, 2]
    assert rp.dtype == np.int64 and c.dtype == np.int32


# ---------------------------------------------------------------------------
# Hoyer projection (DenseFactorSparsityContext::sparsifyF).  The reference never runs
# it, so the pins are the published operator's own properties and a plain
# per-vector float64 restatement of the published algorithm.
def _hoyer_vector_f64(x, l1, l2):
    """Hoyer 2004, section 3.3, one vector, float64."""
    x = np.asarray(x, dtype=np.float64)
    n = x.size
    s = x + (l1 - x.sum()) / n
    z = np.zeros(n, dtype=bool)
    for _ in range(n + 1):
        m = np.where(z, 0.0, l1 / (n - z.sum()))
        d = s - m
        a, b, c = (d * d).sum(), (m * d).sum(), (m * m).sum() - l2 * l2
        alpha = (-b + np.sqrt(max(0.0, b * b - a * c))) / max(a, 1e-30)
        s = m + alpha * d
        if (s >= 0).all():
            return s
        z |= s < 0
        s[z] = 0.0
        s[~z] -= (s.sum() - l1) / (n - z.sum())
    return s


@pytest.mark.parametrize("n,r,sparseness", [(50, 3, 0.3), (400, 8, 0.6), (1000, 5, 0.9), (64, 16, 0.75)])
def test_hoyer_projection_properties(n, r, sparseness):
    rng = np.random.default_rng(n + r)
    W = rng.random((n, r), dtype=np.float32)
    l2 = 1.0
    l1 = (np.sqrt(n) - (np.sqrt(n) - 1.0) * sparseness) * l2
    S, passes, conv = O.hoyer_project(W, l1, l2, rule=0)
    assert conv and 1 <= passes <= n + 1
    assert S.dtype == np.float32 and S.min() >= 0
    assert np.allclose(S.astype(np.float64).sum(axis=0), l1, rtol=2e-5)
    assert np.allclose(np.sqrt((S.astype(np.float64) ** 2).sum(axis=0)), l2, rtol=2e-5)
    # the same answer as the published algorithm, vector by vector in float64
    for t in range(r):
        want = _hoyer_vector_f64(W[:, t], l1, l2)
        assert np.allclose(S[:, t], want, rtol=1e-4, atol=2e-6)
    # a projected vector is a fixed point
    S2, p2, c2 = O.hoyer_project(S, l1, l2, rule=0)
    assert c2 and np.allclose(S2, S, rtol=1e-4, atol=2e-6)


def test_hoyer_reference_alpha_rule_keeps_l1_and_sign_only():
    """The reference's kernel_computeAlpha expression (rule 1) is not the root of the
    quadratic: the result is non-negative with the requested L1 norm, but its L2 norm is
    not the requested one.  Recorded so that the difference between the two rules stays visible."""
    rng = np.random.default_rng(3)
    W = rng.random((500, 8), dtype=np.float32)
    S, passes, conv = O.hoyer_project(W, 8.0, 1.0, rule=1, max_passes=200)
    assert conv and S.min() >= 0
    assert np.allclose(S.astype(np.float64).sum(axis=0), 8.0, rtol=2e-5)
    assert np.all(np.sqrt((S.astype(np.float64) ** 2).sum(axis=0)) > 1.2)


def test_hoyer_empty_and_degenerate():
    S, p, c = O.hoyer_project(np.zeros((0, 4), np.float32), 2.0)
    assert S.shape == (0, 4) and p == 0 and c
    # one row: the only vector with that L1 norm
    S, p, c = O.hoyer_project(np.array([[0.3, 0.9]], np.float32), 2.0, 1.0)
    assert c and np.allclose(S, 2.0)


def test_host_generator_twin_properties():
    """oracle.synth_pef_hashed (the host twin of the device generator the benchmark
    uses): k distinct columns per row, values descending and non-negative, norms = L2
    norms, deterministic in the seed, Zipf head present in (nearly) every row, and a
    row's content independent of how many rows are generated."""
    n, m, k = 24, 20000, 1024
    v, i, nr = O.synth_pef_hashed(n, m, k, alpha=1.1, sigma=1.0, seed=5)
    assert i.min() >= 0 and i.max() < m
    for row in range(n):
        assert len(np.unique(i[row])) == k
        assert np.all(np.diff(v[row]) <= 0) and v[row, -1] >= 0
    assert np.allclose(nr, np.sqrt((v.astype(np.float64) ** 2).sum(1)), rtol=1e-6)
    assert np.mean([(0 in set(r_)) for r_ in i]) > 0.9
    v2, i2, nr2 = O.synth_pef_hashed(n, m, k, alpha=1.1, sigma=1.0, seed=5)
    assert np.array_equal(v, v2) and np.array_equal(i, i2) and np.array_equal(nr, nr2)
    v3, i3, _ = O.synth_pef_hashed(7, m, k, alpha=1.1, sigma=1.0, seed=5)
    assert np.array_equal(v3, v[:7]) and np.array_equal(i3, i[:7])
    v4, i4, _ = O.synth_pef_hashed(n, m, k, alpha=1.1, sigma=1.0, seed=6)
    assert not np.array_equal(i4, i)
    # k == m: every column, whatever the draws
    v5, i5, _ = O.synth_pef_hashed(3, 64, 64, seed=1)
    assert all(sorted(r_) == list(range(64)) for r_ in i5)


def test_problem_steps_match_run():
    """oracle.Problem (what the timed CPU arm iterates) against oracle.run on the same
    preprocessed matrix and seeded factors."""
    n, m, k, r = 40, 3000, 100, 8
    v, i, nr = O.synth_pef_hashed(n, m, k, seed=2)
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    vn = O.normalize_rows(v.ravel(), rowptr, nr)
    pv, pc, prp, n2o = O.prune_columns(vn, i.ravel(), rowptr, m, 1)
    mk = len(n2o)
    scale = float(np.float32(np.sqrt(pv.astype(np.float64).sum() / (n * mk) / r)))
    W0, H0 = O.init_factors(n, mk, r, 2, scale)
    _, _, ls = O.run(pv, pc, prp, mk, W0, H0, 3, 1e-12, acc64=False, losses=True)
    P = O.Problem(n, m, k, r, v, i, nr, min_count=1, eps=1e-12, seed=2)
    assert P.m_kept == mk
    for step in range(3):
        P.step(acc64=False)
        assert abs(P.loss() - ls[step]) < 1e-6 * ls[step]
    P.close()
