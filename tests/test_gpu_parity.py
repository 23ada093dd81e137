"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU
oracle on the same seeded inputs.  Integer / index work must be bit-exact;
floating-point results must agree within the tolerances written beside each
assert (the stated targets: factors 1e-4 relative Frobenius after 50 iterations
from identical initial factors, loss 1e-5 relative)."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

from oracle import oracle as O
from helpers import rel_fro, make_problem, oracle_preprocess, baseline_scale

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


def _dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _engine(params, keep_csr=False, **kw):
    """An engine; `keep_csr` keeps the shard's CSR in input order for export_shard_csr
    (the loader drops that intermediate by default)."""
    from npeff_ref_b200 import MuNmf
    eng = MuNmf(params, **kw)
    if keep_csr:
        eng.set_option("keep_canonical_csr", 1)
    return eng


def _csr_random(rng, rows, cols, lens):
    ptr = np.zeros(rows + 1, dtype=np.int64)
    ptr[1:] = np.cumsum(lens)
    ind = np.concatenate([rng.choice(cols, size=l, replace=False) for l in lens] +
                         [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    vals = rng.random(int(ptr[-1]), dtype=np.float32)
    return vals, ind, ptr


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("r", [4, 8, 32, 48, 64, 128, 256, 512, 5, 130])
def test_op_spmm_matches_oracle(torch_cuda, r):
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(r)
    rows, cols = 300, 900
    # empty rows, rows of 1, rows around the 32-entry chunk, rows past the
    # warp/block threshold (1024) with ragged tails
    lens = rng.integers(0, 70, size=rows)
    lens[:8] = [0, 1, 31, 32, 33, 900, 700, 0]
    vals, ind, ptr = _csr_random(rng, rows, cols, lens)
    big_cols = 5000
    lens2 = np.array([0, 1025, 4097, 3000, 1024, 5000], dtype=np.int64)
    v2, i2, p2 = _csr_random(rng, len(lens2), big_cols, lens2)
    for (va, ia, pa, nc) in ((vals, ind, ptr, cols), (v2, i2, p2, big_cols)):
        D = rng.random((nc, r), dtype=np.float32)
        want = O.spmm(va, ia, pa, D, acc64=True)
        out = torch.full((len(pa) - 1, r), float("nan"), device="cuda")
        dv, di, dp, dD = _dev(torch, va), _dev(torch, ia), _dev(torch, pa), _dev(torch, D)
        st = torch.cuda.current_stream().cuda_stream
        check(lib().dnpeff_op_spmm(dv.data_ptr(), di.data_ptr(), dp.data_ptr(), len(pa) - 1,
                                   dD.data_ptr(), r, out.data_ptr(), st))
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        # fp32 chains of up to ~1000 sequential positive terms against float64:
        # a few sqrt(1000) * 2^-24 relative, bounded here by 1e-5
        assert np.allclose(got, want, rtol=1e-5, atol=1e-7), np.abs(got / np.maximum(want, 1e-30) - 1).max()
        # repeatable bit for bit
        out2 = torch.empty_like(out)
        check(lib().dnpeff_op_spmm(dv.data_ptr(), di.data_ptr(), dp.data_ptr(), len(pa) - 1,
                                   dD.data_ptr(), r, out2.data_ptr(), st))
        torch.cuda.synchronize()
        assert torch.equal(out, out2)


@pytest.mark.parametrize("rows,r", [(1, 4), (1000, 32), (5000, 64), (777, 48), (20000, 128),
                                    (3001, 256), (2500, 512), (40007, 384), (100, 5), (0, 16), (0, 256), (1, 256), (65, 512)])
def test_op_gram_matches_oracle(torch_cuda, rows, r):
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(rows + r)
    X = rng.random((rows, r), dtype=np.float32)
    want = O.gram(X, acc64=True) if rows > 0 else np.zeros((r, r), np.float32)
    G = torch.full((r, r), float("nan"), device="cuda")
    dX = _dev(torch, X) if rows > 0 else torch.zeros((1, r), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(lib().dnpeff_op_gram(dX.data_ptr(), rows, r, G.data_ptr(), st))
    torch.cuda.synchronize()
    got = G.cpu().numpy()
    # fp32 partial sums folded in double: 3e-6 relative to the largest entry
    assert np.abs(got - want).max() <= 3e-6 * max(np.abs(want).max(), 1e-30)
    assert np.array_equal(got, got.T)


@pytest.mark.parametrize("rows,r", [(1, 4), (513, 32), (300, 64), (1000, 48), (4099, 128),
                                    (700, 256), (200, 512), (3000, 384), (50, 5), (64, 516),
                                    (40001, 128), (60000, 64),    # several tiles per block
                                    (1, 128), (100, 64), (127, 128), (129, 64)])  # fewer rows than a tile
def test_op_mu_update_matches_oracle(torch_cuda, rows, r):
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(rows * 7 + r)
    X = rng.random((rows, r), dtype=np.float32)
    Num = rng.random((rows, r), dtype=np.float32)
    B = rng.random((r + 3, r), dtype=np.float32)
    G = (B.T @ B).astype(np.float32)
    want = O.mu_update(X, Num, G, 1e-8, acc64=True)
    dX, dN, dG = _dev(torch, X), _dev(torch, Num), _dev(torch, G)
    st = torch.cuda.current_stream().cuda_stream
    check(lib().dnpeff_op_mu_update(dX.data_ptr(), dN.data_ptr(), dG.data_ptr(), rows, r, 1e-8, st))
    torch.cuda.synchronize()
    got = dX.cpu().numpy()
    # one fp32 dot of length r against float64, then the same fp32 elementwise rule
    assert np.allclose(got, want, rtol=3e-6, atol=0), np.abs(got / want - 1).max()


@pytest.mark.parametrize("rows,r", [(1000, 128), (20000, 64), (300, 32), (257, 256)])
def test_op_mu_update_zero_and_tiny_numerators(torch_cuda, rows, r):
    """Numerators that are exactly zero or below 2^-100, and rows of X that are zero (their
    denominators are then eps alone): the tensor-core update kernels of ranks 64 and 128
    leave their branch-free division for the IEEE one on such batches; every kernel must
    still give the reference's x * (num / (den + eps))."""
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(rows + r)
    X = rng.random((rows, r), dtype=np.float32)
    Num = rng.random((rows, r), dtype=np.float32)
    Num[rng.random((rows, r)) < 0.05] = 0.0
    Num[rng.random((rows, r)) < 0.05] = np.float32(3e-36)
    X[::7] = 0.0
    B = rng.random((r + 3, r), dtype=np.float32)
    G = (B.T @ B).astype(np.float32)
    want = O.mu_update(X, Num, G, 1e-8, acc64=True)
    dX, dN, dG = _dev(torch, X), _dev(torch, Num), _dev(torch, G)
    st = torch.cuda.current_stream().cuda_stream
    check(lib().dnpeff_op_mu_update(dX.data_ptr(), dN.data_ptr(), dG.data_ptr(), rows, r, 1e-8, st))
    torch.cuda.synchronize()
    got = dX.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.array_equal(got == 0, want == 0)
    assert np.allclose(got, want, rtol=3e-6, atol=1e-44), np.abs(got - want).max()


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("min_count", [1, 2, 3])
@pytest.mark.parametrize("n_shards", [1, 3])
def test_loader_bit_exact(torch_cuda, min_count, n_shards):
    """normalise -> prune -> column split -> CSR/CSC against the oracle, bit for bit."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k = 150, 2000, 70
    vals, idx, norms = make_problem(n, m, k, seed=100 + min_count)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m, min_count)
    mk = len(n2o)
    for s in range(n_shards):
        with _engine(MuNmfParams(rank=8), keep_csr=True, shard_index=s, n_shards=n_shards) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, min_count)
            nn, mkept, c0, ms, nnz = eng.shape
            assert (nn, mkept) == (n, mk)
            assert (c0, ms) == O.split_range(mk, n_shards, s)
            assert np.array_equal(eng.new_to_og(), n2o)
            sv, sc, srp = O.split_columns(v, c, rp, c0, ms)
            gv, gc, grp = eng.export_shard_csr()
            assert nnz == len(sv)
            assert np.array_equal(grp, srp)
            assert np.array_equal(gc, sc)
            assert np.array_equal(gv, sv)  # includes the fp32 division by (norm + 1e-9f)
            cv, cr, cp = O.csr_to_csc(sv, sc, srp, ms)
            hv, hr, hp = eng.export_shard_csc()
            assert np.array_equal(hp, cp)
            assert np.array_equal(hr, cr)
            assert np.array_equal(hv, cv)
            assert abs(eng.a_sq_norm() - float((sv.astype(np.float64) ** 2).sum())) < 1e-9 * max(nnz, 1)


def test_loader_cyclic_sharding_bit_exact(torch_cuda):
    """Cyclic sharding: engine d owns kept columns d, d+G, ...; same entries, same order."""
    from npeff_ref_b200 import MuNmfParams, MuNmf
    n, m, k, G = 90, 1500, 60, 3
    vals, idx, norms = make_problem(n, m, k, seed=8)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m, 2)
    mk = len(n2o)
    rows = np.repeat(np.arange(n), np.diff(rp))
    seen = np.zeros(mk, dtype=bool)
    for d in range(G):
        with _engine(MuNmfParams(rank=8, seed=4, init_scale=0.5), keep_csr=True, shard_index=d, n_shards=G,
                     shard_mode=MuNmf.CYCLIC) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, 2)
            kept_ids, og_ids = eng.shard_columns()
            assert np.array_equal(kept_ids, np.arange(d, mk, G))
            assert np.array_equal(og_ids, n2o[kept_ids])
            seen[kept_ids] = True
            sel = (c % G) == d
            gv, gc, grp = eng.export_shard_csr()
            assert np.array_equal(gc, c[sel] // G) and np.array_equal(gv, v[sel])
            assert np.array_equal(np.diff(grp), np.bincount(rows[sel], minlength=n))
            eng.init_factors()
            _, H0 = O.init_factors(n, mk, 8, 4, 0.5)
            assert np.array_equal(eng.load_h_to_host(), H0[:, kept_ids])
    assert seen.all()


def test_loader_ragged_rows_and_empty_rows(torch_cuda):
    from npeff_ref_b200 import MuNmfParams
    rng = np.random.default_rng(5)
    n, m = 130, 500
    lens = rng.integers(0, 40, size=n)
    lens[[0, 7, 129]] = 0
    vals, ind, ptr = _csr_random(rng, n, m, lens)
    v, c, rp, n2o = O.prune_columns(vals, ind, ptr, m, 2)
    with _engine(MuNmfParams(rank=4), keep_csr=True) as eng:
        eng.set_csr(n, m, vals, ind, ptr, 0, None, 2)
        assert np.array_equal(eng.new_to_og(), n2o)
        gv, gc, grp = eng.export_shard_csr()
        assert np.array_equal(grp, rp) and np.array_equal(gc, c) and np.array_equal(gv, v)
        cv, cr, cp = O.csr_to_csc(v, c, rp, len(n2o))
        hv, hr, hp = eng.export_shard_csc()
        assert np.array_equal(hp, cp) and np.array_equal(hr, cr) and np.array_equal(hv, cv)


def test_loader_rejects_bad_input(torch_cuda):
    from npeff_ref_b200 import MuNmfParams, DnpeffError
    with _engine(MuNmfParams(rank=4)) as eng:
        vals = np.ones(6, np.float32)
        with pytest.raises(DnpeffError) as ei:
            eng.set_csr(2, 10, vals, np.array([0, 1, 2, 3, 4, 10], np.int32), None, 3)
        assert ei.value.code == -4
        eng.set_csr(2, 10, vals, np.array([0, 1, 1, 3, 4, 5], np.int32), None, 3)
        eng.init_factors()
        eng.step_w()
        with pytest.raises(DnpeffError) as ei:  # duplicate column inside a row
            eng.step_h()
        assert ei.value.code == -4


def test_seeded_init_bit_exact(torch_cuda):
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r = 40, 300, 20, 8
    vals, idx, norms = make_problem(n, m, k, seed=1)
    for s in range(2):
        with _engine(MuNmfParams(rank=r, seed=99, init_scale=0.25), shard_index=s, n_shards=2) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, 1)
            eng.init_factors()
            _, mk, c0, ms, _ = eng.shape
            W0, H0 = O.init_factors(n, ms, r, 99, 0.25, col_start=c0)
            assert np.array_equal(eng.load_w_to_host(), W0)
            assert np.array_equal(eng.load_h_to_host(), H0)


@pytest.mark.parametrize("M,K,r", [(1, 1, 32), (127, 63, 64), (128, 64, 128), (129, 65, 96), (1000, 777, 128),
                                   (20000, 300, 32), (5000, 4100, 128), (300, 9000, 64),
                                   (700, 1000, 256), (129, 300, 512), (2000, 640, 384)])
def test_op_block_product_matches_float64(torch_cuda, M, K, r):
    """The tensor-core kernel of the dense popular block on its own: C = X Y against a
    float64 product, with the sparsity and value range of a popular block (a quarter
    of X non-zero), ragged tiles and K chunks, several K splits."""
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(M * 31 + K * 7 + r)
    X = (rng.random((M, K), dtype=np.float32) * (rng.random((M, K)) < 0.25)).astype(np.float32)
    Y = rng.random((K, r), dtype=np.float32)
    want = X.astype(np.float64) @ Y.astype(np.float64)
    dX, dY = _dev(torch, X), _dev(torch, Y)
    C_ = torch.full((M, r), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    check(lib().dnpeff_op_block_product(dX.data_ptr(), M, K, dY.data_ptr(), r, C_.data_ptr(), st))
    torch.cuda.synchronize()
    got = C_.cpu().numpy()
    # fp32-equivalent: relative to each row's scale (sum of |x||y|), 3xTF32 leaves ~1e-6
    scale = np.abs(X).astype(np.float64) @ np.abs(Y).astype(np.float64)
    assert np.all(np.isfinite(got))
    assert np.abs(got - want).max() <= 2e-6 * max(scale.max(), 1e-30)
    # twice the same bits
    C2 = torch.empty((M, r), device="cuda")
    check(lib().dnpeff_op_block_product(dX.data_ptr(), M, K, dY.data_ptr(), r, C2.data_ptr(), st))
    torch.cuda.synchronize()
    assert np.array_equal(C2.cpu().numpy(), got)


# ---------------------------------------------------------------------------
CASES = [
    # n, m, k, r, iters, eps
    (64, 700, 40, 8, 50, 1e-12),
    (256, 6000, 300, 32, 50, 1e-12),     # configuration 1's shape, scaled down 8x
    (96, 9000, 1500, 128, 50, 1e-8),     # long rows (block kernel), r = 128 > n: near-exact fit
    (300, 9000, 1500, 128, 50, 1e-12),   # long rows, r = 128 < n
    (80, 3000, 200, 20, 30, 1e-8),       # rank not a power of two
    (50, 400, 30, 7, 20, 1e-8),          # odd rank: generic kernels
    (300, 6000, 800, 256, 20, 1e-12),    # wide rank: the panelled tensor-core update kernel
]


@pytest.mark.parametrize("n,m,k,r,iters,eps", CASES)
def test_full_run_matches_oracle(torch_cuda, n, m, k, r, iters, eps):
    from npeff_ref_b200 import MuNmfParams
    vals, idx, norms = make_problem(n, m, k, seed=n + r)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    with _engine(MuNmfParams(rank=r, eps=eps, seed=0, init_scale=scale)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        eng.init_factors()
        W0, H0 = eng.load_w_to_host(), eng.load_h_to_host()
        Wo0, Ho0 = O.init_factors(n, mk, r, 0, scale)
        assert np.array_equal(W0, Wo0) and np.array_equal(H0, Ho0)
        l0 = eng.compute_uncached_loss()
        assert abs(l0 - O.loss(v, c, rp, mk, W0, H0)) < 1e-5 * l0
        # single half steps
        eng.step_w()
        W1 = eng.load_w_to_host()
        assert rel_fro(W1, O.step_w(v, c, rp, mk, W0, H0, eps)) < 2e-6
        eng.step_h()
        H1 = eng.load_h_to_host()
        assert rel_fro(H1, O.step_h(v, c, rp, mk, W1, H0, eps)) < 2e-6
        # full run from identical initial factors
        eng.init_factors(W0, H0)
        eng.run(iters, log_every=0)
        W, H = eng.load_w_to_host(), eng.load_h_to_host()
        Wo, Ho, ls = O.run(v, c, rp, mk, W0, H0, iters, eps, acc64=True, losses=True)
        assert rel_fro(W, Wo) < 1e-4, rel_fro(W, Wo)      # stated target
        assert rel_fro(H, Ho) < 1e-4, rel_fro(H, Ho)
        l = eng.compute_uncached_loss()
        # The loss is sqrt(|A|^2 + pos - 2 neg): its squared form is accurate to a
        # relative 3e-6 of |A|^2 (the tensor-core Gram products accumulate 64-K runs with
        # truncation, a uniform -1.1e-6 relative bias on each of the two factors of pos);
        # the stated 1e-5 relative target on the loss itself applies where the fit is
        # not near-exact (no catastrophic cancellation).
        a2 = float((v.astype(np.float64) ** 2).sum())
        assert abs(l * l - ls[-1] ** 2) < 3e-6 * a2
        if ls[-1] ** 2 > 0.05 * a2:
            assert abs(l - ls[-1]) < 1e-5 * ls[-1]        # stated target
        assert np.all(np.isfinite(W)) and np.all(np.isfinite(H))
        assert W.min() >= 0 and H.min() >= 0


def test_popular_block_is_dense_and_matches_oracle(torch_cuda):
    """Ranks 32..128 (multiples of 32) keep the popular columns as a dense block
    for the tensor-core kernel (layout reports tile_rows == 0): several row tiles
    and K splits, one half step each way against the oracle."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r, eps = 700, 20000, 2000, 64, 1e-12
    vals, idx, norms = make_problem(n, m, k, seed=123)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    with _engine(MuNmfParams(rank=r, eps=eps, seed=2, init_scale=scale)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        n_pop, pop_nnz, n_blocks, tile_rows = eng.layout()
        assert n_pop > 128 and pop_nnz > 0 and tile_rows == 0
        eng.init_factors()
        W0, H0 = eng.load_w_to_host(), eng.load_h_to_host()
        eng.step_w()
        W1 = eng.load_w_to_host()
        assert rel_fro(W1, O.step_w(v, c, rp, mk, W0, H0, eps)) < 2e-6
        eng.step_h()
        H1 = eng.load_h_to_host()
        Ho1 = O.step_h(v, c, rp, mk, W1, H0, eps)
        assert rel_fro(H1, Ho1) < 2e-6
        # element-wise too: a popular column must not differ from a tail column in accuracy
        assert np.max(np.abs(H1 - Ho1) / (np.abs(Ho1) + 1e-30)) < 1e-4
        # the H update built only the tail part of the CSC; the export completes it
        cv, cr, cp = O.csr_to_csc(v, c, rp, mk)
        hv, hr, hp = eng.export_shard_csc()
        assert np.array_equal(hp, cp) and np.array_equal(hr, cr) and np.array_equal(hv, cv)
    # a rank outside the tensor-core set keeps the sparse tiled kernel
    with _engine(MuNmfParams(rank=48, eps=eps, seed=2, init_scale=scale)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        assert eng.layout()[3] > 0


def test_run_is_repeatable_bit_for_bit(torch_cuda):
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r = 128, 4000, 1200, 64
    vals, idx, norms = make_problem(n, m, k, seed=77)
    outs = []
    for _ in range(2):
        with _engine(MuNmfParams(rank=r, eps=1e-8, seed=5, init_scale=0.01)) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, 1)
            eng.init_factors()
            eng.run(10, log_every=0)
            outs.append((eng.load_w_to_host(), eng.load_h_to_host()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])


def test_fit_w_only_matches_oracle(torch_cuda):
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r = 300, 2000, 100, 32
    vals, idx, norms = make_problem(n, m, k, seed=31)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    rng = np.random.default_rng(3)
    W0, H0 = O.init_factors(n, mk, r, 3, 1.0)
    H0 = (H0 * (rng.random(H0.shape) > 0.9)).astype(np.float32)  # 90 % of H zeroed
    with _engine(MuNmfParams(rank=r, eps=1e-7)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        eng.init_factors(W0, H0)
        loss = eng.fit_w_only(200)
        W = eng.load_w_to_host()
    Wo, lo = O.fit_w_only(v, c, rp, mk, W0, H0, 200, 1e-7)
    assert rel_fro(W, Wo) < 1e-4
    assert abs(loss - lo) < 1e-5 * lo


def test_sharded_engines_match_unsharded_w_update(torch_cuda):
    """Two shards on one device, the exchange emulated on the host: the summed
    partial A_d*H_d^T / H_d*H_d^T give the unsharded W update (column sharding
    needs no other exchange; the H update is local to a shard)."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r, eps = 100, 3000, 150, 16, 1e-8
    vals, idx, norms = make_problem(n, m, k, seed=55)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, 9, 0.05)
    Hs = []
    for s in range(2):
        with _engine(MuNmfParams(rank=r, eps=eps, seed=9, init_scale=0.05), shard_index=s, n_shards=2) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, 1)
            eng.init_factors()
            _, _, c0, ms, _ = eng.shape
            assert np.array_equal(eng.load_h_to_host(), H0[:, c0:c0 + ms])
            # H update needs only the shard: run it with the oracle's new W
            W1 = O.step_w(v, c, rp, mk, W0, H0, eps)
            eng.init_factors(W1, H0[:, c0:c0 + ms])
            eng.step_h()
            Hs.append(eng.load_h_to_host())
    H1 = O.step_h(v, c, rp, mk, W1, H0, eps)
    assert rel_fro(np.concatenate(Hs, axis=1), H1) < 2e-6


def test_synthetic_generator_properties(torch_cuda):
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    n, m, k = 64, 50000, 2048
    vals = torch.empty((n, k), dtype=torch.float32, device="cuda")
    idx = torch.empty((n, k), dtype=torch.int32, device="cuda")
    norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        check(lib().dnpeff_synth_pef_device(n, m, k, 1.1, 1.0, 7, vals.data_ptr(), idx.data_ptr(),
                                            norms.data_ptr(), st))
    v, i, nr = vals.cpu().numpy(), idx.cpu().numpy(), norms.cpu().numpy()
    assert i.min() >= 0 and i.max() < m
    for row in range(n):
        assert len(np.unique(i[row])) == k                      # distinct columns
        assert np.all(np.diff(v[row]) <= 0) and v[row, -1] >= 0  # descending, non-negative
    assert np.allclose(nr, np.sqrt((v.astype(np.float64) ** 2).sum(1)), rtol=1e-6)
    # Zipf: the most popular columns are in (nearly) every row
    assert np.mean([(0 in set(r_)) for r_ in i]) > 0.95
    vals2 = torch.empty_like(vals)
    idx2 = torch.empty_like(idx)
    check(lib().dnpeff_synth_pef_device(n, m, k, 1.1, 1.0, 7, vals2.data_ptr(), idx2.data_ptr(),
                                        norms.data_ptr(), st))
    assert torch.equal(vals, vals2) and torch.equal(idx, idx2)  # deterministic in the seed


# ---- fixtures recorded from the reference engine ------------------------------
_REF_CASES = sorted(glob.glob(os.path.join(GOLDEN, "ref_case_*.npz")))


@pytest.mark.skipif(not _REF_CASES, reason="no reference-engine fixtures recorded yet")
@pytest.mark.parametrize("path", _REF_CASES, ids=[os.path.basename(p) for p in _REF_CASES])
def test_engine_matches_reference_engine_fixture(torch_cuda, path):
    from npeff_ref_b200 import MuNmfParams
    g = np.load(path)
    n, m, k, r = int(g["n"]), int(g["m"]), int(g["k"]), int(g["rank"])
    with _engine(MuNmfParams(rank=r, eps=float(g["eps"])), keep_csr=True) as eng:
        eng.set_csr(n, m, g["in_vals"], g["in_col"], None, k, None, int(g["min_count"]))
        assert np.array_equal(eng.new_to_og(), g["new_to_og"])
        gv, gc, grp = eng.export_shard_csr()
        assert np.array_equal(grp, g["p_rowptr"].astype(np.int64))
        assert np.array_equal(gc, g["p_col"]) and np.array_equal(gv, g["p_vals"])
        eng.init_factors(g["W0"], g["H0"])
        eng.run(int(g["iters"]), log_every=0)
        assert rel_fro(eng.load_w_to_host(), g["W"]) < 1e-4
        assert rel_fro(eng.load_h_to_host(), g["H"]) < 1e-4
        l = eng.compute_uncached_loss()
        assert abs(l - float(g["loss"])) < 1e-3 * l   # the reference sums its loss terms in fp32


_REF_WIDE = sorted(glob.glob(os.path.join(GOLDEN, "ref_wide_*.npz")))


@pytest.mark.skipif(not _REF_WIDE, reason="no wide reference-engine fixtures recorded yet")
@pytest.mark.parametrize("path", _REF_WIDE, ids=[os.path.basename(p) for p in _REF_WIDE])
def test_engine_matches_reference_engine_wide_fixture(torch_cuda, path):
    """Ranks 128 and 256 against the unmodified reference engine (cuSPARSE / cuBLAS) on
    matrices whose popular block spans several row tiles and K splits, with several
    tail column blocks: the fixture holds seeds (input: oracle.synth_pef; initial
    factors: the engine's cuRAND calls repeated here), W, a sample of H's columns and
    the norm of every column of H."""
    import zlib
    from npeff_ref_b200 import MuNmfParams
    from helpers import curand_xorwow_uniform
    g = np.load(path)
    n, m, k, r = int(g["n"]), int(g["m"]), int(g["k"]), int(g["rank"])
    vals, idx, norms = make_problem(n, m, k, seed=int(g["synth_seed"]))
    assert [zlib.crc32(vals.tobytes()), zlib.crc32(idx.tobytes())] == list(g["in_crc"]), \
        "the numpy generator no longer reproduces the fixture's input"
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    v = O.normalize_rows(vals.ravel(), rowptr, norms)       # the harness was fed normalised values
    with _engine(MuNmfParams(rank=r, eps=float(g["eps"])), keep_csr=True) as eng:
        eng.set_option("tail_block_bytes", 4 << 20)
        eng.set_csr(n, m, v, idx, None, k, None, int(g["min_count"]))
        mk = eng.shape[1]
        assert mk == int(g["m_kept"]) and np.array_equal(eng.new_to_og(), g["new_to_og"])
        gv, gc, grp = eng.export_shard_csr()
        assert zlib.crc32(gc.tobytes()) == int(g["p_col_crc"]) and zlib.crc32(gv.tobytes()) == int(g["p_vals_crc"])
        n_pop, _, n_blocks, tile_rows = eng.layout()
        assert n_pop > 256 and tile_rows == 0 and n_blocks >= 2
        w0, h0 = curand_xorwow_uniform(int(g["seed"]), [n * r, r * mk])
        assert np.array_equal(w0[:4096], g["W0_head"]) and np.array_equal(h0[:4096], g["H0_head"])
        eng.init_factors(w0.reshape(r, n).T, h0.reshape(mk, r).T)   # the reference's matrices are column-major
        eng.run(int(g["iters"]), log_every=0)
        W, H = eng.load_w_to_host(), eng.load_h_to_host()
        l = eng.compute_uncached_loss()
    assert rel_fro(W, g["W"]) < 1e-4, rel_fro(W, g["W"])
    assert rel_fro(H[:, g["H_cols"]], g["H_sample"]) < 1e-4
    hn = np.sqrt((H.astype(np.float64) ** 2).sum(axis=0))
    assert rel_fro(hn, g["H_col_norms"]) < 1e-4
    assert abs(l - float(g["loss"])) < 1e-3 * l   # the reference sums its loss terms in fp32


def test_retain_columns_loader_bit_exact(torch_cuda):
    """dnpeff_set_csr_retain against the oracle's RetainColumns_InPlace: an unsorted
    list, a repeated id, ids that no row holds."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k = 90, 3000, 70
    vals, idx, norms = make_problem(n, m, k, seed=17)
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    nv = O.normalize_rows(vals.ravel(), rowptr, norms)
    rng = np.random.default_rng(2)
    used = np.unique(idx)
    retained = rng.permutation(np.concatenate([rng.choice(used, 400, replace=False),
                                               np.setdiff1d(np.arange(m), used)[:20]])).astype(np.int32)
    retained = np.concatenate([retained, retained[:3]])        # three ids listed twice
    ev, ec, erp = O.retain_columns(nv, idx.ravel(), rowptr, m, retained)
    with _engine(MuNmfParams(rank=8), keep_csr=True) as eng:
        eng.set_csr_retain(n, m, vals, idx, retained, None, k, norms)
        assert eng.shape[1] == len(retained)
        assert np.array_equal(eng.new_to_og(), retained)
        v, c, rp = eng.export_shard_csr()
        assert np.array_equal(rp, erp) and np.array_equal(c, ec) and np.array_equal(v, ev)
    with _engine(MuNmfParams(rank=8)) as eng:
        with pytest.raises(Exception):
            eng.set_csr_retain(n, m, vals, idx, np.array([5, m], np.int32), None, k, norms)


@pytest.mark.parametrize("r", [16, 64, 256])   # 256: configuration 4's rank (panelled update kernel)
def test_fit_w_only_with_sparse_h_matches_oracle(torch_cuda, r):
    """The fit_coeffs_to_sparse_H numerics (src/nmf/sparse2/nmf_sparse_H.h:116-127,
    298-345): retained columns, H from CSR arrays, W-only updates with eps 1e-7."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k, iters, eps = 260, 5000, 120, 60, 1e-7
    vals, idx, norms = make_problem(n, m, k, seed=90 + r)
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    nv = O.normalize_rows(vals.ravel(), rowptr, norms)
    rng = np.random.default_rng(r)
    kept = np.sort(rng.choice(np.unique(idx), 1500, replace=False)).astype(np.int32)
    mk = len(kept)
    Hd = (rng.random((r, mk), dtype=np.float32) * (rng.random((r, mk)) > 0.93)).astype(np.float32)
    hv, hrp, hc = O.dense_to_csr(Hd, 1e-30)
    v, c, rp = O.retain_columns(nv, idx.ravel(), rowptr, m, kept)
    with _engine(MuNmfParams(rank=r, eps=eps, seed=11, init_scale=0.5)) as eng:
        eng.set_csr_retain(n, m, vals, idx, kept, None, k, norms)
        eng.init_factors()
        eng.set_h_csr(hrp, hc, hv)
        W0 = eng.load_w_to_host()
        assert np.array_equal(eng.load_h_to_host(), Hd)
        assert np.array_equal(W0, O.init_factors(n, mk, r, 11, 0.5)[0])
        loss = eng.fit_w_only(iters)
        W = eng.load_w_to_host()
    Wo, lo = O.fit_w_only(v, c, rp, mk, W0, Hd, iters, eps)
    assert rel_fro(W, Wo) < 1e-4
    assert abs(loss - lo) < 1e-5 * lo


# ---------------------------------------------------------------------------
# Hoyer projection of W (DenseFactorSparsityContext::sparsifyF and its kernels).
def _hoyer_check(got, want):
    # Column sums are float64 on both sides but in a different order, so an entry within
    # ~1e-8 of zero may fall on the other side of it: tolerate a few such entries.
    flips = (got == 0) != (want == 0)
    assert flips.sum() <= 3, int(flips.sum())
    assert np.all(np.abs(got[flips]) < 1e-6) and np.all(np.abs(want[flips]) < 1e-6)
    assert np.allclose(got, want, rtol=2e-5, atol=1e-6), np.abs(got - want).max()


@pytest.mark.gpu
@pytest.mark.parametrize("rule", [0, 1])
@pytest.mark.parametrize("n,r,sparseness", [(1, 4, 0.5), (257, 5, 0.4), (500, 8, 0.7), (3000, 128, 0.8),
                                            (20000, 32, 0.9), (64, 256, 0.6)])
def test_op_hoyer_project_matches_oracle(torch_cuda, n, r, sparseness, rule):
    import ctypes as C
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    rng = np.random.default_rng(n * 3 + r)
    W = rng.random((n, r), dtype=np.float32)
    l2 = 1.0
    l1 = float(np.sqrt(n) - (np.sqrt(n) - 1.0) * sparseness) * l2
    cap = 300
    want, wp, wc = O.hoyer_project(W, l1, l2, rule=rule, max_passes=cap)
    dW = _dev(torch, W)
    passes, conv = C.c_int32(-1), C.c_int32(-1)
    st = torch.cuda.current_stream().cuda_stream
    check(lib().dnpeff_op_hoyer_project(dW.data_ptr(), n, r, l1, l2, rule, cap, C.byref(passes), C.byref(conv), st))
    torch.cuda.synchronize()
    got = dW.cpu().numpy()
    assert passes.value == wp and bool(conv.value) == wc
    _hoyer_check(got, want)
    if rule == 0 and wc and n > 1:
        # the operator's own guarantees, independent of the oracle
        assert got.min() >= 0
        assert np.allclose(got.astype(np.float64).sum(axis=0), l1, rtol=2e-5)
        assert np.allclose(np.sqrt((got.astype(np.float64) ** 2).sum(axis=0)), l2, rtol=2e-5)


@pytest.mark.gpu
def test_op_hoyer_project_rejects_bad_arguments(torch_cuda):
    from npeff_ref_b200._lib import lib
    torch = torch_cuda
    dW = torch.ones((4, 4), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib().dnpeff_op_hoyer_project(dW.data_ptr(), 4, 4, -1.0, 1.0, 0, 0, None, None, st) != 0
    assert lib().dnpeff_op_hoyer_project(dW.data_ptr(), 4, 4, 1.0, 1.0, 7, 0, None, None, st) != 0
    assert lib().dnpeff_op_hoyer_project(dW.data_ptr(), 0, 4, 1.0, 1.0, 0, 0, None, None, st) == 0  # empty: no-op


@pytest.mark.gpu
def test_engine_sparsify_w_matches_oracle(torch_cuda):
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r = 300, 4000, 200, 16
    vals, idx, norms = make_problem(n, m, k, seed=5)
    with _engine(MuNmfParams(rank=r, eps=1e-12, seed=0, init_scale=1.0)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        eng.init_factors()
        W0 = eng.load_w_to_host()
        l1 = float(np.sqrt(n) - (np.sqrt(n) - 1.0) * 0.8)
        passes, conv = eng.sparsify_w(l1, 1.0)
        W1 = eng.load_w_to_host()
        want, wp, wc = O.hoyer_project(W0, l1, 1.0, rule=0)
        assert conv and wc and passes == wp
        _hoyer_check(W1, want)
        # the run goes on from the projected W
        eng.step_h()
        eng.step_w()
        assert np.all(np.isfinite(eng.load_w_to_host()))
