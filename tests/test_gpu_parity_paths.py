"""GPU parity tests of the paths the benchmark measures: the slab-pipelined host
loader, the loader without the kept input-order CSR, several tail column blocks,
the workload configuration 1 at its stated size with the loss curve, full runs at
the wide ranks, the host twin of the synthetic generator, and the bounded waits of
the warp-specialised tensor-core kernel.  Everything goes through the C ABI."""
import numpy as np
import pytest

from oracle import oracle as O
from helpers import rel_fro, make_problem, oracle_preprocess, baseline_scale

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    return torch


def _engine(params, options=(), **kw):
    from npeff_ref_b200 import MuNmf
    eng = MuNmf(params, **kw)
    for name, value in options:
        eng.set_option(name, value)
    return eng


def _ragged(rng, n, m, lens):
    ptr = np.zeros(n + 1, dtype=np.int64)
    ptr[1:] = np.cumsum(lens)
    ind = np.concatenate([rng.choice(m, size=l, replace=False) for l in lens] +
                         [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    vals = (rng.random(int(ptr[-1]), dtype=np.float32) + 0.01).astype(np.float32)
    return vals, ind, ptr


# ---------------------------------------------------------------------------
@pytest.mark.parametrize("slabs", [2, 4, 8])
@pytest.mark.parametrize("n_shards", [1, 2])
def test_loader_in_slabs_bit_exact(torch_cuda, slabs, n_shards):
    """dnpeff_set_csr with the values uploaded in several row slabs on a second stream
    (the path the end-to-end benchmark takes from 64 Mi entries on), forced here on a
    small ragged matrix whose rows 20..39 are empty, so that some slabs hold no entry:
    CSR, CSC, pruning map and |A|^2 against the oracle, bit for bit."""
    from npeff_ref_b200 import MuNmfParams
    rng = np.random.default_rng(100 + slabs)
    n, m = 67, 900
    lens = rng.integers(0, 60, size=n)
    lens[20:40] = 0
    lens[[0, 66]] = [0, 59]
    vals, ind, ptr = _ragged(rng, n, m, lens)
    norms = (rng.random(n, dtype=np.float32) + 0.5).astype(np.float32)
    v = O.normalize_rows(vals, ptr, norms)
    v, c, rp, n2o = O.prune_columns(v, ind, ptr, m, 2)
    mk = len(n2o)
    for s in range(n_shards):
        with _engine(MuNmfParams(rank=8), [("loader_slabs", slabs), ("keep_canonical_csr", 1)],
                     shard_index=s, n_shards=n_shards) as eng:
            eng.set_csr(n, m, vals, ind, ptr, 0, norms, 2)
            nn, mkept, c0, ms, nnz = eng.shape
            assert (nn, mkept) == (n, mk) and (c0, ms) == O.split_range(mk, n_shards, s)
            assert np.array_equal(eng.new_to_og(), n2o)
            sv, sc, srp = O.split_columns(v, c, rp, c0, ms)
            gv, gc, grp = eng.export_shard_csr()
            assert np.array_equal(grp, srp) and np.array_equal(gc, sc) and np.array_equal(gv, sv)
            cv, cr, cp = O.csr_to_csc(sv, sc, srp, ms)
            hv, hr, hp = eng.export_shard_csc()
            assert np.array_equal(hp, cp) and np.array_equal(hr, cr) and np.array_equal(hv, cv)
            assert abs(eng.a_sq_norm() - float((sv.astype(np.float64) ** 2).sum())) < 1e-9 * max(nnz, 1)


def test_loader_in_slabs_fixed_k_with_dense_block(torch_cuda):
    """The same with the D-PEF file's implicit offsets (k entries per row), a rank that
    keeps the popular columns as a dense block and narrow tail column blocks: the
    slab-wise extraction, bucketing and dense fill must give the factors of the
    one-slab load bit for bit, with and without the kept input-order CSR."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r = 300, 9000, 1200, 32
    vals, idx, norms = make_problem(n, m, k, seed=41)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    outs = []
    for slabs, keep in [(1, 1), (4, 1), (4, 0), (8, 0)]:
        with _engine(MuNmfParams(rank=r, eps=1e-12, seed=3, init_scale=scale),
                     [("loader_slabs", slabs), ("keep_canonical_csr", keep), ("tail_block_bytes", 64 * 1024)]) as eng:
            eng.set_csr(n, m, vals, idx, None, k, norms, 1)
            n_pop, pop_nnz, n_blocks, tile_rows = eng.layout()
            assert n_pop >= 8 and tile_rows == 0 and n_blocks >= 4
            if keep:
                gv, gc, grp = eng.export_shard_csr()
                assert np.array_equal(grp, rp) and np.array_equal(gc, c) and np.array_equal(gv, v)
            else:
                from npeff_ref_b200 import DnpeffError
                with pytest.raises(DnpeffError) as ei:
                    eng.export_shard_csr()
                assert ei.value.code == -1 and "keep_canonical_csr" in str(ei.value)
            eng.init_factors()
            W0, H0 = eng.load_w_to_host(), eng.load_h_to_host()
            eng.run(3, log_every=0)
            outs.append((eng.load_w_to_host(), eng.load_h_to_host(), eng.compute_uncached_loss()))
            cv, cr, cp = O.csr_to_csc(v, c, rp, mk)
            hv, hr, hp = eng.export_shard_csc()   # rebuilt at full size on demand
            assert np.array_equal(hp, cp) and np.array_equal(hr, cr) and np.array_equal(hv, cv)
            eng.step_h()                          # and the engine still iterates afterwards
    for W, H, l in outs[1:]:
        assert np.array_equal(W, outs[0][0]) and np.array_equal(H, outs[0][1]) and l == outs[0][2]
    Wo, Ho = O.run(v, c, rp, mk, W0, H0, 3, 1e-12)
    assert rel_fro(outs[0][0], Wo) < 1e-5 and rel_fro(outs[0][1], Ho) < 1e-5


def test_device_loader_in_internal_slabs(torch_cuda):
    """dnpeff_set_csr_device cuts large inputs into row slabs of its own; the slab
    boundaries must not show in the result (a matrix of 40 rows is one slab, so the
    check runs the slab loop through the host entry point with 8 slabs and compares
    it with the device entry point)."""
    from npeff_ref_b200 import MuNmfParams
    torch = torch_cuda
    n, m, k, r = 40, 700, 90, 8
    vals, idx, norms = make_problem(n, m, k, seed=9)
    res = []
    for device_input in (False, True):
        with _engine(MuNmfParams(rank=r, seed=1, init_scale=0.1), [("loader_slabs", 8), ("keep_canonical_csr", 1)]) as eng:
            if device_input:
                dv, di, dn = (torch.from_numpy(a).cuda() for a in (vals, idx, norms))
                eng.set_csr_device(n, m, dv.data_ptr(), di.data_ptr(), 0, k, dn.data_ptr(), 1)
            else:
                eng.set_csr(n, m, vals, idx, None, k, norms, 1)
            res.append(eng.export_shard_csr() + eng.export_shard_csc())
    for a, b in zip(*res):
        assert np.array_equal(a, b)


# ---------------------------------------------------------------------------
def test_configuration_1_at_stated_size_with_loss_curve(torch_cuda):
    """Workload configuration 1 as stated: n = 2048 examples, m = 65 536 features, 4096
    stored values per row, Zipf(1.1) columns, rank 32, factors Uniform(0,1) *
    sqrt(mean(A)/r), eps = 1e-12, seed 0, 50 iterations.  Targets: W and H within 1e-4
    relative Frobenius of the float64-accumulating oracle from identical initial
    factors, the loss within 1e-5 relative at every 10th step."""
    from npeff_ref_b200 import MuNmfParams
    n, m, k, r, iters, eps = 2048, 65536, 4096, 32, 50, 1e-12
    vals, idx, norms = O.synth_pef_hashed(n, m, k, alpha=1.1, sigma=1.0, seed=0)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    Wo0, Ho0 = O.init_factors(n, mk, r, 0, scale)
    Wo, Ho, ls = O.run(v, c, rp, mk, Wo0, Ho0, iters, eps, acc64=True, losses=True)
    with _engine(MuNmfParams(rank=r, eps=eps, seed=0, init_scale=scale)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        assert eng.shape[1] == mk
        eng.init_factors()
        assert np.array_equal(eng.load_w_to_host(), Wo0) and np.array_equal(eng.load_h_to_host(), Ho0)
        for step in range(10, iters + 1, 10):
            eng.run(10, log_every=0)
            l = eng.compute_uncached_loss()
            assert abs(l - ls[step - 1]) < 1e-5 * ls[step - 1], (step, l, ls[step - 1])   # stated target
        W, H = eng.load_w_to_host(), eng.load_h_to_host()
    assert rel_fro(W, Wo) < 1e-4, rel_fro(W, Wo)      # stated target
    assert rel_fro(H, Ho) < 1e-4, rel_fro(H, Ho)


@pytest.mark.parametrize("n,m,k,r,iters,tail_bytes", [
    (400, 7000, 900, 384, 20, 2 << 20), (560, 7000, 900, 512, 20, 2 << 20),
    (1100, 60000, 6000, 128, 50, 8 << 20), (700, 30000, 1500, 256, 30, 4 << 20)])
def test_full_run_wide_and_headline_ranks(torch_cuda, n, m, k, r, iters, tail_bytes):
    """Full runs at ranks 384 and 512 (panelled tensor-core kernels) and, at ranks 128
    and 256, on matrices whose dense popular block spans several row tiles and K
    splits with several tail column blocks and rows long enough for the block-per-row
    gather kernel; loss compared every 10th step."""
    from npeff_ref_b200 import MuNmfParams
    eps = 1e-12
    vals, idx, norms = make_problem(n, m, k, seed=n + r)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    W0, H0 = O.init_factors(n, mk, r, 5, scale)
    Wo, Ho, ls = O.run(v, c, rp, mk, W0, H0, iters, eps, acc64=True, losses=True)
    a2 = float((v.astype(np.float64) ** 2).sum())
    with _engine(MuNmfParams(rank=r, eps=eps, seed=5, init_scale=scale), [("tail_block_bytes", tail_bytes)]) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        n_pop, _, n_blocks, tile_rows = eng.layout()
        assert n_pop > 128 and tile_rows == 0 and n_blocks >= 2
        eng.init_factors()
        for step in range(10, iters + 1, 10):
            eng.run(10, log_every=0)
            l = eng.compute_uncached_loss()
            # squared form: accurate to 3e-6 of |A|^2 (see test_full_run_matches_oracle);
            # the 1e-5 relative target applies where the fit is not near-exact
            assert abs(l * l - ls[step - 1] ** 2) < 3e-6 * a2
            if ls[step - 1] ** 2 > 0.05 * a2:
                assert abs(l - ls[step - 1]) < 1e-5 * ls[step - 1], (step, l, ls[step - 1])
        W, H = eng.load_w_to_host(), eng.load_h_to_host()
    assert rel_fro(W, Wo) < 1e-4, rel_fro(W, Wo)
    assert rel_fro(H, Ho) < 1e-4, rel_fro(H, Ho)


# ---------------------------------------------------------------------------
def test_host_generator_twin_matches_device_generator(torch_cuda):
    """The timed CPU arm generates its input with the host twin of the device
    generator: the column indices must be identical, the values equal to rounding."""
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    for (n, m, k, alpha, sigma, seed) in [(48, 50000, 2048, 1.1, 1.0, 7), (33, 4096, 1024, 1.4, 2.0, 4),
                                         (5, 300, 300, 1.1, 1.0, 1)]:
        vals = torch.empty((n, k), dtype=torch.float32, device="cuda")
        idx = torch.empty((n, k), dtype=torch.int32, device="cuda")
        norms = torch.empty((n,), dtype=torch.float32, device="cuda")
        st = torch.cuda.current_stream().cuda_stream
        check(lib().dnpeff_synth_pef_device(n, m, k, alpha, sigma, seed, vals.data_ptr(), idx.data_ptr(),
                                            norms.data_ptr(), st))
        hv, hi, hn = O.synth_pef_hashed(n, m, k, alpha=alpha, sigma=sigma, seed=seed)
        assert np.array_equal(idx.cpu().numpy(), hi)
        assert np.allclose(vals.cpu().numpy(), hv, rtol=2e-6, atol=0)
        assert np.allclose(norms.cpu().numpy(), hn, rtol=2e-6)


def test_streamed_file_loader_matches_array_loader(torch_cuda, tmp_path):
    """dnpeff_load_pef_hdf5 reads the engine's rows in 64 MB chunks through two pinned
    staging buffers; a file of 2 600 x 16 384 values (170 MB per dataset) takes three
    chunks, so both buffers are reused.  The loaded matrix must equal, bit for bit, the
    one dnpeff_set_csr builds from the same arrays; the leading-hyperslab arguments
    (--n_examples, --n_fisher_values) are covered too."""
    import ctypes as C
    from npeff_ref_b200 import MuNmfParams
    from npeff_ref_b200._lib import lib, check
    n, m, k = 2600, 300000, 16384
    vals, idx, norms = O.synth_pef_hashed(n, m, k, seed=12)
    path = str(tmp_path / "pef.h5")
    check(lib().dnpeff_write_pef_hdf5(path.encode(), n, k, C.c_void_p(vals.ctypes.data), C.c_void_p(idx.ctypes.data),
                                      C.c_void_p(norms.ctypes.data), m))
    for (ne, nk) in [(0, 0), (1500, 9000)]:
        rows, cols = (ne or n), (nk or k)
        with _engine(MuNmfParams(rank=8), [("keep_canonical_csr", 1)]) as a, \
                _engine(MuNmfParams(rank=8), [("keep_canonical_csr", 1)]) as b:
            check(lib().dnpeff_load_pef_hdf5(a._h, path.encode(), ne, nk, 2))
            b.set_csr(rows, m, np.ascontiguousarray(vals[:rows, :cols]), np.ascontiguousarray(idx[:rows, :cols]),
                      None, cols, norms[:rows], 2)
            assert a.shape == b.shape and np.array_equal(a.new_to_og(), b.new_to_og())
            for x, y in zip(a.export_shard_csr(), b.export_shard_csr()):
                assert np.array_equal(x, y)


def test_device_generator_row_ranges_are_slices_of_the_matrix(torch_cuda):
    """dnpeff_synth_pef_device_rows: a row's content depends on its index and the seed
    only, so a rank of a row-split job generates exactly its slice of the matrix."""
    from npeff_ref_b200._lib import lib, check
    torch = torch_cuda
    n, m, k = 37, 9000, 512
    st = torch.cuda.current_stream().cuda_stream

    def gen(first, rows):
        v = torch.empty((rows, k), dtype=torch.float32, device="cuda")
        i = torch.empty((rows, k), dtype=torch.int32, device="cuda")
        nr = torch.empty((rows,), dtype=torch.float32, device="cuda")
        check(lib().dnpeff_synth_pef_device_rows(first, rows, m, k, 1.1, 1.0, 3, v.data_ptr(), i.data_ptr(),
                                                 nr.data_ptr(), st))
        return v.cpu().numpy(), i.cpu().numpy(), nr.cpu().numpy()

    fv, fi, fn = gen(0, n)
    for first, rows in [(0, 10), (10, 20), (30, 7)]:
        v, i, nr = gen(first, rows)
        assert np.array_equal(v, fv[first:first + rows]) and np.array_equal(i, fi[first:first + rows])
        assert np.array_equal(nr, fn[first:first + rows])


# ---------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_engine_recovers(torch_cuda):
    """The only device-side failure detection in the product: every wait between the
    roles of the warp-specialised tensor-core kernel is bounded.  With the limit set
    to a single poll the first wait for a bulk copy runs out, the kernel leaves
    cleanly (copies and MMAs already issued are waited for with the full limit, its
    TMEM is freed), and the next status read reports DNPEFF_ERR_CUDA.  With the limit
    restored the same engine computes correct results.  No fault, trap or hang is
    involved: the kernel returns by itself."""
    from npeff_ref_b200 import MuNmfParams, DnpeffError
    n, m, k, r, eps = 700, 20000, 2000, 64, 1e-12
    vals, idx, norms = make_problem(n, m, k, seed=123)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    with _engine(MuNmfParams(rank=r, eps=eps, seed=2, init_scale=scale)) as eng:
        eng.set_csr(n, m, vals, idx, None, k, norms, 1)
        assert eng.layout()[3] == 0            # dense popular block: k_block_tc is on the path
        eng.init_factors()
        W0, H0 = eng.load_w_to_host(), eng.load_h_to_host()
        eng.set_option("wait_limit", 1)
        eng.step_w()
        with pytest.raises(DnpeffError) as ei:
            eng.synchronize()
        assert ei.value.code == -2 and "ran out" in str(ei.value)
        eng.set_option("wait_limit", 0)        # back to the default
        eng.synchronize()                      # the status was reported once and cleared
        eng.init_factors(W0, H0)
        eng.step_w()
        W1 = eng.load_w_to_host()
        assert rel_fro(W1, O.step_w(v, c, rp, mk, W0, H0, eps)) < 2e-6


# ---------------------------------------------------------------------------
_NO_TC_SCRIPT = r"""
import sys, numpy as np
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + "/tests")
from npeff_ref_b200 import MuNmf, MuNmfParams
from helpers import make_problem
n, m, k, r = 300, 9000, 1500, 128
vals, idx, norms = make_problem(n, m, k, seed=428)
with MuNmf(MuNmfParams(rank=r, eps=1e-12, seed=0, init_scale=float(sys.argv[3]))) as eng:
    eng.set_csr(n, m, vals, idx, None, k, norms, 1)
    layout = eng.layout()
    eng.init_factors()
    eng.run(20, log_every=0)
    np.savez(sys.argv[2], W=eng.load_w_to_host(), H=eng.load_h_to_host(), loss=eng.compute_uncached_loss(),
             tile_rows=layout[3])
"""


def test_cuda_core_path_at_a_tensor_core_rank(torch_cuda, tmp_path):
    """DNPEFF_NO_TC=1 keeps every contraction on the CUDA-core kernels and the popular
    columns on the shared-memory tiled sparse kernel (the path other ranks take, and the
    A/B comparison for the tensor-core kernels).  At rank 128 it must match the oracle
    like the tensor-core path does."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    n, m, k, r, iters = 300, 9000, 1500, 128, 20
    vals, idx, norms = make_problem(n, m, k, seed=428)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    scale = baseline_scale(v, n, mk, r)
    W0, H0 = O.init_factors(n, mk, r, 0, scale)
    Wo, Ho, ls = O.run(v, c, rp, mk, W0, H0, iters, 1e-12, acc64=True, losses=True)
    outs = {}
    for name, env in (("tc", {}), ("no_tc", {"DNPEFF_NO_TC": "1"})):
        out = str(tmp_path / (name + ".npz"))
        res = subprocess.run([sys.executable, "-c", _NO_TC_SCRIPT, root, out, repr(scale)],
                             env=dict(os.environ, **env), capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        outs[name] = np.load(out)
    assert int(outs["tc"]["tile_rows"]) == 0 and int(outs["no_tc"]["tile_rows"]) > 0   # dense block / tiled sparse kernel
    for name in outs:
        assert rel_fro(outs[name]["W"], Wo) < 1e-4 and rel_fro(outs[name]["H"], Ho) < 1e-4, name
        assert abs(float(outs[name]["loss"]) - ls[-1]) < 1e-5 * ls[-1], name
