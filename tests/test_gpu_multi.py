"""Multi-GPU parity: one engine per GPU (child processes), column shards joined
by NCCL, against the unsharded CPU oracle.  Needs >= 2 CUDA devices."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROBLEMS = {
    "r32": dict(n=160, m=5000, k=220, r=32, eps=1e-8, iters=20, seed=23, scale=0.02),
    # the headline rank and a wide rank: dense popular block on the tensor cores on
    # every shard, tensor-core Gram / update kernels, one allreduce of [A H^T | H H^T]
    "r128": dict(n=300, m=9000, k=1500, r=128, eps=1e-12, iters=20, seed=31, scale=0.01),
    "r256": dict(n=640, m=6000, k=800, r=256, eps=1e-12, iters=20, seed=37, scale=0.01),
}


def _n_gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, uid, out_dir, mode, problem):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from npeff_ref_b200 import MuNmf, MuNmfParams
    from helpers import make_problem
    P = PROBLEMS[problem]
    vals, idx, norms = make_problem(P["n"], P["m"], P["k"], seed=P["seed"])
    with MuNmf(MuNmfParams(rank=P["r"], eps=P["eps"], seed=3, init_scale=P["scale"]), device=rank,
               shard_index=rank, n_shards=world, shard_mode=mode) as eng:
        eng.set_csr(P["n"], P["m"], vals, idx, None, P["k"], norms, 1)
        eng.init_comm(uid)
        eng.init_factors()
        eng.run(P["iters"], log_every=0)
        loss = eng.compute_uncached_loss()
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), W=eng.load_w_to_host(),
                 H=eng.load_h_to_host(), loss=loss, cols=eng.shard_columns()[0])


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("mode", [0, 1], ids=["contiguous", "cyclic"])
@pytest.mark.parametrize("world,problem", [(2, "r32"), (4, "r32"), (8, "r32"), (2, "r128"), (2, "r256")])
def test_nccl_sharded_run_matches_oracle(tmp_path, world, mode, problem):
    if _n_gpus() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    from npeff_ref_b200 import MuNmf
    from oracle import oracle as O
    from helpers import make_problem, oracle_preprocess, rel_fro
    uid = MuNmf.make_unique_id()
    mp.spawn(_worker, args=(world, uid, str(tmp_path), mode, problem), nprocs=world, join=True)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    P = PROBLEMS[problem]
    vals, idx, norms = make_problem(P["n"], P["m"], P["k"], seed=P["seed"])
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, P["m"])
    mk = len(n2o)
    W0, H0 = O.init_factors(P["n"], mk, P["r"], 3, P["scale"])
    W, H, ls = O.run(v, c, rp, mk, W0, H0, P["iters"], P["eps"], losses=True)
    Hg = np.empty_like(H)
    for p in parts:
        Hg[:, p["cols"]] = p["H"]
    a2 = float((v.astype(np.float64) ** 2).sum())
    for p in parts:                      # W is replicated and identical on every rank
        assert np.array_equal(p["W"], parts[0]["W"])
        l = float(p["loss"])
        # squared form to 3e-6 of |A|^2 always; 1e-5 relative where the fit is not near-exact
        assert abs(l * l - ls[-1] ** 2) < 3e-6 * a2
        if ls[-1] ** 2 > 0.05 * a2:
            assert abs(l - ls[-1]) < 1e-5 * ls[-1]
    assert rel_fro(parts[0]["W"], W) < 1e-4
    assert rel_fro(Hg, H) < 1e-4


# ---------------------------------------------------------------------------
SLICED = dict(n=203, m=4000, k=300, r=32, eps=1e-12, iters=10, seed=41, scale=0.02, min_count=2)


def _sliced_worker(rank, world, uid, out_dir, mode):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from npeff_ref_b200 import MuNmf, MuNmfParams
    from helpers import make_problem
    P = SLICED
    vals, idx, norms = make_problem(P["n"], P["m"], P["k"], seed=P["seed"])
    b, c = MuNmf.row_slice(P["n"], world, rank)
    with MuNmf(MuNmfParams(rank=P["r"], eps=P["eps"], seed=3, init_scale=P["scale"]), device=rank,
               shard_index=rank, n_shards=world, shard_mode=mode) as eng:
        eng.set_option("keep_canonical_csr", 1)
        eng.init_comm(uid)
        # only this engine's rows are handed over
        eng.set_csr_rows(P["n"], P["m"], b, vals[b:b + c], idx[b:b + c], None, P["k"], norms[b:b + c],
                         P["min_count"])
        v, ci, rp = eng.export_shard_csr()
        cv, cr, cp = eng.export_shard_csc()
        n2o = eng.new_to_og()
        cols = eng.shard_columns()[0]
        eng.init_factors()
        eng.run(P["iters"], log_every=0)
        np.savez(os.path.join(out_dir, "sliced%d.npz" % rank), v=v, ci=ci, rp=rp, cv=cv, cr=cr, cp=cp, n2o=n2o,
                 cols=cols, W=eng.load_w_to_host(), H=eng.load_h_to_host(), loss=eng.compute_uncached_loss(),
                 a_sq=eng.a_sq_norm())


@pytest.mark.skipif(_n_gpus() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("mode", [0, 1], ids=["contiguous", "cyclic"])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_row_sliced_loader_bit_exact(tmp_path, world, mode):
    """dnpeff_set_csr_rows: every engine uploads its slice of the rows only; the column
    counts are summed with one allreduce and the entries exchanged with grouped
    ncclSend/ncclRecv.  The shard each engine ends up with must be, bit for bit, the
    column split of the oracle's pruned matrix (CSR in input order, CSC, pruning map),
    and a run from there must match the oracle like the whole-matrix loader's."""
    if _n_gpus() < world:
        pytest.skip("needs %d GPUs" % world)
    import torch.multiprocessing as mp
    from npeff_ref_b200 import MuNmf
    from oracle import oracle as O
    from helpers import make_problem, oracle_preprocess, rel_fro
    uid = MuNmf.make_unique_id()
    mp.spawn(_sliced_worker, args=(world, uid, str(tmp_path), mode), nprocs=world, join=True)
    P = SLICED
    vals, idx, norms = make_problem(P["n"], P["m"], P["k"], seed=P["seed"])
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, P["m"], P["min_count"])
    mk = len(n2o)
    rows = np.repeat(np.arange(P["n"]), np.diff(rp))
    parts = [np.load(os.path.join(str(tmp_path), "sliced%d.npz" % r)) for r in range(world)]
    for d, p in enumerate(parts):
        assert np.array_equal(p["n2o"], n2o)
        if mode == 1:
            sel = (c % world) == d
            sv, sc = v[sel], (c[sel] // world).astype(np.int32)
            srp = np.concatenate([[0], np.cumsum(np.bincount(rows[sel], minlength=P["n"]))]).astype(np.int64)
            ms = len(np.arange(d, mk, world))
        else:
            c0, ms = O.split_range(mk, world, d)
            sv, sc, srp = O.split_columns(v, c, rp, c0, ms)
        assert np.array_equal(p["rp"], srp) and np.array_equal(p["ci"], sc) and np.array_equal(p["v"], sv)
        cv, cr, cp = O.csr_to_csc(sv, sc, srp, ms)
        assert np.array_equal(p["cp"], cp) and np.array_equal(p["cr"], cr) and np.array_equal(p["cv"], cv)
        assert abs(float(p["a_sq"]) - float((sv.astype(np.float64) ** 2).sum())) < 1e-9 * max(len(sv), 1)
    W0, H0 = O.init_factors(P["n"], mk, P["r"], 3, P["scale"])
    W, H, ls = O.run(v, c, rp, mk, W0, H0, P["iters"], P["eps"], losses=True)
    Hg = np.empty_like(H)
    for p in parts:
        Hg[:, p["cols"]] = p["H"]
        assert np.array_equal(p["W"], parts[0]["W"])
        assert abs(float(p["loss"]) - ls[-1]) < 1e-5 * ls[-1]
    assert rel_fro(parts[0]["W"], W) < 1e-4 and rel_fro(Hg, H) < 1e-4
