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
