"""Two-rank CPU rendering (gloo) of the multi-GPU exchange: column shards, one
all-reduce of [A_d*H_d^T | H_d*H_d^T] per iteration, replicated W update, local
H update, column-wise gather of H.  The per-shard arithmetic is the oracle's;
what is under test is the sharding rule and the exchange pattern the engine
uses (multi_mu_dense_factors_nmf1.h:293-339), against the unsharded oracle."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, iters, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from helpers import make_problem, oracle_preprocess

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, m, k, r, eps = 48, 600, 40, 6, 1e-8
    vals, idx, norms = make_problem(n, m, k, seed=17)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)     # every rank: same global pruning
    mk = len(n2o)
    c0, w = O.split_range(mk, world, rank)
    sv, sc, srp = O.split_columns(v, c, rp, c0, w)
    W, Hs = O.init_factors(n, w, r, 5, 0.05, col_start=c0)     # W replicated, H shard of the global stream
    for _ in range(iters):
        Hst = np.ascontiguousarray(Hs.T)
        buf = np.concatenate([O.spmm(sv, sc, srp, Hst).ravel(), O.gram(Hst).ravel()])
        t = torch.from_numpy(buf)
        dist.all_reduce(t)                                       # the one exchange per iteration
        AH = t.numpy()[:n * r].reshape(n, r)
        HH = t.numpy()[n * r:].reshape(r, r)
        W = O.mu_update(W, AH, HH, eps)                          # identical on every rank
        Hs = O.step_h(sv, sc, srp, w, W, Hs, eps)                # local to the shard
    gathered = [None] * world
    dist.all_gather_object(gathered, (c0, Hs))
    if rank == 0:
        H = np.concatenate([h for _, h in sorted(gathered, key=lambda x: x[0])], axis=1)
        np.savez(os.path.join(out_dir, "sharded.npz"), W=W, H=H)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_column_sharded_iteration_matches_unsharded(tmp_path, world):
    import torch.multiprocessing as mp
    from oracle import oracle as O
    from helpers import make_problem, oracle_preprocess, rel_fro
    iters = 5
    mp.spawn(_worker, args=(world, _free_port(), iters, str(tmp_path)), nprocs=world, join=True)
    got = np.load(os.path.join(str(tmp_path), "sharded.npz"))
    n, m, k, r, eps = 48, 600, 40, 6, 1e-8
    vals, idx, norms = make_problem(n, m, k, seed=17)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, 5, 0.05)
    W, H = O.run(v, c, rp, mk, W0, H0, iters, eps)
    # the exchange sums fp32 partials that the unsharded run accumulates in double
    assert rel_fro(got["W"], W) < 1e-5
    assert rel_fro(got["H"], H) < 1e-5
