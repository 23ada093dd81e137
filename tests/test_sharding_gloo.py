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


# ---------------------------------------------------------------------------
def _slice_bounds(n, world, idx):
    """dnpeff_row_slice: rows [n*idx/world, n*(idx+1)/world)."""
    b = n * idx // world
    return b, n * (idx + 1) // world - b


def _sliced_loader_worker(rank, world, port, cyclic, out_dir):
    """The exchange of the row-sliced loader (dnpeff_set_csr_rows), host rendering:
    local column counts -> all-reduce -> the same pruning map everywhere -> for every
    destination the slice's entries in that destination's columns, input order kept ->
    all-to-all -> slices concatenated in source order."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from oracle import oracle as O
    from helpers import make_problem

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, m, k, min_count = 53, 500, 30, 2
    vals, idx, norms = make_problem(n, m, k, seed=29)
    b, cnt = _slice_bounds(n, world, rank)
    lv = (vals[b:b + cnt] / (norms[b:b + cnt, None] + np.float32(1e-9))).astype(np.float32)   # pef_fisher_h5.h:38-52
    li = idx[b:b + cnt]
    counts = torch.from_numpy(np.bincount(li.ravel(), minlength=m).astype(np.int32))
    dist.all_reduce(counts)                                   # the integer all-reduce of the loader
    keep = counts.numpy() >= min_count
    og_to_new = np.where(keep, np.cumsum(keep) - 1, -1)
    mk = int(keep.sum())
    new = og_to_new[li]                                       # [cnt, k] kept-column id or -1

    def owner_and_local(c):
        if cyclic:
            return c % world, c // world
        base = mk // world
        d = np.minimum(c // max(base, 1), world - 1) if base > 0 else np.full_like(c, world - 1)
        return d, c - d * base

    send = []
    for d in range(world):
        rows_v, rows_c, lens = [], [], []
        for i in range(cnt):
            sel = new[i] >= 0
            own, loc = owner_and_local(new[i][sel])
            pick = own == d
            rows_v.append(lv[i][sel][pick])
            rows_c.append(loc[pick].astype(np.int32))
            lens.append(int(pick.sum()))
        send.append((np.array(lens, np.int32), np.concatenate(rows_v + [np.zeros(0, np.float32)]),
                     np.concatenate(rows_c + [np.zeros(0, np.int32)])))
    recv = [None] * world
    for d in range(world):                                    # the grouped send/recv, as gathers
        box = [None] * world if rank == d else None
        dist.gather_object(send[d], box, dst=d)
        if rank == d:
            recv = box
    lens = np.concatenate([r_[0] for r_ in recv])             # slices in source (= row) order
    np.savez(os.path.join(out_dir, "sliced%d.npz" % rank), rp=np.concatenate([[0], np.cumsum(lens)]),
             v=np.concatenate([r_[1] for r_ in recv]), c=np.concatenate([r_[2] for r_ in recv]),
             n2o=np.flatnonzero(keep).astype(np.int32))
    dist.destroy_process_group()


@pytest.mark.parametrize("cyclic", [False, True], ids=["contiguous", "cyclic"])
@pytest.mark.parametrize("world", [2, 3])
def test_row_sliced_exchange_layout(tmp_path, world, cyclic):
    import torch.multiprocessing as mp
    from oracle import oracle as O
    from helpers import make_problem, oracle_preprocess
    mp.spawn(_sliced_loader_worker, args=(world, _free_port(), cyclic, str(tmp_path)), nprocs=world, join=True)
    n, m, k, min_count = 53, 500, 30, 2
    vals, idx, norms = make_problem(n, m, k, seed=29)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m, min_count)
    mk = len(n2o)
    rows = np.repeat(np.arange(n), np.diff(rp))
    for d in range(world):
        p = np.load(os.path.join(str(tmp_path), "sliced%d.npz" % d))
        assert np.array_equal(p["n2o"], n2o)
        if cyclic:
            sel = (c % world) == d
            sv, sc = v[sel], (c[sel] // world).astype(np.int32)
            srp = np.concatenate([[0], np.cumsum(np.bincount(rows[sel], minlength=n))])
        else:
            c0, w = O.split_range(mk, world, d)
            sv, sc, srp = O.split_columns(v, c, rp, c0, w)
        assert np.array_equal(p["rp"], srp) and np.array_equal(p["c"], sc) and np.array_equal(p["v"], sv)
