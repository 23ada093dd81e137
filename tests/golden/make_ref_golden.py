"""Generates the reference-engine fixtures in this folder.

Needs a CUDA GPU and ``oracle/_ref/ref_engine`` (``make -C oracle ref`` where
the reference tree is mounted): it runs the UNMODIFIED reference engine
(cuSPARSE/cuBLAS/cuRAND/NCCL) on small seeded matrices and stores its inputs
and outputs as ``ref_case_*.npz``.  The tests compare the CPU oracle, and the
CUDA engine, against these files.

    python tests/golden/make_ref_golden.py [out_dir]

Each fixture holds: the normalised input CSR, the reference's pruned CSR and
``new_to_og`` map, its initial factors (W0, H0), its factors and loss after
``iters`` iterations, and the parameters used.
"""
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

CASES = [
    # name, n, m, k, rank, iters, eps, seed, min_count, synth seed
    ("a", 96, 1500, 48, 8, 20, 1e-8, 43190432042, 1, 11),
    ("b", 200, 4096, 128, 32, 50, 1e-8, 43190432042, 2, 12),
    ("c", 64, 700, 40, 12, 30, 1e-12, 7, 1, 13),
]


def run_case(exe, out_dir, name, n, m, k, rank, iters, eps, seed, min_count, sseed):
    vals, idx, norms = O.synth_pef(n, m, k, alpha=1.1, sigma=1.0, seed=sseed)
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    v = O.normalize_rows(vals.ravel(), rowptr, norms)
    with tempfile.TemporaryDirectory() as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        with open(fin, "wb") as f:
            f.write(struct.pack("<3q", n, m, n * k))
            f.write(rowptr.astype(np.int32).tobytes())
            f.write(idx.astype(np.int32).tobytes())
            f.write(v.astype(np.float32).tobytes())
        res = subprocess.run([exe, fin, fout, str(rank), str(iters), repr(eps), str(seed),
                              str(min_count)], capture_output=True, text=True)
        sys.stdout.write(res.stdout[-2000:])
        if res.returncode != 0:
            sys.stderr.write(res.stderr[-4000:])
            raise SystemExit("ref_engine failed for case %s" % name)
        raw = open(fout, "rb").read()
    off = 0

    def take(dtype, count):
        nonlocal off
        a = np.frombuffer(raw, dtype=dtype, count=count, offset=off).copy()
        off += a.nbytes
        return a

    n_, m_kept, nnz_kept, rank_, ndev = take(np.int64, 5)
    new_to_og = take(np.int32, m_kept)
    p_rowptr = take(np.int32, n + 1)
    p_col = take(np.int32, nnz_kept)
    p_vals = take(np.float32, nnz_kept)
    W0 = take(np.float32, n * rank).reshape(rank, n).T.copy()        # col-major n x r
    H0 = take(np.float32, rank * m_kept).reshape(m_kept, rank).T.copy()  # col-major r x m
    W = take(np.float32, n * rank).reshape(rank, n).T.copy()
    H = take(np.float32, rank * m_kept).reshape(m_kept, rank).T.copy()
    loss0, loss = take(np.float32, 2)
    np.savez_compressed(
        os.path.join(out_dir, "ref_case_%s.npz" % name),
        n=n, m=m, k=k, rank=rank, iters=iters, eps=eps, seed=seed, min_count=min_count,
        n_devices=ndev, in_vals=v.astype(np.float32), in_col=idx.ravel().astype(np.int32),
        new_to_og=new_to_og, p_rowptr=p_rowptr, p_col=p_col, p_vals=p_vals,
        W0=W0, H0=H0, W=W, H=H, loss0=loss0, loss=loss)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_engine")
    if not os.path.exists(exe):
        raise SystemExit("build oracle/_ref/ref_engine first: make -C oracle ref")
    for case in CASES:
        run_case(exe, out_dir, *case)


if __name__ == "__main__":
    main()
