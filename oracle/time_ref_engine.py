"""TEST INFRASTRUCTURE ONLY: times the UNMODIFIED reference engine
(``oracle/_ref/ref_engine``: cuSPARSE SpMM + cuBLAS SGEMM + cuRAND + NCCL, built by
``make -C oracle ref`` where the reference tree is mounted) on the benchmark's
workload, on the GPUs this process can see.  The number goes into the design
notes as the reference's own speed on this hardware; nothing in the product or in
``bench.py`` calls this.

    python oracle/time_ref_engine.py [--config 2] [--iters 30] [--scale-rows F]

The workload is generated on the GPU by the benchmark's generator, normalised the
way the loader does (``v / (norm + 1e-9)``, io/pef_fisher_h5.h:38-52) and handed to
the harness as a flat file.  The engine prints ``step N: <loss> [<ms> ms/step]``
every 10 steps (multi_mu_dense_factors_nmf1.h:171-201); those lines are the result.
"""
import argparse
import ctypes as C
import os
import re
import struct
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import bench
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--scale-rows", type=float, default=1.0)
    ap.add_argument("--tmp", default=None)
    args = ap.parse_args()
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_engine")
    if not os.path.exists(exe):
        raise SystemExit("build oracle/_ref/ref_engine first: make -C oracle ref")
    import torch
    from npeff_ref_b200._lib import lib, check
    c = dict(bench.CONFIGS[args.config])
    c["n"] = max(1, int(c["n"] * args.scale_rows))
    n, m, k, r = c["n"], c["m"], c["k"], c["r"]
    if n * k >= 2 ** 31:
        raise SystemExit("the reference engine's int32 offsets cannot hold this workload")
    d_vals = torch.empty((n, k), dtype=torch.float32, device="cuda")
    d_idx = torch.empty((n, k), dtype=torch.int32, device="cuda")
    d_norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    check(lib().dnpeff_synth_pef_device(n, m, k, c["alpha"], c["sigma"], c["seed"], d_vals.data_ptr(),
                                        d_idx.data_ptr(), d_norms.data_ptr(), 0))
    torch.cuda.synchronize()
    v = (d_vals / (d_norms[:, None] + 1e-9)).cpu().numpy()
    idx = d_idx.cpu().numpy()
    del d_vals, d_idx, d_norms
    torch.cuda.empty_cache()
    rowptr = (np.arange(n + 1, dtype=np.int64) * k).astype(np.int32)
    with tempfile.TemporaryDirectory(dir=args.tmp) as td:
        fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
        with open(fin, "wb") as f:
            f.write(struct.pack("<3q", n, m, n * k))
            f.write(rowptr.tobytes())
            f.write(idx.tobytes())
            f.write(v.tobytes())
        del v, idx
        res = subprocess.run([exe, fin, fout, str(r), str(args.iters), repr(bench.EPS), "1", "1"],
                             capture_output=True, text=True)
    sys.stdout.write(res.stdout[-3000:])
    if res.returncode != 0:
        sys.stderr.write(res.stderr[-3000:])
        raise SystemExit("ref_engine failed (exit %d)" % res.returncode)
    steps = re.findall(r"^step (\d+): ([0-9.eE+-]+) \[([0-9.eE+-]+) ms/step\]", res.stdout, flags=re.M)
    if steps:
        ms = [float(s[2]) for s in steps]
        print("reference engine, %s: %.2f ms/step (best 10-step window of %s) = %.2f iter/s"
              % (bench.workload_name(args.config, c), min(ms), [round(x, 2) for x in ms], 1000.0 / min(ms)))


if __name__ == "__main__":
    main()
