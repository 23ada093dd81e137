"""D-NPEFF NMF benchmark: iterations/s of the multiplicative-update loop and the
HBM roofline of its dominant kernel, on synthetic D-PEFs of the headline workload, configuration 2
(n=20,000 examples, m=4,194,304 features, 32,768 stored values per row, r=128).

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --steps K --warmup W    # CPU baseline arm

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE).  At N > 1 the
SAME matrix is column-sharded over the ranks (strong scaling) and the per-shard
A*H^T and H*H^T partials are all-reduced with NCCL inside the engine.

A "step" is one NMF iteration: W update then H update.  `value` is timed with
the matrix resident in HBM; `e2e` is the same loop timed through the C ABI from
pinned HOST buffers: upload + normalise + prune + shard + K iterations + W and H
read back.  Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes as C
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: n, m, k, r, alpha, sigma, seed   (the benchmark's workload configurations, 1-based)
    1: dict(n=2048, m=65536, k=4096, r=32, alpha=1.1, sigma=1.0, seed=0),
    2: dict(n=20000, m=4194304, k=32768, r=128, alpha=1.1, sigma=1.0, seed=1),
    3: dict(n=50000, m=16777216, k=65536, r=256, alpha=1.1, sigma=1.0, seed=2),
    5: dict(n=50000, m=8388608, k=65536, r=512, alpha=1.4, sigma=2.0, seed=4),
    # coefficient fit only (H fixed, 90 % of it zero; W updated): not a headline line, a
    # measurement of the W-only path; on N GPUs the examples are split by rows, no exchange
    4: dict(n=200000, m=4194304, k=32768, r=256, alpha=1.1, sigma=1.0, seed=3, w_only=True),
}
EPS = 1e-12
METRIC = "dnpeff_nmf_iterations_per_s"
UNIT = "iter/s"

# dram__bytes_read.sum + dram__bytes_write.sum of one A*H^T product (a sequence of
# launches: the dense popular block on tensor cores + one launch per tail column
# block), keyed by (config, ranks, product).  Config 2 on one GPU: scaled from an ncu
# capture of the same workload with a tenth of the rows, where the product moved
# 3.06 GB: 2.01 GB are the dense factor H, read once whatever the row count; the
# other 1.05 GB (dense block of A, tail entries, split-K partials) grow with the
# rows: 2.15e9 (H at full size) + 10 * 1.05e9.
NCU_TRAFFIC_BYTES = {(2, 1, "spmm_ah"): 12.6e9}


def workload_name(cfg_id, c):
    return "config%d: n=%d m=%d k=%d r=%d zipf=%.1f sigma=%.0f seed=%d eps=%g" % (
        cfg_id, c["n"], c["m"], c["k"], c["r"], c["alpha"], c["sigma"], c["seed"], EPS)


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 200 ms (NVML, read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            }
            while True:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                if self._stop_evt.wait(0.2):
                    break
        except Exception as ex:  # no NVML: report that instead of clocks
            self.reasons.add("unsampled: %s" % type(ex).__name__)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ---------------------------------------------------------------------------
CPU_MAX_NNZ = 700 * 1000 * 1000   # entries of the CPU arm's matrix (host memory: ~40 bytes per entry and rank-128 factor rows)


def cpu_rows(c):
    """Rows of the workload the CPU arm iterates on: all of them while the matrix
    stays below CPU_MAX_NNZ stored entries, else the leading rows that fit."""
    return int(min(c["n"], max(1, CPU_MAX_NNZ // c["k"])))


def all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm is one process
    and is meant to use every host thread it may run on."""
    from oracle import oracle as O
    try:
        O.set_num_threads(len(os.sched_getaffinity(0)))
    except Exception:
        pass
    return O.num_threads()


def cpu_arm(c, vals, idx, norms, warmup, steps):
    """The CPU oracle (float-accumulating rendering, OpenMP over all host threads) on
    `vals/idx/norms` ([ns, k] arrays: the workload's leading ns rows, every column):
    normalise + prune + transpose once (untimed, like the GPU arm's resident load),
    then `warmup` + `steps` full iterations, each timed.  Returns (seconds per timed
    step as a list, description, cores, kept columns)."""
    from oracle import oracle as O
    cores = all_host_threads()
    ns, k = vals.shape
    t0 = time.perf_counter()
    prob = O.Problem(ns, c["m"], k, c["r"], vals, idx, norms, min_count=1, eps=EPS, seed=c["seed"])
    t_setup = time.perf_counter() - t0
    times = []
    for _ in range(max(warmup, 0) + max(steps, 1)):
        t0 = time.perf_counter()
        prob.step(acc64=False)
        times.append(time.perf_counter() - t0)
    timed = times[max(warmup, 0):]
    loss = prob.loss()
    m_kept = prob.m_kept
    prob.close()
    whole = ns == c["n"]
    desc = ("%s %d of %d rows, every column (%d kept), the same generator stream as the GPU arm; fp32-accumulating "
            "CPU oracle, %d OpenMP threads; %d warm-up + %d timed full iterations of %.2f s mean (setup %.0f s untimed); "
            "loss after them %.6f" % ("all" if whole else "the leading", ns, c["n"], m_kept, cores, max(warmup, 0),
                                      len(timed), float(np.mean(timed)), t_setup, loss))
    return timed, desc, cores, m_kept


def run_reference_arm(args, c, cfg_id):
    """`--impl reference`: the reference has no CPU implementation of this path (its
    engine is cuSPARSE/cuBLAS on a GPU); the timed CPU arm is the oracle port on all
    host threads, on the workload's own matrix: the host twin of the device generator
    draws the same column indices bit for bit.  Every step is one full iteration on
    all rows and all columns (configurations whose matrix exceeds CPU_MAX_NNZ entries:
    the leading rows that fit, rate scaled by the row ratio and marked extrapolated).
    No GPU is touched."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    all_host_threads()
    ns = cpu_rows(c)
    t0 = time.perf_counter()
    vals, idx, norms = O.synth_pef_hashed(ns, c["m"], c["k"], alpha=c["alpha"], sigma=c["sigma"], seed=c["seed"])
    t_gen = time.perf_counter() - t0
    timed, desc, cores, _ = cpu_arm(c, vals, idx, norms, args.warmup, args.steps)
    sec = float(np.mean(timed))
    extrapolated = ns != c["n"]
    if extrapolated:
        sec *= c["n"] / float(ns)
        desc += "; EXTRAPOLATED to %d rows by the row ratio" % c["n"]
    value = 1.0 / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * sec,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload_name(cfg_id, c), "generate_s": round(t_gen, 1)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc,
                         "extrapolated": extrapolated},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def ref_gpu_engine_ms_per_step(c, h_vals, h_idx, h_norms, iters=10):
    """The unmodified reference engine (cuSPARSE / cuBLAS / cuRAND / NCCL, compiled from
    the reference's own headers into oracle/_ref/ref_engine where that tree was
    mounted) on the same matrix: returns (ms per step as the engine itself prints it
    in its `step N: loss [ms/step]` line, None) or (None, reason)."""
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_engine")
    if not os.path.exists(exe):
        return None, "oracle/_ref/ref_engine is not built (the reference tree was not mounted at build time)"
    n, k = h_vals.shape
    if n * k >= 2 ** 31:
        return None, "the reference engine stops at 2^31 stored entries per device (cublasSnrm2 guard)"
    import re
    import struct
    import tempfile
    tmp = "/dev/shm" if os.path.isdir("/dev/shm") else None
    try:
        with tempfile.TemporaryDirectory(dir=tmp) as td:
            fin, fout = os.path.join(td, "in.bin"), os.path.join(td, "out.bin")
            with open(fin, "wb") as f:
                f.write(struct.pack("<3q", n, c["m"], n * k))
                (np.arange(n + 1, dtype=np.int64) * k).astype(np.int32).tofile(f)
                h_idx.tofile(f)
                (h_vals / (h_norms[:, None] + np.float32(1e-9))).astype(np.float32).tofile(f)
            res = subprocess.run([exe, fin, fout, str(c["r"]), str(iters), repr(EPS), str(c["seed"]), "1", "timing"],
                                 capture_output=True, text=True, timeout=600)
        if res.returncode != 0:
            return None, "ref_engine exited %d: %s" % (res.returncode, res.stderr[-300:].replace("\n", " "))
        found = re.findall(r"step \d+: \S+ \[([0-9.eE+-]+) ms/step\]", res.stdout)
        if not found:
            return None, "ref_engine printed no step line"
        return float(found[-1]), None
    except Exception as ex:  # disk space, time-out
        return None, "%s: %s" % (type(ex).__name__, str(ex)[:200])


# ---------------------------------------------------------------------------
def run_w_only(args, c, cfg_id):
    """Config 4: H fixed (Uniform(0,1), 90 % zeroed), `steps` W-only multiplicative updates
    (`dnpeff_fit_w_only`: A*H^T and H*H^T once, then W *= AH / (W*HH + eps) per step).  The
    rows of W are independent given H, so on N GPUs the examples are split by rows
    (dnpeff_row_slice), H is replicated and there is no exchange at all: every rank runs
    its own engine; the job's rate is that of the slowest rank."""
    import torch
    import torch.distributed as dist
    from npeff_ref_b200 import MuNmf, MuNmfParams
    from npeff_ref_b200._lib import lib, check
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n, m, k, r = c["n"], c["m"], c["k"], c["r"]
    row_b, row_c = MuNmf.row_slice(n, world, rank)
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    stream = side.cuda_stream
    d_vals = torch.empty((row_c, k), dtype=torch.float32, device="cuda")
    d_idx = torch.empty((row_c, k), dtype=torch.int32, device="cuda")
    d_norms = torch.empty((row_c,), dtype=torch.float32, device="cuda")
    check(lib().dnpeff_synth_pef_device_rows(row_b, row_c, m, k, c["alpha"], c["sigma"], c["seed"], d_vals.data_ptr(),
                                             d_idx.data_ptr(), d_norms.data_ptr(), stream))
    eng = MuNmf(MuNmfParams(rank=r, eps=1e-7, seed=c["seed"]), device=local_rank, stream=stream)
    # every column is kept (threshold 0), as with the retained-column list of a decomposition
    # file: all ranks then share one H
    eng.set_csr_device(row_c, m, d_vals.data_ptr(), d_idx.data_ptr(), 0, k, d_norms.data_ptr(), 0)
    del d_vals, d_idx, d_norms
    torch.cuda.empty_cache()
    _, m_kept, _, ms, nnz = eng.shape
    g = torch.Generator(device="cuda").manual_seed(c["seed"])
    H = torch.rand((r, ms), generator=g, device="cuda")
    H = (H * (torch.rand((r, ms), generator=g, device="cuda") > 0.9)).cpu().numpy()
    check(lib().dnpeff_set_w_row_offset(eng._h, row_b))   # W rows as the unsplit run would draw them
    eng.init_factors(None, H)
    del H

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        eng.fit_w_only(iters, want_loss=False)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        timed(1)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    launches0 = eng.launch_count()
    stage1 = min(timed(0) for _ in range(3))           # A*H^T + H*H^T alone
    total = timed(args.steps)
    launches = eng.launch_count() - launches0
    clocks = sampler.stop()
    per_step = max(total - stage1, 0.0) / max(args.steps, 1)
    # loss of the whole job: the row blocks' squared losses add
    l2 = torch.tensor([eng.fit_w_only(0) ** 2, float(nnz)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(l2)
    loss, nnz_job = math.sqrt(float(l2[0].item())), int(l2[1].item())
    if rank == 0:
        upd_bytes = 3 * 4.0 * row_c * r
        print(json.dumps({
            "metric": "dnpeff_w_only_fit_iterations_per_s", "value": 1e3 / per_step if per_step > 0 else None,
            "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(cfg_id, c).replace("eps=%g" % EPS, "eps=1e-07") + " W-only, H 90% zero",
                       "n_cols_kept": m_kept, "nnz": nnz_job, "rows_per_rank": row_c, "shard": "rows/%d, no exchange" % world,
                       "stage1_ms": stage1, "stage1_spmm_GBps": (8.0 * nnz + 4.0 * r * ms + 4.0 * row_c * r) / (stage1 * 1e-3) / 1e9,
                       "loss_after": loss,
                       "l2": "inputs larger than L2 (A %.1f GB, H %.2f GB per rank)" % (8.0 * nnz / 1e9, 4.0 * r * ms / 1e9)},
            "roofline": {"bound": "hbm", "kernel": "mu_update (W side)", "achieved": upd_bytes / (per_step * 1e-3) / 1e9
                         if per_step > 0 else None, "peak": measured_peak_hbm()[0], "unit": "GB/s",
                         "frac": (upd_bytes / (per_step * 1e-3) / 1e9) / measured_peak_hbm()[0] if per_step > 0 else None,
                         "peak_kind": "of " + measured_peak_hbm()[1], "traffic": None,
                         "algorithmic_bytes_per_launch": upd_bytes},
            "cpu_baseline": None, "e2e": None, "gpu_launches": launches, "clocks": clocks}), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument("--no-ref-gpu-engine", action="store_true",
                    help="skip the run of the unmodified reference engine on the same GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--scale-rows", type=float, default=1.0,
                    help="shrink n (profiling captures on a small case); not a bench value")
    ap.add_argument("--scale-cols", type=float, default=1.0,
                    help="shrink m and k alike (profiling captures on a small case); not a bench value")
    args = ap.parse_args()
    cfg_id = args.config
    c = dict(CONFIGS[cfg_id])
    if args.scale_rows != 1.0:
        c["n"] = max(1, int(c["n"] * args.scale_rows))
    if args.scale_cols != 1.0:
        c["m"] = max(1, int(c["m"] * args.scale_cols))
        c["k"] = max(1, min(c["m"], int(c["k"] * args.scale_cols)))
    if c.get("w_only"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "config 4 (W-only fit) is timed on the GPU arm only"}))
            return
        return run_w_only(args, c, cfg_id)
    if args.impl == "reference":
        return run_reference_arm(args, c, cfg_id)

    import torch
    import torch.distributed as dist
    from npeff_ref_b200 import MuNmf, MuNmfParams
    from npeff_ref_b200._lib import lib, check

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch with torchrun --nproc-per-node %d"
                         % (args.gpus, world, args.gpus))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n, m, k, r = c["n"], c["m"], c["k"], c["r"]
    warm = max(args.warmup, 3)
    # a side stream made current: the engine launches on it and torch's events,
    # copies and collectives see the same stream (the legacy default stream is 0,
    # which the C ABI reads as "make your own")
    side = torch.cuda.Stream()
    torch.cuda.set_stream(side)
    stream = side.cuda_stream

    # ---- synthetic D-PEF arrays, generated in HBM (every rank: the same matrix)
    d_vals = torch.empty((n, k), dtype=torch.float32, device="cuda")
    d_idx = torch.empty((n, k), dtype=torch.int32, device="cuda")
    d_norms = torch.empty((n,), dtype=torch.float32, device="cuda")
    t0 = time.perf_counter()
    check(lib().dnpeff_synth_pef_device(n, m, k, c["alpha"], c["sigma"], c["seed"],
                                        d_vals.data_ptr(), d_idx.data_ptr(), d_norms.data_ptr(),
                                        stream))
    t_gen = time.perf_counter() - t0

    def make_engine():
        return MuNmf(MuNmfParams(rank=r, eps=EPS, seed=c["seed"]), device=local_rank,
                     shard_index=rank, n_shards=world, stream=stream,
                     shard_mode=MuNmf.CYCLIC if world > 1 else MuNmf.CONTIGUOUS)

    def join(eng):
        if world > 1:
            box = [MuNmf.make_unique_id() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            eng.init_comm(box[0])

    def global_scale(eng):
        # Uniform(0,1) * sqrt(mean(A)/r), mean over all n * m_kept entries
        s = torch.tensor([eng.a_sum()], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(s)
        return math.sqrt(float(s.item()) / (n * eng.shape[1]) / r)

    # The rows this rank will hand to the end-to-end loader (and rank 0 to the CPU arm)
    # go to pinned host memory now, so that the generator's device arrays can be
    # released as soon as the resident engine has loaded them (at configuration 3 they
    # are 26 GB beside a 130 GB engine).
    need_host = (not args.no_e2e) or (rank == 0 and world == 1 and not (args.no_cpu_baseline and args.no_ref_gpu_engine))
    h_vals = h_idx = h_norms = None
    row_b, row_c = MuNmf.row_slice(n, world, rank)
    if need_host:
        h_vals = torch.empty((row_c, k), dtype=torch.float32, pin_memory=True)
        h_idx = torch.empty((row_c, k), dtype=torch.int32, pin_memory=True)
        h_norms = torch.empty((row_c,), dtype=torch.float32, pin_memory=True)
        h_vals.copy_(d_vals[row_b:row_b + row_c])
        h_idx.copy_(d_idx[row_b:row_b + row_c])
        h_norms.copy_(d_norms[row_b:row_b + row_c])
        torch.cuda.synchronize()

    eng = make_engine()
    t0 = time.perf_counter()
    eng.set_csr_device(n, m, d_vals.data_ptr(), d_idx.data_ptr(), 0, k, d_norms.data_ptr(), 1)
    t_load = time.perf_counter() - t0
    del d_vals, d_idx, d_norms
    torch.cuda.empty_cache()
    join(eng)
    eng.set_init_scale(global_scale(eng))
    eng.init_factors()
    _, m_kept, c0, ms, nnz = eng.shape
    layout = eng.layout()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warm):
        eng.step_w()
        eng.step_h()
    barrier()
    loss_before = eng.compute_uncached_loss()

    # ---- timed region: K iterations, matrix resident in HBM ---------------------
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    eng.enable_timing(True)
    eng.get_timing()
    launches0 = eng.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        eng.step_w()
        eng.step_h()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = eng.launch_count() - launches0
    timing = eng.get_timing()
    eng.enable_timing(False)
    clocks = sampler.stop()
    loss_after = eng.compute_uncached_loss()
    t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    value = 1000.0 / ms_per_step

    # ---- roofline of the dominant kernel (this rank's shard) --------------------
    spmm_bytes = 8.0 * nnz + 4.0 * r * ms + 4.0 * n * r
    per_kernel = {name: (tot / cnt if cnt else None) for name, (tot, cnt) in timing.items()}
    dom = max(("spmm_ah", "spmm_wa"), key=lambda kname: timing[kname][0])
    peak, peak_kind = measured_peak_hbm()
    achieved = spmm_bytes / (per_kernel[dom] * 1e-3) / 1e9
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_kind": "of " + peak_kind,
        "traffic": NCU_TRAFFIC_BYTES.get((cfg_id, world, dom)),
        "algorithmic_bytes_per_launch": spmm_bytes,
        "ms_per_launch": {a: (round(b, 4) if b is not None else None) for a, b in per_kernel.items()},
        # what actually bounds the product at r >= 64: the tail entries' gather of one
        # 4r-byte factor row each through the L2->SM read ports (64 B/clk/SM).  Lower bound
        # of the rate: the whole product's time is charged to the gather, although the
        # dense popular block (tensor cores) is part of it.
        "l2_gather": {"bytes_per_launch": 4.0 * r * (nnz - layout[1]),
                      "achieved_TBps_lower_bound": 4.0 * r * (nnz - layout[1]) / (per_kernel[dom] * 1e-3) / 1e12,
                      "port_peak_TBps": 148 * 64 * (clocks["sm_mhz"] or 1965.0) * 1e6 / 1e12,
                      "what": "tail entries x 4r bytes / product time, against 148 SMs x 64 B/clk at the sampled SM clock"},
        "note": "one product = the dense popular block on tensor cores + one launch per tail column block, timed as a whole; "
                "every stored entry gathers r floats on chip (shared memory or L2), so the SpMM is not "
                "HBM-bound for r >= 64; traffic is scaled from a small-case capture",
    }
    # the loss after exactly K iterations from the seeded initial factors: what the
    # end-to-end run below must arrive at (untimed)
    loss_k_resident = None
    if not args.no_e2e:
        eng.init_factors()
        for _ in range(args.steps):
            eng.step_w()
            eng.step_h()
        loss_k_resident = eng.compute_uncached_loss()
    eng.close()

    # ---- e2e: host buffers -> loader -> K iterations -> W,H back, through the C ABI
    e2e = None
    if not args.no_e2e:
        # every rank hands the loader the rows it holds in pinned host memory: the whole
        # matrix on one GPU, its slice of the rows (dnpeff_row_slice) otherwise
        W_out = torch.empty((n, r), dtype=torch.float32, pin_memory=True)
        H_out = torch.empty((r, ms), dtype=torch.float32, pin_memory=True)
        eng2 = make_engine()
        join(eng2)
        barrier()
        ev0.record()
        tw = [time.perf_counter()]
        check(lib().dnpeff_set_csr_rows(eng2._h, n, m, k, row_b, row_c, None, h_vals.data_ptr(), h_idx.data_ptr(),
                                        h_norms.data_ptr(), 1))
        tw.append(time.perf_counter())
        eng2.set_init_scale(global_scale(eng2))
        eng2.init_factors()
        for _ in range(args.steps):
            eng2.step_w()
            eng2.step_h()
        eng2.synchronize()
        tw.append(time.perf_counter())
        check(lib().dnpeff_get_w(eng2._h, W_out.data_ptr()))
        check(lib().dnpeff_get_h(eng2._h, H_out.data_ptr()))
        tw.append(time.perf_counter())
        ev1.record()
        barrier()
        te = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item())
        # bytes of this rank; the job's total is the sum over the ranks
        h2d = h_vals.numel() * 4 + h_idx.numel() * 4 + h_norms.numel() * 4
        d2h = W_out.numel() * 4 + H_out.numel() * 4
        tb = torch.tensor([h2d, d2h], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(tb)
        h2d_job, d2h_job = float(tb[0].item()), float(tb[1].item())
        loss_k_e2e = eng2.compute_uncached_loss()
        e2e = {"value": args.steps / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": h2d_job / args.steps, "d2h_bytes_per_step": d2h_job / args.steps,
               "h2d_bytes_per_step_per_rank": h2d / args.steps,
               "ms_total": e2e_ms,
               "host_ms": {"load": round(1e3 * (tw[1] - tw[0]), 1), "iterate": round(1e3 * (tw[2] - tw[1]), 1),
                           "read_back": round(1e3 * (tw[3] - tw[2]), 1)},
               "what": "dnpeff_set_csr_rows from pinned host arrays: every rank uploads its 1/N of the rows; "
                       "column counts all-reduced, entries exchanged over NVLink to the rank owning their column; "
                       "normalise, prune, shard, CSC + init + K iterations + dnpeff_get_w/get_h into pinned host arrays",
               # the end-to-end run against the resident run after the same K iterations
               # from the same seeded factors (the slab-pipelined loader against the device loader)
               "self_check": {"loss_after_k_resident": loss_k_resident, "loss_after_k_e2e": loss_k_e2e,
                              "rel_diff": abs(loss_k_e2e - loss_k_resident) / max(abs(loss_k_resident), 1e-300)}}
        if e2e["self_check"]["rel_diff"] > 1e-6:
            raise SystemExit("end-to-end run disagrees with the resident run: %r" % (e2e["self_check"],))
        eng2.close()
        host_arrays = (h_vals.numpy(), h_idx.numpy(), h_norms.numpy())
    else:
        host_arrays = None

    # ---- CPU baseline and the reference's own GPU engine, rank 0 of a 1-GPU run only
    cpu = None
    ref_gpu = None
    if rank == 0 and world == 1 and (not args.no_cpu_baseline or not args.no_ref_gpu_engine):
        if host_arrays is None:
            host_arrays = (h_vals.numpy(), h_idx.numpy(), h_norms.numpy())
        if not args.no_ref_gpu_engine:
            ms_ref, why = ref_gpu_engine_ms_per_step(c, *host_arrays)
            ref_gpu = {"ms_per_step": ms_ref, "unavailable": why,
                       "what": "the unmodified reference engine (cuSPARSE/cuBLAS, oracle/_ref/ref_engine) on the same "
                               "matrix and GPU; its own `step N: loss [ms/step]` print after 10 iterations"}
        if not args.no_cpu_baseline:
            ns = cpu_rows(c)
            timed, desc, cores, _ = cpu_arm(c, host_arrays[0][:ns], host_arrays[1][:ns], host_arrays[2][:ns], 0, 1)
            sec = float(np.mean(timed)) * (n / float(ns))
            cpu = {"value": 1.0 / sec, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc,
                   "extrapolated": ns != n}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(cfg_id, c), "n_cols_kept": m_kept,
                       "nnz_per_rank": nnz, "popular_cols": layout[0], "popular_nnz": layout[1],
                       "tail_blocks": layout[2], "shard": "columns/%d%s" % (world, " cyclic" if world > 1 else ""),
                       "l2": "inputs larger than L2 (A %.1f GB, H %.2f GB per rank)" % (
                           16.0 * nnz / 1e9, 4.0 * r * ms / 1e9),
                       "setup_s": {"generate": round(t_gen, 2), "load_resident": round(t_load, 2)},
                       "loss_before_timed": loss_before, "loss_after_timed": loss_after},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks, "ref_gpu_engine": ref_gpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
