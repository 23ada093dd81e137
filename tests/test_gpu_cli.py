"""The `run_nmf_on_pefs` drop-in executable end to end on a GPU: D-PEF file in,
decomposition file out, same flags and progress lines as the reference
(cc/cuda_d_npeff/mains/run_nmf_on_pefs.cu), checked against the CPU oracle."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from oracle import oracle as O
from helpers import rel_fro, make_problem, oracle_preprocess
from npeff_ref_b200._lib import lib, check

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "npeff_ref_b200", "bin", "run_nmf_on_pefs")
SEED = 43190432042  # compiled into the reference executable (run_nmf_on_pefs.cu:190)


def _write_pef(path, vals, idx, norms, dense):
    n, k = vals.shape
    check(lib().dnpeff_write_pef_hdf5(path.encode(), n, k, C.c_void_p(vals.ctypes.data),
                                      C.c_void_p(idx.ctypes.data), C.c_void_p(norms.ctypes.data), dense))


def _read_decomp(path):
    a, b, c, d = C.c_int64(0), C.c_int32(0), C.c_int64(0), C.c_int64(0)
    check(lib().dnpeff_decomposition_hdf5_info(path.encode(), C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    W = np.empty((a.value, b.value), np.float32)
    H = np.empty((b.value, c.value), np.float32)
    kept = np.empty(c.value, np.int32)
    check(lib().dnpeff_read_decomposition_hdf5(path.encode(), C.c_void_p(W.ctypes.data),
                                               C.c_void_p(H.ctypes.data), C.c_void_p(kept.ctypes.data)))
    return W, H, kept, d.value


def _run(*flags):
    res = subprocess.run([CLI] + list(flags), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    return res.stdout


def test_cli_matches_oracle_and_writes_reference_layout(tmp_path):
    n, m, k, r, iters = 120, 4000, 90, 16, 30
    vals, idx, norms = make_problem(n, m, k, seed=61)
    pef, out = str(tmp_path / "pef.h5"), str(tmp_path / "nmf.h5")
    _write_pef(pef, vals, idx, norms, m)
    stdout = _run("--per_example_fishers=" + pef, "--output_path=" + out, "--nmf_n_components=%d" % r,
                  "--nmf_max_iter=%d" % iters, "--min_values_per_parameter=2", "--some_unknown_flag=1")
    W, H, kept, dense = _read_decomp(out)
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m, 2)
    mk = len(n2o)
    assert dense == m and np.array_equal(kept, n2o)
    assert W.shape == (n, r) and H.shape == (r, mk)
    W0, H0 = O.init_factors(n, mk, r, SEED, 1.0)           # unscaled U(0,1], eps 1e-8: the reference's defaults
    Wo, Ho, ls = O.run(v, c, rp, mk, W0, H0, iters, 1e-8, losses=True)
    assert rel_fro(W, Wo) < 1e-4 and rel_fro(H, Ho) < 1e-4
    # "step N: <loss> [<ms> ms/step]" every 10 steps (multi_mu_dense_factors_nmf1.h:198)
    steps = re.findall(r"^step (\d+): ([0-9.eE+-]+) \[([0-9.eE+-]+) ms/step\]$", stdout, flags=re.M)
    assert [int(s[0]) for s in steps] == [10, 20, 30]
    for s in steps:
        assert abs(float(s[1]) - ls[int(s[0]) - 1]) < 1e-4 * ls[int(s[0]) - 1]   # printed with 6 digits


def test_cli_leading_hyperslab_flags(tmp_path):
    n, m, k, r = 80, 2000, 64, 8
    vals, idx, norms = make_problem(n, m, k, seed=62)
    pef, out = str(tmp_path / "pef.h5"), str(tmp_path / "nmf.h5")
    _write_pef(pef, vals, idx, norms, m)
    _run("--per_example_fishers=" + pef, "--output_path=" + out, "--nmf_n_components=%d" % r,
         "--nmf_max_iter=5", "--n_examples=50", "--n_fisher_values=40", "--log_every=0")
    W, H, kept, _ = _read_decomp(out)
    v, c, rp, n2o = oracle_preprocess(vals[:50, :40], idx[:50, :40], norms[:50], m, 1)
    assert np.array_equal(kept, n2o) and W.shape == (50, r)
    W0, H0 = O.init_factors(50, len(n2o), r, SEED, 1.0)
    Wo, Ho = O.run(v, c, rp, len(n2o), W0, H0, 5, 1e-8)
    assert rel_fro(W, Wo) < 1e-4 and rel_fro(H, Ho) < 1e-4


def test_cli_resume_from_initial_factor_files(tmp_path):
    """--initial_W_path / --initial_H_path (parsed but dead in the reference,
    run_nmf_on_pefs.cu:131-156): 10 + 10 iterations equal 20 in one go, bit for bit."""
    n, m, k, r = 100, 3000, 80, 12
    vals, idx, norms = make_problem(n, m, k, seed=63)
    pef = str(tmp_path / "pef.h5")
    _write_pef(pef, vals, idx, norms, m)
    common = ["--per_example_fishers=" + pef, "--nmf_n_components=%d" % r, "--log_every=0", "--n_devices=1"]
    a, b, full = str(tmp_path / "a.h5"), str(tmp_path / "b.h5"), str(tmp_path / "full.h5")
    _run(*common, "--output_path=" + a, "--nmf_max_iter=10")
    _run(*common, "--output_path=" + b, "--nmf_max_iter=10", "--initial_W_path=" + a, "--initial_H_path=" + a)
    _run(*common, "--output_path=" + full, "--nmf_max_iter=20")
    Wb, Hb, kb, _ = _read_decomp(b)
    Wf, Hf, kf, _ = _read_decomp(full)
    assert np.array_equal(kb, kf) and np.array_equal(Wb, Wf) and np.array_equal(Hb, Hf)


def test_cli_periodic_checkpoint_resumes_bit_for_bit(tmp_path):
    """--checkpoint_every=K writes <output_path>.checkpoint after every K-th step (a
    decomposition file, written under a temporary name and renamed).  A run continued
    from the checkpoint of step 10 for the remaining 10 steps ends exactly where the
    uninterrupted 20-step run ends, and the step numbers of the log continue."""
    n, m, k, r = 100, 3000, 80, 12
    vals, idx, norms = make_problem(n, m, k, seed=64)
    pef = str(tmp_path / "pef.h5")
    _write_pef(pef, vals, idx, norms, m)
    common = ["--per_example_fishers=" + pef, "--nmf_n_components=%d" % r, "--n_devices=1"]
    full, part, cont = str(tmp_path / "full.h5"), str(tmp_path / "part.h5"), str(tmp_path / "cont.h5")
    out_full = _run(*common, "--output_path=" + full, "--nmf_max_iter=20", "--checkpoint_every=10")
    assert "Checkpoint after step 10 written to " + full + ".checkpoint" in out_full
    assert [int(x) for x in re.findall(r"^step (\d+):", out_full, flags=re.M)] == [10, 20]
    assert os.path.exists(full + ".checkpoint") and not os.path.exists(full + ".checkpoint.tmp")
    # the checkpoint IS the state after 10 steps ...
    _run(*common, "--output_path=" + part, "--nmf_max_iter=10", "--log_every=0")
    Wc, Hc, kc, _ = _read_decomp(full + ".checkpoint")
    Wp, Hp, kp, _ = _read_decomp(part)
    assert np.array_equal(kc, kp) and np.array_equal(Wc, Wp) and np.array_equal(Hc, Hp)
    # ... and a run continued from it ends where the uninterrupted one ends
    ck = full + ".checkpoint"
    _run(*common, "--output_path=" + cont, "--nmf_max_iter=10", "--initial_W_path=" + ck, "--initial_H_path=" + ck,
         "--log_every=0")
    Wf, Hf, kf, _ = _read_decomp(full)
    Wr, Hr, kr, _ = _read_decomp(cont)
    assert np.array_equal(kf, kr) and np.array_equal(Wf, Wr) and np.array_equal(Hf, Hr)


def test_cli_truncated_input_file_fails_cleanly(tmp_path):
    """A D-PEF file cut short (host-side fault injection): the executable reports the
    read error and exits non-zero; nothing hangs and nothing is written."""
    n, m, k = 60, 1000, 50
    vals, idx, norms = make_problem(n, m, k, seed=65)
    pef, cut, out = str(tmp_path / "pef.h5"), str(tmp_path / "cut.h5"), str(tmp_path / "nmf.h5")
    _write_pef(pef, vals, idx, norms, m)
    data = open(pef, "rb").read()
    open(cut, "wb").write(data[:len(data) - 8000])
    res = subprocess.run([CLI, "--per_example_fishers=" + cut, "--output_path=" + out, "--nmf_n_components=4",
                          "--nmf_max_iter=2"], capture_output=True, text=True, timeout=300)
    assert res.returncode != 0 and not os.path.exists(out)
    assert "run_nmf_on_pefs" in res.stderr


def test_cli_missing_required_flag_aborts():
    res = subprocess.run([CLI, "--output_path=/tmp/x.h5"], capture_output=True, text=True)
    assert res.returncode != 0 and "Missing flag: per_example_fishers" in res.stdout


CLI_FIT = os.path.join(ROOT, "npeff_ref_b200", "bin", "fit_coeffs_to_sparse_H")


def _read_sparse(path):
    a, b, c, d, e = C.c_int64(0), C.c_int32(0), C.c_int64(0), C.c_int64(0), C.c_int64(0)
    check(lib().dnpeff_sparse_decomposition_hdf5_info(path.encode(), C.byref(a), C.byref(b), C.byref(c),
                                                      C.byref(d), C.byref(e)))
    W = np.empty((a.value, b.value), np.float32)
    rp = np.empty(b.value + 1, np.int64)
    ci = np.empty(max(d.value, 1), np.int32)
    va = np.empty(max(d.value, 1), np.float32)
    kept = np.empty(c.value, np.int32)
    check(lib().dnpeff_read_sparse_decomposition_hdf5(
        path.encode(), C.c_void_p(W.ctypes.data), C.c_void_p(rp.ctypes.data), C.c_void_p(ci.ctypes.data),
        C.c_void_p(va.ctypes.data), C.c_void_p(kept.ctypes.data)))
    return W, rp, ci[:d.value], va[:d.value], kept, e.value


def test_fit_coeffs_cli_matches_oracle_and_is_chunk_invariant(tmp_path):
    """fit_coeffs_to_sparse_H end to end (mains/fit_coeffs_to_sparse_H.cu): sparse
    decomposition + new D-PEFs in, W for the new examples + the same sparse H out;
    --n_row_splits_pefs must not change the result."""
    n, m, k, r, iters = 150, 4000, 80, 12, 40
    vals, idx, norms = make_problem(n, m, k, seed=71)
    rng = np.random.default_rng(7)
    kept = np.sort(rng.choice(np.unique(idx), 1200, replace=False)).astype(np.int32)
    mk = len(kept)
    Hd = (rng.random((r, mk), dtype=np.float32) * (rng.random((r, mk)) > 0.9)).astype(np.float32)
    hv, hrp, hc = O.dense_to_csr(Hd, 1e-30)
    W_old = rng.random((33, r), dtype=np.float32)            # the old examples' W is not used
    pef, hpath = str(tmp_path / "pef.h5"), str(tmp_path / "sp.h5")
    _write_pef(pef, vals, idx, norms, m)
    check(lib().dnpeff_save_sparse_decomposition_hdf5(
        hpath.encode(), C.c_void_p(W_old.ctypes.data), 33, r, C.c_void_p(hrp.ctypes.data),
        C.c_void_p(hc.ctypes.data), C.c_void_p(hv.ctypes.data), C.c_void_p(kept.ctypes.data), mk, m))
    outs = []
    for splits in (1, 4):
        out = str(tmp_path / ("out%d.h5" % splits))
        res = subprocess.run([CLI_FIT, "--pef_path=" + pef, "--H_path=" + hpath, "--output_path=" + out,
                              "--n_splits_sparse_matmul=2", "--n_row_splits_pefs=%d" % splits,
                              "--nmf_max_iter=%d" % iters], capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stdout + res.stderr
        outs.append((_read_sparse(out), res.stdout))
    (W, rp, ci, va, k2, dense), stdout = outs[0]
    assert W.shape == (n, r) and dense == m
    assert np.array_equal(rp, hrp) and np.array_equal(ci, hc) and np.array_equal(va, hv) and np.array_equal(k2, kept)
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    nv = O.normalize_rows(vals.ravel(), rowptr, norms)
    v, c, rpo = O.retain_columns(nv, idx.ravel(), rowptr, m, kept)
    W0 = O.init_factors(n, mk, r, SEED, 1.0)[0]
    Wo, lo = O.fit_w_only(v, c, rpo, mk, W0, Hd, iters, 1e-7)
    assert rel_fro(W, Wo) < 1e-4
    step = re.findall(r"^step (\d+): ([0-9.eE+-]+) \[", stdout, flags=re.M)
    assert len(step) == 1 and int(step[0][0]) == iters and abs(float(step[0][1]) - lo) < 1e-4 * lo
    # four row chunks: the same W (rows are independent given H; a chunk may order the
    # sums of A*H^T differently, so equality is to rounding), the same loss
    W4 = outs[1][0][0]
    assert rel_fro(W4, W) < 1e-5
    step4 = re.findall(r"^step (\d+): ([0-9.eE+-]+) \[", outs[1][1], flags=re.M)
    assert abs(float(step4[0][1]) - lo) < 1e-4 * lo


def test_fit_coeffs_cli_rejects_unknown_and_missing_flags(tmp_path):
    res = subprocess.run([CLI_FIT, "--pef_path=x"], capture_output=True, text=True, timeout=60)
    assert res.returncode != 0 and "Missing flag:" in res.stdout
    res = subprocess.run([CLI_FIT, "--pef_path=x", "--H_path=y", "--output_path=z", "--n_splits_sparse_matmul=1",
                          "--n_row_splits_pefs=1", "--nmf_max_iter=1", "--bogus=1"],
                         capture_output=True, text=True, timeout=60)
    assert res.returncode != 0 and "Unrecognized flags." in res.stdout


def test_cli_sparsity_flag_is_inert_unless_the_projection_is_asked_for(tmp_path):
    """--sparsity_W alone leaves the output unchanged (the reference builds the Hoyer
    context from it and never calls it, multi_mu_dense_factors_nmf1.h:162);
    --sparsify_initial_W=1 makes the commented-out call: the initial W is projected onto
    L1 = sparsity_W, L2 = 1 before the first step."""
    n, m, k, r, iters = 100, 3000, 80, 8, 10
    vals, idx, norms = make_problem(n, m, k, seed=71)
    pef = str(tmp_path / "pef.h5")
    _write_pef(pef, vals, idx, norms, m)
    common = ["--per_example_fishers=" + pef, "--nmf_n_components=%d" % r, "--nmf_max_iter=%d" % iters]
    outs = [str(tmp_path / ("o%d.h5" % i)) for i in range(3)]
    _run(*common, "--output_path=" + outs[0])
    _run(*common, "--output_path=" + outs[1], "--sparsity_W=4.0")
    stdout = _run(*common, "--output_path=" + outs[2], "--sparsity_W=4.0", "--sparsify_initial_W=1")
    Wa, Ha, _, _ = _read_decomp(outs[0])
    Wb, Hb, _, _ = _read_decomp(outs[1])
    Wc, Hc, kept, _ = _read_decomp(outs[2])
    assert np.array_equal(Wa, Wb) and np.array_equal(Ha, Hb)
    assert re.search(r"Projected the initial W onto L1 = 4, L2 = 1: \d+ passes\.", stdout)
    # against the oracle: project the generated W0, then the same iterations
    v, c, rp, n2o = oracle_preprocess(vals, idx, norms, m, 1)
    mk = len(n2o)
    W0, H0 = O.init_factors(n, mk, r, SEED, 1.0)
    W0p, _, conv = O.hoyer_project(W0, 4.0, 1.0, rule=0)
    assert conv
    Wo, Ho = O.run(v, c, rp, mk, W0p, H0, iters, 1e-8)
    assert rel_fro(Wc, Wo) < 1e-4 and rel_fro(Hc, Ho) < 1e-4
    assert rel_fro(Wc, Wa) > 1e-2
