"""Builds the CUDA library in-tree: ``npeff_ref_b200/libdnpeff.so`` (sm_100a only).

Run as ``python -m npeff_ref_b200.build`` or through ``__graft_entry__.build()``.
nvcc cross-compiles without a GPU; the shared object is what the ctypes front
end, the tests and the benchmark load.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdnpeff.so")
CLI = os.path.join(HERE, "bin", "run_nmf_on_pefs")
CLI_FIT = os.path.join(HERE, "bin", "fit_coeffs_to_sparse_H")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(HERE, "..", "include", "dnpeff.h")]


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in _deps())


def build_cli():
    """The `run_nmf_on_pefs` and `fit_coeffs_to_sparse_H` executables: plain C++ over the C ABI."""
    os.makedirs(os.path.dirname(CLI), exist_ok=True)
    for exe, src in ((CLI, "run_nmf_on_pefs.cpp"), (CLI_FIT, "fit_coeffs_to_sparse_H.cpp")):
        cmd = ["g++", "-O2", "-std=c++17", "-o", exe, os.path.join(CSRC, src),
               "-L" + HERE, "-ldnpeff", "-Wl,-rpath,$ORIGIN/..", "-lpthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("g++ failed:\n" + res.stdout + res.stderr)
    return CLI


def build(force=False, verbose=False):
    if not force and not needs_build() and os.path.exists(CLI) and os.path.exists(CLI_FIT):
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
        ["-o", LIB] + _sources() + ["-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    build_cli()
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
