"""Shared test helpers: seeded synthetic D-PEF problems and comparison metrics."""
import numpy as np

from oracle import oracle as O


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b)
    return np.linalg.norm(a - b) / (d if d > 0 else 1.0)


def make_problem(n, m, k, seed, alpha=1.1, sigma=1.0):
    """Unnormalised top-k D-PEF rows as the file holds them, plus row norms."""
    vals, idx, norms = O.synth_pef(n, m, k, alpha=alpha, sigma=sigma, seed=seed)
    return vals, idx, norms


def oracle_preprocess(vals, idx, norms, m, min_count=1):
    """normalise -> prune, on the CPU: (vals, colind, rowptr, new_to_og)."""
    n, k = vals.shape
    rowptr = np.arange(n + 1, dtype=np.int64) * k
    v = O.normalize_rows(vals.ravel(), rowptr, norms)
    return O.prune_columns(v, idx.ravel(), rowptr, m, min_count)


def baseline_scale(vals_pruned, n, m_kept, r):
    """sqrt(mean(A)/r) with mean over all n*m_kept entries of the pruned matrix."""
    return float(np.sqrt(vals_pruned.astype(np.float64).sum() / (n * m_kept) / r))


def curand_xorwow_uniform(seed, counts):
    """The reference engine's initial factors: it draws W and then H with
    curandGenerateUniform from one cuRAND generator of the default pseudo-random type,
    seeded per device (multi_mu_dense_factors_device_contexts1.h:197-207,373-375).
    Re-creating that generator and repeating its calls (same seed, same counts, same
    order) reproduces them, which lets a fixture store the seed instead of the
    initial factors.  Needs a CUDA device and libcurand; returns float32 arrays."""
    import ctypes
    import torch
    lib = None
    for name in ("libcurand.so.10", "libcurand.so"):
        try:
            lib = ctypes.CDLL(name)
            break
        except OSError:
            continue
    if lib is None:
        raise RuntimeError("libcurand not found")
    gen = ctypes.c_void_p()
    CURAND_RNG_PSEUDO_DEFAULT = 100
    assert lib.curandCreateGenerator(ctypes.byref(gen), CURAND_RNG_PSEUDO_DEFAULT) == 0
    assert lib.curandSetPseudoRandomGeneratorSeed(gen, ctypes.c_ulonglong(int(seed))) == 0
    out = []
    for count in counts:
        t = torch.empty(int(count), dtype=torch.float32, device="cuda")
        assert lib.curandGenerateUniform(gen, ctypes.c_void_p(t.data_ptr()), ctypes.c_size_t(int(count))) == 0
        torch.cuda.synchronize()
        out.append(t.cpu().numpy())
    lib.curandDestroyGenerator(gen)
    return out
