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
