"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

Only tests/, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module.  The shipped
package never does.

Layouts at this boundary follow the reference's files: ``W`` is ``[n, r]``
row-major and ``H`` is ``[r, m]`` row-major (io/nmf_decomp_h5.h:38-89).  The C
side works on ``Ht = H.T`` (``[m, r]``, the reference's device layout), so the
wrappers transpose.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libdnpeff_oracle.so")
_lib = None


def build(force=False):
    """Compile the C restatement with the committed Makefile."""
    src = os.path.join(_HERE, "dnpeff_oracle.c")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_loss.restype = C.c_double
        _lib.oracle_fit_w_only.restype = C.c_double
        _lib.oracle_dot.restype = C.c_double
        _lib.oracle_prune_columns.restype = C.c_int64
        _lib.oracle_split_columns.restype = C.c_int64
        _lib.oracle_num_threads.restype = C.c_int
        _lib.oracle_synth_pef.restype = C.c_int
        _lib.oracle_problem_create.restype = C.c_void_p
        _lib.oracle_problem_loss.restype = C.c_double
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def num_threads():
    return int(lib().oracle_num_threads())


def set_num_threads(t):
    lib().oracle_set_num_threads(C.c_int(int(t)))


def init_uniform(first, count, seed, stream, scale):
    out = np.empty(int(count), dtype=np.float32)
    lib().oracle_init_uniform(_p(out, C.c_float), C.c_int64(int(first)), C.c_int64(int(count)),
                              C.c_uint64(int(seed)), C.c_uint64(int(stream)),
                              C.c_float(float(scale)))
    return out


def init_factors(n, m, r, seed, scale, col_start=0, m_total=None):
    """W [n,r] and H [r,m] exactly as the engine's seeded initialiser makes them.

    H is defined on the full kept-column axis (index = column * r + t), so a
    shard ``[col_start, col_start+m)`` takes a slice of the same stream."""
    W = init_uniform(0, n * r, seed, 0, scale).reshape(n, r)
    Ht = init_uniform(col_start * r, m * r, seed, 1, scale).reshape(m, r)
    return W, np.ascontiguousarray(Ht.T)


def normalize_rows(vals, rowptr, norms, eps=1e-9):
    vals = _f32(vals).copy()
    rowptr = _i64(rowptr)
    norms = _f32(norms)
    lib().oracle_normalize_rows(_p(vals, C.c_float), _p(rowptr, C.c_int64),
                                C.c_int64(len(rowptr) - 1), _p(norms, C.c_float),
                                C.c_float(eps))
    return vals


def prune_columns(vals, colind, rowptr, n_cols, min_count=1):
    """Returns (vals, colind, rowptr, new_to_og) of the pruned matrix."""
    vals = _f32(vals).copy()
    colind = _i32(colind).copy()
    rowptr = _i64(rowptr).copy()
    n = len(rowptr) - 1
    new_to_og = np.empty(max(int(n_cols), 1), dtype=np.int32)
    nnz = C.c_int64(0)
    kept = lib().oracle_prune_columns(_p(vals, C.c_float), _p(colind, C.c_int32),
                                      _p(rowptr, C.c_int64), C.c_int64(n), C.c_int64(int(n_cols)),
                                      C.c_int32(int(min_count)), _p(new_to_og, C.c_int32),
                                      C.byref(nnz))
    q = nnz.value
    return vals[:q].copy(), colind[:q].copy(), rowptr, new_to_og[:kept].copy()


def retain_columns(vals, colind, rowptr, n_cols, retained):
    """CsrMatrix::RetainColumns_InPlace (src/cuda/host/sparse_matrix.h:141-170): keep
    the entries whose column is in `retained`; a column's new index is its position
    in that list (a later position overwrites an earlier one for a repeated id);
    order inside a row is kept.  Returns (vals, colind, rowptr)."""
    vals = np.asarray(vals, dtype=np.float32)
    colind = np.asarray(colind)
    rowptr = np.asarray(rowptr, dtype=np.int64)
    old_to_new = np.full(int(n_cols), -1, dtype=np.int64)
    for i, c in enumerate(np.asarray(retained)):      # sequential, as the reference loop
        old_to_new[int(c)] = i
    new = old_to_new[colind]
    keep = new >= 0
    rows = np.repeat(np.arange(len(rowptr) - 1), np.diff(rowptr))
    out_ptr = np.zeros(len(rowptr), dtype=np.int64)
    np.add.at(out_ptr, rows[keep] + 1, 1)
    return vals[keep].copy(), new[keep].astype(np.int32), np.cumsum(out_ptr)


def dense_to_csr(A, threshold):
    """to_csr of scripts/sparsify_d_npeff.py:27-49: entries >= threshold, row by row;
    int64 row offsets and int32 column ids as that script writes them."""
    A = np.asarray(A)
    mask = A >= threshold
    rowptr = np.concatenate([[0], np.cumsum(mask.sum(axis=1))]).astype(np.int64)
    cols = np.nonzero(mask)[1].astype(np.int32)
    return A[mask].astype(np.float32), rowptr, cols


def split_range(total, n_splits, idx):
    s, w = C.c_int64(0), C.c_int64(0)
    lib().oracle_split_range(C.c_int64(int(total)), C.c_int64(int(n_splits)), C.c_int64(int(idx)),
                             C.byref(s), C.byref(w))
    return s.value, w.value


def split_columns(vals, colind, rowptr, c0, w):
    vals, colind, rowptr = _f32(vals), _i32(colind), _i64(rowptr)
    n = len(rowptr) - 1
    q = lib().oracle_split_columns(_p(vals, C.c_float), _p(colind, C.c_int32),
                                   _p(rowptr, C.c_int64), C.c_int64(n), C.c_int64(int(c0)),
                                   C.c_int64(int(w)), None, None, None)
    ov = np.empty(max(q, 1), dtype=np.float32)
    oc = np.empty(max(q, 1), dtype=np.int32)
    orp = np.empty(n + 1, dtype=np.int64)
    lib().oracle_split_columns(_p(vals, C.c_float), _p(colind, C.c_int32), _p(rowptr, C.c_int64),
                               C.c_int64(n), C.c_int64(int(c0)), C.c_int64(int(w)),
                               _p(ov, C.c_float), _p(oc, C.c_int32), _p(orp, C.c_int64))
    return ov[:q], oc[:q], orp


def csr_to_csc(vals, colind, rowptr, m):
    vals, colind, rowptr = _f32(vals), _i32(colind), _i64(rowptr)
    n = len(rowptr) - 1
    nnz = int(rowptr[n])
    cv = np.empty(max(nnz, 1), dtype=np.float32)
    cr = np.empty(max(nnz, 1), dtype=np.int32)
    cp = np.empty(m + 1, dtype=np.int64)
    lib().oracle_csr_to_csc(_p(vals, C.c_float), _p(colind, C.c_int32), _p(rowptr, C.c_int64),
                            C.c_int64(n), C.c_int64(int(m)), _p(cv, C.c_float),
                            _p(cr, C.c_int32), _p(cp, C.c_int64))
    return cv[:nnz], cr[:nnz], cp


def spmm(vals, ind, ptr, D, acc64=True):
    """out[i,:] = sum_p vals[p] * D[ind[p],:] for p in row i."""
    vals, ind, ptr, D = _f32(vals), _i32(ind), _i64(ptr), _f32(D)
    rows, r = len(ptr) - 1, D.shape[1]
    out = np.empty((rows, r), dtype=np.float32)
    lib().oracle_spmm(_p(vals, C.c_float), _p(ind, C.c_int32), _p(ptr, C.c_int64),
                      C.c_int64(rows), _p(D, C.c_float), C.c_int64(r), _p(out, C.c_float),
                      C.c_int(int(acc64)))
    return out


def gram(X, acc64=True):
    X = _f32(X)
    rows, r = X.shape
    G = np.empty((r, r), dtype=np.float32)
    lib().oracle_gram(_p(X, C.c_float), C.c_int64(rows), C.c_int64(r), _p(G, C.c_float),
                      C.c_int(int(acc64)))
    return G


def mu_update(X, Num, G, eps, acc64=True):
    X = _f32(X).copy()
    Num, G = _f32(Num), _f32(G)
    rows, r = X.shape
    lib().oracle_mu_update(_p(X, C.c_float), _p(Num, C.c_float), _p(G, C.c_float),
                           C.c_int64(rows), C.c_int64(r), C.c_float(eps), C.c_int(int(acc64)))
    return X


def _csr_args(vals, colind, rowptr):
    vals, colind, rowptr = _f32(vals), _i32(colind), _i64(rowptr)
    return vals, colind, rowptr, (_p(vals, C.c_float), _p(colind, C.c_int32),
                                  _p(rowptr, C.c_int64), C.c_int64(len(rowptr) - 1))


def run(vals, colind, rowptr, m, W, H, iters, eps, acc64=True, losses=False):
    """`iters` iterations of (W update, then H update); returns (W, H[, losses])."""
    vals, colind, rowptr, a = _csr_args(vals, colind, rowptr)
    W = _f32(W).copy()
    Ht = _f32(np.asarray(H).T).copy()
    r = W.shape[1]
    ls = np.zeros(max(iters, 1), dtype=np.float64)
    lib().oracle_run(*a, C.c_int64(int(m)), C.c_int64(r), _p(W, C.c_float), _p(Ht, C.c_float),
                     C.c_int32(int(iters)), C.c_float(eps), C.c_int(int(acc64)),
                     _p(ls, C.c_double) if losses else None)
    H_out = np.ascontiguousarray(Ht.T)
    return (W, H_out, ls[:iters]) if losses else (W, H_out)


def step_w(vals, colind, rowptr, m, W, H, eps, acc64=True):
    vals, colind, rowptr, a = _csr_args(vals, colind, rowptr)
    W = _f32(W).copy()
    Ht = _f32(np.asarray(H).T)
    lib().oracle_step_w(*a, C.c_int64(int(m)), C.c_int64(W.shape[1]), _p(W, C.c_float),
                        _p(Ht, C.c_float), C.c_float(eps), C.c_int(int(acc64)))
    return W


def step_h(vals, colind, rowptr, m, W, H, eps, acc64=True):
    vals, colind, rowptr, a = _csr_args(vals, colind, rowptr)
    W = _f32(W)
    Ht = _f32(np.asarray(H).T).copy()
    lib().oracle_step_h(*a, C.c_int64(int(m)), C.c_int64(W.shape[1]), _p(W, C.c_float),
                        _p(Ht, C.c_float), C.c_float(eps), C.c_int(int(acc64)))
    return np.ascontiguousarray(Ht.T)


def loss(vals, colind, rowptr, m, W, H, acc64=True):
    vals, colind, rowptr, a = _csr_args(vals, colind, rowptr)
    W = _f32(W)
    Ht = _f32(np.asarray(H).T)
    return float(lib().oracle_loss(*a, C.c_int64(int(m)), C.c_int64(W.shape[1]),
                                   _p(W, C.c_float), _p(Ht, C.c_float), C.c_int(int(acc64))))


def fit_w_only(vals, colind, rowptr, m, W, H, iters, eps, acc64=True):
    vals, colind, rowptr, a = _csr_args(vals, colind, rowptr)
    W = _f32(W).copy()
    Ht = _f32(np.asarray(H).T)
    l = lib().oracle_fit_w_only(*a, C.c_int64(int(m)), C.c_int64(W.shape[1]), _p(W, C.c_float),
                                _p(Ht, C.c_float), C.c_int32(int(iters)), C.c_float(eps),
                                C.c_int(int(acc64)))
    return W, float(l)


# ---------------------------------------------------------------------------
# Independent second opinion: dense float64 numpy rendering of the same rule,
# usable only at small sizes.  It shares no code with the C file above.
def numpy_run(vals, colind, rowptr, m, W, H, iters, eps):
    rowptr = np.asarray(rowptr)
    n = len(rowptr) - 1
    A = np.zeros((n, m), dtype=np.float64)
    rows = np.repeat(np.arange(n), np.diff(rowptr))
    np.add.at(A, (rows, np.asarray(colind)), np.asarray(vals, dtype=np.float64))
    W = np.asarray(W, dtype=np.float64).copy()
    H = np.asarray(H, dtype=np.float64).copy()
    losses = []
    for _ in range(iters):
        W *= (A @ H.T) / (W @ (H @ H.T) + eps)
        H *= (W.T @ A) / ((W.T @ W) @ H + eps)
        losses.append(np.linalg.norm(A - W @ H))
    return W, H, np.array(losses)


# ---------------------------------------------------------------------------
# Hoyer's sparseness projection of the columns of W (n x r), the reference's
# DenseFactorSparsityContext::sparsifyF: the sequence of
# src/nmf/sparse/dense_factor_sparsity_constraints.h:205-237 (set-up: Y = 1,
# column sums, computeInitialS; then per pass: sums and dot products, alpha,
# updateSAfterAlpha, active columns, updateYAndS, updateSLastStep) with the
# elementwise rules of src/nmf/sparse/sparsity_constraint_kernels.h:14-141.
# The reference never calls it (multi_mu_dense_factors_nmf1.h:162), so there is
# no output of the reference to pin this against: the pins are the properties of
# the published projection (Hoyer 2004, section 3.3) checked in tests/.
# Column sums are taken in float64 and rounded to float32 (the reference: cuBLAS
# fp32 sums); every elementwise operation is a single float32 operation, in the
# order of the kernels.  rule 0: alpha = non-negative root of
# |m + alpha (s - m)| = L2 (as published); rule 1: the reference's
# kernel_computeAlpha expression.  Returns (S, passes, converged).
def hoyer_project(W, l1, l2=1.0, rule=0, max_passes=None):
    f = np.float32
    S = np.array(W, dtype=f, copy=True)
    n, r = S.shape
    if n == 0 or r == 0:
        return S, 0, True
    l1, l2 = f(l1), f(l2)
    Y = np.ones((n, r), dtype=bool)
    active = np.ones(r, dtype=bool)
    if max_passes is None or max_passes <= 0:
        max_passes = n + 1

    def colsum(M):
        return M.astype(np.float64).sum(axis=0).astype(f)

    S = S + (l1 - colsum(S)) / f(n)                               # kernel_computeInitialS
    passes, converged = 0, False
    for _ in range(max_passes):
        yy = colsum(Y)
        ss = (S.astype(np.float64) ** 2).sum(axis=0).astype(f)
        sy = (S.astype(np.float64) * Y).sum(axis=0).astype(f)
        with np.errstate(divide="ignore", invalid="ignore"):
            beta = l1 / yy
            m2 = (beta * beta) * yy
            ms = beta * sy
            d2 = np.maximum(f(1e-9), (m2 + ss) - f(2.0) * ms)
            if rule == 1:                                          # kernel_computeAlpha as written
                alpha = ((l2 * np.sqrt(d2) + m2) - ms) / d2
            else:
                b = ms - m2
                c = m2 - l2 * l2
                disc = np.maximum(f(0.0), b * b - d2 * c)
                alpha = (np.sqrt(disc) - b) / d2
            alpha = np.where(yy > 0, alpha, f(0.0)).astype(f)
            mid = np.where(yy > 0, l1 / yy, f(0.0)).astype(f)
        M = np.where(Y, mid[None, :], f(0.0)).astype(f)           # kernel_updateSAfterAlpha
        S_new = (M + alpha[None, :] * (S - M)).astype(f)
        S = np.where(active[None, :], S_new, S)
        neg = ((S < 0) & active[None, :]).sum(axis=0)
        active = active & (neg > 0)
        passes += 1
        if not active.any():
            converged = True
            break
        a = active[None, :]                                        # kernel_updateYAndS
        Y = np.where(a & Y & (S < 0), False, Y)
        S = np.where(a & ~Y, f(0.0), S).astype(f)
        sum_s, sum_y = colsum(S), colsum(Y)                        # kernel_updateSLastStep
        with np.errstate(divide="ignore", invalid="ignore"):
            cshift = ((sum_s - l1) / sum_y).astype(f)
        S = np.where(a & Y, S - cshift[None, :], S).astype(f)
    return S, passes, converged


# ---------------------------------------------------------------------------
# Synthetic D-PEF generator for tests (numpy; small sizes).  Column popularity
# Zipf(alpha), k distinct columns per row drawn without replacement
# (exponential-race form of successive sampling), value = g^2 * row scale with
# g ~ N(0,1), scale ~ LogNormal(0, sigma); entries ordered by descending value
# as tf.math.top_k leaves them (npeff/fishers/d_pefs_computer.py:127-129).
# Returns unnormalised values plus the row L2 norms, the form the D-PEF file
# holds (values + dense_fisher_norms).
def synth_pef(n, m, k, alpha=1.1, sigma=1.0, seed=0):
    rng = np.random.default_rng(seed)
    p = (np.arange(m, dtype=np.float64) + 1.0) ** (-alpha)
    p /= p.sum()
    vals = np.empty((n, k), dtype=np.float32)
    idx = np.empty((n, k), dtype=np.int32)
    for i in range(n):
        keys = rng.exponential(size=m) / p
        cols = np.argpartition(keys, k - 1)[:k] if k < m else np.arange(m)
        cols = rng.permutation(cols)
        v = rng.standard_normal(k) ** 2 * rng.lognormal(0.0, sigma)
        order = np.argsort(-v, kind="stable")
        vals[i] = v[order].astype(np.float32)
        idx[i] = cols.astype(np.int32)
    norms = np.sqrt((vals.astype(np.float64) ** 2).sum(axis=1)).astype(np.float32)
    return vals, idx, norms


def synth_pef_hashed(n, m, k, alpha=1.1, sigma=1.0, seed=0):
    """The benchmark's synthetic D-PEF rows, generated on the host by the twin of the
    device generator (``dnpeff_synth_pef_device``): the same column indices bit for
    bit, values to a few ulp.  Returns (vals [n,k], idx [n,k], norms [n])."""
    vals = np.empty((n, k), dtype=np.float32)
    idx = np.empty((n, k), dtype=np.int32)
    norms = np.empty(n, dtype=np.float32)
    rc = lib().oracle_synth_pef(C.c_int64(n), C.c_int64(m), C.c_int64(k), C.c_double(alpha), C.c_double(sigma),
                                C.c_uint64(seed), _p(vals, C.c_float), _p(idx, C.c_int32), _p(norms, C.c_float))
    if rc != 0:
        raise ValueError("bad synthetic shape")
    return vals, idx, norms


class Problem:
    """A D-PEF matrix loaded once (normalise, prune, CSC, seeded initial factors with
    the benchmark's Uniform * sqrt(mean(A)/r) scale when ``init_scale <= 0``), then
    iterated one step per call: what the timed CPU arm of the benchmark runs."""

    def __init__(self, n, m, k, r, vals, idx, norms, min_count=1, eps=1e-12, seed=0, init_scale=0.0):
        vals, idx = _f32(vals), _i32(idx)
        norms = None if norms is None else _f32(norms)
        mk = C.c_int64(0)
        self._h = lib().oracle_problem_create(
            C.c_int64(n), C.c_int64(m), C.c_int64(k), C.c_int64(r), _p(vals, C.c_float), _p(idx, C.c_int32),
            None if norms is None else _p(norms, C.c_float), C.c_int32(min_count), C.c_float(eps),
            C.c_uint64(seed), C.c_float(init_scale), C.byref(mk))
        if not self._h:
            raise MemoryError("the CPU problem does not fit host memory")
        self.m_kept = mk.value

    def step(self, acc64=False):
        lib().oracle_problem_step(C.c_void_p(self._h), C.c_int(int(acc64)))

    def loss(self):
        return float(lib().oracle_problem_loss(C.c_void_p(self._h)))

    def close(self):
        if self._h:
            lib().oracle_problem_free(C.c_void_p(self._h))
            self._h = None

    def __del__(self):
        self.close()
