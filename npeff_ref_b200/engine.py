"""Host-side mirror of the reference's ``MuNmf<IndT>`` for one column shard.

Reference surface (src/nmf/sparse/multi_mu_dense_factors_nmf1.h): constructor
from host CSR partitions + ``MuNmfParams`` (:81), ``run()`` (:152),
``loadWToHostSync()`` (:207), ``loadHToHostSync()`` (:222),
``computeUncachedLoss()`` (:242).  The reference drives every visible GPU from
one process; here one ``MuNmf`` object is one shard on one device, and a
multi-GPU job is one object per process joined by :meth:`MuNmf.init_comm`.
The preprocessing the reference does on the host before constructing the
engine (normalise rows, prune columns, split by columns;
mains/run_nmf_on_pefs.cu:122-182) happens on the device inside the loader.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import Params, check, lib


@dataclass
class MuNmfParams:
    """``MuNmfParams`` (…device_contexts1.h:36-55) with the executable's defaults
    (mains/run_nmf_on_pefs.cu:190-192)."""
    rank: int
    max_iters: int = 0
    eps: float = 1e-8
    seed: int = 43190432042
    init_scale: float = 0.0  # <= 0: unscaled U(0,1] like the reference


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


class MuNmf:
    CONTIGUOUS, CYCLIC = 0, 1

    def __init__(self, params, device=0, shard_index=0, n_shards=1, stream=None, shard_mode=0):
        self.params = params
        self._h = C.c_void_p()
        p = Params(int(params.rank), float(params.eps), int(params.seed),
                   float(params.init_scale), int(shard_index), int(n_shards), int(shard_mode))
        check(lib().dnpeff_create(C.byref(p), int(device), C.c_void_p(stream or 0),
                                  C.byref(self._h)))
        self.device = device
        self.shard_index = shard_index
        self.n_shards = n_shards

    # -- lifetime -----------------------------------------------------------
    def close(self):
        if self._h:
            lib().dnpeff_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_option(self, name, value):
        """Tuning values and test hooks of the engine (``dnpeff_set_option``)."""
        check(lib().dnpeff_set_option(self._h, name.encode(), int(value)))

    # -- loader ---------------------------------------------------------------
    def set_csr(self, n_rows, n_cols_full, vals, colind, rowptr=None, k_per_row=0, norms=None,
                min_values_per_parameter=1):
        """Host buffers (numpy).  ``rowptr=None`` means ``k_per_row`` entries per row."""
        vals = np.ascontiguousarray(vals, dtype=np.float32).reshape(-1)
        colind = np.ascontiguousarray(colind, dtype=np.int32).reshape(-1)
        if rowptr is not None:
            rowptr = np.ascontiguousarray(rowptr, dtype=np.int64)
        if norms is not None:
            norms = np.ascontiguousarray(norms, dtype=np.float32)
        check(lib().dnpeff_set_csr(self._h, int(n_rows), int(n_cols_full), int(k_per_row),
                                   _ptr(rowptr), _ptr(vals), _ptr(colind), _ptr(norms),
                                   int(min_values_per_parameter)))

    @staticmethod
    def row_slice(n_rows_total, n_engines, index):
        """(row_begin, n_rows) of the slice engine ``index`` of ``n_engines`` passes to
        :meth:`set_csr_rows`."""
        b, c = C.c_int64(0), C.c_int64(0)
        check(lib().dnpeff_row_slice(int(n_rows_total), int(n_engines), int(index), C.byref(b), C.byref(c)))
        return b.value, c.value

    def set_csr_rows(self, n_rows_total, n_cols_full, row_begin, vals, colind, rowptr=None, k_per_row=0,
                     norms=None, min_values_per_parameter=1):
        """Collective loader: this engine passes only its row slice of the matrix
        (``vals``/``colind``/``norms`` of rows ``[row_begin, row_begin + n_rows)``); every
        engine of the job calls it after :meth:`init_comm`.  The reference uploads to each
        device only that device's partition (…device_contexts1.h:180-194)."""
        vals = np.ascontiguousarray(vals, dtype=np.float32)
        n_rows = (len(rowptr) - 1) if rowptr is not None else (vals.size // max(int(k_per_row), 1))
        vals = vals.reshape(-1)
        colind = np.ascontiguousarray(colind, dtype=np.int32).reshape(-1)
        if rowptr is not None:
            rowptr = np.ascontiguousarray(rowptr, dtype=np.int64)
        if norms is not None:
            norms = np.ascontiguousarray(norms, dtype=np.float32)
        check(lib().dnpeff_set_csr_rows(self._h, int(n_rows_total), int(n_cols_full), int(k_per_row),
                                        int(row_begin), int(n_rows), _ptr(rowptr), _ptr(vals), _ptr(colind),
                                        _ptr(norms), int(min_values_per_parameter)))

    def set_csr_retain(self, n_rows, n_cols_full, vals, colind, retained_cols, rowptr=None, k_per_row=0,
                       norms=None):
        """As ``set_csr`` with the kept columns given as a list of original column ids
        (``CsrMatrix::RetainColumns_InPlace``, src/cuda/host/sparse_matrix.h:141-170):
        a column's new index is its position in the list."""
        vals = np.ascontiguousarray(vals, dtype=np.float32).reshape(-1)
        colind = np.ascontiguousarray(colind, dtype=np.int32).reshape(-1)
        retained_cols = np.ascontiguousarray(retained_cols, dtype=np.int32).reshape(-1)
        if rowptr is not None:
            rowptr = np.ascontiguousarray(rowptr, dtype=np.int64)
        if norms is not None:
            norms = np.ascontiguousarray(norms, dtype=np.float32)
        check(lib().dnpeff_set_csr_retain(self._h, int(n_rows), int(n_cols_full), int(k_per_row),
                                          _ptr(rowptr), _ptr(vals), _ptr(colind), _ptr(norms),
                                          _ptr(retained_cols), int(retained_cols.size)))

    def set_h_csr(self, h_rowptr, h_colind, h_vals):
        """H (rank x n_cols_kept) from CSR arrays; zero elsewhere (the sparse
        decomposition file's form, src/io/nmf_decomp_h5.h:134-170)."""
        h_rowptr = np.ascontiguousarray(h_rowptr, dtype=np.int64)
        h_colind = np.ascontiguousarray(h_colind, dtype=np.int32)
        h_vals = np.ascontiguousarray(h_vals, dtype=np.float32)
        check(lib().dnpeff_set_h_csr(self._h, _ptr(h_rowptr), _ptr(h_colind), _ptr(h_vals)))

    def set_csr_device(self, n_rows, n_cols_full, d_vals, d_colind, d_rowptr=0, k_per_row=0,
                       d_norms=0, min_values_per_parameter=1):
        """Device pointers (ints), inputs already resident in HBM."""
        check(lib().dnpeff_set_csr_device(self._h, int(n_rows), int(n_cols_full), int(k_per_row),
                                          C.c_void_p(d_rowptr or 0), C.c_void_p(d_vals),
                                          C.c_void_p(d_colind), C.c_void_p(d_norms or 0),
                                          int(min_values_per_parameter)))

    @property
    def shape(self):
        """(n_rows, n_cols_kept, col_start, n_cols_shard, nnz_shard)"""
        v = [C.c_int64(0) for _ in range(5)]
        check(lib().dnpeff_get_shape(self._h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def layout(self):
        """(n_popular_cols, popular_nnz, n_tail_blocks, tile_rows) of the internal layout."""
        a, b, c, d = C.c_int64(0), C.c_int64(0), C.c_int32(0), C.c_int32(0)
        check(lib().dnpeff_get_layout(self._h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return a.value, b.value, c.value, d.value

    def new_to_og(self):
        out = np.empty(max(self.shape[1], 1), dtype=np.int32)
        check(lib().dnpeff_get_new_to_og(self._h, _ptr(out)))
        return out[:self.shape[1]]

    def shard_columns(self):
        """(kept_ids, original_ids) of this shard's local columns."""
        ms = self.shape[3]
        a = np.empty(max(ms, 1), dtype=np.int32)
        b = np.empty(max(ms, 1), dtype=np.int32)
        check(lib().dnpeff_get_shard_columns(self._h, _ptr(a), _ptr(b)))
        return a[:ms], b[:ms]

    def export_shard_csr(self):
        n, _, _, _, nnz = self.shape
        rp = np.empty(n + 1, dtype=np.int64)
        ci = np.empty(max(nnz, 1), dtype=np.int32)
        va = np.empty(max(nnz, 1), dtype=np.float32)
        check(lib().dnpeff_export_shard_csr(self._h, _ptr(rp), _ptr(ci), _ptr(va)))
        return va[:nnz], ci[:nnz], rp

    def export_shard_csc(self):
        _, _, _, ms, nnz = self.shape
        cp = np.empty(ms + 1, dtype=np.int64)
        ri = np.empty(max(nnz, 1), dtype=np.int32)
        va = np.empty(max(nnz, 1), dtype=np.float32)
        check(lib().dnpeff_export_shard_csc(self._h, _ptr(cp), _ptr(ri), _ptr(va)))
        return va[:nnz], ri[:nnz], cp

    def a_sq_norm(self):
        v = C.c_double(0)
        check(lib().dnpeff_a_sq_norm(self._h, C.byref(v)))
        return v.value

    def a_sum(self):
        v = C.c_double(0)
        check(lib().dnpeff_a_sum(self._h, C.byref(v)))
        return v.value

    # -- factors --------------------------------------------------------------
    def set_init_scale(self, scale):
        check(lib().dnpeff_set_init_scale(self._h, float(scale)))

    def init_factors(self, W=None, H=None):
        """``None`` = seeded generation on the device; arrays are ``W [n, r]`` and
        this shard's ``H [r, n_cols_shard]``, row-major."""
        if W is not None:
            W = np.ascontiguousarray(W, dtype=np.float32)
        if H is not None:
            H = np.ascontiguousarray(H, dtype=np.float32)
        check(lib().dnpeff_init_factors(self._h, _ptr(W), _ptr(H)))

    def load_w_to_host(self):
        """``loadWToHostSync`` + ``toRowMajor_inPlace``: ``[n_rows, rank]``."""
        out = np.empty((self.shape[0], self.params.rank), dtype=np.float32)
        check(lib().dnpeff_get_w(self._h, _ptr(out)))
        return out

    def load_h_to_host(self):
        """``loadHToHostSync`` + ``toRowMajor_inPlace`` for this shard: ``[rank, n_cols_shard]``."""
        out = np.empty((self.params.rank, self.shape[3]), dtype=np.float32)
        check(lib().dnpeff_get_h(self._h, _ptr(out)))
        return out

    # -- multi-GPU --------------------------------------------------------------
    @staticmethod
    def make_unique_id():
        buf = (C.c_ubyte * 128)()
        check(lib().dnpeff_nccl_unique_id(C.byref(buf)))
        return bytes(buf)

    def init_comm(self, unique_id):
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        check(lib().dnpeff_comm_init(self._h, C.byref(buf), int(self.shard_index),
                                     int(self.n_shards)))

    # -- iteration --------------------------------------------------------------
    def step_w(self):
        check(lib().dnpeff_step_w(self._h))

    def step_h(self):
        check(lib().dnpeff_step_h(self._h))

    def run(self, iters=None, log_every=10):
        """``MuNmf::run``: ``iters`` x (update W, update H); logs the reference's
        ``step N: loss [ms/step]`` line every ``log_every`` steps."""
        check(lib().dnpeff_run(self._h, int(self.params.max_iters if iters is None else iters),
                               int(log_every)))

    def synchronize(self):
        check(lib().dnpeff_synchronize(self._h))

    def compute_uncached_loss(self):
        v = C.c_double(0)
        check(lib().dnpeff_loss(self._h, C.byref(v)))
        return v.value

    def fit_w_only(self, iters, want_loss=True):
        v = C.c_double(0)
        check(lib().dnpeff_fit_w_only(self._h, int(iters), C.byref(v) if want_loss else None))
        return v.value if want_loss else None

    def sparsify_w(self, l1_norm, l2_norm=1.0, alpha_rule=0):
        """Hoyer's sparseness projection of every component (column) of W onto the given
        L1 / L2 norms (``DenseFactorSparsityContext::sparsifyF``, built by the reference from
        ``--sparsity_W`` but never called).  Returns (passes, converged)."""
        passes, conv = C.c_int32(0), C.c_int32(0)
        check(lib().dnpeff_sparsify_w(self._h, float(l1_norm), float(l2_norm), int(alpha_rule),
                                      C.byref(passes), C.byref(conv)))
        return passes.value, bool(conv.value)

    # -- measurement --------------------------------------------------------------
    def enable_timing(self, on=True):
        check(lib().dnpeff_enable_timing(self._h, 1 if on else 0))

    def get_timing(self):
        ms = (C.c_double * _lib.N_TIMERS)()
        cnt = (C.c_int64 * _lib.N_TIMERS)()
        check(lib().dnpeff_get_timing(self._h, ms, cnt))
        return {name: (ms[i], cnt[i]) for i, name in enumerate(_lib.TIMER_NAMES)}

    def launch_count(self):
        v = C.c_int64(0)
        check(lib().dnpeff_launch_count(self._h, C.byref(v)))
        return v.value


def preprocess_and_split(params, n_rows, n_cols_full, vals, colind, norms, k_per_row,
                         min_values_per_parameter=1, device=0, shard_index=0, n_shards=1,
                         stream=None):
    """``readAndPreprocessPef`` + engine construction (mains/run_nmf_on_pefs.cu:122-200)
    for one shard: returns a loaded :class:`MuNmf`."""
    eng = MuNmf(params, device=device, shard_index=shard_index, n_shards=n_shards, stream=stream)
    eng.set_csr(n_rows, n_cols_full, vals, colind, None, k_per_row, norms, min_values_per_parameter)
    return eng
