"""CPU-only checks of the built-in HDF5 codec (no libhdf5 / h5py exists in this
image): write -> read round trips of both file layouts of the path, structural
checks of the bytes written, and a read of a real libhdf5-written file where
one is available."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from npeff_ref_b200._lib import lib, check


def _info(path, name):
    rank, isf, ts = C.c_int32(0), C.c_int32(0), C.c_int32(0)
    dims = (C.c_int64 * 4)()
    check(lib().dnpeff_hdf5_dataset_info(path.encode(), name.encode(), C.byref(rank), dims,
                                         C.byref(isf), C.byref(ts)))
    return tuple(dims[i] for i in range(rank.value)), bool(isf.value), ts.value


def _read(path, name, rows, cols):
    out = np.empty((rows, cols), dtype=np.float64)
    check(lib().dnpeff_hdf5_read_f64(path.encode(), name.encode(), rows, cols,
                                     C.c_void_p(out.ctypes.data)))
    return out


def test_pef_file_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    n, k, dense = 37, 19, 123457
    vals = rng.random((n, k), dtype=np.float32)
    idx = rng.integers(0, dense, size=(n, k)).astype(np.int32)
    norms = rng.random(n, dtype=np.float32)
    path = str(tmp_path / "pef.h5")
    check(lib().dnpeff_write_pef_hdf5(path.encode(), n, k, C.c_void_p(vals.ctypes.data),
                                      C.c_void_p(idx.ctypes.data), C.c_void_p(norms.ctypes.data), dense))
    a, b, c = C.c_int64(0), C.c_int64(0), C.c_int64(0)
    check(lib().dnpeff_pef_hdf5_info(path.encode(), C.byref(a), C.byref(b), C.byref(c)))
    assert (a.value, b.value, c.value) == (n, k, dense)
    assert _info(path, "data/fisher/values") == ((n, k), True, 4)
    assert _info(path, "data/fisher/indices") == ((n, k), False, 4)
    assert _info(path, "data/dense_fisher_norms") == ((n,), True, 4)
    # full read and the leading hyperslab selected by --n_examples / --n_fisher_values
    for (nn, kk) in ((0, 0), (11, 7), (n, 5), (3, k)):
        rn, rk = nn or n, kk or k
        v = np.empty((rn, rk), np.float32)
        i = np.empty((rn, rk), np.int32)
        no = np.empty(rn, np.float32)
        check(lib().dnpeff_read_pef_hdf5(path.encode(), nn, kk, C.c_void_p(v.ctypes.data),
                                         C.c_void_p(i.ctypes.data), C.c_void_p(no.ctypes.data)))
        assert np.array_equal(v, vals[:rn, :rk]) and np.array_equal(i, idx[:rn, :rk])
        assert np.array_equal(no, norms[:rn])
    assert lib().dnpeff_read_pef_hdf5(path.encode(), n + 1, 0, None, None, None) == -1


def test_decomposition_file_round_trip_and_layout(tmp_path):
    rng = np.random.default_rng(1)
    n, r, m, dense = 23, 5, 41, 1000
    W = rng.random((n, r), dtype=np.float32)
    H = rng.random((r, m), dtype=np.float32)
    kept = np.sort(rng.choice(dense, size=m, replace=False)).astype(np.int32)
    path = str(tmp_path / "decomp.h5")
    check(lib().dnpeff_save_decomposition_hdf5(path.encode(), C.c_void_p(W.ctypes.data),
                                               C.c_void_p(H.ctypes.data), C.c_void_p(kept.ctypes.data),
                                               n, r, m, dense))
    a, b, c, d = C.c_int64(0), C.c_int32(0), C.c_int64(0), C.c_int64(0)
    check(lib().dnpeff_decomposition_hdf5_info(path.encode(), C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
    assert (a.value, b.value, c.value, d.value) == (n, r, m, dense)
    W2, H2, k2 = np.empty_like(W), np.empty_like(H), np.empty_like(kept)
    check(lib().dnpeff_read_decomposition_hdf5(path.encode(), C.c_void_p(W2.ctypes.data),
                                               C.c_void_p(H2.ctypes.data), C.c_void_p(k2.ctypes.data)))
    assert np.array_equal(W, W2) and np.array_equal(H, H2) and np.array_equal(kept, k2)
    assert _info(path, "data/reduce_kept_indices") == ((m,), False, 4)
    # structural checks of the bytes against the format specification
    raw = open(path, "rb").read()
    assert raw[:8] == b"\x89HDF\r\n\x1a\n"
    assert raw[8] == 0 and raw[13] == 8 and raw[14] == 8           # superblock v0, 8-byte offsets/lengths
    leaf_k, internal_k = struct.unpack_from("<HH", raw, 16)
    assert (leaf_k, internal_k) == (4, 16)
    base, freesp, eof, drv = struct.unpack_from("<QQQQ", raw, 24)
    assert base == 0 and freesp == 2 ** 64 - 1 and drv == 2 ** 64 - 1 and eof == len(raw)
    name_off, root_hdr, cache, _, btree, heap = struct.unpack_from("<QQIIQQ", raw, 56)
    assert cache == 1 and raw[btree:btree + 4] == b"TREE" and raw[heap:heap + 4] == b"HEAP"
    assert raw[root_hdr] == 1                                          # version-1 object header
    nmsg, refc, hsize = struct.unpack_from("<HII", raw, root_hdr + 2)
    assert nmsg == 1 and refc == 1 and hsize % 8 == 0
    mtype, msize = struct.unpack_from("<HH", raw, root_hdr + 16)
    assert mtype == 0x11 and msize == 16
    assert struct.unpack_from("<QQ", raw, root_hdr + 24) == (btree, heap)
    used = struct.unpack_from("<H", raw, btree + 6)[0]
    assert used == 1
    snod = struct.unpack_from("<Q", raw, btree + 24 + 8)[0]
    assert raw[snod:snod + 4] == b"SNOD" and struct.unpack_from("<H", raw, snod + 6)[0] == 1
    dsize, free_head, daddr = struct.unpack_from("<QQQ", raw, heap + 8)
    assert raw[daddr + 8:daddr + 12] == b"data" and free_head == dsize - 16
    assert struct.unpack_from("<QQ", raw, daddr + free_head) == (1, 16)
    assert len(raw) % 8 == 0


def test_missing_objects_and_bad_files_report_errors(tmp_path):
    bad = str(tmp_path / "not_hdf5.bin")
    open(bad, "wb").write(b"x" * 4096)
    assert lib().dnpeff_pef_hdf5_info(bad.encode(), None, None, None) == -6
    assert b"not an HDF5 file" in lib().dnpeff_last_error()
    assert lib().dnpeff_pef_hdf5_info(b"/nonexistent/file.h5", None, None, None) == -6
    W = np.zeros((2, 2), np.float32)
    k = np.zeros(2, np.int32)
    path = str(tmp_path / "d.h5")
    check(lib().dnpeff_save_decomposition_hdf5(path.encode(), C.c_void_p(W.ctypes.data),
                                               C.c_void_p(W.ctypes.data), C.c_void_p(k.ctypes.data), 2, 2, 2, 9))
    assert lib().dnpeff_pef_hdf5_info(path.encode(), None, None, None) == -6  # a decomposition is not a D-PEF file
    # a truncated file must fail cleanly, not crash
    raw = open(path, "rb").read()
    trunc = str(tmp_path / "t.h5")
    open(trunc, "wb").write(raw[:len(raw) // 2])
    assert lib().dnpeff_read_decomposition_hdf5(trunc.encode(), C.c_void_p(W.ctypes.data), None, None) in (-6, 0)


def _real_hdf5_file():
    try:
        import scipy.io
        p = os.path.join(os.path.dirname(scipy.io.__file__), "matlab", "tests", "data",
                         "testhdf5_7.4_GLNX86.mat")
        return p if os.path.exists(p) else None
    except Exception:
        return None


@pytest.mark.skipif(_real_hdf5_file() is None, reason="no libhdf5-written file available")
def test_reader_parses_a_file_written_by_libhdf5():
    """A MATLAB v7.3 file is an HDF5 file written by libhdf5 itself (512-byte user
    block, version-0 superblock, old-style groups): the same structures h5py's
    default settings produce for D-PEF files."""
    path = _real_hdf5_file()
    dims, is_float, size = _info(path, "testdouble")
    assert dims == (9, 1) and is_float and size == 8
    vals = _read(path, "testdouble", 9, 1).ravel()
    assert np.allclose(vals, np.arange(9) * np.pi / 4, rtol=0, atol=1e-15)   # MATLAB's 0:pi/4:2*pi


def _sparse_info(path):
    a, b, c, d, e = C.c_int64(0), C.c_int32(0), C.c_int64(0), C.c_int64(0), C.c_int64(0)
    check(lib().dnpeff_sparse_decomposition_hdf5_info(path.encode(), C.byref(a), C.byref(b), C.byref(c),
                                                      C.byref(d), C.byref(e)))
    return a.value, b.value, c.value, d.value, e.value


def test_sparse_decomposition_file_round_trip_and_layout(tmp_path):
    """SparseNmfDecomposition::save / ::read (src/io/nmf_decomp_h5.h:134-237): W, H as
    CSR under data/H with its shape attribute, reduce_kept_indices + full_dense_size."""
    rng = np.random.default_rng(5)
    n, r, m, dense = 17, 6, 53, 4000
    W = rng.random((n, r), dtype=np.float32)
    H = rng.random((r, m), dtype=np.float32)
    H[H < 0.8] = 0
    H[2] = 0                                               # an empty row
    mask = H != 0
    rowptr = np.concatenate([[0], np.cumsum(mask.sum(1))]).astype(np.int64)
    cols = np.nonzero(mask)[1].astype(np.int32)
    vals = H[mask].astype(np.float32)
    kept = np.sort(rng.choice(dense, m, replace=False)).astype(np.int32)
    path = str(tmp_path / "sp.h5")
    check(lib().dnpeff_save_sparse_decomposition_hdf5(
        path.encode(), C.c_void_p(W.ctypes.data), n, r, C.c_void_p(rowptr.ctypes.data),
        C.c_void_p(cols.ctypes.data), C.c_void_p(vals.ctypes.data), C.c_void_p(kept.ctypes.data), m, dense))
    assert _sparse_info(path) == (n, r, m, len(vals), dense)
    assert _info(path, "data/W") == ((n, r), True, 4)
    assert _info(path, "data/H/values") == ((len(vals),), True, 4)
    assert _info(path, "data/H/row_indices") == ((r + 1,), False, 8)      # int64, as the sparsify script writes
    assert _info(path, "data/H/column_indices") == ((len(vals),), False, 4)
    assert _info(path, "data/reduce_kept_indices") == ((m,), False, 4)
    W2 = np.empty_like(W)
    rp2 = np.empty(r + 1, np.int64)
    c2 = np.empty(len(vals), np.int32)
    v2 = np.empty(len(vals), np.float32)
    k2 = np.empty(m, np.int32)
    check(lib().dnpeff_read_sparse_decomposition_hdf5(
        path.encode(), C.c_void_p(W2.ctypes.data), C.c_void_p(rp2.ctypes.data), C.c_void_p(c2.ctypes.data),
        C.c_void_p(v2.ctypes.data), C.c_void_p(k2.ctypes.data)))
    assert np.array_equal(W2, W) and np.array_equal(rp2, rowptr) and np.array_equal(c2, cols)
    assert np.array_equal(v2, vals) and np.array_equal(k2, kept)
    # a dense decomposition file is not a sparse one, and the other way round
    dpath = str(tmp_path / "dense.h5")
    check(lib().dnpeff_save_decomposition_hdf5(dpath.encode(), C.c_void_p(W.ctypes.data), C.c_void_p(H.ctypes.data),
                                               C.c_void_p(kept.ctypes.data), n, r, m, dense))
    assert lib().dnpeff_sparse_decomposition_hdf5_info(dpath.encode(), None, None, None, None, None) != 0
    assert lib().dnpeff_decomposition_hdf5_info(path.encode(), None, None, None, None) != 0
