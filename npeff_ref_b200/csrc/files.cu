// File entry points of the C ABI: D-PEF input (src/io/pef_fisher_h5.h:57-226) and
// decomposition output/input (src/io/nmf_decomp_h5.h:38-126) through the built-in
// HDF5 codec.  Host code only.
#include <algorithm>
#include <vector>

#include "../../include/dnpeff_synth.h"
#include "common.cuh"
#include "h5lite.hpp"

using namespace dnpeff;

namespace {

struct PefShape {
    int64_t n = 0, k = 0, dense = 0;
};

// Dimensions of data/fisher/values plus the dense_fisher_size attribute of
// data/fisher (pef_fisher_h5.h:117-154; the reference insists on a 4-byte
// attribute, here any integer width is accepted).
PefShape pef_shape(h5lite::Reader& rd) {
    h5lite::ObjectInfo v = rd.dataset("data/fisher/values");
    if (v.space.dims.size() != 2) throw h5lite::Error("data/fisher/values must have rank 2");
    h5lite::ObjectInfo i = rd.dataset("data/fisher/indices");
    if (i.space.dims != v.space.dims) throw h5lite::Error("data/fisher/indices and values differ in shape");
    PefShape s;
    s.n = (int64_t)v.space.dims[0];
    s.k = (int64_t)v.space.dims[1];
    s.dense = rd.attr_int(rd.object(rd.find("data/fisher")), "dense_fisher_size");
    return s;
}

}  // namespace

extern "C" {

int dnpeff_pef_hdf5_info(const char* path, int64_t* n_examples, int64_t* n_values_per_example,
                         int64_t* dense_fisher_size) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        PefShape s = pef_shape(rd);
        if (n_examples) *n_examples = s.n;
        if (n_values_per_example) *n_values_per_example = s.k;
        if (dense_fisher_size) *dense_fisher_size = s.dense;
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

int dnpeff_read_pef_hdf5(const char* path, int64_t n_examples, int64_t n_fisher_values, float* vals,
                         int32_t* indices, float* norms) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        PefShape s = pef_shape(rd);
        int64_t n = n_examples > 0 ? n_examples : s.n, k = n_fisher_values > 0 ? n_fisher_values : s.k;
        if (n > s.n || k > s.k) return fail(DNPEFF_ERR_INVALID, "requested %ld x %ld of a %ld x %ld file",
                                            (long)n, (long)k, (long)s.n, (long)s.k);
        if (vals) rd.read_leading(rd.dataset("data/fisher/values"), n, k, h5lite::DType::f32(), vals);
        if (indices) rd.read_leading(rd.dataset("data/fisher/indices"), n, k, h5lite::DType::i32(), indices);
        if (norms) rd.read_leading(rd.dataset("data/dense_fisher_norms"), n, 1, h5lite::DType::f32(), norms);
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

// PefSparseFishers::read (src/io/pef_fisher_h5.h:175-220) reads the whole file into
// malloc'd arrays before anything is uploaded.  Here the engine's slice of the rows is
// read in chunks into two page-locked staging buffers per dataset; chunk i crosses
// PCIe while chunk i+1 is being read from the file, and no whole-file host copy exists.
int dnpeff_load_pef_hdf5(dnpeff_engine* eng, const char* path, int64_t n_examples,
                         int64_t n_fisher_values, int32_t min_values_per_parameter) {
    if (!eng || !path) return fail(DNPEFF_ERR_INVALID, "null argument");
    int32_t shard = 0, n_shards = 1, device = 0;
    DN_TRY(dnpeff_get_shard(eng, &shard, &n_shards, &device));
    // the staging and device buffers belong on the engine's device; the caller's
    // current device is put back on return
    struct DeviceScope {
        int prev = -1;
        explicit DeviceScope(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
        ~DeviceScope() { if (prev >= 0) cudaSetDevice(prev); }
    } device_scope(device);
    int64_t n = 0, k = 0, dense = 0;
    int status = dnpeff_pef_hdf5_info(path, &n, &k, &dense);
    if (status == DNPEFF_OK && n_examples > 0) {
        if (n_examples > n) status = fail(DNPEFF_ERR_INVALID, "--n_examples exceeds the file's %ld rows", (long)n);
        n = n_examples;
    }
    if (status == DNPEFF_OK && n_fisher_values > 0) {
        if (n_fisher_values > k) status = fail(DNPEFF_ERR_INVALID, "--n_fisher_values exceeds the file's %ld", (long)k);
        k = n_fisher_values;
    }
    int64_t row_begin = 0, rows = 0;
    if (status == DNPEFF_OK) status = dnpeff_row_slice(n, n_shards, shard, &row_begin, &rows);

    float *d_vals = nullptr, *d_norms = nullptr;
    int32_t* d_idx = nullptr;
    float* h_vals[2] = {nullptr, nullptr};
    int32_t* h_idx[2] = {nullptr, nullptr};
    float* h_norms = nullptr;
    cudaStream_t up = nullptr;
    cudaEvent_t done[2] = {nullptr, nullptr};
    char msg[1024] = {0};
    auto keep_msg = [&]() { snprintf(msg, sizeof(msg), "%s", dnpeff_last_error()); };
    if (status != DNPEFF_OK) keep_msg();

    // about 64 MB per staging buffer
    const int64_t chunk_rows = std::max<int64_t>(1, ((int64_t)64 << 20) / std::max<int64_t>(4 * k, 1));
    if (status == DNPEFF_OK) {
        const size_t cnt = (size_t)std::max<int64_t>(rows * k, 1), stage = (size_t)std::max<int64_t>(chunk_rows * k, 1);
        bool ok = cudaMalloc((void**)&d_vals, sizeof(float) * cnt) == cudaSuccess &&
                  cudaMalloc((void**)&d_idx, sizeof(int32_t) * cnt) == cudaSuccess &&
                  cudaMalloc((void**)&d_norms, sizeof(float) * (size_t)std::max<int64_t>(rows, 1)) == cudaSuccess &&
                  cudaMallocHost((void**)&h_norms, sizeof(float) * (size_t)std::max<int64_t>(rows, 1)) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&up, cudaStreamNonBlocking) == cudaSuccess;
        for (int b2 = 0; b2 < 2 && ok; b2++)
            ok = cudaMallocHost((void**)&h_vals[b2], sizeof(float) * stage) == cudaSuccess &&
                 cudaMallocHost((void**)&h_idx[b2], sizeof(int32_t) * stage) == cudaSuccess &&
                 cudaEventCreateWithFlags(&done[b2], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            status = fail(DNPEFF_ERR_CUDA, "device or page-locked memory for the D-PEF rows could not be allocated");
            keep_msg();
        }
    }
    if (status == DNPEFF_OK) {
        try {
            h5lite::Reader rd(path);
            h5lite::ObjectInfo dv = rd.dataset("data/fisher/values"), di = rd.dataset("data/fisher/indices");
            rd.read_block(rd.dataset("data/dense_fisher_norms"), (uint64_t)row_begin, (uint64_t)rows, 1, h5lite::DType::f32(),
                          h_norms);
            if (rows > 0 && cudaMemcpyAsync(d_norms, h_norms, sizeof(float) * (size_t)rows, cudaMemcpyHostToDevice, up) != cudaSuccess)
                throw h5lite::Error("upload of the row norms failed");
            int buf = 0;
            for (int64_t r0 = 0; r0 < rows; r0 += chunk_rows, buf ^= 1) {
                const int64_t nr = std::min(chunk_rows, rows - r0);
                if (r0 >= 2 * chunk_rows) cudaEventSynchronize(done[buf]);  // the staging buffer's previous upload
                rd.read_block(dv, (uint64_t)(row_begin + r0), (uint64_t)nr, (uint64_t)k, h5lite::DType::f32(), h_vals[buf]);
                rd.read_block(di, (uint64_t)(row_begin + r0), (uint64_t)nr, (uint64_t)k, h5lite::DType::i32(), h_idx[buf]);
                if (cudaMemcpyAsync(d_vals + r0 * k, h_vals[buf], sizeof(float) * (size_t)(nr * k), cudaMemcpyHostToDevice, up) != cudaSuccess ||
                    cudaMemcpyAsync(d_idx + r0 * k, h_idx[buf], sizeof(int32_t) * (size_t)(nr * k), cudaMemcpyHostToDevice, up) != cudaSuccess ||
                    cudaEventRecord(done[buf], up) != cudaSuccess)
                    throw h5lite::Error("upload of a chunk of D-PEF rows failed");
            }
            if (cudaStreamSynchronize(up) != cudaSuccess) throw h5lite::Error("upload of the D-PEF rows failed");
        } catch (const std::exception& ex) {
            cudaGetLastError();
            status = fail(DNPEFF_ERR_IO, "%s", ex.what());
            keep_msg();
        }
    }
    // every engine of the job gets here, whatever happened to its own part of the file,
    // and they enter the collective loader only if all of them could read theirs
    int32_t all_ok = 0;
    int s2 = dnpeff_comm_agree(eng, status == DNPEFF_OK ? 1 : 0, &all_ok);
    if (status == DNPEFF_OK && s2 != DNPEFF_OK) { status = s2; keep_msg(); }
    if (status == DNPEFF_OK && !all_ok) {
        status = fail(DNPEFF_ERR_IO, "another engine of the job could not read its rows of %s", path);
        keep_msg();
    }
    if (status == DNPEFF_OK) {
        status = dnpeff_set_csr_rows_device(eng, n, dense, k, row_begin, rows, nullptr, d_vals, d_idx, d_norms,
                                            min_values_per_parameter);
        if (status != DNPEFF_OK) keep_msg();
    }
    if (up) { cudaStreamSynchronize(up); cudaStreamDestroy(up); }
    for (int b2 = 0; b2 < 2; b2++) {
        if (done[b2]) cudaEventDestroy(done[b2]);
        cudaFreeHost(h_vals[b2]);
        cudaFreeHost(h_idx[b2]);
    }
    cudaFreeHost(h_norms);
    cudaFree(d_vals); cudaFree(d_idx); cudaFree(d_norms);
    if (status != DNPEFF_OK) return fail(status, "%s", msg);
    return DNPEFF_OK;
}

int dnpeff_save_decomposition_hdf5(const char* path, const float* W, const float* H,
                                   const int32_t* reduce_kept_indices, int64_t n_examples,
                                   int32_t rank, int64_t n_kept, int64_t full_dense_size) {
    if (!path || !W || !H || (!reduce_kept_indices && n_kept > 0)) return fail(DNPEFF_ERR_INVALID, "null argument");
    try {
        h5lite::Writer w(path);
        w.add_group("data");
        w.add_dataset("data/W", h5lite::DType::f32(), {(uint64_t)n_examples, (uint64_t)rank}, W);
        w.add_dataset("data/H", h5lite::DType::f32(), {(uint64_t)rank, (uint64_t)n_kept}, H);
        w.add_dataset("data/reduce_kept_indices", h5lite::DType::i32(), {(uint64_t)n_kept}, reduce_kept_indices);
        int32_t fds = (int32_t)full_dense_size;
        w.add_attr("data/reduce_kept_indices", "full_dense_size", h5lite::DType::i32(), {1}, &fds);
        w.finish();
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

int dnpeff_decomposition_hdf5_info(const char* path, int64_t* n_examples, int32_t* rank,
                                   int64_t* n_kept, int64_t* full_dense_size) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        h5lite::ObjectInfo W = rd.dataset("data/W"), H = rd.dataset("data/H");
        h5lite::ObjectInfo K = rd.dataset("data/reduce_kept_indices");
        if (W.space.dims.size() != 2 || H.space.dims.size() != 2 || W.space.dims[1] != H.space.dims[0])
            return fail(DNPEFF_ERR_IO, "data/W and data/H do not form a decomposition");
        if (n_examples) *n_examples = (int64_t)W.space.dims[0];
        if (rank) *rank = (int32_t)W.space.dims[1];
        if (n_kept) *n_kept = (int64_t)H.space.dims[1];
        if (full_dense_size) *full_dense_size = rd.attr_int(K, "full_dense_size");
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

int dnpeff_read_decomposition_hdf5(const char* path, float* W, float* H, int32_t* reduce_kept_indices) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        if (W) {
            h5lite::ObjectInfo o = rd.dataset("data/W");
            rd.read_leading(o, o.space.dims[0], o.space.dims[1], h5lite::DType::f32(), W);
        }
        if (H) {
            h5lite::ObjectInfo o = rd.dataset("data/H");
            rd.read_leading(o, o.space.dims[0], o.space.dims[1], h5lite::DType::f32(), H);
        }
        if (reduce_kept_indices) {
            h5lite::ObjectInfo o = rd.dataset("data/reduce_kept_indices");
            rd.read_leading(o, o.space.dims[0], 1, h5lite::DType::i32(), reduce_kept_indices);
        }
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

// ---- decomposition with H in CSR form (SparseNmfDecomposition, src/io/nmf_decomp_h5.h:134-237;
// written by scripts/sparsify_d_npeff.py:27-73 with int64 row offsets and int32 column ids) ----
int dnpeff_save_sparse_decomposition_hdf5(const char* path, const float* W, int64_t n_examples, int32_t rank,
                                          const int64_t* h_rowptr, const int32_t* h_colind, const float* h_vals,
                                          const int32_t* reduce_kept_indices, int64_t n_kept,
                                          int64_t full_dense_size) {
    if (!path || !W || !h_rowptr || (!reduce_kept_indices && n_kept > 0))
        return fail(DNPEFF_ERR_INVALID, "null argument");
    const int64_t nnz = h_rowptr[rank];
    if (nnz < 0 || (nnz > 0 && (!h_colind || !h_vals))) return fail(DNPEFF_ERR_INVALID, "bad CSR arrays");
    try {
        h5lite::Writer w(path);
        w.add_group("data");
        w.add_dataset("data/W", h5lite::DType::f32(), {(uint64_t)n_examples, (uint64_t)rank}, W);
        w.add_group("data/H");
        float dummy_f = 0.f;
        int32_t dummy_i = 0;
        w.add_dataset("data/H/values", h5lite::DType::f32(), {(uint64_t)nnz}, nnz ? (const void*)h_vals : &dummy_f);
        w.add_dataset("data/H/row_indices", h5lite::DType::i64(), {(uint64_t)rank + 1}, h_rowptr);
        w.add_dataset("data/H/column_indices", h5lite::DType::i32(), {(uint64_t)nnz},
                      nnz ? (const void*)h_colind : &dummy_i);
        int64_t shape[2] = {rank, n_kept};
        w.add_attr("data/H", "shape", h5lite::DType::i64(), {2}, shape);
        w.add_dataset("data/reduce_kept_indices", h5lite::DType::i32(), {(uint64_t)n_kept},
                      n_kept ? (const void*)reduce_kept_indices : &dummy_i);
        int32_t fds = (int32_t)full_dense_size;
        w.add_attr("data/reduce_kept_indices", "full_dense_size", h5lite::DType::i32(), {1}, &fds);
        w.finish();
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

int dnpeff_sparse_decomposition_hdf5_info(const char* path, int64_t* n_examples, int32_t* rank, int64_t* n_kept,
                                          int64_t* h_nnz, int64_t* full_dense_size) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        h5lite::ObjectInfo W = rd.dataset("data/W"), V = rd.dataset("data/H/values");
        h5lite::ObjectInfo R = rd.dataset("data/H/row_indices"), C = rd.dataset("data/H/column_indices");
        h5lite::ObjectInfo K = rd.dataset("data/reduce_kept_indices");
        std::vector<int64_t> shape = rd.attr_ints(rd.object(rd.find("data/H")), "shape");
        if (W.space.dims.size() != 2 || shape.size() != 2 || V.space.dims.size() != 1 || R.space.dims.size() != 1 ||
            C.space.dims.size() != 1)
            return fail(DNPEFF_ERR_IO, "not a sparse decomposition file");
        if ((int64_t)W.space.dims[1] != shape[0] || (int64_t)R.space.dims[0] != shape[0] + 1 ||
            V.space.dims[0] != C.space.dims[0] || K.space.count() != (uint64_t)shape[1])
            return fail(DNPEFF_ERR_IO, "data/W, data/H and data/reduce_kept_indices do not agree in shape");
        if (n_examples) *n_examples = (int64_t)W.space.dims[0];
        if (rank) *rank = (int32_t)shape[0];
        if (n_kept) *n_kept = shape[1];
        if (h_nnz) *h_nnz = (int64_t)V.space.dims[0];
        if (full_dense_size) *full_dense_size = rd.attr_int(K, "full_dense_size");
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

int dnpeff_read_sparse_decomposition_hdf5(const char* path, float* W, int64_t* h_rowptr, int32_t* h_colind,
                                          float* h_vals, int32_t* reduce_kept_indices) {
    if (!path) return fail(DNPEFF_ERR_INVALID, "null path");
    try {
        h5lite::Reader rd(path);
        if (W) {
            h5lite::ObjectInfo o = rd.dataset("data/W");
            rd.read_leading(o, o.space.dims[0], o.space.dims[1], h5lite::DType::f32(), W);
        }
        if (h_rowptr) {
            h5lite::ObjectInfo o = rd.dataset("data/H/row_indices");
            rd.read_leading(o, o.space.dims[0], 1, h5lite::DType::i64(), h_rowptr);
        }
        if (h_colind) {
            h5lite::ObjectInfo o = rd.dataset("data/H/column_indices");
            if (o.space.count() > 0) rd.read_leading(o, o.space.dims[0], 1, h5lite::DType::i32(), h_colind);
        }
        if (h_vals) {
            h5lite::ObjectInfo o = rd.dataset("data/H/values");
            if (o.space.count() > 0) rd.read_leading(o, o.space.dims[0], 1, h5lite::DType::f32(), h_vals);
        }
        if (reduce_kept_indices) {
            h5lite::ObjectInfo o = rd.dataset("data/reduce_kept_indices");
            if (o.space.count() > 0) rd.read_leading(o, o.space.dims[0], 1, h5lite::DType::i32(), reduce_kept_indices);
        }
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

// Generic probe used by the tests: shape and type of any dataset.
int dnpeff_hdf5_dataset_info(const char* path, const char* dataset, int32_t* rank, int64_t dims[4],
                             int32_t* is_float, int32_t* type_size) {
    if (!path || !dataset) return fail(DNPEFF_ERR_INVALID, "null argument");
    try {
        h5lite::Reader rd(path);
        h5lite::ObjectInfo o = rd.dataset(dataset);
        if (o.space.dims.size() > 4) return fail(DNPEFF_ERR_UNSUPPORTED, "rank > 4");
        if (rank) *rank = (int32_t)o.space.dims.size();
        for (size_t i = 0; i < o.space.dims.size() && dims; i++) dims[i] = (int64_t)o.space.dims[i];
        if (is_float) *is_float = o.type.cls == h5lite::TypeClass::Float;
        if (type_size) *type_size = o.type.size;
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

// Reads the leading rows x cols block of a rank <= 2 dataset as float64.
int dnpeff_hdf5_read_f64(const char* path, const char* dataset, int64_t rows, int64_t cols, double* out) {
    if (!path || !dataset || !out) return fail(DNPEFF_ERR_INVALID, "null argument");
    try {
        h5lite::Reader rd(path);
        h5lite::ObjectInfo o = rd.dataset(dataset);
        h5lite::DType f64 = {h5lite::TypeClass::Float, 8, true, false};
        rd.read_leading(o, (uint64_t)rows, (uint64_t)cols, f64, out);
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

// Writes a D-PEF file with the layout of npeff/fishers/d_pefs_computer.py:235-251
// (data/fisher/{values,indices} + attribute dense_fisher_size, data/dense_fisher_norms).
int dnpeff_write_pef_hdf5(const char* path, int64_t n_examples, int64_t n_values_per_example,
                          const float* vals, const int32_t* indices, const float* norms,
                          int64_t dense_fisher_size) {
    if (!path || !vals || !indices || !norms) return fail(DNPEFF_ERR_INVALID, "null argument");
    try {
        h5lite::Writer w(path);
        w.add_group("data");
        w.add_group("data/fisher");
        int64_t dfs64 = dense_fisher_size;
        int32_t dfs32 = (int32_t)dense_fisher_size;
        // the reference reader demands a 4-byte attribute (pef_fisher_h5.h:145-154)
        if (dense_fisher_size <= INT32_MAX) w.add_attr("data/fisher", "dense_fisher_size", h5lite::DType::i32(), {}, &dfs32);
        else w.add_attr("data/fisher", "dense_fisher_size", h5lite::DType::i64(), {}, &dfs64);
        w.add_dataset("data/fisher/values", h5lite::DType::f32(),
                      {(uint64_t)n_examples, (uint64_t)n_values_per_example}, vals);
        w.add_dataset("data/fisher/indices", h5lite::DType::i32(),
                      {(uint64_t)n_examples, (uint64_t)n_values_per_example}, indices);
        w.add_dataset("data/dense_fisher_norms", h5lite::DType::f32(), {(uint64_t)n_examples}, norms);
        w.finish();
    } catch (const std::exception& ex) {
        return fail(DNPEFF_ERR_IO, "%s", ex.what());
    }
    return DNPEFF_OK;
}

}  // extern "C"
