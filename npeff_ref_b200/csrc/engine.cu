// Host side of the D-NPEFF engine and its C ABI (see include/dnpeff.h).
//
// One engine = one column shard of the pruned PEF matrix A on one device:
//   A  as CSR (rows = examples) and CSC (rows = features), fp32 + int32 + int64 offsets
//   W  [n_rows, r] row-major, replicated on every engine of a job
//   H  [n_cols_shard, r] row-major: the reference's column-major r x m_s matrix
//      (multi_mu_dense_factors_device_contexts1.h:413-429), byte for byte
// Iteration (multi_mu_dense_factors_nmf1.h:175-182): W first, then H.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <functional>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels_dense.cuh"
#include "kernels_hoyer.cuh"
#include "kernels_prep.cuh"
#include "kernels_spmm.cuh"
#include "kernels_tc.cuh"
#include "nccl_dyn.h"

using namespace dnpeff;

namespace {

// While a PoolScope is alive on this thread, DevBuf takes its memory from the
// device's stream-ordered pool on that stream: cudaFree waits for every stream of
// the device -- also for an upload that is meant to overlap the loader -- whereas
// cudaFreeAsync only orders the release behind the work queued so far.
struct PoolScope {
    static thread_local cudaStream_t stream;
    static thread_local int depth;
    int device = 0;
    uint64_t saved_threshold = 0;
    bool have_saved = false;
    explicit PoolScope(cudaStream_t st) {
        if (depth++ == 0) {
            stream = st;
            cudaGetDevice(&device);
            cudaMemPool_t pool;
            if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
                have_saved = cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &saved_threshold) == cudaSuccess;
                uint64_t keep = UINT64_MAX;  // no release to the OS in the middle of the work
                cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            }
        }
    }
    ~PoolScope() {
        if (--depth == 0) {
            cudaStreamSynchronize(stream);
            cudaMemPool_t pool;
            if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
                // the pool gets the caller's setting back; what this scope parked in it
                // goes back to the device unless the caller wants memory kept
                if (have_saved) cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &saved_threshold);
                if (!have_saved || saved_threshold == 0) cudaMemPoolTrimTo(pool, 0);
            }
            stream = nullptr;
        }
    }
    static bool active() { return depth > 0; }
};
thread_local cudaStream_t PoolScope::stream = nullptr;
thread_local int PoolScope::depth = 0;

template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t count = 0;
    bool pooled = false;
    cudaStream_t pool_stream = nullptr;
    DevBuf() {}
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    ~DevBuf() { release(); }
    int alloc(size_t n) {
        release();
        count = n;
        // (large buffers stay with cudaMalloc: growing and trimming the pool by
        // gigabytes costs far more than the synchronisation it avoids)
        if (PoolScope::active() && sizeof(T) * n <= ((size_t)64 << 20)) {
            pooled = true;
            pool_stream = PoolScope::stream;
            DN_CUDA(cudaMallocAsync((void**)&p, sizeof(T) * (n ? n : 1), pool_stream));
        } else {
            pooled = false;
            DN_CUDA(cudaMalloc((void**)&p, sizeof(T) * (n ? n : 1)));
        }
        return DNPEFF_OK;
    }
    int alloc_zero(size_t n, cudaStream_t st) {
        DN_TRY(alloc(n));
        DN_CUDA(cudaMemsetAsync(p, 0, sizeof(T) * (n ? n : 1), st));
        return DNPEFF_OK;
    }
    void release() {
        if (p) {
            if (pooled) cudaFreeAsync(p, pool_stream);
            else cudaFree(p);
        }
        p = nullptr;
        count = 0;
    }
    T* take() {
        T* q = p;
        p = nullptr;
        count = 0;
        return q;
    }
};

template <typename T>
void dev_free(T*& p) {
    if (p) cudaFree(p);
    p = nullptr;
}

// Exclusive scan of N items into out[0..N) (int64).  Callers that want the
// total pass N+1 items whose last one is zero.
template <typename TIn>
int scan_exclusive(const TIn* in, int64_t* out, int64_t N, cudaStream_t st) {
    if (N <= 0) return DNPEFF_OK;
    int64_t nb = ceil_div(N, 4096);
    if (nb == 1) {
        k_scan_block<TIn><<<1, 1024, 0, st>>>(in, out, nullptr, N);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
        return DNPEFF_OK;
    }
    DevBuf<int64_t> bs, bsp;
    DN_TRY(bs.alloc((size_t)nb));
    DN_TRY(bsp.alloc((size_t)nb));
    k_scan_block<TIn><<<(unsigned)nb, 1024, 0, st>>>(in, out, bs.p, N);
    DN_LAUNCH_CHECK();
    DN_TRY(scan_exclusive<int64_t>(bs.p, bsp.p, nb, st));
    k_scan_add<<<(unsigned)nb, 1024, 0, st>>>(out, bsp.p, N);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(2);
    DN_CUDA(cudaStreamSynchronize(st));  // bs/bsp are released on return
    return DNPEFF_OK;
}

struct TimedRegion {
    int id;
    cudaEvent_t a, b;
};

}  // namespace

struct dnpeff_engine {
    dnpeff_params p;
    int device = 0;
    cudaStream_t st = nullptr;
    bool own_stream = false;

    int64_t n = 0, m_full = 0, m_kept = 0, c0 = 0, ms = 0, nnz = 0;
    ShardMap map = {0, 0, 1, 0, 0};
    bool loaded = false, have_factors = false, csc_ready = false, csc_hot_ready = false;

    float* a_vals = nullptr;
    int32_t* a_col = nullptr;
    int64_t* a_rowptr = nullptr;
    // CSC arrays.  With the popular block kept dense only the other columns are ever
    // read from the CSC: the arrays then hold entries [c_base, nnz) of the full CSC
    // (c_base = c_colptr[n_hot]) and are addressed through csc_vals()/csc_rows(),
    // which shift the pointers so that the offsets in c_colptr apply unchanged.
    float* c_vals = nullptr;
    int32_t* c_row = nullptr;
    int64_t* c_colptr = nullptr;
    int64_t c_base = 0;
    float* w_spare = nullptr;  // n x r, wide ranks only: a W update is written here, then W and w_spare change places
    int32_t* new_to_og = nullptr;

    // Internal column order: [n_hot popular columns][the rest], each in local-id
    // order.  H, WA and the CSC use it; perm[jp] = local id, inv_perm[local] = jp.
    int32_t* perm = nullptr;
    int32_t* inv_perm = nullptr;
    int64_t n_hot = 0;
    BucketMap bm = {0, 1, 1, 0, 0};
    int n_tail_blocks = 0;
    float* b_vals = nullptr;      // rows of A with entries grouped by bucket, internal ids
    int32_t* b_col = nullptr;
    uint32_t* tail_off = nullptr;  // [n][n_tail_blocks + 1]
    std::vector<int64_t> tail_nnz;  // stored entries per tail block
    int* work_counter = nullptr;
    int* d_err = nullptr;
    // Popular block of A kept dense for the tensor-core product (null: the popular
    // part goes through the tiled sparse kernel): x1 = rows x popular columns,
    // x2 = its transpose, both in the blocked layout of k_block_tc.
    float* x1 = nullptr;
    float* x2 = nullptr;
    BlockTcPlan plan_x1 = {}, plan_x2 = {};
    float* blk_ysplit = nullptr;
    float* blk_partial = nullptr;

    float* W = nullptr;
    float* H = nullptr;
    float* AHG = nullptr;  // [n*r | r*r]: A*H^T partial and H*H^T partial, one allreduce
    float* WA = nullptr;   // [ms*r], made on the first H update
    float* WW = nullptr;   // [r*r]
    float* gram_scratch = nullptr;
    size_t gram_scratch_floats = 0;
    float* tc_scratch = nullptr;  // 2*r*r: the update's small matrix split for the tensor cores
    double* red_partial = nullptr;  // device, 2*kRedBlocks doubles
    double* red_out = nullptr;      // device, 4 doubles
    void* h_pinned = nullptr;       // 256 bytes of page-locked host memory for scalar read-backs
    SpmmPlan plan_csr, plan_csc;

    double a_sq = 0.0, a_sum = 0.0;
    double a_sq_global = -1.0;
    int64_t w_row_offset = 0;  // global index of this engine's first row (generated W only)

    ncclComm_t comm = nullptr;
    int comm_rank = 0, comm_size = 1;

    bool timing = false;
    std::vector<TimedRegion> regions;
    std::vector<cudaEvent_t> ev_pool;
    double t_ms[DNPEFF_N_TIMERS] = {0};
    int64_t t_n[DNPEFF_N_TIMERS] = {0};
    int64_t launches0 = 0;

    // dnpeff_set_option values; 0 = the built-in default
    int opt_loader_slabs = 0;
    int64_t opt_tail_block_bytes = 0;
    int opt_popular_divisor = 0;
    uint32_t opt_wait_limit = kTiledSpinLimit;
    bool opt_keep_csr = false;
};

namespace {

int check_kernel_status(dnpeff_engine* e);

// A pointer `base` elements before p (never dereferenced below p + base).
template <typename T>
T* shifted(T* p, int64_t base) {
    return reinterpret_cast<T*>(reinterpret_cast<uintptr_t>(p) - (uintptr_t)base * sizeof(T));
}
float* csc_vals(const dnpeff_engine* e) { return shifted(e->c_vals, e->c_base); }
int32_t* csc_rows(const dnpeff_engine* e) { return shifted(e->c_row, e->c_base); }

constexpr int kRedBlocks = 4 * kNumSMs;
constexpr int kMaxHotTiles = 1024;            // tiles of popular columns per row walk
// Slice of H gathered per tail launch.  It has to stay L2-resident (126 MB, shared
// with the A*H^T accumulator and the streamed entries) while all rows sweep it, and
// every further launch costs about 11 us: 48 MB is the measured optimum on B200.
constexpr int64_t kTailBlockBytes = 48 << 20;
constexpr int kMaxTailBlocks = 512;

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

struct ScopedTimer {
    dnpeff_engine* e;
    int id;
    cudaEvent_t a = nullptr, b = nullptr;
    ScopedTimer(dnpeff_engine* e_, int id_) : e(e_), id(id_) {
        if (!e->timing) return;
        a = get();
        b = get();
        cudaEventRecord(a, e->st);
    }
    ~ScopedTimer() {
        if (!e->timing) return;
        cudaEventRecord(b, e->st);
        e->regions.push_back({id, a, b});
    }
    cudaEvent_t get() {
        if (!e->ev_pool.empty()) {
            cudaEvent_t x = e->ev_pool.back();
            e->ev_pool.pop_back();
            return x;
        }
        cudaEvent_t x;
        cudaEventCreate(&x);
        return x;
    }
};

// DNPEFF_NO_TC=1 keeps the dense contractions on the CUDA-core kernels (A/B runs).
bool tensor_cores_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* s = getenv("DNPEFF_NO_TC");
        v = (s && s[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

// DNPEFF_TRACE=1 prints the wall time of the loader's phases to stderr (each
// phase is closed with a stream synchronisation, so the trace slows the load).
struct PhaseTrace {
    cudaStream_t st;
    bool on;
    std::chrono::high_resolution_clock::time_point t;
    explicit PhaseTrace(cudaStream_t s) : st(s) {
        const char* v = getenv("DNPEFF_TRACE");
        on = v && v[0] == '1';
        if (on) t = std::chrono::high_resolution_clock::now();
    }
    void mark(const char* what) {
        if (!on) return;
        cudaStreamSynchronize(st);
        auto n = std::chrono::high_resolution_clock::now();
        fprintf(stderr, "[dnpeff] %-28s %8.2f ms\n", what, std::chrono::duration<double, std::milli>(n - t).count());
        t = n;
    }
};

// Popular columns hold at least ceil(n / div) entries.  With the dense tensor-core
// block a column pays off from a few percent of density on; the sparse tiled
// kernel needs longer columns.
int hot_divisor(const dnpeff_engine* e, bool dense) {
    if (e->opt_popular_divisor >= 2) return e->opt_popular_divisor;
    return dense ? 16 : 8;
}

// G = X^T X: tcgen05 kernel where the rank allows, CUDA-core kernel otherwise.
int gram_any(const float* X, int64_t rows, int r, float* G, float* scratch, int* err, cudaStream_t st,
             uint32_t wait_limit = kTiledSpinLimit) {
    if (tensor_cores_enabled() && gram_tc_ok(r)) return gram_blk_launch(X, rows, r, G, scratch, err, st, wait_limit);
    if (tensor_cores_enabled() && gram_wide_ok(r) && rows > 0)
        return gram_wide_launch(X, rows, r, G, scratch, err, st, wait_limit);
    return gram_launch(X, rows, r, G, scratch, st);
}

size_t gram_any_scratch(int64_t rows, int r) {
    size_t a = gram_plan(rows, r).scratch_floats;
    size_t b = gram_tc_ok(r) ? gram_blk_plan(rows).scratch_floats : 0;
    if (gram_wide_ok(r)) b = gram_wide_plan(rows, r).scratch_floats;
    return a > b ? a : b;
}

// tc_scratch: 2*r*r floats.
// The wide-rank kernels cannot update X in place: their result goes to Num when the caller
// is done with it (num_is_scratch), else to the caller's spare buffer of rows * r floats
// (out_buf), else to a temporary.  With `moved` given, the result stays there and *moved
// tells the caller to exchange its two buffers; without it, one device copy brings the
// result back to X.
int mu_update_any(float* X, const float* Num, const float* G, int64_t rows, int r, float eps,
                  float* tc_scratch, int* err, cudaStream_t st, bool num_is_scratch = false,
                  float* out_buf = nullptr, uint32_t wait_limit = kTiledSpinLimit, bool* moved = nullptr) {
    if (moved) *moved = false;
    if (tensor_cores_enabled() && mu_update_ws_ok(r))
        return mu_update_ws_launch(X, Num, X, G, rows, r, eps, tc_scratch, err, st, wait_limit);
    if (tensor_cores_enabled() && mu_update_tc_ok(r))
        return mu_update_tc_launch(X, Num, G, rows, r, eps, tc_scratch, err, st);
    if (tensor_cores_enabled() && mu_update_ws_wide_ok(r) && rows > 0) {
        DevBuf<float> tmp;
        float* out = num_is_scratch ? const_cast<float*>(Num) : out_buf;
        if (!out) {
            DN_TRY(tmp.alloc((size_t)(rows * r)));
            out = tmp.p;
        }
        DN_TRY(mu_update_ws_launch(X, Num, out, G, rows, r, eps, tc_scratch, err, st, wait_limit));
        if (moved && !tmp.p) {
            *moved = true;
            return DNPEFF_OK;
        }
        DN_CUDA(cudaMemcpyAsync(X, out, sizeof(float) * (size_t)(rows * r), cudaMemcpyDeviceToDevice, st));
        if (tmp.p) DN_CUDA(cudaStreamSynchronize(st));  // tmp is released on return
        return DNPEFF_OK;
    }
    return mu_update_launch(X, Num, G, rows, r, eps, st);
}

void free_matrix(dnpeff_engine* e) {
    dev_free(e->a_vals); dev_free(e->a_col); dev_free(e->a_rowptr);
    dev_free(e->c_vals); dev_free(e->c_row); dev_free(e->c_colptr);
    e->c_base = 0;
    dev_free(e->w_spare);
    dev_free(e->new_to_og);
    dev_free(e->perm); dev_free(e->inv_perm);
    dev_free(e->b_vals); dev_free(e->b_col); dev_free(e->tail_off);
    dev_free(e->x1); dev_free(e->x2); dev_free(e->blk_ysplit); dev_free(e->blk_partial);
    e->tail_nnz.clear();
    e->n_hot = 0; e->n_tail_blocks = 0;
    dev_free(e->W); dev_free(e->H); dev_free(e->AHG); dev_free(e->WA); dev_free(e->WW);
    dev_free(e->gram_scratch);
    dev_free(e->tc_scratch);
    e->gram_scratch_floats = 0;
    dev_free(e->plan_csr.long_list);
    dev_free(e->plan_csc.long_list);
    e->plan_csr = SpmmPlan();
    e->plan_csc = SpmmPlan();
    e->loaded = e->have_factors = e->csc_ready = e->csc_hot_ready = false;
    e->a_sq_global = -1.0;
}

// Small device -> host read through the engine's page-locked scratch: a copy into
// pageable memory would queue behind a large upload that is still in flight.
int read_small(dnpeff_engine* e, const void* dptr, size_t bytes, void* out) {
    if (bytes > 256 || !e->h_pinned) {
        DN_CUDA(cudaMemcpyAsync(out, dptr, bytes, cudaMemcpyDeviceToHost, e->st));
        DN_CUDA(cudaStreamSynchronize(e->st));
        return DNPEFF_OK;
    }
    DN_CUDA(cudaMemcpyAsync(e->h_pinned, dptr, bytes, cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    memcpy(out, e->h_pinned, bytes);
    return DNPEFF_OK;
}

int read_err_flag(int* d_err, cudaStream_t st, int* host) {
    DN_CUDA(cudaMemcpyAsync(host, d_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    DN_CUDA(cudaStreamSynchronize(st));
    return DNPEFF_OK;
}

int data_error(int flags) {
    if (flags & kErrColRange) return fail(DNPEFF_ERR_DATA, "column index outside [0, n_cols_full)");
    if (flags & kErrRowPtr) return fail(DNPEFF_ERR_DATA, "row offsets are not non-decreasing");
    if (flags & kErrDuplicate) return fail(DNPEFF_ERR_DATA, "a row holds the same column twice");
    return DNPEFF_OK;
}

// getSizeOfSplit (src/util/matrix_util.h:10-20): equal widths, remainder to the last.
void shard_range(int64_t total, int n_shards, int idx, int64_t* start, int64_t* size) {
    int64_t base = total / n_shards;
    *start = base * idx;
    *size = (idx == n_shards - 1) ? base + total % n_shards : base;
}

// The values may arrive in slabs of rows (a host upload still in flight): rows
// [row_end[s-1], row_end[s]) are valid once ready[s] has fired (a null event: valid
// already).  Everything that needs the column ids only runs before the first wait.
struct LoadSlabs {
    std::vector<int64_t> row_end;
    std::vector<cudaEvent_t> ready;
    int count() const { return (int)row_end.size(); }
};

// d_retained != nullptr: the kept columns are that list of original ids (device
// pointer, n_retained of them) instead of the columns with >= min_count entries.
// The rows every engine of a job holds when the matrix arrives in row slices
// (dnpeff_set_csr_rows): equal-size contiguous ranges, the remainder spread over
// the leading engines.
void row_slice(int64_t n_total, int n_parts, int idx, int64_t* begin, int64_t* count) {
    *begin = n_total * idx / n_parts;
    *count = n_total * (idx + 1) / n_parts - *begin;
}

// Row slice of the input (dnpeff_set_csr_rows): the arrays hold rows
// [row_begin, row_begin + n_in) of the matrix and every engine of the job is making
// the same call on its own slice.  Column counts are summed over the engines, and
// every entry travels to the engine that owns its column.
struct RowSlice {
    int64_t n_in;
    int64_t row_begin;
};

int load_device(dnpeff_engine* e, int64_t n, int64_t m_full, int64_t k, const int64_t* d_rowptr,
                const float* d_vals, const int32_t* d_col, const float* d_norms, int32_t min_count,
                const int32_t* d_retained = nullptr, int64_t n_retained = 0, const LoadSlabs* slabs = nullptr,
                const RowSlice* slice = nullptr) {
    if (n < 0 || m_full < 0 || (d_rowptr == nullptr && k < 0))
        return fail(DNPEFF_ERR_INVALID, "negative shape");
    if (n >= INT32_MAX || m_full >= INT32_MAX)
        return fail(DNPEFF_ERR_UNSUPPORTED, "n_rows and n_cols_full must fit int32");
    cudaStream_t st = e->st;
    free_matrix(e);
    PoolScope pool_scope(st);
    const int r = e->p.rank;
    const int64_t n_in = slice ? slice->n_in : n;  // rows the input arrays hold

    int64_t nnz_in = n_in * k;
    if (d_rowptr) {
        if (n_in > 0) {
            DN_TRY(read_small(e, d_rowptr + n_in, sizeof(int64_t), &nnz_in));
        } else {
            nnz_in = 0;
        }
    }
    if (nnz_in < 0) return fail(DNPEFF_ERR_DATA, "negative nnz");

    DevBuf<int> err;
    DN_TRY(err.alloc_zero(1, st));
    int herr = 0;
    PhaseTrace trace(st);
    trace.mark("upload / inputs ready");

    // 1. explicit entries per original column
    DevBuf<int32_t> counts, flags, og_to_new;
    DevBuf<int64_t> pos;
    DN_TRY(counts.alloc_zero((size_t)m_full + 1, st));
    if (nnz_in > 0) {
        int64_t blocks = std::min<int64_t>(ceil_div(nnz_in, 256), (int64_t)kNumSMs * 16);
        k_count_columns<<<(unsigned)blocks, 256, 0, st>>>(d_col, nnz_in, m_full, counts.p, err.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    if (slice) {
        // the pruning decision needs the counts over all rows: one integer sum over the
        // engines; a bad index seen by any of them fails the load on all of them
        DN_NCCL(nccl_api().AllReduce(counts.p, counts.p, (size_t)m_full + 1, ncclInt32, ncclSum, e->comm, st));
        DN_NCCL(nccl_api().AllReduce(err.p, err.p, 1, ncclInt32, ncclMax, e->comm, st));
    }
    DN_TRY(read_small(e, err.p, sizeof(int), &herr));
    if (herr) return data_error(herr);

    trace.mark("count columns");
    // 2. keep mask -> ascending renumbering, or the caller's list of kept columns
    DN_TRY(og_to_new.alloc((size_t)m_full + 1));
    int64_t m_kept = 0;
    if (d_retained) {
        if (n_retained < 0 || n_retained >= INT32_MAX) return fail(DNPEFF_ERR_INVALID, "bad retained-column count");
        m_kept = n_retained;
        DN_CUDA(cudaMalloc((void**)&e->new_to_og, sizeof(int32_t) * (size_t)std::max<int64_t>(m_kept, 1)));
        DN_CUDA(cudaMemsetAsync(og_to_new.p, 0xFF, sizeof(int32_t) * ((size_t)m_full + 1), st));
        if (m_kept > 0) {
            k_retain_maps<<<(unsigned)ceil_div(m_kept, 256), 256, 0, st>>>(d_retained, m_kept, m_full, og_to_new.p,
                                                                          e->new_to_og, err.p);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
        }
        DN_TRY(read_err_flag(err.p, st, &herr));
        if (herr) return fail(DNPEFF_ERR_DATA, "retained column id outside [0, n_cols_full)");
    } else {
        DN_TRY(flags.alloc_zero((size_t)m_full + 1, st));
        DN_TRY(pos.alloc((size_t)m_full + 1));
        if (m_full > 0) {
            k_keep_flags<<<(unsigned)ceil_div(m_full, 256), 256, 0, st>>>(counts.p, m_full, min_count, flags.p);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
        }
        DN_TRY(scan_exclusive<int32_t>(flags.p, pos.p, m_full + 1, st));
        DN_TRY(read_small(e, pos.p + m_full, sizeof(int64_t), &m_kept));
        DN_CUDA(cudaMalloc((void**)&e->new_to_og, sizeof(int32_t) * (size_t)std::max<int64_t>(m_kept, 1)));
        if (m_full > 0) {
            k_build_maps<<<(unsigned)ceil_div(m_full, 256), 256, 0, st>>>(flags.p, pos.p, m_full,
                                                                         og_to_new.p, e->new_to_og);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
        }
    }

    trace.mark("pruning maps");
    // 3. this engine's range of kept columns
    int64_t c0 = 0, ms = 0;
    ShardMap map;
    if (e->p.shard_mode == DNPEFF_SHARD_CYCLIC) {
        int64_t G = e->p.n_shards, d = e->p.shard_index;
        ms = m_kept > d ? (m_kept - d + G - 1) / G : 0;
        c0 = d;
        map = {c0, ms, (int32_t)G, (int32_t)d, 1};
    } else {
        shard_range(m_kept, e->p.n_shards, e->p.shard_index, &c0, &ms);
        map = {c0, ms, 1, 0, 0};
    }

    // 4. shard row lengths -> row offsets
    DevBuf<int32_t> row_count;
    DN_TRY(row_count.alloc_zero((size_t)n + 1, st));
    DN_CUDA(cudaMalloc((void**)&e->a_rowptr, sizeof(int64_t) * (size_t)(n + 1)));
    // Row slices: for every engine d of the job, the lengths of this slice's rows
    // inside d's columns (rc_to[d], with offsets off_to[d] for the extraction); the
    // lengths travel to d, which puts the slices of all engines one after the other.
    const int G = slice ? e->comm_size : 1;
    std::vector<ShardMap> map_of((size_t)G);
    // (one allocation each for all destinations: device allocations are driver calls
    // that the processes of a box serialise on)
    DevBuf<int32_t> rc_all;
    DevBuf<int64_t> off_all;
    std::vector<int32_t*> rc_to((size_t)G, nullptr);
    std::vector<int64_t*> off_to((size_t)G, nullptr);
    if (slice) {
        DN_TRY(rc_all.alloc_zero((size_t)G * ((size_t)n_in + 1), st));
        DN_TRY(off_all.alloc((size_t)G * ((size_t)n_in + 1)));
        for (int d = 0; d < G; d++) {
            rc_to[(size_t)d] = rc_all.p + (size_t)d * ((size_t)n_in + 1);
            off_to[(size_t)d] = off_all.p + (size_t)d * ((size_t)n_in + 1);
        }
    }
    std::vector<int64_t> send_count((size_t)G, 0), slice_begin((size_t)G + 1, 0);
    if (slice) {
        for (int d = 0; d < G; d++) {
            if (e->p.shard_mode == DNPEFF_SHARD_CYCLIC) {
                int64_t w = m_kept > d ? (m_kept - d + G - 1) / G : 0;
                map_of[(size_t)d] = {d, w, (int32_t)G, (int32_t)d, 1};
            } else {
                int64_t b = 0, w = 0;
                shard_range(m_kept, G, d, &b, &w);
                map_of[(size_t)d] = {b, w, 1, 0, 0};
            }
            int64_t sb = 0, sc = 0;
            row_slice(n, G, d, &sb, &sc);
            slice_begin[(size_t)d] = sb;
            if (n_in > 0) {
                int64_t blocks = std::min<int64_t>(n_in, (int64_t)kNumSMs * 32);
                k_row_counts<<<(unsigned)blocks, 256, 0, st>>>(d_col, d_rowptr, k, n_in, og_to_new.p, map_of[(size_t)d],
                                                              rc_to[(size_t)d], err.p);
                DN_LAUNCH_CHECK();
                DN_COUNT_LAUNCH(1);
            }
            DN_TRY(scan_exclusive<int32_t>(rc_to[(size_t)d], off_to[(size_t)d], n_in + 1, st));
        }
        // entries bound for each engine: the last offset of every destination, one read-back
        if (e->h_pinned && (size_t)G * sizeof(int64_t) <= 256) {
            DN_CUDA(cudaMemcpy2DAsync(e->h_pinned, sizeof(int64_t), off_all.p + n_in, sizeof(int64_t) * ((size_t)n_in + 1),
                                      sizeof(int64_t), (size_t)G, cudaMemcpyDeviceToHost, st));
            DN_CUDA(cudaStreamSynchronize(st));
            memcpy(send_count.data(), e->h_pinned, sizeof(int64_t) * (size_t)G);
        } else {
            for (int d = 0; d < G; d++)
                DN_TRY(read_small(e, off_to[(size_t)d] + n_in, sizeof(int64_t), &send_count[(size_t)d]));
        }
        slice_begin[(size_t)G] = n;
        if (slice->row_begin != slice_begin[(size_t)e->comm_rank] ||
            n_in != slice_begin[(size_t)e->comm_rank + 1] - slice_begin[(size_t)e->comm_rank])
            return fail(DNPEFF_ERR_INVALID, "row slice of engine %d must be rows [%lld, %lld)", e->comm_rank,
                        (long long)slice_begin[(size_t)e->comm_rank], (long long)slice_begin[(size_t)e->comm_rank + 1]);
        int gs = DNPEFF_OK;
        DN_NCCL(nccl_api().GroupStart());
        for (int d = 0; d < G; d++) {
            const int64_t cnt_d = slice_begin[(size_t)d + 1] - slice_begin[(size_t)d];
            if (d == e->comm_rank) continue;
            if (n_in > 0) DN_NCCL_IN_GROUP(gs, nccl_api().Send(rc_to[(size_t)d], (size_t)n_in, ncclInt32, d, e->comm, st));
            if (cnt_d > 0)
                DN_NCCL_IN_GROUP(gs, nccl_api().Recv(row_count.p + slice_begin[(size_t)d], (size_t)cnt_d, ncclInt32, d,
                                                     e->comm, st));
        }
        DN_NCCL(nccl_api().GroupEnd());
        DN_TRY(gs);
        if (n_in > 0)
            DN_CUDA(cudaMemcpyAsync(row_count.p + slice->row_begin, rc_to[(size_t)e->comm_rank], sizeof(int32_t) * (size_t)n_in,
                                    cudaMemcpyDeviceToDevice, st));
    } else if (n > 0) {
        int64_t blocks = std::min<int64_t>(n, (int64_t)kNumSMs * 32);
        k_row_counts<<<(unsigned)blocks, 256, 0, st>>>(d_col, d_rowptr, k, n, og_to_new.p, map,
                                                      row_count.p, err.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    DN_TRY(scan_exclusive<int32_t>(row_count.p, e->a_rowptr, n + 1, st));
    int64_t nnz = 0;
    DN_TRY(read_small(e, e->a_rowptr + n, sizeof(int64_t), &nnz));
    DN_TRY(read_small(e, err.p, sizeof(int), &herr));
    if (herr) return data_error(herr);

    trace.mark("row counts + scan");
    // 5. (the order-preserving extraction needs the values and comes further down,
    //    slab by slab; everything up to there needs the column ids only)
    // The shard's CSR in input order is an intermediate: it is kept only on request
    // (option keep_canonical_csr, for dnpeff_export_shard_csr); otherwise one slab
    // of it at a time lives in a temporary on its way into the bucketed layout.
    if (e->opt_keep_csr) {
        DN_CUDA(cudaMalloc((void**)&e->a_vals, sizeof(float) * (size_t)std::max<int64_t>(nnz, 1)));
        DN_CUDA(cudaMalloc((void**)&e->a_col, sizeof(int32_t) * (size_t)std::max<int64_t>(nnz, 1)));
    }
    // 6. internal column order: popular columns first (they get the tiled,
    //    shared-memory kernels), then the rest; both parts in local-id order
    DevBuf<int32_t> cnt_s, hot_flags, cnt_p;
    DevBuf<int64_t> hot_pos;
    DN_TRY(cnt_s.alloc((size_t)ms + 1));
    k_gather_counts<<<(unsigned)ceil_div(ms + 1, 256), 256, 0, st>>>(counts.p, e->new_to_og, map, cnt_s.p);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    const bool fast = spmm_fast_rank(r);
    bool dense = fast && tensor_cores_enabled() && block_tc_ok(r);
    int tile = fast ? spmm_tile_rows(r) : 128;
    int32_t hot_thr = (int32_t)std::max<int64_t>(2, ceil_div(n, hot_divisor(e, dense)));
    if (!fast || n < 32) hot_thr = INT32_MAX;  // no hot part
    DN_TRY(hot_flags.alloc((size_t)ms + 1));
    DN_TRY(hot_pos.alloc((size_t)ms + 1));
    k_hot_flags<<<(unsigned)ceil_div(ms + 1, 256), 256, 0, st>>>(cnt_s.p, ms, hot_thr, hot_flags.p);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    DN_TRY(scan_exclusive<int32_t>(hot_flags.p, hot_pos.p, ms + 1, st));
    int64_t n_hot = 0;
    DN_TRY(read_small(e, hot_pos.p + ms, sizeof(int64_t), &n_hot));
    int64_t max_hot = (int64_t)kMaxHotTiles * tile;
    if (dense) {
        // both dense copies (8 bytes per element of the block) within a third of
        // the memory that is free now
        size_t free_b = 0, total_b = 0;
        DN_CUDA(cudaMemGetInfo(&free_b, &total_b));
        max_hot = (int64_t)(free_b / 3 / (8 * (size_t)std::max<int64_t>(n, 1)));
        max_hot = std::min<int64_t>(max_hot / 128 * 128, (int64_t)1 << 21);
        if (max_hot < 128) {
            dense = false;
            max_hot = (int64_t)kMaxHotTiles * tile;
        }
    }
    if (n_hot > max_hot || n_hot < 8) {
        // too many (cap the tile loop) or too few to be worth a launch: raise the
        // bar until the count fits, or drop the hot part
        if (n_hot > max_hot) {
            // keep the max_hot most popular: find the count threshold by bisection on the host
            std::vector<int32_t> hc((size_t)ms);
            DN_CUDA(cudaMemcpyAsync(hc.data(), cnt_s.p, sizeof(int32_t) * (size_t)ms, cudaMemcpyDeviceToHost, st));
            DN_CUDA(cudaStreamSynchronize(st));
            std::vector<int32_t> sorted(hc);
            std::nth_element(sorted.begin(), sorted.begin() + (size_t)max_hot, sorted.end(), std::greater<int32_t>());
            hot_thr = sorted[(size_t)max_hot] + 1;
        } else {
            hot_thr = INT32_MAX;
        }
        k_hot_flags<<<(unsigned)ceil_div(ms + 1, 256), 256, 0, st>>>(cnt_s.p, ms, hot_thr, hot_flags.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
        DN_TRY(scan_exclusive<int32_t>(hot_flags.p, hot_pos.p, ms + 1, st));
        DN_TRY(read_small(e, hot_pos.p + ms, sizeof(int64_t), &n_hot));
    }
    DN_CUDA(cudaMalloc((void**)&e->perm, sizeof(int32_t) * (size_t)std::max<int64_t>(ms, 1)));
    DN_CUDA(cudaMalloc((void**)&e->inv_perm, sizeof(int32_t) * (size_t)std::max<int64_t>(ms, 1)));
    if (ms > 0) {
        k_build_perm<<<(unsigned)ceil_div(ms, 256), 256, 0, st>>>(hot_flags.p, hot_pos.p, ms, n_hot, e->perm, e->inv_perm);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    // column offsets of the CSC in internal order (the arrays are filled on first use)
    DN_TRY(cnt_p.alloc((size_t)ms + 1));
    DN_CUDA(cudaMalloc((void**)&e->c_colptr, sizeof(int64_t) * (size_t)(ms + 1)));
    k_permute_counts<<<(unsigned)ceil_div(ms + 1, 256), 256, 0, st>>>(cnt_s.p, e->perm, ms, cnt_p.p);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    DN_TRY(scan_exclusive<int32_t>(cnt_p.p, e->c_colptr, ms + 1, st));

    trace.mark("popular columns, permutation");
    // 6b. rows of A partitioned into buckets: hot tiles, then tail column blocks
    //     narrow enough for their slice of H to stay in L2 while it is gathered
    {
        int64_t tail_cols = ms - n_hot;
        const int64_t tail_bytes = e->opt_tail_block_bytes > 0 ? e->opt_tail_block_bytes : kTailBlockBytes;
        const int64_t min_block = e->opt_tail_block_bytes > 0 ? 32 : 4096;
        int64_t block = std::max<int64_t>(min_block, (tail_bytes / (4 * (int64_t)r)) / 32 * 32);
        int64_t nb = ceil_div(std::max<int64_t>(tail_cols, 1), block);
        if (nb > kMaxTailBlocks) {
            block = ceil_div(ceil_div(tail_cols, kMaxTailBlocks), 32) * 32;
            nb = ceil_div(tail_cols, block);
        }
        if (tail_cols <= 0) nb = 0;
        if (n_hot <= 0) dense = false;
        if (dense) tile = (int)std::max<int64_t>(n_hot, 1);  // the dense block needs no tiles: one hot bucket
        BucketMap bm;
        bm.n_hot = n_hot;
        bm.tile = tile;
        bm.block = (int32_t)block;
        bm.n_hot_tiles = (int32_t)ceil_div(n_hot, tile);
        bm.n_buckets = bm.n_hot_tiles + (int32_t)nb;
        e->bm = bm;
        e->n_hot = n_hot;
        e->n_tail_blocks = (int)nb;
        DN_CUDA(cudaMalloc((void**)&e->b_vals, sizeof(float) * (size_t)std::max<int64_t>(nnz, 1)));
        DN_CUDA(cudaMalloc((void**)&e->b_col, sizeof(int32_t) * (size_t)std::max<int64_t>(nnz, 1)));
        DN_CUDA(cudaMalloc((void**)&e->tail_off, sizeof(uint32_t) * (size_t)std::max<int64_t>(n * (nb + 1), 1)));
        if (dense) {
            e->plan_x1 = block_tc_plan(n, n_hot, r);
            e->plan_x2 = block_tc_plan(n_hot, n, r);
            DN_CUDA(cudaMalloc((void**)&e->x1, sizeof(float) * e->plan_x1.x_floats));
            DN_CUDA(cudaMalloc((void**)&e->x2, sizeof(float) * e->plan_x2.x_floats));
            DN_CUDA(cudaMalloc((void**)&e->blk_ysplit,
                               sizeof(float) * std::max(e->plan_x1.ysplit_floats, e->plan_x2.ysplit_floats)));
            DN_CUDA(cudaMalloc((void**)&e->blk_partial,
                               sizeof(float) * std::max(e->plan_x1.partial_floats, e->plan_x2.partial_floats)));
            DN_CUDA(cudaMemsetAsync(e->x1, 0, sizeof(float) * e->plan_x1.x_floats, st));
        }
        trace.mark("index-only phases done");
        // slab by slab, as the values arrive: extraction with the row normalisation
        // applied, bucketing of the rows, the dense copy of the popular part
        // Row slices: every engine extracts, for each engine d, its slice's entries in
        // d's columns (normalised, column ids local to d, input order) and sends them;
        // what arrives from engine s lands at rows [slice_begin[s], slice_begin[s+1]) of
        // this shard's CSR in input order, which is then complete and bucketed below.
        DevBuf<float> canon_v;
        DevBuf<int32_t> canon_c;
        if (slice) {
            if (slabs)
                for (cudaEvent_t ev : slabs->ready)
                    if (ev) DN_CUDA(cudaStreamWaitEvent(st, ev, 0));
            slabs = nullptr;
            if (!e->opt_keep_csr) {
                DN_TRY(canon_v.alloc((size_t)std::max<int64_t>(nnz, 1)));
                DN_TRY(canon_c.alloc((size_t)std::max<int64_t>(nnz, 1)));
            }
            float* const cv = e->opt_keep_csr ? e->a_vals : canon_v.p;
            int32_t* const cc = e->opt_keep_csr ? e->a_col : canon_c.p;
            // one pair of send buffers, the destinations' parts one after the other
            DevBuf<float> sv_all;
            DevBuf<int32_t> sc_all;
            std::vector<int64_t> send_off((size_t)G + 1, 0);
            for (int d = 0; d < G; d++)
                send_off[(size_t)d + 1] = send_off[(size_t)d] + (d == e->comm_rank ? 0 : send_count[(size_t)d]);
            DN_TRY(sv_all.alloc((size_t)std::max<int64_t>(send_off[(size_t)G], 1)));
            DN_TRY(sc_all.alloc((size_t)std::max<int64_t>(send_off[(size_t)G], 1)));
            std::vector<int64_t> recv_off((size_t)G + 1, 0);
            for (int d = 0; d <= G; d++)
                DN_TRY(read_small(e, e->a_rowptr + slice_begin[(size_t)d], sizeof(int64_t), &recv_off[(size_t)d]));
            for (int d = 0; d < G; d++) {
                const bool self = d == e->comm_rank;
                // this engine's own part goes straight to its place
                float* ov = self ? cv + recv_off[(size_t)d] : nullptr;
                int32_t* oc = self ? cc + recv_off[(size_t)d] : nullptr;
                if (!self) {
                    ov = sv_all.p + send_off[(size_t)d];
                    oc = sc_all.p + send_off[(size_t)d];
                } else if (send_count[(size_t)d] != recv_off[(size_t)d + 1] - recv_off[(size_t)d]) {
                    return fail(DNPEFF_ERR_INVALID, "internal: row-slice bookkeeping out of step");
                }
                if (n_in > 0) {
                    k_extract_shard<<<(unsigned)std::min<int64_t>(n_in, (int64_t)kNumSMs * 32), 256, 0, st>>>(
                        d_vals, d_col, d_rowptr, k, 0, n_in, d_norms, og_to_new.p, map_of[(size_t)d], off_to[(size_t)d],
                        ov, oc);
                    DN_LAUNCH_CHECK();
                    DN_COUNT_LAUNCH(1);
                }
            }
            int gs = DNPEFF_OK;
            DN_NCCL(nccl_api().GroupStart());
            for (int d = 0; d < G; d++) {
                if (d == e->comm_rank) continue;
                if (send_count[(size_t)d] > 0) {
                    DN_NCCL_IN_GROUP(gs, nccl_api().Send(sv_all.p + send_off[(size_t)d], (size_t)send_count[(size_t)d],
                                                         ncclFloat, d, e->comm, st));
                    DN_NCCL_IN_GROUP(gs, nccl_api().Send(sc_all.p + send_off[(size_t)d], (size_t)send_count[(size_t)d],
                                                         ncclInt32, d, e->comm, st));
                }
                const int64_t cnt = recv_off[(size_t)d + 1] - recv_off[(size_t)d];
                if (cnt > 0) {
                    DN_NCCL_IN_GROUP(gs, nccl_api().Recv(cv + recv_off[(size_t)d], (size_t)cnt, ncclFloat, d, e->comm, st));
                    DN_NCCL_IN_GROUP(gs, nccl_api().Recv(cc + recv_off[(size_t)d], (size_t)cnt, ncclInt32, d, e->comm, st));
                }
            }
            DN_NCCL(nccl_api().GroupEnd());
            DN_TRY(gs);
            DN_CUDA(cudaStreamSynchronize(st));  // the send buffers are released here
            trace.mark("row slices exchanged");
        }
        // Row slabs: the caller's (an upload in flight), or cuts of about 256 Mi input
        // entries, which bound the temporary that holds a slab in input order.
        LoadSlabs own;
        if (!slabs) {
            const int64_t S = std::min<int64_t>(std::max<int64_t>(ceil_div(slice ? nnz : nnz_in, (int64_t)256 << 20), 1), 64);
            for (int64_t sl = 0; sl < S; sl++) {
                own.row_end.push_back(sl + 1 == S ? n : n * (sl + 1) / S);
                own.ready.push_back(nullptr);
            }
            slabs = &own;
        }
        const int n_slabs = slabs->count();
        std::vector<int64_t> slab_off((size_t)n_slabs + 1, 0);  // a_rowptr at the slab boundaries
        for (int sl = 0; sl < n_slabs && n > 0; sl++)
            DN_TRY(read_small(e, e->a_rowptr + slabs->row_end[sl], sizeof(int64_t), &slab_off[(size_t)sl + 1]));
        DevBuf<float> t_vals;
        DevBuf<int32_t> t_col;
        if (!e->opt_keep_csr && !slice && n > 0) {
            int64_t longest = 1;
            for (int sl = 0; sl < n_slabs; sl++) longest = std::max(longest, slab_off[(size_t)sl + 1] - slab_off[(size_t)sl]);
            DN_TRY(t_vals.alloc((size_t)longest));
            DN_TRY(t_col.alloc((size_t)longest));
        }
        int64_t row0 = 0;
        for (int sl = 0; sl < n_slabs && n > 0; sl++) {
            const int64_t row1 = slabs->row_end[sl];
            if (slabs->ready[sl]) DN_CUDA(cudaStreamWaitEvent(st, slabs->ready[sl], 0));
            if (row1 <= row0) continue;
            const int64_t rows = row1 - row0;
            // the slab in input order: at its place in the kept CSR, or in the temporary
            // (addressed through a_rowptr all the same: the pointers are shifted)
            float* cv = e->opt_keep_csr ? e->a_vals : (slice ? canon_v.p : shifted(t_vals.p, slab_off[(size_t)sl]));
            int32_t* cc = e->opt_keep_csr ? e->a_col : (slice ? canon_c.p : shifted(t_col.p, slab_off[(size_t)sl]));
            if (!slice) {
                k_extract_shard<<<(unsigned)std::min<int64_t>(rows, (int64_t)kNumSMs * 32), 256, 0, st>>>(
                    d_vals, d_col, d_rowptr, k, row0, row1, d_norms, og_to_new.p, map, e->a_rowptr, cv, cc);
                DN_LAUNCH_CHECK();
                DN_COUNT_LAUNCH(1);
            }
            size_t smem = sizeof(int) * 8 * (size_t)std::max(bm.n_buckets, 1);
            k_bucket_rows<<<(unsigned)std::min<int64_t>(rows, (int64_t)kNumSMs * 16), 256, smem, st>>>(
                cv, cc, e->a_rowptr, row0, row1, e->inv_perm, bm, e->b_vals, e->b_col, e->tail_off);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
            if (dense) {
                k_fill_blocks<<<(unsigned)std::min<int64_t>(ceil_div(rows, 8), (int64_t)kNumSMs * 16), 256, 0, st>>>(
                    e->b_vals, e->b_col, e->a_rowptr, e->tail_off, (int)(nb + 1), row0, row1, e->plan_x1.k_chunks,
                    e->x1);
                DN_LAUNCH_CHECK();
                DN_COUNT_LAUNCH(1);
            }
            row0 = row1;
        }
        if (t_vals.p || canon_v.p) DN_CUDA(cudaStreamSynchronize(st));  // the temporaries are released at the end of this scope
        trace.mark("extract, bucket, dense fill");
        if (dense) {
            dim3 tgrid((unsigned)e->plan_x1.m_tiles, (unsigned)e->plan_x2.m_tiles);
            k_block_transpose<<<tgrid, 256, 0, st>>>(e->x1, e->plan_x1.m_tiles, e->plan_x1.k_chunks, e->x2,
                                                    e->plan_x2.m_tiles, e->plan_x2.k_chunks);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
        }
        trace.mark("transposed dense block");
        // stored entries per tail block (decides warp-per-row or block-per-row launches)
        std::vector<int64_t> colptr_h;
        e->tail_nnz.assign((size_t)nb, 0);
        for (int64_t b = 0; b < nb; b++) {
            int64_t lo = n_hot + b * block, hi = std::min<int64_t>(ms, lo + block);
            int64_t v[2];
            DN_TRY(read_small(e, e->c_colptr + lo, sizeof(int64_t), &v[0]));
            DN_TRY(read_small(e, e->c_colptr + hi, sizeof(int64_t), &v[1]));
            e->tail_nnz[(size_t)b] = v[1] - v[0];
        }
    }

    trace.mark("tail block sizes");
    // 7. |A|^2 and sum(A) of the shard
    k_sum_sumsq<<<kRedBlocks, 256, 0, st>>>(e->b_vals, nnz, e->red_partial);
    DN_LAUNCH_CHECK();
    k_fold<<<1, 256, 0, st>>>(e->red_partial, kRedBlocks, 2, e->red_out);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(2);
    double hs[2] = {0, 0};
    DN_CUDA(cudaMemcpyAsync(hs, e->red_out, sizeof(double) * 2, cudaMemcpyDeviceToHost, st));
    DN_CUDA(cudaStreamSynchronize(st));
    e->a_sum = hs[0];
    e->a_sq = hs[1];

    e->n = n; e->m_full = m_full; e->m_kept = m_kept; e->c0 = c0; e->ms = ms; e->nnz = nnz;
    e->map = map;

    // 8. factor and work buffers, long-row lists
    DN_CUDA(cudaMalloc((void**)&e->W, sizeof(float) * (size_t)std::max<int64_t>(n * r, 1)));
    DN_CUDA(cudaMalloc((void**)&e->H, sizeof(float) * (size_t)std::max<int64_t>(ms * r, 1)));
    DN_CUDA(cudaMalloc((void**)&e->AHG, sizeof(float) * (size_t)(n * r + (int64_t)r * r)));
    DN_CUDA(cudaMalloc((void**)&e->WW, sizeof(float) * (size_t)((int64_t)r * r)));
    e->gram_scratch_floats = std::max(gram_any_scratch(n, r), gram_any_scratch(ms, r));
    DN_CUDA(cudaMalloc((void**)&e->gram_scratch, sizeof(float) * e->gram_scratch_floats));
    DN_CUDA(cudaMalloc((void**)&e->tc_scratch, sizeof(float) * 2 * (size_t)r * r));
    DN_TRY(spmm_make_plan(e->a_rowptr, 0, n, &e->plan_csr, st));
    DN_TRY(spmm_make_plan(e->c_colptr, e->n_hot, ms - e->n_hot, &e->plan_csc, st));
    e->loaded = true;
    trace.mark("norms, factor buffers, plans");
    return DNPEFF_OK;
}

// CSC fill (see kernels_prep.cuh): every entry takes the next slot of its column in a
// temporary copy, then every column is put in row order.  `mode`: 0 every entry, 1
// only the entries outside the popular columns, 2 only those inside.  The column
// offsets cover all entries in every mode.
int fill_csc(dnpeff_engine* e, int mode) {
    cudaStream_t st = e->st;
    if (e->nnz <= 0 || e->n <= 0 || e->ms <= 0) return DNPEFF_OK;
    const int n_seg_all = e->n_tail_blocks + 1;  // segment 0 = popular part, s >= 1 = tail block s-1
    const int seg_first = mode == 1 ? 1 : 0, seg_last = mode == 2 ? 1 : n_seg_all;
    const int64_t col_first = mode == 1 ? e->n_hot : 0, col_last = mode == 2 ? e->n_hot : e->ms;
    if (seg_first >= seg_last || col_first >= col_last) return DNPEFF_OK;
    RowSegments segs = {e->tail_off, e->n_tail_blocks + 1};
    const size_t bitmap_bytes = 2 * (size_t)ceil_div(e->n, 32) * sizeof(uint32_t);
    PoolScope pool_scope(st);
    PhaseTrace trace(st);
    // the temporary copy covers the CSC entries of the columns being filled:
    // offsets [t_base, t_end) of c_colptr
    int64_t t_base = 0, t_end = e->nnz;
    if (mode != 0) {
        int64_t split = 0;
        DN_TRY(read_small(e, e->c_colptr + e->n_hot, sizeof(int64_t), &split));
        if (mode == 1) t_base = split; else t_end = split;
    }
    if (t_base < e->c_base) return fail(DNPEFF_ERR_INVALID, "internal: CSC arrays do not cover the requested columns");
    DevBuf<float> tvals_buf;
    DevBuf<int32_t> trow_buf, cursor, long_cols;
    DevBuf<int> err, n_long;
    DN_TRY(tvals_buf.alloc((size_t)std::max<int64_t>(t_end - t_base, 1)));
    DN_TRY(trow_buf.alloc((size_t)std::max<int64_t>(t_end - t_base, 1)));
    float* const tvals = shifted(tvals_buf.p, t_base);
    int32_t* const trow = shifted(trow_buf.p, t_base);
    float* const cvals = csc_vals(e);
    int32_t* const crows = csc_rows(e);
    DN_TRY(cursor.alloc_zero((size_t)e->ms, st));
    DN_TRY(long_cols.alloc((size_t)(col_last - col_first)));
    DN_TRY(err.alloc_zero(1, st));
    DN_TRY(n_long.alloc_zero(1, st));
    trace.mark("  csc: scratch");
    for (int seg = seg_first; seg < seg_last; seg++) {
        k_csc_scatter<<<(unsigned)ceil_div(e->n, 8), 256, 0, st>>>(e->a_rowptr, e->b_col, e->b_vals, e->n, segs, seg,
                                                                  e->c_colptr, cursor.p, tvals, trow);
        DN_COUNT_LAUNCH(1);
    }
    DN_LAUNCH_CHECK();
    trace.mark("  csc: slots");
    k_csc_list_long<<<(unsigned)ceil_div(col_last - col_first, 256), 256, 0, st>>>(e->c_colptr, col_first, col_last,
                                                                                  long_cols.p, n_long.p);
    DN_LAUNCH_CHECK();
    int h_long = 0;
    DN_CUDA(cudaMemcpyAsync(&h_long, n_long.p, sizeof(int), cudaMemcpyDeviceToHost, st));
    DN_CUDA(cudaStreamSynchronize(st));
    {
        int64_t blocks = std::min<int64_t>(ceil_div(col_last - col_first, 8), (int64_t)kNumSMs * 32);
        k_csc_order_short<<<(unsigned)blocks, 256, 0, st>>>(e->c_colptr, col_first, col_last, tvals, trow,
                                                           cvals, crows, err.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(2);
    }
    if (h_long > 0) {
        if (bitmap_bytes > 200 * 1024)
            return fail(DNPEFF_ERR_UNSUPPORTED, "columns longer than 512 entries need n_rows <= 819200");
        DN_CUDA(cudaFuncSetAttribute(k_csc_order_long, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bitmap_bytes));
        int blocks = std::min(h_long, kNumSMs * 8);
        k_csc_order_long<<<blocks, 256, bitmap_bytes, st>>>(e->c_colptr, long_cols.p, h_long, e->n, tvals, trow,
                                                           cvals, crows, err.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    trace.mark("  csc: row order");
    int herr = 0;
    DN_TRY(read_err_flag(err.p, st, &herr));
    if (herr) return data_error(herr);
    return DNPEFF_OK;
}

// The CSC the H update needs.  With the popular block kept dense the popular
// columns are never read from the CSC, so they are filled only on demand
// (`full`: the export call).
int build_csc(dnpeff_engine* e, bool full = false) {
    PhaseTrace trace(e->st);
    if (full && e->csc_ready && e->c_base > 0) {
        // the arrays were sized for the unpopular columns only: start over at full size
        DN_CUDA(cudaStreamSynchronize(e->st));
        dev_free(e->c_vals);
        dev_free(e->c_row);
        e->c_base = 0;
        e->csc_ready = e->csc_hot_ready = false;
    }
    if (!e->csc_ready) {
        trace.mark("(before CSC build)");
        const bool tail_only = e->x2 != nullptr && !full;
        int64_t base = 0;
        if (tail_only) DN_TRY(read_small(e, e->c_colptr + e->n_hot, sizeof(int64_t), &base));
        DN_CUDA(cudaMalloc((void**)&e->c_vals, sizeof(float) * (size_t)std::max<int64_t>(e->nnz - base, 1)));
        DN_CUDA(cudaMalloc((void**)&e->c_row, sizeof(int32_t) * (size_t)std::max<int64_t>(e->nnz - base, 1)));
        e->c_base = base;
        trace.mark("  csc: arrays allocated");
        DN_TRY(fill_csc(e, tail_only ? 1 : 0));
        e->csc_ready = true;
        e->csc_hot_ready = !tail_only;
        trace.mark("CSC build");
    }
    if (full && !e->csc_hot_ready) {
        DN_TRY(fill_csc(e, 2));
        e->csc_hot_ready = true;
    }
    return DNPEFF_OK;
}

int allreduce_f32(dnpeff_engine* e, float* buf, size_t count) {
    if (e->comm_size <= 1) return DNPEFF_OK;
    ScopedTimer t(e, 4);
    DN_NCCL(nccl_api().AllReduce(buf, buf, count, ncclFloat, ncclSum, e->comm, e->st));
    return DNPEFF_OK;
}

int device_dot(dnpeff_engine* e, const float* a, const float* b, int64_t count, double* d_out) {
    k_dot<<<kRedBlocks, 256, 0, e->st>>>(a, b, count, e->red_partial);
    DN_LAUNCH_CHECK();
    k_fold<<<1, 256, 0, e->st>>>(e->red_partial, kRedBlocks, 1, d_out);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(2);
    return DNPEFF_OK;
}

// A*H^T: the popular columns through the tiled kernel (H tiles staged in shared
// memory), then one launch per tail column block, each adding to AH, so that the
// slice of H being gathered stays L2-resident.
int spmm_ah(dnpeff_engine* e, float* AH) {
    const int r = e->p.rank;
    if (!spmm_fast_rank(r))
        return spmm_dispatch(e->b_vals, e->b_col, e->a_rowptr, e->n, e->H, r, AH, e->plan_csr, e->st);
    if (e->n <= 0) return DNPEFF_OK;
    int accumulate = 0;
    const int stride = e->n_tail_blocks + 1;
    if (e->x1) {
        // popular block on the tensor cores: AH = A_pop * H_pop (H's first n_hot rows)
        DN_TRY(block_tc_launch(e->x1, e->plan_x1, e->H, e->n, e->n_hot, r, AH, e->blk_ysplit, e->blk_partial,
                               e->d_err, e->st, e->opt_wait_limit));
        accumulate = 1;
    } else if (e->n_hot > 0) {
        SpmmCall c;
        c.kind = kSpmmTiled;
        c.vals = e->b_vals; c.ind = e->b_col;
        c.seg = {e->a_rowptr, nullptr, 0, 0};
        c.rows = e->n; c.D = e->H; c.r = r; c.out = AH;
        c.row_len = e->tail_off; c.row_len_stride = stride;
        c.d_rows = e->n_hot;
        c.work_counter = e->work_counter; c.err = e->d_err;
        DN_TRY(spmm_call(c, e->st));
        accumulate = 1;
    }
    for (int b = 0; b < e->n_tail_blocks; b++) {
        SpmmCall c;
        c.kind = (e->tail_nnz[(size_t)b] / e->n > 512) ? kSpmmBucketBlock : kSpmmBucketWarp;
        c.vals = e->b_vals; c.ind = e->b_col;
        c.seg = {e->a_rowptr, e->tail_off, stride, b};
        c.rows = e->n; c.D = e->H; c.r = r; c.out = AH;
        c.accumulate = accumulate;
        DN_TRY(spmm_call(c, e->st));
        accumulate = 1;
    }
    if (!accumulate) DN_CUDA(cudaMemsetAsync(AH, 0, sizeof(float) * (size_t)(e->n * r), e->st));
    return DNPEFF_OK;
}

// A^T*W: the popular columns (long CSC rows) through the tiled kernel with W
// staged tile by tile, the rest by warp/block gathers from the L2-resident W.
int spmm_wa(dnpeff_engine* e) {
    const int r = e->p.rank;
    if (!spmm_fast_rank(r))
        return spmm_dispatch(csc_vals(e), csc_rows(e), e->c_colptr, e->ms, e->W, r, e->WA, e->plan_csc, e->st);
    if (e->x2) {
        // popular columns on the tensor cores: WA[0, n_hot) = A_pop^T * W
        DN_TRY(block_tc_launch(e->x2, e->plan_x2, e->W, e->n_hot, e->n, r, e->WA, e->blk_ysplit, e->blk_partial,
                               e->d_err, e->st, e->opt_wait_limit));
    } else if (e->n_hot > 0) {
        SpmmCall c;
        c.kind = kSpmmTiled;
        c.vals = csc_vals(e); c.ind = csc_rows(e);
        c.seg = {e->c_colptr, nullptr, 0, 0};
        c.rows = e->n_hot; c.D = e->W; c.r = r; c.out = e->WA;
        c.d_rows = e->n;
        c.work_counter = e->work_counter; c.err = e->d_err;
        DN_TRY(spmm_call(c, e->st));
    }
    if (e->ms > e->n_hot) {
        SpmmCall c;
        c.kind = kSpmmRows;
        c.vals = csc_vals(e); c.ind = csc_rows(e);
        c.seg = {e->c_colptr, nullptr, 0, 0};
        c.row_first = e->n_hot; c.rows = e->ms - e->n_hot;
        c.D = e->W; c.r = r; c.out = e->WA; c.plan = &e->plan_csc;
        DN_TRY(spmm_call(c, e->st));
    }
    return DNPEFF_OK;
}

int compute_ah_hh(dnpeff_engine* e) {
    const int r = e->p.rank;
    float* AH = e->AHG;
    float* HH = e->AHG + e->n * r;
    {
        ScopedTimer t(e, 0);
        DN_TRY(spmm_ah(e, AH));
    }
    {
        ScopedTimer t(e, 2);
        DN_TRY(gram_any(e->H, e->ms, r, HH, e->gram_scratch, e->d_err, e->st, e->opt_wait_limit));
    }
    DN_TRY(allreduce_f32(e, e->AHG, (size_t)(e->n * r + (int64_t)r * r)));
    return DNPEFF_OK;
}

int step_w(dnpeff_engine* e) {
    const int r = e->p.rank;
    DN_TRY(compute_ah_hh(e));
    // Wide ranks write the updated W beside the old one, into the engine's spare n x r
    // buffer (allocated once), and the two buffers change places.
    if (tensor_cores_enabled() && mu_update_ws_wide_ok(r) && e->n > 0 && !e->w_spare)
        DN_CUDA(cudaMalloc((void**)&e->w_spare, sizeof(float) * (size_t)(e->n * r)));
    ScopedTimer t(e, 3);
    bool moved = false;
    DN_TRY(mu_update_any(e->W, e->AHG, e->AHG + e->n * r, e->n, r, e->p.eps, e->tc_scratch, e->d_err, e->st, false,
                         e->w_spare, e->opt_wait_limit, &moved));
    if (moved) std::swap(e->W, e->w_spare);
    return DNPEFF_OK;
}

int step_h(dnpeff_engine* e) {
    const int r = e->p.rank;
    DN_TRY(build_csc(e));
    if (!e->WA) DN_CUDA(cudaMalloc((void**)&e->WA, sizeof(float) * (size_t)std::max<int64_t>(e->ms * r, 1)));
    {
        ScopedTimer t(e, 1);
        DN_TRY(spmm_wa(e));
    }
    {
        ScopedTimer t(e, 2);
        DN_TRY(gram_any(e->W, e->n, r, e->WW, e->gram_scratch, e->d_err, e->st, e->opt_wait_limit));
    }
    ScopedTimer t(e, 3);
    // wide ranks: the new H is written over W^T*A (not used again), and the buffers change places
    bool moved = false;
    DN_TRY(mu_update_any(e->H, e->WA, e->WW, e->ms, r, e->p.eps, e->tc_scratch, e->d_err, e->st, true, nullptr,
                         e->opt_wait_limit, &moved));
    if (moved) std::swap(e->H, e->WA);
    return DNPEFF_OK;
}

int global_a_sq(dnpeff_engine* e, double* out) {
    if (e->a_sq_global < 0.0) {
        if (e->comm_size > 1) {
            DN_CUDA(cudaMemcpyAsync(e->red_out + 3, &e->a_sq, sizeof(double), cudaMemcpyHostToDevice, e->st));
            DN_NCCL(nccl_api().AllReduce(e->red_out + 3, e->red_out + 3, 1, ncclDouble, ncclSum, e->comm, e->st));
            double v = 0;
            DN_CUDA(cudaMemcpyAsync(&v, e->red_out + 3, sizeof(double), cudaMemcpyDeviceToHost, e->st));
            DN_CUDA(cudaStreamSynchronize(e->st));
            e->a_sq_global = v;
        } else {
            e->a_sq_global = e->a_sq;
        }
    }
    *out = e->a_sq_global;
    return DNPEFF_OK;
}

// sqrt(|A|^2 + <W^T W, H H^T> - 2 <A H^T, W>).  <H,(W^T W)H> = <W^T W, H H^T> and
// <W^T A, H> = <A H^T, W> are the reference's two Frobenius products
// (…device_contexts1.h:337-354) written on the small side; after the allreduce
// both are global, so every engine returns the same number.  The three terms
// are accumulated in double.
int loss_from_current(dnpeff_engine* e, bool recompute_ah, double* out) {
    const int r = e->p.rank;
    ScopedTimer t(e, 5);
    if (recompute_ah) DN_TRY(compute_ah_hh(e));
    DN_TRY(gram_any(e->W, e->n, r, e->WW, e->gram_scratch, e->d_err, e->st, e->opt_wait_limit));
    DN_TRY(device_dot(e, e->AHG, e->W, e->n * r, e->red_out + 0));
    DN_TRY(device_dot(e, e->WW, e->AHG + e->n * r, (int64_t)r * r, e->red_out + 1));
    double h[2];
    DN_CUDA(cudaMemcpyAsync(h, e->red_out, sizeof(double) * 2, cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    DN_TRY(check_kernel_status(e));
    double a2 = 0;
    DN_TRY(global_a_sq(e, &a2));
    double sq = a2 + h[1] - 2.0 * h[0];
    *out = sq > 0.0 ? sqrt(sq) : 0.0;
    return DNPEFF_OK;
}

int init_generated(dnpeff_engine* e, bool do_w, bool do_h) {
    const int r = e->p.rank;
    float scale = e->p.init_scale > 0.f ? e->p.init_scale : 1.0f;
    if (do_w && e->n > 0) {
        k_init_uniform<<<kNumSMs * 8, 256, 0, e->st>>>(e->W, e->w_row_offset * r, e->n * r,
                                                       stream_key(e->p.seed, 0), scale);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    if (do_h && e->ms > 0) {
        k_init_uniform_cols<<<kNumSMs * 8, 256, 0, e->st>>>(e->H, e->ms, r, e->map, e->perm,
                                                          stream_key(e->p.seed, 1), scale);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    return DNPEFF_OK;
}

// Reads the device error word the bounded waits write (synchronises the stream).
int check_kernel_status(dnpeff_engine* e) {
    int h = 0;
    DN_CUDA(cudaMemcpyAsync(&h, e->d_err, sizeof(int), cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    if (h) {
        // reported once: the word is cleared so that the engine can be used again
        // (after new factors are set; what the interrupted kernels wrote is invalid)
        cudaMemsetAsync(e->d_err, 0, sizeof(int), e->st);
        cudaStreamSynchronize(e->st);
    }
    if (h & kErrTiledTimeout)
        return fail(DNPEFF_ERR_CUDA, "a bulk-copy wait in the tiled SpMM kernel ran out; results are invalid");
    if (h & kErrTcTimeout)
        return fail(DNPEFF_ERR_CUDA, "a wait in a tensor-core kernel ran out; results are invalid");
    return DNPEFF_OK;
}

int check_ready(dnpeff_engine* e, bool need_factors) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (!e->loaded) return fail(DNPEFF_ERR_INVALID, "no matrix loaded: call dnpeff_set_csr first");
    if (need_factors && !e->have_factors)
        return fail(DNPEFF_ERR_INVALID, "factors not initialised: call dnpeff_init_factors first");
    return DNPEFF_OK;
}

// Scratch for the single-kernel entry points, one grow-only buffer per device.
struct OpWorkspace {
    std::mutex mu;
    float* scratch[64] = {nullptr};
    size_t floats[64] = {0};
    int* err[64] = {nullptr};
};
OpWorkspace& op_ws() {
    static OpWorkspace w;
    return w;
}

int op_scratch(size_t floats, float** out) {
    int dev = 0;
    DN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(DNPEFF_ERR_UNSUPPORTED, "device ordinal %d", dev);
    OpWorkspace& w = op_ws();
    std::lock_guard<std::mutex> lk(w.mu);
    if (w.floats[dev] < floats) {
        if (w.scratch[dev]) {
            DN_CUDA(cudaDeviceSynchronize());
            cudaFree(w.scratch[dev]);
            w.scratch[dev] = nullptr;
            w.floats[dev] = 0;
        }
        DN_CUDA(cudaMalloc((void**)&w.scratch[dev], sizeof(float) * floats));
        w.floats[dev] = floats;
    }
    *out = w.scratch[dev];
    return DNPEFF_OK;
}

// Error word of the single-kernel entry points (one per device), read after the call.
int op_err_word(int** out) {
    int dev = 0;
    DN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(DNPEFF_ERR_UNSUPPORTED, "device ordinal %d", dev);
    OpWorkspace& w = op_ws();
    std::lock_guard<std::mutex> lk(w.mu);
    if (!w.err[dev]) {
        DN_CUDA(cudaMalloc((void**)&w.err[dev], sizeof(int)));
        DN_CUDA(cudaMemset(w.err[dev], 0, sizeof(int)));
    }
    *out = w.err[dev];
    return DNPEFF_OK;
}

int op_check_err(int* d_err, cudaStream_t st) {
    int h = 0;
    DN_CUDA(cudaMemcpyAsync(&h, d_err, sizeof(int), cudaMemcpyDeviceToHost, st));
    DN_CUDA(cudaStreamSynchronize(st));
    if (h) {
        cudaMemsetAsync(d_err, 0, sizeof(int), st);
        return fail(DNPEFF_ERR_CUDA, "a bounded wait inside a kernel ran out (status %d); results are invalid", h);
    }
    return DNPEFF_OK;
}

}  // namespace

// ===========================================================================
extern "C" {

const char* dnpeff_last_error(void) { return err_buf(); }
int dnpeff_abi_version(void) { return DNPEFF_ABI_VERSION; }

int dnpeff_device_count(int* count) {
    if (!count) return fail(DNPEFF_ERR_INVALID, "null argument");
    *count = 0;
    DN_CUDA(cudaGetDeviceCount(count));
    return DNPEFF_OK;
}

int dnpeff_create(const dnpeff_params* params, int device, void* stream, dnpeff_engine** out) {
    if (!params || !out) return fail(DNPEFF_ERR_INVALID, "null argument");
    if (params->rank <= 0) return fail(DNPEFF_ERR_INVALID, "rank must be positive");
    if (params->n_shards <= 0 || params->shard_index < 0 || params->shard_index >= params->n_shards)
        return fail(DNPEFF_ERR_INVALID, "shard_index/n_shards out of range");
    if (params->shard_mode != DNPEFF_SHARD_CONTIGUOUS && params->shard_mode != DNPEFF_SHARD_CYCLIC)
        return fail(DNPEFF_ERR_INVALID, "unknown shard_mode %d", (int)params->shard_mode);
    int ndev = 0;
    DN_CUDA(cudaGetDeviceCount(&ndev));
    if (device < 0 || device >= ndev)
        return fail(DNPEFF_ERR_CUDA, "device %d not available (%d visible)", device, ndev);
    DN_CUDA(cudaSetDevice(device));
    dnpeff_engine* e = new dnpeff_engine();
    e->p = *params;
    e->device = device;
    if (stream) {
        e->st = (cudaStream_t)stream;
    } else {
        cudaError_t ce = cudaStreamCreateWithFlags(&e->st, cudaStreamNonBlocking);
        if (ce != cudaSuccess) {
            delete e;
            return fail(DNPEFF_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(ce));
        }
        e->own_stream = true;
    }
    if (cudaMalloc((void**)&e->red_partial, sizeof(double) * 2 * kRedBlocks) != cudaSuccess ||
        cudaMalloc((void**)&e->red_out, sizeof(double) * 4) != cudaSuccess ||
        cudaMalloc((void**)&e->work_counter, sizeof(int)) != cudaSuccess ||
        cudaMalloc((void**)&e->d_err, sizeof(int)) != cudaSuccess ||
        cudaMemset(e->d_err, 0, sizeof(int)) != cudaSuccess) {
        dnpeff_destroy(e);
        return fail(DNPEFF_ERR_CUDA, "cudaMalloc of reduction buffers failed");
    }
    if (cudaHostAlloc(&e->h_pinned, 256, cudaHostAllocDefault) != cudaSuccess) {
        e->h_pinned = nullptr;  // read_small falls back to pageable copies
        cudaGetLastError();
    }
    e->launches0 = launch_counter();
    *out = e;
    return DNPEFF_OK;
}

int dnpeff_destroy(dnpeff_engine* e) {
    if (!e) return DNPEFF_OK;
    DeviceGuard g(e->device);
    cudaStreamSynchronize(e->st);
    if (e->comm) nccl_api().CommDestroy(e->comm);
    free_matrix(e);
    dev_free(e->red_partial);
    dev_free(e->red_out);
    if (e->h_pinned) cudaFreeHost(e->h_pinned);
    e->h_pinned = nullptr;
    dev_free(e->work_counter);
    dev_free(e->d_err);
    for (auto& r : e->regions) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
    for (auto ev : e->ev_pool) cudaEventDestroy(ev);
    if (e->own_stream) cudaStreamDestroy(e->st);
    delete e;
    return DNPEFF_OK;
}

int dnpeff_set_option(dnpeff_engine* e, const char* name, int64_t value) {
    if (!e || !name) return fail(DNPEFF_ERR_INVALID, "null argument");
    if (value < 0) return fail(DNPEFF_ERR_INVALID, "option values are non-negative");
    if (!strcmp(name, "loader_slabs")) {
        if (value > 8) return fail(DNPEFF_ERR_INVALID, "loader_slabs: at most 8");
        e->opt_loader_slabs = (int)value;
    } else if (!strcmp(name, "tail_block_bytes")) {
        e->opt_tail_block_bytes = value;
    } else if (!strcmp(name, "popular_divisor")) {
        if (value == 1 || value > INT32_MAX) return fail(DNPEFF_ERR_INVALID, "popular_divisor: 0 or >= 2");
        e->opt_popular_divisor = (int)value;
    } else if (!strcmp(name, "keep_canonical_csr")) {
        e->opt_keep_csr = value != 0;
    } else if (!strcmp(name, "wait_limit")) {
        e->opt_wait_limit = value == 0 || value > kTiledSpinLimit ? kTiledSpinLimit : (uint32_t)value;
    } else {
        return fail(DNPEFF_ERR_INVALID, "unknown option '%s'", name);
    }
    return DNPEFF_OK;
}

int dnpeff_set_csr_device(dnpeff_engine* e, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                          const int64_t* d_rowptr, const float* d_vals, const int32_t* d_colind,
                          const float* d_norms, int32_t min_values_per_parameter) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    DeviceGuard g(e->device);
    int s = load_device(e, n_rows, n_cols_full, k_per_row, d_rowptr, d_vals, d_colind, d_norms,
                        min_values_per_parameter);
    if (s != DNPEFF_OK) free_matrix(e);
    return s;
}

namespace {
int set_csr_host(dnpeff_engine* e, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                 const int64_t* rowptr, const float* vals, const int32_t* colind, const float* norms,
                 int32_t min_values_per_parameter, const int32_t* retained, int64_t n_retained,
                 int64_t n_rows_total = -1, int64_t row_begin = 0);
}

int dnpeff_set_csr(dnpeff_engine* e, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                   const int64_t* rowptr, const float* vals, const int32_t* colind,
                   const float* norms, int32_t min_values_per_parameter) {
    return set_csr_host(e, n_rows, n_cols_full, k_per_row, rowptr, vals, colind, norms,
                        min_values_per_parameter, nullptr, 0);
}

int dnpeff_row_slice(int64_t n_rows_total, int32_t n_engines, int32_t index, int64_t* row_begin, int64_t* n_rows) {
    if (n_rows_total < 0 || n_engines <= 0 || index < 0 || index >= n_engines || !row_begin || !n_rows)
        return fail(DNPEFF_ERR_INVALID, "bad argument");
    row_slice(n_rows_total, n_engines, index, row_begin, n_rows);
    return DNPEFF_OK;
}

int dnpeff_set_csr_rows(dnpeff_engine* e, int64_t n_rows_total, int64_t n_cols_full, int64_t k_per_row,
                        int64_t row_begin, int64_t n_rows, const int64_t* rowptr, const float* vals,
                        const int32_t* colind, const float* norms, int32_t min_values_per_parameter) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (n_rows_total < 0 || n_rows < 0 || row_begin < 0 || row_begin + n_rows > n_rows_total)
        return fail(DNPEFF_ERR_INVALID, "row slice outside the matrix");
    if (e->p.n_shards == 1) {
        if (row_begin != 0 || n_rows != n_rows_total)
            return fail(DNPEFF_ERR_INVALID, "a single engine takes the whole matrix");
        return set_csr_host(e, n_rows, n_cols_full, k_per_row, rowptr, vals, colind, norms, min_values_per_parameter,
                            nullptr, 0);
    }
    if (e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init first");
    return set_csr_host(e, n_rows, n_cols_full, k_per_row, rowptr, vals, colind, norms, min_values_per_parameter,
                        nullptr, 0, n_rows_total, row_begin);
}

int dnpeff_set_csr_rows_device(dnpeff_engine* e, int64_t n_rows_total, int64_t n_cols_full, int64_t k_per_row,
                               int64_t row_begin, int64_t n_rows, const int64_t* d_rowptr, const float* d_vals,
                               const int32_t* d_colind, const float* d_norms, int32_t min_values_per_parameter) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (n_rows_total < 0 || n_rows < 0 || row_begin < 0 || row_begin + n_rows > n_rows_total)
        return fail(DNPEFF_ERR_INVALID, "row slice outside the matrix");
    DeviceGuard g(e->device);
    int s;
    if (e->p.n_shards == 1) {
        if (row_begin != 0 || n_rows != n_rows_total)
            return fail(DNPEFF_ERR_INVALID, "a single engine takes the whole matrix");
        s = load_device(e, n_rows, n_cols_full, k_per_row, d_rowptr, d_vals, d_colind, d_norms, min_values_per_parameter);
    } else {
        if (e->comm_size != e->p.n_shards)
            return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init first");
        RowSlice slice = {n_rows, row_begin};
        s = load_device(e, n_rows_total, n_cols_full, k_per_row, d_rowptr, d_vals, d_colind, d_norms,
                        min_values_per_parameter, nullptr, 0, nullptr, &slice);
    }
    if (s != DNPEFF_OK) free_matrix(e);
    return s;
}

int dnpeff_get_shard(dnpeff_engine* e, int32_t* shard_index, int32_t* n_shards, int32_t* device) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (shard_index) *shard_index = e->p.shard_index;
    if (n_shards) *n_shards = e->p.n_shards;
    if (device) *device = e->device;
    return DNPEFF_OK;
}

int dnpeff_comm_agree(dnpeff_engine* e, int32_t ok, int32_t* all_ok) {
    if (!e || !all_ok) return fail(DNPEFF_ERR_INVALID, "null argument");
    *all_ok = ok ? 1 : 0;
    if (e->p.n_shards == 1) return DNPEFF_OK;
    if (e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init first");
    DeviceGuard g(e->device);
    DevBuf<int32_t> flag;
    DN_TRY(flag.alloc(1));
    int32_t h = ok ? 1 : 0;
    DN_CUDA(cudaMemcpyAsync(flag.p, &h, sizeof(int32_t), cudaMemcpyHostToDevice, e->st));
    DN_NCCL(nccl_api().AllReduce(flag.p, flag.p, 1, ncclInt32, ncclMin, e->comm, e->st));
    DN_CUDA(cudaMemcpyAsync(&h, flag.p, sizeof(int32_t), cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    *all_ok = h;
    return DNPEFF_OK;
}

int dnpeff_set_csr_retain(dnpeff_engine* e, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                          const int64_t* rowptr, const float* vals, const int32_t* colind,
                          const float* norms, const int32_t* retained_cols, int64_t n_retained) {
    if (!retained_cols && n_retained > 0) return fail(DNPEFF_ERR_INVALID, "null retained_cols");
    static const int32_t none = 0;
    return set_csr_host(e, n_rows, n_cols_full, k_per_row, rowptr, vals, colind, norms, 1,
                        retained_cols ? retained_cols : &none, n_retained);
}

namespace {
// n_rows_total >= 0: the arrays hold rows [row_begin, row_begin + n_rows) of a matrix of
// n_rows_total rows and every engine of the job makes this call on its own slice.
int set_csr_host(dnpeff_engine* e, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                 const int64_t* rowptr, const float* vals, const int32_t* colind, const float* norms,
                 int32_t min_values_per_parameter, const int32_t* retained, int64_t n_retained,
                 int64_t n_rows_total, int64_t row_begin) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (n_rows < 0) return fail(DNPEFF_ERR_INVALID, "negative shape");
    DeviceGuard g(e->device);
    int64_t nnz = rowptr ? (n_rows > 0 ? rowptr[n_rows] : 0) : n_rows * k_per_row;
    if (nnz < 0) return fail(DNPEFF_ERR_DATA, "negative nnz");
    if (nnz > 0 && (!vals || !colind)) return fail(DNPEFF_ERR_INVALID, "null vals/colind");
    free_matrix(e);
    PoolScope pool_scope(e->st);
    DevBuf<float> dv, dn;
    DevBuf<int32_t> dc;
    DevBuf<int64_t> dr;
    DN_TRY(dv.alloc((size_t)nnz));
    DN_TRY(dc.alloc((size_t)nnz));
    // The column ids go first, on the engine's stream; the values follow on a second
    // stream in slabs of rows, so that counting, pruning, row offsets and the column
    // permutation overlap their upload and every slab is processed as it lands.
    cudaStream_t up = nullptr;
    LoadSlabs slabs;
    struct UploadGuard {
        cudaStream_t& s;
        LoadSlabs& sl;
        ~UploadGuard() {
            if (s) { cudaStreamSynchronize(s); cudaStreamDestroy(s); }
            for (cudaEvent_t ev : sl.ready) cudaEventDestroy(ev);
        }
    } upload_guard{up, slabs};
    if (nnz > 0) {
        DN_CUDA(cudaMemcpyAsync(dc.p, colind, sizeof(int32_t) * (size_t)nnz, cudaMemcpyHostToDevice, e->st));
        DN_CUDA(cudaStreamCreateWithFlags(&up, cudaStreamNonBlocking));
        // the copy engine takes the transfers in issue order: ids first
        cudaEvent_t ids_issued = nullptr;
        DN_CUDA(cudaEventCreateWithFlags(&ids_issued, cudaEventDisableTiming));
        DN_CUDA(cudaEventRecord(ids_issued, e->st));
        DN_CUDA(cudaStreamWaitEvent(up, ids_issued, 0));
        cudaEventDestroy(ids_issued);
        int n_slabs = nnz >= ((int64_t)64 << 20) ? 4 : 1;
        if (e->opt_loader_slabs > 0) n_slabs = std::min(e->opt_loader_slabs, 8);
        int64_t off0 = 0;
        for (int i = 0; i < n_slabs; i++) {
            const int64_t row1 = i + 1 == n_slabs ? n_rows : n_rows * (i + 1) / n_slabs;
            const int64_t off1 = rowptr ? rowptr[row1] : row1 * k_per_row;
            if (off1 > off0)
                DN_CUDA(cudaMemcpyAsync(dv.p + off0, vals + off0, sizeof(float) * (size_t)(off1 - off0),
                                        cudaMemcpyHostToDevice, up));
            cudaEvent_t ev = nullptr;
            DN_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            slabs.row_end.push_back(row1);
            slabs.ready.push_back(ev);
            DN_CUDA(cudaEventRecord(ev, up));
            off0 = off1;
        }
    }
    if (rowptr) {
        DN_TRY(dr.alloc((size_t)n_rows + 1));
        DN_CUDA(cudaMemcpyAsync(dr.p, rowptr, sizeof(int64_t) * (size_t)(n_rows + 1), cudaMemcpyHostToDevice, e->st));
    }
    if (norms) {
        DN_TRY(dn.alloc((size_t)n_rows));
        if (n_rows > 0)
            DN_CUDA(cudaMemcpyAsync(dn.p, norms, sizeof(float) * (size_t)n_rows, cudaMemcpyHostToDevice, e->st));
    }
    DevBuf<int32_t> dret;
    if (retained) {
        DN_TRY(dret.alloc((size_t)std::max<int64_t>(n_retained, 1)));
        if (n_retained > 0)
            DN_CUDA(cudaMemcpyAsync(dret.p, retained, sizeof(int32_t) * (size_t)n_retained, cudaMemcpyHostToDevice, e->st));
    }
    RowSlice slice = {n_rows, row_begin};
    const bool sliced = n_rows_total >= 0;
    int s = load_device(e, sliced ? n_rows_total : n_rows, n_cols_full, k_per_row, rowptr ? dr.p : nullptr, dv.p, dc.p,
                        norms ? dn.p : nullptr, min_values_per_parameter, retained ? dret.p : nullptr, n_retained,
                        slabs.count() > 0 ? &slabs : nullptr, sliced ? &slice : nullptr);
    if (s != DNPEFF_OK) free_matrix(e);
    cudaStreamSynchronize(e->st);
    return s;
}
}  // namespace

int dnpeff_get_shape(dnpeff_engine* e, int64_t* n_rows, int64_t* n_cols_kept, int64_t* col_start,
                     int64_t* n_cols_shard, int64_t* nnz_shard) {
    DN_TRY(check_ready(e, false));
    if (n_rows) *n_rows = e->n;
    if (n_cols_kept) *n_cols_kept = e->m_kept;
    if (col_start) *col_start = e->c0;
    if (n_cols_shard) *n_cols_shard = e->ms;
    if (nnz_shard) *nnz_shard = e->nnz;
    return DNPEFF_OK;
}

int dnpeff_get_layout(dnpeff_engine* e, int64_t* n_hot_cols, int64_t* hot_nnz, int32_t* n_tail_blocks,
                      int32_t* tile_rows) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    int64_t v = 0;
    DN_CUDA(cudaMemcpyAsync(&v, e->c_colptr + e->n_hot, sizeof(int64_t), cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    if (n_hot_cols) *n_hot_cols = e->n_hot;
    if (hot_nnz) *hot_nnz = v;
    if (n_tail_blocks) *n_tail_blocks = e->n_tail_blocks;
    if (tile_rows) *tile_rows = e->x1 ? 0 : e->bm.tile;
    return DNPEFF_OK;
}

int dnpeff_get_new_to_og(dnpeff_engine* e, int32_t* out) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    if (e->m_kept > 0) {
        DN_CUDA(cudaMemcpyAsync(out, e->new_to_og, sizeof(int32_t) * (size_t)e->m_kept, cudaMemcpyDeviceToHost, e->st));
        DN_CUDA(cudaStreamSynchronize(e->st));
    }
    return DNPEFF_OK;
}

int dnpeff_get_shard_columns(dnpeff_engine* e, int32_t* kept_ids, int32_t* original_ids) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    if (e->ms <= 0) return DNPEFF_OK;
    DevBuf<int32_t> a, b;
    DN_TRY(a.alloc((size_t)e->ms));
    DN_TRY(b.alloc((size_t)e->ms));
    k_shard_columns<<<(unsigned)ceil_div(e->ms, 256), 256, 0, e->st>>>(e->new_to_og, e->map, a.p, b.p);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    if (kept_ids) DN_CUDA(cudaMemcpyAsync(kept_ids, a.p, sizeof(int32_t) * (size_t)e->ms, cudaMemcpyDeviceToHost, e->st));
    if (original_ids) DN_CUDA(cudaMemcpyAsync(original_ids, b.p, sizeof(int32_t) * (size_t)e->ms, cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    return DNPEFF_OK;
}

int dnpeff_export_shard_csr(dnpeff_engine* e, int64_t* rowptr, int32_t* colind, float* vals) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    if ((colind || vals) && e->nnz > 0 && !e->a_vals)
        return fail(DNPEFF_ERR_INVALID,
                    "the CSR in input order was not kept: set option keep_canonical_csr to 1 before loading");
    if (rowptr) DN_CUDA(cudaMemcpyAsync(rowptr, e->a_rowptr, sizeof(int64_t) * (size_t)(e->n + 1), cudaMemcpyDeviceToHost, e->st));
    if (colind && e->nnz > 0) DN_CUDA(cudaMemcpyAsync(colind, e->a_col, sizeof(int32_t) * (size_t)e->nnz, cudaMemcpyDeviceToHost, e->st));
    if (vals && e->nnz > 0) DN_CUDA(cudaMemcpyAsync(vals, e->a_vals, sizeof(float) * (size_t)e->nnz, cudaMemcpyDeviceToHost, e->st));
    DN_CUDA(cudaStreamSynchronize(e->st));
    return DNPEFF_OK;
}

int dnpeff_export_shard_csc(dnpeff_engine* e, int64_t* colptr, int32_t* rowind, float* vals) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    DN_TRY(build_csc(e, true));
    // The device CSC is in the engine's internal column order; hand it out in
    // local column order (a test/debug path: reordered on the host).
    std::vector<int64_t> cp((size_t)e->ms + 1);
    std::vector<int32_t> perm((size_t)e->ms), ri((size_t)e->nnz);
    std::vector<float> va((size_t)e->nnz);
    DN_CUDA(cudaMemcpyAsync(cp.data(), e->c_colptr, sizeof(int64_t) * (size_t)(e->ms + 1), cudaMemcpyDeviceToHost, e->st));
    if (e->ms > 0) DN_CUDA(cudaMemcpyAsync(perm.data(), e->inv_perm, sizeof(int32_t) * (size_t)e->ms, cudaMemcpyDeviceToHost, e->st));
    if (e->nnz > 0) {
        DN_CUDA(cudaMemcpyAsync(ri.data(), csc_rows(e), sizeof(int32_t) * (size_t)e->nnz, cudaMemcpyDeviceToHost, e->st));
        DN_CUDA(cudaMemcpyAsync(va.data(), csc_vals(e), sizeof(float) * (size_t)e->nnz, cudaMemcpyDeviceToHost, e->st));
    }
    DN_CUDA(cudaStreamSynchronize(e->st));
    int64_t q = 0;
    for (int64_t j = 0; j < e->ms; j++) {
        int64_t jp = perm[(size_t)j];
        if (colptr) colptr[j] = q;
        for (int64_t p = cp[(size_t)jp]; p < cp[(size_t)jp + 1]; p++, q++) {
            if (rowind) rowind[q] = ri[(size_t)p];
            if (vals) vals[q] = va[(size_t)p];
        }
    }
    if (colptr) colptr[e->ms] = q;
    return DNPEFF_OK;
}

int dnpeff_a_sq_norm(dnpeff_engine* e, double* out) {
    DN_TRY(check_ready(e, false));
    *out = e->a_sq;
    return DNPEFF_OK;
}

int dnpeff_a_sum(dnpeff_engine* e, double* out) {
    DN_TRY(check_ready(e, false));
    *out = e->a_sum;
    return DNPEFF_OK;
}

int dnpeff_set_init_scale(dnpeff_engine* e, float init_scale) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    e->p.init_scale = init_scale;
    return DNPEFF_OK;
}

int dnpeff_init_factors(dnpeff_engine* e, const float* W, const float* H) {
    DN_TRY(check_ready(e, false));
    DeviceGuard g(e->device);
    const int r = e->p.rank;
    DN_TRY(init_generated(e, W == nullptr, H == nullptr));
    if (W && e->n > 0)
        DN_CUDA(cudaMemcpyAsync(e->W, W, sizeof(float) * (size_t)(e->n * r), cudaMemcpyHostToDevice, e->st));
    if (H && e->ms > 0) {
        DevBuf<float> tmp;
        DN_TRY(tmp.alloc((size_t)(e->ms * r)));
        DevBuf<float> tmp2;
        DN_TRY(tmp2.alloc((size_t)(e->ms * r)));
        DN_CUDA(cudaMemcpyAsync(tmp.p, H, sizeof(float) * (size_t)(e->ms * r), cudaMemcpyHostToDevice, e->st));
        k_transpose<<<kNumSMs * 8, dim3(32, 8), 0, e->st>>>(tmp.p, tmp2.p, r, e->ms);
        DN_LAUNCH_CHECK();
        // internal row jp holds local column perm[jp]
        k_gather_rows<<<kNumSMs * 8, 256, 0, e->st>>>(tmp2.p, e->perm, e->ms, r, e->H);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(2);
        DN_CUDA(cudaStreamSynchronize(e->st));
    }
    DN_CUDA(cudaStreamSynchronize(e->st));
    e->have_factors = true;
    return DNPEFF_OK;
}

int dnpeff_set_w_row_offset(dnpeff_engine* e, int64_t first_row) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    if (first_row < 0) return fail(DNPEFF_ERR_INVALID, "negative row offset");
    e->w_row_offset = first_row;
    return DNPEFF_OK;
}

int dnpeff_set_h_csr(dnpeff_engine* e, const int64_t* h_rowptr, const int32_t* h_colind, const float* h_vals) {
    DN_TRY(check_ready(e, false));
    if (!h_rowptr) return fail(DNPEFF_ERR_INVALID, "null h_rowptr");
    DeviceGuard g(e->device);
    const int r = e->p.rank;
    const int64_t nnz = h_rowptr[r];
    if (h_rowptr[0] != 0 || nnz < 0) return fail(DNPEFF_ERR_DATA, "row offsets of H must start at 0");
    for (int t = 0; t < r; t++)
        if (h_rowptr[t + 1] < h_rowptr[t]) return fail(DNPEFF_ERR_DATA, "row offsets of H are not non-decreasing");
    if (nnz > 0 && (!h_colind || !h_vals)) return fail(DNPEFF_ERR_INVALID, "null column ids / values of H");
    if (!e->have_factors) DN_TRY(init_generated(e, true, false));  // W as dnpeff_init_factors(NULL, .) makes it
    DN_CUDA(cudaMemsetAsync(e->H, 0, sizeof(float) * (size_t)std::max<int64_t>(e->ms * r, 1), e->st));
    if (nnz > 0 && e->ms > 0) {
        DevBuf<int64_t> drp;
        DevBuf<int32_t> dc;
        DevBuf<float> dv;
        DevBuf<int> err;
        DN_TRY(drp.alloc((size_t)r + 1));
        DN_TRY(dc.alloc((size_t)nnz));
        DN_TRY(dv.alloc((size_t)nnz));
        DN_TRY(err.alloc_zero(1, e->st));
        DN_CUDA(cudaMemcpyAsync(drp.p, h_rowptr, sizeof(int64_t) * (size_t)(r + 1), cudaMemcpyHostToDevice, e->st));
        DN_CUDA(cudaMemcpyAsync(dc.p, h_colind, sizeof(int32_t) * (size_t)nnz, cudaMemcpyHostToDevice, e->st));
        DN_CUDA(cudaMemcpyAsync(dv.p, h_vals, sizeof(float) * (size_t)nnz, cudaMemcpyHostToDevice, e->st));
        k_scatter_h_csr<<<(unsigned)ceil_div(nnz, 256), 256, 0, e->st>>>(drp.p, dc.p, dv.p, r, nnz, e->m_kept, e->map,
                                                                         e->inv_perm, e->H, err.p);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
        int herr = 0;
        DN_TRY(read_err_flag(err.p, e->st, &herr));
        if (herr) return fail(DNPEFF_ERR_DATA, "a column id of H is outside [0, n_cols_kept)");
    }
    DN_CUDA(cudaStreamSynchronize(e->st));
    e->have_factors = true;
    return DNPEFF_OK;
}

int dnpeff_get_w(dnpeff_engine* e, float* out) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    if (e->n > 0)
        DN_CUDA(cudaMemcpyAsync(out, e->W, sizeof(float) * (size_t)(e->n * e->p.rank), cudaMemcpyDeviceToHost, e->st));
    return check_kernel_status(e);
}

int dnpeff_get_h(dnpeff_engine* e, float* out) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    const int r = e->p.rank;
    if (e->ms > 0) {
        DevBuf<float> tmp2;
        float* t = e->WA;  // free between iterations
        if (!t) {
            DN_TRY(tmp2.alloc((size_t)(e->ms * r)));
            t = tmp2.p;
        }
        // local column j is internal row inv_perm[j]; gathered and transposed in one pass
        k_gather_transpose<<<kNumSMs * 8, dim3(32, 8), 0, e->st>>>(e->H, e->inv_perm, e->ms, r, t);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
        DN_CUDA(cudaMemcpyAsync(out, t, sizeof(float) * (size_t)(e->ms * r), cudaMemcpyDeviceToHost, e->st));
        DN_TRY(check_kernel_status(e));
    }
    return DNPEFF_OK;
}

int dnpeff_nccl_unique_id(void* id128) {
    if (!id128) return fail(DNPEFF_ERR_INVALID, "null argument");
    DN_TRY(nccl_load());
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    DN_NCCL(nccl_api().GetUniqueId(&id));
    memcpy(id128, &id, 128);
    return DNPEFF_OK;
}

int dnpeff_comm_init(dnpeff_engine* e, const void* id128, int comm_rank, int comm_size) {
    if (!e || !id128) return fail(DNPEFF_ERR_INVALID, "null argument");
    if (comm_size != e->p.n_shards || comm_rank != e->p.shard_index)
        return fail(DNPEFF_ERR_INVALID, "communicator rank/size must equal shard_index/n_shards");
    DeviceGuard g(e->device);
    DN_TRY(nccl_load());
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    DN_NCCL(nccl_api().CommInitRank(&e->comm, comm_size, id, comm_rank));
    e->comm_rank = comm_rank;
    e->comm_size = comm_size;
    e->a_sq_global = -1.0;
    // NCCL connects its channels on the first collective (hundreds of ms): do that
    // here, as part of joining, not inside the first iteration
    // ... and the point-to-point channels the row-sliced loader uses: NCCL opens as many
    // channels per peer as a transfer's size calls for, the first time it is that large,
    // so the first exchange here is of the loader's order of size (4 MB per peer), not a
    // token one
    const size_t kWarm = (size_t)1 << 20;  // floats per peer and direction
    DevBuf<float> one;
    DN_TRY(one.alloc_zero(32 + 2 * kWarm * (size_t)comm_size, e->st));
    DN_NCCL(nccl_api().AllReduce(one.p, one.p, 32, ncclFloat, ncclSum, e->comm, e->st));
    int gs = DNPEFF_OK;
    DN_NCCL(nccl_api().GroupStart());
    for (int d = 0; d < comm_size; d++) {
        if (d == comm_rank) continue;
        DN_NCCL_IN_GROUP(gs, nccl_api().Send(one.p + 32 + kWarm * (size_t)d, kWarm, ncclFloat, d, e->comm, e->st));
        DN_NCCL_IN_GROUP(gs, nccl_api().Recv(one.p + 32 + kWarm * (size_t)(comm_size + d), kWarm, ncclFloat, d, e->comm,
                                             e->st));
    }
    DN_NCCL(nccl_api().GroupEnd());
    DN_TRY(gs);
    DN_CUDA(cudaStreamSynchronize(e->st));
    return DNPEFF_OK;
}

int dnpeff_step_w(dnpeff_engine* e) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    if (e->p.n_shards > 1 && e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init");
    return step_w(e);
}

int dnpeff_step_h(dnpeff_engine* e) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    return step_h(e);
}

int dnpeff_synchronize(dnpeff_engine* e) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    DeviceGuard g(e->device);
    return check_kernel_status(e);
}

int dnpeff_loss(dnpeff_engine* e, double* out) {
    DN_TRY(check_ready(e, true));
    if (!out) return fail(DNPEFF_ERR_INVALID, "null argument");
    DeviceGuard g(e->device);
    if (e->p.n_shards > 1 && e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init");
    return loss_from_current(e, true, out);
}

int dnpeff_run(dnpeff_engine* e, int32_t iters, int32_t log_every) { return dnpeff_run_steps(e, 0, iters, log_every); }

int dnpeff_run_steps(dnpeff_engine* e, int32_t first_step, int32_t iters, int32_t log_every) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    if (e->p.n_shards > 1 && e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init");
    if (first_step < 0) return fail(DNPEFF_ERR_INVALID, "negative first step");
    auto t0 = std::chrono::high_resolution_clock::now();
    for (int step = first_step; step < first_step + iters; step++) {
        DN_TRY(step_w(e));
        DN_TRY(step_h(e));
        // "step N: <loss> [<ms> ms/step]" every log_every steps, loss time
        // excluded from the rate (multi_mu_dense_factors_nmf1.h:187-201).
        if (log_every > 0 && (step + 1) % log_every == 0) {
            DN_CUDA(cudaStreamSynchronize(e->st));
            auto t1 = std::chrono::high_resolution_clock::now();
            double ms = std::chrono::duration<double, std::milli>(t1 - t0).count();
            double loss = 0;
            DN_TRY(loss_from_current(e, true, &loss));
            if (e->comm_rank == 0) {
                printf("step %d: %g [%g ms/step]\n", step + 1, loss, ms / (double)log_every);
                fflush(stdout);
            }
            t0 = std::chrono::high_resolution_clock::now();
        }
    }
    return DNPEFF_OK;
}

int dnpeff_fit_w_only(dnpeff_engine* e, int32_t iters, double* loss) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    if (e->p.n_shards > 1 && e->comm_size != e->p.n_shards)
        return fail(DNPEFF_ERR_INVALID, "sharded engine without a communicator: call dnpeff_comm_init");
    const int r = e->p.rank;
    DN_TRY(compute_ah_hh(e));
    // wide ranks write the updated W beside the old one: the engine's spare n x r buffer
    if (tensor_cores_enabled() && mu_update_ws_wide_ok(r) && e->n > 0 && !e->w_spare)
        DN_CUDA(cudaMalloc((void**)&e->w_spare, sizeof(float) * (size_t)(e->n * r)));
    for (int it = 0; it < iters; it++) {
        ScopedTimer t(e, 3);
        bool moved = false;
        DN_TRY(mu_update_any(e->W, e->AHG, e->AHG + e->n * r, e->n, r, e->p.eps, e->tc_scratch, e->d_err, e->st, false,
                             e->w_spare, e->opt_wait_limit, &moved));
        if (moved) std::swap(e->W, e->w_spare);
    }
    if (loss) DN_TRY(loss_from_current(e, false, loss));
    return DNPEFF_OK;
}

int dnpeff_enable_timing(dnpeff_engine* e, int enable) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    e->timing = enable != 0;
    return DNPEFF_OK;
}

int dnpeff_get_timing(dnpeff_engine* e, double ms_total[DNPEFF_N_TIMERS], int64_t launches[DNPEFF_N_TIMERS]) {
    if (!e) return fail(DNPEFF_ERR_INVALID, "null engine");
    DeviceGuard g(e->device);
    DN_CUDA(cudaStreamSynchronize(e->st));
    for (auto& r : e->regions) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            e->t_ms[r.id] += ms;
            e->t_n[r.id] += 1;
        }
        e->ev_pool.push_back(r.a);
        e->ev_pool.push_back(r.b);
    }
    e->regions.clear();
    for (int i = 0; i < DNPEFF_N_TIMERS; i++) {
        if (ms_total) ms_total[i] = e->t_ms[i];
        if (launches) launches[i] = e->t_n[i];
        e->t_ms[i] = 0;
        e->t_n[i] = 0;
    }
    return DNPEFF_OK;
}

int dnpeff_launch_count(dnpeff_engine* e, int64_t* out) {
    if (!e || !out) return fail(DNPEFF_ERR_INVALID, "null argument");
    *out = launch_counter() - e->launches0;
    return DNPEFF_OK;
}

// ---- single kernels ---------------------------------------------------------
int dnpeff_op_spmm(const float* vals, const int32_t* ind, const int64_t* ptr, int64_t rows,
                   const float* D, int32_t r, float* out, void* stream) {
    if (rows < 0 || r <= 0) return fail(DNPEFF_ERR_INVALID, "bad shape");
    cudaStream_t st = (cudaStream_t)stream;
    SpmmPlan plan;
    plan.n_short = rows;
    if (spmm_fast_rank(r)) DN_TRY(spmm_make_plan(ptr, 0, rows, &plan, st));
    int s = spmm_dispatch(vals, ind, ptr, rows, D, r, out, plan, st);
    if (plan.long_list) {
        cudaStreamSynchronize(st);
        cudaFree(plan.long_list);
    }
    return s;
}

int dnpeff_op_gram(const float* X, int64_t rows, int32_t r, float* G, void* stream) {
    if (rows < 0 || r <= 0) return fail(DNPEFF_ERR_INVALID, "bad shape");
    float* scratch = nullptr;
    int* err = nullptr;
    DN_TRY(op_scratch(gram_any_scratch(rows, r), &scratch));
    DN_TRY(op_err_word(&err));
    DN_TRY(gram_any(X, rows, r, G, scratch, err, (cudaStream_t)stream));
    return op_check_err(err, (cudaStream_t)stream);
}

int dnpeff_op_mu_update(float* X, const float* Num, const float* G, int64_t rows, int32_t r,
                        float eps, void* stream) {
    if (rows < 0 || r <= 0) return fail(DNPEFF_ERR_INVALID, "bad shape");
    float* scratch = nullptr;
    int* err = nullptr;
    DN_TRY(op_scratch(2 * (size_t)r * r, &scratch));
    DN_TRY(op_err_word(&err));
    DN_TRY(mu_update_any(X, Num, G, rows, r, eps, scratch, err, (cudaStream_t)stream));
    return op_check_err(err, (cudaStream_t)stream);
}

// The projection with its own scratch (released on return; the call synchronises).
static int hoyer_run(float* W, int64_t n, int32_t r, float l1, float l2, int32_t rule, int32_t max_passes,
                     int32_t* passes, int32_t* converged, cudaStream_t st) {
    if (n < 0 || r <= 0) return fail(DNPEFF_ERR_INVALID, "bad shape");
    if (!(l1 > 0.f) || !(l2 > 0.f)) return fail(DNPEFF_ERR_INVALID, "the L1 and L2 norms must be positive");
    if (rule != 0 && rule != 1) return fail(DNPEFF_ERR_INVALID, "alpha_rule must be 0 or 1");
    if (max_passes <= 0) max_passes = (int32_t)std::min<int64_t>(n + 1, INT32_MAX);  // a pass zeroes >= 1 entry per active column
    int np = 0, conv = 1;
    if (n > 0) {
        HoyerPlan plan = hoyer_plan(n, r);
        DevBuf<unsigned char> scratch;
        DN_TRY(scratch.alloc(plan.bytes));
        int* h_count = nullptr;
        DN_CUDA(cudaHostAlloc((void**)&h_count, sizeof(int), cudaHostAllocDefault));
        int s = hoyer_project(W, n, r, l1, l2, rule, max_passes, scratch.p, plan, h_count, &np, &conv, st);
        cudaStreamSynchronize(st);
        cudaFreeHost(h_count);
        if (s != DNPEFF_OK) return s;
    }
    if (passes) *passes = np;
    if (converged) *converged = conv;
    return DNPEFF_OK;
}

int dnpeff_op_hoyer_project(float* W, int64_t n, int32_t r, float l1_norm, float l2_norm, int32_t alpha_rule,
                            int32_t max_passes, int32_t* passes, int32_t* converged, void* stream) {
    return hoyer_run(W, n, r, l1_norm, l2_norm, alpha_rule, max_passes, passes, converged, (cudaStream_t)stream);
}

int dnpeff_sparsify_w(dnpeff_engine* e, float l1_norm, float l2_norm, int32_t alpha_rule, int32_t* passes,
                      int32_t* converged) {
    DN_TRY(check_ready(e, true));
    DeviceGuard g(e->device);
    return hoyer_run(e->W, e->n, e->p.rank, l1_norm, l2_norm, alpha_rule, 0, passes, converged, e->st);
}

int dnpeff_op_block_product(const float* X, int64_t M, int64_t K, const float* Y, int32_t r, float* C,
                            void* stream) {
    if (M < 0 || K < 0 || r <= 0) return fail(DNPEFF_ERR_INVALID, "bad shape");
    if (!block_tc_ok(r)) return fail(DNPEFF_ERR_UNSUPPORTED, "rank must be 32, 64, 96, 128, 256, 384 or 512");
    if (M == 0) return DNPEFF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (K == 0) {
        DN_CUDA(cudaMemsetAsync(C, 0, sizeof(float) * (size_t)(M * r), st));
        return DNPEFF_OK;
    }
    BlockTcPlan p = block_tc_plan(M, K, r);
    DevBuf<float> xb, ysplit, partial;
    DN_TRY(xb.alloc(p.x_floats));
    DN_TRY(ysplit.alloc(p.ysplit_floats));
    DN_TRY(partial.alloc(p.partial_floats));
    int* err = nullptr;
    DN_TRY(op_err_word(&err));
    k_block_layout<<<(unsigned)ceil_div((int64_t)(p.x_floats / 4), 256), 256, 0, st>>>(X, M, K, p.m_tiles, p.k_chunks,
                                                                                      xb.p);
    DN_LAUNCH_CHECK();
    DN_TRY(block_tc_launch(xb.p, p, Y, M, K, r, C, ysplit.p, partial.p, err, st));
    int s = op_check_err(err, st);
    DN_CUDA(cudaStreamSynchronize(st));  // the scratch buffers are released on return
    return s;
}

}  // extern "C"
