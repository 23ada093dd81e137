/*
 * dnpeff.h -- C ABI of the B200 D-NPEFF factorization engine.
 *
 * The reference (mmatena/npeff_ref, cc/cuda_d_npeff) has no FFI or plugin
 * interface for this path: it is reached through the `run_nmf_on_pefs` process
 * (mains/run_nmf_on_pefs.cu) and, in process, through the public members of
 * MuNmf<IndT> (src/nmf/sparse/multi_mu_dense_factors_nmf1.h:81,152,207,222,242)
 * plus three host preprocessing functions.  Each entry point below names the
 * reference interface it replaces.
 *
 * Conventions
 *   - every function returns DNPEFF_OK (0) or a negative dnpeff_status; the
 *     message of the last failure on the calling thread is dnpeff_last_error();
 *     nothing throws or aborts across this boundary (the reference terminates
 *     on every error, src/cuda/cuda_statuses.h:15-38);
 *   - one engine owns ONE column shard of A on ONE device; a multi-GPU job is
 *     one engine per device (one process or thread each) joined by
 *     dnpeff_comm_init; calls on one engine must be serialised by the caller;
 *   - host buffers are caller-owned; device memory is engine-owned and is
 *     released by dnpeff_destroy;
 *   - W is [n_rows, rank] row-major, H is [rank, n_cols] row-major at this
 *     boundary: the layouts of the output file (src/io/nmf_decomp_h5.h:38-89);
 *   - values are fp32, column ids int32, row offsets int64.
 *   - there is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails with DNPEFF_ERR_CUDA.
 */
#ifndef DNPEFF_H_
#define DNPEFF_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DNPEFF_ABI_VERSION 1

typedef enum {
    DNPEFF_OK = 0,
    DNPEFF_ERR_INVALID = -1,   /* bad argument, shape or call order */
    DNPEFF_ERR_CUDA = -2,      /* CUDA runtime failure, or no device */
    DNPEFF_ERR_NCCL = -3,      /* NCCL missing or failed */
    DNPEFF_ERR_DATA = -4,      /* malformed matrix: index out of range, duplicate column in a row */
    DNPEFF_ERR_UNSUPPORTED = -5,
    DNPEFF_ERR_IO = -6         /* file could not be read or written */
} dnpeff_status;

typedef struct dnpeff_engine dnpeff_engine;

/* MuNmfParams (src/nmf/sparse/multi_mu_dense_factors_device_contexts1.h:36-55)
 * and the values run_nmf_on_pefs.cu:190-200 fills in. */
typedef struct {
    int32_t rank;       /* --nmf_n_components */
    float eps;          /* added to the denominator; the executable hard-codes 1e-8f */
    uint64_t seed;      /* the executable hard-codes 43190432042 */
    float init_scale;   /* factors start as init_scale * U(0,1]; <= 0 means 1.0 (reference) */
    int32_t shard_index; /* which part of the kept columns this engine owns */
    int32_t n_shards;    /* number of parts (== number of engines in the job) */
    int32_t shard_mode;  /* DNPEFF_SHARD_CONTIGUOUS (reference) or DNPEFF_SHARD_CYCLIC */
} dnpeff_params;

/* How the kept columns are dealt to the engines of a job.
 * CONTIGUOUS: equal-width ranges, the last takes the remainder -- splitColumnWise /
 *   getSizeOfSplit (src/util/matrix_util.h:10-69); H shards concatenate in order.
 * CYCLIC: engine d owns kept columns d, d+n_shards, ...; balances stored entries
 *   when column popularity follows the column order (the reference's split puts
 *   every popular column on engine 0).  dnpeff_get_shard_columns tells where each
 *   local column of H belongs. */
#define DNPEFF_SHARD_CONTIGUOUS 0
#define DNPEFF_SHARD_CYCLIC 1

const char* dnpeff_last_error(void);
int dnpeff_abi_version(void);

/* Number of CUDA devices visible; replaces cudaGetDeviceCount at
 * run_nmf_on_pefs.cu:126 / multi_mu_dense_factors_nmf1.h:84. */
int dnpeff_device_count(int* count);

/* DeviceContext ctor + initializeCuda (…device_contexts1.h:129-170,360-376).
 * `stream` is a cudaStream_t the engine launches on, or NULL to create one. */
int dnpeff_create(const dnpeff_params* params, int device, void* stream, dnpeff_engine** out);
int dnpeff_destroy(dnpeff_engine* eng);

/* Engine options: tuning values and test hooks (no reference counterpart; the
 * reference has no tunables beyond MuNmfParams).  Set before the call they affect;
 * value 0 restores the built-in default.
 *   "loader_slabs"      dnpeff_set_csr uploads the values in this many row slabs on a
 *                       second stream and processes each as it lands (1..8; default: 4
 *                       from 64 Mi entries on, else 1)
 *   "tail_block_bytes"  bytes of H covered by one column block of the unpopular
 *                       columns, i.e. per gather launch (default 48 MiB)
 *   "popular_divisor"   a column is popular from ceil(n_rows / d) entries on (d >= 2;
 *                       default 16 with the dense tensor-core block, else 8)
 *   "keep_canonical_csr" 1: keep the shard's CSR in input order after the loader has
 *                       built its own layout (needed by dnpeff_export_shard_csr;
 *                       costs 8 bytes per stored entry; default 0)
 *   "wait_limit"        polls after which a wait between the roles of a
 *                       warp-specialised tensor-core kernel (dense block, Gram, update)
 *                       gives up (default 2^24); the kernel then leaves cleanly and the
 *                       next call that reads the engine's status returns DNPEFF_ERR_CUDA
 * Unknown names fail with DNPEFF_ERR_INVALID. */
int dnpeff_set_option(dnpeff_engine* eng, const char* name, int64_t value);

/* ---- loader: normalize -> prune -> shard -> CSR + CSC on the device -------
 * Replaces PefSparseFishers::normalizeFishers_inPlace (src/io/pef_fisher_h5.h:38-52),
 * removeSmallestL0NormColumns_inPlace (src/util/sparse_util.h:79-159),
 * splitColumnWise (src/util/matrix_util.h:24-69) and moveAToDeviceAsync
 * (…device_contexts1.h:182-195).
 *   vals, colind : nnz entries; row i owns [rowptr[i], rowptr[i+1]), or
 *                  [i*k, (i+1)*k) when rowptr == NULL (the D-PEF file's
 *                  implicit offsets, pef_fisher_h5.h:175-177)
 *   norms        : n_rows row norms (data/dense_fisher_norms) or NULL to skip
 *                  the normalisation
 *   n_cols_full  : dense_fisher_size
 * The *_device form takes device pointers (inputs already resident in HBM);
 * the inputs are not modified and may be released after the call returns. */
int dnpeff_set_csr(dnpeff_engine* eng, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                   const int64_t* rowptr, const float* vals, const int32_t* colind,
                   const float* norms, int32_t min_values_per_parameter);
int dnpeff_set_csr_device(dnpeff_engine* eng, int64_t n_rows, int64_t n_cols_full,
                          int64_t k_per_row, const int64_t* d_rowptr, const float* d_vals,
                          const int32_t* d_colind, const float* d_norms,
                          int32_t min_values_per_parameter);

/* The loader for a matrix that arrives in row slices, one per engine of a job: the
 * multi-GPU form of moveAToDeviceAsync (…device_contexts1.h:180-194), where the
 * reference uploads to every device only that device's column partition (made on the
 * host by splitColumnWise, src/util/matrix_util.h:24-69).  Here engine i of G passes
 * rows [row_begin, row_begin + n_rows) of the matrix -- the range dnpeff_row_slice
 * gives for (n_rows_total, G, i) -- so every engine uploads 1/G of the entries; the
 * per-column counts are summed over the engines (one integer allreduce), every
 * engine derives the same pruning map, and each entry travels over NVLink to the
 * engine that owns its column (grouped ncclSend / ncclRecv).  The resulting shard is
 * the same, bit for bit, as the one dnpeff_set_csr builds from the whole matrix.
 * Collective: every engine of the job must make the call, after dnpeff_comm_init.
 * rowptr (or NULL with k_per_row), vals, colind and norms describe the slice only;
 * rowptr starts at 0. */
int dnpeff_row_slice(int64_t n_rows_total, int32_t n_engines, int32_t index, int64_t* row_begin, int64_t* n_rows);
int dnpeff_set_csr_rows(dnpeff_engine* eng, int64_t n_rows_total, int64_t n_cols_full, int64_t k_per_row,
                        int64_t row_begin, int64_t n_rows, const int64_t* rowptr, const float* vals,
                        const int32_t* colind, const float* norms, int32_t min_values_per_parameter);

/* dnpeff_set_csr_rows with the slice already in device memory. */
int dnpeff_set_csr_rows_device(dnpeff_engine* eng, int64_t n_rows_total, int64_t n_cols_full, int64_t k_per_row,
                               int64_t row_begin, int64_t n_rows, const int64_t* d_rowptr, const float* d_vals,
                               const int32_t* d_colind, const float* d_norms, int32_t min_values_per_parameter);
/* shard_index / n_shards the engine was created with, and its device (any may be NULL). */
int dnpeff_get_shard(dnpeff_engine* eng, int32_t* shard_index, int32_t* n_shards, int32_t* device);
/* Collective AND over the engines of a job: *all_ok = 1 only if every engine passed
 * ok != 0.  Lets the engines agree, before a collective loader call, that each of
 * them could read its part of a file (an engine that stayed out of a collective
 * would leave the others waiting).  No reference counterpart (single process). */
int dnpeff_comm_agree(dnpeff_engine* eng, int32_t ok, int32_t* all_ok);

/* The same loader with the kept columns given as a list of original column ids
 * instead of a count threshold: CsrMatrix::RetainColumns_InPlace
 * (src/cuda/host/sparse_matrix.h:141-170) as fit_coeffs_to_sparse_H applies it
 * with a decomposition's reduce_kept_indices (mains/fit_coeffs_to_sparse_H.cu:
 * 137-140).  A column's new index is its position in the list; entries in other
 * columns are dropped; an id listed twice keeps its last position. */
int dnpeff_set_csr_retain(dnpeff_engine* eng, int64_t n_rows, int64_t n_cols_full, int64_t k_per_row,
                          const int64_t* rowptr, const float* vals, const int32_t* colind,
                          const float* norms, const int32_t* retained_cols, int64_t n_retained);

/* Shapes after the loader ran.  n_cols_kept = columns surviving the pruning
 * (over all shards); this engine owns kept columns [col_start, col_start+n_cols_shard)
 * (getSizeOfSplit, src/util/matrix_util.h:10-20). */
int dnpeff_get_shape(dnpeff_engine* eng, int64_t* n_rows, int64_t* n_cols_kept,
                     int64_t* col_start, int64_t* n_cols_shard, int64_t* nnz_shard);
/* How the engine laid the shard out internally (no reference counterpart;
 * reported by the benchmark): columns held by a sizeable share of the rows are
 * "popular"; that block of A is kept a second time as a dense matrix and its part
 * of both products runs on the tensor cores (ranks 32..128, multiples of 32;
 * tile_rows = 0 then) or, for other ranks, through the shared-memory tiled SpMM
 * kernel (tile_rows = rows of the dense factor per tile).  The rest is cut into
 * column blocks whose slice of H stays L2-resident while it is gathered. */
int dnpeff_get_layout(dnpeff_engine* eng, int64_t* n_popular_cols, int64_t* popular_nnz,
                      int32_t* n_tail_blocks, int32_t* tile_rows);
/* newToOgIndex of removeSmallestL0NormColumns_inPlace: n_cols_kept original ids. */
int dnpeff_get_new_to_og(dnpeff_engine* eng, int32_t* out);
/* For each of the n_cols_shard local columns: its index among the kept columns
 * (position in the full H / in reduce_kept_indices) and its original column id.
 * Either output may be NULL. */
int dnpeff_get_shard_columns(dnpeff_engine* eng, int32_t* kept_ids, int32_t* original_ids);
/* The shard's CSR as splitColumnWise leaves it (bit-exact partition check). */
int dnpeff_export_shard_csr(dnpeff_engine* eng, int64_t* rowptr, int32_t* colind, float* vals);
/* The shard's CSC (values, row ids, n_cols_shard+1 offsets), rows ascending in a column. */
int dnpeff_export_shard_csc(dnpeff_engine* eng, int64_t* colptr, int32_t* rowind, float* vals);
/* sum of squares of the shard's stored values (computeASqNorm, …device_contexts1.h:274-294). */
int dnpeff_a_sq_norm(dnpeff_engine* eng, double* out);
/* sum of the shard's stored values (for the Uniform*sqrt(mean(A)/r) initial scale). */
int dnpeff_a_sum(dnpeff_engine* eng, double* out);

/* ---- files ------------------------------------------------------------------
 * The D-PEF input file (written by npeff/fishers/d_pefs_computer.py:235-251):
 *   data/fisher/values  float32 [n, k],  data/fisher/indices int32 [n, k],
 *   attribute dense_fisher_size on group data/fisher,
 *   data/dense_fisher_norms float32 [n].
 * dnpeff_pef_hdf5_info replaces the dimension probe of
 * Pef::pefRequiresInt64Indices (src/io/pef_fisher_h5.h:57-90);
 * dnpeff_read_pef_hdf5 / dnpeff_load_pef_hdf5 replace PefSparseFishers::read
 * (:107-226): n_examples / n_fisher_values <= 0 mean "all", otherwise the leading
 * rows / leading values per row are taken (--n_examples, --n_fisher_values).
 * dnpeff_load_pef_hdf5 = read + load, streamed: the engine reads only its slice of
 * the rows (dnpeff_row_slice; the whole file for a single engine) in chunks into two
 * page-locked staging buffers and uploads each chunk while the next is being read,
 * then runs the row-sliced loader (dnpeff_set_csr_rows_device); a multi-engine job
 * calls it on every engine after dnpeff_comm_init (collective).  Files are read and
 * written by a built-in HDF5 codec (contiguous, uncompressed datasets only). */
int dnpeff_pef_hdf5_info(const char* path, int64_t* n_examples, int64_t* n_values_per_example,
                         int64_t* dense_fisher_size);
int dnpeff_read_pef_hdf5(const char* path, int64_t n_examples, int64_t n_fisher_values, float* vals,
                         int32_t* indices, float* norms);
int dnpeff_load_pef_hdf5(dnpeff_engine* eng, const char* path, int64_t n_examples,
                         int64_t n_fisher_values, int32_t min_values_per_parameter);
/* NmfDecomposition<IndT>::save (src/io/nmf_decomp_h5.h:38-89): data/W [n, r],
 * data/H [r, n_kept], data/reduce_kept_indices [n_kept] (int32) with attribute
 * full_dense_size of shape {1}; the file npeff/decomp/decomps.py:55-71 loads. */
int dnpeff_save_decomposition_hdf5(const char* path, const float* W, const float* H,
                                   const int32_t* reduce_kept_indices, int64_t n_examples,
                                   int32_t rank, int64_t n_kept, int64_t full_dense_size);
/* NmfDecomposition<IndT>::read (src/io/nmf_decomp_h5.h:100-126), used for
 * --initial_W_path / --initial_H_path.  Any output may be NULL. */
int dnpeff_decomposition_hdf5_info(const char* path, int64_t* n_examples, int32_t* rank,
                                   int64_t* n_kept, int64_t* full_dense_size);
int dnpeff_read_decomposition_hdf5(const char* path, float* W, float* H, int32_t* reduce_kept_indices);
/* Decomposition with H in CSR form (SparseNmfDecomposition::save / ::read,
 * src/io/nmf_decomp_h5.h:134-237; scripts/sparsify_d_npeff.py:27-73 writes the
 * same file): data/W, data/H/{values, row_indices, column_indices} with the
 * attribute data/H.shape = {rank, n_kept}, data/reduce_kept_indices with the
 * attribute full_dense_size.  Row offsets are written as int64, column ids as
 * int32 (the script's types); any integer width is read.  Outputs may be NULL. */
int dnpeff_save_sparse_decomposition_hdf5(const char* path, const float* W, int64_t n_examples, int32_t rank,
                                          const int64_t* h_rowptr, const int32_t* h_colind,
                                          const float* h_vals, const int32_t* reduce_kept_indices,
                                          int64_t n_kept, int64_t full_dense_size);
int dnpeff_sparse_decomposition_hdf5_info(const char* path, int64_t* n_examples, int32_t* rank,
                                          int64_t* n_kept, int64_t* h_nnz, int64_t* full_dense_size);
int dnpeff_read_sparse_decomposition_hdf5(const char* path, float* W, int64_t* h_rowptr, int32_t* h_colind,
                                          float* h_vals, int32_t* reduce_kept_indices);
/* Shape/type of any dataset, and its leading rows x cols block as float64
 * (src/util/h5_util.h helpers). */
int dnpeff_hdf5_dataset_info(const char* path, const char* dataset, int32_t* rank, int64_t dims[4],
                             int32_t* is_float, int32_t* type_size);
int dnpeff_hdf5_read_f64(const char* path, const char* dataset, int64_t rows, int64_t cols, double* out);

/* ---- factors --------------------------------------------------------------
 * initializeW / initializeH / broadcastInitializedW (…device_contexts1.h:197-233,
 * multi_mu_dense_factors_nmf1.h:131-135,358-375).  W: [n_rows, rank] row-major
 * or NULL; H: this shard's [rank, n_cols_shard] row-major or NULL.  NULL means
 * "generate": init_scale * U(0,1] from a counter-based hash of (seed, global
 * element index), identical on every shard layout and reproducible on a CPU. */
int dnpeff_init_factors(dnpeff_engine* eng, const float* W, const float* H);
/* H from its CSR form (rank rows x n_cols_kept columns; int64 row offsets, int32
 * column ids, as the sparse decomposition file holds them, src/io/nmf_decomp_h5.h:
 * 134-170): zero elsewhere.  The engine keeps H dense (the sparse-sparse products
 * of Nmf::OnlyW::SparseH::Learner, src/nmf/sparse2/nmf_sparse_H.h:157-166,
 * 252-262, become the engine's A*H^T and H*H^T); on a sharded engine entries of
 * other shards' columns are skipped.  W is generated if no factors were set yet. */
int dnpeff_set_h_csr(dnpeff_engine* eng, const int64_t* h_rowptr, const int32_t* h_colind,
                     const float* h_vals);
/* Global index of the engine's first row, used only where W is generated: the
 * row chunks of one matrix (SplitRowWise, src/cuda/host/sparse_matrix.h:219-245,
 * as fit_coeffs_to_sparse_H feeds them) then draw the rows an unchunked engine
 * would.  No reference counterpart (its generator is cuRAND over the whole W). */
int dnpeff_set_w_row_offset(dnpeff_engine* eng, int64_t first_row);
int dnpeff_set_init_scale(dnpeff_engine* eng, float init_scale);
/* loadWToHostSync / loadHToHostSync + toRowMajor_inPlace
 * (multi_mu_dense_factors_nmf1.h:207-240, src/util/matrices.h:49-62). */
int dnpeff_get_w(dnpeff_engine* eng, float* out);
int dnpeff_get_h(dnpeff_engine* eng, float* out);

/* ---- multi-GPU ------------------------------------------------------------
 * initializeNccl (multi_mu_dense_factors_nmf1.h:341-349).  The reference uses
 * ncclCommInitAll in one process; here every engine joins with the 128-byte
 * id made by dnpeff_nccl_unique_id on one of them. */
int dnpeff_nccl_unique_id(void* id128);
int dnpeff_comm_init(dnpeff_engine* eng, const void* id128, int comm_rank, int comm_size);

/* ---- iteration ------------------------------------------------------------
 * updateW / updateH / run (multi_mu_dense_factors_nmf1.h:152-205,293-339).
 * dnpeff_run does `iters` x (step_w, step_h); when log_every > 0 it prints the
 * reference's "step N: <loss> [<ms> ms/step]" line every log_every steps.
 * All three are asynchronous on the engine's stream unless they log. */
int dnpeff_step_w(dnpeff_engine* eng);
int dnpeff_step_h(dnpeff_engine* eng);
int dnpeff_run(dnpeff_engine* eng, int32_t iters, int32_t log_every);
/* dnpeff_run for a run made in several calls (periodic checkpoints): the logged
 * step numbers continue from first_step. */
int dnpeff_run_steps(dnpeff_engine* eng, int32_t first_step, int32_t iters, int32_t log_every);
int dnpeff_synchronize(dnpeff_engine* eng);
/* computeUncachedLoss (multi_mu_dense_factors_nmf1.h:242-274): the global
 * sqrt(|A|^2 + <H,(W^T W)H> - 2<W^T A,H>), identical on every engine. */
int dnpeff_loss(dnpeff_engine* eng, double* out);

/* W-only fit with H fixed (Nmf::OnlyW::SparseH::Learner, src/nmf/sparse2/
 * nmf_sparse_H.h:116-127,157-211,298-345): A*H^T and H*H^T once, then `iters`
 * x  W *= AH / (W*HH + eps).  Uses the engine's current H; returns the loss
 * sqrt(|A|^2 + <W*HH,W> - 2<AH,W>) when loss != NULL. */
int dnpeff_fit_w_only(dnpeff_engine* eng, int32_t iters, double* loss);

/* ---- measurement ----------------------------------------------------------
 * Per-kernel device time (CUDA events on the engine's stream).  Kernel ids:
 * 0 spmm A*H^T, 1 spmm A^T*W, 2 gram, 3 update, 4 allreduce, 5 loss. */
#define DNPEFF_N_TIMERS 6
int dnpeff_enable_timing(dnpeff_engine* eng, int enable);
int dnpeff_get_timing(dnpeff_engine* eng, double ms_total[DNPEFF_N_TIMERS],
                      int64_t launches[DNPEFF_N_TIMERS]);
/* Number of kernel launches of this library since the engine was made. */
int dnpeff_launch_count(dnpeff_engine* eng, int64_t* out);

/* ---- single kernels on caller-owned device buffers ------------------------
 * The building blocks above, exposed for kernel-level parity tests and
 * benchmarks.  All pointers are device pointers; `stream` is a cudaStream_t.
 *
 * dnpeff_op_spmm: out[i,:] = sum_{p in [ptr[i],ptr[i+1])} vals[p] * D[ind[p],:],
 *   out is [rows, r], D is [*, r], both row-major.  Replaces the two
 *   cusparseSpMM calls (…device_contexts1.h:255-265; device_matrix_util.h:184-192).
 * dnpeff_op_gram: G[r,r] = X^T X for X [rows, r].  Replaces the cublasSgemm
 *   calls for H*H^T and W^T*W (…device_contexts1.h:303,322).
 * dnpeff_op_mu_update: X[i,c] *= Num[i,c] / (sum_t X[i,t]*G[t,c] + eps).
 *   Replaces cublasSgemm W*(HH^T) / (W^T W)*H (…device_contexts1.h:306,329)
 *   fused with kernelNmfMuUpdate (src/nmf/sparse/kernels.h:24-34). */
int dnpeff_op_spmm(const float* vals, const int32_t* ind, const int64_t* ptr, int64_t rows,
                   const float* D, int32_t r, float* out, void* stream);
int dnpeff_op_gram(const float* X, int64_t rows, int32_t r, float* G, void* stream);
int dnpeff_op_mu_update(float* X, const float* Num, const float* G, int64_t rows, int32_t r,
                        float eps, void* stream);
/* dnpeff_op_block_product: C[M,r] = X[M,K] * Y[K,r], all row-major and dense, on
 *   the tensor-core kernel that multiplies the dense popular block of A (ranks
 *   32, 64, 96, 128 in one go, 256, 384, 512 in panels of 128 columns;
 *   fp32-equivalent 3xTF32; other ranks: DNPEFF_ERR_UNSUPPORTED).  It stands for the popular columns'
 *   share of the same two cusparseSpMM calls; exposed for kernel-level tests. */
int dnpeff_op_block_product(const float* X, int64_t M, int64_t K, const float* Y, int32_t r, float* C,
                            void* stream);

/* Hoyer's sparseness projection of the components of W: every column of the
 * row-major W[n, r] is replaced by the closest non-negative vector whose entries
 * sum to l1_norm and whose Euclidean norm is l2_norm ("Non-negative Matrix
 * Factorization with Sparseness Constraints", Hoyer 2004, projection operator).
 * Replaces DenseFactorSparsityContext::sparsifyF
 * (src/nmf/sparse/dense_factor_sparsity_constraints.h:205-237) and its kernels
 * (src/nmf/sparse/sparsity_constraint_kernels.h:14-141), which the reference
 * builds for W on device 0 from --sparsity_W (= l1_norm; l2_norm 1,
 * mains/run_nmf_on_pefs.cu:200) but never calls (the call in MuNmf::run,
 * multi_mu_dense_factors_nmf1.h:162, is commented out).
 *   alpha_rule 0: alpha is the non-negative root of |m + alpha (s - m)| = l2_norm,
 *     as published; the result has exactly the requested norms.
 *   alpha_rule 1: the reference's kernel_computeAlpha expression, which is that root
 *     only when m and s - m are parallel.
 *   max_passes <= 0: n + 1 (a pass removes at least one entry of every column that
 *     is still active); the reference loops without a limit.
 *   passes / converged (may be NULL): passes made; 1 when no column is left active.
 * The call synchronises the stream once per pass (as the reference's
 * isFinishedSync) and allocates its scratch (9 bytes per element of W at most).
 * dnpeff_sparsify_w applies it to the engine's W (every rank of a column-sharded
 * run holds the same W and gets the same result). */
int dnpeff_op_hoyer_project(float* W, int64_t n, int32_t r, float l1_norm, float l2_norm, int32_t alpha_rule,
                            int32_t max_passes, int32_t* passes, int32_t* converged, void* stream);
int dnpeff_sparsify_w(dnpeff_engine* eng, float l1_norm, float l2_norm, int32_t alpha_rule, int32_t* passes,
                      int32_t* converged);

/* Allocation-free variant of dnpeff_op_gram (no counterpart in the reference).
 *
 * For callers that must not allocate device memory at call time: code running
 * inside another framework's memory pool, a loop with a fixed memory budget, or
 * any place where cudaMalloc's implicit device synchronisation is unacceptable.
 * The slab partials go to a fixed DNPEFF_NOALLOC_SCRATCH_BYTES array that is part
 * of the library image (every GPU that loads the library holds it until the
 * process exits) instead of an allocated buffer; the call makes no cudaMalloc,
 * cudaFree or other allocating call.  Inputs and outputs are the caller's, as
 * for dnpeff_op_gram.  The partial sums always come from the CUDA-core kernel
 * (fp32 FMA, slabs folded in double), whereas dnpeff_op_gram takes the tensor-core
 * kernel at the ranks that one supports: the two results agree to about 3e-6 of
 * the largest entry, not bit for bit.  A row count whose default slab split would
 * not fit the array is cut into fewer, longer slabs.
 *   - rank above DNPEFF_NOALLOC_MAX_RANK fails with DNPEFF_ERR_UNSUPPORTED;
 *   - the first call on a device looks up the array's device address; under
 *     CUDA's lazy module loading that lookup may load the library's module onto
 *     the device, which materialises the array and can synchronise the device --
 *     the only point where this entry point can cause either.  Make that first
 *     call at set-up time, before starting any stream capture on that device;
 *   - all calls on a device share the one array: calls that can overlap on the
 *     GPU (different streams, different threads) race and must be serialised by
 *     the caller.  Nothing in the array needs clearing between calls. */
#define DNPEFF_NOALLOC_SCRATCH_BYTES (16 * 1024 * 1024)
#define DNPEFF_NOALLOC_MAX_RANK 1024
int dnpeff_op_gram_noalloc(const float* X, int64_t rows, int32_t r, float* G, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DNPEFF_H_ */
