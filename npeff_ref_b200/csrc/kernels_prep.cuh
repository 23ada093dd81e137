// Loader kernels: column counting, pruning map, shard extraction, CSC build,
// plus the small elementwise helpers (init, transpose, reductions).
// These are integer/byte passes bound by HBM bandwidth; every index is 64-bit
// because nnz and rank*n_cols exceed 2^31 at the large configurations.
#pragma once
#include "common.cuh"

namespace dnpeff {

enum : int { kErrColRange = 1, kErrDuplicate = 2, kErrRowPtr = 4 };

// Which kept columns an engine owns, and their local numbering.
//   contiguous: [c0, c0+w), local = c - c0  -- the reference's equal-width split
//               (src/util/matrix_util.h:10-20)
//   cyclic:     c % stride == offset, local = c / stride -- spreads popular
//               columns evenly over the engines (the equal-width split puts every
//               popular column of a popularity-ordered feature axis on engine 0)
struct ShardMap {
    int64_t c0, w;
    int32_t stride, offset;
    int32_t cyclic;
    __host__ __device__ bool owns(int64_t c) const {
        return cyclic ? (c >= 0 && (c % stride) == offset) : (c >= c0 && c < c0 + w);
    }
    __host__ __device__ int64_t local(int64_t c) const { return cyclic ? c / stride : c - c0; }
    __host__ __device__ int64_t global(int64_t j) const {
        return cyclic ? j * stride + offset : c0 + j;
    }
};

// Row i of the input owns [rowptr[i], rowptr[i+1]) or, with rowptr == NULL,
// [i*k, (i+1)*k): the implicit offsets of a D-PEF file (src/io/pef_fisher_h5.h:175-177).
__device__ __forceinline__ void row_range(const int64_t* rowptr, int64_t k, int64_t row,
                                          int64_t& b, int64_t& e) {
    if (rowptr) { b = rowptr[row]; e = rowptr[row + 1]; }
    else { b = row * k; e = b + k; }
}

// colMask[csrColIndA[i]] += 1 of removeSmallestL0NormColumns_inPlace
// (src/util/sparse_util.h:95-98), as integer atomics (order-independent).
__global__ void k_count_columns(const int32_t* __restrict__ colind, int64_t nnz, int64_t n_cols,
                                int32_t* __restrict__ counts, int* __restrict__ err) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz; p += stride) {
        int32_t c = __ldcs(colind + p);
        if ((uint32_t)c >= (uint64_t)n_cols) atomicOr(err, kErrColRange);
        else atomicAdd(counts + c, 1);
    }
}

// keep[c] = counts[c] >= min  (src/util/sparse_util.h:110-118)
__global__ void k_keep_flags(const int32_t* __restrict__ counts, int64_t n_cols, int32_t min_count,
                             int32_t* __restrict__ flags) {
    int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c < n_cols) flags[c] = counts[c] >= min_count ? 1 : 0;
}

// ---- exclusive scan (1024 threads x 4 items per block) ----------------------
template <typename TIn>
__global__ void k_scan_block(const TIn* __restrict__ in, int64_t* __restrict__ out,
                             int64_t* __restrict__ block_sums, int64_t N) {
    __shared__ int64_t wsum[32];
    int64_t base = ((int64_t)blockIdx.x * 1024 + threadIdx.x) * 4;
    int64_t v[4];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[i] = (base + i < N) ? (int64_t)in[base + i] : 0;
        s += v[i];
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int64_t inc = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int64_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) wsum[w] = inc;
    __syncthreads();
    if (w == 0) {
        int64_t x = wsum[lane];
        int64_t xi = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int64_t t = __shfl_up_sync(0xffffffffu, xi, o);
            if (lane >= o) xi += t;
        }
        wsum[lane] = xi - x;  // exclusive prefix of warp sums
        if (lane == 31 && block_sums) block_sums[blockIdx.x] = xi;
    }
    __syncthreads();
    int64_t run = wsum[w] + inc - s;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (base + i < N) out[base + i] = run;
        run += v[i];
    }
}

__global__ void k_scan_add(int64_t* __restrict__ out, const int64_t* __restrict__ block_prefix,
                           int64_t N) {
    int64_t base = ((int64_t)blockIdx.x * 1024 + threadIdx.x) * 4;
    int64_t add = block_prefix[blockIdx.x];
#pragma unroll
    for (int i = 0; i < 4; i++)
        if (base + i < N) out[base + i] += add;
}

// og_to_new / new_to_og of src/util/sparse_util.h:105-120 from the scanned flags.
__global__ void k_build_maps(const int32_t* __restrict__ flags, const int64_t* __restrict__ pos,
                             int64_t n_cols, int32_t* __restrict__ og_to_new,
                             int32_t* __restrict__ new_to_og) {
    int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n_cols) return;
    if (flags[c]) {
        og_to_new[c] = (int32_t)pos[c];
        new_to_og[pos[c]] = (int32_t)c;
    } else {
        og_to_new[c] = -1;
    }
}

// RetainColumns_InPlace (src/cuda/host/sparse_matrix.h:141-170): the kept columns
// are a given list of original ids and a column's new index is its position in
// the list (the last position wins if an id is listed twice, as in the sequential
// loop there).  og_to_new must be filled with -1 before.
__global__ void k_retain_maps(const int32_t* __restrict__ retained, int64_t n_retained, int64_t n_cols,
                              int32_t* __restrict__ og_to_new, int32_t* __restrict__ new_to_og,
                              int* __restrict__ err) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_retained) return;
    int32_t c = retained[i];
    new_to_og[i] = c;
    if (c < 0 || c >= n_cols) {
        atomicOr(err, kErrColRange);
        return;
    }
    atomicMax(&og_to_new[c], (int32_t)i);
}

// H given in CSR form (rank rows x kept columns) scattered into this shard's dense
// H (internal row order, zeroed before).  One thread per stored entry; an entry
// whose column another shard owns is skipped.
__global__ void k_scatter_h_csr(const int64_t* __restrict__ rowptr, const int32_t* __restrict__ colind,
                                const float* __restrict__ vals, int r, int64_t nnz, int64_t m_kept,
                                ShardMap map, const int32_t* __restrict__ inv_perm, float* __restrict__ H,
                                int* __restrict__ err) {
    int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= nnz) return;
    // the row of H that holds entry p: last t with rowptr[t] <= p
    int lo = 0, hi = r;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (rowptr[mid] <= p) lo = mid; else hi = mid;
    }
    const int64_t c = colind[p];
    if (c < 0 || c >= m_kept) {
        atomicOr(err, kErrColRange);
        return;
    }
    if (!map.owns(c)) return;
    H[(int64_t)inv_perm[map.local(c)] * r + lo] = vals[p];
}

// Entries of each row that fall into kept columns [c0, c0+w) of this shard:
// the counting pass of splitColumnWise (src/util/matrix_util.h:39-44) merged
// with the pruning test (src/util/sparse_util.h:139).  One block per row.
__global__ void k_row_counts(const int32_t* __restrict__ colind, const int64_t* __restrict__ rowptr,
                             int64_t k, int64_t n_rows, const int32_t* __restrict__ og_to_new,
                             ShardMap map, int32_t* __restrict__ row_count,
                             int* __restrict__ err) {
    __shared__ int ws[32];
    for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
        int64_t b, e;
        row_range(rowptr, k, row, b, e);
        if (e < b) { if (threadIdx.x == 0) atomicOr(err, kErrRowPtr); e = b; }
        int cnt = 0;
        for (int64_t p = b + threadIdx.x; p < e; p += blockDim.x) {
            int64_t c = og_to_new[__ldcs(colind + p)];
            cnt += map.owns(c) ? 1 : 0;
        }
        cnt = warp_sum_i(cnt);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = cnt;
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = 0;
            for (int i = 0; i < (int)(blockDim.x >> 5); i++) t += ws[i];
            row_count[row] = t;
        }
    }
}

// Order-preserving extraction of the shard's entries, with the row
// normalisation val / (norm + 1e-9f) of src/io/pef_fisher_h5.h:38-52 applied on
// the way and the column ids rebased to the shard start
// (src/util/matrix_util.h:57-61).  One block of 256 threads per row.
__global__ void k_extract_shard(const float* __restrict__ vals, const int32_t* __restrict__ colind,
                                const int64_t* __restrict__ rowptr, int64_t k, int64_t row_begin, int64_t n_rows,
                                const float* __restrict__ norms,
                                const int32_t* __restrict__ og_to_new, ShardMap map,
                                const int64_t* __restrict__ out_rowptr, float* __restrict__ out_vals,
                                int32_t* __restrict__ out_colind) {
    __shared__ int wtot[8];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int64_t row = row_begin + blockIdx.x; row < n_rows; row += gridDim.x) {
        int64_t b, e;
        row_range(rowptr, k, row, b, e);
        if (e < b) e = b;
        float denom = norms ? (norms[row] + 1e-9f) : 1.0f;
        int64_t run = out_rowptr[row];
        for (int64_t base = b; base < e; base += 256) {
            int64_t p = base + threadIdx.x;
            bool keep = false;
            int64_t c = 0;
            float v = 0.f;
            if (p < e) {
                c = og_to_new[__ldcs(colind + p)];
                keep = map.owns(c);
                v = __ldcs(vals + p);
            }
            unsigned bal = __ballot_sync(0xffffffffu, keep);
            if (lane == 0) wtot[wid] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                int t = wtot[i];
                before += (i < wid) ? t : 0;
                total += t;
            }
            if (keep) {
                int64_t q = run + before + __popc(bal & ((1u << lane) - 1u));
                out_colind[q] = (int32_t)map.local(c);
                out_vals[q] = norms ? v / denom : v;
            }
            run += total;
            __syncthreads();
        }
    }
}

__global__ void k_max_rowlen(const int64_t* __restrict__ rowptr, int64_t n_rows,
                             unsigned long long* __restrict__ out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n_rows) atomicMax(out, (unsigned long long)(rowptr[i + 1] - rowptr[i]));
}

// cnt_s[j] = counts[new_to_og[global(j)]]: every stored entry of a kept column
// survives, so the pruning counts are also the shard's column lengths.
__global__ void k_gather_counts(const int32_t* __restrict__ counts,
                                const int32_t* __restrict__ new_to_og, ShardMap map,
                                int32_t* __restrict__ cnt_s) {
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j < map.w) cnt_s[j] = counts[new_to_og[map.global(j)]];
    else if (j == map.w) cnt_s[j] = 0;
}

// ---- CSC build --------------------------------------------------------------
// A transpose with rows ascending inside every column, in two steps.  (1) Every
// entry takes the next free slot of its column (integer atomicAdd on a per-column
// cursor) in a temporary copy of the CSC arrays: the columns are complete but in
// arrival order.  This runs one launch per segment of the bucketed rows (segment
// 0 = a row's popular part, segment s >= 1 = its entries in tail column block
// s-1), so that the cursors and the slots being written belong to one block of
// columns and stay in L2.  (2) Every column is put in row order into the final
// arrays: a row occurs at most once per column, so the order -- and with it the
// result -- does not depend on the arrival order.  Short columns are ranked by
// comparison (keys in shared memory), long ones through a bitmap of their rows.
// A row that holds a column twice shows up as two equal keys: kErrDuplicate.
struct RowSegments {
    const uint32_t* tail_off;  // [rows][n_tail + 1]
    int stride;                // n_tail + 1
    __device__ void range(const int64_t* rowptr, int64_t row, int seg, int64_t& b, int64_t& e) const {
        const int64_t r0 = rowptr[row];
        const uint32_t* t = tail_off + row * stride;
        b = r0 + (seg == 0 ? 0u : t[seg - 1]);
        e = r0 + t[seg];
    }
};

// grid = ceil(rows / 8), 256 threads: one warp per row, segment `seg` of it
__global__ void k_csc_scatter(const int64_t* __restrict__ rowptr, const int32_t* __restrict__ colind,
                              const float* __restrict__ vals, int64_t n_rows, RowSegments segs, int seg,
                              const int64_t* __restrict__ colptr, int32_t* __restrict__ cursor,
                              float* __restrict__ tvals, int32_t* __restrict__ trow) {
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    int64_t beg, end;
    segs.range(rowptr, row, seg, beg, end);
    for (int64_t p = beg + (threadIdx.x & 31); p < end; p += 32) {
        const int32_t j = colind[p];
        const int64_t q = colptr[j] + atomicAdd(cursor + j, 1);
        tvals[q] = vals[p];
        trow[q] = (int32_t)row;
    }
}

constexpr int kCscShortMax = 512;  // longest column ranked by comparison (keys per warp in shared memory)

// Columns [col_first, col_last) with at most kCscShortMax entries: one warp per column.
__global__ void __launch_bounds__(256)
k_csc_order_short(const int64_t* __restrict__ colptr, int64_t col_first, int64_t col_last,
                  const float* __restrict__ tvals, const int32_t* __restrict__ trow,
                  float* __restrict__ cvals, int32_t* __restrict__ crow, int* __restrict__ err) {
    __shared__ int32_t keys[8][kCscShortMax];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t warps = (int64_t)gridDim.x * 8;
    for (int64_t j = col_first + (int64_t)blockIdx.x * 8 + w; j < col_last; j += warps) {
        const int64_t b = colptr[j];
        const int len = (int)(colptr[j + 1] - b);
        if (len > kCscShortMax || len <= 0) continue;
        if (len == 1) {
            if (lane == 0) { cvals[b] = tvals[b]; crow[b] = trow[b]; }
            continue;
        }
        for (int e = lane; e < len; e += 32) keys[w][e] = trow[b + e];
        __syncwarp();
        for (int e = lane; e < len; e += 32) {
            const int32_t k = keys[w][e];
            int rank = 0, same = 0;
            for (int t = 0; t < len; t++) {
                const int32_t o = keys[w][t];
                rank += o < k;
                same += o == k;
            }
            if (same > 1) atomicOr(err, kErrDuplicate);
            // with a repeated row the ranks collide; keep the writes inside the column
            crow[b + rank] = k;
            cvals[b + rank] = tvals[b + e];
        }
        __syncwarp();
    }
}

// Columns longer than kCscShortMax: one block per column, a bitmap of the column's
// rows in shared memory (n_rows bits), rank = set bits below the row.
// Dynamic shared memory: 2 * ceil(n_rows / 32) words.
__global__ void __launch_bounds__(256)
k_csc_order_long(const int64_t* __restrict__ colptr, const int32_t* __restrict__ long_cols, int n_long,
                 int64_t n_rows, const float* __restrict__ tvals, const int32_t* __restrict__ trow,
                 float* __restrict__ cvals, int32_t* __restrict__ crow, int* __restrict__ err) {
    extern __shared__ uint32_t bm[];  // [words] bits, then [words] exclusive prefix of popcounts
    const int words = (int)((n_rows + 31) / 32);
    uint32_t* pre = bm + words;
    __shared__ uint32_t carry;
    for (int c = blockIdx.x; c < n_long; c += gridDim.x) {
        const int64_t j = long_cols[c];
        const int64_t b = colptr[j];
        const int len = (int)(colptr[j + 1] - b);
        for (int i = threadIdx.x; i < words; i += 256) bm[i] = 0u;
        __syncthreads();
        for (int e = threadIdx.x; e < len; e += 256) {
            const int32_t k = trow[b + e];
            const uint32_t bit = 1u << (k & 31);
            if (atomicOr(bm + (k >> 5), bit) & bit) atomicOr(err, kErrDuplicate);
        }
        __syncthreads();
        // exclusive prefix of the word popcounts, 256 words at a time
        if (threadIdx.x == 0) carry = 0u;
        __syncthreads();
        for (int base = 0; base < words; base += 256) {
            const int i = base + threadIdx.x;
            uint32_t v = i < words ? (uint32_t)__popc(bm[i]) : 0u;
            // block-wide inclusive scan of v (warp scans + warp totals)
            uint32_t inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                if ((threadIdx.x & 31) >= o) inc += t;
            }
            __shared__ uint32_t wtot[8];
            if ((threadIdx.x & 31) == 31) wtot[threadIdx.x >> 5] = inc;
            __syncthreads();
            uint32_t add = carry;
            for (int ww = 0; ww < (threadIdx.x >> 5); ww++) add += wtot[ww];
            if (i < words) pre[i] = add + inc - v;
            __syncthreads();
            if (threadIdx.x == 255) carry = add + inc;
            __syncthreads();
        }
        for (int e = threadIdx.x; e < len; e += 256) {
            const int32_t k = trow[b + e];
            const int rank = (int)(pre[k >> 5] + (uint32_t)__popc(bm[k >> 5] & ((1u << (k & 31)) - 1u)));
            crow[b + rank] = k;
            cvals[b + rank] = tvals[b + e];
        }
        __syncthreads();
    }
}

// long_cols <- ids of the columns in [col_first, col_last) longer than kCscShortMax.
__global__ void k_csc_list_long(const int64_t* __restrict__ colptr, int64_t col_first, int64_t col_last,
                                int32_t* __restrict__ long_cols, int* __restrict__ n_long) {
    int64_t j = col_first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= col_last) return;
    if (colptr[j + 1] - colptr[j] > kCscShortMax) long_cols[atomicAdd(n_long, 1)] = (int32_t)j;
}

// ---- internal column order and row buckets -----------------------------------
// The engine renumbers a shard's columns as [popular ("hot") columns in id
// order][the rest in id order].  hot_pos is the exclusive scan of the hot flags.
__global__ void k_hot_flags(const int32_t* __restrict__ col_count, int64_t n_cols, int32_t threshold,
                            int32_t* __restrict__ flags) {
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n_cols) flags[j] = col_count[j] >= threshold ? 1 : 0;
    else if (j == n_cols) flags[j] = 0;
}

__global__ void k_build_perm(const int32_t* __restrict__ flags, const int64_t* __restrict__ hot_pos,
                             int64_t n_cols, int64_t n_hot, int32_t* __restrict__ perm,
                             int32_t* __restrict__ inv_perm) {
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_cols) return;
    int64_t jp = flags[j] ? hot_pos[j] : n_hot + (j - hot_pos[j]);
    inv_perm[j] = (int32_t)jp;
    perm[jp] = (int32_t)j;
}

// cnt_p[jp] = col_count[perm[jp]] (+ a trailing zero for the scan).
__global__ void k_permute_counts(const int32_t* __restrict__ col_count, const int32_t* __restrict__ perm,
                                 int64_t n_cols, int32_t* __restrict__ cnt_p) {
    int64_t jp = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (jp < n_cols) cnt_p[jp] = col_count[perm[jp]];
    else if (jp == n_cols) cnt_p[jp] = 0;
}

// Bucket of an internal column: hot columns are cut into tiles of `tile` columns
// (buckets 0..n_hot_tiles-1), the rest into blocks of `block` columns.
struct BucketMap {
    int64_t n_hot;
    int32_t tile, block, n_hot_tiles, n_buckets;
    __host__ __device__ int bucket(int64_t jp) const {
        return jp < n_hot ? (int)(jp / tile) : n_hot_tiles + (int)((jp - n_hot) / block);
    }
};

// Stable partition of every row's entries by bucket (one block of 8 warps per
// row, dynamic shared memory 8 * n_buckets ints).  Input: the shard's CSR with
// local column ids; output: the same rows with internal column ids, entries
// grouped by ascending bucket, original order kept inside a bucket, plus
// tail_off[row][b] = offset inside the row of tail block b (b = 0 is the end of
// the hot part; n_tail_blocks + 1 entries per row).
__global__ void __launch_bounds__(256)
k_bucket_rows(const float* __restrict__ vals, const int32_t* __restrict__ col,
              const int64_t* __restrict__ rowptr, int64_t row_begin, int64_t n_rows,
              const int32_t* __restrict__ inv_perm,
              BucketMap bm, float* __restrict__ out_vals, int32_t* __restrict__ out_col,
              uint32_t* __restrict__ tail_off) {
    extern __shared__ int cnt[];  // [8][n_buckets]
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int NB = bm.n_buckets;
    const int n_tail = NB - bm.n_hot_tiles;
    for (int64_t row = row_begin + blockIdx.x; row < n_rows; row += gridDim.x) {
        const int64_t beg = rowptr[row], end = rowptr[row + 1];
        const int64_t len = end - beg;
        int64_t chunk = ((len + 7) / 8 + 31) / 32 * 32;  // per-warp share, a multiple of 32
        const int64_t wb = beg + w * chunk < end ? beg + w * chunk : end;
        const int64_t we = wb + chunk < end ? wb + chunk : end;
        for (int i = threadIdx.x; i < 8 * NB; i += 256) cnt[i] = 0;
        __syncthreads();
        // 1. per-warp bucket counts
        for (int64_t base = wb; base < we; base += 32) {
            int64_t p = base + lane;
            int b = -1 - lane;  // inactive lanes: distinct negative keys
            if (p < we) b = bm.bucket(inv_perm[col[p]]);
            unsigned peers = __match_any_sync(0xffffffffu, b);
            if (p < we && lane == __ffs(peers) - 1) cnt[w * NB + b] += __popc(peers);
            __syncwarp();
        }
        __syncthreads();
        // 2. start of every (bucket, warp) run: buckets ascending, warps ascending inside
        if (w == 0) {
            int run = 0;
            for (int b0 = 0; b0 < NB; b0 += 32) {
                int b = b0 + lane;
                int tot = 0;
                if (b < NB)
                    for (int ww = 0; ww < 8; ww++) tot += cnt[ww * NB + b];
                int inc = tot;
                for (int o = 1; o < 32; o <<= 1) {
                    int t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += t;
                }
                int start = run + inc - tot;
                if (b < NB) {
                    if (b >= bm.n_hot_tiles) tail_off[row * (n_tail + 1) + (b - bm.n_hot_tiles)] = (uint32_t)start;
                    for (int ww = 0; ww < 8; ww++) {
                        int c = cnt[ww * NB + b];
                        cnt[ww * NB + b] = start;
                        start += c;
                    }
                }
                run += __shfl_sync(0xffffffffu, inc, 31);
            }
            if (lane == 0) tail_off[row * (n_tail + 1) + n_tail] = (uint32_t)len;
        }
        __syncthreads();
        // 3. stable scatter
        for (int64_t base = wb; base < we; base += 32) {
            int64_t p = base + lane;
            int b = -1 - lane;
            int jp = 0;
            float v = 0.f;
            if (p < we) {
                jp = inv_perm[col[p]];
                b = bm.bucket(jp);
                v = vals[p];
            }
            unsigned peers = __match_any_sync(0xffffffffu, b);
            if (p < we) {
                int rank = __popc(peers & ((1u << lane) - 1u));
                int64_t q = beg + cnt[w * NB + b] + rank;
                out_col[q] = jp;
                out_vals[q] = v;
            }
            __syncwarp();
            if (p < we && lane == __ffs(peers) - 1) cnt[w * NB + b] += __popc(peers);
            __syncwarp();
        }
        __syncthreads();
    }
}

// rows_out[i] = rows_in[index[i]] for r floats per row (float4 when r % 4 == 0).
__global__ void k_gather_rows(const float* __restrict__ in, const int32_t* __restrict__ index,
                              int64_t n_rows, int r, float* __restrict__ out) {
    int64_t total = n_rows * r;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t row = i / r;
        int c = (int)(i - row * r);
        out[i] = in[(int64_t)index[row] * r + c];
    }
}

// ---- reductions over the stored values --------------------------------------
// partial[b] = (sum v, sum v*v) of block b, then one block folds the partials in
// index order: double accumulation, fixed order.
__global__ void k_sum_sumsq(const float* __restrict__ v, int64_t count, double* __restrict__ partial) {
    __shared__ double sm[32];
    double s = 0.0, q = 0.0;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        double x = (double)v[i];
        s += x;
        q += x * x;
    }
    double ts = block_sum(s, sm);
    double tq = block_sum(q, sm);
    if (threadIdx.x == 0) {
        partial[2 * blockIdx.x] = ts;
        partial[2 * blockIdx.x + 1] = tq;
    }
}

// partial[b] = sum a[i]*b[i] over block b's grid-stride share (double).
__global__ void k_dot(const float* __restrict__ a, const float* __restrict__ b, int64_t count,
                      double* __restrict__ partial) {
    __shared__ double sm[32];
    double s = 0.0;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        s += (double)a[i] * (double)b[i];
    double t = block_sum(s, sm);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// out[c] = sum_b partial[b*ncomp + c], one block, fixed order.
__global__ void k_fold(const double* __restrict__ partial, int nblocks, int ncomp,
                       double* __restrict__ out) {
    __shared__ double sm[32];
    for (int c = 0; c < ncomp; c++) {
        double s = 0.0;
        for (int b = threadIdx.x; b < nblocks; b += blockDim.x) s += partial[b * ncomp + c];
        double t = block_sum(s, sm);
        if (threadIdx.x == 0) out[c] = t;
    }
}

// ---- factor helpers ---------------------------------------------------------
__global__ void k_init_uniform(float* __restrict__ out, int64_t first, int64_t count, uint64_t key,
                               float scale) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        out[i] = uniform01_from_key(key, (uint64_t)(first + i)) * scale;
}

// H[j, t] = scale * U(0,1] at global index (global column of j) * r + t, so every
// sharding of the feature axis starts from the same matrix.
// Row jp of `out` is internal column jp = local column perm[jp].
__global__ void k_init_uniform_cols(float* __restrict__ out, int64_t n_local_cols, int r,
                                    ShardMap map, const int32_t* __restrict__ perm, uint64_t key,
                                    float scale) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t count = n_local_cols * r;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        int64_t jp = i / r;
        int t = (int)(i - jp * r);
        out[i] = uniform01_from_key(key, (uint64_t)(map.global(perm[jp]) * r + t)) * scale;
    }
}

// out[j] = original (dense_fisher_size) id of local column j.
__global__ void k_shard_columns(const int32_t* __restrict__ new_to_og, ShardMap map,
                                int32_t* __restrict__ kept_ids, int32_t* __restrict__ og_ids) {
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= map.w) return;
    int64_t g = map.global(j);
    if (kept_ids) kept_ids[j] = (int32_t)g;
    if (og_ids) og_ids[j] = new_to_og[g];
}

// out[c, r] = in[r, c] for in of shape [rows, cols] (row-major both).  Used to
// go between the file layout H[rank, n_cols] and the device layout [n_cols, rank]
// (the reference does this on the host, src/util/matrices.h:49-62).
__global__ void k_transpose(const float* __restrict__ in, float* __restrict__ out, int64_t rows,
                            int64_t cols) {
    __shared__ float tile[32][33];
    int64_t tiles_c = (cols + 31) / 32;
    int64_t tiles_r = (rows + 31) / 32;
    for (int64_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        int64_t tr = t / tiles_c, tc = t % tiles_c;
        for (int i = threadIdx.y; i < 32; i += blockDim.y) {
            int64_t r_ = tr * 32 + i, c_ = tc * 32 + threadIdx.x;
            tile[i][threadIdx.x] = (r_ < rows && c_ < cols) ? in[r_ * cols + c_] : 0.f;
        }
        __syncthreads();
        for (int i = threadIdx.y; i < 32; i += blockDim.y) {
            int64_t c_ = tc * 32 + i, r_ = tr * 32 + threadIdx.x;
            if (c_ < cols && r_ < rows) out[c_ * rows + r_] = tile[threadIdx.x][i];
        }
        __syncthreads();
    }
}

// out[c, j] = in[index[j], c]: the rows of `in` ([*, cols] row-major) picked by `index`
// (n_out of them) and transposed in one pass (the gather of the internal column order
// fused with the device -> file layout transpose).
__global__ void k_gather_transpose(const float* __restrict__ in, const int32_t* __restrict__ index, int64_t n_out,
                                   int64_t cols, float* __restrict__ out) {
    __shared__ float tile[32][33];
    int64_t tiles_c = (cols + 31) / 32;
    int64_t tiles_r = (n_out + 31) / 32;
    for (int64_t t = blockIdx.x; t < tiles_c * tiles_r; t += gridDim.x) {
        int64_t tr = t / tiles_c, tc = t % tiles_c;
        for (int i = threadIdx.y; i < 32; i += blockDim.y) {
            int64_t j = tr * 32 + i, c_ = tc * 32 + threadIdx.x;
            tile[i][threadIdx.x] = (j < n_out && c_ < cols) ? in[(int64_t)index[j] * cols + c_] : 0.f;
        }
        __syncthreads();
        for (int i = threadIdx.y; i < 32; i += blockDim.y) {
            int64_t c_ = tc * 32 + i, j = tr * 32 + threadIdx.x;
            if (c_ < cols && j < n_out) out[c_ * n_out + j] = tile[threadIdx.x][i];
        }
        __syncthreads();
    }
}

}  // namespace dnpeff
