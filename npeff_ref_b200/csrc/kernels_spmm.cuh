// Sparse x dense-rows product  out[i,:] = sum_{p in row i} vals[p] * D[ind[p],:].
//
// One kernel family serves both multiplicative-update products:
//   A   * H^T : S = CSR(A) (rows = examples),  D = H stored [n_cols, r]
//   A^T * W   : S = CSC(A) (rows = features),  D = W stored [n_rows, r]
// (the two cusparseSpMM calls of multi_mu_dense_factors_device_contexts1.h:255-265).
//
// Work split: a row shorter than kLongRow entries is done by one warp; longer
// rows are listed once and done by a whole block whose warps interleave 32-entry
// chunks and fold their partial rows through shared memory in warp order.  The
// summation order of every output element is fixed, so results repeat bit for bit.
//
// Inside a warp the lanes are cut into 32/G groups; a group owns one stored
// entry at a time and its lanes cover the r floats of the gathered D row with
// V 128-bit loads each.  U entries are in flight per group so that U*V >= 8
// independent 16-byte loads per lane hide the gather latency.
#pragma once
#include "common.cuh"

namespace dnpeff {

constexpr int kLongRow = 1024;      // entries; longer rows go to the block kernel
constexpr int kSpmmWarps = 8;       // warps per block in both kernels

template <int G, int V>
__device__ __forceinline__ void spmm_accumulate(const float* __restrict__ vals,
                                                const int32_t* __restrict__ ind, int64_t beg,
                                                int64_t end, int64_t chunk_stride,
                                                const float4* __restrict__ D4, int r4,
                                                float4 (&acc)[V]) {
    constexpr int NG = 32 / G;
    constexpr int U = (V >= 8) ? 1 : (8 / V);
    const int lane = threadIdx.x & 31;
    const int g = lane / G, l = lane % G;
    // Lanes past the end of the row (r4 not a multiple of G) gather the last
    // float4 instead: their accumulators are never stored, so no masking is needed.
    int cq[V];
#pragma unroll
    for (int q = 0; q < V; q++) cq[q] = (l + G * q < r4) ? l + G * q : r4 - 1;
    for (int64_t base = beg; base < end; base += chunk_stride) {
        int64_t p = base + lane;
        float v = 0.f;
        int j = 0;
        if (p < end) {
            v = __ldcs(vals + p);
            j = __ldcs(ind + p);
        }
        int cnt = (int)((end - base) < 32 ? (end - base) : 32);
        // NG*U divides 32, so every shuffle source below is a lane of this chunk;
        // lanes past `cnt` hold v = 0, j = 0 and add nothing.
        for (int t0 = 0; t0 < cnt; t0 += NG * U) {
            float vv[U];
            int jj[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                int src = t0 + u * NG + g;
                vv[u] = __shfl_sync(0xffffffffu, v, src);
                jj[u] = __shfl_sync(0xffffffffu, j, src);
            }
            float4 h[U][V];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const float4* drow = D4 + (int64_t)jj[u] * r4;
#pragma unroll
                for (int q = 0; q < V; q++) h[u][q] = __ldg(drow + cq[q]);
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
#pragma unroll
                for (int q = 0; q < V; q++) {
                    acc[q].x = fmaf(vv[u], h[u][q].x, acc[q].x);
                    acc[q].y = fmaf(vv[u], h[u][q].y, acc[q].y);
                    acc[q].z = fmaf(vv[u], h[u][q].z, acc[q].z);
                    acc[q].w = fmaf(vv[u], h[u][q].w, acc[q].w);
                }
            }
        }
    }
    // fold the NG groups (butterfly: every lane ends with the group-order sum)
#pragma unroll
    for (int o = G; o < 32; o <<= 1) {
#pragma unroll
        for (int q = 0; q < V; q++) {
            acc[q].x += __shfl_xor_sync(0xffffffffu, acc[q].x, o);
            acc[q].y += __shfl_xor_sync(0xffffffffu, acc[q].y, o);
            acc[q].z += __shfl_xor_sync(0xffffffffu, acc[q].z, o);
            acc[q].w += __shfl_xor_sync(0xffffffffu, acc[q].w, o);
        }
    }
}

// Which stored entries of a row one launch covers: the whole row, or -- for a
// matrix whose rows were partitioned into column buckets -- bucket `b` of it.
struct SegView {
    const int64_t* ptr;    // row offsets
    const uint32_t* boff;  // optional bucket offsets inside each row, [rows][stride]
    int stride;
    int b;
    __device__ __forceinline__ void range(int64_t row, int64_t& beg, int64_t& end) const {
        if (boff) {
            int64_t base = ptr[row];
            const uint32_t* o = boff + row * stride + b;
            beg = base + o[0];
            end = base + o[1];
        } else {
            beg = ptr[row];
            end = ptr[row + 1];
        }
    }
};

__device__ __forceinline__ void store_or_add(float4* dst, const float4& v, int accumulate) {
    if (accumulate) {
        float4 o = *dst;
        *dst = make_float4(o.x + v.x, o.y + v.y, o.z + v.z, o.w + v.w);
    } else {
        *dst = v;
    }
}

// Lists the rows of [row_first, row_first+rows) longer than kLongRow (once per
// matrix: the structure is static).  The list order depends on atomic timing; it
// only decides which block takes which row, never a summation order.
__global__ void k_classify_rows(const int64_t* __restrict__ ptr, int64_t row_first, int64_t rows,
                                int32_t* __restrict__ long_list, int* __restrict__ n_long) {
    int64_t row = row_first + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row < row_first + rows && ptr[row + 1] - ptr[row] > kLongRow)
        long_list[atomicAdd(n_long, 1)] = (int32_t)row;
}

// One warp per row; rows longer than `long_thresh` are left to the block kernel.
template <int G, int V>
__global__ void __launch_bounds__(kSpmmWarps * 32)
k_spmm_warp(const float* __restrict__ vals, const int32_t* __restrict__ ind, SegView seg,
            int64_t row_first, int64_t rows, int64_t long_thresh, const float4* __restrict__ D4,
            int r4, float4* __restrict__ out4, int accumulate) {
    const int lane = threadIdx.x & 31;
    int64_t row = (int64_t)blockIdx.x * kSpmmWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    row += row_first;
    int64_t beg, end;
    seg.range(row, beg, end);
    if (end - beg > long_thresh) return;
    float4 acc[V];
#pragma unroll
    for (int q = 0; q < V; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    spmm_accumulate<G, V>(vals, ind, beg, end, 32, D4, r4, acc);
    if (lane < G) {
#pragma unroll
        for (int q = 0; q < V; q++) {
            int c = lane + G * q;
            if (c < r4) store_or_add(out4 + row * r4 + c, acc[q], accumulate);
        }
    }
}

// One block per row: the rows of `long_list`, or rows row_first + item when the
// list is NULL.  Dynamic shared memory: kSpmmWarps * r4 float4.
template <int G, int V>
__global__ void __launch_bounds__(kSpmmWarps * 32)
k_spmm_block(const float* __restrict__ vals, const int32_t* __restrict__ ind, SegView seg,
             const int32_t* __restrict__ long_list, int64_t row_first, int64_t n_items,
             const float4* __restrict__ D4, int r4, float4* __restrict__ out4, int accumulate) {
    extern __shared__ float4 red[];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int64_t item = blockIdx.x; item < n_items; item += gridDim.x) {
        int64_t row = long_list ? (int64_t)long_list[item] : row_first + item;
        int64_t beg, end;
        seg.range(row, beg, end);
        float4 acc[V];
#pragma unroll
        for (int q = 0; q < V; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        spmm_accumulate<G, V>(vals, ind, beg + 32 * w, end, 32 * kSpmmWarps, D4, r4, acc);
        if (lane < G) {
#pragma unroll
            for (int q = 0; q < V; q++) {
                int c = lane + G * q;
                if (c < r4) red[w * r4 + c] = acc[q];
            }
        }
        __syncthreads();
        for (int c = threadIdx.x; c < r4; c += blockDim.x) {
            float4 s = red[c];
#pragma unroll
            for (int i = 1; i < kSpmmWarps; i++) {
                float4 t = red[i * r4 + c];
                s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
            }
            store_or_add(out4 + row * r4 + c, s, accumulate);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Tiled product for the dense part of the matrix: rows whose stored entries
// cover a small range of D rows many times over (the popular feature columns
// in A*H^T; the popular features' own columns in A^T*W).  D is cut into tiles of
// `tile_rows` rows; a tile (tile_rows * r floats, contiguous in memory) is
// brought into shared memory once per block with ONE bulk async copy (TMA,
// cp.async.bulk + mbarrier) and every warp of the block gathers from shared
// memory instead of L2, two tiles in flight.  Each warp owns one row of S and
// walks its entries tile by tile: the entries of a row must be grouped by tile
// in ascending tile order (any order inside a tile).
//
// Persistent blocks fetch groups of rows (one per warp) from an atomic counter.
// Every wait on the copy barrier is bounded: on expiry the block records the
// error and leaves without touching the output again.
// Warps (= rows) per block of the tiled kernel: 32 while the kernel fits 64
// registers per thread (up to 4 float4 accumulators per lane), 16 above.
template <int V>
struct TiledWarps {
    static constexpr int value = (V <= 4) ? 32 : 16;
};
constexpr uint32_t kTiledSpinLimit = 1u << 24;
enum : int { kErrTiledTimeout = 8 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void bulk_load_tile(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Returns false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done = 0;
    for (uint32_t spin = 0; spin < kTiledSpinLimit; spin++) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

template <int G, int V>
__global__ void __launch_bounds__(TiledWarps<V>::value * 32, 1)
k_spmm_tiled(const float* __restrict__ vals, const int32_t* __restrict__ ind,
             const int64_t* __restrict__ ptr, const uint32_t* __restrict__ row_len,
             int row_len_stride, int64_t rows, const float* __restrict__ D, int r4, int64_t d_rows, int tile_rows,
             float4* __restrict__ out4, int accumulate, int* __restrict__ work_counter,
             int* __restrict__ err) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[2];
    __shared__ int s_group;
    constexpr int NG = 32 / G;
    constexpr int U = (V >= 8) ? 1 : (8 / V);
    const int kTiledWarps = blockDim.x >> 5;  // rows per group, chosen by the launcher
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int g = lane / G, l = lane % G;
    const size_t tile_floats4 = (size_t)tile_rows * r4;
    float4* const tile0 = (float4*)smem_raw;
    const uint32_t tile_smem = smem_u32(smem_raw);
    const uint32_t row_bytes = (uint32_t)r4 * 16u;
    const uint32_t tile_bytes = (uint32_t)tile_rows * row_bytes;
    const int n_tiles = (int)((d_rows + tile_rows - 1) / tile_rows);
    const int64_t n_groups = (rows + kTiledWarps - 1) / kTiledWarps;

    if (threadIdx.x == 0) {
        mbar_init(&full_bar[0], 1);
        mbar_init(&full_bar[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t phase_bits = 0;  // bit b: parity the next wait on buffer b expects
    // byte offset of this lane's float4s inside a tile row; lanes past the end of
    // the row read the last float4 (their accumulators are never stored)
    uint32_t lane_off[V];
#pragma unroll
    for (int q = 0; q < V; q++) lane_off[q] = (uint32_t)((l + G * q < r4) ? l + G * q : r4 - 1) * 16u;

    auto issue = [&](int t) {  // thread 0 only
        int64_t first = (int64_t)t * tile_rows;
        int64_t nrow = d_rows - first < tile_rows ? d_rows - first : tile_rows;
        bulk_load_tile(tile0 + (size_t)(t & 1) * tile_floats4, D + first * (int64_t)r4 * 4,
                       (uint32_t)(nrow * r4 * 16), &full_bar[t & 1]);
    };

    while (true) {
        if (threadIdx.x == 0) s_group = atomicAdd(work_counter, 1);
        __syncthreads();
        const int64_t group = s_group;
        if (group >= n_groups) break;
        const int64_t row = group * kTiledWarps + w;
        int64_t cursor = 0, end = 0;
        if (row < rows) {
            cursor = ptr[row];
            end = row_len ? cursor + row_len[row * row_len_stride] : ptr[row + 1];
        }
        float4 acc[V];
#pragma unroll
        for (int q = 0; q < V; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);

        if (threadIdx.x == 0) issue(0);
        // A window of 64 stored entries is kept in registers: (v, j) are the 32 at the
        // cursor, (vb, jb) the 32 after them.  When the cursor moves the window is
        // re-aligned with shuffles and only the far half is fetched again, so the
        // entries needed next are always already on their way.
        float v = 0.f, vb = 0.f;
        int j = INT32_MAX, jb = INT32_MAX;
        auto load_far = [&]() {
            int64_t p = cursor + 32 + lane;
            vb = 0.f;
            jb = INT32_MAX;
            if (p < end) {
                vb = __ldcs(vals + p);
                jb = __ldcs(ind + p);
            }
        };
        {
            int64_t p = cursor + lane;
            if (p < end) {
                v = __ldcs(vals + p);
                j = __ldcs(ind + p);
            }
            load_far();
        }
        auto advance = [&](int cnt) {
            cursor += cnt;
            if (cnt == 32) {
                v = vb;
                j = jb;
            } else {
                const int src = lane + cnt;
                const float v0 = __shfl_sync(0xffffffffu, v, src & 31);
                const float v1 = __shfl_sync(0xffffffffu, vb, src & 31);
                const int j0 = __shfl_sync(0xffffffffu, j, src & 31);
                const int j1 = __shfl_sync(0xffffffffu, jb, src & 31);
                v = src < 32 ? v0 : v1;
                j = src < 32 ? j0 : j1;
            }
            load_far();
        };
        bool ok = true;
        for (int t = 0; t < n_tiles; t++) {
            const int buf = t & 1;
            if (threadIdx.x == 0 && t + 1 < n_tiles) issue(t + 1);
            if (!mbar_wait(&full_bar[buf], (phase_bits >> buf) & 1u)) ok = false;
            phase_bits ^= 1u << buf;
            if (!__syncthreads_and(ok ? 1 : 0)) { ok = false; break; }
            // 32-bit shared-memory address of this lane's 16 bytes of tile row 0
            const uint32_t buf_base = tile_smem + (uint32_t)buf * tile_bytes;
            const int64_t tile_base = (int64_t)t * tile_rows;
            const int64_t tile_end = tile_base + tile_rows;
            while (true) {
                const bool in = (int64_t)j < tile_end;
                const unsigned mask = __ballot_sync(0xffffffffu, in);
                const int cnt = __popc(mask);  // entries are grouped by tile: a prefix of the chunk
                if (cnt == 0) break;
                // byte offset of the gathered tile row, computed once by the owning lane
                const uint32_t off = in ? (uint32_t)((int64_t)j - tile_base) * row_bytes : 0u;
                const float vz = in ? v : 0.f;
                for (int t0 = 0; t0 < cnt; t0 += NG * U) {
                    float vv[U];
                    uint32_t oo[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        int src = t0 + u * NG + g;
                        vv[u] = __shfl_sync(0xffffffffu, vz, src);
                        oo[u] = __shfl_sync(0xffffffffu, off, src);
                    }
                    float4 h[U][V];
#pragma unroll
                    for (int u = 0; u < U; u++) {
#pragma unroll
                        for (int q = 0; q < V; q++) {
                            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                         : "=f"(h[u][q].x), "=f"(h[u][q].y), "=f"(h[u][q].z), "=f"(h[u][q].w)
                                         : "r"(buf_base + oo[u] + lane_off[q]));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; u++) {
#pragma unroll
                        for (int q = 0; q < V; q++) {
                            acc[q].x = fmaf(vv[u], h[u][q].x, acc[q].x);
                            acc[q].y = fmaf(vv[u], h[u][q].y, acc[q].y);
                            acc[q].z = fmaf(vv[u], h[u][q].z, acc[q].z);
                            acc[q].w = fmaf(vv[u], h[u][q].w, acc[q].w);
                        }
                    }
                }
                advance(cnt);
                if (cnt < 32) break;
            }
            __syncthreads();  // everybody is done with this buffer before it is refilled
        }
        if (!ok) {
            // let the copies still in flight land (bounded) before the block leaves
            if (threadIdx.x == 0) {
                atomicOr(err, kErrTiledTimeout);
                mbar_wait(&full_bar[0], phase_bits & 1u);
                mbar_wait(&full_bar[1], (phase_bits >> 1) & 1u);
            }
            break;
        }
#pragma unroll
        for (int o = G; o < 32; o <<= 1) {
#pragma unroll
            for (int q = 0; q < V; q++) {
                acc[q].x += __shfl_xor_sync(0xffffffffu, acc[q].x, o);
                acc[q].y += __shfl_xor_sync(0xffffffffu, acc[q].y, o);
                acc[q].z += __shfl_xor_sync(0xffffffffu, acc[q].z, o);
                acc[q].w += __shfl_xor_sync(0xffffffffu, acc[q].w, o);
            }
        }
        if (row < rows && lane < G) {
#pragma unroll
            for (int q = 0; q < V; q++) {
                int c = lane + G * q;
                if (c < r4) store_or_add(out4 + row * r4 + c, acc[q], accumulate);
            }
        }
    }
}

// Any rank (r not a multiple of 4, or r > 1024): one warp per row, lanes stride
// over the r columns, entries taken one at a time.  Correct, not fast.
__global__ void k_spmm_generic(const float* __restrict__ vals, const int32_t* __restrict__ ind,
                               const int64_t* __restrict__ ptr, int64_t rows,
                               const float* __restrict__ D, int r, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int64_t beg = ptr[row], end = ptr[row + 1];
    for (int c0 = 0; c0 < r; c0 += 32) {
        int c = c0 + lane;
        float acc = 0.f;
        for (int64_t p = beg; p < end; p++) {
            float v = vals[p];
            int64_t j = ind[p];
            if (c < r) acc = fmaf(v, D[j * r + c], acc);
        }
        if (c < r) out[row * r + c] = acc;
    }
}

// ---- host-side dispatch ------------------------------------------------------
struct SpmmPlan {
    int32_t* long_list = nullptr;  // device, capacity = rows
    int n_long = 0;                // rows done by the block kernel
    int64_t n_short = 0;           // rows done by the warp kernel
};

inline bool spmm_fast_rank(int r) { return r > 0 && (r % 4) == 0 && r <= 1024; }

// Rows of D per shared-memory tile of the tiled kernel (about 64 KB per buffer).
inline int spmm_tile_rows(int r) {
    int t = 16384 / r;
    if (t < 8) t = 8;
    if (t > 1024) t = 1024;
    return t;
}

enum SpmmKind { kSpmmRows, kSpmmBucketWarp, kSpmmBucketBlock, kSpmmTiled };

struct SpmmCall {
    SpmmKind kind = kSpmmRows;
    const float* vals = nullptr;
    const int32_t* ind = nullptr;
    SegView seg = {nullptr, nullptr, 0, 0};
    int64_t row_first = 0, rows = 0;
    const float* D = nullptr;
    int r = 0;
    float* out = nullptr;
    int accumulate = 0;
    const SpmmPlan* plan = nullptr;      // kSpmmRows
    const uint32_t* row_len = nullptr;   // kSpmmTiled: entries per row to use (NULL: whole row)
    int row_len_stride = 1;
    int64_t d_rows = 0;                  // kSpmmTiled: rows of D that are tiled
    int* work_counter = nullptr;         // kSpmmTiled
    int* err = nullptr;                  // kSpmmTiled
};

template <int G, int V>
inline int spmm_launch_t(const SpmmCall& c, cudaStream_t st) {
    const int r4 = c.r / 4;
    const float4* D4 = (const float4*)c.D;
    float4* out4 = (float4*)c.out;
    size_t red_smem = (size_t)kSpmmWarps * r4 * sizeof(float4);
    switch (c.kind) {
        case kSpmmRows: {
            if (c.plan->n_short > 0) {
                k_spmm_warp<G, V><<<(unsigned)ceil_div(c.rows, kSpmmWarps), kSpmmWarps * 32, 0, st>>>(
                    c.vals, c.ind, c.seg, c.row_first, c.rows, kLongRow, D4, r4, out4, c.accumulate);
                DN_LAUNCH_CHECK();
                DN_COUNT_LAUNCH(1);
            }
            if (c.plan->n_long > 0) {
                k_spmm_block<G, V><<<(unsigned)c.plan->n_long, kSpmmWarps * 32, red_smem, st>>>(
                    c.vals, c.ind, c.seg, c.plan->long_list, 0, c.plan->n_long, D4, r4, out4, c.accumulate);
                DN_LAUNCH_CHECK();
                DN_COUNT_LAUNCH(1);
            }
            break;
        }
        case kSpmmBucketWarp:
            k_spmm_warp<G, V><<<(unsigned)ceil_div(c.rows, kSpmmWarps), kSpmmWarps * 32, 0, st>>>(
                c.vals, c.ind, c.seg, c.row_first, c.rows, INT64_MAX, D4, r4, out4, c.accumulate);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
            break;
        case kSpmmBucketBlock:
            k_spmm_block<G, V><<<(unsigned)c.rows, kSpmmWarps * 32, red_smem, st>>>(
                c.vals, c.ind, c.seg, nullptr, c.row_first, c.rows, D4, r4, out4, c.accumulate);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
            break;
        case kSpmmTiled: {
            int tile_rows = spmm_tile_rows(c.r);
            size_t smem = 2 * (size_t)tile_rows * r4 * sizeof(float4);
            DN_CUDA(cudaFuncSetAttribute(k_spmm_tiled<G, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
            DN_CUDA(cudaMemsetAsync(c.work_counter, 0, sizeof(int), st));
            // Rows per group (= warps per block): the smallest count that lets every
            // SM take the same whole number of groups, so the last round is full.
            constexpr int kMaxWarps = TiledWarps<V>::value;
            int warps = kMaxWarps;
            for (int k = 1; k <= 64; k++) {
                int64_t per = ceil_div(c.rows, (int64_t)kNumSMs * k);
                if (per <= kMaxWarps) { warps = (int)(per < 4 ? 4 : per); break; }
            }
            int64_t groups = ceil_div(c.rows, warps);
            int grid = (int)(groups < kNumSMs ? groups : kNumSMs);
            k_spmm_tiled<G, V><<<grid, warps * 32, smem, st>>>(
                c.vals, c.ind, c.seg.ptr, c.row_len, c.row_len_stride, c.rows, c.D, r4, c.d_rows, tile_rows, out4,
                c.accumulate, c.work_counter, c.err);
            DN_LAUNCH_CHECK();
            DN_COUNT_LAUNCH(1);
            break;
        }
    }
    return DNPEFF_OK;
}

inline int spmm_call(const SpmmCall& c, cudaStream_t st) {
    if (c.rows <= 0) return DNPEFF_OK;
    if (!spmm_fast_rank(c.r)) return fail(DNPEFF_ERR_INVALID, "internal: fast SpMM called with rank %d", c.r);
#define DN_SPMM_CASE(G, V) return spmm_launch_t<G, V>(c, st)
    int r4 = c.r / 4;
    if (c.kind == kSpmmTiled) {
        // Shared-memory gathers: groups of 8 lanes (128 bytes of the tile row per
        // group and load) keep four entries in flight per warp instruction and need
        // a quarter of the shuffles of a whole-warp-per-entry layout; shuffles and
        // shared loads share the pipe that bounds this kernel.
        if (r4 <= 8) DN_SPMM_CASE(8, 1);
        if (r4 <= 16) DN_SPMM_CASE(8, 2);
        if (r4 <= 32) DN_SPMM_CASE(8, 4);
        if (r4 <= 64) DN_SPMM_CASE(8, 8);
        if (r4 <= 128) DN_SPMM_CASE(16, 8);
        DN_SPMM_CASE(32, 8);
    }
    // L2/HBM gathers: one whole row of D per warp-wide 128-bit load where r allows
    // (measured faster than the grouped layout for these).
    if (r4 <= 8) DN_SPMM_CASE(8, 1);
    if (r4 <= 16) DN_SPMM_CASE(16, 1);
    if (r4 <= 32) DN_SPMM_CASE(32, 1);
    if (r4 <= 64) DN_SPMM_CASE(32, 2);
    if (r4 <= 128) DN_SPMM_CASE(32, 4);
    DN_SPMM_CASE(32, 8);
#undef DN_SPMM_CASE
}

// out[rows, r] = S * D over whole rows.  `plan` may be empty (n_long = 0,
// n_short = rows) only if no row is longer than kLongRow.
inline int spmm_dispatch(const float* vals, const int32_t* ind, const int64_t* ptr, int64_t rows,
                         const float* D, int r, float* out, const SpmmPlan& plan,
                         cudaStream_t st) {
    if (rows <= 0) return DNPEFF_OK;
    if (!spmm_fast_rank(r)) {
        k_spmm_generic<<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(vals, ind, ptr, rows, D, r, out);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
        return DNPEFF_OK;
    }
    SpmmCall c;
    c.kind = kSpmmRows;
    c.vals = vals; c.ind = ind;
    c.seg = {ptr, nullptr, 0, 0};
    c.rows = rows; c.D = D; c.r = r; c.out = out; c.plan = &plan;
    return spmm_call(c, st);
}

// Builds the long-row list of rows [row_first, row_first+rows) (allocates
// plan->long_list; synchronises).
inline int spmm_make_plan(const int64_t* ptr, int64_t row_first, int64_t rows, SpmmPlan* plan,
                          cudaStream_t st) {
    plan->n_long = 0;
    plan->n_short = rows;
    if (rows <= 0) return DNPEFF_OK;
    int* d_n = nullptr;
    DN_CUDA(cudaMalloc(&d_n, sizeof(int)));
    if (!plan->long_list) DN_CUDA(cudaMalloc(&plan->long_list, sizeof(int32_t) * (size_t)rows));
    DN_CUDA(cudaMemsetAsync(d_n, 0, sizeof(int), st));
    k_classify_rows<<<(unsigned)ceil_div(rows, 256), 256, 0, st>>>(ptr, row_first, rows, plan->long_list, d_n);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(1);
    int n = 0;
    DN_CUDA(cudaMemcpyAsync(&n, d_n, sizeof(int), cudaMemcpyDeviceToHost, st));
    DN_CUDA(cudaStreamSynchronize(st));
    DN_CUDA(cudaFree(d_n));
    plan->n_long = n;
    plan->n_short = rows - n;
    return DNPEFF_OK;
}

}  // namespace dnpeff
