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
                for (int q = 0; q < V; q++) {
                    int c = l + G * q;
                    h[u][q] = (c < r4) ? __ldg(drow + c) : make_float4(0.f, 0.f, 0.f, 0.f);
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

// Lists the rows longer than kLongRow (once per matrix: the structure is static).
// The list order depends on atomic timing; it only decides which block takes
// which row, never a summation order.
__global__ void k_classify_rows(const int64_t* __restrict__ ptr, int64_t rows,
                                int32_t* __restrict__ long_list, int* __restrict__ n_long) {
    int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row < rows && ptr[row + 1] - ptr[row] > kLongRow)
        long_list[atomicAdd(n_long, 1)] = (int32_t)row;
}

// One warp per row; rows longer than kLongRow are left to the block kernel.
template <int G, int V>
__global__ void __launch_bounds__(kSpmmWarps * 32)
k_spmm_warp(const float* __restrict__ vals, const int32_t* __restrict__ ind,
            const int64_t* __restrict__ ptr, int64_t rows, const float4* __restrict__ D4, int r4,
            float4* __restrict__ out4) {
    const int lane = threadIdx.x & 31;
    int64_t row = (int64_t)blockIdx.x * kSpmmWarps + (threadIdx.x >> 5);
    if (row >= rows) return;
    int64_t beg = ptr[row], end = ptr[row + 1];
    if (end - beg > kLongRow) return;
    float4 acc[V];
#pragma unroll
    for (int q = 0; q < V; q++) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    spmm_accumulate<G, V>(vals, ind, beg, end, 32, D4, r4, acc);
    if (lane < G) {
#pragma unroll
        for (int q = 0; q < V; q++) {
            int c = lane + G * q;
            if (c < r4) out4[row * r4 + c] = acc[q];
        }
    }
}

// One block per listed row.  Dynamic shared memory: kSpmmWarps * r4 float4.
template <int G, int V>
__global__ void __launch_bounds__(kSpmmWarps * 32)
k_spmm_block(const float* __restrict__ vals, const int32_t* __restrict__ ind,
             const int64_t* __restrict__ ptr, const int32_t* __restrict__ long_list, int n_long,
             const float4* __restrict__ D4, int r4, float4* __restrict__ out4) {
    extern __shared__ float4 red[];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (int item = blockIdx.x; item < n_long; item += gridDim.x) {
        int64_t row = long_list[item];
        int64_t beg = ptr[row], end = ptr[row + 1];
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
            out4[row * r4 + c] = s;
        }
        __syncthreads();
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

template <int G, int V>
inline int spmm_launch_t(const float* vals, const int32_t* ind, const int64_t* ptr, int64_t rows,
                         const float* D, int r, float* out, const SpmmPlan& plan,
                         cudaStream_t st) {
    const int r4 = r / 4;
    if (plan.n_short > 0) {
        int64_t blocks = ceil_div(rows, kSpmmWarps);
        k_spmm_warp<G, V><<<(unsigned)blocks, kSpmmWarps * 32, 0, st>>>(
            vals, ind, ptr, rows, (const float4*)D, r4, (float4*)out);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    if (plan.n_long > 0) {
        size_t smem = (size_t)kSpmmWarps * r4 * sizeof(float4);
        k_spmm_block<G, V><<<(unsigned)plan.n_long, kSpmmWarps * 32, smem, st>>>(
            vals, ind, ptr, plan.long_list, plan.n_long, (const float4*)D, r4, (float4*)out);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(1);
    }
    return DNPEFF_OK;
}

inline bool spmm_fast_rank(int r) { return r > 0 && (r % 4) == 0 && r <= 1024; }

// out[rows, r] = S * D.  `plan` may be empty (n_long = 0, n_short = rows) only
// if no row is longer than kLongRow.
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
#define DN_SPMM_CASE(G, V) return spmm_launch_t<G, V>(vals, ind, ptr, rows, D, r, out, plan, st)
    int r4 = r / 4;
    if (r4 <= 8) DN_SPMM_CASE(8, 1);
    if (r4 <= 16) DN_SPMM_CASE(16, 1);
    if (r4 <= 32) DN_SPMM_CASE(32, 1);
    if (r4 <= 64) DN_SPMM_CASE(32, 2);
    if (r4 <= 128) DN_SPMM_CASE(32, 4);
    DN_SPMM_CASE(32, 8);
#undef DN_SPMM_CASE
}

// Builds the long-row list of a matrix (allocates plan->long_list; synchronises).
inline int spmm_make_plan(const int64_t* ptr, int64_t rows, SpmmPlan* plan, cudaStream_t st) {
    plan->n_long = 0;
    plan->n_short = rows;
    if (rows <= 0) return DNPEFF_OK;
    int* d_n = nullptr;
    DN_CUDA(cudaMalloc(&d_n, sizeof(int)));
    if (!plan->long_list) DN_CUDA(cudaMalloc(&plan->long_list, sizeof(int32_t) * (size_t)rows));
    DN_CUDA(cudaMemsetAsync(d_n, 0, sizeof(int), st));
    k_classify_rows<<<(unsigned)ceil_div(rows, 256), 256, 0, st>>>(ptr, rows, plan->long_list, d_n);
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
