// Hoyer's sparseness projection of the columns of W (n x r, row-major: component t is
// column t): the closest non-negative vector with a given L1 and L2 norm, for every
// component at once.  Follows the reference's unfinished DenseFactorSparsityContext
// (src/nmf/sparse/dense_factor_sparsity_constraints.h:205-237 for the sequence,
// sparsity_constraint_kernels.h:14-141 for the elementwise rules), which implements
// "Non-negative Matrix Factorization with Sparseness Constraints" (Hoyer 2004, the
// projection operator of section 3.3):
//   s = x + (L1 - sum x)/n;  Y = all ones (1 - Z)
//   repeat
//     m = Y * L1 / size(Y);  s = m + alpha (s - m)  with alpha >= 0 so that |s|_2 = L2
//     finished where no entry of s is negative
//     Y = 0 and s = 0 where s < 0;  s -= (sum s - L1) / size(Y) on the entries left
// Column sums are accumulated in double in a fixed order (the reference: cublasSgemv /
// cublasSgemmStridedBatched in fp32), the elementwise rules in fp32 without
// contraction, so that the result repeats bit for bit and matches a numpy restatement.
#pragma once

#include <cstdint>

#include "common.cuh"

namespace dnpeff {

constexpr int kHoyerThreads = 256;  // 32 column lanes x 8 row lanes

// Per column and block: sum s, sum y, sum s*s, sum s*y over the block's rows.
// partial: [gridDim.x][r][4] doubles.
static __global__ void __launch_bounds__(kHoyerThreads)
k_hoyer_reduce(const float* __restrict__ S, const uint8_t* __restrict__ Y, int64_t n, int r,
               int64_t rows_per_block, double* __restrict__ partial) {
    __shared__ double red[8][32][4];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
    const int64_t row1 = row0 + rows_per_block < n ? row0 + rows_per_block : n;
    for (int c0 = 0; c0 < r; c0 += 32) {
        const int c = c0 + tx;
        double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
        if (c < r) {
            for (int64_t i = row0 + ty; i < row1; i += 8) {
                const double s = (double)S[i * r + c];
                const double y = Y[i * r + c] ? 1.0 : 0.0;
                a0 += s;
                a1 += y;
                a2 += s * s;
                a3 += s * y;
            }
        }
        red[ty][tx][0] = a0;
        red[ty][tx][1] = a1;
        red[ty][tx][2] = a2;
        red[ty][tx][3] = a3;
        __syncthreads();
        if (ty < 4 && c < r) {  // thread (ty, tx) folds quantity ty of column c over the 8 row lanes, in order
            double t = 0;
            for (int k = 0; k < 8; k++) t += red[k][tx][ty];
            partial[((int64_t)blockIdx.x * r + c) * 4 + ty] = t;
        }
        __syncthreads();
    }
}

// col[t][q] = sum over blocks, in block order, as float (what the elementwise rules read).
static __global__ void k_hoyer_fold(const double* __restrict__ partial, int n_blocks, int r, float* __restrict__ col) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= r * 4) return;
    double t = 0;
    for (int b = 0; b < n_blocks; b++) t += partial[(int64_t)b * r * 4 + idx];
    col[idx] = (float)t;
}

// kernel_computeInitialS (sparsity_constraint_kernels.h:14-26): s = x + (L1 - sum x) / n
static __global__ void k_hoyer_init(float* __restrict__ S, uint8_t* __restrict__ Y, int64_t total, int r, float n_f,
                                    const float* __restrict__ col, float l1) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % r);
        S[i] = __fadd_rn(S[i], __fdiv_rn(__fsub_rn(l1, col[c * 4 + 0]), n_f));
        Y[i] = 1;
    }
}

// kernel_computeAlpha (sparsity_constraint_kernels.h:40-68).  rule 0: the non-negative
// root of |m + alpha (s - m)|^2 = L2^2 (the published algorithm); rule 1: the
// reference's expression (L2 sqrt(|s-m|^2) + |m|^2 - <m,s>) / |s-m|^2, which equals
// that root only when m and s - m are parallel.
static __global__ void k_hoyer_alpha(const float* __restrict__ col, int r, float l1, float l2, int rule,
                                     float* __restrict__ alpha) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= r) return;
    const float yy = col[t * 4 + 1], ss = col[t * 4 + 2], sy = col[t * 4 + 3];
    if (!(yy > 0.f)) {  // nothing left of the column: it stays all zero
        alpha[t] = 0.f;
        return;
    }
    const float beta = __fdiv_rn(l1, yy);
    const float m2 = __fmul_rn(__fmul_rn(beta, beta), yy);
    const float ms = __fmul_rn(beta, sy);
    const float d2 = fmaxf(1e-9f, __fsub_rn(__fadd_rn(m2, ss), __fmul_rn(2.0f, ms)));  // |s - m|^2
    if (rule == 1) {
        alpha[t] = __fdiv_rn(__fsub_rn(__fadd_rn(__fmul_rn(l2, __fsqrt_rn(d2)), m2), ms), d2);
    } else {
        const float b = __fsub_rn(ms, m2);                      // <m, s - m>
        const float c = __fsub_rn(m2, __fmul_rn(l2, l2));       // |m|^2 - L2^2
        const float disc = fmaxf(0.f, __fsub_rn(__fmul_rn(b, b), __fmul_rn(d2, c)));
        alpha[t] = __fdiv_rn(__fsub_rn(__fsqrt_rn(disc), b), d2);
    }
}

// kernel_updateSAfterAlpha (sparsity_constraint_kernels.h:71-92) on the active columns,
// with the count of negative entries per column and block (the reference: a float mask
// matrix summed by cublasSgemv).  neg: [gridDim.x][r] ints.
static __global__ void __launch_bounds__(kHoyerThreads)
k_hoyer_step(float* __restrict__ S, const uint8_t* __restrict__ Y, int64_t n, int r, int64_t rows_per_block,
             const float* __restrict__ col, const float* __restrict__ alpha, const int* __restrict__ active, float l1,
             int* __restrict__ neg) {
    __shared__ int red[8][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t row0 = (int64_t)blockIdx.x * rows_per_block;
    const int64_t row1 = row0 + rows_per_block < n ? row0 + rows_per_block : n;
    for (int c0 = 0; c0 < r; c0 += 32) {
        const int c = c0 + tx;
        int cnt = 0;
        if (c < r && active[c]) {
            const float yy = col[c * 4 + 1], al = alpha[c];
            const float mid = yy > 0.f ? __fdiv_rn(l1, yy) : 0.f;
            for (int64_t i = row0 + ty; i < row1; i += 8) {
                const float m = Y[i * r + c] ? mid : 0.f;
                const float s = __fadd_rn(m, __fmul_rn(al, __fsub_rn(S[i * r + c], m)));
                S[i * r + c] = s;
                cnt += s < 0.f;
            }
        }
        red[ty][tx] = cnt;
        __syncthreads();
        if (ty == 0 && c < r) {
            int t = 0;
            for (int k = 0; k < 8; k++) t += red[k][tx];
            neg[(int64_t)blockIdx.x * r + c] = t;
        }
        __syncthreads();
    }
}

// A column stays active while its last step left a negative entry
// (updateAndReadActiveMask, dense_factor_sparsity_constraints.h:343-352).
static __global__ void k_hoyer_active(const int* __restrict__ neg, int n_blocks, int r, int* __restrict__ active,
                                      int* __restrict__ n_active) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= r) return;
    if (active[t]) {
        int s = 0;
        for (int b = 0; b < n_blocks; b++) s += neg[(int64_t)b * r + t];
        active[t] = s > 0;
        if (s > 0) atomicAdd(n_active, 1);
    }
}

// kernel_updateYAndS (sparsity_constraint_kernels.h:95-119)
static __global__ void k_hoyer_clip(float* __restrict__ S, uint8_t* __restrict__ Y, int64_t total, int r,
                                    const int* __restrict__ active) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        if (!active[(int)(i % r)]) continue;
        if (Y[i] && S[i] < 0.f) Y[i] = 0;
        if (!Y[i]) S[i] = 0.f;
    }
}

// kernel_updateSLastStep (sparsity_constraint_kernels.h:122-141): s -= (sum s - L1) / size(Y)
static __global__ void k_hoyer_shift(float* __restrict__ S, const uint8_t* __restrict__ Y, int64_t total, int r,
                                     const float* __restrict__ col, const int* __restrict__ active, float l1) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % r);
        if (active[c] && Y[i]) S[i] = __fsub_rn(S[i], __fdiv_rn(__fsub_rn(col[c * 4 + 0], l1), col[c * 4 + 1]));
    }
}

static __global__ void k_hoyer_set_active(int* active, int r) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < r) active[t] = 1;
}

struct HoyerPlan {
    int n_blocks;
    int64_t rows_per_block;
    size_t bytes;  // device scratch: partial | neg | col | alpha | active | n_active | Y
    size_t off_neg, off_col, off_alpha, off_active, off_count, off_y;
};

inline HoyerPlan hoyer_plan(int64_t n, int r) {
    HoyerPlan p;
    p.n_blocks = (int)std::max<int64_t>(1, std::min<int64_t>(2 * kNumSMs, ceil_div(n, 64)));
    p.rows_per_block = ceil_div(std::max<int64_t>(n, 1), p.n_blocks);
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    size_t o = up((size_t)p.n_blocks * r * 4 * sizeof(double));
    p.off_neg = o;
    o += up((size_t)p.n_blocks * r * sizeof(int));
    p.off_col = o;
    o += up((size_t)r * 4 * sizeof(float));
    p.off_alpha = o;
    o += up((size_t)r * sizeof(float));
    p.off_active = o;
    o += up((size_t)r * sizeof(int));
    p.off_count = o;
    o += 256;
    p.off_y = o;
    o += up((size_t)n * r);
    p.bytes = o;
    return p;
}

// Projects the r columns of S in place.  h_count: page-locked int the loop reads the
// number of active columns through (one stream synchronisation per pass, as the
// reference's isFinishedSync).  Returns the passes made in *passes and whether every
// column finished in *converged (the reference loops without a limit).
inline int hoyer_project(float* S, int64_t n, int r, float l1, float l2, int rule, int max_passes,
                         unsigned char* scratch, const HoyerPlan& p, int* h_count, int* passes, int* converged,
                         cudaStream_t st) {
    double* partial = (double*)scratch;
    int* neg = (int*)(scratch + p.off_neg);
    float* col = (float*)(scratch + p.off_col);
    float* alpha = (float*)(scratch + p.off_alpha);
    int* active = (int*)(scratch + p.off_active);
    int* count = (int*)(scratch + p.off_count);
    uint8_t* Y = scratch + p.off_y;
    const int64_t total = n * r;
    const unsigned eg = (unsigned)std::min<int64_t>(ceil_div(total, 256), (int64_t)kNumSMs * 8);
    const unsigned rg = (unsigned)ceil_div(r, 128);
    auto reduce = [&]() -> int {
        k_hoyer_reduce<<<p.n_blocks, kHoyerThreads, 0, st>>>(S, Y, n, r, p.rows_per_block, partial);
        DN_LAUNCH_CHECK();
        k_hoyer_fold<<<(unsigned)ceil_div(r * 4, 128), 128, 0, st>>>(partial, p.n_blocks, r, col);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(2);
        return DNPEFF_OK;
    };
    *passes = 0;
    *converged = 1;
    if (total == 0) return DNPEFF_OK;
    // set-up: Y = 1 (needed by the first reduction: set before it), s = x + (L1 - sum x)/n
    DN_CUDA(cudaMemsetAsync(Y, 1, (size_t)total, st));
    k_hoyer_set_active<<<rg, 128, 0, st>>>(active, r);
    DN_LAUNCH_CHECK();
    DN_TRY(reduce());
    k_hoyer_init<<<eg, 256, 0, st>>>(S, Y, total, r, (float)n, col, l1);
    DN_LAUNCH_CHECK();
    DN_COUNT_LAUNCH(2);
    *converged = 0;
    for (int pass = 0; pass < max_passes; pass++) {
        DN_TRY(reduce());
        k_hoyer_alpha<<<rg, 128, 0, st>>>(col, r, l1, l2, rule, alpha);
        DN_LAUNCH_CHECK();
        k_hoyer_step<<<p.n_blocks, kHoyerThreads, 0, st>>>(S, Y, n, r, p.rows_per_block, col, alpha, active, l1, neg);
        DN_LAUNCH_CHECK();
        DN_CUDA(cudaMemsetAsync(count, 0, sizeof(int), st));
        k_hoyer_active<<<rg, 128, 0, st>>>(neg, p.n_blocks, r, active, count);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(3);
        DN_CUDA(cudaMemcpyAsync(h_count, count, sizeof(int), cudaMemcpyDeviceToHost, st));
        DN_CUDA(cudaStreamSynchronize(st));
        *passes = pass + 1;
        if (*h_count == 0) {
            *converged = 1;
            break;
        }
        k_hoyer_clip<<<eg, 256, 0, st>>>(S, Y, total, r, active);
        DN_LAUNCH_CHECK();
        DN_TRY(reduce());
        k_hoyer_shift<<<eg, 256, 0, st>>>(S, Y, total, r, col, active, l1);
        DN_LAUNCH_CHECK();
        DN_COUNT_LAUNCH(2);
    }
    return DNPEFF_OK;
}

}  // namespace dnpeff
