// Synthetic D-PEF generator on the device (benchmark / test support; the
// reference has no counterpart: it reads real D-PEF files written by
// npeff/fishers/d_pefs_computer.py).  It fills the two arrays a D-PEF file
// holds -- data/fisher/values [n,k] and data/fisher/indices [n,k] -- plus
// data/dense_fisher_norms [n], directly in HBM:
//   * column popularity p_c ~ (c+1)^-alpha over m columns (Zipf);
//   * each row holds k DISTINCT columns, drawn by successive sampling with
//     rejection of repeats (inverse-CDF draws against a per-block bitmap);
//   * values are g^2 * s_row, g ~ N(0,1), s_row ~ LogNormal(0, sigma), laid
//     out in descending order like tf.math.top_k leaves them
//     (d_pefs_computer.py:127-129): the sorted chi-square(1) sample is generated
//     directly as order statistics (exponential spacings), no sort needed;
//   * the norm is the L2 norm of the row's values.
#include <math.h>

#include <vector>

#include "../../include/dnpeff_synth.h"
#include "common.cuh"

using namespace dnpeff;

namespace {

constexpr int kSynthThreads = 1024;
constexpr uint64_t kSynthMaxRounds = 1ull << 15;

__device__ __forceinline__ double u01_open(uint64_t h) {  // (0,1]
    return (double)((h >> 11) + 1ull) * (1.0 / 9007199254740992.0);
}

// Bijection on [0, 2^bits): two multiply-add / xorshift rounds.
__device__ __forceinline__ uint32_t perm_bits(uint32_t x, int bits, uint32_t key) {
    uint32_t mask = (bits >= 32) ? 0xffffffffu : ((1u << bits) - 1u);
    int half = bits > 1 ? bits / 2 : 1;
    x = (x * 0x9E3779B1u + key) & mask;
    x ^= x >> half;
    x = (x * 0x85EBCA6Bu + (key >> 7) * 2u + 1u) & mask;
    x ^= x >> half;
    return x & mask;
}

__global__ void __launch_bounds__(kSynthThreads)
k_synth_rows(int64_t row_first, int64_t n, int64_t m, int k, const double* __restrict__ cdf, double sigma,
             uint64_t seed, uint32_t* __restrict__ bitmaps, int64_t bitmap_words,
             int32_t* __restrict__ claimed_all, float* __restrict__ out_vals,
             int32_t* __restrict__ out_idx, float* __restrict__ out_norms) {
    __shared__ int s_count;
    __shared__ int s_warp[32];
    __shared__ int s_newcols[kSynthThreads];
    __shared__ double s_red[32];
    __shared__ double s_scan[32];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    uint32_t* bitmap = bitmaps + (int64_t)blockIdx.x * bitmap_words;
    int32_t* claimed = claimed_all + (int64_t)blockIdx.x * k;
    int bits = 1;
    while ((1ll << bits) < k) bits++;

    // output row `row` is row row_first + row of the matrix: its draws depend on that index only
    for (int64_t row = blockIdx.x; row < n; row += gridDim.x) {
        const uint64_t rkey = mix64(stream_key(seed, 2) + (uint64_t)(row_first + row));
        if (tid == 0) s_count = 0;
        __syncthreads();
        // ---- k distinct columns --------------------------------------------
        for (uint64_t round = 0;; round++) {
            int count = s_count;
            if (count >= k) break;
            if (round >= kSynthMaxRounds) {
                // Bounded: the draws are not finding the last unclaimed columns
                // (k close to n_cols); take the lowest-numbered free ones instead.
                if (tid == 0) {
                    for (int64_t c = 0; c < m && count < k; c++) {
                        uint32_t b = 1u << (c & 31);
                        if (!(bitmap[c >> 5] & b)) {
                            bitmap[c >> 5] |= b;
                            count++;
                        }
                    }
                    s_count = count;
                }
                __syncthreads();
                break;
            }
            uint64_t h = mix64(rkey + round * kSynthThreads + tid + 0x1234567ull);
            double u = u01_open(h) * cdf[m - 1];
            // first c with cdf[c] >= u
            int64_t lo = 0, hi = m - 1;
            while (lo < hi) {
                int64_t mid = (lo + hi) >> 1;
                if (cdf[mid] >= u) hi = mid; else lo = mid + 1;
            }
            int c = (int)lo;
            uint32_t bit = 1u << (c & 31);
            uint32_t old = atomicOr(bitmap + (c >> 5), bit);
            bool isnew = !(old & bit);
            unsigned bal = __ballot_sync(0xffffffffu, isnew);
            if (lane == 0) s_warp[wid] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
            for (int i = 0; i < kSynthThreads / 32; i++) {
                int t = s_warp[i];
                before += (i < wid) ? t : 0;
                total += t;
            }
            if (count + total > k) {
                // Last round overshoots: keep the (k - count) new columns with the
                // smallest keyed hash.  The set of new columns of a round does not
                // depend on which thread won a repeated draw, so neither does this.
                int slot = before + __popc(bal & ((1u << lane) - 1u));
                if (isnew) s_newcols[slot] = c;
                __syncthreads();
                if (isnew) {
                    uint64_t mine = mix64(rkey ^ (uint64_t)c);
                    int rank = 0;
                    for (int i = 0; i < total; i++) {
                        int o = s_newcols[i];
                        uint64_t hv = mix64(rkey ^ (uint64_t)o);
                        rank += (hv < mine || (hv == mine && o < c)) ? 1 : 0;
                    }
                    if (rank >= k - count) atomicAnd(bitmap + (c >> 5), ~bit);
                }
                total = k - count;
            }
            __syncthreads();
            if (tid == 0) s_count = count + total;
            __syncthreads();
        }
        // ---- the claimed set in ascending column order (read back from the bitmap,
        //      which is cleared on the way): independent of any thread timing --------
        {
            int64_t wpt = (bitmap_words + kSynthThreads - 1) / kSynthThreads;
            int64_t w0 = (int64_t)tid * wpt;
            int64_t w1 = w0 + wpt < bitmap_words ? w0 + wpt : bitmap_words;
            int cnt = 0;
            for (int64_t w = w0; w < w1; w++) cnt += __popc(bitmap[w]);
            int inc = cnt;
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += t;
            }
            __syncthreads();
            if (lane == 31) s_warp[wid] = inc;
            __syncthreads();
            int base = inc - cnt;
            for (int i = 0; i < wid; i++) base += s_warp[i];
            for (int64_t w = w0; w < w1; w++) {
                uint32_t bitsw = bitmap[w];
                if (bitsw) bitmap[w] = 0u;
                while (bitsw) {
                    int b = __ffs(bitsw) - 1;
                    claimed[base++] = (int)(w * 32 + b);
                    bitsw &= bitsw - 1u;
                }
            }
            __syncthreads();
        }
        // ---- values: descending order statistics of k chi-square(1) draws ---
        double zu1 = u01_open(mix64(rkey + 0xABCDEFull)), zu2 = u01_open(mix64(rkey + 0xFEDCBAull));
        double z = sqrt(-2.0 * log(zu1)) * cos(6.283185307179586 * zu2);
        double srow = exp(sigma * z);
        int per = (k + kSynthThreads - 1) / kSynthThreads;
        int j0 = tid * per, j1 = min(k, j0 + per);
        double local = 0.0;
        for (int j = j0; j < j1; j++) {
            double e = -log(u01_open(mix64(rkey ^ (0x5555ull << 32) ^ (uint64_t)(j + 1) * 0x9E3779B97F4A7C15ull)));
            local += e / (double)(k - j);
        }
        // exclusive block scan of `local`
        double inc = local;
        for (int o = 1; o < 32; o <<= 1) {
            double t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) s_scan[wid] = inc;
        __syncthreads();
        if (wid == 0) {
            double x = s_scan[lane], xi = x;
            for (int o = 1; o < 32; o <<= 1) {
                double t = __shfl_up_sync(0xffffffffu, xi, o);
                if (lane >= o) xi += t;
            }
            s_scan[lane] = xi - x;
        }
        __syncthreads();
        double run = s_scan[wid] + inc - local;
        double sq = 0.0;
        for (int j = j0; j < j1; j++) {
            double e = -log(u01_open(mix64(rkey ^ (0x5555ull << 32) ^ (uint64_t)(j + 1) * 0x9E3779B97F4A7C15ull)));
            run += e / (double)(k - j);
            double surv = -expm1(-run);      // P(X > x) for this order statistic
            double q = erfcinv(surv);
            double x = 2.0 * q * q * srow;
            float xf = (float)x;
            // column: a keyed permutation of the claim order (cycle-walk into [0,k))
            uint32_t pj = (uint32_t)j;
            do { pj = perm_bits(pj, bits, (uint32_t)(rkey >> 17)); } while (pj >= (uint32_t)k);
            out_vals[row * k + j] = xf;
            out_idx[row * k + j] = claimed[pj];
            sq += (double)xf * (double)xf;
        }
        double tot = block_sum(sq, s_red);
        if (tid == 0) out_norms[row] = (float)sqrt(tot);
        __syncthreads();
    }
}

}  // namespace

extern "C" int dnpeff_synth_pef_device(int64_t n_rows, int64_t n_cols, int64_t k_per_row,
                                       double alpha, double sigma, uint64_t seed, float* d_vals,
                                       int32_t* d_idx, float* d_norms, void* stream) {
    return dnpeff_synth_pef_device_rows(0, n_rows, n_cols, k_per_row, alpha, sigma, seed, d_vals, d_idx, d_norms,
                                        stream);
}

extern "C" int dnpeff_synth_pef_device_rows(int64_t row_first, int64_t n_rows, int64_t n_cols, int64_t k_per_row,
                                            double alpha, double sigma, uint64_t seed, float* d_vals,
                                            int32_t* d_idx, float* d_norms, void* stream) {
    if (row_first < 0 || n_rows < 0 || n_cols <= 0 || k_per_row <= 0 || k_per_row > n_cols || k_per_row > (1 << 30))
        return fail(DNPEFF_ERR_INVALID, "bad synthetic shape (need 0 < k <= n_cols)");
    if (n_cols >= INT32_MAX) return fail(DNPEFF_ERR_UNSUPPORTED, "n_cols must fit int32");
    if (n_rows == 0) return DNPEFF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    std::vector<double> cdf((size_t)n_cols);
    double acc = 0.0;
    for (int64_t c = 0; c < n_cols; c++) {
        acc += pow((double)(c + 1), -alpha);
        cdf[(size_t)c] = acc;
    }
    double* d_cdf = nullptr;
    uint32_t* d_bitmaps = nullptr;
    int32_t* d_claimed = nullptr;
    int grid = (int)(n_rows < 2 * kNumSMs ? n_rows : 2 * kNumSMs);
    int64_t words = (n_cols + 31) / 32;
    int status = DNPEFF_OK;
    do {
        if (cudaMalloc((void**)&d_cdf, sizeof(double) * (size_t)n_cols) != cudaSuccess ||
            cudaMalloc((void**)&d_bitmaps, sizeof(uint32_t) * (size_t)(words * grid)) != cudaSuccess ||
            cudaMalloc((void**)&d_claimed, sizeof(int32_t) * (size_t)(k_per_row * grid)) != cudaSuccess) {
            status = fail(DNPEFF_ERR_CUDA, "cudaMalloc failed in the synthetic generator");
            break;
        }
        cudaMemcpyAsync(d_cdf, cdf.data(), sizeof(double) * (size_t)n_cols, cudaMemcpyHostToDevice, st);
        cudaMemsetAsync(d_bitmaps, 0, sizeof(uint32_t) * (size_t)(words * grid), st);
        k_synth_rows<<<grid, kSynthThreads, 0, st>>>(row_first, n_rows, n_cols, (int)k_per_row, d_cdf, sigma, seed,
                                                    d_bitmaps, words, d_claimed, d_vals, d_idx, d_norms);
        DN_COUNT_LAUNCH(1);
        cudaError_t e = cudaStreamSynchronize(st);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) status = fail(DNPEFF_ERR_CUDA, "synthetic generator: %s", cudaGetErrorString(e));
    } while (0);
    cudaFree(d_cdf);
    cudaFree(d_bitmaps);
    cudaFree(d_claimed);
    return status;
}
