// Shared host/device helpers of the D-NPEFF engine (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <atomic>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>

#include "../../include/dnpeff.h"

namespace dnpeff {

// ---- error plumbing -------------------------------------------------------
// The reference terminates the process on any failure
// (src/cuda/cuda_statuses.h:15-38); here every failure becomes a status code
// plus a thread-local message.
inline char* err_buf() {
    static thread_local char buf[1024] = {0};
    return buf;
}

inline int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), 1024, fmt, ap);
    va_end(ap);
    return code;
}

#define DN_CUDA(call)                                                                     \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return ::dnpeff::fail(DNPEFF_ERR_CUDA, "%s:%d: %s -> %s", __FILE__, __LINE__, \
                                  #call, cudaGetErrorString(e_));                         \
    } while (0)

#define DN_TRY(call)             \
    do {                         \
        int s_ = (call);         \
        if (s_ != DNPEFF_OK) return s_; \
    } while (0)

#define DN_LAUNCH_CHECK() DN_CUDA(cudaGetLastError())

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Counts the kernel launches this library makes (reported by the bench).
inline std::atomic<int64_t>& launch_counter() {
    static std::atomic<int64_t> c{0};
    return c;
}
#define DN_COUNT_LAUNCH(n) (::dnpeff::launch_counter() += (n))

// ---- counter-based uniform generator --------------------------------------
// Same integer hash as the CPU checker uses, so a seeded initialisation is
// bit-identical on both sides.  The reference draws cuRAND XORWOW uniforms in
// (0,1] (multi_mu_dense_factors_device_contexts1.h:197-207); the (0,1] range is
// kept, the generator is replaced by one that does not depend on the sharding.
__host__ __device__ inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__host__ __device__ inline uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return mix64(seed ^ (stream * 0xD1B54A32D192ED03ull));
}

__host__ __device__ inline float uniform01_from_key(uint64_t key, uint64_t index) {
    uint64_t h = mix64(key + index);
    return (float)((uint32_t)(h >> 40) + 1u) * (1.0f / 16777216.0f);
}

// ---- warp / block reductions -----------------------------------------------
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a block of up to 1024 threads; result valid in thread 0.
// Fixed combination order, so the result does not vary run to run.
__device__ __forceinline__ double block_sum(double v, double* smem32) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[w] = v;
    __syncthreads();
    double t = 0.0;
    if (w == 0) {
        int nw = (blockDim.x + 31) >> 5;
        t = lane < nw ? smem32[lane] : 0.0;
        t = warp_sum(t);
    }
    return t;
}

}  // namespace dnpeff
