// Allocation-free Gram entry point (see dnpeff_op_gram_noalloc in include/dnpeff.h).
//
// Some hosts may not allocate device memory when they call into this library:
// a plugin running inside another framework's memory pool, a real-time loop
// with a fixed memory budget, or code running where cudaMalloc would
// synchronise the device.  For them the slab partials of the Gram kernel live
// in a fixed array that is part of the loaded module instead of a buffer from
// cudaMalloc.
//
// The array's name is only a host-side handle in host code; the address the
// kernels need comes from cudaGetSymbolAddress, looked up once per device (with
// that device current) on the first call made on it.  Under CUDA's lazy module
// loading that first lookup may be what loads this module onto the device: the
// 16 MiB array is materialised then, and the load can synchronise the device.
// Every later call on that device neither allocates nor synchronises.
#include <mutex>

#include "common.cuh"
#include "kernels_dense.cuh"

using namespace dnpeff;

namespace {

constexpr size_t kNoAllocScratchFloats = (size_t)DNPEFF_NOALLOC_SCRATCH_BYTES / sizeof(float);

// 16 MiB per device that loads the library, held until the process exits.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Resolves the device address of the static array for the current device.
int scratch_for_current_device(float** out) {
    int dev = -1;
    DN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(DNPEFF_ERR_UNSUPPORTED, "device ordinal %d", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();  // the failed lookup must not surface again in a later, unrelated call
            return fail(DNPEFF_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev,
                        cudaGetErrorString(e));
        }
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return DNPEFF_OK;
}

}  // namespace

extern "C" int dnpeff_op_gram_noalloc(const float* X, int64_t rows, int32_t r, float* G,
                                      void* stream) {
    if (rows < 0 || r <= 0 || !G || (rows > 0 && !X)) return fail(DNPEFF_ERR_INVALID, "bad argument");
    if (r > DNPEFF_NOALLOC_MAX_RANK)
        return fail(DNPEFF_ERR_UNSUPPORTED,
                    "rank %d exceeds the allocation-free limit of %d (use dnpeff_op_gram)", (int)r,
                    DNPEFF_NOALLOC_MAX_RANK);
    GramPlan g = gram_plan(rows, r);
    // Same slab split as dnpeff_op_gram while it fits the fixed array; otherwise
    // fewer, longer slabs (identical maths, a different but still fixed order).
    size_t per_slab = (size_t)g.npairs * g.tile * g.tile;
    if (per_slab > kNoAllocScratchFloats)
        return fail(DNPEFF_ERR_UNSUPPORTED, "rank %d needs %zu scratch floats per slab, limit %zu",
                    (int)r, per_slab, kNoAllocScratchFloats);
    if (g.scratch_floats > kNoAllocScratchFloats) {
        int nslab = (int)(kNoAllocScratchFloats / per_slab);
        g.rows_per_slab = ceil_div(ceil_div(rows, nslab), kGramBK) * kGramBK;
        g.nslab = (int)ceil_div(rows, g.rows_per_slab);
        g.scratch_floats = (size_t)g.nslab * per_slab;
    }
    float* scratch = nullptr;
    DN_TRY(scratch_for_current_device(&scratch));
    // Every partial tile is written in full before it is read, so nothing in the
    // shared array has to be cleared between calls.
    return gram_launch_plan(X, rows, r, G, scratch, g, (cudaStream_t)stream);
}
