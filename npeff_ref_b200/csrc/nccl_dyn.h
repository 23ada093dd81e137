// NCCL bound at run time.  The library is looked up with dlopen the first time
// a communicator is made, so a single-GPU job needs no NCCL at all, and inside
// a process that already loaded an NCCL (for instance through PyTorch) that
// same copy is reused instead of a second one being mapped.
#pragma once
#include <dlfcn.h>
#include <nccl.h>

#include "common.cuh"

namespace dnpeff {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

inline NcclApi& nccl_api() {
    static NcclApi api;
    return api;
}

inline int nccl_load() {
    NcclApi& a = nccl_api();
    if (a.ok) return DNPEFF_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* nm : names) {
        a.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) return fail(DNPEFF_ERR_NCCL, "NCCL not found: %s", dlerror());
#define DN_SYM(field, name)                                                        \
    *(void**)(&a.field) = dlsym(a.handle, name);                                   \
    if (!a.field) return fail(DNPEFF_ERR_NCCL, "NCCL symbol %s missing", name);
    DN_SYM(GetUniqueId, "ncclGetUniqueId")
    DN_SYM(CommInitRank, "ncclCommInitRank")
    DN_SYM(CommDestroy, "ncclCommDestroy")
    DN_SYM(AllReduce, "ncclAllReduce")
    DN_SYM(Broadcast, "ncclBroadcast")
    DN_SYM(Send, "ncclSend")
    DN_SYM(Recv, "ncclRecv")
    DN_SYM(GroupStart, "ncclGroupStart")
    DN_SYM(GroupEnd, "ncclGroupEnd")
    DN_SYM(GetErrorString, "ncclGetErrorString")
#undef DN_SYM
    a.ok = true;
    return DNPEFF_OK;
}

#define DN_NCCL(call)                                                                  \
    do {                                                                               \
        ncclResult_t r_ = (call);                                                      \
        if (r_ != ncclSuccess)                                                         \
            return ::dnpeff::fail(DNPEFF_ERR_NCCL, "%s:%d: %s -> %s", __FILE__, __LINE__, \
                                  #call, ::dnpeff::nccl_api().GetErrorString(r_));     \
    } while (0)

// Inside an ncclGroupStart / ncclGroupEnd section a failed call must not return before
// the group is closed: it records the failure in `status` instead and the later calls
// of the section are skipped.
#define DN_NCCL_IN_GROUP(status, call)                                                        \
    do {                                                                                      \
        if ((status) == DNPEFF_OK) {                                                          \
            ncclResult_t r_ = (call);                                                         \
            if (r_ != ncclSuccess)                                                            \
                (status) = ::dnpeff::fail(DNPEFF_ERR_NCCL, "%s:%d: %s -> %s", __FILE__, __LINE__, \
                                          #call, ::dnpeff::nccl_api().GetErrorString(r_));    \
        }                                                                                     \
    } while (0)

}  // namespace dnpeff
