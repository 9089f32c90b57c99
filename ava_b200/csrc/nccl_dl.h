// NCCL reached at run time (dlopen), so that the engine's library links against nothing but the CUDA runtime: a host
// program that never splits a sequence over GPUs needs no NCCL at all.  Only the handful of entry points the split
// step uses are looked up; the types below restate NCCL's public ABI for them (nccl.h: ncclComm_t is an opaque pointer,
// ncclUniqueId 128 bytes, ncclResult_t and ncclDataType_t ints with ncclSuccess = 0 and ncclFloat32 = 7).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

namespace ava {

struct NcclUniqueId { char internal[128]; };

struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId*);
    int (*CommInitRank)(void** comm, int nranks, NcclUniqueId id, int rank);
    int (*CommDestroy)(void* comm);
    int (*Broadcast)(const void* send, void* recv, size_t count, int dtype, int root, void* comm, cudaStream_t st);
    int (*AllGather)(const void* send, void* recv, size_t sendcount, int dtype, void* comm, cudaStream_t st);
    const char* (*GetErrorString)(int);
    int (*GetVersion)(int*);
    // Optional (null when the library has none): the communicator's asynchronous error state, and the abort that ends
    // its kernels in flight.
    int (*CommGetAsyncError)(void* comm, int* async_error);
    int (*CommAbort)(void* comm);
};
constexpr int NCCL_IN_PROGRESS = 7;
constexpr int NCCL_FLOAT32 = 7;

// nullptr when no NCCL library could be loaded (why: nccl_dl_error()).  The library named by AVA_NCCL_LIB is tried
// first, then libnccl.so.2 (a copy already loaded into the process, e.g. by a host framework, is the one found).
const NcclApi* nccl_api();
const char* nccl_dl_error();

}  // namespace ava
