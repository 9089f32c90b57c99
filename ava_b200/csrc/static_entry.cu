// One entry point that allocates nothing, for callers that cannot call cudaMalloc.
//
// Who that is: code that runs where device allocation is forbidden or would stall everything else — a latency-critical
// service thread that must not take the allocator's device-wide lock (cudaMalloc and cudaFree synchronise the whole
// device), or a process whose GPU memory was handed out in full at start-up (a serving runtime that owns the whole GPU
// and gives its plug-ins fixed buffers).  Such a caller already holds its inputs and outputs in device memory and only
// needs the fast-weight update + read done on them.
//
// ava_mem_heads_static is ava_op_mem_heads (update + read of m independent fast-weight heads) with two differences:
// every pointer is DEVICE memory, and the kernel's scratch (the slice-major copy of the heads it works on, plus its
// status word) lives in a file-scope __device__ array of fixed size instead of a fresh allocation.  Consequences a
// user must know:
//   * the array is part of the library image: every GPU that loads the library holds AVA_STATIC_SCRATCH_BYTES (16 MiB)
//     until the process exits;
//   * m * hs * hs may not exceed AVA_STATIC_SCRATCH_FLOATS; larger calls are refused with AVA_ERR_CAPACITY;
//   * every call on a device shares the one array and it keeps the last call's contents: the entry point overwrites
//     all it reads and clears its status word itself, but two calls that overlap on the GPU (different streams, or
//     different host threads) race on it.  Serialise them;
//   * the first call on each device looks the array's device address up (cudaGetSymbolAddress, with that device
//     current).  Make that first call before any stream capture begins;
//   * the kernel fetches e, v, w, ah, qg and ex with bulk copies, which need 16-byte-aligned addresses: a pointer into
//     the middle of a larger buffer must keep that alignment, or the call is refused with AVA_ERR_ARG before anything
//     is launched (f, y, qw and qa need only their natural 4-byte alignment);
//   * the call makes `device` the calling thread's current device and leaves it so, and it returns only after `stream`
//     has drained (it reads the kernel's status word back).
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/ava_engine.h"
#include "kernels.cuh"

namespace {

constexpr size_t SCRATCH_FLOATS = AVA_STATIC_SCRATCH_FLOATS;

// In host code these names are host-side stand-ins, not device addresses: they are only ever handed to
// cudaGetSymbolAddress below, never to a kernel.
static __device__ __align__(256) float g_scratch[SCRATCH_FLOATS];
static __device__ __align__(256) uint32_t g_status_word[64];

constexpr int MAX_DEVICES = 64;
struct PerDevice {
    float* scratch = nullptr;
    uint32_t* status = nullptr;
};
PerDevice g_dev[MAX_DEVICES];

thread_local std::string g_static_error;

int fail(int code, const std::string& msg) {
    g_static_error = msg;
    return code;
}

// once per device, with that device current
int set_up(int device, PerDevice** out) {
    PerDevice& d = g_dev[device];
    if (!d.scratch) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);
        if (e != cudaSuccess) return fail(AVA_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        void* s = nullptr;
        e = cudaGetSymbolAddress(&s, g_status_word);
        if (e != cudaSuccess) return fail(AVA_ERR_CUDA, std::string("cudaGetSymbolAddress(status): ") + cudaGetErrorString(e));
        d.status = static_cast<uint32_t*>(s);
        d.scratch = static_cast<float*>(p);
    }
    *out = &d;
    return AVA_OK;
}

}  // namespace

extern "C" {

const char* ava_static_last_error(void) { return g_static_error.c_str(); }

int ava_mem_heads_static(int device, void* stream, int32_t m, int32_t hs, const float* e, const float* v, const float* w, const float* ah,
                         const float* qg, const float* ex, const float* qw, const float* qa, float* f, float* y) {
    using namespace ava;
    if (!e || !v || !w || !ah || !qg || !ex || !qw || !qa || !f || !y || m <= 0 || hs <= 0) return fail(AVA_ERR_ARG, "null pointer or non-positive size");
    int cw = 0, chunk_rows = 0;
    if (hs % 16 || !mem_heads_tiling(hs, &cw, &chunk_rows)) return fail(AVA_NOT_APPLICABLE, "head size not covered (a multiple of 16 whose column slice fits shared memory)");
    const size_t need = (size_t)m * hs * hs;
    if (need > SCRATCH_FLOATS)
        return fail(AVA_ERR_CAPACITY, "ava_mem_heads_static: " + std::to_string(m) + " heads of " + std::to_string(hs) + " x " + std::to_string(hs) +
                                          " need " + std::to_string(need) + " floats of scratch; the built-in array holds " +
                                          std::to_string(SCRATCH_FLOATS) + " (use ava_op_mem_heads or an engine state for more)");
    // the kernel's bulk copies fault on a source that is not 16-byte aligned, and a fault would end the caller's context
    const void* bulk[6] = {e, v, w, ah, qg, ex};
    static const char* const bulk_name[6] = {"e", "v", "w", "ah", "qg", "ex"};
    for (int i = 0; i < 6; ++i)
        if (reinterpret_cast<uintptr_t>(bulk[i]) & 15)
            return fail(AVA_ERR_ARG, std::string("ava_mem_heads_static: ") + bulk_name[i] + " must be 16-byte aligned (the kernel reads it with bulk copies)");
    if ((hs * sizeof(float)) % 16) return fail(AVA_ERR_ARG, "ava_mem_heads_static: rows of hs floats must be a multiple of 16 bytes");
    const void* word[4] = {qw, qa, f, y};
    for (int i = 0; i < 4; ++i)
        if (reinterpret_cast<uintptr_t>(word[i]) & 3) return fail(AVA_ERR_ARG, "ava_mem_heads_static: qw, qa, f and y must be 4-byte aligned");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count || device >= MAX_DEVICES)
        return fail(AVA_ERR_CUDA, "no such CUDA device (this library has no CPU path)");
    cudaError_t ce = cudaSetDevice(device);
    if (ce != cudaSuccess) return fail(AVA_ERR_CUDA, cudaGetErrorString(ce));
    PerDevice* d = nullptr;
    int rc = set_up(device, &d);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // the status word must start at zero; the scratch itself is overwritten in full before it is read
    if ((ce = cudaMemsetAsync(d->status, 0, sizeof(uint32_t), st)) != cudaSuccess) return fail(AVA_ERR_CUDA, cudaGetErrorString(ce));
    launch_retile(st, f, d->scratch, m, hs, cw, 1);
    MemHeadsArgs a{};
    a.f = d->scratch;
    a.M = m; a.nh = 1; a.hs = hs; a.cw = cw; a.chunk_rows = chunk_rows;
    a.e = e; a.v = v; a.w = w; a.ah = ah; a.qg = qg; a.ex = ex; a.qw = qw; a.qa = qa;
    a.y = y;
    a.status = d->status;
    launch_mem_heads_seq(st, a, 1);
    launch_retile(st, d->scratch, f, m, hs, cw, 0);
    if ((ce = cudaGetLastError()) != cudaSuccess) return fail(AVA_ERR_CUDA, std::string("launch: ") + cudaGetErrorString(ce));
    uint32_t status = 0;
    if ((ce = cudaMemcpyAsync(&status, d->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, st)) != cudaSuccess ||
        (ce = cudaStreamSynchronize(st)) != cudaSuccess)
        return fail(AVA_ERR_CUDA, cudaGetErrorString(ce));
    if (status) return fail(AVA_ERR_CUDA, "a bounded wait on a bulk-copy barrier ran out inside the memory kernel");
    return AVA_OK;
}

}  // extern "C"
