// b200_reduce_full_noalloc: the whole-tensor reduction of b200_reduce_full for
// callers that must not allocate device memory.
//
// Some users of this library run where a cudaMalloc is not allowed at call
// time: inside a framework's memory pool that owns the whole device, inside a
// real-time loop that may not take the allocator lock, or after the process
// has handed all free memory to another component.  Everything else in the
// library either allocates (the arena, the op-tree backend's scratch) or asks
// the caller for scratch space.  This entry point does neither: the partial
// results and the arrival counter of the split reduction live in a fixed array
// that is part of the library image, so each GPU that loads the library carries
// kNoAllocScratchBytes of it until the process exits.
//
// The kernel and the launch geometry are exactly those of b200_reduce_full
// (b200_detail_reduce_full in kernels.cu); only where the scratch comes from
// differs.

#include "b200ew.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

extern "C" int b200_detail_reduce_full(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                                       uint64_t out, uint64_t scratch, int sm_count, void* stream);
extern "C" void* b200_detail_stream(uint64_t stream);
extern "C" int32_t b200_detail_fail(int32_t code, const char* message);

namespace {

// counter block (256 bytes) + one fp32 partial per block of the split (at most 4096)
enum { kNoAllocScratchBytes = 256 + 4 * 4096, kMaxDevices = 64 };

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol table, not an address a kernel could use: the device address is looked
// up with cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

struct PerDevice {
    void* scratch = nullptr;     // device address of g_noalloc_scratch on this device
    int sm_count = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_dev_mu;

}  // namespace

extern "C" uint64_t b200_reduce_full_noalloc_max_count(void) { return B200_NOALLOC_MAX_COUNT; }

extern "C" b200_status b200_reduce_full_noalloc(uint64_t in, int32_t dtype, uint64_t count, int32_t op,
                                               int32_t absolute, uint64_t out, uint64_t stream) {
    if (!in || !out) return b200_detail_fail(B200_ERR_INVALID, "b200_reduce_full_noalloc: null device pointer");
    if (!count) return b200_detail_fail(B200_ERR_INVALID, "b200_reduce_full_noalloc: empty input");
    if (count > B200_NOALLOC_MAX_COUNT) {
        char msg[160];
        snprintf(msg, sizeof msg, "b200_reduce_full_noalloc: %llu elements exceed the supported maximum of %llu; "
                 "use b200_reduce_full with caller-provided scratch",
                 (unsigned long long)count, (unsigned long long)B200_NOALLOC_MAX_COUNT);
        return b200_detail_fail(B200_ERR_INVALID, msg);
    }
    if (dtype != B200_F32 && dtype != B200_F16 && dtype != B200_BF16)
        return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_reduce_full_noalloc: only f32, f16 and bf16 inputs");
    if (op != B200_SUM && op != B200_MAX && op != B200_MIN)
        return b200_detail_fail(B200_ERR_INVALID, "b200_reduce_full_noalloc: bad reduction op");

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return b200_detail_fail(B200_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return b200_detail_fail(B200_ERR_UNSUPPORTED, "device ordinal out of range");

    PerDevice& d = g_dev[dev];
    std::lock_guard<std::mutex> lock(g_dev_mu);      // two host threads may make the first call together
    if (!d.scratch) {
        // first call on this device (it is the current one): resolve the array's device address
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return b200_detail_fail(B200_ERR_CUDA, e != cudaSuccess ? cudaGetErrorString(e)
                                                                    : "cudaGetSymbolAddress returned null");
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return b200_detail_fail(B200_ERR_CUDA, cudaGetErrorString(e));
        d.sm_count = sms;
        d.scratch = p;
    }

    cudaStream_t s = static_cast<cudaStream_t>(b200_detail_stream(stream));
    // the array keeps whatever the previous call left: the arrival counter must start at zero
    e = cudaMemsetAsync(d.scratch, 0, 256, s);
    if (e != cudaSuccess) return b200_detail_fail(B200_ERR_CUDA, cudaGetErrorString(e));
    int r = b200_detail_reduce_full(in, dtype, count, op, absolute, out,
                                    reinterpret_cast<uint64_t>(d.scratch), d.sm_count, s);
    if (r) return b200_detail_fail(B200_ERR_CUDA, cudaGetErrorString(static_cast<cudaError_t>(r)));
    return B200_OK;
}
