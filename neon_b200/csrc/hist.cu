// b200_log2_hist: histogram of round(log2(|x|)) over a tensor, the device side of
// GPUTensor.hist (neon/backends/nervanagpu.py:619-637; kernel text and launch in
// neon/backends/float_ew.py:1069-1158), which neon's histogram callback uses to watch the
// dynamic range of activations and weights.  Bin b counts the elements with
// round(log2|x|) - offset == b, clamped to [0, nbins - 1]; zero lands in bin 0, infinity in
// the last bin, NaN in bin 0 (what the reference's MIN/MAX macros and float -> int
// conversion make of them).  The histogram (nbins int32) is zeroed by the call.
//
// One pass over the data with 16-byte loads, counts kept per block in shared memory
// (one copy per warp to keep atomics off each other) and added to the result once per
// block.  HBM bound: the element size per element.

#include "b200ew.h"
#include "optree_templates.cuh"

#include <cuda_runtime.h>

#include <cstdio>

extern "C" void* b200_detail_stream(uint64_t stream);
extern "C" int32_t b200_detail_fail(int32_t code, const char* message);

namespace {

enum { kMaxBins = B200_HIST_MAX_BINS, kWarps = 8 };

struct HP {
    u64 in, hist;
    i64 nvec, count;         // whole vectors, then a scalar tail up to count
    int nbins, offset;
};

__device__ __forceinline__ int hist_bin(float a, int nbins, float offset) {
    const float t = roundf(log2f(fabsf(a))) - offset;
    return !(t > 0.f) ? 0 : (t < (float)(nbins - 1) ? (int)t : nbins - 1);
}

template <int DT, int V>
__global__ void __launch_bounds__(32 * kWarps) hist_kernel(const __grid_constant__ HP p) {
    using namespace b200;
    __shared__ int s[kWarps][kMaxBins];
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < kWarps * kMaxBins; i += 32 * kWarps) (&s[0][0])[i] = 0;
    __syncthreads();
    const float off = (float)p.offset;
    const i64 step = (i64)gridDim.x * blockDim.x;
    for (i64 v = (i64)blockIdx.x * blockDim.x + tid; v < p.nvec; v += step) {
        float a[V];
        ld_f<DT, V, true>(p.in, v * V, a);
#pragma unroll
        for (int i = 0; i < V; ++i) atomicAdd(&s[warp][hist_bin(a[i], p.nbins, off)], 1);
    }
    if (blockIdx.x == 0) {                              // the elements after the last whole vector
        for (i64 n = p.nvec * V + tid; n < p.count; n += blockDim.x) {
            float a[1];
            ld_f<DT, 1, true>(p.in, n, a);
            atomicAdd(&s[warp][hist_bin(a[0], p.nbins, off)], 1);
        }
    }
    __syncthreads();
    for (int b = tid; b < p.nbins; b += blockDim.x) {
        int c = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) c += s[w][b];
        if (c) atomicAdd(reinterpret_cast<int*>(p.hist) + b, c);
    }
}

template <int DT>
cudaError_t launch(const HP& p0, bool aligned, int sms, cudaStream_t s) {
    constexpr int V = 16 / b200::dt_size<DT>::value;
    HP p = p0;
    if (aligned) {
        p.nvec = p.count / V;
        i64 blocks = (p.nvec + 32 * kWarps - 1) / (32 * kWarps);
        if (blocks > (i64)sms * 8) blocks = (i64)sms * 8;
        if (blocks < 1) blocks = 1;
        hist_kernel<DT, V><<<(unsigned)blocks, 32 * kWarps, 0, s>>>(p);
    } else {
        p.nvec = p.count;
        i64 blocks = (p.nvec + 32 * kWarps - 1) / (32 * kWarps);
        if (blocks > (i64)sms * 8) blocks = (i64)sms * 8;
        hist_kernel<DT, 1><<<(unsigned)blocks, 32 * kWarps, 0, s>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace

extern "C" b200_status b200_log2_hist(uint64_t in, int32_t dtype, uint64_t count, uint64_t hist, int32_t nbins,
                                     int32_t offset, uint64_t stream) {
    if (!in || !hist) return b200_detail_fail(B200_ERR_INVALID, "b200_log2_hist: null device pointer");
    if (nbins < 1 || nbins > kMaxBins) return b200_detail_fail(B200_ERR_INVALID, "b200_log2_hist: 1 to 128 bins");
    if (dtype < B200_F32 || dtype > B200_U8) return b200_detail_fail(B200_ERR_INVALID, "b200_log2_hist: unknown dtype");
    if (hist % 4) return b200_detail_fail(B200_ERR_INVALID, "b200_log2_hist: histogram not 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(b200_detail_stream(stream));
    cudaError_t e = cudaMemsetAsync(reinterpret_cast<void*>(hist), 0, 4u * (unsigned)nbins, s);
    if (e == cudaSuccess && count) {
        int dev = 0, sms = 0;
        e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) {
            HP p;
            p.in = in; p.hist = hist; p.count = (i64)count; p.nvec = 0; p.nbins = nbins; p.offset = offset;
            const bool aligned = in % 16 == 0;
            switch (dtype) {                  // integer tensors are binned by their value as a float
            case B200_F32: e = launch<b200::F32>(p, aligned, sms, s); break;
            case B200_F16: e = launch<b200::F16>(p, aligned, sms, s); break;
            case B200_BF16: e = launch<b200::BF16>(p, aligned, sms, s); break;
            case B200_I32: e = launch<b200::I32>(p, aligned, sms, s); break;
            case B200_U32: e = launch<b200::U32>(p, aligned, sms, s); break;
            case B200_I16: e = launch<b200::I16>(p, aligned, sms, s); break;
            case B200_U16: e = launch<b200::U16>(p, aligned, sms, s); break;
            case B200_I8: e = launch<b200::I8>(p, aligned, sms, s); break;
            default: e = launch<b200::U8>(p, aligned, sms, s); break;
            }
        }
    }
    if (e != cudaSuccess) {
        char msg[160];
        snprintf(msg, sizeof msg, "b200_log2_hist: %s", cudaGetErrorString(e));
        return b200_detail_fail(B200_ERR_CUDA, msg);
    }
    return B200_OK;
}
