// b200_compensated_sum: Kahan-compensated in-place accumulation with optional
// stochastic rounding of the running sum, the device side of
// NervanaGPU.compensated_sum (neon/backends/nervanagpu.py:1896-1917, kernel text
// neon/backends/float_ew.py:944-1037).  Per element, in fp32:
//
//     y   = add * add_scale - cmp * cmp_scale        amount to add, corrected
//     t   = round(sum + y)                            to the storage type; stochastic
//                                                     when rounding_bits > 0, else nearest
//     cmp = nearest((t - sum) - y)                    what the rounding lost
//     sum = t
//
// The three tensors are contiguous and of one dtype (f32, f16 or bf16).  Random
// bits come from the library's counter-based generator exactly as for an
// op-tree store of the same element index, so a given (seed, launch counter)
// reproduces the result whatever the launch geometry.
// HBM traffic: 3 reads + 2 writes of the element size.

#include "b200ew.h"
#include "optree_templates.cuh"

#include <cuda_runtime.h>

#include <cstdio>

extern "C" void* b200_detail_stream(uint64_t stream);
extern "C" int32_t b200_detail_fail(int32_t code, const char* message);

namespace {

struct KP {
    u64 sum, cmp, add;
    i64 first, count;        // element range [first, first + count * V)
    float cmp_scale, add_scale;
    u32 k0, k1;
    int mb, pad_;
};

template <int DT, int V, bool SR>
__global__ void __launch_bounds__(256) kahan_kernel(const __grid_constant__ KP p) {
    using namespace b200;
    constexpr bool PAIR = DT != F32;
    constexpr int B = dt_size<DT>::value * V;
    constexpr int W = (B + 3) / 4;
    const i64 j = (i64)blockIdx.x * 256 + threadIdx.x;
    if (j >= p.count) return;
    const i64 e = p.first + j * V;
    float s[V], c[V], a[V], y[V], t[V];
    ld_f<DT, V, false>(p.sum, e, s);
    ld_f<DT, V, false>(p.cmp, e, c);
    ld_f<DT, V, true>(p.add, e, a);
#pragma unroll
    for (int i = 0; i < V; ++i) {
        y[i] = a[i] * p.add_scale - c[i] * p.cmp_scale;
        t[i] = s[i] + y[i];
    }
    u32 ur[V];
    SrCtx cx = sr_ctx(SR ? p.mb : 23);
    if constexpr (SR) {
        Rng g; g.k0 = p.k0; g.k1 = p.k1;
        if constexpr (V > 1) rng_lanes<V, PAIR, true>(g, (u64)e, 1, ur);
        else rng_lanes<V, PAIR, false>(g, (u64)e, 1, ur);
    }
    u32 w[W];
    cvt_out<DT, V, SR>(t, w, cx, ur);
    cvt_in<DT, V>(w, t);                   // the sum as it is stored
    st_raw<B>(reinterpret_cast<char*>(p.sum) + e * dt_size<DT>::value, w);
#pragma unroll
    for (int i = 0; i < V; ++i) c[i] = (t[i] - s[i]) - y[i];
    cvt_out<DT, V, false>(c, w, cx, ur);
    st_raw<B>(reinterpret_cast<char*>(p.cmp) + e * dt_size<DT>::value, w);
}

template <int DT, int V>
cudaError_t launch_v(const KP& p, cudaStream_t s) {
    const unsigned grid = (unsigned)((p.count + 255) / 256);
    if (p.mb > 0) kahan_kernel<DT, V, true><<<grid, 256, 0, s>>>(p);
    else kahan_kernel<DT, V, false><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}

template <int DT>
cudaError_t launch_dt(KP p, u64 count, bool aligned, cudaStream_t s) {
    constexpr int V = 16 / b200::dt_size<DT>::value;
    u64 done = 0;
    if (aligned && count >= (u64)V) {
        p.first = 0; p.count = (i64)(count / V);
        cudaError_t e = launch_v<DT, V>(p, s);
        if (e != cudaSuccess) return e;
        done = (count / V) * V;
    }
    if (done < count) {
        p.first = (i64)done; p.count = (i64)(count - done);
        return launch_v<DT, 1>(p, s);
    }
    return cudaSuccess;
}

}  // namespace

extern "C" b200_status b200_compensated_sum(uint64_t sum, uint64_t cmp, uint64_t add, int32_t dtype, uint64_t count,
                                           float cmp_scale, float add_scale, int32_t rounding_bits,
                                           uint64_t stream) {
    if (!sum || !cmp || !add) return b200_detail_fail(B200_ERR_INVALID, "b200_compensated_sum: null device pointer");
    if (dtype != B200_F32 && dtype != B200_F16 && dtype != B200_BF16)
        return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_compensated_sum: only f32, f16 and bf16 tensors");
    if (count == 0) return B200_OK;
    if (count > (1ull << 36)) return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_compensated_sum: more than 2^36 elements");
    const int cap = dtype == B200_F32 ? 15 : dtype == B200_F16 ? 10 : 7;     // as for op-tree stores
    if (rounding_bits < 0) return b200_detail_fail(B200_ERR_INVALID, "b200_compensated_sum: negative rounding bits");
    KP p;
    p.sum = sum; p.cmp = cmp; p.add = add;
    p.first = 0; p.count = 0;
    p.cmp_scale = cmp_scale; p.add_scale = add_scale;
    p.mb = rounding_bits > cap ? cap : rounding_bits;
    p.pad_ = 0; p.k0 = 0; p.k1 = 0;
    if (p.mb > 0) {
        uint32_t key[2];
        b200_status st = b200_rng_next_key(key);
        if (st) return st;
        p.k0 = key[0]; p.k1 = key[1];
    }
    const bool aligned = (sum % 16 == 0) && (cmp % 16 == 0) && (add % 16 == 0);
    cudaStream_t s = static_cast<cudaStream_t>(b200_detail_stream(stream));
    cudaError_t e;
    if (dtype == B200_F32) e = launch_dt<b200::F32>(p, count, aligned, s);
    else if (dtype == B200_F16) e = launch_dt<b200::F16>(p, count, aligned, s);
    else e = launch_dt<b200::BF16>(p, count, aligned, s);
    if (e != cudaSuccess) {
        char msg[160];
        snprintf(msg, sizeof msg, "b200_compensated_sum: %s", cudaGetErrorString(e));
        return b200_detail_fail(B200_ERR_CUDA, msg);
    }
    return B200_OK;
}
