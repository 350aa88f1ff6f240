// Kernels that are compiled into libb200ew.so at build time (no NVRTC needed):
// pattern fills behind b200_memset, and the whole-tensor reduction behind
// b200_reduce_full, which instantiates the same red_rows_kernel skeleton the
// run-time generated op-tree kernels use.

#include "b200ew.h"
#include "optree_templates.cuh"

#include <cuda_runtime.h>

namespace {

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* dst, T value, u64 count) {
    u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x;
    const u64 step = (u64)gridDim.x * blockDim.x;
    for (; i < count; i += step) dst[i] = value;
}

// ---- whole-tensor reduction: one kept index (K = 1), row = all elements
struct RP {
    u64 t0, part_v, part_i, counters, o;
    i64 K, N, nvec, seg;
    int split, pad_;
};

template <int DT, int OP, bool ABS>
struct FullRed {
    template <int V>
    struct S {
        enum { NRED = 1, FUSED = (OP == b200::OP_SUM && !ABS && DT != b200::F32) ? 1 : 0, XCHG = 0 };
        static DEV constexpr int op(int) { return OP; }
        struct H { int unused_; };
        struct L { u32 a0[(b200::dt_size<DT>::value * V + 3) / 4]; };
        static DEV void load_h(const RP&, i64, H&) {}
        static DEV void load_l(const RP& p, i64, i64 n, L& l) { b200::ld_w<DT, V, true>(p.t0, n, l.a0); }
        static DEV void eval(const RP&, const H&, const L& l, i64, i64, float (&out)[1][V]) {
            float a0[V];
            b200::cvt_in<DT, V>(l.a0, a0);
#pragma unroll
            for (int i = 0; i < V; ++i) out[0][i] = ABS ? fabsf(a0[i]) : a0[i];
        }
        // plain sums of 16-bit floats: the add takes the stored value as it is
        static DEV void accum(const RP&, const H&, const L& l, i64, i64, float (&acc)[1][V], int (&)[1][V]) {
            if constexpr (DT != b200::F32) {
#pragma unroll
                for (int i = 0; i < V; ++i) acc[0][i] = b200::mx_add<DT, V>(l.a0, i, acc[0][i]);
            }
        }
        static DEV void epilogue(const RP& p, i64, const float* r, const int*) {
            *reinterpret_cast<float*>(p.o) = r[0];
        }
    };
};

template <int DT, int OP, bool ABS, int V>
__global__ void __launch_bounds__(256) full_reduce_kernel(const __grid_constant__ RP p) {
    b200::red_rows_kernel<FullRed<DT, OP, ABS>::template S, RP, V, 256, 256, 4>(p);
}

template <int DT, int OP, bool ABS>
cudaError_t launch_full(const RP& p, bool vec, unsigned grid, cudaStream_t s) {
    constexpr int V = 16 / b200::dt_size<DT>::value;
    if (vec) full_reduce_kernel<DT, OP, ABS, V><<<grid, 256, 0, s>>>(p);
    else full_reduce_kernel<DT, OP, ABS, 1><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}

template <int DT>
cudaError_t launch_full_dt(const RP& p, int op, bool absolute, bool vec, unsigned grid, cudaStream_t s) {
    if (op == B200_SUM) return absolute ? launch_full<DT, b200::OP_SUM, true>(p, vec, grid, s) : launch_full<DT, b200::OP_SUM, false>(p, vec, grid, s);
    if (op == B200_MAX) return absolute ? launch_full<DT, b200::OP_MAX, true>(p, vec, grid, s) : launch_full<DT, b200::OP_MAX, false>(p, vec, grid, s);
    return absolute ? launch_full<DT, b200::OP_MIN, true>(p, vec, grid, s) : launch_full<DT, b200::OP_MIN, false>(p, vec, grid, s);
}

// ---- plain tiled GEMM for `dot` nodes inside op-trees (conformance, not a performance path):
// C[m,n] = alpha * sum_k A[m,k] * B[k,n] + beta * C[m,n], any element strides, fp32 accumulation
struct GemmP {
    u64 a, b, c;
    i64 a_s0, a_s1, b_s0, b_s1, c_s0, c_s1;
    int m, n, k, pad_;
    float alpha, beta;
};

template <int DA, int DB, int DC>
__global__ void __launch_bounds__(256) gemm_kernel(const __grid_constant__ GemmP p) {
    __shared__ float sa[16][17], sb[16][17];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
    float acc = 0.f;
    for (int k0 = 0; k0 < p.k; k0 += 16) {
        float va = 0.f, vb = 0.f;
        if (row < p.m && k0 + tx < p.k) b200::ld_f<DA, 1, false>(p.a, (i64)row * p.a_s0 + (i64)(k0 + tx) * p.a_s1, &va);
        if (k0 + ty < p.k && col < p.n) b200::ld_f<DB, 1, false>(p.b, (i64)(k0 + ty) * p.b_s0 + (i64)col * p.b_s1, &vb);
        sa[ty][tx] = va; sb[ty][tx] = vb;
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) acc = fmaf(sa[ty][kk], sb[kk][tx], acc);
        __syncthreads();
    }
    if (row < p.m && col < p.n) {
        const i64 o = (i64)row * p.c_s0 + (i64)col * p.c_s1;
        float prev = 0.f;
        if (p.beta != 0.f) b200::ld_f<DC, 1, false>(p.c, o, &prev);
        b200::st_one<DC>(p.c, o, p.alpha * acc + p.beta * prev);
    }
}

template <int DA, int DB>
cudaError_t launch_gemm_c(const GemmP& p, int dc, dim3 grid, cudaStream_t s) {
    if (dc == B200_F32) gemm_kernel<DA, DB, b200::F32><<<grid, 256, 0, s>>>(p);
    else gemm_kernel<DA, DB, b200::F16><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

extern "C" int b200_detail_gemm(uint64_t a, int da, int64_t a_s0, int64_t a_s1,
                                uint64_t b, int db, int64_t b_s0, int64_t b_s1,
                                uint64_t c, int dc, int64_t c_s0, int64_t c_s1,
                                int m, int n, int k, float alpha, float beta, void* stream) {
    GemmP p;
    p.a = a; p.b = b; p.c = c;
    p.a_s0 = a_s0; p.a_s1 = a_s1; p.b_s0 = b_s0; p.b_s1 = b_s1; p.c_s0 = c_s0; p.c_s1 = c_s1;
    p.m = m; p.n = n; p.k = k; p.pad_ = 0; p.alpha = alpha; p.beta = beta;
    dim3 grid((n + 15) / 16, (m + 15) / 16, 1);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool af = da == B200_F32, bf = db == B200_F32;
    cudaError_t e;
    if (af && bf) e = launch_gemm_c<b200::F32, b200::F32>(p, dc, grid, s);
    else if (af) e = launch_gemm_c<b200::F32, b200::F16>(p, dc, grid, s);
    else if (bf) e = launch_gemm_c<b200::F16, b200::F32>(p, dc, grid, s);
    else e = launch_gemm_c<b200::F16, b200::F16>(p, dc, grid, s);
    return (int)e;
}

enum { kMaxSplit = 4096, kCounterBytes = 256 };

// used by runtime.cpp
extern "C" int b200_detail_fill(void* dst, uint32_t value, int width, uint64_t count, void* stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    u64 blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (width == 2) fill_kernel<u16><<<(unsigned)blocks, 256, 0, s>>>(static_cast<u16*>(dst), (u16)value, count);
    else fill_kernel<u32><<<(unsigned)blocks, 256, 0, s>>>(static_cast<u32*>(dst), value, count);
    return (int)cudaGetLastError();
}

extern "C" uint64_t b200_reduce_scratch_bytes(void) { return kCounterBytes + 4ull * kMaxSplit; }

// Fills the parameter block and picks the grid; shared with the variant that
// keeps its scratch in a static device array.
extern "C" int b200_detail_reduce_full(uint64_t in, int32_t dtype, uint64_t count, int32_t op, int32_t absolute,
                                       uint64_t out, uint64_t scratch, int sm_count, void* stream) {
    RP p;
    const int isz = dtype == B200_F32 ? 4 : 2;
    const int V = 16 / isz;
    const bool vec = (in % 16) == 0 && count >= (uint64_t)V;
    const int v = vec ? V : 1;
    p.t0 = in; p.o = out;
    p.counters = scratch;
    p.part_v = scratch + kCounterBytes;
    p.part_i = 0;
    p.K = 1; p.N = (i64)count; p.nvec = (i64)(count / v);
    i64 split = p.nvec / (256 * 4);
    const i64 target = (i64)sm_count * 8;
    if (split > target) split = target;
    if (split > kMaxSplit) split = kMaxSplit;
    if (split < 1) split = 1;
    p.seg = (p.nvec + split - 1) / split;
    split = (p.nvec + p.seg - 1) / p.seg;
    if (split < 1) split = 1;
    p.split = (int)split; p.pad_ = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (dtype == B200_F32) e = launch_full_dt<b200::F32>(p, op, absolute != 0, vec, (unsigned)split, s);
    else if (dtype == B200_F16) e = launch_full_dt<b200::F16>(p, op, absolute != 0, vec, (unsigned)split, s);
    else e = launch_full_dt<b200::BF16>(p, op, absolute != 0, vec, (unsigned)split, s);
    return (int)e;
}
