// b200_dimshuffle: out = transpose(a, axes) for tensors of any rank, the
// device side of copy_transpose (neon/backends/nervanagpu.py:3077-3118; the
// reference generates a 32x32 shared-memory tile kernel per shape in
// neon/backends/convolution.py, _get_copy_transpose_kernel).
//
// The caller describes the copy in OUTPUT dimension order: for every output
// dimension its extent, the output's element stride and the input's element
// stride of the axis that lands there.  The host code below drops extent-1
// dimensions, merges neighbours that are contiguous in both tensors and then
// picks one of two kernels:
//
//   tile  when the input's unit-stride dimension and the output's unit-stride
//         dimension differ: a T x T element tile goes through shared memory so
//         that global reads run along the input's fast dimension and global
//         writes along the output's.  T = 32 elements of 4 or 8 bytes, 64 of 2
//         bytes, 128 of 1 byte, so a warp always moves 128 contiguous bytes
//         per row (as one 32-bit access per lane when alignment allows).
//   copy  otherwise (same fast dimension, or no unit stride at all): lanes run
//         along the output's innermost dimension; when that dimension is
//         contiguous in both tensors and everything is 16-byte aligned the
//         elements are widened to 16 bytes first.
//
// Both are pure data movement, bound by HBM: 2 x elem_bytes per element.

#include "b200ew.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

extern "C" void* b200_detail_stream(uint64_t stream);
extern "C" int32_t b200_detail_fail(int32_t code, const char* message);

namespace {

typedef unsigned long long u64;
typedef long long i64;
typedef unsigned int u32;

enum { kMaxDims = B200_SHUFFLE_MAX_DIMS };

// dims[0], dims[1] are the two tile dimensions (tile kernel) or dims[0] the lane
// dimension (copy kernel); the rest are walked by the block index.
struct ShP {
    u64 dst, src;
    i64 n[kMaxDims], ds[kMaxDims], ss[kMaxDims];
    i64 tiles0, tiles1;
    int nd, src_vec, dst_vec, pad_;
};

template <int ES> struct elem_t;
template <> struct elem_t<1> { typedef unsigned char type; };
template <> struct elem_t<2> { typedef unsigned short type; };
template <> struct elem_t<4> { typedef unsigned int type; };
template <> struct elem_t<8> { typedef unsigned long long type; };
template <> struct elem_t<16> { typedef uint4 type; };

// offsets of the block's slice in the dimensions from `first` on
__device__ __forceinline__ void rest_offsets(const ShP& p, int first, i64 r, i64& so, i64& dof) {
    for (int d = p.nd - 1; d >= first; --d) {
        const i64 q = r / p.n[d];
        const i64 c = r - q * p.n[d];
        so += c * p.ss[d];
        dof += c * p.ds[d];
        r = q;
    }
}

// dims[0]: input stride 1 (index i);  dims[1]: output stride 1 (index o)
template <int ES>
__global__ void __launch_bounds__(256) shuffle_tile_kernel(const __grid_constant__ ShP p) {
    typedef typename elem_t<ES>::type E;
    constexpr int VEC = ES >= 4 ? 1 : 4 / ES;      // elements per 32-bit word
    constexpr int T = 32 * VEC;
    __shared__ __align__(16) E tile[T][T + VEC];   // [o][i]; the pad keeps column reads off one bank

    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    i64 b = blockIdx.x;
    const i64 t0 = b % p.tiles0; b /= p.tiles0;
    const i64 t1 = b % p.tiles1; b /= p.tiles1;
    i64 so = 0, dof = 0;
    rest_offsets(p, 2, b, so, dof);
    const i64 i0 = t0 * T, o0 = t1 * T;
    const E* __restrict__ src = reinterpret_cast<const E*>(p.src) + so;
    E* __restrict__ dst = reinterpret_cast<E*>(p.dst) + dof;
    const i64 ni = p.n[0], no = p.n[1];

    // global -> shared, lanes along i
#pragma unroll 4
    for (int ol = ty; ol < T; ol += 8) {
        const i64 o = o0 + ol;
        if (o >= no) break;
        const i64 i = i0 + tx * VEC;
        const E* row = src + o * p.ss[1];
        bool done = false;
        if constexpr (VEC > 1) {
            if (p.src_vec && i + VEC <= ni) {
                const u32 w = __ldg(reinterpret_cast<const u32*>(row + i));
                *reinterpret_cast<u32*>(&tile[ol][tx * VEC]) = w;
                done = true;
            }
        }
        if (!done) {
#pragma unroll
            for (int v = 0; v < VEC; ++v)
                if (i + v < ni) tile[ol][tx * VEC + v] = __ldg(row + i + v);
        }
    }
    __syncthreads();
    // shared -> global, lanes along o
#pragma unroll 4
    for (int il = ty; il < T; il += 8) {
        const i64 i = i0 + il;
        if (i >= ni) break;
        const i64 o = o0 + tx * VEC;
        E* row = dst + i * p.ds[0];
        bool done = false;
        if constexpr (VEC > 1) {
            if (p.dst_vec && o + VEC <= no) {
                u32 w = 0;
#pragma unroll
                for (int v = 0; v < VEC; ++v) w |= (u32)tile[tx * VEC + v][il] << (8 * ES * v);
                *reinterpret_cast<u32*>(row + o) = w;
                done = true;
            }
        }
        if (!done) {
#pragma unroll
            for (int v = 0; v < VEC; ++v)
                if (o + v < no) row[o + v] = tile[tx * VEC + v][il];
        }
    }
}

// dims[0]: lane dimension with any strides; a block moves 1024 consecutive indices of it
template <int ES>
__global__ void __launch_bounds__(256) shuffle_copy_kernel(const __grid_constant__ ShP p) {
    typedef typename elem_t<ES>::type E;
    i64 b = blockIdx.x;
    const i64 c = b % p.tiles0; b /= p.tiles0;
    i64 so = 0, dof = 0;
    rest_offsets(p, 1, b, so, dof);
    const E* __restrict__ src = reinterpret_cast<const E*>(p.src) + so;
    E* __restrict__ dst = reinterpret_cast<E*>(p.dst) + dof;
    const i64 base = c * 1024 + threadIdx.x;
    E v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const i64 i = base + u * 256;
        if (i < p.n[0]) v[u] = src[i * p.ss[0]];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const i64 i = base + u * 256;
        if (i < p.n[0]) dst[i * p.ds[0]] = v[u];
    }
}

template <int ES> cudaError_t launch_tile(const ShP& p, unsigned grid, cudaStream_t s) {
    shuffle_tile_kernel<ES><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}
template <int ES> cudaError_t launch_copy(const ShP& p, unsigned grid, cudaStream_t s) {
    shuffle_copy_kernel<ES><<<grid, 256, 0, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

extern "C" b200_status b200_dimshuffle(uint64_t dst, uint64_t src, int32_t elem_bytes, int32_t ndim,
                                      const int64_t* shape, const int64_t* dst_strides,
                                      const int64_t* src_strides, uint64_t stream) {
    if (!dst || !src) return b200_detail_fail(B200_ERR_INVALID, "b200_dimshuffle: null device pointer");
    if (dst == src) return b200_detail_fail(B200_ERR_INVALID, "b200_dimshuffle: input and output are the same memory");
    if (ndim < 1 || ndim > kMaxDims) return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_dimshuffle: 1 to 8 dimensions");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
        return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_dimshuffle: elements of 1, 2, 4 or 8 bytes");
    if (!shape || !dst_strides || !src_strides) return b200_detail_fail(B200_ERR_INVALID, "b200_dimshuffle: null array");
    if (dst % elem_bytes || src % elem_bytes)
        return b200_detail_fail(B200_ERR_INVALID, "b200_dimshuffle: pointer not aligned to the element size");

    // 1. keep the dimensions with more than one index
    i64 n[kMaxDims], ds[kMaxDims], ss[kMaxDims];
    int nd = 0;
    for (int d = 0; d < ndim; ++d) {
        if (shape[d] < 0 || dst_strides[d] < 0 || src_strides[d] < 0)
            return b200_detail_fail(B200_ERR_INVALID, "b200_dimshuffle: negative extent or stride");
        if (shape[d] == 0) return B200_OK;
        if (shape[d] == 1) continue;
        n[nd] = shape[d]; ds[nd] = dst_strides[d]; ss[nd] = src_strides[d];
        ++nd;
    }
    if (nd == 0) { n[0] = 1; ds[0] = 1; ss[0] = 1; nd = 1; }
    // 2. merge neighbours that are contiguous in both tensors
    int m = 0;
    for (int d = 1; d < nd; ++d) {
        if (ds[m] == ds[d] * n[d] && ss[m] == ss[d] * n[d]) {
            n[m] *= n[d]; ds[m] = ds[d]; ss[m] = ss[d];
        } else {
            ++m;
            n[m] = n[d]; ds[m] = ds[d]; ss[m] = ss[d];
        }
    }
    nd = m + 1;

    // 3. which dimension is fast in the output, which in the input
    int od = -1, id = -1;
    for (int d = 0; d < nd; ++d) {
        if (ds[d] == 1 && (od < 0 || n[d] > n[od])) od = d;
        if (ss[d] == 1 && (id < 0 || n[d] > n[id])) id = d;
    }
    const bool tiled = od >= 0 && id >= 0 && od != id && n[od] >= 8 && n[id] >= 8;

    ShP p;
    p.dst = dst; p.src = src; p.pad_ = 0; p.src_vec = 0; p.dst_vec = 0; p.tiles1 = 1;
    int es = elem_bytes;
    int lead[2] = {-1, -1};
    if (tiled) { lead[0] = id; lead[1] = od; }
    else {
        int lane = od;
        if (lane < 0) {             // no unit stride in the output: lanes along its smallest stride
            lane = 0;
            for (int d = 1; d < nd; ++d) if (ds[d] < ds[lane]) lane = d;
        }
        lead[0] = lane;
        if (ds[lane] == 1 && ss[lane] == 1) {
            // widen the element while every offset stays a whole number of wide elements
            for (int w = 16; w > es; w >>= 1) {
                bool ok = (n[lane] * es) % w == 0 && dst % w == 0 && src % w == 0;
                for (int d = 0; ok && d < nd; ++d)
                    if (d != lane && ((ds[d] * es) % w || (ss[d] * es) % w)) ok = false;
                if (!ok) continue;
                const int f = w / es;
                n[lane] /= f;
                for (int d = 0; d < nd; ++d) if (d != lane) { ds[d] /= f; ss[d] /= f; }
                es = w;
                break;
            }
        }
    }
    int k = 0;
    for (int j = 0; j < 2; ++j)
        if (lead[j] >= 0) { p.n[k] = n[lead[j]]; p.ds[k] = ds[lead[j]]; p.ss[k] = ss[lead[j]]; ++k; }
    i64 rest = 1;
    for (int d = 0; d < nd; ++d) {
        if (d == lead[0] || d == lead[1]) continue;
        p.n[k] = n[d]; p.ds[k] = ds[d]; p.ss[k] = ss[d]; ++k;
        rest *= n[d];
    }
    p.nd = k;
    for (int d = k; d < kMaxDims; ++d) { p.n[d] = 1; p.ds[d] = 0; p.ss[d] = 0; }

    cudaStream_t s = static_cast<cudaStream_t>(b200_detail_stream(stream));
    cudaError_t e;
    i64 blocks;
    if (tiled) {
        const int T = es >= 4 ? 32 : 32 * (4 / es);
        p.tiles0 = (p.n[0] + T - 1) / T;
        p.tiles1 = (p.n[1] + T - 1) / T;
        blocks = p.tiles0 * p.tiles1 * rest;
        bool sv = src % 4 == 0, dv = dst % 4 == 0;
        for (int d = 0; d < k; ++d) {
            if (d != 0 && (p.ss[d] * es) % 4) sv = false;
            if (d != 1 && (p.ds[d] * es) % 4) dv = false;
        }
        p.src_vec = sv; p.dst_vec = dv;
    } else {
        p.tiles0 = (p.n[0] + 1023) / 1024;
        blocks = p.tiles0 * rest;
    }
    if (blocks > 0x7fffffffll) return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_dimshuffle: more than 2^31 blocks");
    const unsigned grid = (unsigned)blocks;
    if (tiled) {
        e = es == 1 ? launch_tile<1>(p, grid, s) : es == 2 ? launch_tile<2>(p, grid, s)
          : es == 4 ? launch_tile<4>(p, grid, s) : launch_tile<8>(p, grid, s);
    } else {
        e = es == 1 ? launch_copy<1>(p, grid, s) : es == 2 ? launch_copy<2>(p, grid, s)
          : es == 4 ? launch_copy<4>(p, grid, s) : es == 8 ? launch_copy<8>(p, grid, s) : launch_copy<16>(p, grid, s);
    }
    if (e != cudaSuccess) {
        char msg[160];
        snprintf(msg, sizeof msg, "b200_dimshuffle: %s", cudaGetErrorString(e));
        return b200_detail_fail(B200_ERR_CUDA, msg);
    }
    return B200_OK;
}
