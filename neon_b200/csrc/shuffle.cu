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
//         writes along the output's.  Lanes move 16-byte vectors (8 or 4 bytes
//         when the two tile dimensions are short), sixteen lanes to a row, and
//         each thread transposes an N x N micro-block in registers, so shared
//         memory sees only whole vectors and no bank conflicts.
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
    int nd, src_vec, dst_vec;    // tile kernel: vector access allowed on the input / output side
    int bx_log2;                  // copy kernel: log2 of the lanes along dims[0]
};

template <int ES> struct elem_t;
template <> struct elem_t<1> { typedef unsigned char type; };
template <> struct elem_t<2> { typedef unsigned short type; };
template <> struct elem_t<4> { typedef unsigned int type; };
template <> struct elem_t<8> { typedef unsigned long long type; };
template <> struct elem_t<16> { typedef uint4 type; };

// offsets of the block's slice in the dimensions from `first` on (the grid has fewer than 2^31
// blocks, so block coordinates are 32-bit quantities)
__device__ __forceinline__ void rest_offsets(const ShP& p, int first, u32 r, i64& so, i64& dof) {
    for (int d = p.nd - 1; d >= first; --d) {
        const u32 nd = (u32)p.n[d];
        const u32 q = r / nd;
        const u32 c = r - q * nd;
        so += (i64)c * p.ss[d];
        dof += (i64)c * p.ds[d];
        r = q;
    }
}

// ---- vectors of U bytes held as 32-bit words; element k of such a vector
template <int ES> __device__ __forceinline__ u64 vget(const u32* w, int k) {
    if constexpr (ES == 8) return (u64)w[2 * k] | ((u64)w[2 * k + 1] << 32);
    else if constexpr (ES == 4) return w[k];
    else if constexpr (ES == 2) return (w[k >> 1] >> (16 * (k & 1))) & 0xffffu;
    else return (w[k >> 2] >> (8 * (k & 3))) & 0xffu;
}
template <int ES> __device__ __forceinline__ void vor(u32* w, int k, u64 x) {      // into a zeroed vector
    if constexpr (ES == 8) { w[2 * k] = (u32)x; w[2 * k + 1] = (u32)(x >> 32); }
    else if constexpr (ES == 4) w[k] = (u32)x;
    else if constexpr (ES == 2) w[k >> 1] |= (u32)x << (16 * (k & 1));
    else w[k >> 2] |= (u32)x << (8 * (k & 3));
}
template <int U> __device__ __forceinline__ void vld_global(const unsigned char* p, u32* w) {
    if constexpr (U == 16) { const uint4 a = __ldg(reinterpret_cast<const uint4*>(p)); w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; }
    else if constexpr (U == 8) { const uint2 a = __ldg(reinterpret_cast<const uint2*>(p)); w[0] = a.x; w[1] = a.y; }
    else w[0] = __ldg(reinterpret_cast<const u32*>(p));
}
template <int U> __device__ __forceinline__ void vst(void* p, const u32* w) {
    if constexpr (U == 16) *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    else if constexpr (U == 8) *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
    else *reinterpret_cast<u32*>(p) = w[0];
}
template <int U> __device__ __forceinline__ void vld_shared(const void* p, u32* w) {
    if constexpr (U == 16) { const uint4 a = *reinterpret_cast<const uint4*>(p); w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; }
    else if constexpr (U == 8) { const uint2 a = *reinterpret_cast<const uint2*>(p); w[0] = a.x; w[1] = a.y; }
    else w[0] = *reinterpret_cast<const u32*>(p);
}

// Tile kernel.  dims[0]: input stride 1 (index i);  dims[1]: output stride 1 (index o).
// A lane moves vectors of U bytes = N elements.  The tile is T x T elements, T = 16 N:
// thread (l, r) loads the N x N micro-block at columns i = N l .., rows o = N r .. as N
// vectors (sixteen lanes cover 16 U contiguous bytes of an input row), transposes it in
// registers, and stores N vectors into the shared tile, which is laid out [i][o] so that
// the second phase reads whole vectors along o and writes 16 U contiguous bytes of an
// output row.  Column vectors of tile row i are rotated by i / N: both phases then touch
// every bank group once per wavefront.
template <int ES, int U>
__global__ void __launch_bounds__(256) shuffle_tile_kernel(const __grid_constant__ ShP p) {
    typedef typename elem_t<ES>::type E;
    constexpr int N = U / ES;
    constexpr int T = 16 * N;
    constexpr int UW = U / 4;
    __shared__ __align__(16) u32 tile[T][16 * UW];

    const int l = threadIdx.x & 15, r = threadIdx.x >> 4;
    u32 b = blockIdx.x;
    const u32 nt0 = (u32)p.tiles0, nt1 = (u32)p.tiles1;
    const i64 t0 = b % nt0; b /= nt0;
    const i64 t1 = b % nt1; b /= nt1;
    i64 so = 0, dof = 0;
    rest_offsets(p, 2, b, so, dof);
    const i64 ni = p.n[0], no = p.n[1];
    const E* __restrict__ src = reinterpret_cast<const E*>(p.src) + so;
    E* __restrict__ dst = reinterpret_cast<E*>(p.dst) + dof;

    {   // global -> registers -> shared
        const i64 i = t0 * T + N * l;
        const i64 o = t1 * T + N * r;
        u32 in[N][UW];
        const bool whole = p.src_vec && i + N <= ni;
#pragma unroll
        for (int v = 0; v < N; ++v) {
#pragma unroll
            for (int q = 0; q < UW; ++q) in[v][q] = 0;
            if (o + v < no) {
                const E* row = src + (o + v) * p.ss[1] + i;
                if (whole) vld_global<U>(reinterpret_cast<const unsigned char*>(row), in[v]);
                else {
#pragma unroll
                    for (int e = 0; e < N; ++e)
                        if (i + e < ni) vor<ES>(in[v], e, (u64)__ldg(row + e));
                }
            }
        }
#pragma unroll
        for (int w = 0; w < N; ++w) {
            u32 out[UW];
            if constexpr (ES == 2) {
                // element w of rows 2q and 2q+1 -> word q: one byte permute
#pragma unroll
                for (int q = 0; q < UW; ++q)
                    out[q] = __byte_perm(in[2 * q][w >> 1], in[2 * q + 1][w >> 1], (w & 1) ? 0x7632 : 0x5410);
            } else if constexpr (ES == 1) {
                // byte w of rows 4q .. 4q+3 -> word q: two permutes pick the byte from row pairs, one joins them
                const u32 sel = ((4u + (w & 3)) << 4) | (u32)(w & 3);
#pragma unroll
                for (int q = 0; q < UW; ++q) {
                    const u32 lo = __byte_perm(in[4 * q][w >> 2], in[4 * q + 1][w >> 2], sel);
                    const u32 hi = __byte_perm(in[4 * q + 2][w >> 2], in[4 * q + 3][w >> 2], sel);
                    out[q] = __byte_perm(lo, hi, 0x5410);
                }
            } else {
#pragma unroll
                for (int q = 0; q < UW; ++q) out[q] = 0;
#pragma unroll
                for (int v = 0; v < N; ++v) vor<ES>(out, v, vget<ES>(in[v], w));
            }
            vst<U>(&tile[N * l + w][((r + l) & 15) * UW], out);
        }
    }
    __syncthreads();
    {   // shared -> global: lane l covers o = N l .., thread row r covers i = N r ..
        const i64 o = t1 * T + N * l;
        const bool whole = p.dst_vec && o + N <= no;
#pragma unroll
        for (int w = 0; w < N; ++w) {
            const i64 i = t0 * T + N * r + w;
            if (i >= ni || o >= no) continue;
            u32 x[UW];
            vld_shared<U>(&tile[N * r + w][((l + r) & 15) * UW], x);
            E* row = dst + i * p.ds[0] + o;
            if (whole) vst<U>(row, x);
            else {
#pragma unroll
                for (int e = 0; e < N; ++e)
                    if (o + e < no) row[e] = (E)vget<ES>(x, e);
            }
        }
    }
}

// Copy kernel.  dims[0]: lane dimension (any strides), dims[1]: the next one (extent 1 when
// there is none).  The 256 threads form bx lanes x (256 / bx) rows, bx a power of two picked by
// the host so that short lane dimensions still fill the block; a thread moves up to four
// elements, bx apart.
template <int ES>
__global__ void __launch_bounds__(256) shuffle_copy_kernel(const __grid_constant__ ShP p) {
    typedef typename elem_t<ES>::type E;
    const int bx_log2 = p.bx_log2;
    const int bx = 1 << bx_log2;
    const int tx = threadIdx.x & (bx - 1), ty = threadIdx.x >> bx_log2;
    u32 b = blockIdx.x;
    const u32 nt0 = (u32)p.tiles0, nt1 = (u32)p.tiles1;
    const i64 t0 = b % nt0; b /= nt0;
    const i64 t1 = b % nt1; b /= nt1;
    i64 so = 0, dof = 0;
    rest_offsets(p, 2, b, so, dof);
    const i64 j = t1 * (256 >> bx_log2) + ty;
    if (j >= p.n[1]) return;
    const E* __restrict__ src = reinterpret_cast<const E*>(p.src) + so + j * p.ss[1];
    E* __restrict__ dst = reinterpret_cast<E*>(p.dst) + dof + j * p.ds[1];
    const i64 base = t0 * (4 * bx) + tx;
    E v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const i64 i = base + u * bx;
        if (i < p.n[0]) v[u] = src[i * p.ss[0]];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const i64 i = base + u * bx;
        if (i < p.n[0]) dst[i * p.ds[0]] = v[u];
    }
}

template <int ES, int U> cudaError_t launch_tile(const ShP& p, unsigned grid, cudaStream_t s) {
    shuffle_tile_kernel<ES, U><<<grid, 256, 0, s>>>(p);
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
    p.dst = dst; p.src = src; p.bx_log2 = 8; p.src_vec = 0; p.dst_vec = 0; p.tiles1 = 1;
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
    if (!tiled) {
        // second block dimension of the copy kernel: the innermost of the other dimensions
        for (int d = nd - 1; d >= 0; --d)
            if (d != lead[0]) { lead[1] = d; break; }
    }
    int k = 0;
    for (int j = 0; j < 2; ++j) {
        if (lead[j] >= 0) { p.n[k] = n[lead[j]]; p.ds[k] = ds[lead[j]]; p.ss[k] = ss[lead[j]]; }
        else { p.n[k] = 1; p.ds[k] = 0; p.ss[k] = 0; }
        ++k;
    }
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
    int U = 0;                                   // bytes a lane of the tile kernel moves at once
    if (tiled) {
        // vector width: tiles are T = 16 U / es elements a side, so short dimensions waste part of
        // a wide tile, while narrow vectors move fewer bytes per instruction (measured: about 0.7 of
        // the 16-byte rate at 8 bytes, 0.4 at 4).  Take the smallest padded area / rate.
        double best = 0;
        for (int u = es == 1 ? 8 : 16; u >= 2 * es && u >= 4; u >>= 1) {
            const i64 T = 16 * (u / es);
            const double area = (double)((p.n[0] + T - 1) / T * T) * (double)((p.n[1] + T - 1) / T * T);
            const double cost = area / (u == 16 ? 1.0 : u == 8 ? (es == 1 ? 1.0 : 0.7) : (es == 1 ? 0.7 : 0.4));
            if (!U || cost < best) { U = u; best = cost; }
        }
        const int T = 16 * (U / es);
        p.tiles0 = (p.n[0] + T - 1) / T;
        p.tiles1 = (p.n[1] + T - 1) / T;
        blocks = p.tiles0 * p.tiles1 * rest;
        bool sv = src % U == 0, dv = dst % U == 0;
        for (int d = 0; d < k; ++d) {
            if (d != 0 && (p.ss[d] * es) % U) sv = false;
            if (d != 1 && (p.ds[d] * es) % U) dv = false;
        }
        p.src_vec = sv; p.dst_vec = dv;
    } else {
        // lanes along dims[0]: the widest of 256/128/64/32 that wastes the fewest slots of the
        // 4 bx elements a block row covers
        int bx_log2 = 8;
        if (p.n[1] > 1) {
            i64 best = (p.n[0] + 1023) / 1024 * 1024;
            for (int bl = 7; bl >= 5; --bl) {
                const i64 chunk = 4ll << bl;
                const i64 padded = (p.n[0] + chunk - 1) / chunk * chunk;
                if (padded < best) { best = padded; bx_log2 = bl; }
            }
        }
        p.bx_log2 = bx_log2;
        p.tiles0 = (p.n[0] + (4ll << bx_log2) - 1) / (4ll << bx_log2);
        p.tiles1 = (p.n[1] + (256 >> bx_log2) - 1) / (256 >> bx_log2);
        blocks = p.tiles0 * p.tiles1 * rest;
    }
    if (blocks > 0x7fffffffll) return b200_detail_fail(B200_ERR_UNSUPPORTED, "b200_dimshuffle: more than 2^31 blocks");
    const unsigned grid = (unsigned)blocks;
    if (tiled) {
        switch (es * 100 + U) {
        case 108: e = launch_tile<1, 8>(p, grid, s); break;
        case 104: e = launch_tile<1, 4>(p, grid, s); break;
        case 216: e = launch_tile<2, 16>(p, grid, s); break;
        case 208: e = launch_tile<2, 8>(p, grid, s); break;
        case 204: e = launch_tile<2, 4>(p, grid, s); break;
        case 416: e = launch_tile<4, 16>(p, grid, s); break;
        case 408: e = launch_tile<4, 8>(p, grid, s); break;
        default: e = launch_tile<8, 16>(p, grid, s); break;
        }
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
