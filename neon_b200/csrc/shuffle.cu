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
//   tma   the tile case for 1- and 2-byte elements when both tensors allow it (16-byte aligned
//         bases and pitches, output extent a multiple of the vector): the tile is fetched by one
//         tiled bulk-tensor copy into a swizzled shared-memory image and written back by one
//         bulk-tensor store, so no lane computes a global address; threads only move 16-byte
//         vectors between the two shared images and transpose micro-blocks in registers.
//
// All are pure data movement, bound by HBM: 2 x elem_bytes per element.

#include "b200ew.h"

#include <cuda.h>            // CUtensorMap and the encoder's signature; the function itself is looked up at run time
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>

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

// ---- bulk-tensor tile kernel (1- and 2-byte elements) --------------------------------------
// N = 16 / ES elements make a 16-byte vector.  A block moves the tile of TI = 128 / ES input
// columns (i: one 128-byte line) by 256 output columns (o).  The input is described to the copy
// engine as (i, o / N, o % N, rest...), so the 128-byte lines of the shared image are ordered
// [o % N][o / N]: with the 128-byte swizzle (16-byte unit u of line n sits at unit u ^ (n & 7))
// the eight lanes of a quarter warp, which hold consecutive o / N, read one unit each of eight
// lines N apart without a bank conflict.  Thread (l, r) reads the N x N micro-block (lines o =
// N r + v, unit l), transposes it in registers and writes N vectors into the dense output image
// [i][o], where the same eight lanes fill 128 contiguous bytes.  One bulk-tensor store writes the
// image; edges need no code (loads beyond the extents read zeros, stores are clipped).
struct TmP {
    u32 tiles_i, tiles_o, n2, tiles;   // tiles along i and o, extent of the first batch dimension, tiles in all
    u64 status;       // mapped host word: set when the wait for a tile's copy runs out
    u64 wait_ns;
};

__device__ __forceinline__ u32 smem_addr(const void* p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ u64 now_ns() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

// start the copy of tile t into the image at `image`; completion is counted on `bar`
template <int ES>
__device__ __forceinline__ void tma_fetch(const CUtensorMap* map, const TmP& p, u32 t, u32 image, u32 bar) {
    constexpr int N = 16 / ES, R = 256 / N, TI = 128 / ES;
    const u32 ti = t % p.tiles_i; t /= p.tiles_i;
    const u32 to = t % p.tiles_o; t /= p.tiles_o;
    const u32 c2 = t % p.n2, c3 = t / p.n2;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(32768u) : "memory");
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 :: "r"(image), "l"(map), "r"(ti * TI), "r"(to * R), "r"(0u), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// Persistent: block b moves tiles b, b + grid, ...; two input images (the copy of the tile after
// next starts as soon as every thread has its micro-block of the current one in registers) and
// one output image (its store is waited for just before the next tile's vectors are written).
template <int ES>
__global__ void __launch_bounds__(ES == 2 ? 256 : 128)
shuffle_tma_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                   const __grid_constant__ TmP p) {
    constexpr int N = 16 / ES;            // micro-block side
    constexpr int R = 256 / N;            // micro-block rows of a tile
    constexpr int TI = 128 / ES;          // tile extent along i
    constexpr u32 kTile = 32768;          // bytes of an image
    extern __shared__ unsigned char dyn[];
    __shared__ __align__(8) u64 bars[2];

    const int r = threadIdx.x % R, l = threadIdx.x / R;
    const u32 in_s = (smem_addr(dyn) + 1023u) & ~1023u;       // the swizzle pattern repeats every 1024 bytes
    const u32 out_s = in_s + 2 * kTile;
    const u32 bar_s = smem_addr(bars);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar_s + 8));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (blockIdx.x < p.tiles) tma_fetch<ES>(&in_map, p, blockIdx.x, in_s, bar_s);
        if (blockIdx.x + gridDim.x < p.tiles) tma_fetch<ES>(&in_map, p, blockIdx.x + gridDim.x, in_s + kTile, bar_s + 8);
    }
    u32 it = 0;
    for (u32 t = blockIdx.x; t < p.tiles; t += gridDim.x, ++it) {
        const u32 stage = it & 1u, parity = (it >> 1) & 1u;
        {   // wait for the tile, at most p.wait_ns
            u32 done = 0;
            u64 t0 = 0;
            while (true) {
                asm volatile("{ .reg .pred q; mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2, %3; selp.u32 %0, 1, 0, q; }"
                             : "=r"(done) : "r"(bar_s + 8 * stage), "r"(parity), "r"(20000u) : "memory");
                if (done) break;
                const u64 now = now_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > p.wait_ns) {
                    if (p.status) *reinterpret_cast<volatile u32*>(p.status) = 1u;
                    return;
                }
            }
        }
        u32 in[N][4];
        const u32 image = in_s + stage * kTile;
#pragma unroll
        for (int v = 0; v < N; ++v) {
            const u32 a = image + (u32)(v * R + r) * 128u + (u32)((l ^ (r & 7)) * 16);
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(in[v][0]), "=r"(in[v][1]), "=r"(in[v][2]), "=r"(in[v][3]) : "r"(a));
        }
        // the previous tile's store has read the output image; everyone has read this input image
        if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0 && t + 2 * gridDim.x < p.tiles)
            tma_fetch<ES>(&in_map, p, t + 2 * gridDim.x, image, bar_s + 8 * stage);
#pragma unroll
        for (int w = 0; w < N; ++w) {
            u32 out[4];
            if constexpr (ES == 2) {
                // element w of rows 2q and 2q+1 -> word q
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    out[q] = __byte_perm(in[2 * q][w >> 1], in[2 * q + 1][w >> 1], (w & 1) ? 0x7632 : 0x5410);
            } else {
                // byte w of rows 4q .. 4q+3 -> word q
                const u32 sel = ((4u + (w & 3)) << 4) | (u32)(w & 3);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const u32 lo = __byte_perm(in[4 * q][w >> 2], in[4 * q + 1][w >> 2], sel);
                    const u32 hi = __byte_perm(in[4 * q + 2][w >> 2], in[4 * q + 3][w >> 2], sel);
                    out[q] = __byte_perm(lo, hi, 0x5410);
                }
            }
            const u32 a = out_s + (u32)(N * l + w) * (256u * ES) + (u32)r * 16u;
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" :: "r"(a), "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            u32 q = t;
            const u32 ti = q % p.tiles_i; q /= p.tiles_i;
            const u32 to = q % p.tiles_o; q /= p.tiles_o;
            const u32 c2 = q % p.n2, c3 = q / p.n2;
            asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                         :: "l"(&out_map), "r"(to * 256u), "r"(ti * TI), "r"(c2), "r"(c3), "r"(out_s) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    if (threadIdx.x == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

typedef CUresult (*tensor_map_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

enum { kTmaSmem = 3 * 32768 + 1024 };     // two input images, one output image, alignment slack

struct TmaHost {
    int sm_count = 0;
    std::mutex mu;
    bool tried = false;
    tensor_map_encode_fn encode = nullptr;
    volatile u32* status_host = nullptr;
    u64 status_dev = 0;
};
TmaHost g_tma;

// the encoder and the mapped status word, once per process; false when the driver offers neither
bool tma_ready() {
    std::lock_guard<std::mutex> lock(g_tma.mu);
    if (g_tma.tried) return g_tma.encode != nullptr;
    g_tma.tried = true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess || !fn) { cudaGetLastError(); return false; }
    void* host = nullptr; void* dev = nullptr;
    if (cudaHostAlloc(&host, 64, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(&dev, host, 0) != cudaSuccess) { cudaGetLastError(); return false; }
    int dev_id = 0;
    if (cudaGetDevice(&dev_id) != cudaSuccess ||
        cudaDeviceGetAttribute(&g_tma.sm_count, cudaDevAttrMultiProcessorCount, dev_id) != cudaSuccess || g_tma.sm_count < 1) {
        cudaGetLastError();
        return false;
    }
    *static_cast<volatile u32*>(host) = 0;
    g_tma.status_host = static_cast<volatile u32*>(host);
    g_tma.status_dev = (u64)dev;
    for (int es = 1; es <= 2; ++es) {
        const void* k = es == 1 ? (const void*)shuffle_tma_kernel<1> : (const void*)shuffle_tma_kernel<2>;
        if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kTmaSmem) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
    }
    g_tma.encode = reinterpret_cast<tensor_map_encode_fn>(fn);
    return true;
}

// Can the tile case in p (dims[0] = i, dims[1] = o, then the rest) go through the copy engine?
bool tma_eligible(const ShP& p, int k, int es, u64 dst, u64 src) {
    if (es > 2 || k > 4) return false;
    const i64 N = 16 / es, TI = 128 / es;
    if (dst % 16 || src % 16) return false;
    if (p.ss[0] != 1 || p.ds[1] != 1 || p.n[1] % N) return false;
    for (int d = 0; d < k; ++d) {
        if (d != 0 && (p.ss[d] * es) % 16) return false;
        if (d != 1 && (p.ds[d] * es) % 16) return false;
        if (p.n[d] >= (1ll << 31) || p.ss[d] * es >= (1ll << 40) || p.ds[d] * es >= (1ll << 40)) return false;
    }
    // whole tiles are moved: not worth it when the padding exceeds a quarter
    const double area = (double)((p.n[0] + TI - 1) / TI * TI) * (double)((p.n[1] + 255) / 256 * 256);
    return area <= 1.25 * (double)p.n[0] * (double)p.n[1];
}

template <int ES> cudaError_t launch_tma(const ShP& p, int k, cudaStream_t s, bool* encoded) {
    constexpr i64 N = 16 / ES, TI = 128 / ES, R = 256 / N;
    const CUtensorMapDataType dt = ES == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
    const i64 n2 = k > 2 ? p.n[2] : 1, n3 = k > 3 ? p.n[3] : 1;
    const i64 ss2 = k > 2 ? p.ss[2] * ES : 16, ss3 = k > 3 ? p.ss[3] * ES : 16;
    const i64 ds2 = k > 2 ? p.ds[2] * ES : 16, ds3 = k > 3 ? p.ds[3] * ES : 16;
    CUtensorMap in_map, out_map;
    {
        const cuuint64_t dims[5] = {(cuuint64_t)p.n[0], (cuuint64_t)(p.n[1] / N), (cuuint64_t)N, (cuuint64_t)n2, (cuuint64_t)n3};
        const cuuint64_t strides[4] = {(cuuint64_t)(p.ss[1] * N * ES), (cuuint64_t)(p.ss[1] * ES), (cuuint64_t)ss2, (cuuint64_t)ss3};
        const cuuint32_t box[5] = {(cuuint32_t)TI, (cuuint32_t)R, (cuuint32_t)N, 1, 1};
        const cuuint32_t one[5] = {1, 1, 1, 1, 1};
        if (g_tma.encode(&in_map, dt, 5, reinterpret_cast<void*>(p.src), dims, strides, box, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { *encoded = false; return cudaSuccess; }
    }
    {
        const cuuint64_t dims[4] = {(cuuint64_t)p.n[1], (cuuint64_t)p.n[0], (cuuint64_t)n2, (cuuint64_t)n3};
        const cuuint64_t strides[3] = {(cuuint64_t)(p.ds[0] * ES), (cuuint64_t)ds2, (cuuint64_t)ds3};
        const cuuint32_t box[4] = {256, (cuuint32_t)TI, 1, 1};
        const cuuint32_t one[4] = {1, 1, 1, 1};
        if (g_tma.encode(&out_map, dt, 4, reinterpret_cast<void*>(p.dst), dims, strides, box, one, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { *encoded = false; return cudaSuccess; }
    }
    *encoded = true;
    TmP t;
    t.tiles_i = (u32)((p.n[0] + TI - 1) / TI);
    t.tiles_o = (u32)((p.n[1] + 255) / 256);
    t.n2 = (u32)n2;
    t.status = g_tma.status_dev;
    t.wait_ns = 2000000000ull;
    const i64 tiles = (i64)t.tiles_i * t.tiles_o * n2 * n3;
    if (tiles > 0x7fffffffll) { *encoded = false; return cudaSuccess; }
    t.tiles = (u32)tiles;
    const i64 resident = 2ll * g_tma.sm_count;                 // two blocks per SM (shared memory)
    const unsigned grid = (unsigned)(tiles < resident ? tiles : resident);
    shuffle_tma_kernel<ES><<<grid, ES == 2 ? 256 : 128, kTmaSmem, s>>>(in_map, out_map, t);
    return cudaGetLastError();
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
    if (g_tma.status_host && *g_tma.status_host) {
        *g_tma.status_host = 0;
        return b200_detail_fail(B200_ERR_TIMEOUT, "b200_dimshuffle: an earlier call gave up waiting for a tile copy; its output is incomplete");
    }
    if (tiled && tma_eligible(p, k, es, dst, src) && tma_ready()) {
        bool encoded = false;
        e = es == 1 ? launch_tma<1>(p, k, s, &encoded) : launch_tma<2>(p, k, s, &encoded);
        if (encoded) {
            if (e != cudaSuccess) {
                char msg[160];
                snprintf(msg, sizeof msg, "b200_dimshuffle: %s", cudaGetErrorString(e));
                return b200_detail_fail(B200_ERR_CUDA, msg);
            }
            return B200_OK;
        }
    }
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
