// Kernel skeletons of the compound-optree engine for sm_100a.
//
// One op-tree assignment is lowered on the host into one or more *passes*; for
// each pass the code generator emits a small struct `S<V>` (operand loads, the
// fused element expression, the store or the reduction epilogue) and one of the
// skeletons below supplies everything else: the thread mapping, 128-bit
// vectorised coalesced access, warp-shuffle / shared-memory block reductions,
// split reductions finished by the last block to arrive, and the conversions
// and rounding on store.  The file is self-contained (no system headers) so the
// same text compiles under NVRTC at run time and under nvcc at build time.
//
// Frame.  A pass sees every tensor as (K, N): K = extent of the axis that is
// kept, N = extent of the axis the loop runs along (the reduced axis, or the
// contiguous axis of an element-wise pass).  Strides are in elements.
// "Lanes" are the V elements one thread handles per step: along N in
// ew_kernel / red_rows_kernel, along K in red_cols_kernel.
//
// What replaces what in neon (neon/backends/cuda_templates.py):
//   ew_kernel        -- _ew_template + "loop" stage with ew_out  (:45-86)
//   red_rows_kernel  -- "loop" + "red32"/"red" + "red_out" stages (:88-135);
//                       one block (or sub-warp) per kept index, optionally
//                       several blocks per index
//   red_cols_kernel  -- the same stages when the reduced axis is the strided
//                       one (axis 0 of a row-major tensor): threads map to
//                       neighbouring kept indices so every load is coalesced,
//                       where the reference walks down columns
//   conversions      -- _common_round / _common_fp16_to_fp32 (:189-372)
//   rng_bits, frand  -- _common_urand_gen / _common_frand (:165-186), replaced
//                       by a counter-based generator (no state pool, no race)
//   red_* helpers    -- _reduction_ops (:577-613)
#pragma once

typedef long long i64;
typedef unsigned long long u64;
typedef unsigned int u32;
typedef unsigned short u16;
typedef unsigned char u8;

#define DEV __device__ __forceinline__
#define B200_FLT_MAX 3.402823466e+38f

namespace b200 {

// First statement of every generated kernel.  Launched with the "programmatic stream
// serialization" attribute, a kernel's blocks may become resident while the previous kernel of
// the stream still runs: griddepcontrol.wait holds them until that kernel has completed and its
// writes are visible (a no-op after a plain launch); launch_dependents lets the next kernel's
// blocks in as soon as every block of this one has started.
DEV void grid_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

enum { F32 = 0, F16 = 1, BF16 = 2, I32 = 3, U32 = 4, I16 = 5, U16 = 6, I8 = 7, U8 = 8 };
// OP_MOM_MEAN / OP_MOM_M2 are a PAIR of neighbouring reduction slots (r, r + 1) that together
// carry the first two moments of one expression: see "moments" below.
enum { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2, OP_ARGMAX = 3, OP_ARGMIN = 4, OP_MOM_MEAN = 5, OP_MOM_M2 = 6 };

template <int DT> struct dt_size { enum { value = (DT == F32 || DT == I32 || DT == U32) ? 4 : (DT == I8 || DT == U8) ? 1 : 2 }; };

// ------------------------------------------------------------------ raw access
// BYTES in {1,2,4,8,16,32}; data lands in 32-bit words (sub-word loads zero-extend).
template <int BYTES, bool NC> DEV void ld_raw(const char* p, u32* w) {
    if constexpr (BYTES == 32) {
        uint4 a, b;
        if constexpr (NC) { a = __ldg(reinterpret_cast<const uint4*>(p)); b = __ldg(reinterpret_cast<const uint4*>(p) + 1); }
        else { a = *reinterpret_cast<const uint4*>(p); b = *(reinterpret_cast<const uint4*>(p) + 1); }
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
    } else if constexpr (BYTES == 16) {
        uint4 a;
        if constexpr (NC) a = __ldg(reinterpret_cast<const uint4*>(p)); else a = *reinterpret_cast<const uint4*>(p);
        w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    } else if constexpr (BYTES == 8) {
        uint2 a;
        if constexpr (NC) a = __ldg(reinterpret_cast<const uint2*>(p)); else a = *reinterpret_cast<const uint2*>(p);
        w[0] = a.x; w[1] = a.y;
    } else if constexpr (BYTES == 4) {
        if constexpr (NC) w[0] = __ldg(reinterpret_cast<const u32*>(p)); else w[0] = *reinterpret_cast<const u32*>(p);
    } else if constexpr (BYTES == 2) {
        if constexpr (NC) w[0] = __ldg(reinterpret_cast<const u16*>(p)); else w[0] = *reinterpret_cast<const u16*>(p);
    } else {
        if constexpr (NC) w[0] = __ldg(reinterpret_cast<const u8*>(p)); else w[0] = *reinterpret_cast<const u8*>(p);
    }
}

template <int BYTES> DEV void st_raw(char* p, const u32* w) {
    if constexpr (BYTES == 32) {
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
        *(reinterpret_cast<uint4*>(p) + 1) = make_uint4(w[4], w[5], w[6], w[7]);
    } else if constexpr (BYTES == 16) {
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2*>(p) = make_uint2(w[0], w[1]);
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<u32*>(p) = w[0];
    } else if constexpr (BYTES == 2) {
        *reinterpret_cast<u16*>(p) = (u16)w[0];
    } else {
        *reinterpret_cast<u8*>(p) = (u8)w[0];
    }
}

// ------------------------------------------------------------------ conversions
DEV float h2f(u32 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"((u16)h)); return f; }
DEV void h2f2(u32 hh, float& lo, float& hi) {
    asm("{.reg .b16 a, b; mov.b32 {a, b}, %2; cvt.f32.f16 %0, a; cvt.f32.f16 %1, b;}" : "=f"(lo), "=f"(hi) : "r"(hh));
}
DEV u32 f2h_rn(float f) { u16 r; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
DEV u32 f2h_rz(float f) { u16 r; asm("cvt.rz.f16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
DEV u32 f2h2_rn(float lo, float hi) { u32 r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
DEV float bf2f(u32 b) { return __uint_as_float(b << 16); }
DEV u32 f2bf_rn(float f) { u16 r; asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
DEV u32 f2bf2_rn(float lo, float hi) { u32 r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }

// words of V stored elements -> V floats
template <int DT, int V> DEV void cvt_in(const u32* w, float* out) {
    if constexpr (DT == F32) {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = __uint_as_float(w[i]);
    } else if constexpr (DT == I32) {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = (float)(int)w[i];
    } else if constexpr (DT == U32) {
#pragma unroll
        for (int i = 0; i < V; ++i) out[i] = (float)w[i];
    } else if constexpr (DT == F16) {
        if constexpr (V == 1) out[0] = h2f(w[0]);
        else {
#pragma unroll
            for (int i = 0; i < V / 2; ++i) h2f2(w[i], out[2 * i], out[2 * i + 1]);
        }
    } else if constexpr (DT == BF16) {
        if constexpr (V == 1) out[0] = bf2f(w[0]);
        else {
#pragma unroll
            for (int i = 0; i < V / 2; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
        }
    } else if constexpr (DT == I16 || DT == U16) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            u32 x = (V == 1) ? w[0] : ((w[i / 2] >> (16 * (i & 1))) & 0xffffu);
            out[i] = (DT == I16) ? (float)(short)x : (float)x;
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            u32 x = (V == 1) ? w[0] : ((w[i / 4] >> (8 * (i & 3))) & 0xffu);
            out[i] = (DT == I8) ? (float)(signed char)x : (float)x;
        }
    }
}

// typed vector load of V consecutive elements starting `off` elements after base
template <int DT, int V, bool NC> DEV void ld_f(u64 base, i64 off, float* out) {
    constexpr int B = dt_size<DT>::value * V;
    u32 w[(B + 3) / 4];
    ld_raw<B, NC>(reinterpret_cast<const char*>(base) + off * dt_size<DT>::value, w);
    cvt_in<DT, V>(w, out);
}
template <int DT, int V, bool NC> DEV void ld_w(u64 base, i64 off, u32* w) {
    ld_raw<dt_size<DT>::value * V, NC>(reinterpret_cast<const char*>(base) + off * dt_size<DT>::value, w);
}
// int32 index load (take / one-hot addressing)
DEV int ld_idx(u64 base, i64 off) { return __ldg(reinterpret_cast<const int*>(base) + off); }

// ------------------------------------------------------------------ mixed-precision add / subtract
// d = a + c and d = a - c with a a stored 16-bit float and c, d fp32: one instruction
// (add.f32.f16 / sub.f32.f16, sm_100) instead of a conversion followed by an fp32 add.  The
// 16-bit operand is converted exactly, so the result is bit for bit that of cvt + add.rn.f32.
// `w` are the loaded words of a V-element vector, `i` the lane (a constant once unrolled).
template <int DT, int HI, bool SUB> DEV float mx_half(u32 w, float c) {
    float d;
    if constexpr (DT == F16) {
        if constexpr (SUB) {
            if constexpr (HI) asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; sub.rn.f32.f16 %0, hi, %2;}" : "=f"(d) : "r"(w), "f"(c));
            else asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; sub.rn.f32.f16 %0, lo, %2;}" : "=f"(d) : "r"(w), "f"(c));
        } else {
            if constexpr (HI) asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f32.f16 %0, hi, %2;}" : "=f"(d) : "r"(w), "f"(c));
            else asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f32.f16 %0, lo, %2;}" : "=f"(d) : "r"(w), "f"(c));
        }
    } else {
        if constexpr (SUB) {
            if constexpr (HI) asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; sub.rn.f32.bf16 %0, hi, %2;}" : "=f"(d) : "r"(w), "f"(c));
            else asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; sub.rn.f32.bf16 %0, lo, %2;}" : "=f"(d) : "r"(w), "f"(c));
        } else {
            if constexpr (HI) asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f32.bf16 %0, hi, %2;}" : "=f"(d) : "r"(w), "f"(c));
            else asm("{.reg .b16 lo, hi; mov.b32 {lo, hi}, %1; add.rn.f32.bf16 %0, lo, %2;}" : "=f"(d) : "r"(w), "f"(c));
        }
    }
    return d;
}
template <int DT, int V> DEV float mx_add(const u32* w, int i, float c) {
    if constexpr (V == 1) return mx_half<DT, 0, false>(w[0], c);
    else return (i & 1) ? mx_half<DT, 1, false>(w[i >> 1], c) : mx_half<DT, 0, false>(w[i >> 1], c);
}
template <int DT, int V> DEV float mx_sub(const u32* w, int i, float c) {
    if constexpr (V == 1) return mx_half<DT, 0, true>(w[0], c);
    else return (i & 1) ? mx_half<DT, 1, true>(w[i >> 1], c) : mx_half<DT, 0, true>(w[i >> 1], c);
}

// ------------------------------------------------------------------ fast math
// Used by generated code unless the backend asks for IEEE / libm versions.
// Each stays within a few fp32 ulp (far inside the 1e-5 parity bound) and
// costs a fraction of the instructions, which is what bounds kernels with few
// bytes per element.
DEV float ex2_approx(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
DEV float rcp_approx(float x) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
DEV float fast_sqrt(float x) { float r; asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
DEV float fast_div(float a, float b) { float r; asm("div.approx.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
// exp: 2^(x log2 e) with the product carried in two pieces (t + r), so that the error does not
// grow with |x| as it does for ex2(x * log2e) alone; at most 3 ulp.  Results below the normal
// range are flushed to zero.
DEV float fast_exp(float x) {
    const float t = x * 1.44269502162933349609375f;              // log2(e) rounded to fp32
    float r = __fmaf_rn(x, 1.44269502162933349609375f, -t);      // what that product lost, exactly
    r = __fmaf_rn(x, 1.925963033500011e-8f, r);                  // + x * (log2(e) - its fp32 value)
    return ex2_approx(t) * (1.0f + r * 0.693147182464599609375f);   // 2^(t + r) ~ 2^t (1 + r ln 2)
}
// tanh: odd polynomial x + x^3 Q(x^2) below 0.6 (least-squares fit, 1.2 ulp),
// 1 - 2/(e^(2|x|) + 1) with the sign of x above it
DEV float fast_tanh(float x) {
    const float ax = fabsf(x);
    const float e = ex2_approx(ax * 2.885390082f);
    float big = __fmaf_rn(rcp_approx(e + 1.0f), -2.0f, 1.0f);
    big = copysignf(big, x);
    const float u = x * x;
    float q = __fmaf_rn(u, -0.005895146634429693f, 0.02079596184194088f);
    q = __fmaf_rn(q, u, -0.053783826529979706f);
    q = __fmaf_rn(q, u, 0.13331924378871918f);
    q = __fmaf_rn(q, u, -0.33333298563957214f);
    const float small = __fmaf_rn(x * u, q, x);
    return ax < 0.6f ? small : big;
}

// ------------------------------------------------------------------ random bits
struct Rng { u32 k0, k1; };

// 32 random bits for a 64-bit counter: one multiplicative hash, keyed per launch
DEV u32 rng_hash(const Rng& g, u32 lo, u32 hi) {
    u32 x = lo * 0x9E3779B1u + g.k0;
    x ^= x >> 16; x *= 0x21F0AAADu;
    x ^= x >> 15; x *= 0x735A2D97u;
    x ^= x >> 15;
    x ^= g.k1 + hi * 0x632BE5ABu;
    return x;
}
DEV u32 rng_bits(const Rng& g, u64 idx) { return rng_hash(g, (u32)idx, (u32)(idx >> 32)); }
// The key of a launch's random stream: its parameters -- or, for a launch that is replayed from a
// recorded graph, the two words at `tab`, which the host fills before every replay with the key
// an eager launch would have been given at that point.
DEV Rng rng_key(u32 k0, u32 k1, u64 tab) {
    Rng g{k0, k1};
    if (tab) {
        const uint2 k = *reinterpret_cast<const uint2*>(tab);
        g.k0 = k.x; g.k1 = k.y;
    }
    return g;
}
// 16-bit float stores need at most 13 random bits per element (the top bits of
// the word), so eight neighbouring elements share ONE hash: group = idx >> 3 is
// hashed, the four element pairs of the group take successive steps of a linear
// congruential chain from it, the even element of a pair reads the pair's word
// as it is and the odd element reads it rotated left by 19, so that at the full
// fp16 width the even element's rounding is decided by the word's top 13 bits
// and the odd element's by its low 13 bits.
DEV u32 rng_chain(u32 h) { return h * 0x2C9277B5u + 0xAC564B05u; }
DEV u32 rng_chain_word(u32 h) { return h ^ (h >> 16); }
DEV u32 rng_bits_pair(const Rng& g, u64 idx) {
    u32 h = rng_bits(g, idx >> 3);
    const int s = (int)(idx >> 1) & 3;
    for (int j = 0; j < s; ++j) h = rng_chain(h);
    const u32 w = s ? rng_chain_word(h) : h;
    return (idx & 1) ? __funnelshift_l(w, w, 19) : w;
}
DEV float frand(const Rng& g, u64 idx) { return __uint2float_rn(rng_bits(g, idx)) * 2.3283064365386963e-10f; }

// ------------------------------------------------------------------ rounding on store
// Stochastic rounding of an fp32 value to `mb` mantissa bits: add a uniform
// fraction of one mb-bit ulp to the magnitude, truncate.  Done on the bit
// pattern: the top (23-mb) bits of the random word are added below the kept
// mantissa and the discarded bits cleared; a carry rounds the magnitude up with
// probability equal to the discarded fraction.  (Same stored value as the
// float formulation e = val & 0xff800000; e *= 2^(-32-mb); fma.rz(e, rz(urand),
// val) & mask: only the carry out of the discarded bits matters, and that is
// decided by the top 23-mb bits of urand.)
struct SrCtx { u32 shift; u32 mask; };
DEV SrCtx sr_ctx(int mb) { SrCtx c; c.shift = (u32)(9 + mb); c.mask = 0xffffffffu << (23 - mb); return c; }
DEV float sr_f32(float v, u32 urand, const SrCtx& c) {
    return __uint_as_float((__float_as_uint(v) + (urand >> c.shift)) & c.mask);
}
DEV float sr_int_pre(float v, u32 urand) {     // value to truncate for integer stores
    float fr = copysignf(__uint2float_rz(urand), v);
    fr = __fmul_rz(fr, 2.3283064365386963e-10f);
    return __fadd_rz(fr, v);
}
DEV u32 f2h2_rz(float lo, float hi) { u32 r; asm("cvt.rz.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
DEV u32 f2bf2_rz(float lo, float hi) { u32 r; asm("cvt.rz.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
DEV u32 f2bf_rz(float f) { u16 r; asm("cvt.rz.bf16.f32 %0, %1;" : "=h"(r) : "f"(f)); return r; }
template <int DT> DEV u32 f2i_rn(float v) {
    if constexpr (DT == I32) { int r; asm("cvt.rni.sat.s32.f32 %0, %1;" : "=r"(r) : "f"(v)); return (u32)r; }
    else if constexpr (DT == U32) { u32 r; asm("cvt.rni.sat.u32.f32 %0, %1;" : "=r"(r) : "f"(v)); return r; }
    else if constexpr (DT == I16) { short r; asm("cvt.rni.sat.s16.f32 %0, %1;" : "=h"(r) : "f"(v)); return (u32)(u16)r; }
    else if constexpr (DT == U16) { u16 r; asm("cvt.rni.sat.u16.f32 %0, %1;" : "=h"(r) : "f"(v)); return r; }
    else if constexpr (DT == I8) { int r; asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v)); return (u32)r & 0xffu; }
    else { u32 r; asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(r) : "f"(v)); return r & 0xffu; }
}
template <int DT> DEV u32 f2i_rz(float v) {
    if constexpr (DT == I32) { int r; asm("cvt.rzi.sat.s32.f32 %0, %1;" : "=r"(r) : "f"(v)); return (u32)r; }
    else if constexpr (DT == I16) { short r; asm("cvt.rzi.sat.s16.f32 %0, %1;" : "=h"(r) : "f"(v)); return (u32)(u16)r; }
    else { int r; asm("cvt.rzi.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v)); return (u32)r & 0xffu; }
}

// V floats -> words of V stored elements.  SR: 0 nearest, else stochastic with
// ctx `c` and per-lane random words `ur`.
template <int DT, int V, bool SR> DEV void cvt_out(const float* v, u32* w, const SrCtx& c, const u32* ur) {
    if constexpr (DT == F32) {
#pragma unroll
        for (int i = 0; i < V; ++i) w[i] = __float_as_uint(SR ? sr_f32(v[i], ur[i], c) : v[i]);
    } else if constexpr (DT == F16) {
        if constexpr (SR) {
            if constexpr (V == 1) w[0] = f2h_rz(sr_f32(v[0], ur[0], c));
            else {
#pragma unroll
                for (int i = 0; i < V / 2; ++i)
                    w[i] = f2h2_rz(sr_f32(v[2 * i], ur[2 * i], c), sr_f32(v[2 * i + 1], ur[2 * i + 1], c));
            }
        } else {
            if constexpr (V == 1) w[0] = f2h_rn(v[0]);
            else {
#pragma unroll
                for (int i = 0; i < V / 2; ++i) w[i] = f2h2_rn(v[2 * i], v[2 * i + 1]);
            }
        }
    } else if constexpr (DT == BF16) {
        if constexpr (SR) {
            if constexpr (V == 1) w[0] = f2bf_rz(sr_f32(v[0], ur[0], c));
            else {
#pragma unroll
                for (int i = 0; i < V / 2; ++i)
                    w[i] = f2bf2_rz(sr_f32(v[2 * i], ur[2 * i], c), sr_f32(v[2 * i + 1], ur[2 * i + 1], c));
            }
        } else {
            if constexpr (V == 1) w[0] = f2bf_rn(v[0]);
            else {
#pragma unroll
                for (int i = 0; i < V / 2; ++i) w[i] = f2bf2_rn(v[2 * i], v[2 * i + 1]);
            }
        }
    } else {
        constexpr bool SRI = SR && (DT == I32 || DT == I16 || DT == I8);   // unsigned: nearest only
        constexpr int PER = 4 / dt_size<DT>::value;
#pragma unroll
        for (int i = 0; i < (V + PER - 1) / PER; ++i) w[i] = 0;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            u32 x;
            if constexpr (SRI) x = f2i_rz<DT>(sr_int_pre(v[i], ur[i])); else x = f2i_rn<DT>(v[i]);
            if constexpr (PER == 1) w[i] = x;
            else w[i / PER] |= x << ((32 / PER) * (i % PER));
        }
    }
}

// Random words for the V lanes of a store whose lane i has element index idx0 + i*step.
// PAIR: 16-bit float stores (eight elements per hash).  ALIGNED: idx0 % V == 0 and
// step == 1, so a vector never straddles a group or a 2^32 boundary and the
// 64-bit arithmetic is done once per vector instead of once per lane.
// TOP13: the caller only looks at the top 13 bits of each word (an fp16 store at 10
// mantissa bits), so the odd element's rotation can be a plain shift.
template <int V, bool PAIR, bool ALIGNED, bool TOP13 = false>
DEV void rng_lanes(const Rng& g, u64 idx0, i64 step, u32* ur) {
    if constexpr (ALIGNED && V > 1) {
        if constexpr (PAIR) {
            // V divides 8 and idx0 % V == 0: the vector lies inside one group of eight
            const u64 grp = idx0 >> 3;
            u32 h = rng_hash(g, (u32)grp, (u32)(grp >> 32));
            const int s0 = (int)(idx0 >> 1) & 3;          // 0 when V == 8
            for (int j = 0; j < s0; ++j) h = rng_chain(h);
#pragma unroll
            for (int j = 0; j < V / 2; ++j) {
                const u32 w = (V == 8) ? (j ? rng_chain_word(h) : h) : ((s0 + j) ? rng_chain_word(h) : h);
                ur[2 * j] = w;
                ur[2 * j + 1] = TOP13 ? (w << 19) : __funnelshift_l(w, w, 19);
                h = rng_chain(h);
            }
        } else {
            const u32 lo = (u32)idx0, hi = (u32)(idx0 >> 32);
#pragma unroll
            for (int i = 0; i < V; ++i) ur[i] = rng_hash(g, lo + i, hi);
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const u64 idx = idx0 + (u64)(i * step);
            ur[i] = PAIR ? rng_bits_pair(g, idx) : rng_bits(g, idx);
        }
    }
}

template <int DT, int V, bool SR> DEV void st_f(u64 base, i64 off, const float* v, const SrCtx& c, const u32* ur) {
    constexpr int B = dt_size<DT>::value * V;
    u32 w[(B + 3) / 4];
    cvt_out<DT, V, SR>(v, w, c, ur);
    st_raw<B>(reinterpret_cast<char*>(base) + off * dt_size<DT>::value, w);
}
template <int DT> DEV void st_one(u64 base, i64 off, float v) {
    SrCtx c; c.shift = 0; c.mask = 0;
    st_f<DT, 1, false>(base, off, &v, c, nullptr);
}
// arg-reduction index straight into an integer tensor (float_ew.py:451-454)
template <int DT> DEV void st_index(u64 base, i64 off, int idx) {
    if constexpr (DT == F32 || DT == F16 || DT == BF16) st_one<DT>(base, off, (float)idx);
    else { u32 w = (u32)idx; st_raw<dt_size<DT>::value>(reinterpret_cast<char*>(base) + off * dt_size<DT>::value, &w); }
}

// ------------------------------------------------------------------ reduction algebra
DEV float red_init(int op) { return (op == OP_SUM || op >= OP_MOM_MEAN) ? 0.f : (op == OP_MAX || op == OP_ARGMAX) ? -B200_FLT_MAX : B200_FLT_MAX; }
DEV int red_init_idx(int op) { return op >= OP_MOM_MEAN ? 0 : -1; }
// the slot carries an int next to its value: the index of an arg reduction, the count of a moments pair
DEV bool red_is_arg(int op) { return op >= OP_ARGMAX; }
// fold one element in; strict comparison keeps the first index a thread sees
DEV void red_acc(int op, float& a, int& ai, float v, int vi) {
    switch (op) {
        case OP_SUM: a += v; break;
        case OP_MAX: a = fmaxf(a, v); break;
        case OP_MIN: a = fminf(a, v); break;
        case OP_ARGMAX: if (v > a) { a = v; ai = vi; } break;
        default: if (v < a) { a = v; ai = vi; } break;
    }
}
// merge two partial results; equal extrema resolve to the smaller index
DEV void red_merge(int op, float& a, int& ai, float b, int bi) {
    switch (op) {
        case OP_SUM: a += b; break;
        case OP_MAX: a = fmaxf(a, b); break;
        case OP_MIN: a = fminf(a, b); break;
        case OP_ARGMAX: if (b > a || (b == a && (unsigned)bi < (unsigned)ai)) { a = b; ai = bi; } break;
        default: if (b < a || (b == a && (unsigned)bi < (unsigned)ai)) { a = b; ai = bi; } break;
    }
}

// ------------------------------------------------------------------ moments
// sum(e) and sum((e - m)^2) of one expression e in ONE pass over the data, for statements such
// as a variance whose second sum is centred on a value m that itself needs the first sum (the
// reference makes two passes, cuda_templates.py "loop" stage per reduction).  Slots r and r + 1
// of a pass hold the pair.
//   while a thread accumulates:  acc[r][i]   sum of (e - K) over the lane's elements
//                                acc[r+1][i] sum of (e - K)^2
//                                acci[r][0]  elements seen so far, acci[r+1][0] bits of K,
//     K = the first element the thread saw (a shift that keeps the squares small);
//   from the thread level up:    a[r] mean, ai[r] count, a[r+1] sum of squared deviations from
//     that mean; two such triples merge exactly (Chan, Golub, LeVeque 1979):
//     mean = mean_a + d * n_b / n,  M2 = M2_a + M2_b + d^2 * n_a * n_b / n,  d = mean_b - mean_a;
//   before generated code sees them (finish_slots): a[r] = mean * count = sum(e), a[r+1] = M2.
// Generated code then turns M2 into sum((e - m)^2) = M2 + n (mean - m)^2 for its own m.
template <int V> DEV void mom_acc_vec(float (&s1)[V], float (&s2)[V], int& cnt, int& kbits, const float (&x)[V]) {
    if (cnt == 0) kbits = __float_as_int(x[0]);
    const float K = __int_as_float(kbits);
#pragma unroll
    for (int i = 0; i < V; ++i) { const float d = x[i] - K; s1[i] += d; s2[i] = __fmaf_rn(d, d, s2[i]); }
    cnt += V;
}
DEV void mom_acc_one(float& s1, float& s2, int& cnt, int& kbits, float x) {
    if (cnt == 0) kbits = __float_as_int(x);
    const float d = x - __int_as_float(kbits);
    s1 += d; s2 = __fmaf_rn(d, d, s2); cnt += 1;
}
DEV void mom_merge(float& mean, int& n, float& m2, float mean_b, int n_b, float m2_b) {
    if (n_b > 0) {
        const int na = n, nt = n + n_b;
        const float f = (float)n_b * rcp_approx((float)nt);     // a weight: one ulp of it is far below the result's
        const float d = mean_b - mean;
        m2 = m2 + m2_b + d * d * ((float)na * f);
        mean = __fmaf_rn(d, f, mean);
        n = nt;
    }
}
// slot r of a pass and its partner (r + 1, clamped so that dead code stays in bounds)
#define B200_PARTNER(r, NR) ((r) + 1 < (NR) ? (r) + 1 : (r))

// per-lane accumulators of a thread -> one value per slot
template <class S, int NR, int V>
DEV void lanes_to_thread(float (&acc)[NR][V], int (&acci)[NR][V], float* a, int* ai) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        if (S::op(r) == OP_MOM_MEAN) {
            const int r2 = B200_PARTNER(r, NR);
            float s1 = acc[r][0], s2 = acc[r2][0];
#pragma unroll
            for (int i = 1; i < V; ++i) { s1 += acc[r][i]; s2 += acc[r2][i]; }
            const int n = acci[r][0];
            float mean = 0.f, m2 = 0.f;
            if (n > 0) {
                const float dm = s1 * rcp_approx((float)n);
                mean = __int_as_float(acci[r2][0]) + dm;
                m2 = fmaxf(__fmaf_rn(-s1, dm, s2), 0.f);
            }
            a[r] = mean; ai[r] = n; a[r2] = m2; ai[r2] = 0;
        } else if (S::op(r) != OP_MOM_M2) {
            a[r] = acc[r][0]; ai[r] = acci[r][0];
#pragma unroll
            for (int i = 1; i < V; ++i) red_merge(S::op(r), a[r], ai[r], acc[r][i], acci[r][i]);
        }
    }
}
// a <- a merged with b, slot by slot (pairs jointly)
template <class S, int NR> DEV void merge_slots(float* a, int* ai, const float* b, const int* bi) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        if (S::op(r) == OP_MOM_MEAN) {
            const int r2 = B200_PARTNER(r, NR);
            mom_merge(a[r], ai[r], a[r2], b[r], bi[r], b[r2]);
        } else if (S::op(r) != OP_MOM_M2) {
            red_merge(S::op(r), a[r], ai[r], b[r], bi[r]);
        }
    }
}
// merge with the thread `o` lanes away (xor butterfly step)
template <class S, int NR> DEV void shfl_merge(float* a, int* ai, int o) {
    float b[NR]; int bi[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        b[r] = __shfl_xor_sync(0xffffffffu, a[r], o);
        bi[r] = red_is_arg(S::op(r)) ? __shfl_xor_sync(0xffffffffu, ai[r], o) : -1;
    }
    merge_slots<S, NR>(a, ai, b, bi);
}
// what generated epilogues read: the mean slot of a moments pair becomes the plain sum
template <class S, int NR> DEV void finish_slots(float* a, const int* ai) {
#pragma unroll
    for (int r = 0; r < NR; ++r) if (S::op(r) == OP_MOM_MEAN) a[r] *= (float)ai[r];
}

// ================================================================== element-wise
// MODE 0: 2-d, vector index -> (k, n) by division; grid.x * BLOCK * UNROLL >= K * nvec.
// MODE 1: flat (K == 1, all operands contiguous), scalar tail of N % V elements.
// MODE 2: 2-d with long rows: blockIdx.y/z select the row, blockIdx.x tiles it.
// MODE 3: flat over a contiguous 2-d tensor whose row length is p.flat_bpr times the elements
//         one block handles: like MODE 1, but k carries the row of the block for statements
//         that need element coordinates; the grid is (p.flat_bpr, rows), so the row is
//         blockIdx.y/z and no thread divides.
// IDX32: the host guarantees that element counts and byte offsets fit 32 bits, so vector
//        indices are computed in 32-bit arithmetic (widening multiply-adds for addresses).
// One evaluated vector into the per-lane accumulators.  Generated code sets S::FUSED and
// provides S::accum when every reduction of the pass is a sum and the accumulation can absorb
// an operand's conversion (mx_add); otherwise eval + the generic reduction step.  Lane i has
// element index idx0 + i * idx_step (arg reductions).
template <class S, class P, int NR, int V>
DEV void accumulate(const P& p, const typename S::H& h, const typename S::L& l, i64 k, i64 n,
                    int idx0, int idx_step, float (&acc)[NR][V], int (&acci)[NR][V]) {
    if constexpr (S::FUSED) {
        S::accum(p, h, l, k, n, acc, acci);
    } else {
        float out[NR][V];
        S::eval(p, h, l, k, n, out);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            if (S::op(r) == OP_MOM_MEAN) {
                const int r2 = B200_PARTNER(r, NR);
                mom_acc_vec<V>(acc[r], acc[r2], acci[r][0], acci[r2][0], out[r]);
            } else if (S::op(r) != OP_MOM_M2) {
#pragma unroll
                for (int i = 0; i < V; ++i) red_acc(S::op(r), acc[r][i], acci[r][i], out[r][i], idx0 + i * idx_step);
            }
        }
    }
}
// the same for one element of a row's scalar tail (lane 0 of the accumulators)
template <class S, int NR, int V>
DEV void accumulate_one(const float (&out)[NR][1], int idx, float (&acc)[NR][V], int (&acci)[NR][V]) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        if (S::op(r) == OP_MOM_MEAN) {
            const int r2 = B200_PARTNER(r, NR);
            mom_acc_one(acc[r][0], acc[r2][0], acci[r][0], acci[r2][0], out[r][0]);
        } else if (S::op(r) != OP_MOM_M2) {
            red_acc(S::op(r), acc[r][0], acci[r][0], out[r][0], idx);
        }
    }
}

// The work of one block: `bx` is the block's index along x (MODE 3: among all blocks), `row` its
// row (MODE 2 and 3).
template <template <int> class SV, class P, int V, int BLOCK, int UNROLL, int MODE, bool IDX32 = false>
DEV void ew_body(const P& p, u32 bx, i64 row) {
    typedef SV<V> S;
    constexpr bool FLAT = MODE == 1 || MODE == 3;
    const i64 nvec = p.nvec;                     // vectors per row (FLAT: all vectors)
    const i64 total = MODE == 0 ? p.K * nvec : nvec;
    const i64 base = IDX32 ? (i64)(bx * (u32)(BLOCK * UNROLL) + threadIdx.x)
                           : (i64)bx * (BLOCK * UNROLL) + threadIdx.x;
    i64 krow = 0;
    if constexpr (MODE == 2) krow = row;
    // MODE 3: k carries, instead of the row r itself, the amount to add to a flat index of row r to
    // get the element index in the enclosing tensor: lin_0 + r * lin_r
    if constexpr (MODE == 3) krow = p.lin_0 + row * p.lin_r;
    if (MODE == 2 && krow >= p.K) return;
    typename S::L l[UNROLL];
    typename S::H h[UNROLL];
    i64 kk[UNROLL], nn[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        i64 g = base + (i64)u * BLOCK;
        if (g < total) {
            if constexpr (MODE != 0 && IDX32) { kk[u] = krow; nn[u] = (i64)((u32)g * (u32)V); }
            else if constexpr (MODE != 0) { kk[u] = krow; nn[u] = g * V; }
            else if (nvec <= 0x7fffffffLL && g <= 0x7fffffffLL) {
                u32 q = (u32)g / (u32)nvec; kk[u] = q; nn[u] = (i64)((u32)g - q * (u32)nvec) * V;
            } else { kk[u] = g / nvec; nn[u] = (g - kk[u] * nvec) * V; }
            S::load_l(p, kk[u], nn[u], l[u]);
            if (MODE != 2 || u == 0) S::load_h(p, kk[u], h[u]);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        i64 g = base + (i64)u * BLOCK;
        if (g < total) {
            float out[1][V];
            S::eval(p, MODE == 2 ? h[0] : h[u], l[u], kk[u], nn[u], out);
            S::store(p, kk[u], nn[u], out[0]);
        }
    }
    if constexpr (FLAT && V > 1) {               // scalar tail: N % V elements
        typedef SV<1> S1;
        const i64 t = nvec * V + (i64)bx * BLOCK + threadIdx.x;
        if (bx == 0 && t < p.N) {
            typename S1::L l1; typename S1::H h1;
            S1::load_l(p, 0, t, l1); S1::load_h(p, 0, h1);
            float out[1][1];
            S1::eval(p, h1, l1, 0, t, out);
            S1::store(p, 0, t, out[0]);
        }
    }
}

template <template <int> class SV, class P, int V, int BLOCK, int UNROLL, int MODE, bool IDX32 = false>
DEV void ew_kernel(const P& p) {
    const i64 row = (MODE == 2 || MODE == 3) ? (i64)blockIdx.y + (i64)blockIdx.z * gridDim.y : 0;
    if constexpr (MODE == 3) {
        if (row >= p.flat_rows) return;              // a grid padded in z
        ew_body<SV, P, V, BLOCK, UNROLL, MODE, IDX32>(p, (u32)row * p.flat_bpr + blockIdx.x, row);
    } else {
        ew_body<SV, P, V, BLOCK, UNROLL, MODE, IDX32>(p, blockIdx.x, row);
    }
}
// ================================================================== split-reduction finish
// Partials of reduction r, kept index k, split j live at r*K*SPLIT + j*pj + k*pk.
template <class S, class P>
DEV void write_partial(const P& p, i64 k, int j, i64 pj, i64 pk, const float* a, const int* ai) {
    float* pv = reinterpret_cast<float*>(p.part_v);
    int* pi = reinterpret_cast<int*>(p.part_i);
#pragma unroll
    for (int r = 0; r < S::NRED; ++r) {
        i64 o = (i64)r * p.K * p.split + j * pj + k * pk;
        pv[o] = a[r];
        if (red_is_arg(S::op(r))) pi[o] = ai[r];
    }
}

// ================================================================== finishing a reduction across GPUs
// One process per GPU, tensors sharded by columns: a reduction along the rows of a shard ends
// with the other GPUs' results for the same rows.  Instead of leaving that to a collective
// launched after the kernel, the thread that holds a row's final local result exchanges it
// itself: it stores the result into the exchange area of EVERY rank (peer-mapped memory, plain
// stores over NVLink), waits until its own area holds every rank's result for that row, and
// merges the W results in rank order -- the same order on every GPU, so all of them end up with
// the same bits.  Nothing is read from a peer.
// Every 32-bit word travels in an aligned 64-bit store together with the launch number
// (payload in the low half, launch number in the high half): such a store arrives whole or not
// at all, so a word is valid exactly when its high half shows the current launch number, and
// no fence is needed between "data" and "flag" -- a system-scope fence in the tail of a
// bandwidth-bound kernel costs several microseconds, two of them cost more than the exchange.
// A launch uses half `epoch & 1` of the area, so a rank that is one launch ahead never
// overwrites what a slower rank still reads (it cannot get two ahead: it needs this rank's
// results first).  The wait is bounded in time: a rank that never arrives sets bit 2 of the
// status word and the kernel carries on to its end.
// Area layout, both halves alike: entry[W][cap] of two 64-bit words (value, index or count).
//   P fields: x_table (device array of W area addresses), x_epoch and x_base (the launch number
//   is x_epoch + the 32-bit word at x_base, never 0 and the same on every rank: the word lets a
//   recorded launch sequence be replayed with fresh numbers without touching its parameters),
//   x_rank, x_world, x_cap, x_col0 (first global column of the shard, added to arg-reduction indices).
//   S::XCHG enables it; S::xc(r) says whether slot r spans the shards (a reduction of a
//   replicated operand does not: every rank already holds the full result).
DEV void st_sys_u64(u64* p, u64 v) { asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory"); }
DEV u64 ld_sys_u64(const u64* p) { u64 v; asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
DEV u64 xchg_ns() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

// PUT: this thread also publishes (a, ai) as this GPU's result; without it the thread only
// collects (a block of a cluster whose leader block publishes).  `base`: first entry slot of the
// pass when one launch exchanges the results of several passes.
template <class S, class P, int NR, bool PUT = true>
DEV void xchg_rows(const P& p, i64 k, float* a, int* ai, u32 base = 0) {
    const u32 W = p.x_world, me = p.x_rank;
    const u32 epoch = p.x_epoch + *reinterpret_cast<const u32*>(p.x_base);
    const u64 tag = (u64)epoch << 32;
    const u64* table = reinterpret_cast<const u64*>(p.x_table);
    const u64 half = (u64)(epoch & 1u) * ((u64)W * p.x_cap * 16u);
#pragma unroll
    for (int r = 0; r < NR; ++r)
        if (S::xc(r) && (S::op(r) == OP_ARGMAX || S::op(r) == OP_ARGMIN)) ai[r] += p.x_col0;
    for (u32 q = 0; PUT && q < W; ++q) {
        u64* entry = reinterpret_cast<u64*>(__ldg(table + q) + half) + (u64)me * p.x_cap * 2u;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            if (!S::xc(r)) continue;
            u64* e = entry + ((u64)(base + r) * p.K + k) * 2u;
            st_sys_u64(e, tag | __float_as_uint(a[r]));
            if (red_is_arg(S::op(r))) st_sys_u64(e + 1, tag | (u32)ai[r]);
        }
    }
    float own[NR]; int owni[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) { own[r] = a[r]; owni[r] = ai[r]; }
    const u64* mine = reinterpret_cast<const u64*>(__ldg(table + me) + half);
    u64 t0 = 0;
    bool gave_up = false;
    for (u32 q = 0; q < W; ++q) {
        const u64* entry = mine + (u64)q * p.x_cap * 2u;
        float b[NR]; int bi[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            b[r] = red_init(S::op(r)); bi[r] = red_init_idx(S::op(r));
            if (!S::xc(r)) continue;
            const u64* e = entry + ((u64)(base + r) * p.K + k) * 2u;
#pragma unroll
            for (int w = 0; w < 2; ++w) {
                if (w == 1 && !red_is_arg(S::op(r))) continue;
                u64 v = ld_sys_u64(e + w);
                while ((v >> 32) != (tag >> 32) && !gave_up) {
                    if (t0 == 0) {
                        t0 = xchg_ns();
                        // a wait of this launch has already run out: do not wait the limit again
                        if (p.status && (*reinterpret_cast<volatile int*>(p.status) & 4)) gave_up = true;
                    } else if (xchg_ns() - t0 > p.wait_ns) {
                        if (p.status) atomicOr(reinterpret_cast<int*>(p.status), 4);
                        gave_up = true;
                    }
                    v = ld_sys_u64(e + w);
                }
                if (w == 0) b[r] = __uint_as_float((u32)v); else bi[r] = (int)(u32)v;
            }
        }
        if (q == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) { a[r] = b[r]; ai[r] = bi[r]; }
        } else {
            merge_slots<S, NR>(a, ai, b, bi);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) if (!S::xc(r)) { a[r] = own[r]; ai[r] = owni[r]; }
}

// ================================================================== reduce along lanes (rows)
// TPR threads cooperate on one kept index; BLOCK/TPR indices per block.
// TPR == BLOCK: one index per block and the row may be split over p.split blocks.
// The work of block number `bid` of the pass.  Returns the kept index whose epilogue this block
// has just run (its thread 0; the results of that index are complete), or -1.
template <template <int> class SV, class P, int V, int BLOCK, int TPR, int UNROLL>
DEV i64 red_rows_body(const P& p, i64 bid) {
    typedef SV<V> S;
    constexpr int NR = S::NRED;
    constexpr int RPC = BLOCK / TPR;
    const int tid = threadIdx.x;
    const int sub = tid % TPR;
    i64 k; int j;
    if constexpr (RPC == 1) { k = bid / p.split; j = (int)(bid - k * p.split); }
    else { k = bid * RPC + tid / TPR; j = 0; }
    const bool live = k < p.K;
    const i64 nvec = p.nvec;
    i64 v0 = 0, v1 = nvec;
    if constexpr (RPC == 1) { v0 = (i64)j * p.seg; v1 = v0 + p.seg < nvec ? v0 + p.seg : nvec; }

    float acc[NR][V]; int acci[NR][V];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[r][i] = red_init(S::op(r)); acci[r][i] = red_init_idx(S::op(r)); }

    if (live) {
        typename S::H h;
        S::load_h(p, k, h);
        for (i64 v = v0 + sub; v < v1; v += (i64)TPR * UNROLL) {
            typename S::L l[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) if (v + (i64)u * TPR < v1) S::load_l(p, k, (v + (i64)u * TPR) * V, l[u]);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (v + (i64)u * TPR < v1) {
                    const i64 n = (v + (i64)u * TPR) * V;
                    accumulate<S, P, NR, V>(p, h, l[u], k, n, (int)n, 1, acc, acci);
                }
            }
        }
        // scalar tail of the row (N % V elements), first split only
        if constexpr (V > 1) {
            typedef SV<1> S1;
            if (j == 0) {
                typename S1::H h1;
                S1::load_h(p, k, h1);
                for (i64 n = nvec * V + sub; n < p.N; n += TPR) {
                    typename S1::L l1;
                    S1::load_l(p, k, n, l1);
                    float out[NR][1];
                    S1::eval(p, h1, l1, k, n, out);
                    accumulate_one<S, NR, V>(out, (int)n, acc, acci);
                }
            }
        }
    }
    // lanes -> one value per thread
    float a[NR]; int ai[NR];
    lanes_to_thread<S, NR, V>(acc, acci, a, ai);
    // threads of one index -> one value
    constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) shfl_merge<S, NR>(a, ai, o);
    if constexpr (TPR > 32) {
        __shared__ float sv[NR][BLOCK / 32];
        __shared__ int si[NR][BLOCK / 32];
        const int warp = tid >> 5, lane = tid & 31;
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) { sv[r][warp] = a[r]; si[r][warp] = ai[r]; }
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                a[r] = lane < BLOCK / 32 ? sv[r][lane] : red_init(S::op(r));
                ai[r] = lane < BLOCK / 32 ? si[r][lane] : red_init_idx(S::op(r));
            }
#pragma unroll
            for (int o = (BLOCK / 32) / 2; o > 0; o >>= 1) shfl_merge<S, NR>(a, ai, o);
        }
    }
    if constexpr (RPC > 1) {
        if (live && sub == 0) {
            if constexpr (S::XCHG) xchg_rows<S, P, NR>(p, k, a, ai);
            finish_slots<S, NR>(a, ai); S::epilogue(p, k, a, ai);
        }
        return -1;
    } else {
        if (p.split == 1) {
            if (tid == 0) {
                if constexpr (S::XCHG) xchg_rows<S, P, NR>(p, k, a, ai);
                finish_slots<S, NR>(a, ai); S::epilogue(p, k, a, ai);
            }
            return k;
        }
        // several blocks per index: publish, count arrivals, last one combines in split order
        __shared__ int s_last;
        if (tid == 0) {
            write_partial<S>(p, k, j, 1, p.split, a, ai);
            __threadfence();
            int* cnt = reinterpret_cast<int*>(p.counters) + k;
            int seen = atomicAdd(cnt, 1);
            s_last = (seen == p.split - 1);
            if (s_last) *cnt = 0;                      // leave the counter clean for the next launch
        }
        __syncthreads();
        if (!s_last) return -1;
        __threadfence();
        if (tid < 32) {
            const float* pv = reinterpret_cast<const float*>(p.part_v);
            const int* pi = reinterpret_cast<const int*>(p.part_i);
#pragma unroll
            for (int r = 0; r < NR; ++r) { a[r] = red_init(S::op(r)); ai[r] = red_init_idx(S::op(r)); }
            for (int s = tid; s < p.split; s += 32) {
                float b[NR]; int bi[NR];
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    const i64 o = ((i64)r * p.K + k) * p.split;
                    b[r] = __ldcg(pv + o + s);
                    bi[r] = red_is_arg(S::op(r)) ? __ldcg(pi + o + s) : -1;
                }
                merge_slots<S, NR>(a, ai, b, bi);
            }
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) shfl_merge<S, NR>(a, ai, o2);
            if (tid == 0) {
                if constexpr (S::XCHG) xchg_rows<S, P, NR>(p, k, a, ai);
                finish_slots<S, NR>(a, ai); S::epilogue(p, k, a, ai);
            }
        }
        return k;
    }
}
template <template <int> class SV, class P, int V, int BLOCK, int TPR, int UNROLL>
DEV void red_rows_kernel(const P& p) {
    red_rows_body<SV, P, V, BLOCK, TPR, UNROLL>(p, (i64)blockIdx.x);
}
// ================================================================== reduce across lanes (cols)
// Block = CW x RH threads (CW*RH == BLOCK).  threadIdx % CW picks V neighbouring
// kept indices, threadIdx / CW a residue class of the reduced axis.
// grid = (tiles of CW*V kept indices, p.split slices of the reduced axis).
template <template <int> class SV, class P, int V, int BLOCK, int CW, int UNROLL>
DEV void red_cols_kernel(const P& p) {
    typedef SV<V> S;
    constexpr int NR = S::NRED;
    constexpr int RH = BLOCK / CW;
    const int tx = threadIdx.x % CW, ty = threadIdx.x / CW;
    const i64 k0 = ((i64)blockIdx.x * CW + tx) * V;
    const int j = blockIdx.y;
    const bool live = k0 < p.K;
    const i64 n0 = (i64)j * p.seg;
    const i64 n1 = n0 + p.seg < p.N ? n0 + p.seg : p.N;

    float acc[NR][V]; int acci[NR][V];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[r][i] = red_init(S::op(r)); acci[r][i] = red_init_idx(S::op(r)); }

    if (live) {
        typename S::H h;
        S::load_h(p, k0, h);
        for (i64 n = n0 + ty; n < n1; n += (i64)RH * UNROLL) {
            typename S::L l[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) if (n + (i64)u * RH < n1) S::load_l(p, k0, n + (i64)u * RH, l[u]);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                if (n + (i64)u * RH < n1) {
                    accumulate<S, P, NR, V>(p, h, l[u], k0, n + (i64)u * RH, (int)(n + (i64)u * RH), 0, acc, acci);
                }
            }
        }
    }
    // combine the RH residue classes through shared memory, in class order
    __shared__ float sv[NR][RH][CW * V + 1];
    __shared__ int si[NR][RH][CW * V + 1];
    __shared__ int s_last;
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int i = 0; i < V; ++i) {
            sv[r][ty][tx * V + i] = acc[r][i];
            if (red_is_arg(S::op(r))) si[r][ty][tx * V + i] = acci[r][i];
        }
    __syncthreads();
    // thread t finishes kept index (tile base + t) for t < CW*V
    const int t = threadIdx.x;
    const i64 kt = (i64)blockIdx.x * CW * V + t;
    const bool owner = t < CW * V && kt < p.K;
    float a[NR]; int ai[NR];
    if (owner) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            a[r] = sv[r][0][t]; ai[r] = red_is_arg(S::op(r)) ? si[r][0][t] : -1;
            for (int y = 1; y < RH; ++y) red_merge(S::op(r), a[r], ai[r], sv[r][y][t], red_is_arg(S::op(r)) ? si[r][y][t] : -1);
        }
    }
    if (p.split == 1) {
        if (owner) S::epilogue(p, kt, a, ai);
        return;
    }
    if (owner) write_partial<S>(p, kt, j, p.K, 1, a, ai);
    __threadfence();
    __syncthreads();
    if (t == 0) {
        int* cnt = reinterpret_cast<int*>(p.counters) + blockIdx.x;
        int seen = atomicAdd(cnt, 1);
        s_last = (seen == p.split - 1);
        if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last block of this tile: every thread folds a residue class of the splits, then as above
    {
        const float* pv = reinterpret_cast<const float*>(p.part_v);
        const int* pi = reinterpret_cast<const int*>(p.part_i);
        const int cx = threadIdx.x % (CW * V), cy = threadIdx.x / (CW * V);
        constexpr int CH = BLOCK / (CW * V) > 0 ? BLOCK / (CW * V) : 1;
        const i64 kc = (i64)blockIdx.x * CW * V + cx;
        __syncthreads();
        if (cy < CH && threadIdx.x < CH * CW * V) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                float b = red_init(S::op(r)); int bi = -1;
                if (kc < p.K) {
                    const i64 o0 = (i64)r * p.K * p.split + kc;
                    int s = cy;
                    for (; s + 3 * CH < p.split; s += 4 * CH) {       // four loads in flight
                        float v4[4]; int i4[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            v4[q] = __ldcg(pv + o0 + (i64)(s + q * CH) * p.K);
                            i4[q] = red_is_arg(S::op(r)) ? __ldcg(pi + o0 + (i64)(s + q * CH) * p.K) : -1;
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) red_merge(S::op(r), b, bi, v4[q], i4[q]);
                    }
                    for (; s < p.split; s += CH)
                        red_merge(S::op(r), b, bi, __ldcg(pv + o0 + (i64)s * p.K),
                                  red_is_arg(S::op(r)) ? __ldcg(pi + o0 + (i64)s * p.K) : -1);
                }
                sv[r][cy % RH][cx] = b;
                if (red_is_arg(S::op(r))) si[r][cy % RH][cx] = bi;
            }
        }
        __syncthreads();
        if (owner) {
            constexpr int CHR = CH < RH ? CH : RH;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                a[r] = sv[r][0][t]; ai[r] = red_is_arg(S::op(r)) ? si[r][0][t] : -1;
                for (int y = 1; y < CHR; ++y) red_merge(S::op(r), a[r], ai[r], sv[r][y][t], red_is_arg(S::op(r)) ? si[r][y][t] : -1);
            }
            S::epilogue(p, kt, a, ai);
        }
    }
}


// ================================================================== row-resident statements
// A statement with several passes over the same rows (mean -> variance ->
// normalise, row softmax ...) normally re-reads its operands from HBM once per
// pass.  When a row of the full-size operands fits in the shared memory of a
// thread-block cluster, the kernel below reads it from HBM exactly once: the
// C blocks of a cluster each stage a contiguous slice of the row with TMA bulk
// copies (cp.async.bulk, completion on an mbarrier), every pass then runs out
// of shared memory, partial reductions are exchanged through distributed
// shared memory between two hardware cluster barriers, and the last pass
// streams the result to HBM.  Clusters walk over rows persistently.
//
// The slice is staged in chunks, each with its own mbarrier: the first pass of a
// row consumes chunk by chunk as the copies land, and the last pass hands each
// chunk it has finished with to the copies of the next row, so HBM reads run
// underneath the passes.  The generated driver calls rr_begin, rr_issue_row for
// the first row, then per row rr_pass (+ rr_combine after reductions) and
// rr_row_end.  Waits are bounded in time: a copy that never completes sets
// *status and the kernel carries on to its end instead of spinning.

DEV u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }
DEV u32 cluster_rank() { u32 r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
DEV u32 cluster_index() { u32 r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r; }
DEV u32 cluster_count() { u32 r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r; }
DEV void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The same barrier when only warp 0 has written something its cluster peers will read (the
// block's exchange slot): warp 0 arrives with release semantics, the other warps relaxed, so
// they do not have to wait until their own earlier global stores have drained.
DEV void cluster_barrier_warp0_releases() {
    if ((threadIdx.x >> 5) == 0) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    else asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// store into the same shared-memory location of block `rank` of this cluster
DEV void dsmem_st(void* local, u32 rank, u32 v) {
    u32 addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
DEV u32 dsmem_ld(const void* local, u32 rank) {
    u32 addr, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
DEV void mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
DEV void mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
DEV void mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One try: the thread may be suspended by the hardware until the phase completes or, at the
// latest, for about RR_WAIT_HINT_NS -- so a waiting warp issues a handful of instructions per
// hint period instead of spinning (and taking issue slots from the block it shares the SM with).
#define RR_WAIT_HINT_NS 20000
DEV bool mbar_try_wait(u64* bar, u32 parity) {
    u32 ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(RR_WAIT_HINT_NS) : "memory");
    return ok != 0;
}
// global -> this block's shared memory, 16-byte aligned on both sides, bytes % 16 == 0
DEV void bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

enum { RR_MAX_CHUNKS = 32 };

struct RowCtx {
    u32 rank;            // block's rank in its cluster
    u32 v0, v1;          // this block's slice of the row, in V-wide vectors
    u32 cv, nc;          // vectors per chunk, chunks in the slice (each chunk has its own mbarrier)
    u32 phase;           // mbarrier parity of the row being consumed
    u32 row_parity;      // which set of exchange slots this row uses
    bool failed;
};

// THREADS * UNROLL vectors per chunk: one trip of the pass loops
template <int C, int THREADS, int UNROLL> DEV void rr_begin(RowCtx& cx, i64 nvec, u64* bars) {
    cx.rank = C > 1 ? cluster_rank() : 0;
    const u32 per = (u32)((nvec + C - 1) / C);
    cx.v0 = cx.rank * per;
    cx.v1 = cx.v0 + per < (u32)nvec ? cx.v0 + per : (u32)nvec;
    if (cx.v0 > cx.v1) cx.v0 = cx.v1;
    cx.cv = THREADS * UNROLL;
    cx.nc = (cx.v1 - cx.v0 + cx.cv - 1) / cx.cv;
    cx.phase = 0; cx.row_parity = 0; cx.failed = false;
    if (threadIdx.x == 0) {
        for (u32 c = 0; c < cx.nc; ++c) {
            // bars[c]: chunk c has landed (one arrival + its bytes); bars[RR_MAX_CHUNKS + c]:
            // every warp is done reading chunk c in the row's last pass
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bars + c)), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bars + RR_MAX_CHUNKS + c)), "r"(THREADS / 32) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
}
// one operand's part of chunk c: global -> shared, at most 32 KB per bulk copy
DEV void rr_copy(unsigned char* dst, u64 src, u32 bytes, u64* bar) {
    for (u32 off = 0; off < bytes; off += 32768u) {
        const u32 n = bytes - off < 32768u ? bytes - off : 32768u;
        bulk_g2s(dst + off, reinterpret_cast<const char*>(src) + off, n, bar);
    }
}
// ST::issue(p, cx, k, c, dyn, bars) (generated) announces and starts the copies of chunk c of row k
template <class ST, class P>
DEV void rr_issue_row(const P& p, const RowCtx& cx, i64 k, unsigned char* dyn, u64* bars) {
    if (threadIdx.x == 0 && !cx.failed)
        for (u32 c = 0; c < cx.nc; ++c) ST::issue(p, cx, k, c, dyn, bars);
}
DEV u64 global_ns() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
// Wait for one chunk, for at most limit_ns.  When the time runs out the thread
// records it in *status and stops waiting; rr_row_end makes that the outcome for
// the whole block, which then stops staging (its results are meaningless, the
// host raises on the status) but keeps taking part in every barrier so that its
// cluster peers are never left waiting.
DEV void rr_wait_parity(RowCtx& cx, u64* bar, u32 parity, u64 status, u64 limit_ns) {
    if (cx.failed || mbar_try_wait(bar, parity)) return;
    const u64 t0 = global_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_ns() - t0 > limit_ns) {
            cx.failed = true;
            if (status) atomicExch(reinterpret_cast<int*>(status), 1);
            return;
        }
    }
}
DEV void rr_wait_chunk(RowCtx& cx, u64* bar, u64 status, u64 limit_ns) {
    rr_wait_parity(cx, bar, cx.phase, status, limit_ns);
}
DEV void rr_row_end(RowCtx& cx) {
    cx.failed = __syncthreads_or(cx.failed) != 0;
    cx.phase ^= 1;
    cx.row_parity ^= 1;
}

// The work of one thread on chunk c of its block's slice: UNROLL vectors, element-wise (NR == 0:
// evaluate and store) or folded into the accumulators.
template <class S, class P, int NA, int V, int THREADS, int UNROLL>
DEV void rr_chunk(const P& q, const typename S::H& h, i64 k, const RowCtx& cx, u32 c, u32 nfull,
                  float (&acc)[NA][V], int (&acci)[NA][V]) {
    constexpr int NR = S::NRED;
    const u32 vb = cx.v0 + c * cx.cv + threadIdx.x;
    typename S::L l[UNROLL];
    if (c < nfull) {                                 // every thread has all its vectors: no bounds checks
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) S::load_l(q, k, (i64)((vb + u * THREADS) * (u32)V), l[u]);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const i64 n = (i64)((vb + u * THREADS) * (u32)V);
            if constexpr (NR == 0) {
                float out[1][V];
                S::eval(q, h, l[u], k, n, out);
                S::store(q, k, n, out[0]);
            } else {
                accumulate<S, P, NA, V>(q, h, l[u], k, n, (int)n, 1, acc, acci);
            }
        }
    } else {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u)
            if (vb + u * THREADS < cx.v1) S::load_l(q, k, (i64)((vb + u * THREADS) * (u32)V), l[u]);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            if (vb + u * THREADS < cx.v1) {
                const i64 n = (i64)((vb + u * THREADS) * (u32)V);
                if constexpr (NR == 0) {
                    float out[1][V];
                    S::eval(q, h, l[u], k, n, out);
                    S::store(q, k, n, out[0]);
                } else {
                    accumulate<S, P, NA, V>(q, h, l[u], k, n, (int)n, 1, acc, acci);
                }
            }
        }
    }
}
// every warp reports that it is done with chunk c of the row; thread 0 alone waits for all of
// them (bounded) and then starts the next row's copies into the chunk, so the other warps run
// on without a block-wide barrier
template <class ST, class P>
DEV void rr_release_chunk(const P& p, RowCtx& cx, i64 knext, u32 c, unsigned char* dyn, u64* bars) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bars + RR_MAX_CHUNKS + c);
    if (threadIdx.x == 0 && knext < p.K) {
        rr_wait_chunk(cx, bars + RR_MAX_CHUNKS + c, p.status, p.wait_ns);
        if (!cx.failed) ST::issue(p, cx, knext, c, dyn, bars);
    }
}
// accumulators of a reduction pass -> one value per warp, left in sv / si by lane 0
template <class S, int NA, int V, int THREADS>
DEV void rr_reduce_tail(float (&acc)[NA][V], int (&acci)[NA][V], float* a, int* ai,
                        float (*sv)[THREADS / 32], int (*si)[THREADS / 32]) {
    constexpr int NR = S::NRED;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    lanes_to_thread<S, NA, V>(acc, acci, a, ai);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) shfl_merge<S, NA>(a, ai, o);
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < NR; ++r) { sv[r][warp] = a[r]; if (red_is_arg(S::op(r))) si[r][warp] = ai[r]; }
    }
}

// One pass over this block's slice, chunk by chunk (operands already point at shared memory).
//   WAIT     first pass of a row: wait for each chunk's copies before touching it
//   RELEASE  last pass of a row: once all warps are done with a chunk, start the copies of
//            the same chunk of the next row (knext), so loads overlap the rest of this pass
//   NR == 0  element-wise pass (stores through S::store), else reductions into a / ai
template <template <int> class SV, class ST, class P, int V, int THREADS, int UNROLL, bool WAIT, bool RELEASE>
DEV void rr_pass(const P& q, const P& p, i64 k, i64 knext, RowCtx& cx, unsigned char* dyn, u64* bars,
                 float* a, int* ai, float (*sv)[THREADS / 32], int (*si)[THREADS / 32]) {
    typedef SV<V> S;
    constexpr int NR = S::NRED;
    constexpr int NA = NR > 0 ? NR : 1;
    float acc[NA][V]; int acci[NA][V];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[r][i] = red_init(S::op(r)); acci[r][i] = red_init_idx(S::op(r)); }
    typename S::H h;
    S::load_h(q, k, h);
    const u32 nfull = (cx.v1 - cx.v0) / cx.cv;       // chunks in which every thread has all its vectors
    for (u32 c = 0; c < cx.nc; ++c) {
        if constexpr (WAIT) rr_wait_chunk(cx, bars + c, p.status, p.wait_ns);
        rr_chunk<S, P, NA, V, THREADS, UNROLL>(q, h, k, cx, c, nfull, acc, acci);
        if constexpr (RELEASE) rr_release_chunk<ST>(p, cx, knext, c, dyn, bars);
    }
    if constexpr (NR > 0) rr_reduce_tail<S, NA, V, THREADS>(acc, acci, a, ai, sv, si);
}

// Block results of one pass -> row result, left in res[0..NR) (value bits, or the index for arg
// reductions) for every thread to read, and in a / ai of warp 0.  S::fixup (generated) may
// rewrite the finished values before they are published (the centring term of a moments pair).  Warp 0 does the combining,
// lane w standing for warp w and then for block w of the cluster, with xor butterflies (a fixed
// order, so results repeat exactly); the other warps only take part in the barriers.  Blocks
// PUSH their result into every peer's slots before the cluster barrier, so that after it each
// block reads only its own shared memory.
template <template <int> class SV, class P, int V, int C, int THREADS, int XBASE = 0>
DEV void rr_combine(const P& q, i64 k, const RowCtx& cx, float* a, int* ai, float (*sv)[THREADS / 32],
                    int (*si)[THREADS / 32], u32* slots /* [2 parities][NR][C][2] of this pass */, u32* res) {
    typedef SV<V> S;
    constexpr int NR = S::NRED;
    constexpr int NW = THREADS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    u32* mine = slots + cx.row_parity * NR * C * 2;
    __syncthreads();                                  // the warps' results are in sv / si
    if (warp == 0) {
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            a[r] = lane < NW ? sv[r][lane] : red_init(S::op(r));
            ai[r] = (red_is_arg(S::op(r)) && lane < NW) ? si[r][lane] : red_init_idx(S::op(r));
        }
#pragma unroll
        for (int o = NW / 2; o > 0; o >>= 1) shfl_merge<S, NR>(a, ai, o);
        if (C > 1 && lane < C) {                      // lane w writes this block's entry at block w
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                u32* entry = mine + (r * C + (int)cx.rank) * 2;
                dsmem_st(entry, (u32)lane, __float_as_uint(a[r]));
                if (red_is_arg(S::op(r))) dsmem_st(entry + 1, (u32)lane, (u32)ai[r]);
            }
        }
    }
    if constexpr (C > 1 && S::XCHG) {
        // the row also spans other GPUs: warp 0 folds the C block results, thread 0 of the
        // cluster's first block publishes the GPU's result to every rank, thread 0 of every
        // block collects the W results (xchg_rows) and leaves the row's result in res
        cluster_barrier_warp0_releases();
        if (warp == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const u32* entry = mine + (r * C + (lane < C ? lane : 0)) * 2;
                a[r] = __uint_as_float(entry[0]);
                ai[r] = red_is_arg(S::op(r)) ? (int)entry[1] : -1;
            }
#pragma unroll
            for (int o = C / 2; o > 0; o >>= 1) shfl_merge<S, NR>(a, ai, o);
            if (lane == 0) {
                if (cx.rank == 0) xchg_rows<S, P, NR, true>(q, k, a, ai, XBASE);
                else xchg_rows<S, P, NR, false>(q, k, a, ai, XBASE);
                finish_slots<S, NR>(a, ai);
                S::fixup(q, k, a, ai);
#pragma unroll
                for (int r = 0; r < NR; ++r) res[r] = (S::op(r) == OP_ARGMAX || S::op(r) == OP_ARGMIN) ? (u32)ai[r] : __float_as_uint(a[r]);
            }
        }
        __syncthreads();
    } else if constexpr (C > 1) {
        cluster_barrier_warp0_releases();
        // every warp folds the C block results for itself (same values, same order) and leaves
        // them in res: no hand-over between warps, so no block barrier.  res of this pass is next
        // written one row later, after a cluster barrier every warp has passed since reading it.
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const u32* entry = mine + (r * C + (lane < C ? lane : 0)) * 2;
            a[r] = __uint_as_float(entry[0]);
            ai[r] = red_is_arg(S::op(r)) ? (int)entry[1] : -1;
        }
#pragma unroll
        for (int o = C / 2; o > 0; o >>= 1) shfl_merge<S, NR>(a, ai, o);
        finish_slots<S, NR>(a, ai);
        S::fixup(q, k, a, ai);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r) res[r] = (S::op(r) == OP_ARGMAX || S::op(r) == OP_ARGMIN) ? (u32)ai[r] : __float_as_uint(a[r]);
        }
        __syncwarp();
    } else {
        if (threadIdx.x == 0) {
            if constexpr (S::XCHG) xchg_rows<S, P, NR, true>(q, k, a, ai, XBASE);
            finish_slots<S, NR>(a, ai);
            S::fixup(q, k, a, ai);
#pragma unroll
            for (int r = 0; r < NR; ++r) res[r] = (S::op(r) == OP_ARGMAX || S::op(r) == OP_ARGMIN) ? (u32)ai[r] : __float_as_uint(a[r]);
        }
        __syncthreads();
    }
}

}  // namespace b200
