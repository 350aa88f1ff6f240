"""
TEST INFRASTRUCTURE ONLY -- CPU restatement of the rounding-on-store rules.

neon's NervanaCPU has no stochastic rounding (nervanacpu.py:548 ignores the
flag), so the reference for it is the GPU kernel text.  This module restates,
with numpy integer / float64 arithmetic, exactly what that text computes:

  * ``sr_f32`` / ``sr_f16``   -- cuda_templates.py:189-235
        e   = val & 0xff800000            (sign and exponent: +-2^E)
        e  *= 2^(-32 - mantissa_bits)
        r   = cvt.rz.f32.u32(urand)
        res = fma.rz(e, r, val)           (adds a uniform fraction of one
                                           mantissa_bits-ulp, away from zero)
        res &= 0xffffffff << (23 - mantissa_bits)
        [fp16]  cvt.rz.f16.f32
  * ``sr_int``                -- cuda_templates.py:236-287 (copysign(urand*2^-32)
                                 added with rz, then cvt.rzi, saturating)
  * ``nearest_*``             -- cuda_templates.py:290-350 (cvt.rn / cvt.rni.sat)
  * ``mantissa_bits``         -- float_ew.py:833-844 (True -> 10; fp32 <= 15,
                                 fp16 <= 10, never below 1)
  * ``frand``                 -- cuda_templates.py:176-186 (urand * 2^-32)

The random words themselves do NOT follow the reference: its 3-LFSR pool is
indexed by launch geometry (cuda_templates.py:138-173) and races when more than
65536 threads run.  The CUDA backend uses a counter-based generator keyed by
(seed, launch number, element index) instead; ``rng_bits`` (and ``rng_bits_pair``
for 16-bit float stores) is the same generator in numpy so that stored values
can be compared bit for bit.  The kernels apply the rounding rule on the bit
pattern (integer add of the top random bits, mask) rather than with fma.rz;
``sr_f32`` below keeps the reference's float formulation, and the bit-exact GPU
test shows the two agree.

``compensated_sum`` restates the Kahan accumulation kernel (float_ew.py:944-1037),
which exists only as GPU kernel text in the reference.

Parity status: pinned by known answers in tests/test_sround.py, among them the
case of neon's tests/test_backend_sr.py:52-71 (1.1 at one mantissa bit gives
only 1.0 or 1.5, with the up-probability equal to the discarded fraction).
"""

import numpy as np

U32 = np.uint32
M32 = 0xFFFFFFFF


def splitmix64(x):
    """One step of the splitmix64 sequence on python ints."""
    x = (x + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    return x, z ^ (z >> 31)


def launch_key(seed, launch):
    """(key0, key1) for launch number ``launch`` of a generator seeded ``seed``."""
    _, a = splitmix64((seed & 0xFFFFFFFFFFFFFFFF) ^ 0x6A09E667F3BCC909)
    _, b = splitmix64(a ^ ((launch * 0xD1342543DE82EF95) & 0xFFFFFFFFFFFFFFFF))
    return int(b & M32), int(b >> 32)


def rng_bits(key0, key1, idx):
    """32 random bits for every element index in ``idx`` (uint64 array)."""
    idx = np.asarray(idx, dtype=np.uint64)
    lo = (idx & np.uint64(M32)).astype(np.uint64)
    hi = (idx >> np.uint64(32)).astype(np.uint64)
    m = np.uint64(M32)
    x = (lo * np.uint64(0x9E3779B1) + np.uint64(key0)) & m
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x21F0AAAD)) & m
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x735A2D97)) & m
    x ^= x >> np.uint64(15)
    x ^= (np.uint64(key1) + hi * np.uint64(0x632BE5AB)) & m
    return x.astype(U32)


def rng_bits_pair(key0, key1, idx):
    """Random word of element ``idx`` of a 16-bit float store: the eight elements of
    group idx >> 3 share one hash; pair s = (idx >> 1) & 3 of the group takes s steps
    of the chain h -> h * 0x2C9277B5 + 0xAC564B05 (and, past the first, h ^ (h >> 16));
    the even element of a pair reads the word as it is, the odd element reads it rotated
    left by 19 bits (at the full fp16 width the word's top 13 bits decide the even element's
    rounding and its low 13 bits the odd element's)."""
    idx = np.asarray(idx, dtype=np.uint64)
    h = rng_bits(key0, key1, idx >> np.uint64(3)).astype(np.uint64)
    s = ((idx >> np.uint64(1)) & np.uint64(3)).astype(np.int64)
    m = np.uint64(M32)
    for step in (1, 2, 3):
        nxt = (h * np.uint64(0x2C9277B5) + np.uint64(0xAC564B05)) & m
        h = np.where(s >= step, nxt, h)
    w = np.where(s > 0, h ^ (h >> np.uint64(16)), h).astype(U32)
    shifted = ((w << U32(19)) | (w >> U32(13))).astype(U32)
    return np.where((idx & np.uint64(1)).astype(bool), shifted, w).astype(U32)


def frand(bits):
    """cvt.rn.f32.u32 then * 2^-32."""
    return (np.asarray(bits, U32).astype(np.float32) * np.float32(2.0 ** -32)).astype(np.float32)


def _f64_to_f32_rz(x):
    x = np.asarray(x, np.float64)
    f = x.astype(np.float32)
    over = np.abs(f.astype(np.float64)) > np.abs(x)
    toward0 = np.nextafter(f, np.float32(0))
    return np.where(over, toward0, f).astype(np.float32)


def _f32_to_f16_rz(x):
    x = np.asarray(x, np.float32)
    with np.errstate(over="ignore"):
        h = x.astype(np.float16)
    big = np.isinf(h) & np.isfinite(x)
    h = np.where(big, np.copysign(np.float16(65504), x.astype(np.float16)), h).astype(np.float16)
    over = np.abs(h.astype(np.float32)) > np.abs(x)
    return np.where(over, np.nextafter(h, np.float16(0)), h).astype(np.float16)


def mantissa_bits(rounding, dtype):
    """Effective number of kept mantissa bits (float_ew.py:833-844)."""
    if not rounding:
        return 0
    if rounding is True:
        rounding = 10
    elif np.dtype(dtype) == np.float32:
        rounding = min(int(rounding), 15)
    elif np.dtype(dtype) == np.float16:
        rounding = min(int(rounding), 10)
    return max(int(rounding), 1)


def sr_f32(val, urand, mb):
    val = np.asarray(val, np.float32)
    urand = np.asarray(urand, U32)
    e = (val.view(U32) & U32(0xFF800000)).view(np.float32)
    e = (e * np.float32(2.0 ** (-32 - mb))).astype(np.float32)
    r = _f64_to_f32_rz(urand.astype(np.float64))
    res = _f64_to_f32_rz(e.astype(np.float64) * r.astype(np.float64) + val.astype(np.float64))
    mask = U32((M32 << (23 - mb)) & M32)
    return (res.view(U32) & mask).view(np.float32)


def sr_f16(val, urand, mb):
    return _f32_to_f16_rz(sr_f32(val, urand, mb))


_INT_RANGE = {"i1": (-128, 127), "i2": (-32768, 32767), "i4": (-2 ** 31, 2 ** 31 - 1),
              "u1": (0, 255), "u2": (0, 65535), "u4": (0, 2 ** 32 - 1)}


def _code(dtype):
    return np.dtype(dtype).str[1:]


def sr_int(val, urand, dtype):
    """copysign(urand * 2^-32, val) added toward zero, then truncated, saturating."""
    code = _code(dtype)
    if code[0] == "u":
        return nearest_int(val, dtype)      # cuda_templates.py:352-354
    val = np.asarray(val, np.float32)
    r = _f64_to_f32_rz(np.asarray(urand, U32).astype(np.float64))
    fr = _f64_to_f32_rz(np.copysign(r, val).astype(np.float64) * 2.0 ** -32)
    s = _f64_to_f32_rz(fr.astype(np.float64) + val.astype(np.float64))
    lo, hi = _INT_RANGE[code]
    return np.clip(np.trunc(s.astype(np.float64)), lo, hi).astype(np.dtype(dtype))


def nearest_int(val, dtype):
    """cvt.rni.<int>.f32: round to nearest even, saturating."""
    lo, hi = _INT_RANGE[_code(dtype)]
    v = np.rint(np.asarray(val, np.float32).astype(np.float64))
    v = np.where(np.isnan(v), 0, v)
    return np.clip(v, lo, hi).astype(np.dtype(dtype))


def nearest_f16(val):
    return np.asarray(val, np.float32).astype(np.float16)


def store(val, dtype, rounding=0, urand=None):
    """fp32 value -> stored element, as the kernel epilogue does (float_ew.py:437-470)."""
    dtype = np.dtype(dtype)
    mb = mantissa_bits(rounding, dtype)
    if dtype == np.float32:
        return sr_f32(val, urand, mb) if mb else np.asarray(val, np.float32)
    if dtype == np.float16:
        return sr_f16(val, urand, mb) if mb else nearest_f16(val)
    if dtype.name == "bfloat16":            # no counterpart in the reference: fp32 rule, 7 bits at most
        if mb:
            return sr_f32(val, urand, min(mb, 7)).astype(dtype)     # exact: low 16 bits are clear
        return np.asarray(val, np.float32).astype(dtype)
    return sr_int(val, urand, dtype) if mb else nearest_int(val, dtype)


def compensated_sum(s, c, a, cmp_scale=1.0, add_scale=1.0, rounding=0, urand=None):
    """One step of the Kahan accumulation kernel (float_ew.py:958-993): returns the new
    (sum, cmp) arrays in the dtype of ``s``.  fp32 arithmetic; the new sum is rounded
    with ``store`` (stochastically when ``rounding``), the compensation to nearest.
    The kernel text leaves a*add_scale - c*cmp_scale to the compiler, which may fuse
    it; the difference is taken exactly here and rounded once, which is the same
    value whenever the two products are exact (scales that are powers of two)."""
    dtype = np.asarray(s).dtype
    s32 = np.asarray(s).astype(np.float32)
    c32 = np.asarray(c).astype(np.float32)
    a32 = np.asarray(a).astype(np.float32)
    y32 = (a32.astype(np.float64) * np.float64(np.float32(add_scale))
           - c32.astype(np.float64) * np.float64(np.float32(cmp_scale))).astype(np.float32)
    t = store((s32 + y32).astype(np.float32), dtype, rounding, urand)
    t32 = t.astype(np.float32)
    cmp_new = store(((t32 - s32).astype(np.float32) - y32).astype(np.float32), dtype)
    return t, cmp_new
