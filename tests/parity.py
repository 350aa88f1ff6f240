"""Comparison rules of the parity tests (the bar the backend is held to):
integer / index outputs bit-exact; fp32 within 1e-5 relative of the float64
checker (plus 1e-6 of the largest magnitude, for values that cancel); fp16 within
one unit in the last place of the float64 checker (plus the same 1e-6 term)."""
import numpy as np

RTOL_F32 = 1e-5


def ulp16(x):
    """Spacing of fp16 at |x| (float64 array), never below the smallest subnormal step."""
    h = np.abs(np.asarray(x, np.float64)).astype(np.float16)
    h = np.where(np.isfinite(h), h, np.float16(65504))
    return np.maximum(np.spacing(h).astype(np.float64), 2.0 ** -24)


def ulp_bf16(x):
    """Spacing of bfloat16 (8 significant bits) at |x|."""
    a = np.maximum(np.abs(np.asarray(x, np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


def check_output(name, got, want64, dtype, scale=None):
    """Assert ``got`` (device result, storage dtype) matches ``want64`` (checker run in float64)."""
    dtype = np.dtype(dtype)
    want64 = np.asarray(want64)
    assert got.shape == want64.shape, (name, got.shape, want64.shape)
    if dtype.kind in "iu":
        assert np.array_equal(got.astype(np.int64), want64.astype(np.int64)), \
            "%s: %d of %d indices differ" % (name, int((got != want64).sum()), got.size)
        return
    g = got.astype(np.float64)
    w = want64.astype(np.float64)
    if dtype.name == "bfloat16":
        noise = 1e-6 * (float(np.max(np.abs(w))) if w.size else 0.0)
        err = (np.abs(g - w) - noise) / ulp_bf16(w)
        assert np.all(err <= 1.0 + 1e-3), "%s: bf16 error %.3f ulp" % (name, err.max())
        return
    if dtype == np.float16:
        # beyond the fp16 range both sides must overflow the same way (cvt.rn gives inf, as numpy does)
        with np.errstate(over="ignore"):
            w16 = w.astype(np.float16)
        over = ~np.isfinite(w16)
        if over.any():
            edge = np.abs(w) < 65520.0 * (1 + 1e-5)          # within fp32 noise of the overflow threshold
            assert np.all((got[over] == w16[over]) | edge[over]), "%s: overflow handling differs" % name
            g, w = g[~over], w[~over]
            if not w.size:
                return
        # one fp16 ulp of the exact value, plus the fp32 rounding noise of the terms that
        # were combined (matters only where the result cancels to almost nothing and an
        # fp16 ulp is smaller than fp32 arithmetic on the operands can resolve)
        noise = 1e-6 * (float(np.max(np.abs(w))) if w.size else 0.0)
        err = (np.abs(g - w) - noise) / ulp16(w)
        assert np.all(err <= 1.0 + 1e-3), "%s: fp16 error %.3f ulp" % (name, err.max())
        return
    mag = float(np.max(np.abs(w))) if w.size else 0.0
    if scale is not None:
        atol = RTOL_F32 * scale            # caller states the magnitude the error is relative to
    else:
        atol = RTOL_F32 * max(mag, 1e-30) * 0.1
    bad = np.abs(g - w) > RTOL_F32 * np.abs(w) + atol
    assert not bad.any(), "%s: %d of %d fp32 values off; worst rel %.3g" % (
        name, int(bad.sum()), g.size, float(np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-30))))


def check_fingerprint(name, got, golden, prefix):
    """Compare a device result with the committed fingerprint of neon's NervanaCPU result."""
    from tests.cases import summarize
    fp = summarize(got)
    if "full" in fp:
        want = golden[prefix + "/full"]
        return fp["full"], want
    step = int(golden[prefix + "/step"])
    return got.reshape(-1)[::step], golden[prefix + "/sample"]
