"""CPU tests of B200Tensor subscripting: the view a subscript produces (shape, element strides,
offset) addresses exactly the elements numpy's subscript selects, for slices with steps, negative
positions, ellipsis and integer subscripts on 2- to 4-d tensors; and the errors GPUTensor raises
(neon/backends/nervanagpu.py:193-323) are raised for the same subscripts.  No device is touched:
the tensors of the dry-run backend carry made-up addresses."""
import numpy as np
import pytest

from tests.dryrun import DryRunBackend


def _random_subscript(rng, shape):
    parts = []
    for extent in shape:
        kind = rng.randint(0, 4)
        if kind == 0:
            parts.append(slice(None))
        elif kind == 1:
            parts.append(int(rng.randint(-extent, extent)))
        else:
            lo, hi = sorted(int(v) for v in rng.randint(-extent, extent + 1, 2))
            step = int(rng.choice([1, 1, 2, 3, -1, -2]))
            parts.append(slice(hi, lo, step) if step < 0 else slice(lo, hi, step))
    cut = rng.randint(0, len(parts) + 1)
    if rng.rand() < 0.3:
        keep_tail = rng.randint(0, len(parts) - cut + 1)
        parts = parts[:cut] + [Ellipsis] + (parts[len(parts) - keep_tail:] if keep_tail else [])
    elif rng.rand() < 0.3:
        parts = parts[:max(cut, 1)]                       # trailing axes left out
    return tuple(parts)


@pytest.mark.parametrize("seed", range(40))
def test_views_address_what_numpy_selects(seed):
    rng = np.random.RandomState(seed)
    be = DryRunBackend()
    for _ in range(25):
        shape = tuple(int(d) for d in rng.randint(1, 7, rng.randint(2, 5)))
        host = np.arange(int(np.prod(shape)), dtype=np.int64).reshape(shape)
        t = be.empty(shape, np.float32)
        idx = _random_subscript(rng, shape)
        want = host[idx]
        if want.size == 0 and any(isinstance(e, slice) for e in idx):
            pass                                          # empty views are legal; nothing to address
        view = t[idx]
        assert view.size == want.size, (shape, idx, view.shape, want.shape)
        offset = (view.ptr - t.ptr) // 4
        grid = np.indices(view.shape).reshape(len(view.shape), -1)
        flat = offset + sum(g * s for g, s in zip(grid, view.strides)) if view.size else np.zeros(0, np.int64)
        assert np.array_equal(np.asarray(flat, np.int64).reshape(-1), want.reshape(-1)), (shape, idx)
        # a matrix stays 2-d under integer subscripts, higher ranks drop the axis like numpy
        if len(shape) == 2:
            assert len(view.shape) == 2
        else:                                              # (tensors never have fewer than two axes)
            assert view.shape == want.shape + (1,) * max(0, 2 - want.ndim), (shape, idx)
        assert view.base is t and view._block is t._block


def test_subscript_errors():
    be = DryRunBackend()
    t = be.empty((4, 6), np.float32)
    for idx, text in (((1, 2, 3), "too many axes"), ((Ellipsis, Ellipsis), "more than one ellipsis"),
                      ((7,), "out of range"), ((0, -7), "out of range"), (("a",), "invalid subindex"),
                      ((1.5,), "invalid subindex")):
        with pytest.raises(IndexError) as e:
            t[idx]
        assert text in str(e.value), (idx, str(e.value))
    assert t[:] is t
    rows = be.empty((1, 3), np.int32)
    v = t[rows]                                           # fancy index along axis 0
    assert v.take_array[1] == 0 and v.shape == (3, 6)
    with pytest.raises(IndexError):
        t[rows, rows]
    with pytest.raises(IndexError):
        t[be.empty((1, 3), np.float32)]
    with pytest.raises(IndexError):
        t[be.empty((2, 3), np.int32)]
