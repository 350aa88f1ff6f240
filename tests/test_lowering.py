"""CPU tests of the host lowering: every statement of the standard cases plans,
every generated kernel compiles for sm_100a, and the reference's error behaviour
for malformed programs is kept."""
import numpy as np
import pytest

from tests.cases import cfg4, standard_cases
from tests.dryrun import DryRunBackend


def _run_dry(be, case):
    arrays = case.inputs(np.random.RandomState(0))
    t = {k: be.empty(a.shape, a.dtype) for k, a in arrays.items()}
    for k, (shape, dt) in case.outputs.items():
        t[k] = be.empty(shape, dt)
    case.run(be, t)
    return t


@pytest.fixture(scope="module")
def dry():
    return DryRunBackend()


@pytest.mark.parametrize("case", standard_cases(), ids=lambda c: c.name)
def test_case_lowers_and_compiles(case, dry):
    before = len(dry.passes)
    _run_dry(dry, case)
    assert len(dry.passes) > before


def test_softmax_is_three_passes_with_deduplicated_max(dry):
    dry2 = DryRunBackend()
    dry2.compile = False
    x = dry2.empty((32000, 256))
    y = dry2.empty((32000, 256))
    y[:] = dry2.exp(x - dry2.max(x, axis=0)) / dry2.sum(dry2.exp(x - dry2.max(x, axis=0)), axis=0)
    kinds = [p.kind for p in dry2.passes]
    assert kinds == ["red_cols", "red_cols", "ew_2d"]          # max computed once


def test_axis1_statistics_use_row_kernels_and_vector_width_8_for_fp16():
    be = DryRunBackend()
    be.compile = False
    be._planner.rowres = False
    be._planner.fuse_moments = False
    _run_dry(be, cfg4(256, 401408))
    assert [p.kind for p in be.passes] == ["red_rows", "red_rows", "ew_2d"]
    assert all("V=8" in p.desc for p in be.passes)


def test_mean_and_centred_squares_share_one_pass():
    """var(x) = sum(sqr(x - sum(x) * c)) * c needs sum(x) before its own sum can start; the
    planner computes both from one pass over x (first two moments) instead of two."""
    be = DryRunBackend()
    be.compile = False
    be._planner.rowres = False
    _run_dry(be, cfg4(256, 401408))
    assert [p.kind for p in be.passes] == ["red_rows", "ew_2d"]
    assert "OP_MOM_MEAN : OP_MOM_M2" in be.passes[0].source
    # a centre that is not the mean works the same way: sum(sqr(max(x) - x))
    x, out = be.empty((64, 5000)), be.empty((64, 1))
    be.passes = []
    out[:] = be.sum(be.square(be.max(x, axis=1) - x), axis=1)
    assert [p.kind for p in be.passes] == ["red_rows"]
    assert "OP_MAX" in be.passes[0].source and "OP_MOM_M2" in be.passes[0].source
    # a centre that needs nothing from this pass leaves the statement as it is
    m = be.empty((64, 1))
    be.passes = []
    out[:] = be.sum(be.square(x - m), axis=1)
    assert [p.kind for p in be.passes] == ["red_rows"] and "OP_MOM" not in be.passes[0].source
    # reductions down the strided axis keep the two-pass form
    col = be.empty((1, 5000))
    be.passes = []
    col[:] = be.var(x, axis=0)
    assert [p.kind for p in be.passes] == ["red_cols", "red_cols"]


def test_rows_that_fit_cluster_shared_memory_become_one_row_resident_kernel():
    be = DryRunBackend()
    be.compile = False
    _run_dry(be, cfg4(256, 401408))          # 802,816-byte rows: eight blocks of 100,352 bytes, two per SM
    assert [p.kind for p in be.passes] == ["rowres"]
    pz = be.passes[0]
    assert pz.cluster == 8 and pz.smem == 100352 and pz.block == (512, 1, 1)
    be.passes = []
    _run_dry(be, cfg4(32, 4096))             # short rows: the multi-pass kernels
    assert [p.kind for p in be.passes] == ["red_rows", "ew_2d"]
    be.passes = []
    _run_dry(be, cfg4(8, 4000000))           # a row larger than eight blocks can hold
    assert "rowres" not in [p.kind for p in be.passes]


def test_rows_that_would_stage_on_8_byte_boundaries_are_not_row_resident():
    """The row-resident kernel stages rows with bulk copies, which need 16-byte aligned
    addresses and sizes: fp32 rows of 4n+2 elements and fp16 rows of 8n+4 elements put
    every other row 8 bytes off, so those statements take the multi-pass kernels."""
    be = DryRunBackend()
    be.compile = False
    for shape, dt in (((128, 4098), np.float32), ((128, 8196), np.float16), ((128, 1026), np.float32),
                      ((128, 2052), np.float16)):
        x, y = be.empty(shape, dt), be.empty(shape, dt)
        be.passes = []
        y[:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)
        assert "rowres" not in [p.kind for p in be.passes], shape
    # the same row lengths rounded to whole 16-byte units do stay resident
    for shape, dt in (((128, 4096), np.float32), ((128, 8192), np.float16)):
        x, y = be.empty(shape, dt), be.empty(shape, dt)
        be.passes = []
        y[:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)
        assert [p.kind for p in be.passes] == ["rowres"], shape
    # a view that starts 8 bytes into a 16-byte unit
    base = be.empty((128, 4100), np.float32)
    x, y = base[:, 2:4098], be.empty((128, 4096), np.float32)
    be.passes = []
    y[:] = (x - be.mean(x, axis=1)) / (be.std(x, axis=1) + 1e-3)
    assert "rowres" not in [p.kind for p in be.passes]


def test_whole_tensor_reduction_is_one_flat_pass():
    be = DryRunBackend()
    be.compile = False
    z = be.empty((512, 384), np.float16)
    tot = be.empty((1, 1))
    tot[:] = be.sum(z)
    tot[:] = be.max(be.absolute(z))
    assert [p.kind for p in be.passes] == ["red_rows", "red_rows"]
    assert "K=1 N=196608" in be.passes[0].desc


def test_reference_error_behaviour():
    be = DryRunBackend()
    be.compile = False
    a, b = be.empty((4, 6)), be.empty((5, 6))
    out = be.empty((4, 6))
    with pytest.raises(TypeError):
        out[:] = a + b                                   # float_ew.py:824-825
    with pytest.raises(TypeError):
        out[:] = be.rint(a)                              # not in the kernel vocabulary
    with pytest.raises(ValueError):
        be.onehot(be.empty((1, 6), np.int32), axis=2)


def test_whole_tensor_reductions_of_different_sizes_do_not_share_a_pass():
    """The squared-gradient norm over all layers (neon/optimizers/optimizer.py:72-96) adds
    sum(square(g)) over tensors of different sizes: one pass each, then the scalar part."""
    be = DryRunBackend()
    be.compile = False
    be.bsz = 4
    g0, g1, g2 = be.empty((96, 160)), be.empty((50, 1)), be.empty((96, 160))
    norm = be.empty((1, 1))
    norm[:] = be.sqrt(sum(be.sum(be.square(g)) for g in (g0, g1))) / be.bsz
    assert ["N=15360" in p.desc for p in be.passes] == [True, False]
    assert "N=50" in be.passes[1].desc
    be.passes = []
    norm[:] = be.sqrt(sum(be.sum(be.square(g)) for g in (g0, g2))) / be.bsz       # same size: one pass
    assert len(be.passes) == 1
    # and the lowering itself refuses what the splitter must never hand it
    from neon_b200.lowering import Statement
    from neon_b200.optree import OpTreeNode
    a, b = g0.reshape(1, g0.size), g1.reshape(1, g1.size)
    tree = OpTreeNode({"op": "assign"}, norm, be.sum(a, axis=1) + be.sum(b, axis=1))
    with pytest.raises(ValueError):
        Statement(tree.traverse([]))
    # the same for reductions along an axis: rows of 100 and of 300 elements
    s1, s2, col = be.empty((64, 100)), be.empty((64, 300)), be.empty((64, 1))
    be.passes = []
    col[:] = be.sum(s1, axis=1) + be.max(s2, axis=1)
    assert ["N=100" in p.desc for p in be.passes] == [True, False] and "N=300" in be.passes[1].desc


def test_unaligned_views_fall_back_to_narrower_vectors():
    be = DryRunBackend()
    be.compile = False
    x = be.empty((64, 100))
    out = be.empty((64, 99))
    out[:] = x[:, 1:] * 2.0                              # 4-byte aligned only, odd row length
    assert "V=1" in be.passes[-1].desc


def test_dot_inside_an_op_tree_is_split_into_its_own_launch():
    """tests/test_backend_compound_optree.py:39-58 builds trees around be.dot."""
    be = DryRunBackend()
    be.compile = False
    a, b, c = be.empty((20, 30)), be.empty((30, 40)), be.empty((20, 40))
    out = be.empty((20, 40))
    out[:] = be.dot(a, b)
    assert be.dots == 1 and not be.passes
    out[:] = be.dot(a * 2.0, b) + c
    assert be.dots == 2 and [p.kind for p in be.passes] == ["ew_flat", "ew_flat"]
    col = be.empty((20, 1))
    col[:] = be.sum(be.dot(a, b.T.T if False else b), axis=1) * 0.5
    assert be.dots == 3
