"""CPU: host-side logic of the product (shapes, op planning, autograd bookkeeping in shallow
mode) and the C-ABI library itself: it must load without a GPU and export every symbol
include/litenn_b200.h declares."""
import ctypes
import os
import re

import numpy as np
import pytest

import litenn_b200 as nn
from litenn_b200 import _lib
from litenn_b200.info import InfoBroadcast, InfoConv2D, InfoReduction, InfoReshape, InfoSlice
from litenn_b200.ops import _ReduceOp, _hashable_slices
from litenn_b200.shape import TensorAxes, TensorShape

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "litenn_b200.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(lnn_\w+)\s*\(", header, re.M))
    assert len(declared) >= 45
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, f"library lacks {missing}"
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)


def test_library_fails_loudly_without_gpu():
    lib = _lib.get_lib()
    assert lib.lnn_version() == 100
    n = ctypes.c_int(-1)
    try:
        lib.lnn_device_count(ctypes.byref(n))
    except _lib.LnnError as e:
        assert e.code == _lib.E_CUDA
    if n.value <= 0:
        with pytest.raises(_lib.LnnError) as ei:
            lib.lnn_sync(0)
        assert ei.value.code == _lib.E_NOTINIT
        assert "not initialised" in str(ei.value)


def test_conv_geometry_matches_reference_rules():
    # 'same': floor/ceil split of the effective kernel, OH = max(1, int((H+PT+PB-EKH)/s + 1))
    ci = InfoConv2D(112, 112, 2, 2, 2, 1, "same")
    assert (ci.PADL, ci.PADT, ci.PADR, ci.PADB, ci.OH, ci.OW) == (0, 0, 1, 1, 56, 56)
    ci = InfoConv2D(56, 56, 3, 3, 2, 1, 1)
    assert (ci.OH, ci.OW) == (28, 28)
    ci = InfoConv2D(12, 12, 3, 3, 1, 2, "same")
    assert (ci.PADL, ci.PADR, ci.OH) == (2, 2, 12)
    with pytest.raises(ValueError):
        InfoConv2D(8, 8, 3, 3, 1, 1, (1, 2, 3))


def test_broadcast_and_reduction_info():
    b = InfoBroadcast(TensorShape((3,)), TensorShape((3, 1)))
    assert b.output_shape == (3, 3) and b.a_shape_reduction_axes == (0,) and b.b_shape_reduction_axes == (1,)
    with pytest.raises(ValueError):
        InfoBroadcast(TensorShape((2, 3)), TensorShape((4, 3)))
    r = InfoReduction(TensorShape((2, 3, 4)), TensorAxes(None), False)
    assert r.output_shape == (1,) and r.output_shape_keepdims == (1, 1, 1)
    with pytest.raises(ValueError):
        InfoReduction(TensorShape((256, 512, 1024)), TensorAxes((2, 3)), False)   # invalid on rank 3


@pytest.mark.parametrize("shape,axes,dims,needs_transpose", [
    ((256, 512, 1024), (1,), (256, 1, 1, 512, 1024), False),
    ((256, 512, 1024), None, (1, 1, 1, 256 * 512 * 1024, 1), False),
    ((256, 512, 32, 32), (2, 3), (256 * 512, 1, 1, 1024, 1), False),
    ((8, 16, 4, 4), (0, 2, 3), (1, 8, 16, 16, 1), False),
    ((4, 1000), (0,), (1, 1, 1, 4, 1000), False),
    ((2, 3, 4, 5, 6, 7), (0, 2, 4), None, True),
])
def test_reduce_plan(shape, axes, dims, needs_transpose):
    op = _ReduceOp("sum", TensorShape(shape), TensorAxes(axes, len(shape)), False)
    assert (op.transpose_axes is not None) == needs_transpose
    if dims is not None:
        assert op.dims == dims
    outer, r0, mid, r1, inner = op.dims
    assert outer * r0 * mid * r1 * inner == int(np.prod(shape))


def test_reshape_and_slice_info():
    assert InfoReshape(TensorShape((2, 512, 8, 8)), (2, -1)).output_shape == (2, 32768)
    with pytest.raises(ValueError):
        InfoReshape(TensorShape((2, 3)), (4, -1))
    s = InfoSlice(TensorShape((5, 6, 7)), _hashable_slices((2, Ellipsis, slice(None, None, -1))))
    assert s.output_shape == (6, 7) and s.begin_step == ((2, 1), (0, 1), (6, -1)) and not s.output_is_reshaped
    s = InfoSlice(TensorShape((1, 6)), _hashable_slices((0,)))
    assert s.output_is_reshaped and s.output_shape == (6,)


def test_shape_algebra():
    assert TensorShape(()) == (1,)
    assert (1,) * 2 + TensorShape((3,)) == (1, 1, 3)
    assert TensorAxes((0, 2, 3, 1)).inversed() == (0, 3, 1, 2)
    assert TensorAxes((0, 1, 2, 3)) - TensorAxes((1, 3)) == (0, 2)
    with pytest.raises(ValueError):
        TensorShape((2, 0))
    with pytest.raises(ValueError):
        TensorAxes((-1,))


def test_shard_bounds():
    from litenn_b200 import parallel
    assert [parallel.shard_bounds(4096, 8, r) for r in (0, 7)] == [(0, 512), (3584, 4096)]
    with pytest.raises(ValueError):
        parallel.shard_bounds(10, 4, 0)


def test_matmul_shape_errors():
    from litenn_b200.ops import _matmul_shapes
    assert _matmul_shapes(TensorShape((2, 3, 4, 5)), TensorShape((2, 3, 5, 6)))[:4] == (6, 4, 6, 5)
    with pytest.raises(ValueError):
        _matmul_shapes(TensorShape((4, 5)), TensorShape((6, 7)))
    with pytest.raises(ValueError):
        _matmul_shapes(TensorShape((4, 5)), TensorShape((2, 5, 7)))
