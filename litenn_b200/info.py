"""Pure shape calculators with the exact semantics of litenn/core/info/*.py: they decide
output shapes, paddings and reduction axes before any kernel is launched and raise the
same ValueErrors."""
import math
from collections.abc import Iterable

from .shape import TensorAxes, TensorShape


class InfoConv2D:
    """Paddings and output extents of a 2-D window op (info/InfoConv2D.py:41-77).

    'same' pads floor((EK-1)/2) on the left/top and ceil((EK-1)/2) on the right/bottom;
    OH = max(1, int((H + PADT + PADB - EKH) / stride + 1)).
    """
    __slots__ = ["PADL", "PADR", "PADT", "PADB", "OH", "OW", "OH_T", "OW_T"]

    def __init__(self, H, W, KH, KW, stride, dilation, padding):
        EKH = (KH - 1) * dilation + 1
        EKW = (KW - 1) * dilation + 1
        OH_T = OW_T = None
        if padding == "valid":
            PADL = PADT = PADR = PADB = 0
            OH_T = H * stride + max(EKH - stride, 0)
            OW_T = W * stride + max(EKW - stride, 0)
        elif padding == "same":
            PADL = (EKW - 1) // 2
            PADT = (EKH - 1) // 2
            PADR = EKW - 1 - PADL
            PADB = EKH - 1 - PADT
            OH_T, OW_T = H * stride, W * stride
        elif isinstance(padding, int):
            PADL = PADT = PADR = PADB = padding
        elif isinstance(padding, Iterable) and not isinstance(padding, str):
            padding = tuple(int(x) for x in padding)
            if len(padding) != 4:
                raise ValueError("Invalid paddings list length.")
            PADL, PADT, PADR, PADB = padding
        else:
            raise ValueError("Invalid padding value.")
        self.PADL, self.PADR, self.PADT, self.PADB = PADL, PADR, PADT, PADB
        self.OH = max(1, int((H + PADT + PADB - EKH) / stride + 1))
        self.OW = max(1, int((W + PADL + PADR - EKW) / stride + 1))
        self.OH_T, self.OW_T = OH_T, OW_T


class InfoBroadcast:
    """numpy-style broadcast of two shapes (info/InfoBroadcast.py:40-86)."""
    __slots__ = ["a_br_shape", "a_shape_reduction_axes", "b_br_shape", "b_shape_reduction_axes", "output_shape"]

    def __init__(self, a_shape, b_shape):
        a_shape, b_shape = TensorShape(a_shape), TensorShape(b_shape)
        rank = max(a_shape.rank, b_shape.rank)
        a_br = (1,) * (rank - a_shape.rank) + a_shape
        b_br = (1,) * (rank - b_shape.rank) + b_shape
        a_red, b_red, out = [], [], []
        for axis in range(rank):
            a, b = a_br[axis], b_br[axis]
            if a != b:
                if a == 1:
                    a_red.append(axis)
                elif b == 1:
                    b_red.append(axis)
                else:
                    raise ValueError(f"operands could not be broadcast together with shapes {a_shape} {b_shape}")
            out.append(max(a, b))
        self.output_shape = TensorShape(out)
        self.a_br_shape, self.b_br_shape = TensorShape(a_br), TensorShape(b_br)
        self.a_shape_reduction_axes = TensorAxes(a_red)
        self.b_shape_reduction_axes = TensorAxes(b_red)


class InfoReduction:
    """Reduction axes bookkeeping (info/InfoReduction.py:25-50)."""
    __slots__ = ["reduction_axes", "output_axes", "output_shape", "output_shape_keepdims"]

    def __init__(self, shape, axes, keepdims):
        shape_axes = shape.axes_arange()
        if axes.is_none_axes():
            axes = shape_axes
        for axis in axes:
            if axis not in shape_axes:
                raise ValueError(f"Wrong axis {axis} not in {shape_axes}")
        self.reduction_axes = axes.sorted()
        self.output_axes = shape_axes - axes
        self.output_shape = shape[self.output_axes]          # () becomes (1,)
        self.output_shape_keepdims = TensorShape(
            1 if axis in self.reduction_axes else shape[axis] for axis in range(shape.rank))
        if keepdims:
            self.output_shape = self.output_shape_keepdims


class InfoTranspose:
    """info/InfoTranspose.py:24-35"""
    __slots__ = ["no_changes", "output_shape"]

    def __init__(self, shape, axes_order):
        if shape.rank != axes_order.rank:
            raise ValueError("axes must match the shape")
        self.output_shape = shape[axes_order]
        self.no_changes = axes_order == shape.axes_arange()


class InfoReshape:
    """Target shape with at most one -1 (info/InfoReshape.py:21-43)."""
    __slots__ = ["output_shape"]

    def __init__(self, shape, target_shape):
        out, remain, unk = [], shape.size, None
        for t in target_shape:
            t = int(t)
            if t != -1:
                if remain % t != 0:
                    raise ValueError(f"Cannot reshape {shape} to {target_shape}.")
                remain //= t
            else:
                if unk is not None:
                    raise ValueError("Can specify only one unknown dimension.")
                unk = len(out)
            out.append(t)
        if unk is not None:
            out[unk] = int(remain)
        elif remain != 1:
            raise ValueError(f"Cannot reshape {shape} to {target_shape}.")
        self.output_shape = TensorShape(out)


class InfoSlice:
    """Normalises a __getitem__ argument the way op/slice.py:54-160 does.  Result:
    output_shape, output_shape_krn (one extent per input axis), begin_step per input axis,
    output_is_reshaped (the slice selects everything, so the result is a view)."""
    __slots__ = ["output_shape", "output_shape_krn", "begin_step", "output_is_reshaped"]

    def __init__(self, input_shape, slices):
        new_slices, before_ellipsis = [], None
        for s in slices:
            if s is Ellipsis:
                before_ellipsis, new_slices = new_slices, []
                continue
            if s is not None and not isinstance(s, (int, tuple)):
                raise ValueError(f"unknown slice argument {s} of type {s.__class__}")
            new_slices.append(s)
        if before_ellipsis is not None:
            n_after = sum(1 for x in new_slices if x is not None)
            n_before = sum(1 for x in before_ellipsis if x is not None)
            new_slices = before_ellipsis + [(None, None, None)] * max(0, input_shape.rank - n_before - n_after) + new_slices
        n_axes = sum(1 for x in new_slices if x is not None)
        if n_axes > input_shape.rank:
            raise ValueError("slices arguments more than shape axes")
        new_slices += [(None, None, None)] * (input_shape.rank - n_axes)

        reshaped, out_shape, out_krn, begin_step = True, [], [], []
        i_axis = 0
        for v in new_slices:
            if v is None:
                out_shape.append(1)
                continue
            size = input_shape[i_axis]
            i_axis += 1
            if isinstance(v, int):
                if v < 0:
                    v += size
                if v < 0 or v >= size:
                    raise ValueError(f"index {v} is out of bounds for axis {i_axis} with size {size}")
                b, e, s = v, v, 1
            else:
                b, e, s = v
            if s is None:
                s = 1
            if s == 0:
                raise ValueError("slice step cannot be zero")
            if b is None:
                b = 0 if s > 0 else size - 1
            if e is None:
                e = size if s > 0 else -1
            elif e < 0:
                e += size
            if b < 0:
                b += size
            if s > 0:
                b, e = min(max(b, 0), size), min(max(e, 0), size)
            else:
                b, e = min(max(b, 0), size - 1), min(max(e, -1), size)
            if size != 1 and not (b == 0 and e == size and s == 1):
                reshaped = False
            n_out = max(0, math.ceil((e - b) / s))
            if n_out >= 1:
                out_shape.append(n_out)
            out_krn.append(max(1, n_out))
            begin_step.append((int(b), int(s)))
        self.output_is_reshaped = reshaped
        self.output_shape = TensorShape(out_shape)
        self.output_shape_krn = TensorShape(out_krn)
        self.begin_step = tuple(begin_step)
