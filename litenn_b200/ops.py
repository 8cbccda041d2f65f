"""The op layer: one Python function per operator with the names, keyword arguments,
defaults, shape errors and `output_t=` / `is_add_to_output=` conventions of
litenn/core/op/*.py.  Each function validates shapes on the host, allocates the result
Tensor, registers the grad functions and makes ONE C-ABI call per current device; the
kernels live in liblitenn_b200.so.  There is no host-side arithmetic fallback.
"""
import ctypes
import functools

import numpy as np
from collections.abc import Iterable

from . import _lib
from . import deferred as _deferred
from . import initializer as _initializer
from .devices import devices
from .info import (InfoBroadcast, InfoConv2D, InfoReduction, InfoReshape, InfoSlice, InfoTranspose)
from .shape import TensorAxes, TensorShape
from .tensor import Tensor, Tensor_zeros_like

_slice_cls = slice


def _each_device():
    """(position in the current-device list, C-ABI device slot) pairs; empty in shallow mode."""
    if devices._shallow > 0:
        return []
    return [(i, d.index) for i, d in enumerate(devices.get_current())]


def _lib_():
    return _lib.get_lib()


_UNINIT = _initializer.Uninitialized()


def _out(shape):
    """Result tensor of an op: its kernel writes every element, so no zero fill."""
    return Tensor(shape, init=_UNINIT)


# =============================================================================================
# element-wise (ref: op/element_wise_op.py)
# =============================================================================================
def _ew(name, args, input_t, output_t=None, is_add_to_output=False):
    """O (+)= f(I); registers dI += g(I, O, dO) unless output_t is given
    (element_wise_op.py:48-80)."""
    is_add_to_output = False if output_t is None else is_add_to_output
    p0, p1, flag = args
    n = input_t.shape.size
    if output_t is None:
        output_t = _out(input_t.shape)
        output_t._set_op_name(name)
        output_t._assign_gradfn(input_t, lambda O_t, dO_t: _ew_grad(name, args, input_t, O_t, dO_t))
    elif output_t.shape.size != n:
        raise ValueError(f"output_t must have size {n}")
    op = _lib.EW[name]
    for i, dev in _each_device():
        _lib_().lnn_eltwise_fwd(dev, op, output_t._ptr(i), input_t._ptr(i), n, p0, p1, flag, int(is_add_to_output))
    return output_t


def _ew_grad(name, args, input_t, O_t, dO_t):
    p0, p1, flag = args
    g = input_t.get_grad()
    for i, dev in _each_device():
        _lib_().lnn_eltwise_bwd(dev, _lib.EW[name], g._ptr(i), input_t._ptr(i), O_t._ptr(i), dO_t._ptr(i),
                                input_t.shape.size, p0, p1, flag)


def abs_op(input_t, output_t=None, is_add_to_output=False): return _ew("abs", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def abs(input_t): return abs_op(input_t)
def add_const_op(input_t, value, output_t=None, is_add_to_output=False): return _ew("add_const", (float(value), 0.0, 0), input_t, output_t, is_add_to_output)
def add_const(input_t, value): return add_const_op(input_t, value)
def sub_const_op(input_t, value, output_t=None, is_add_to_output=False): return add_const_op(input_t, -value, output_t, is_add_to_output)
def sub_const(input_t, value): return add_const(input_t, -value)


def clip_op(input_t, min_value, max_value, preserve_gradient=False, output_t=None, is_add_to_output=False):
    """Element-wise clip; with preserve_gradient=False the gradient is zero outside the range."""
    if min_value > max_value:
        raise ValueError(f"{min_value} > {max_value}")
    return _ew("clip", (float(min_value), float(max_value), int(bool(preserve_gradient))), input_t, output_t, is_add_to_output)
def clip(input_t, min_value, max_value, preserve_gradient=False): return clip_op(input_t, min_value, max_value, preserve_gradient)

def cos_op(input_t, output_t=None, is_add_to_output=False): return _ew("cos", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def cos(input_t): return cos_op(input_t)
def exp_op(input_t, output_t=None, is_add_to_output=False): return _ew("exp", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def exp(input_t): return exp_op(input_t)
def leaky_relu_op(input_t, alpha, output_t=None, is_add_to_output=False): return _ew("leaky_relu", (float(alpha), 0.0, 0), input_t, output_t, is_add_to_output)
def leaky_relu(input_t, alpha=0.1):
    fused = _deferred.try_act(input_t, alpha)       # joins a convolution that has not been launched yet
    return fused if fused is not None else leaky_relu_op(input_t, alpha)
def log_op(input_t, output_t=None, is_add_to_output=False): return _ew("log", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def log(input_t): return log_op(input_t)
def mul_const_op(input_t, value, output_t=None, is_add_to_output=False): return _ew("mul_const", (float(value), 0.0, 0), input_t, output_t, is_add_to_output)
def mul_const(input_t, value): return mul_const_op(input_t, value)
def div_const_op(input_t, value, output_t=None, is_add_to_output=False): return mul_const_op(input_t, 1.0 / value, output_t, is_add_to_output)
def div_const(input_t, value): return mul_const(input_t, 1.0 / value)
def rdiv_const_op(input_t, value, output_t=None, is_add_to_output=False): return _ew("rdiv_const", (float(value), 0.0, 0), input_t, output_t, is_add_to_output)
def rdiv_const(input_t, value): return rdiv_const_op(input_t, value)
def rsub_const_op(input_t, value, output_t=None, is_add_to_output=False): return _ew("rsub_const", (float(value), 0.0, 0), input_t, output_t, is_add_to_output)
def rsub_const(input_t, value): return rsub_const_op(input_t, value)
def relu_op(input_t, output_t=None, is_add_to_output=False): return _ew("relu", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def relu(input_t): return relu_op(input_t)
def sigmoid_op(input_t, output_t=None, is_add_to_output=False): return _ew("sigmoid", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def sigmoid(input_t): return sigmoid_op(input_t)
def sin_op(input_t, output_t=None, is_add_to_output=False): return _ew("sin", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def sin(input_t): return sin_op(input_t)
def sqrt_op(input_t, output_t=None, is_add_to_output=False): return _ew("sqrt", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def sqrt(input_t): return sqrt_op(input_t)
def square_op(input_t, output_t=None, is_add_to_output=False): return _ew("square", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def square(input_t): return square_op(input_t)
def tanh_op(input_t, output_t=None, is_add_to_output=False): return _ew("tanh", (0.0, 0.0, 0), input_t, output_t, is_add_to_output)
def tanh(input_t): return tanh_op(input_t)


_FUSED_ROW_MAX = 8192      # columns the fused row kernels keep in shared memory


def softmax(input_t, axis=-1):
    """exp(x) / sum(exp(x)) with no max-subtraction (element_wise_op.py:309-314).  Over the last
    axis of a matrix it is one kernel (and one for the gradient) with the values of the
    reference's exp / reduce_sum / div composition; other cases run that composition."""
    rank = input_t.shape.rank
    if rank == 2 and axis in (-1, 1) and input_t.shape[1] <= _FUSED_ROW_MAX and not _deferred.composed_softmax[0]:
        rows, cols = input_t.shape
        output_t = _out(input_t.shape)
        output_t._set_op_name("softmax")

        def grad(O_t, dO_t):
            g = input_t.get_grad()
            for i, dev in _each_device():
                _lib_().lnn_softmax_bwd(dev, g._ptr(i), input_t._ptr(i), dO_t._ptr(i), rows, cols)

        output_t._assign_gradfn(input_t, grad)
        for i, dev in _each_device():
            _lib_().lnn_softmax_fwd(dev, output_t._ptr(i), input_t._ptr(i), rows, cols)
        return output_t
    e = exp(input_t)
    return e / e.sum(axis, keepdims=True)


# =============================================================================================
# broadcast binary (ref: op/dual_wise_op.py)
# =============================================================================================
@functools.lru_cache(maxsize=4096)
def _bcast_info(a_shape, b_shape):
    return InfoBroadcast(a_shape, b_shape)


def _bin(name, a_t, b_t, output_t=None, is_add_to_output=False):
    is_add_to_output = False if output_t is None else is_add_to_output
    info = _bcast_info(a_t.shape, b_t.shape)
    if info.output_shape.rank > _lib.MAX_DIMS:
        raise ValueError(f"broadcast rank {info.output_shape.rank} > {_lib.MAX_DIMS} is not supported")
    if output_t is None:
        output_t = _out(info.output_shape)
        output_t._set_op_name(name)
        output_t._assign_gradfn(a_t, lambda O_t, dO_t: _bin_grad(name, info, 0, a_t, b_t, O_t, dO_t))
        output_t._assign_gradfn(b_t, lambda O_t, dO_t: _bin_grad(name, info, 1, a_t, b_t, O_t, dO_t))
    elif output_t.shape.size != info.output_shape.size:
        raise ValueError(f"output_t must have size {info.output_shape.size}")
    rank = info.output_shape.rank
    o, a, b = _lib.i64_array(info.output_shape), _lib.i64_array(info.a_br_shape), _lib.i64_array(info.b_br_shape)
    for i, dev in _each_device():
        _lib_().lnn_binary_fwd(dev, _lib.BIN[name], output_t._ptr(i), a_t._ptr(i), b_t._ptr(i), rank, o, a, b,
                               int(is_add_to_output))
    return output_t


def _bin_grad(name, info, which, a_t, b_t, O_t, dO_t):
    """Gradient of operand `which`.  When that operand was broadcast the full-size
    gradient goes to a zeroed temporary which is then reduce_sum'ed (+=) over the broadcast
    axes, exactly the reference's two steps (dual_wise_op.py:110-130)."""
    target = a_t if which == 0 else b_t
    red = info.a_shape_reduction_axes if which == 0 else info.b_shape_reduction_axes
    dst = target.get_grad()
    if red.rank != 0:
        dst = Tensor_zeros_like(dO_t)
    rank = info.output_shape.rank
    o, a, b = _lib.i64_array(info.output_shape), _lib.i64_array(info.a_br_shape), _lib.i64_array(info.b_br_shape)
    for i, dev in _each_device():
        _lib_().lnn_binary_bwd(dev, _lib.BIN[name], which, dst._ptr(i), a_t._ptr(i), b_t._ptr(i), O_t._ptr(i),
                               dO_t._ptr(i), rank, o, a, b)
    if red.rank != 0:
        reduce_sum_op(dst, red, output_t=target.get_grad(), is_add_to_output=True)


def add_op(a_t, b_t, output_t=None, is_add_to_output=False):
    if output_t is None:
        # conv2D(...) + bias.reshape(1, OC, 1, 1): the bias joins the convolution's epilogue
        fused = _deferred.try_bias(a_t, b_t) or _deferred.try_bias(b_t, a_t)
        if fused is not None:
            return fused
    return _bin("add", a_t, b_t, output_t, is_add_to_output)
def add(a_t, b_t): return add_op(a_t, b_t)
def sub_op(a_t, b_t, output_t=None, is_add_to_output=False): return _bin("sub", a_t, b_t, output_t, is_add_to_output)
def sub(a_t, b_t): return sub_op(a_t, b_t)
def mul_op(a_t, b_t, output_t=None, is_add_to_output=False): return _bin("mul", a_t, b_t, output_t, is_add_to_output)
def mul(a_t, b_t): return mul_op(a_t, b_t)
def div_op(a_t, b_t, output_t=None, is_add_to_output=False): return _bin("div", a_t, b_t, output_t, is_add_to_output)
def div(a_t, b_t): return div_op(a_t, b_t)
def max_op(a_t, b_t, output_t=None, is_add_to_output=False): return _bin("max", a_t, b_t, output_t, is_add_to_output)
def max(a_t, b_t): return max_op(a_t, b_t)
def min_op(a_t, b_t, output_t=None, is_add_to_output=False): return _bin("min", a_t, b_t, output_t, is_add_to_output)
def min(a_t, b_t): return min_op(a_t, b_t)
def binary_crossentropy_op(input_t, target_t, output_t=None, is_add_to_output=False): return _bin("binary_crossentropy", input_t, target_t, output_t, is_add_to_output)
def binary_crossentropy(input_t, target_t): return binary_crossentropy_op(input_t, target_t)


def categorical_crossentropy(input_t, target_t):
    """reduce_sum(-target * log(clip(p, 1e-7, 1-1e-7)), -1) (dual_wise_op.py:228-250)."""
    if input_t.shape.rank != 2:
        raise ValueError("input_t.shape.rank != 2")
    if target_t.shape.rank not in (1, 2):
        raise ValueError("target_t.shape.rank != 1 or 2")
    rows, cols = input_t.shape
    t_ok = tuple(target_t.shape.shape) in ((cols,), (rows, cols))
    if t_ok and cols <= _FUSED_ROW_MAX and not _deferred.composed_softmax[0] and not _deferred.reaches_trainable(target_t):
        # one kernel (and one for the gradient of the probabilities) with the values of the
        # composition below; a target that needs a gradient itself takes the composition
        t_stride = cols if target_t.shape.rank == 2 else 0
        output_t = _out((rows,))
        output_t._set_op_name("categorical_crossentropy")

        def grad(O_t, dO_t):
            g = input_t.get_grad()
            for i, dev in _each_device():
                _lib_().lnn_cce_bwd(dev, g._ptr(i), input_t._ptr(i), target_t._ptr(i), dO_t._ptr(i), rows, cols, t_stride)

        output_t._assign_gradfn(input_t, grad)
        for i, dev in _each_device():
            _lib_().lnn_cce_fwd(dev, output_t._ptr(i), input_t._ptr(i), target_t._ptr(i), rows, cols, t_stride)
        return output_t
    input_t = clip(input_t, 1e-7, 1 - 1e-7)
    return reduce_sum(-target_t * log(input_t), axes=-1)


def scale_bias_leaky_relu(x_t, g_t, b_t, alpha=0.1, output_t=None, is_add_to_output=False):
    """leaky_relu(x*g + b, alpha) for x (N,C,H,W) and g, b of C elements in ONE pass.
    Forward-only fusion of nn.mul, nn.add and nn.leaky_relu with identical roundings
    (no grad functions are registered; build the chain from the three ops to train)."""
    if x_t.shape.rank != 4 or g_t.shape.size != x_t.shape[1] or b_t.shape.size != x_t.shape[1]:
        raise ValueError("expected x (N,C,H,W) and g, b with C elements")
    is_add_to_output = False if output_t is None else is_add_to_output
    if output_t is None:
        output_t = _out(x_t.shape)
        output_t._set_op_name("scale_bias_leaky_relu")
    elif output_t.shape.size != x_t.shape.size:
        raise ValueError(f"output_t must have size {x_t.shape.size}")
    N, C, H, W = x_t.shape
    for i, dev in _each_device():
        _lib_().lnn_scale_bias_lrelu(dev, output_t._ptr(i), x_t._ptr(i), g_t._ptr(i), b_t._ptr(i), N, C, H * W,
                                     float(alpha), int(is_add_to_output))
    return output_t


# =============================================================================================
# reductions (ref: op/reduce.py)
# =============================================================================================
class _ReduceOp:
    """Host plan of one reduction: the reduced axes as at most two contiguous groups around
    one kept group ([outer][r0][mid][r1][inner]); other axis sets go through a transpose
    that moves the reduced axes last, as the reference always does (reduce.py:190-191)."""

    def __init__(self, op_type, input_shape, axes, keepdims):
        if op_type not in ("sum", "mean", "min", "max"):
            raise ValueError(f"unknown op_type {op_type}")
        self.op_type = op_type
        self.info = info = InfoReduction(input_shape, axes, keepdims)
        red = set(info.reduction_axes)
        # run-length encode axes into kept / reduced groups (size-1 axes join either kind)
        groups = []   # [is_reduced, size]
        for ax in range(input_shape.rank):
            size = input_shape[ax]
            if size == 1:
                continue
            r = ax in red
            if groups and groups[-1][0] == r:
                groups[-1][1] *= size
            else:
                groups.append([r, size])
        self.transpose_axes = None
        kinds = [g[0] for g in groups]
        sizes = [g[1] for g in groups]
        n_red_groups = sum(kinds)
        if n_red_groups == 0:
            self.dims = (input_shape.size, 1, 1, 1, 1)
        elif n_red_groups <= 2 and len(groups) <= 5 and self._fits(kinds):
            self.dims = self._layout(kinds, sizes)
        else:
            self.transpose_axes = info.output_axes + info.reduction_axes
            cols = 1
            for ax in info.reduction_axes:
                cols *= input_shape[ax]
            self.dims = (input_shape.size // cols, 1, 1, cols, 1)

    @staticmethod
    def _fits(kinds):
        # patterns K?RK?R?K? with at most two R groups and a K group between them
        s = "".join("R" if k else "K" for k in kinds)
        return s in ("R", "KR", "RK", "KRK", "RKR", "KRKR", "RKRK", "KRKRK")

    @staticmethod
    def _layout(kinds, sizes):
        s = "".join("R" if k else "K" for k in kinds)
        outer = r0 = mid = r1 = inner = 1
        if s == "R": r1 = sizes[0]
        elif s == "KR": outer, r1 = sizes
        elif s == "RK": r1, inner = sizes
        elif s == "KRK": outer, r1, inner = sizes
        elif s == "RKR": r0, mid, r1 = sizes
        elif s == "KRKR": outer, r0, mid, r1 = sizes
        elif s == "RKRK": r0, mid, r1, inner = sizes
        elif s == "KRKRK": outer, r0, mid, r1, inner = sizes
        return (outer, r0, mid, r1, inner)


@functools.lru_cache(maxsize=4096)
def _reduce_plan(op_type, input_shape, axes, keepdims):
    return _ReduceOp(op_type, input_shape, axes, keepdims)


def reduce_op(op_type, input_t, axes=None, keepdims=False, output_t=None, is_add_to_output=False):
    """op_type 'sum' | 'mean' | 'min' | 'max' (reduce.py:166-205)."""
    is_add_to_output = False if output_t is None else is_add_to_output
    op = _reduce_plan(op_type, input_t.shape, TensorAxes(axes, input_t.shape.rank), bool(keepdims))
    if output_t is None:
        output_t = _out(op.info.output_shape)
        output_t._op = op
        output_t._set_op_name(f"reduce_{op_type}")
        output_t._assign_gradfn(input_t, lambda O_t, dO_t: _reduce_grad(op, input_t, O_t, dO_t))
    elif output_t.shape.size != op.info.output_shape.size:
        raise ValueError(f"output_t must have size {op.info.output_shape.size}")
    src = input_t if op.transpose_axes is None else transpose(input_t, op.transpose_axes)
    for i, dev in _each_device():
        _lib_().lnn_reduce(dev, _lib.RED[op_type], output_t._ptr(i), src._ptr(i), *op.dims, int(is_add_to_output))
    return output_t


def _reduce_grad(op, input_t, O_t, dO_t):
    g = input_t.get_grad()
    if op.transpose_axes is None:
        for i, dev in _each_device():
            _lib_().lnn_reduce_bwd(dev, _lib.RED[op.op_type], g._ptr(i), input_t._ptr(i), dO_t._ptr(i), O_t._ptr(i), *op.dims)
        return
    # rare axis sets: gradient in the transposed layout, then transposed back with "+="
    src = transpose(input_t, op.transpose_axes)
    tmp = Tensor_zeros_like(src)
    for i, dev in _each_device():
        _lib_().lnn_reduce_bwd(dev, _lib.RED[op.op_type], tmp._ptr(i), src._ptr(i), dO_t._ptr(i), O_t._ptr(i), *op.dims)
    transpose_op(tmp, TensorAxes(op.transpose_axes).inversed(), output_t=g, is_add_to_output=True)


def reduce_sum_op(input_t, axes=None, keepdims=False, output_t=None, is_add_to_output=False): return reduce_op("sum", input_t, axes, keepdims, output_t, is_add_to_output)
def reduce_sum(input_t, axes=None, keepdims=False): return reduce_sum_op(input_t, axes, keepdims)
def reduce_mean_op(input_t, axes=None, keepdims=False, output_t=None, is_add_to_output=False): return reduce_op("mean", input_t, axes, keepdims, output_t, is_add_to_output)
def reduce_mean(input_t, axes=None, keepdims=False): return reduce_mean_op(input_t, axes, keepdims)
def reduce_min_op(input_t, axes=None, keepdims=False, output_t=None, is_add_to_output=False): return reduce_op("min", input_t, axes, keepdims, output_t, is_add_to_output)
def reduce_min(input_t, axes=None, keepdims=False): return reduce_min_op(input_t, axes, keepdims)
def reduce_max_op(input_t, axes=None, keepdims=False, output_t=None, is_add_to_output=False): return reduce_op("max", input_t, axes, keepdims, output_t, is_add_to_output)
def reduce_max(input_t, axes=None, keepdims=False): return reduce_max_op(input_t, axes, keepdims)


def reduce_variance(input_t, axes=None, keepdims=False):
    mean = reduce_mean(input_t, axes, keepdims=True)
    return reduce_mean(square(input_t - mean), axes, keepdims)


def reduce_std(input_t, axes=None, keepdims=False):
    return sqrt(reduce_variance(input_t, axes, keepdims))


def moments(input_t, axes=None, keepdims=False):
    mean = reduce_mean(input_t, axes, keepdims)
    var = reduce_mean(square(input_t - mean.reshape(mean._op.info.output_shape_keepdims)), axes, keepdims)
    return mean, var


# =============================================================================================
# data movement (ref: op/transpose.py, op/reshape.py, op/slice.py)
# =============================================================================================
def transpose_op(input_t, axes_order, output_t=None, is_add_to_output=False):
    is_add_to_output = False if output_t is None else is_add_to_output
    axes_order = TensorAxes(axes_order, input_t.shape.rank)
    info = InfoTranspose(input_t.shape, axes_order)
    if input_t.shape.rank > _lib.MAX_DIMS:
        raise ValueError(f"rank {input_t.shape.rank} > {_lib.MAX_DIMS} is not supported")
    if output_t is None:
        output_t = _out(info.output_shape)
        output_t._set_op_name("transpose")
        output_t._assign_gradfn(input_t, lambda O_t, dO_t: transpose_op(
            dO_t, axes_order.inversed(), output_t=input_t.get_grad(), is_add_to_output=True))
    elif output_t.shape.size != info.output_shape.size:
        raise ValueError(f"output_t must have size {info.output_shape.size}")
    shape = _lib.i64_array(input_t.shape)
    axes = (ctypes.c_int * axes_order.rank)(*axes_order.axes)
    for i, dev in _each_device():
        _lib_().lnn_transpose(dev, output_t._ptr(i), input_t._ptr(i), input_t.shape.rank, shape, axes, int(is_add_to_output))
    return output_t


def transpose(input_t, axes_order):
    return transpose_op(input_t, axes_order)


def reshape(input_t, target_shape):
    """Zero-copy view with a new shape (reshape.py:7-18)."""
    info = InfoReshape(input_t.shape, tuple(int(x) for x in target_shape))
    return input_t._as_ref(info.output_shape)


def flatten(input_t):
    return reshape(input_t, (input_t.shape[0], -1))


def _hashable_slices(slices):
    if not isinstance(slices, Iterable):
        slices = (slices,)
    out = []
    for x in slices:
        if isinstance(x, _slice_cls):
            out.append((x.start, x.stop, x.step))
        elif x is Ellipsis or x is None:
            out.append(x)
        else:
            out.append(int(x))
    return tuple(out)


def slice_op(input_t, slices, output_t=None, is_add_to_output=False):
    is_add_to_output = False if output_t is None else is_add_to_output
    info = InfoSlice(input_t.shape, _hashable_slices(slices))
    if input_t.shape.rank > _lib.MAX_DIMS:
        raise ValueError(f"rank {input_t.shape.rank} > {_lib.MAX_DIMS} is not supported")
    if output_t is None:
        if info.output_is_reshaped:
            return input_t.reshape(info.output_shape)
        output_t = _out(info.output_shape)
        output_t._set_op_name("slice")
        output_t._assign_gradfn(input_t, lambda O_t, dO_t: _slice_grad(info, input_t, dO_t))
    elif output_t.shape.size != info.output_shape.size:
        raise ValueError(f"output_t must have size {info.output_shape.size}")
    args = _slice_args(info, input_t.shape)
    for i, dev in _each_device():
        _lib_().lnn_slice_fwd(dev, output_t._ptr(i), input_t._ptr(i), input_t.shape.rank, *args, int(is_add_to_output))
    return output_t


def _slice_args(info, in_shape):
    return (_lib.i64_array(in_shape), _lib.i64_array(info.output_shape_krn),
            _lib.i64_array([b for b, _ in info.begin_step]), _lib.i64_array([s for _, s in info.begin_step]))


def _slice_grad(info, input_t, dO_t):
    g = input_t.get_grad()
    args = _slice_args(info, input_t.shape)
    for i, dev in _each_device():
        _lib_().lnn_slice_bwd(dev, g._ptr(i), dO_t._ptr(i), input_t.shape.rank, *args)


def slice(input_t, slices):
    return slice_op(input_t, slices)


# =============================================================================================
# pooling (ref: op/pool2D.py)
# =============================================================================================
def pool2D_op(op_type, input_t, pool_size=2, stride=2, padding="same"):
    if op_type not in ("avg", "min", "max"):
        raise ValueError(f"unknown op_type {op_type}")
    pool_size, stride = int(pool_size), int(stride)
    if pool_size < 2:
        raise ValueError(f"pool_size {pool_size} must be at least 2")
    fused = _deferred.try_pool(op_type, input_t, pool_size, stride, padding)
    if fused is not None:
        return fused
    N, IC, IH, IW = input_t.shape
    ci = InfoConv2D(IH, IW, pool_size, pool_size, stride, 1, padding)
    geom = (N, IC, IH, IW, ci.OH, ci.OW, pool_size, stride, ci.PADL, ci.PADT)
    output_t = _out((N, IC, ci.OH, ci.OW))
    output_t._set_op_name(f"{op_type}_pool2D")
    output_t._assign_gradfn(input_t, lambda O_t, dO_t: _pool_grad(op_type, geom, input_t, dO_t, O_t))
    for i, dev in _each_device():
        _lib_().lnn_pool2d_fwd(dev, _lib.POOL[op_type], output_t._ptr(i), input_t._ptr(i), *geom)
    return output_t


def _pool_grad(op_type, geom, input_t, dO_t, O_t):
    g = input_t.get_grad()
    for i, dev in _each_device():
        _lib_().lnn_pool2d_bwd(dev, _lib.POOL[op_type], g._ptr(i), input_t._ptr(i), dO_t._ptr(i), O_t._ptr(i), *geom)


def avg_pool2D(input_t, pool_size=2, stride=2, padding="same"): return pool2D_op("avg", input_t, pool_size, stride, padding)
def max_pool2D(input_t, pool_size=2, stride=2, padding="same"): return pool2D_op("max", input_t, pool_size, stride, padding)
def min_pool2D(input_t, pool_size=2, stride=2, padding="same"): return pool2D_op("min", input_t, pool_size, stride, padding)


# =============================================================================================
# matmul (ref: op/matmul.py)
# =============================================================================================
def _matmul_shapes(a_shape, b_shape):
    """A(...,M,K) x B(...,K,N) -> (...,M,N) with the reference's checks (matmul.py:75-100)."""
    if a_shape.rank != b_shape.rank:
        raise ValueError(f"Ranks are not equal. {a_shape.rank} != {b_shape.rank}")
    if a_shape.rank < 2:
        raise ValueError("Tensors rank must be at least 2.")
    M, K = a_shape[-2], a_shape[-1]
    K2, N = b_shape[-2], b_shape[-1]
    if K != K2:
        raise ValueError("A_ROWS != B_COLS")
    batch = a_shape[0:-2].size if a_shape.rank > 2 else 1
    b_batch = b_shape[0:-2].size if b_shape.rank > 2 else 1
    if batch != b_batch:
        raise ValueError(f"BATCH size {batch} != {b_batch} in shapes {a_shape} {b_shape}")
    out = TensorShape((M, N)) if a_shape.rank == 2 else TensorShape(a_shape[:-2] + (M, N))
    return batch, M, N, K, out


def _gemm(out_t, a_t, b_t, bias_t, batch, m, n, k, trans_a, trans_b, accumulate):
    passes = _lib.precision()
    for i, dev in _each_device():
        _lib_().lnn_gemm_f32(dev, out_t._ptr(i), a_t._ptr(i), b_t._ptr(i), bias_t._ptr(i) if bias_t is not None else 0,
                             batch, m, n, k, int(trans_a), int(trans_b), int(accumulate), passes)


def matmul_op(a_t, b_t, output_t=None, is_add_to_output=False):
    """Row-major A(...,M,K) x B(...,K,N).  The gradients are the transposed GEMMs
    dA += dO.B^T and dB += A^T.dO (matmul.py:64-72) issued without materialising a
    transpose: the tile engine reads either operand K-major or MN-major."""
    is_add_to_output = False if output_t is None else is_add_to_output
    batch, M, N, K, out_shape = _matmul_shapes(a_t.shape, b_t.shape)
    if output_t is None:
        output_t = _out(out_shape)
        output_t._set_op_name("matmul")
        output_t._assign_gradfn(a_t, lambda O_t, dO_t: _gemm(a_t.get_grad(), dO_t, b_t, None, batch, M, K, N, 0, 1, 1))
        output_t._assign_gradfn(b_t, lambda O_t, dO_t: _gemm(b_t.get_grad(), a_t, dO_t, None, batch, K, N, M, 1, 0, 1))
    elif output_t.shape.size != out_shape.size:
        raise ValueError(f"output_t must have size {out_shape.size}")
    _gemm(output_t, a_t, b_t, None, batch, M, N, K, 0, 0, is_add_to_output)
    return output_t


def matmul(a_t, b_t):
    return matmul_op(a_t, b_t)


def matmulc_op(a_t, b_t, output_t=None, is_add_to_output=False):
    """Column-major form A(...,K,M) x B(...,N,K) = (...,N,M) (matmul.py:33-62)."""
    return matmul_op(b_t, a_t, output_t=output_t, is_add_to_output=is_add_to_output)


def dense(input_t, weight_t, bias_t=None):
    """x.W (+ bias) in one GEMM with the bias in the epilogue; same value as nn.matmul
    followed by a broadcast add (module/Dense.py:44-48)."""
    batch, M, N, K, out_shape = _matmul_shapes(input_t.shape, weight_t.shape)
    if bias_t is not None and bias_t.shape.size != N:
        raise ValueError(f"bias must have {N} elements")
    output_t = _out(out_shape)
    output_t._set_op_name("dense")
    output_t._assign_gradfn(input_t, lambda O_t, dO_t: _gemm(input_t.get_grad(), dO_t, weight_t, None, batch, M, K, N, 0, 1, 1))
    output_t._assign_gradfn(weight_t, lambda O_t, dO_t: _gemm(weight_t.get_grad(), input_t, dO_t, None, batch, K, N, M, 1, 0, 1))
    if bias_t is not None:
        output_t._assign_gradfn(bias_t, lambda O_t, dO_t: reduce_sum_op(
            dO_t.reshape((-1, N)), 0, output_t=bias_t.get_grad(), is_add_to_output=True))
    _gemm(output_t, input_t, weight_t, bias_t, batch, M, N, K, 0, 0, 0)
    return output_t


# =============================================================================================
# convolution (ref: op/conv2D.py)
# =============================================================================================
def _conv_geom(input_shape, kernel_shape, stride, dilation, padding):
    N, IC, IH, IW = input_shape
    KO, KI, KH, KW = kernel_shape
    if KI != IC:
        raise ValueError(f"Kernel input channels {KI} does not match tensor input channels {IC}.")
    ci = InfoConv2D(IH, IW, KH, KW, stride, dilation, padding)
    g = _lib.ConvGeom(N, IC, IH, IW, KO, KH, KW, ci.OH, ci.OW, stride, dilation, ci.PADL, ci.PADT)
    return g, TensorShape((N, KO, ci.OH, ci.OW))


def conv2D(input_t, kernel_t, stride=1, dilation=1, padding="same", bias_t=None, activation=None, alpha=0.1,
           _pooled=False):
    """2-D convolution, input (N,IC,H,W), kernel (OC,IC,KH,KW) (conv2D.py:9-44).

    bias_t / activation ('leaky_relu') are optional epilogue fusions that give the same
    values as the separate nn.add / nn.leaky_relu ops; the default call is the reference's.
    """
    if input_t.shape.rank != 4 or kernel_t.shape.rank != 4:
        raise ValueError("conv2D expects (N,IC,H,W) input and (OC,IC,KH,KW) kernel")
    stride, dilation = int(stride), int(dilation)
    g, out_shape = _conv_geom(input_t.shape, kernel_t.shape, stride, dilation, padding)
    if activation not in (None, "leaky_relu"):
        raise ValueError(f"unknown activation {activation}")
    if bias_t is not None and bias_t.shape.size != g.oc:
        raise ValueError(f"bias must have {g.oc} elements")
    if activation == "leaky_relu" and alpha <= 0.0:
        # the fused gradient reads leaky_relu' off the sign of the OUTPUT, which only mirrors the
        # sign of the input for alpha > 0: other slopes run as the separate operators
        y = leaky_relu(conv2D(input_t, kernel_t, stride, dilation, padding, bias_t=bias_t), alpha)
        return pool2D_op("max", y, 2, 2, "same") if _pooled else y
    act = 1 if activation == "leaky_relu" else 0
    if not _pooled:
        # nothing upstream needs a gradient: the launch waits until the consumer is known
        lazy = _deferred.start(input_t, kernel_t, stride, dilation, padding, g, out_shape, bias_t, act, alpha)
        if lazy is not None:
            return lazy
    passes = _lib.precision()
    output_t = _out(out_shape)
    output_t._set_op_name("conv2D")
    idx_t = None
    if _pooled:
        # conv2D_block: the pool runs in the convolution's epilogue and the full-resolution
        # activation is never written; the backward pass gets the map of winning window positions
        # instead (one byte per pooled element, kept in a flat tensor used as raw storage)
        output_t = _out((g.n, g.oc, g.oh // 2, g.ow // 2))
        output_t._set_op_name("conv2D_block")
        idx_t = _out(((output_t.shape.size + 3) // 4,))
    full_shape = out_shape

    # The grad functions below are stored inside output_t, so they must not capture output_t itself
    # (a reference cycle would keep the whole chain of activations alive until the cycle collector
    # runs): they receive it as O_t.

    def pre_act_grad(O_t, dO_t):
        # gradient w.r.t. the convolution output (before the fused activation)
        if _pooled:
            cached = getattr(O_t, "_pre_act_grad", None)
            if cached is None or cached[0] is not dO_t:
                d = _out(full_shape)                    # every element is written
                t = _out(O_t.shape)                     # the winners' gradients: what the bias gradient sums
                for i, dev in _each_device():
                    _lib_().lnn_pool2x2_idx_lrelu_bwd(dev, d._ptr(i), t._ptr(i), idx_t._ptr(i), O_t._ptr(i),
                                                      dO_t._ptr(i), g.n, g.oc, g.oh, g.ow, float(alpha), act)
                cached = (dO_t, d, t)
                O_t._pre_act_grad = cached
            return cached[1]
        if not act:
            return dO_t
        cached = getattr(O_t, "_pre_act_grad", None)
        if cached is None or cached[0] is not dO_t:
            d = Tensor(O_t.shape)
            # leaky_relu'(y) from the OUTPUT sign: sign(lrelu(y)) == sign(y) for alpha > 0
            _ew_grad_into(d, "leaky_relu", (float(alpha), 0.0, 0), O_t, O_t, dO_t)
            cached = (dO_t, d)
            O_t._pre_act_grad = cached
        return cached[1]

    # Layers that run on the tensor cores read channel-innermost hi/lo copies of their operands.
    # The copy of the input made for the forward pass is kept for the kernel gradient, and the
    # copy of dY is made once for both gradients (three repacking passes per layer instead of five).
    keep_packed = g.ic > 4
    packed_x = pack_activation(input_t) if keep_packed else None

    # a pooled block whose gradients all read the packed format never needs dZ as an NCHW tensor
    direct_packed = _pooled and keep_packed and passes == 2
    # a pooled first layer (few input channels): the kernel gradient walks the winners of the
    # pooling windows, so dZ is only built if somebody asks for the input gradient
    winners_dw = (_pooled and not keep_packed and g.kh == 3 and g.kw == 3 and stride == 1 and dilation == 1 and
                  g.padl == 1 and g.padt == 1 and g.ow % 64 == 0)

    def winner_grads(O_t, dO_t):
        cached = getattr(O_t, "_winner_grads", None)
        if cached is None or cached[0] is not dO_t:
            t = _out(O_t.shape)
            for i, dev in _each_device():
                _lib_().lnn_pool2x2_winner_grad(dev, t._ptr(i), idx_t._ptr(i), O_t._ptr(i), dO_t._ptr(i), g.n, g.oc,
                                                g.oh // 2, g.ow // 2, float(alpha), act)
            cached = (dO_t, t)
            O_t._winner_grads = cached
        return cached[1]

    def packed_dy(O_t, dO_t):
        if direct_packed:
            cached = getattr(O_t, "_packed_dy", None)
            if cached is None or cached[0] is not dO_t:
                pd = _packed_like(g.n, g.oc, g.oh, g.ow)
                t = _out(O_t.shape)                 # the winners' gradients: what the bias gradient sums
                for i, dev in _each_device():
                    _lib_().lnn_pool2x2_idx_lrelu_bwd_packed(dev, pd.hi._ptr(i), pd.lo._ptr(i), t._ptr(i), idx_t._ptr(i),
                                                             O_t._ptr(i), dO_t._ptr(i), g.n, g.oc, g.oh, g.ow,
                                                             float(alpha), act)
                cached = (dO_t, pd, t)
                O_t._packed_dy = cached
            return cached[1]
        d = pre_act_grad(O_t, dO_t)
        cached = getattr(O_t, "_packed_dy", None)
        if cached is None or cached[0] is not d:
            cached = (d, pack_activation(d))
            O_t._packed_dy = cached
        return cached[1]

    def _lo(p, i):
        return p.lo._ptr(i) if p.lo is not None else 0

    def grad_x(O_t, dO_t):
        gx = input_t.get_grad()
        if keep_packed:
            pd = packed_dy(O_t, dO_t)
            for i, dev in _each_device():
                _lib_().lnn_conv2d_dx_packed(dev, ctypes.byref(g), gx._ptr(i), pd.hi._ptr(i), _lo(pd, i), kernel_t._ptr(i), passes)
            return
        d = pre_act_grad(O_t, dO_t)
        for i, dev in _each_device():
            _lib_().lnn_conv2d_dx(dev, ctypes.byref(g), gx._ptr(i), d._ptr(i), kernel_t._ptr(i), passes)

    def grad_w(O_t, dO_t):
        gw = kernel_t.get_grad()
        if winners_dw:
            t = winner_grads(O_t, dO_t)
            for i, dev in _each_device():
                _lib_().lnn_conv2d_dw_winners(dev, ctypes.byref(g), gw._ptr(i), t._ptr(i), idx_t._ptr(i), input_t._ptr(i))
            return
        if keep_packed:
            pd = packed_dy(O_t, dO_t)
            for i, dev in _each_device():
                _lib_().lnn_conv2d_dw_packed(dev, ctypes.byref(g), gw._ptr(i), pd.hi._ptr(i), _lo(pd, i),
                                             packed_x.hi._ptr(i), _lo(packed_x, i), passes)
            return
        d = pre_act_grad(O_t, dO_t)
        for i, dev in _each_device():
            _lib_().lnn_conv2d_dw(dev, ctypes.byref(g), gw._ptr(i), d._ptr(i), input_t._ptr(i), passes)

    def grad_b(O_t, dO_t):
        if winners_dw:
            d = winner_grads(O_t, dO_t)
        elif direct_packed:
            packed_dy(O_t, dO_t)
            d = O_t._packed_dy[2]
        else:
            d = pre_act_grad(O_t, dO_t)
            if _pooled:
                # every other element of d is zero: sum the winners (pooled size) instead
                d = O_t._pre_act_grad[2]
        reduce_sum_op(d, (0, 2, 3), output_t=bias_t.get_grad(), is_add_to_output=True)

    output_t._assign_gradfn(input_t, grad_x)
    output_t._assign_gradfn(kernel_t, grad_w)
    if bias_t is not None:
        output_t._assign_gradfn(bias_t, grad_b)
    bias_ptr = (lambda i: bias_t._ptr(i)) if bias_t is not None else (lambda i: 0)
    for i, dev in _each_device():
        if _pooled:
            x, x_lo = (packed_x.hi._ptr(i), _lo(packed_x, i)) if keep_packed else (input_t._ptr(i), 0)
            _lib_().lnn_conv2d_fwd_packed(dev, ctypes.byref(g), output_t._ptr(i), idx_t._ptr(i), x, x_lo,
                                          kernel_t._ptr(i), bias_ptr(i), act, float(alpha), 1,
                                          1 if keep_packed else 0, 0, passes)
        elif keep_packed:
            _lib_().lnn_conv2d_fwd_packed(dev, ctypes.byref(g), output_t._ptr(i), 0, packed_x.hi._ptr(i), _lo(packed_x, i),
                                          kernel_t._ptr(i), bias_ptr(i), act, float(alpha), 0, 1, 0, passes)
        else:
            _lib_().lnn_conv2d_fwd(dev, ctypes.byref(g), output_t._ptr(i), input_t._ptr(i), kernel_t._ptr(i),
                                   bias_ptr(i), act, float(alpha), 0, passes)
    return output_t


def conv2D_block(input_t, kernel_t, stride=1, dilation=1, padding="same", bias_t=None, activation=None, alpha=0.1):
    """max_pool2D(activation(conv2D(x, k) + bias), 2, 2, 'same') as ONE trainable op: same values
    and gradients as the chain nn.conv2D -> nn.leaky_relu -> nn.max_pool2D (the bias gradient sums
    the same non-zero terms in another order).  The pool runs in the convolution's epilogue,
    which also records the winning position of every window, so the full-resolution activation is
    never written; the backward pass computes the gradient of the convolution output from the
    pooled gradient and that map in a single kernel
    instead of two zero fills and two read-modify-write passes over full-resolution tensors
    (pool2D.py:147-230, element_wise_op.py:207-221).  Shapes the fused gradient kernel does not
    cover (odd height, width not a multiple of 4) run as the chain."""
    g, _ = _conv_geom(input_t.shape, kernel_t.shape, int(stride), int(dilation), padding)
    if (g.oh % 2) or (g.ow % 4):
        y = conv2D(input_t, kernel_t, stride, dilation, padding, bias_t, activation, alpha)
        return pool2D_op("max", y, 2, 2, "same")
    return conv2D(input_t, kernel_t, stride, dilation, padding, bias_t, activation, alpha, _pooled=True)


def conv2DTranspose(input_t, kernel_t, stride=2, dilation=1, padding="same"):
    """Transposed convolution, input (N,IC,H,W), kernel (OC,IC,KH,KW), padding 'same' | 'valid'
    (conv2DTranspose.py:8-46).  Forward, dI and dK are the three GEMMs of a convolution with the
    roles swapped, issued on the tile engine without materialising an unfolded buffer."""
    if padding not in ("valid", "same"):
        raise ValueError("Wrong padding value, only valid or same supported for conv2DTranspose.")
    if input_t.shape.rank != 4 or kernel_t.shape.rank != 4:
        raise ValueError("conv2DTranspose expects (N,IC,H,W) input and (OC,IC,KH,KW) kernel")
    stride, dilation = int(stride), int(dilation)
    N, IC, IH, IW = input_t.shape
    KO, KI, KH, KW = kernel_t.shape
    if KI != IC:
        raise ValueError(f"Kernel input channels {KI} does not match input channels {IC}.")
    ci = InfoConv2D(IH, IW, KH, KW, stride, dilation, padding)
    OH, OW = ci.OH_T, ci.OW_T
    # geometry of the convolution [N,KO,OH,OW] -> [N,IC,IH,IW] whose input gradient this is
    g = _lib.ConvGeom(N, KO, OH, OW, IC, KH, KW, IH, IW, stride, dilation, ci.PADL, ci.PADT)
    passes = _lib.precision()
    output_t = _out((N, KO, OH, OW))
    output_t._set_op_name("conv2DTranspose")

    def grad_x(O_t, dO_t):
        gx = input_t.get_grad()
        for i, dev in _each_device():
            _lib_().lnn_conv2d_transpose_dx(dev, ctypes.byref(g), gx._ptr(i), dO_t._ptr(i), kernel_t._ptr(i), passes)

    def grad_k(O_t, dO_t):
        gk = kernel_t.get_grad()
        for i, dev in _each_device():
            _lib_().lnn_conv2d_transpose_dk(dev, ctypes.byref(g), gk._ptr(i), dO_t._ptr(i), input_t._ptr(i), passes)

    output_t._assign_gradfn(input_t, grad_x)
    output_t._assign_gradfn(kernel_t, grad_k)
    for i, dev in _each_device():
        _lib_().lnn_conv2d_transpose_fwd(dev, ctypes.byref(g), output_t._ptr(i), input_t._ptr(i), kernel_t._ptr(i), 0, passes)
    return output_t


def depthwise_conv2D(input_t, kernel_t, stride=1, dilation=1, padding="same"):
    """Depthwise convolution, input (N,IC,H,W), kernel (IC,KH,KW) (depthwise_conv2D.py:9-123)."""
    if kernel_t.shape.rank != 3:
        raise ValueError("Kernel shape rank must be == 3")
    if input_t.shape.rank != 4:
        raise ValueError("depthwise_conv2D expects an (N,IC,H,W) input")
    stride, dilation = int(stride), int(dilation)
    N, IC, IH, IW = input_t.shape
    KI, KH, KW = kernel_t.shape
    if KI != IC:
        raise ValueError(f"Kernel input channels {KI} does not match tensor input channels {IC}.")
    ci = InfoConv2D(IH, IW, KH, KW, stride, dilation, padding)
    g = _lib.ConvGeom(N, IC, IH, IW, IC, KH, KW, ci.OH, ci.OW, stride, dilation, ci.PADL, ci.PADT)
    output_t = _out((N, IC, ci.OH, ci.OW))
    output_t._set_op_name("depthwise_conv2D")

    def grad_x(O_t, dO_t):
        gx = input_t.get_grad()
        for i, dev in _each_device():
            _lib_().lnn_depthwise_conv2d_dx(dev, ctypes.byref(g), gx._ptr(i), dO_t._ptr(i), kernel_t._ptr(i))

    def grad_k(O_t, dO_t):
        gk = kernel_t.get_grad()
        for i, dev in _each_device():
            _lib_().lnn_depthwise_conv2d_dk(dev, ctypes.byref(g), gk._ptr(i), dO_t._ptr(i), input_t._ptr(i))

    output_t._assign_gradfn(input_t, grad_x)
    output_t._assign_gradfn(kernel_t, grad_k)
    for i, dev in _each_device():
        _lib_().lnn_depthwise_conv2d_fwd(dev, ctypes.byref(g), output_t._ptr(i), input_t._ptr(i), kernel_t._ptr(i), 0)
    return output_t


class PackedActivation:
    """An activation kept in the tensor-core convolution's operand format between the layers of
    an inference chain: channel-innermost copies hi and lo, each (N, H, W, C rounded up to 8).
    Split FP16 (the default precision): fp16 values of x / s with s a power of two derived from
    the tensor's largest magnitude or an upper bound of it, whose bit pattern sits in a trailer
    behind hi.  Split TF32:
    hi = tf32(x), lo = tf32(x - hi) as fp32.  Only conv2D_infer / conv2D_pool and the gradient
    entries consume it; the reference has no counterpart (its conv2D builds an im2col buffer per
    call, conv2D.py:39-41).  hi / lo are flat fp32-typed tensors used as raw storage."""

    def __init__(self, shape_nchw, hi_t, lo_t, precision):
        self.shape = TensorShape(shape_nchw)
        self.hi, self.lo, self.precision = hi_t, lo_t, precision

    def _elems(self):
        n, c, h, w = self.shape.shape
        return n * h * w * ((c + 7) & ~7)

    def _part(self, t):
        n, c, h, w = self.shape.shape
        elems = self._elems()
        if self.precision == 2:
            v = t.np().view(np.uint8)[:elems * 2].view(np.float16)
        else:
            v = t.np().reshape(-1)[:elems]
        return v.reshape(n, h, w, (c + 7) & ~7)

    def hi_np(self):
        """The stored hi elements, (N, H, W, C padded to 8): float16 (split FP16) or float32."""
        return self._part(self.hi)

    def lo_np(self):
        return self._part(self.lo) if self.lo is not None else None

    def scale_exponent(self):
        """e such that the activation is (hi + lo) * 2**e (0 unless split FP16)."""
        if self.precision != 2:
            return 0
        off = (self._elems() * 2 + 15) & ~15
        return scale_exponent_of(int(self.hi.np().view(np.uint8)[off:off + 4].view(np.uint32)[0]))

    def largest_magnitude(self):
        """The largest |x| of the activation as measured by the kernel that wrote it (split FP16
        only).  A convolution that writes this format takes its scale from an upper bound of its
        result (trailer word 0) and records the measured maximum in trailer word 1; the split
        pre-pass measures first and leaves word 1 zero."""
        off = (self._elems() * 2 + 15) & ~15
        w = self.hi.np().view(np.uint8)[off:off + 8].view(np.uint32)
        return float(w[1:2].view(np.float32)[0] if w[1] else w[0:1].view(np.float32)[0])

    def np(self):
        """(hi + lo) * 2**e as an NCHW array: the fp32 activation up to its last two mantissa bits."""
        c = self.shape.shape[1]
        v = self.hi_np().astype(np.float64)
        if self.lo is not None:
            v = v + self.lo_np()
        v = v * 2.0 ** self.scale_exponent()
        return np.ascontiguousarray(v[..., :c].transpose(0, 3, 1, 2)).astype(np.float32)


def scale_exponent_of(amax_bits):
    """Scale exponent of the split-FP16 format from the fp32 bit pattern of a tensor's largest
    magnitude: that element times 2**-e lies in [2**14, 2**15); 0 for zero / non-finite maxima."""
    e = (amax_bits >> 23) & 0xFF
    if amax_bits == 0 or e == 255:
        return 0
    return (e if e > 0 else 1) - 127 - 14     # (max / min are tensor ops in this module)


def _packed_like(n, c, h, w):
    prec = _lib.precision()
    hb, lb = ctypes.c_uint64(), ctypes.c_uint64()
    _lib_().lnn_packed_bytes(n, c, h, w, prec, ctypes.byref(hb), ctypes.byref(lb))
    hi = _out(((hb.value + 3) // 4,))
    lo = _out(((lb.value + 3) // 4,)) if lb.value else None
    return PackedActivation((n, c, h, w), hi, lo, prec)


def pack_activation(input_t):
    """NCHW tensor -> PackedActivation (the pre-pass nn.conv2D runs on every call)."""
    n, c, h, w = input_t.shape.shape
    out = _packed_like(n, c, h, w)
    for i, dev in _each_device():
        _lib_().lnn_nhwc_split(dev, out.hi._ptr(i), out.lo._ptr(i) if out.lo is not None else 0, input_t._ptr(i),
                               n, c, h, w, out.precision)
    return out


def conv2D_infer(input_t, kernel_t, stride=1, dilation=1, padding="same", bias_t=None, activation=None, alpha=0.1,
                 pool=False, packed_output=False):
    """Inference convolution: [max_pool2D(]activation(conv2D(x, k) + bias)[, 2, 2, 'same')] in one
    call, without grad functions.  input_t is a Tensor or a PackedActivation; with
    packed_output=True the result is a PackedActivation for the next convolution, so the NCHW
    activation between two layers is never written.  Same values as the un-fused chain
    (conv2D.py:9-44, Conv2D.py:58-62, element_wise_op.py:207-221, pool2D.py:47-146)."""
    packed_in = isinstance(input_t, PackedActivation)
    if input_t.shape.rank != 4 or kernel_t.shape.rank != 4:
        raise ValueError("conv2D expects (N,IC,H,W) input and (OC,IC,KH,KW) kernel")
    g, out_shape = _conv_geom(input_t.shape, kernel_t.shape, int(stride), int(dilation), padding)
    if activation not in (None, "leaky_relu"):
        raise ValueError(f"unknown activation {activation}")
    if bias_t is not None and bias_t.shape.size != g.oc:
        raise ValueError(f"bias must have {g.oc} elements")
    oh, ow = ((g.oh + 1) // 2, (g.ow + 1) // 2) if pool else (g.oh, g.ow)
    if packed_output:
        result = _packed_like(g.n, g.oc, oh, ow)
        y, y_lo = result.hi, result.lo
    else:
        result = y = _out((g.n, g.oc, oh, ow))
        y_lo = None
        result._set_op_name("conv2D_infer")
    for i, dev in _each_device():
        x = input_t.hi._ptr(i) if packed_in else input_t._ptr(i)
        x_lo = input_t.lo._ptr(i) if (packed_in and input_t.lo is not None) else 0
        _lib_().lnn_conv2d_fwd_packed(dev, ctypes.byref(g), y._ptr(i), y_lo._ptr(i) if y_lo is not None else 0, x, x_lo,
                                      kernel_t._ptr(i), bias_t._ptr(i) if bias_t is not None else 0,
                                      1 if activation == "leaky_relu" else 0, float(alpha), 1 if pool else 0,
                                      1 if packed_in else 0, 1 if packed_output else 0, _lib.precision())
    return result


def conv2D_pool(input_t, kernel_t, stride=1, dilation=1, padding="same", bias_t=None, activation=None, alpha=0.1,
                packed_output=False):
    """max_pool2D(activation(conv2D(x, k) + bias), 2, 2, 'same') in one call, for inference:
    no grad functions are registered (build the chain from nn.conv2D / nn.leaky_relu /
    nn.max_pool2D to train).  Same values as that chain."""
    return conv2D_infer(input_t, kernel_t, stride, dilation, padding, bias_t, activation, alpha, pool=True,
                        packed_output=packed_output)


def _ew_grad_into(dst_zeroed, name, args, I_t, O_t, dO_t):
    p0, p1, flag = args
    for i, dev in _each_device():
        _lib_().lnn_eltwise_bwd(dev, _lib.EW[name], dst_zeroed._ptr(i), I_t._ptr(i), O_t._ptr(i), dO_t._ptr(i),
                                I_t.shape.size, p0, p1, flag)
