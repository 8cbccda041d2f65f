"""Deferred convolutions: how the stock operator chain reaches the fused kernels.

A model written the way LiteNN's user guide writes it -- `nn.Conv2D` (conv2D, then `+ bias`),
`nn.leaky_relu`, `nn.max_pool2D`, the next `nn.Conv2D` -- asks for four kernels and three
intermediate tensors per block (litenn/core/module/Conv2D.py:58-62, op/element_wise_op.py:207-221,
op/pool2D.py:47-146).  The library has one kernel for the whole block and an operand format that lets
the next convolution start from it without an NCHW tensor in between, but it can only use them if it
knows what follows a convolution.  So `conv2D` does not launch: it returns a tensor that carries a
record of the work (a `Pending`).  `add` with a per-channel bias, `leaky_relu` and
`max_pool2D(2, 2, 'same')` on such a tensor return a new tensor with the extended record; a
convolution whose input is such a tensor chains to it.  The launch happens when somebody needs the
values: any other operator, `np()`, `set()` (through `Tensor._get_buffers`).  A convolution that
consumes a deferred tensor asks for it in the packed operand format, so the activation between two
convolutions is never written as NCHW.  Values are those of the separate kernels, bit for bit (the
fused epilogues apply the same roundings in the same order).

Intermediate tensors stay valid: each carries its own record and launches its own (shorter) chain if
its values are ever asked for.

Only graphs that need no gradient are deferred (no trainable tensor upstream, or inside
`optimizer.freeze()`): a training step takes the eager path with its grad functions.  If a gradient
is asked for anyway (`backward(..., grad_for_non_trainables=True)`), the tape edges of a deferred
tensor are built at that moment by running the trainable form of the same block once.
"""
import ctypes

from . import _lib
from .devices import devices
from .info import InfoConv2D
from .shape import TensorShape

import contextlib
import os

_enabled = [os.environ.get("LNN_EAGER", "0") != "1"]      # LNN_EAGER=1: every operator launches at once


composed_softmax = [False]      # True: softmax / categorical_crossentropy run as the reference's compositions


@contextlib.contextmanager
def disabled():
    """Inside this context every operator is the reference's own composition, one kernel per
    operator: conv2D launches eagerly, softmax and categorical_crossentropy are built from exp,
    reduce_sum, div, clip, log, mul."""
    old = _enabled[0], composed_softmax[0]
    _enabled[0], composed_softmax[0] = False, True
    try:
        yield
    finally:
        _enabled[0], composed_softmax[0] = old


class Pending:
    """conv2D(x, kernel) [+ bias] [leaky_relu] [max_pool2D(2, 2, 'same')] not yet launched."""
    __slots__ = ("x", "kernel", "stride", "dilation", "padding", "geom", "conv_shape", "bias", "act", "alpha",
                 "pool", "done")

    def __init__(self, x, kernel, stride, dilation, padding, geom, conv_shape):
        self.x, self.kernel = x, kernel
        self.stride, self.dilation, self.padding = stride, dilation, padding
        self.geom, self.conv_shape = geom, conv_shape
        self.bias, self.act, self.alpha, self.pool = None, 0, 0.0, False
        self.done = False

    def extended(self, **changes):
        p = Pending(self.x, self.kernel, self.stride, self.dilation, self.padding, self.geom, self.conv_shape)
        p.bias, p.act, p.alpha, p.pool = self.bias, self.act, self.alpha, self.pool
        for k, v in changes.items():
            setattr(p, k, v)
        return p

    def out_shape(self):
        n, oc, oh, ow = self.conv_shape
        return (n, oc, (oh + 1) // 2, (ow + 1) // 2) if self.pool else (n, oc, oh, ow)


def _source(t):
    return t._get_top_reference_source() if t._is_reference() else t


def reaches_trainable(t, _memo=None):
    """True when a gradient could have to flow through t to a trainable tensor."""
    t = _source(t)
    if t._is_trainable():
        return True
    memo = {} if _memo is None else _memo
    key = id(t)
    if key in memo:
        return memo[key]
    memo[key] = False
    r = False
    for inp in t._tape_inputs():
        if reaches_trainable(inp, memo):
            r = True
            break
    memo[key] = r
    return r


def is_deferred(t):
    """t is a tensor whose convolution has not been launched."""
    t = _source(t)
    p = getattr(t, "_pending", None)
    return p is not None and not p.done


def _no_tape_needed(*tensors):
    from .tensor import Tensor
    if Tensor._freeze_stack != 0:
        return True
    return not any(t is not None and reaches_trainable(t) for t in tensors)


def _new(p, op_name):
    from . import ops
    t = ops._out(p.out_shape())
    t._set_op_name(op_name)
    t._pending = p
    return t


def start(input_t, kernel_t, stride, dilation, padding, geom, conv_shape, bias_t=None, act=0, alpha=0.0):
    """The deferred result of conv2D, or None when the call has to run eagerly."""
    if not _enabled[0] or devices._shallow > 0 or not _no_tape_needed(input_t, kernel_t, bias_t):
        return None
    p = Pending(input_t, kernel_t, stride, dilation, padding, geom, tuple(conv_shape))
    p.bias, p.act, p.alpha = bias_t, act, float(alpha)
    if is_deferred(input_t) and not input_t._is_reference():
        input_t._packed_users = getattr(input_t, "_packed_users", 0) + 1     # its packed copy is wanted once more
    return _new(p, "conv2D")


def try_bias(a_t, b_t):
    """a + b where a is a deferred convolution without epilogue and b a per-channel bias."""
    if not is_deferred(a_t) or a_t._is_reference():
        return None
    p = a_t._pending
    oc = p.conv_shape[1]
    if p.bias is not None or p.act or p.pool or is_deferred(b_t):
        return None
    if tuple(b_t.shape.shape) != (1, oc, 1, 1) or not _no_tape_needed(b_t):
        return None
    return _new(p.extended(bias=b_t), "add")


def try_act(t, alpha):
    if not is_deferred(t) or t._is_reference():
        return None
    p = t._pending
    if p.act or p.pool or not _no_tape_needed():
        return None
    return _new(p.extended(act=1, alpha=float(alpha)), "leaky_relu")


def try_pool(op_type, t, pool_size, stride, padding):
    if op_type != "max" or pool_size != 2 or stride != 2 or padding != "same":
        return None
    if not is_deferred(t) or t._is_reference():
        return None
    p = t._pending
    if p.pool or not _no_tape_needed():
        return None
    return _new(p.extended(pool=True), "max_pool2D")


def _launch(p, y_ptrs, y_lo_ptrs, out_packed, precision):
    """One lnn_conv2d_fwd_packed per device.  A deferred input is taken in the packed format."""
    from . import ops
    x = p.x
    packed_in = None
    if isinstance(x, ops.PackedActivation):
        packed_in = x
    elif is_deferred(x) and not x._is_reference():
        packed_in = materialize_packed(x)
    lib = _lib.get_lib()
    for i, d in enumerate(devices.get_current()):
        if packed_in is not None:
            xp = packed_in.hi._ptr(i)
            xl = packed_in.lo._ptr(i) if packed_in.lo is not None else 0
        else:
            xp, xl = x._ptr(i), 0
        lib.lnn_conv2d_fwd_packed(d.index, ctypes.byref(p.geom), y_ptrs[i], y_lo_ptrs[i] if y_lo_ptrs else 0, xp, xl,
                                  p.kernel._ptr(i), p.bias._ptr(i) if p.bias is not None else 0, int(p.act),
                                  float(p.alpha), 1 if p.pool else 0, 1 if packed_in is not None else 0,
                                  1 if out_packed else 0, precision)
    if packed_in is not None and packed_in is not x:
        x._packed_users = getattr(x, "_packed_users", 1) - 1
        if x._packed_users <= 0:
            x._packed = None      # the packed copy of the intermediate has served its last consumer


def materialize(t):
    """Launch the work of a deferred tensor into its own (NCHW) buffers."""
    p = t._pending
    if p is None or p.done:
        return
    p.done = True                 # before the launch: the buffers are about to be requested
    bufs = t._buffers
    _launch(p, [b.ptr() for b in bufs], None, False, _lib.precision())


def materialize_packed(t):
    """The values of a deferred tensor in the packed operand format (no NCHW tensor is written)."""
    from . import ops
    cached = getattr(t, "_packed", None)
    if cached is not None:
        return cached
    p = t._pending
    n, oc, oh, ow = p.out_shape()
    out = ops._packed_like(n, oc, oh, ow)
    ndev = len(devices.get_current())
    _launch(p, [out.hi._ptr(i) for i in range(ndev)],
            [out.lo._ptr(i) if out.lo is not None else 0 for i in range(ndev)], True, out.precision)
    t._packed = out
    return out


def tape_inputs(t):
    """The tensors a deferred tensor was computed from (what reachability walks need)."""
    p = t._pending
    from . import ops
    ins = [p.kernel]
    if not isinstance(p.x, ops.PackedActivation):
        ins.insert(0, p.x)
    if p.bias is not None:
        ins.append(p.bias)
    return ins


def build_gradfns(t):
    """Tape edges of a deferred tensor, built on demand: the trainable form of the same block runs
    once (its values equal the deferred ones) and its grad functions become t's."""
    from . import ops
    p = t._pending
    if isinstance(p.x, ops.PackedActivation):
        return None
    _enabled[0] = False
    try:
        bias_1d = None
        if p.bias is not None:
            bias_1d = p.bias if p.bias.shape.rank == 1 else p.bias.reshape((p.conv_shape[1],))
        act = "leaky_relu" if p.act else None
        if p.pool:
            r = ops.conv2D_block(p.x, p.kernel, p.stride, p.dilation, p.padding, bias_t=bias_1d, activation=act,
                                 alpha=p.alpha if p.act else 0.1)
        else:
            r = ops.conv2D(p.x, p.kernel, p.stride, p.dilation, p.padding, bias_t=bias_1d, activation=act,
                           alpha=p.alpha if p.act else 0.1)
    finally:
        _enabled[0] = True
    return r._get_gradfns()
