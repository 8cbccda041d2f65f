"""Tensor, TensorRef, TensorGrad and the constructors of the `nn` namespace.

A Tensor is a shape plus one lazily allocated fp32 device buffer per current device, an
optional lazily created zero gradient, and the tape edges (grad functions per input) that
`backward` walks -- the contract of litenn/core/Tensor.py:6-553.
"""
import numpy as np

from . import initializer as _init
from .devices import DevicesBuffers, devices
from .shape import TensorShape


class Tensor(DevicesBuffers):
    """Tensor(shape, init=None): fp32 tensor; scalar shape () is stored as (1,)."""

    _object_count = 0
    _seq_id = 0
    _freeze_stack = 0

    def __init__(self, shape, init=None):
        self.shape = shape = TensorShape(shape)
        if init is None:
            init = _init.Scalar(0.0)
        Tensor._object_count += 1
        self._seq_id = Tensor._seq_id = Tensor._seq_id + 1
        self._freezed = Tensor._freeze_stack != 0
        self._trainable = False
        self._grad_t = None
        self._gradfns = None
        self._op_name = None
        self._op = None
        self._parent_module_w = None
        self._pending = None        # work not launched yet (deferred.py); None for ordinary tensors
        super().__init__(shape.size * 4, init_func=lambda buf: init.initialize_buffer(buf, shape))

    def __del__(self):
        Tensor._object_count -= 1
        if Tensor._object_count == 0:
            Tensor._seq_id = 0

    # ---- autograd -------------------------------------------------------------------
    def backward(self, stop_grad=None, grad_for_non_trainables=False):
        from .autograd import backward
        backward(self, stop_grad=stop_grad, grad_for_non_trainables=grad_for_non_trainables)

    def has_grad(self):
        return self._grad_t is not None

    def get_grad(self):
        """Gradient tensor, created zero-filled on first access (Tensor.py:37-46)."""
        if self._is_grad():
            raise Exception("Gradient of gradient is unsupported.")
        if self._grad_t is None:
            self._grad_t = TensorGrad(self.shape, init=_init.Scalar(0.0))
        return self._grad_t

    def free_grad(self):
        self._grad_t = None

    def zero_grad(self):
        self.free_grad()

    # ---- host access ----------------------------------------------------------------
    def np(self, device_id=0):
        return self._get_buffers()[device_id].np(self.shape, dtype=np.float32)

    def np_combined(self):
        return np.concatenate([self.np(i) for i in range(self.np_count())], 0)

    def np_count(self):
        return len(self._get_buffers())

    def fill(self, value, device_id=None):
        value = np.float32(value)
        bufs = self._get_buffers()
        for b in (bufs if device_id is None else [bufs[device_id]]):
            b.fill(value)

    def set(self, value, device_id=None):
        if isinstance(value, Tensor):
            if self.shape.size != value.shape.size:
                raise ValueError("Unable to set data from other tensor: shape.size is not the same.")
            for mine, other in zip(self._get_buffers(), value._get_buffers()):
                mine.set(other)
            return
        if isinstance(value, np.ndarray):
            value = value.astype(np.float32)
        elif isinstance(value, (int, float)):
            value = np.array([value], dtype=np.float32)
        elif isinstance(value, (list, tuple)):
            value = np.array(value, dtype=np.float32)
        else:
            raise ValueError(f"Unknown type {value.__class__}")
        bufs = self._get_buffers()
        for b in (bufs if device_id is None else [bufs[device_id]]):
            b.set(value)

    def copy(self, shape=None):
        shape = self.shape if shape is None else TensorShape(shape)
        if shape.size != self.shape.size:
            raise ValueError("shapes size mismatch")
        t = Tensor(shape)
        t.set(self)
        return t

    # ---- operator sugar -------------------------------------------------------------
    def max(self, axes=None, keepdims=False):
        from . import ops
        return ops.reduce_max(self, axes, keepdims=keepdims)

    def mean(self, axes=None, keepdims=False):
        from . import ops
        return ops.reduce_mean(self, axes, keepdims=keepdims)

    def min(self, axes=None, keepdims=False):
        from . import ops
        return ops.reduce_min(self, axes, keepdims=keepdims)

    def sum(self, axes=None, keepdims=False):
        from . import ops
        return ops.reduce_sum(self, axes, keepdims=keepdims)

    def reshape(self, target_shape):
        from . import ops
        return ops.reshape(self, target_shape)

    def transpose(self, axes_order):
        from . import ops
        return ops.transpose(self, axes_order)

    def T(self):
        return self.transpose(tuple(range(self.shape.rank - 1, -1, -1)))

    def __getitem__(self, slices):
        from . import ops
        return ops.slice(self, slices)

    # x+x, x-x, x*x shortcuts as Tensor.py:301-379
    def _coerce(self, t):
        return t if isinstance(t, Tensor) else Tensor_from_value(t)

    def __add__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.add_const(self, t)
        t = self._coerce(t)
        return ops.mul_const(self, 2.0) if t is self else ops.add(self, t)

    def __radd__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.add_const(self, t)
        t = self._coerce(t)
        return ops.mul_const(self, 2.0) if t is self else ops.add(t, self)

    def __sub__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.sub_const(self, t)
        t = self._coerce(t)
        return ops.mul_const(self, 0.0) if t is self else ops.sub(self, t)

    def __rsub__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.rsub_const(self, t)
        t = self._coerce(t)
        return ops.mul_const(self, 0.0) if t is self else ops.sub(t, self)

    def __mul__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.mul_const(self, t)
        t = self._coerce(t)
        return ops.square(self) if t is self else ops.mul(self, t)

    def __rmul__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.mul_const(self, t)
        t = self._coerce(t)
        return ops.square(self) if t is self else ops.mul(t, self)

    def __truediv__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.div_const(self, t)
        return ops.div(self, self._coerce(t))

    def __rtruediv__(self, t):
        from . import ops
        if isinstance(t, (int, float)):
            return ops.rdiv_const(self, t)
        return ops.div(self._coerce(t), self)

    def __neg__(self):
        return self * -1

    # Tensors are dict keys on the tape: identity hash / equality
    __hash__ = object.__hash__

    def __eq__(self, other):
        return self is other

    # ---- internals --------------------------------------------------------------------
    def get_name(self, top_parent=None):
        if self._parent_module_w is None:
            name = f"#{self._get_seq_id()}"
            if self._op_name is not None:
                name += f"({self._op_name})"
            if self._is_reference():
                name += "(ref)"
            return name
        parent = self._parent_module_w()
        return f"{parent.get_name(top_parent)}.{parent._get_child_name(self)}"

    def __str__(self):
        return f"T {self.get_name()} {self.shape}"

    def __repr__(self):
        s = str(self) + "\n"
        for i, buf in enumerate(self._get_buffers()):
            s += f"{buf.device}\n{self.np(i)}\n"
        return s + str(self)

    def _set_op_name(self, op_name):
        self._op_name = op_name

    def _assign_gradfn(self, input_t, func):
        """Register func(O_t, dO_t), which must ADD the gradient into input_t.get_grad()
        (Tensor.py:387-412)."""
        if self._gradfns is None:
            self._gradfns = {}
        self._gradfns.setdefault(input_t, []).append(func)

    def _as_ref(self, shape):
        return TensorRef(self, shape)

    def _get_buffers(self):
        """The device buffers; a deferred convolution is launched first (deferred.py)."""
        if self._pending is not None and not self._pending.done:
            from . import deferred
            deferred.materialize(self)
        return self._buffers

    def _is_freezed(self): return self._freezed
    def _is_reference(self): return False
    def _is_grad(self): return False
    def _is_trainable(self): return self._trainable
    def _is_produced_by_op(self): return self._gradfns is not None or self._pending is not None

    def _get_gradfns(self):
        if self._gradfns is None and self._pending is not None:
            from . import deferred
            self._gradfns = deferred.build_gradfns(self)
        return self._gradfns

    def _tape_inputs(self):
        """Input tensors of the op that produced this one (empty for leaves)."""
        if self._gradfns is None and self._pending is not None:
            from . import deferred
            return deferred.tape_inputs(self)
        return list(self._gradfns.keys()) if self._gradfns is not None else []
    def _get_reference_source(self): return self
    def _get_seq_id(self): return self._seq_id

    def _get_top_reference_source(self):
        t = self
        while t._is_reference():
            t = t._get_reference_source()
        return t

    def _set_trainable(self, trainable): self._trainable = trainable

    def _ptr(self, device_id):
        """Device pointer of this tensor's buffer on current device number device_id."""
        return self._get_buffers()[device_id].ptr()


class TensorRef(Tensor):
    """Zero-copy view of another Tensor under a different shape of equal size; shares the
    buffers, the gradient, the tape edges and the sequence id (Tensor.py:444-471)."""

    def __init__(self, t, shape):
        shape = TensorShape(shape)
        if t.shape.size != shape.size:
            raise ValueError(f"Cannot interpet shape {t.shape} as ref shape {shape}")
        # no buffers of its own
        self.shape = shape
        Tensor._object_count += 1
        self._seq_id = None
        self._freezed = False
        self._trainable = False
        self._grad_t = None
        self._gradfns = None
        self._op_name = None
        self._op = None
        self._parent_module_w = None
        self._buffers = None
        self._t = t

    def has_grad(self): return self._t.has_grad()
    def get_grad(self): return self._t.get_grad()._as_ref(self.shape)
    def free_grad(self): self._t.free_grad()
    def zero_grad(self): self._t.zero_grad()
    def _assign_gradfn(self, *a, **k): self._t._assign_gradfn(*a, **k)
    def _is_freezed(self): return self._t._is_freezed()
    def _is_reference(self): return True
    def _is_grad(self): return self._t._is_grad()
    def _is_trainable(self): return self._t._is_trainable()
    def _get_buffers(self): return self._t._get_buffers()
    def _get_gradfns(self): return self._t._get_gradfns()
    def _tape_inputs(self): return self._t._tape_inputs()
    def _is_produced_by_op(self): return self._t._is_produced_by_op()
    def _get_reference_source(self): return self._t
    def _get_seq_id(self): return self._t._get_seq_id()
    def _set_trainable(self, *a, **k): self._t._set_trainable(*a, **k)


class TensorGrad(Tensor):
    def _is_grad(self): return True


def Tensor_like(t, init=None):
    return Tensor(t.shape, init=init)


def Tensor_zeros_like(t):
    return Tensor(t.shape, init=_init.Scalar(0.0))


def Tensor_ones_like(t):
    return Tensor(t.shape, init=_init.Scalar(1.0))


def Tensor_from_value(value):
    """New tensor holding `value` (Tensor, number, list or ndarray) (Tensor.py:495-514)."""
    if isinstance(value, list):
        value = np.array(value, np.float32)
    elif isinstance(value, (int, float, np.int32, np.float32, np.float64)):
        value = np.array([value], np.float32)
    elif not isinstance(value, (Tensor, np.ndarray)):
        raise ValueError(f"Unsupported value {value} ({value.__class__})")
    t = Tensor(value.shape)
    t.set(value)
    return t


def Tensor_sliced_from_value(value):
    """Shard an ndarray along axis 0 over the current devices (Tensor.py:516-552)."""
    if not isinstance(value, (Tensor, np.ndarray)):
        raise ValueError("Value must be np.ndarray type")
    if len(value.shape) < 1:
        raise ValueError("Shape rank must be >= 1")
    n_dev = len(devices.get_current())
    if value.shape[0] % n_dev != 0:
        raise ValueError(f"Unable to evenly slice shape {value.shape} to {n_dev} devices.")
    per = value.shape[0] // n_dev
    t = Tensor((per,) + tuple(value.shape[1:]))
    for i in range(n_dev):
        t.set(value[i * per:(i + 1) * per, ...], i)
    return t
