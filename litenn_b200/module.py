"""Module, Conv2D and Dense: thin parameter holders over the op layer, with the reference's
constructor arguments, `forward`, `trainables()`, training flag and a numpy state dict
(litenn/core/module/Module.py, ModuleBase.py:131-199, Conv2D.py, Dense.py)."""
import pickle
import weakref

import numpy as np

from . import initializer as _init
from . import ops
from .devices import devices
from .tensor import Tensor


class Module:
    def __init__(self, saveables=None, trainables=None):
        self._saveables = saveables
        self._trainables = trainables

    def forward(self, *args, **kwargs):
        raise NotImplementedError()

    def shallow_forward(self, *args, **kwargs):
        """forward() without kernel launches or allocations: output-shape inference."""
        with devices._shallow_mode():
            return self.forward(*args, **kwargs)

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def is_training(self):
        return getattr(self, "_tr", False)

    def set_training(self, is_training):
        Module._nested_set_training(self, is_training)

    def trainables(self):
        out = []
        names = getattr(self, "_trainables", None)
        if names is None:
            names = getattr(self, "_saveables", None)
        for var_name in vars(self):
            if names is not None:
                if var_name not in names:
                    continue
            elif var_name[0] == "_":
                continue
            Module._collect(getattr(self, var_name), out)
        return out

    # ---- state dict: {hierarchical name: ndarray} ------------------------------------------
    def _named_tensors(self, prefix=""):
        names = getattr(self, "_saveables", None)
        for var_name, obj in vars(self).items():
            if names is not None:
                if var_name not in names:
                    continue
            elif var_name[0] == "_":
                continue
            yield from Module._named(obj, f"{prefix}{var_name}")

    @staticmethod
    def _named(obj, name):
        if isinstance(obj, Module):
            yield from obj._named_tensors(name + ".")
        elif isinstance(obj, Tensor):
            yield name, obj
        elif isinstance(obj, list):
            for i, o in enumerate(obj):
                yield from Module._named(o, f"{name}[{i}]")
        elif isinstance(obj, dict):
            for k, o in obj.items():
                yield from Module._named(o, f"{name}[{k}]")

    def dump_state(self):
        return {name: ("np.ndarray", t.np()) for name, t in self._named_tensors()}

    def load_state(self, state):
        for name, t in self._named_tensors():
            entry = state.get(name)
            if entry is None:
                continue
            value = entry[1] if isinstance(entry, tuple) else entry
            if tuple(value.shape) != t.shape.shape:
                raise ValueError(f"{name}: stored shape {value.shape} != {t.shape}")
            t.set(value)

    def save(self, filepath):
        with open(filepath, "wb") as f:
            pickle.dump(self.dump_state(), f, protocol=4)

    def load(self, filepath):
        with open(filepath, "rb") as f:
            self.load_state(pickle.load(f))

    @staticmethod
    def _collect(obj, out):
        if isinstance(obj, Module):
            out.extend(obj.trainables())
        elif isinstance(obj, Tensor):
            out.append(obj)
        elif isinstance(obj, list):
            for o in obj:
                Module._collect(o, out)
        elif isinstance(obj, dict):
            for o in obj.values():
                Module._collect(o, out)

    @staticmethod
    def _nested_set_training(obj, is_training):
        if isinstance(obj, Module):
            obj._tr = is_training
            for o in list(vars(obj).values()):
                Module._nested_set_training(o, is_training)
        elif isinstance(obj, list):
            for o in obj:
                Module._nested_set_training(o, is_training)
        elif isinstance(obj, dict):
            for o in obj.values():
                Module._nested_set_training(o, is_training)


class Conv2D(Module):
    """Conv2D(in_ch, out_ch, kernel_size, stride=1, dilation=1, padding='same', use_bias=True,
    kernel_initializer=None, bias_initializer=None); forward = nn.conv2D + bias
    (module/Conv2D.py:28-62).  `fused=True` folds the bias into the convolution epilogue
    (same values, one pass less)."""

    def __init__(self, in_ch, out_ch, kernel_size, stride=1, dilation=1, padding="same", use_bias=True,
                 kernel_initializer=None, bias_initializer=None, fused=True):
        self.in_ch, self.out_ch, self.kernel_size = in_ch, out_ch, kernel_size
        self.stride, self.padding, self.dilation, self.use_bias = stride, padding, dilation, use_bias
        self._fused = fused
        if kernel_initializer is None:
            kernel_initializer = _init.GlorotUniform()
        if getattr(kernel_initializer, "fan_in", 0) is None:
            kernel_initializer.fan_in = in_ch * kernel_size * kernel_size
        if getattr(kernel_initializer, "fan_out", 0) is None:
            kernel_initializer.fan_out = out_ch * kernel_size * kernel_size
        self.kernel = Tensor((out_ch, in_ch, kernel_size, kernel_size), init=kernel_initializer)
        self.bias = None
        if use_bias:
            self.bias = Tensor((out_ch,), init=bias_initializer or _init.Scalar(0.0))
        super().__init__(saveables=["kernel", "bias"])

    def forward(self, x, **kwargs):
        if self.use_bias and self._fused:
            return ops.conv2D(x, self.kernel, self.stride, self.dilation, padding=self.padding, bias_t=self.bias)
        x = ops.conv2D(x, self.kernel, self.stride, self.dilation, padding=self.padding)
        if self.use_bias:
            x = x + self.bias.reshape((1, -1, 1, 1))
        return x

    def __str__(self):
        return f"{self.__class__.__name__} : in_ch:{self.in_ch} out_ch:{self.out_ch} "

    __repr__ = __str__


class Dense(Module):
    """Dense(in_ch, out_ch, use_bias=True, weight_initializer=None, bias_initializer=None);
    forward = nn.matmul(x, weight) + bias (module/Dense.py:20-48)."""

    def __init__(self, in_ch, out_ch, use_bias=True, weight_initializer=None, bias_initializer=None, fused=True):
        self.in_ch, self.out_ch, self.use_bias = in_ch, out_ch, use_bias
        self._fused = fused
        if weight_initializer is None:
            weight_initializer = _init.GlorotUniform()
        if getattr(weight_initializer, "fan_in", 0) is None:
            weight_initializer.fan_in = in_ch
        if getattr(weight_initializer, "fan_out", 0) is None:
            weight_initializer.fan_out = out_ch
        self.weight = Tensor((in_ch, out_ch), init=weight_initializer)
        self.bias = None
        if use_bias:
            self.bias = Tensor((out_ch,), init=bias_initializer or _init.Scalar(0.0))
        super().__init__(saveables=["weight", "bias"])

    def forward(self, x, **kwargs):
        if self.use_bias and self._fused:
            return ops.dense(x, self.weight, self.bias)
        x = ops.matmul(x, self.weight)
        if self.use_bias:
            x = x + self.bias
        return x

    def __str__(self):
        return f"{self.__class__.__name__} : in_ch:{self.in_ch} out_ch:{self.out_ch} "

    __repr__ = __str__
