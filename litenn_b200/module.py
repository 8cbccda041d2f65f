"""ModuleBase, Module, Conv2D and Dense: parameter holders over the op layer with the reference's
constructor arguments, `forward`, `trainables()`, training flag, hierarchical tensor names and
the state dict its checkpoints are made of (litenn/core/module/ModuleBase.py:16-199,
Module.py:45-180, Saveable.py:24-42, Conv2D.py, Dense.py).  A file written by the reference's
`save()` loads here and the other way round: same keys, same entry forms."""
import logging
import pickle
import weakref
from pathlib import Path

from . import initializer as _init
from . import ops
from .devices import devices
from .tensor import Tensor

log = logging.getLogger("litenn_b200")


def _is_saved_name(owner, var_name):
    """The rule that decides which attributes a module saves / names: those listed in its
    `_saveables`, or, without a list, the ones not starting with an underscore."""
    names = getattr(owner, "_saveables", None)
    if names is not None:
        return var_name in names
    return var_name[0] != "_"


class ModuleBase:
    """What Module and Optimizer share: children learn their parent and their name when they are
    assigned (also inside lists and dicts), names are built by walking up to the top parent, and
    the state dict is produced / consumed by one walk over the saved attributes."""

    def __init__(self, saveables=None):
        self._saveables = saveables

    # ---- naming ---------------------------------------------------------------------------
    def get_name(self, top_parent=None):
        """Dotted path from the top parent (its class name when top_parent is None) down to this
        module; a module that is top_parent itself has the empty name."""
        parts = []
        module = self
        while module is not None:
            if top_parent is not None and module is top_parent:
                break
            parent = module._get_parent_module()
            parts.append(parent._get_child_name(module) if parent is not None else module.__class__.__name__)
            module = parent
        return ".".join(str(p) for p in reversed(parts))

    def _get_parent_module(self):
        ref = getattr(self, "_parent_module_w", None)
        return ref() if ref is not None else None

    def _get_child_name(self, child):
        return getattr(self, "_child_names", {}).get(id(child))

    def __setattr__(self, var_name, obj):
        object.__setattr__(self, var_name, obj)
        if not _is_saved_name(self, var_name) and var_name[0] == "_":
            return
        ModuleBase._adopt(self, obj, var_name)

    @staticmethod
    def _adopt(parent, obj, name):
        if isinstance(obj, (Tensor, ModuleBase)):
            if isinstance(obj, Tensor):
                if obj._is_reference():
                    raise Exception("You cannot assign Reference Tensor to the Module")
                if obj._is_produced_by_op():
                    raise Exception("You cannot assign Tensor produced by operator to the Module")
                if obj._parent_module_w is not None:
                    raise Exception(f"Tensor {obj.get_name()} is already assigned to the Module.")
            object.__setattr__(obj, "_parent_module_w", weakref.ref(parent))
            names = getattr(parent, "_child_names", None)
            if names is None:
                names = {}
                object.__setattr__(parent, "_child_names", names)
            names[id(obj)] = name
        elif isinstance(obj, list):
            if len(obj) == 0:
                raise Exception(f"Empty list '{name}' set to {parent.__class__.__name__}: lists of a Module must be "
                                f"filled before they are assigned (use an _underscore name for dynamic lists; "
                                f"those are not saved).")
            for i, element in enumerate(obj):
                ModuleBase._adopt(parent, element, f"{name}[{i}]")
        elif isinstance(obj, dict):
            if len(obj) == 0:
                raise Exception(f"Empty dict '{name}' set to {parent.__class__.__name__}: dicts of a Module must be "
                                f"filled before they are assigned (use an _underscore name for dynamic dicts; "
                                f"those are not saved).")
            for key, element in obj.items():
                ModuleBase._adopt(parent, element, f"{name}[{key}]")
        elif isinstance(obj, set):
            raise Exception("You cannot assign sets to the Module")

    # ---- state dict -------------------------------------------------------------------------
    # Entry forms: tensor -> ('np.ndarray', array) under its name relative to the module being
    # dumped; int / float / complex / str -> ('python-var', (class name, value)); a list adds
    # '<name>__len' -> length.  Loading skips, with a warning, whatever is missing or mismatched.
    def dump_state(self):
        state = {}
        ModuleBase._walk(self, None, self, state, None, True, None)
        return state

    def load_state(self, state_dict):
        ModuleBase._walk(self, None, self, state_dict, None, False, None)

    @staticmethod
    def _walk(top, parent, obj, state, var_name, dump, set_func):
        if isinstance(obj, ModuleBase):
            for name in list(vars(obj)):
                if not _is_saved_name(obj, name):
                    continue
                ModuleBase._walk(top, obj, getattr(obj, name), state, name, dump,
                                 lambda val, o=obj, n=name: setattr(o, n, val))
        elif isinstance(obj, Tensor):
            key = obj.get_name(top)
            if dump:
                state[key] = ("np.ndarray", obj.np())
                return
            entry = state.get(key)
            if entry is None:
                log.warning(f"Tensor {key} is not loaded, because saved data is not found.")
            elif entry[0] != "np.ndarray":
                log.warning(f"Tensor {key} is not loaded, because saved type is {entry[0]}, but must be np.ndarray")
            elif tuple(obj.shape) != tuple(entry[1].shape):
                log.warning(f"Tensor {key} is not loaded, because saved Tensor shape is {entry[1].shape}, "
                            f"but must be {tuple(obj.shape)}")
            else:
                obj.set(entry[1])
        elif isinstance(obj, list):
            key = f"{parent.get_name(top)}.{var_name}".lstrip(".")
            if dump:
                state[f"{key}__len"] = len(obj)
            else:
                saved_len = state.get(f"{key}__len")
                if saved_len is None or saved_len != len(obj):
                    log.warning(f"List {key} is not loaded, because length of list {len(obj)} != saved list len {saved_len}")
                    return
            for i, element in enumerate(obj):
                ModuleBase._walk(top, parent, element, state, f"{var_name}[{i}]", dump,
                                 lambda val, o=obj, k=i: o.__setitem__(k, val))
        elif isinstance(obj, dict):
            for k in obj:
                ModuleBase._walk(top, parent, obj[k], state, f"{var_name}[{k}]", dump,
                                 lambda val, o=obj, kk=k: o.__setitem__(kk, val))
        elif isinstance(obj, (int, float, complex, str)):
            key = f"{parent.get_name(top)}.{var_name}".lstrip(".")
            if dump:
                state[key] = ("python-var", (obj.__class__.__name__, obj))
                return
            entry = state.get(key)
            if entry is None:
                log.warning(f"Variable {key} is not loaded, because saved data is not found.")
            elif entry[0] != "python-var":
                log.warning(f"Variable {key} is not loaded, because saved type is {entry[0]}, but must be python-var")
            elif entry[1][0] != obj.__class__.__name__:
                log.warning(f"Variable {key} is not loaded, because saved class_name is {entry[1][0]}, "
                            f"but must be {obj.__class__.__name__}")
            else:
                set_func(entry[1][1])

    def save(self, filepath):
        """Pickle (protocol 4) of dump_state(), the reference's checkpoint format."""
        Path(filepath).write_bytes(pickle.dumps(self.dump_state(), 4))

    def load(self, filepath):
        """load_state() from a file written by save(); returns False when it does not exist."""
        filepath = Path(filepath)
        if not filepath.exists():
            return False
        self.load_state(pickle.loads(filepath.read_bytes()))
        return True


class Module(ModuleBase):
    """Base class of layers and models.  Calling the constructor may be omitted, as in the
    reference: without `_saveables` / `_trainables` every public attribute counts."""

    def __init__(self, saveables=None, trainables=None):
        super().__init__(saveables=saveables)
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
        """Tensors of this module and its sub-modules, in attribute order (Module.py:96-128):
        those named in `_trainables`, else in `_saveables`, else every public attribute."""
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
            object.__setattr__(obj, "_tr", is_training)
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


def _prepare_fans(initializer, fan_in, fan_out):
    """Give an initializer the fans of the layer unless the caller fixed them."""
    if initializer is None:
        initializer = _init.GlorotUniform()
    if getattr(initializer, "fan_in", 0) is None:
        initializer.fan_in = fan_in
    if getattr(initializer, "fan_out", 0) is None:
        initializer.fan_out = fan_out
    return initializer


class _BiasedConvModule(Module):
    """Shared part of the convolution modules below: a kernel, an optional per-channel bias added
    as a (1, C, 1, 1) broadcast, saveables 'kernel' and 'bias'."""

    def _make_bias(self, channels, use_bias, bias_initializer):
        self.use_bias = use_bias
        self.bias = Tensor((channels,), init=bias_initializer or _init.Scalar(0.0)) if use_bias else None

    def _add_bias(self, x):
        return x + self.bias.reshape((1, -1, 1, 1)) if self.use_bias else x


class Conv2DTranspose(_BiasedConvModule):
    """Conv2DTranspose(in_ch, out_ch, kernel_size, stride=2, dilation=1, padding='same',
    use_bias=True, kernel_initializer=None, bias_initializer=None); forward =
    nn.conv2DTranspose + bias; kernel (out_ch, in_ch, k, k) (module/Conv2DTranspose.py:22-58)."""

    def __init__(self, in_ch, out_ch, kernel_size, stride=2, dilation=1, padding="same", use_bias=True,
                 kernel_initializer=None, bias_initializer=None):
        self.in_ch, self.out_ch, self.kernel_size = in_ch, out_ch, kernel_size
        self.stride, self.padding, self.dilation = stride, padding, dilation
        taps = kernel_size * kernel_size
        self.kernel = Tensor((out_ch, in_ch, kernel_size, kernel_size),
                             init=_prepare_fans(kernel_initializer, in_ch * taps, out_ch * taps))
        self._make_bias(out_ch, use_bias, bias_initializer)
        super().__init__(saveables=["kernel", "bias"])

    def forward(self, x, **kwargs):
        return self._add_bias(ops.conv2DTranspose(x, self.kernel, self.stride, self.dilation, padding=self.padding))

    def __str__(self):
        return f"{self.__class__.__name__} : in_ch:{self.in_ch} out_ch:{self.out_ch} "

    __repr__ = __str__


class DepthwiseConv2D(_BiasedConvModule):
    """DepthwiseConv2D(in_ch, kernel_size, stride=1, dilation=1, padding='same', use_bias=True,
    depthwise_initializer=None, pointwise_initializer=None, bias_initializer=None); forward =
    nn.depthwise_conv2D + bias; kernel (in_ch, k, k) (module/DepthwiseConv2D.py:24-56; the
    reference accepts and ignores pointwise_initializer as well)."""

    def __init__(self, in_ch, kernel_size, stride=1, dilation=1, padding="same", use_bias=True,
                 depthwise_initializer=None, pointwise_initializer=None, bias_initializer=None):
        self.in_ch, self.kernel_size = in_ch, kernel_size
        self.stride, self.padding, self.dilation = stride, padding, dilation
        self.kernel = Tensor((in_ch, kernel_size, kernel_size),
                             init=_prepare_fans(depthwise_initializer, in_ch * kernel_size * kernel_size, 0))
        self._make_bias(in_ch, use_bias, bias_initializer)
        super().__init__(saveables=["kernel", "bias"])

    def forward(self, x, **kwargs):
        return self._add_bias(ops.depthwise_conv2D(x, self.kernel, self.stride, self.dilation, padding=self.padding))

    def __str__(self):
        return f"{self.__class__.__name__} : in_ch:{self.in_ch} "

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
