"""Optimizer base, SGD (momentum, nesterov), RMSprop, Adam and `freeze`
(litenn/core/optimizer/Optimizer.py:36-203, SGD.py:28-83, RMSprop.py:26-69, Adam.py:28-84,
optimizer/__init__.py:9-25).  An optimizer is a saveable module: `iteration` and its state
tensors (`_accs`, or `_ms` / `_vs`) appear in checkpoints under the reference's keys.

Each tensor's update is ONE fused kernel (the reference launches two or three), with the same
operations in the same order.  The multi-device step all-reduces the GRADIENTS over NCCL and
folds 1/replicas into the update, so replicas stay identical; for plain SGD started from
identical weights that equals the reference's host-side weight averaging
(Optimizer.py:149-153)."""
import ctypes

import numpy as np

from . import _lib
from . import ops
from . import parallel
from .devices import devices
from .module import ModuleBase
from .tensor import Tensor, Tensor_zeros_like


class freeze:
    """with nn.optimizer.freeze(): tensors produced inside do not pass gradient to
    trainable inputs (backward.py:135-137)."""

    def __enter__(self):
        Tensor._freeze_stack += 1
        return self

    def __exit__(self, *exc):
        Tensor._freeze_stack -= 1
        if Tensor._freeze_stack < 0:
            raise ValueError("Wrong _freeze_stack")


class OptParams(ctypes.Structure):
    """Mirror of struct lnn_opt_params."""
    _fields_ = [("lr", ctypes.c_float), ("lr_decay", ctypes.c_float), ("lr_dropout", ctypes.c_float),
                ("gscale", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("iteration", ctypes.c_uint32), ("seed_a", ctypes.c_uint32), ("seed_b", ctypes.c_uint32),
                ("nesterov", ctypes.c_int)]


SGD_KIND, RMSPROP_KIND, ADAM_KIND = 0, 1, 2


class Optimizer(ModuleBase):
    """Base class: Optimizer(tensors_list, lr, lr_decay, lr_dropout, clipnorm, saveables)."""

    def __init__(self, _tensors_list, lr=0.001, lr_decay=0.0, lr_dropout=0.0, clipnorm=0.0, saveables=None):
        if _tensors_list is None:
            raise ValueError("_tensors_list must be specified.")
        _tensors_list = list(_tensors_list)
        seen, names = set(), {}
        for i, t in enumerate(_tensors_list):
            if id(t) in seen:
                raise ValueError(f"Tensor {t.get_name()} has duplicate in a list.")
            seen.add(id(t))
            name = t.get_name()
            if name in names:
                raise ValueError(f"Different tensors with the same name '{name}' indexes {names[name]} {i}. "
                                 f"If the same module class is used twice, subclass it under two names.")
            names[name] = i
        for t in _tensors_list:
            if t._is_reference():
                raise ValueError(f"Tensor {t.get_name()} is reference, and cannot be trained in optimizer.")
            if t._is_grad():
                raise ValueError(f"Tensor {t.get_name()} is gradient tensor, and cannot be trained in optimizer.")
            if t._is_trainable():
                raise ValueError(f"Tensor {t.get_name()} is already used by another optimizer.")
            if t._get_gradfns() is not None:
                raise Exception(f"Tensor {t.get_name()} is produced by operator and cannot be trained in optimizer.")
            t._set_trainable(True)
        self._tensors_list = _tensors_list
        self.lr = lr
        self.lr_decay = lr_decay
        self.lr_dropout = lr_dropout
        self.clipnorm = clipnorm
        self.iteration = 0
        super().__init__((saveables or []) + ["iteration"])

    def get_trainable_tensors(self):
        return self._tensors_list

    def get_iteration(self):
        return self.iteration

    def set_iteration(self, iteration):
        self.iteration = iteration

    def zero_grad(self):
        for t in self._tensors_list:
            t.zero_grad()

    def print_no_grad(self):
        for t in self.get_trainable_tensors():
            if not t.has_grad():
                print(f"Tensor has no gradient : {t.get_name()}")

    def step(self, multi_gpu_step=False):
        """Apply one update.  multi_gpu_step=True keeps the replicas in step: gradients are summed
        over all devices / ranks with one group of NCCL all-reduces and the update uses their mean.
        With several current devices and no communicator yet, the single-process communicator is
        created here (the reference averages whenever more than one device is current,
        Optimizer.py:149-153)."""
        tensors = [t for t in self._tensors_list if t.has_grad()]
        gscale = 1.0
        if multi_gpu_step and devices._shallow == 0:
            if parallel.world_size() == 1 and len(devices.get_current()) > 1:
                parallel.init_single_process()
            if parallel.world_size() > 1:
                parallel.allreduce_grads(tensors)
                gscale = 1.0 / parallel.world_size()
        if self.clipnorm != 0.0:
            sums = [ops.square(t.get_grad()).sum().np()[0] for t in tensors]
            l2 = float(np.sqrt(np.sum(sums))) * gscale
            if l2 > self.clipnorm:
                gscale *= self.clipnorm / l2
        self._on_step(tensors, gscale)
        self.iteration += 1

    def _state_tensors(self):
        """{tensor name at construction: zero tensor}, the reference's accumulator dicts."""
        return {t.get_name(): Tensor_zeros_like(t) for t in self.get_trainable_tensors()}

    def _seed(self):
        # one draw per kernel that takes the learning rate, as the reference (Optimizer.py:176-180):
        # the host random stream stays in step with a run on the reference
        return int(np.random.randint(2147483648))

    def _launch(self, kind, t, s1, s2, gscale, beta1, beta2, nesterov, seed_a, seed_b):
        if devices._shallow > 0:
            return
        lib = _lib.get_lib()
        p = OptParams(float(self.lr), float(self.lr_decay), float(self.lr_dropout), float(gscale), float(beta1),
                      float(beta2), int(self.iteration) & 0xFFFFFFFF, seed_a, seed_b, int(bool(nesterov)))
        g = t.get_grad()
        for i, d in enumerate(devices.get_current()):
            lib.lnn_optimizer_step(d.index, kind, t._ptr(i), g._ptr(i), s1._ptr(i), s2._ptr(i) if s2 is not None else 0,
                                   t.shape.size, ctypes.byref(p))

    def _on_step(self, tensors, gscale):
        raise NotImplementedError()


class SGD(Optimizer):
    """SGD(tensors_list, momentum=0.0, nesterov=False, lr=0.001, lr_decay=0.0, lr_dropout=0.0,
    clipnorm=0.0): A = momentum*A - lr*G; V += A (nesterov: V += momentum*A - lr*G)."""

    def __init__(self, tensors_list, momentum=0.0, nesterov=False, lr=0.001, lr_decay=0.0, lr_dropout=0.0, clipnorm=0.0):
        super().__init__(tensors_list, lr=lr, lr_decay=lr_decay, lr_dropout=lr_dropout, clipnorm=clipnorm,
                         saveables=["_accs"])
        self.momentum = momentum
        self.nesterov = nesterov
        self._accs = self._state_tensors()
        self._names = {id(t): t.get_name() for t in self.get_trainable_tensors()}

    def _on_step(self, tensors, gscale):
        for t in tensors:
            seed_a, seed_b = self._seed(), self._seed()
            self._launch(SGD_KIND, t, self._accs[self._names[id(t)]], None, gscale, self.momentum, 0.0, self.nesterov,
                         seed_a, seed_b)


class RMSprop(Optimizer):
    """RMSprop(tensors_list, rho=0.9, lr=0.001, ...): A = rho*A + (1-rho)*G*G;
    V += -lr*G / (sqrt(A) + 1e-7)."""

    def __init__(self, tensors_list, rho=0.9, lr=0.001, lr_decay=0.0, lr_dropout=0.0, clipnorm=0.0):
        super().__init__(tensors_list, lr=lr, lr_decay=lr_decay, lr_dropout=lr_dropout, clipnorm=clipnorm,
                         saveables=["_accs"])
        self._accs = self._state_tensors()
        self._names = {id(t): t.get_name() for t in self.get_trainable_tensors()}
        self.rho = rho

    def _on_step(self, tensors, gscale):
        for t in tensors:
            seed = self._seed()
            self._launch(RMSPROP_KIND, t, self._accs[self._names[id(t)]], None, gscale, self.rho, 0.0, False, seed, seed)


class Adam(Optimizer):
    """Adam(tensors_list, beta_1=0.9, beta_2=0.999, lr=0.001, ...) without bias correction, as the
    reference: M = b1*M + (1-b1)*G; U = b2*U + (1-b2)*G*G; V += -lr*M / (sqrt(U) + 1e-7)."""

    def __init__(self, tensors_list, beta_1=0.9, beta_2=0.999, lr=0.001, lr_decay=0.0, lr_dropout=0.0, clipnorm=0.0):
        super().__init__(tensors_list, lr=lr, lr_decay=lr_decay, lr_dropout=lr_dropout, clipnorm=clipnorm,
                         saveables=["_ms", "_vs"])
        self.beta_1 = beta_1
        self.beta_2 = beta_2
        self._ms = self._state_tensors()
        self._vs = self._state_tensors()
        self._names = {id(t): t.get_name() for t in self.get_trainable_tensors()}

    def _on_step(self, tensors, gscale):
        for t in tensors:
            seed = self._seed()
            name = self._names[id(t)]
            self._launch(ADAM_KIND, t, self._ms[name], self._vs[name], gscale, self.beta_1, self.beta_2, False, seed, seed)
