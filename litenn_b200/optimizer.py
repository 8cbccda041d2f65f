"""Optimizer base, SGD (momentum 0) and `freeze` (litenn/core/optimizer/Optimizer.py,
SGD.py:42-83, optimizer/__init__.py).  The multi-device step all-reduces the GRADIENTS over
NCCL and folds 1/replicas into the update; for plain SGD started from identical weights
that equals the reference's host-side weight averaging (Optimizer.py:149-153)."""
import numpy as np

from . import _lib
from . import ops
from . import parallel
from .devices import devices
from .tensor import Tensor


class freeze:
    """with nn.optimizer.freeze(): tensors produced inside do not pass gradient to
    trainable inputs (backward.py:135-137)."""

    def __enter__(self):
        Tensor._freeze_stack += 1
        return self

    def __exit__(self, *exc):
        Tensor._freeze_stack -= 1


class Optimizer:
    def __init__(self, tensors_list, lr=0.001, clipnorm=0.0):
        tensors_list = list(tensors_list)
        for t in tensors_list:
            if t._is_trainable():
                raise ValueError(f"Tensor {t.get_name()} is already used in another optimizer")
            t._set_trainable(True)
        self._tensors_list = tensors_list
        self.lr = lr
        self.clipnorm = clipnorm
        self.iteration = 0

    def get_trainable_tensors(self):
        return self._tensors_list

    def zero_grad(self):
        for t in self._tensors_list:
            t.zero_grad()

    def step(self, multi_gpu_step=False):
        """Apply one update.  multi_gpu_step=True synchronises replicas: gradients are summed
        across all ranks/devices with one NCCL all-reduce per tensor group first."""
        tensors = [t for t in self._tensors_list if t.has_grad()]
        gscale = 1.0
        if multi_gpu_step and parallel.world_size() > 1:
            parallel.allreduce_grads(tensors)
            gscale = 1.0 / parallel.world_size()
        if self.clipnorm != 0.0:
            sums = [ops.square(t.get_grad()).sum().np()[0] for t in tensors]
            l2 = float(np.sqrt(np.sum(sums))) * gscale
            if l2 > self.clipnorm:
                gscale *= self.clipnorm / l2
        self._on_step(tensors, gscale)
        self.iteration += 1

    def _on_step(self, tensors, gscale):
        raise NotImplementedError()


class SGD(Optimizer):
    """SGD(tensors_list, lr=0.001): V += -lr * G (SGD.py with momentum 0)."""

    def __init__(self, tensors_list, momentum=0.0, nesterov=False, lr=0.001, lr_decay=0.0, lr_dropout=0.0, clipnorm=0.0):
        if momentum != 0.0 or nesterov or lr_decay != 0.0 or lr_dropout != 0.0:
            raise NotImplementedError("only plain SGD (momentum=0, no decay/dropout) is implemented")
        super().__init__(tensors_list, lr=lr, clipnorm=clipnorm)

    def _on_step(self, tensors, gscale):
        if devices._shallow > 0:
            return
        lib = _lib.get_lib()
        for t in tensors:
            g = t.get_grad()
            for i, d in enumerate(devices.get_current()):
                lib.lnn_sgd_step(d.index, t._ptr(i), g._ptr(i), t.shape.size, float(self.lr), float(gscale))
