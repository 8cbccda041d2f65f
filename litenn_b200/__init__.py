"""litenn_b200 -- the `litenn` user namespace over a B200-native device backend.

    import litenn_b200 as nn

Classes and Modules are upper case, operators lower case, initializers under
`nn.initializer`, optimizers under `nn.optimizer` -- the layout of litenn/__init__.py.
Every operator runs hand-written sm_100a kernels through a C-ABI shared library
(include/litenn_b200.h); there is no CPU or PyTorch fallback.
"""
from . import deferred, info, initializer, optimizer, ops, parallel
from ._lib import LnnError
from .autograd import backward
from .devices import devices
from .module import Conv2D, Conv2DTranspose, Dense, DepthwiseConv2D, Module, ModuleBase
from .ops import (abs, add, add_const, avg_pool2D, binary_crossentropy, categorical_crossentropy, clip,
                  conv2D, conv2DTranspose, conv2D_block, conv2D_infer, conv2D_pool, depthwise_conv2D, pack_activation, PackedActivation, cos, dense, div, div_const, exp, flatten, leaky_relu, log, matmul, max, max_pool2D,
                  min, min_pool2D, moments, mul, mul_const, rdiv_const, reduce_max, reduce_mean, reduce_min,
                  reduce_std, reduce_sum, reduce_variance, relu, reshape, rsub_const, scale_bias_leaky_relu,
                  sigmoid, sin, slice, softmax, sqrt, square, sub, sub_const, tanh, transpose)
from .shape import TensorAxes, TensorShape
from .tensor import (Tensor, Tensor_from_value, Tensor_like, Tensor_ones_like, Tensor_sliced_from_value,
                     Tensor_zeros_like)

op = ops   # the reference exposes `_op` variants as nn.core.op.<name>_op


def cleanup():
    """Free device memory of all current devices; no Tensor may be alive (litenn/__init__.py:117-125)."""
    ops._bcast_info.cache_clear()
    ops._reduce_plan.cache_clear()
    if Tensor._object_count != 0:
        raise Exception(f"Unable to cleanup while {Tensor._object_count} Tensor objects exist.")
    parallel.shutdown()
    devices.cleanup()
