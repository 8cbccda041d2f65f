"""ctypes binding of liblitenn_b200.so (declared in include/litenn_b200.h).

Plays the part litenn/core/minicl/api/OpenCL/OpenCL.py plays in the reference: every
entry point gets argtypes, and a non-zero return code raises LnnError carrying
lnn_last_error() (the reference raises CLException from its errcheck hook,
OpenCL.py:175-198).  There is no fallback: if the shared library is missing the first
device call fails loudly.
"""
import ctypes
import os
from ctypes import (POINTER, c_char_p, c_float, c_int, c_int64, c_uint64, c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LNN_LIB") or os.path.join(_HERE, "liblitenn_b200.so")

OK, E_INVALID, E_CUDA, E_NOMEM, E_NOTINIT, E_UNSUPPORTED, E_NCCL, E_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7
MAX_DIMS = 6

EW = {name: i for i, name in enumerate(
    ["abs", "add_const", "clip", "cos", "exp", "leaky_relu", "log", "mul_const", "rdiv_const",
     "rsub_const", "relu", "sigmoid", "sin", "sqrt", "square", "tanh"])}
BIN = {name: i for i, name in enumerate(["add", "sub", "mul", "div", "max", "min", "binary_crossentropy"])}
POOL = {"avg": 0, "max": 1, "min": 2}
RED = {"sum": 0, "mean": 1, "max": 2, "min": 3}


class LnnError(Exception):
    """A C-ABI call returned a negative status."""

    def __init__(self, code, message, func=None):
        self.code = code
        self.func = func
        super().__init__(f"{func or 'lnn'}: [{code}] {message}")


class ConvGeom(ctypes.Structure):
    """Mirror of struct lnn_conv_geom."""
    _fields_ = [(n, c_int) for n in
                ("n", "ic", "ih", "iw", "oc", "kh", "kw", "oh", "ow", "stride", "dilation", "padl", "padt")]


_I64P = POINTER(c_int64)
_SIGNATURES = {
    "lnn_version": (c_int, []),
    "lnn_last_error": (c_char_p, []),
    "lnn_device_count": (c_int, [POINTER(c_int)]),
    "lnn_device_info": (c_int, [c_int, c_char_p, c_int, POINTER(c_uint64), POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "lnn_init": (c_int, [c_int]),
    "lnn_shutdown": (c_int, [c_int]),
    "lnn_alloc": (c_int, [c_int, c_uint64, POINTER(c_uint64)]),
    "lnn_free": (c_int, [c_int, c_uint64, c_uint64]),
    "lnn_mem_stats": (c_int, [c_int, POINTER(c_uint64), POINTER(c_uint64)]),
    "lnn_pool_trim": (c_int, [c_int]),
    "lnn_h2d": (c_int, [c_int, c_uint64, c_void_p, c_uint64]),
    "lnn_d2h": (c_int, [c_int, c_void_p, c_uint64, c_uint64]),
    "lnn_d2d": (c_int, [c_int, c_uint64, c_uint64, c_uint64]),
    "lnn_fill_f32": (c_int, [c_int, c_uint64, c_int64, c_float]),
    "lnn_init_uniform": (c_int, [c_int, c_uint64, c_int64, ctypes.c_uint32, c_float, c_float]),
    "lnn_init_normal": (c_int, [c_int, c_uint64, c_int64, ctypes.c_uint32, c_float, c_float]),
    "lnn_sync": (c_int, [c_int]),
    "lnn_h2d_async": (c_int, [c_int, c_uint64, c_void_p, c_uint64]),
    "lnn_d2h_async": (c_int, [c_int, c_void_p, c_uint64, c_uint64]),
    "lnn_h2d_prefetch": (c_int, [c_int, c_uint64, c_void_p, c_uint64, c_uint64]),
    "lnn_wait_prefetch": (c_int, [c_int]),
    "lnn_d2h_readback": (c_int, [c_int, c_void_p, c_uint64, c_uint64]),
    "lnn_wait_readback": (c_int, [c_int]),
    "lnn_host_alloc": (c_int, [c_uint64, POINTER(c_void_p)]),
    "lnn_host_free": (c_int, [c_void_p]),
    "lnn_launch_count": (c_int, [c_int, POINTER(c_uint64)]),
    "lnn_device_status": (c_int, [c_int, POINTER(c_int)]),
    "lnn_debug_set_status": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "lnn_event_create": (c_int, [c_int, POINTER(c_uint64)]),
    "lnn_event_record": (c_int, [c_int, c_uint64]),
    "lnn_event_elapsed_ms": (c_int, [c_int, c_uint64, c_uint64, POINTER(c_float)]),
    "lnn_event_destroy": (c_int, [c_int, c_uint64]),
    "lnn_profile_enable": (c_int, [c_int, c_int]),
    "lnn_profile_read": (c_int, [c_int, c_int, POINTER(c_uint64), POINTER(c_float)]),
    "lnn_eltwise_fwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_int64, c_float, c_float, c_int, c_int]),
    "lnn_eltwise_bwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_float, c_float, c_int]),
    "lnn_binary_fwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_uint64, c_int, _I64P, _I64P, _I64P, c_int]),
    "lnn_binary_bwd": (c_int, [c_int, c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_int, _I64P, _I64P, _I64P]),
    "lnn_softmax_fwd": (c_int, [c_int, c_uint64, c_uint64, c_int64, c_int64]),
    "lnn_softmax_bwd": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_int64, c_int64]),
    "lnn_cce_fwd": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int64]),
    "lnn_cce_bwd": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int64]),
    "lnn_scale_bias_lrelu": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int64, c_float, c_int]),
    "lnn_pool2d_fwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_int64, c_int64] + [c_int] * 8),
    "lnn_pool2d_bwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64] + [c_int] * 8),
    "lnn_pool2x2_lrelu_bwd": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int, c_int, c_float, c_int]),
    "lnn_pool2x2_idx_lrelu_bwd": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int, c_int, c_float, c_int]),
    "lnn_pool2x2_winner_grad": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int, c_int, c_float, c_int]),
    "lnn_conv2d_dw_winners": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64]),
    "lnn_pool2x2_idx_lrelu_bwd_packed": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int, c_int, c_float, c_int]),
    "lnn_reduce": (c_int, [c_int, c_int, c_uint64, c_uint64] + [c_int64] * 5 + [c_int]),
    "lnn_reduce_noalloc": (c_int, [c_int, c_int, c_uint64, c_uint64] + [c_int64] * 5 + [c_int]),
    "lnn_reduce_bwd": (c_int, [c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64] + [c_int64] * 5),
    "lnn_transpose": (c_int, [c_int, c_uint64, c_uint64, c_int, _I64P, POINTER(c_int), c_int]),
    "lnn_slice_fwd": (c_int, [c_int, c_uint64, c_uint64, c_int, _I64P, _I64P, _I64P, _I64P, c_int]),
    "lnn_slice_bwd": (c_int, [c_int, c_uint64, c_uint64, c_int, _I64P, _I64P, _I64P, _I64P]),
    "lnn_gemm_f32": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int]),
    "lnn_conv2d_fwd": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_float, c_int, c_int]),
    "lnn_conv2d_pool_fwd": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_float, c_int]),
    "lnn_packed_bytes": (c_int, [c_int64, c_int64, c_int64, c_int64, c_int, POINTER(c_uint64), POINTER(c_uint64)]),
    "lnn_nhwc_split": (c_int, [c_int, c_uint64, c_uint64, c_uint64, c_int, c_int, c_int, c_int, c_int]),
    "lnn_conv2d_fwd_packed": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_uint64,
                                      c_int, c_float, c_int, c_int, c_int, c_int]),
    "lnn_conv2d_dx": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_conv2d_dw": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_conv2d_dx_packed": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_conv2d_dw_packed": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_conv2d_transpose_fwd": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int, c_int]),
    "lnn_conv2d_transpose_dx": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_conv2d_transpose_dk": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_depthwise_conv2d_fwd": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64, c_int]),
    "lnn_depthwise_conv2d_dx": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64]),
    "lnn_depthwise_conv2d_dk": (c_int, [c_int, POINTER(ConvGeom), c_uint64, c_uint64, c_uint64]),
    "lnn_sgd_step": (c_int, [c_int, c_uint64, c_uint64, c_int64, c_float, c_float]),
    "lnn_optimizer_step": (c_int, [c_int, c_int, c_uint64, c_uint64, c_uint64, c_uint64, c_int64, c_void_p]),
    "lnn_nccl_unique_id": (c_int, [c_void_p]),
    "lnn_nccl_init_rank": (c_int, [c_int, c_int, c_int, c_void_p]),
    "lnn_nccl_init_all": (c_int, [POINTER(c_int), c_int]),
    "lnn_nccl_allreduce_sum": (c_int, [c_int, c_uint64, c_int64]),
    "lnn_nccl_group_start": (c_int, []),
    "lnn_nccl_group_end": (c_int, []),
    "lnn_nccl_destroy": (c_int, [c_int]),
}
# entry points that report status through their return value
_NO_ERRCHECK = {"lnn_version", "lnn_last_error"}

EXPORTS = tuple(_SIGNATURES)

_lib = None


def _make_errcheck(name):
    def errcheck(result, func, args):
        if result != 0:
            msg = _lib.lnn_last_error()
            raise LnnError(result, msg.decode("utf-8", "replace") if msg else "", name)
        return result
    return errcheck


def get_lib():
    """Load the shared library once and type every export.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LnnError(E_NOTINIT,
                       f"{LIB_PATH} not found: build it with `python -m litenn_b200.csrc.build` "
                       f"(there is no CPU fallback)", "get_lib")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(lib, name)     # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    for name in _SIGNATURES:
        if name not in _NO_ERRCHECK:
            getattr(lib, name).errcheck = _make_errcheck(name)
    return lib


def i64_array(values, pad_to=None, pad_value=1):
    vals = [int(v) for v in values]
    if pad_to is not None:
        vals = vals + [pad_value] * (pad_to - len(vals))
    return (c_int64 * len(vals))(*vals)


def precision():
    """Operand split of the tensor-core contractions (the `precision` argument of the C entries):
    2 = split FP16 (default), 3 = split TF32, 1 = plain TF32.  LNN_PRECISION overrides it."""
    v = int(os.environ.get("LNN_PRECISION", "2"))
    if v not in (1, 2, 3):
        raise ValueError("LNN_PRECISION must be 1, 2 or 3")
    return v


# older name of the same setting
tf32_passes = precision
