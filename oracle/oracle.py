"""numpy front end of the CPU oracle (oracle/lnn_oracle.c).  TEST INFRASTRUCTURE ONLY:
imported by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs; the product
package never imports it.  Every function takes and returns float32 ndarrays and mirrors one
C-ABI entry point of include/litenn_b200.h."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liblnn_oracle.so")
_lib = None

EW = {n: i for i, n in enumerate(
    ["abs", "add_const", "clip", "cos", "exp", "leaky_relu", "log", "mul_const", "rdiv_const",
     "rsub_const", "relu", "sigmoid", "sin", "sqrt", "square", "tanh"])}
BIN = {n: i for i, n in enumerate(["add", "sub", "mul", "div", "max", "min", "binary_crossentropy"])}
POOL = {"avg": 0, "max": 1, "min": 2}
RED = {"sum": 0, "mean": 1, "max": 2, "min": 3}


class ConvGeom(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in
                ("n", "ic", "ih", "iw", "oc", "kh", "kw", "oh", "ow", "stride", "dilation", "padl", "padt")]


def build(force=False):
    src = os.path.join(_HERE, "lnn_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
    return _lib


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _i64(vals):
    return (ctypes.c_int64 * len(vals))(*[int(v) for v in vals])


I64, F32, INT = ctypes.c_int64, ctypes.c_float, ctypes.c_int


def eltwise_fwd(name, I, p0=0.0, p1=0.0, flag=0, out=None):
    I = _f(I)
    acc = out is not None
    O = _f(out).copy() if acc else np.empty_like(I)
    lib().lnn_o_eltwise_fwd(INT(EW[name]), _p(O), _p(I), I64(I.size), F32(p0), F32(p1), INT(flag), INT(acc))
    return O


def eltwise_bwd(name, dI, I, O, dO, p0=0.0, p1=0.0, flag=0):
    dI, I, O, dO = _f(dI).copy(), _f(I), _f(O), _f(dO)
    lib().lnn_o_eltwise_bwd(INT(EW[name]), _p(dI), _p(I), _p(O), _p(dO), I64(I.size), F32(p0), F32(p1), INT(flag))
    return dI


def _bshapes(A, B):
    rank = max(A.ndim, B.ndim)
    a = (1,) * (rank - A.ndim) + A.shape
    b = (1,) * (rank - B.ndim) + B.shape
    o = tuple(max(x, y) for x, y in zip(a, b))
    return rank, o, a, b


def binary_fwd(name, A, B, out=None):
    A, B = _f(A), _f(B)
    rank, o, a, b = _bshapes(A, B)
    acc = out is not None
    O = _f(out).copy() if acc else np.empty(o, np.float32)
    lib().lnn_o_binary_fwd(INT(BIN[name]), _p(O), _p(A), _p(B), INT(rank), _i64(o), _i64(a), _i64(b), INT(acc))
    return O


def binary_bwd(name, which, dX, A, B, O, dO):
    A, B, O, dO, dX = _f(A), _f(B), _f(O), _f(dO), _f(dX).copy()
    rank, o, a, b = _bshapes(A, B)
    lib().lnn_o_binary_bwd(INT(BIN[name]), INT(which), _p(dX), _p(A), _p(B), _p(O), _p(dO), INT(rank), _i64(o), _i64(a), _i64(b))
    return dX


def scale_bias_lrelu(X, G, Bv, alpha=0.1, out=None):
    X, G, Bv = _f(X), _f(G).reshape(-1), _f(Bv).reshape(-1)
    N, C, H, W = X.shape
    acc = out is not None
    Y = _f(out).copy() if acc else np.empty_like(X)
    lib().lnn_o_scale_bias_lrelu(_p(Y), _p(X), _p(G), _p(Bv), I64(N), I64(C), I64(H * W), F32(alpha), INT(acc))
    return Y


def pool_out(ih, iw, pool, stride, padding="same"):
    """(OH, OW, PADL, PADT) as info/InfoConv2D.py:41-77 with dilation 1."""
    if padding == "same":
        padl = padt = (pool - 1) // 2
        padr = padb = pool - 1 - padl
    elif padding == "valid":
        padl = padt = padr = padb = 0
    elif isinstance(padding, int):
        padl = padt = padr = padb = padding
    else:
        padl, padt, padr, padb = padding
    oh = max(1, int((ih + padt + padb - pool) / stride + 1))
    ow = max(1, int((iw + padl + padr - pool) / stride + 1))
    return oh, ow, padl, padt


def pool2d_fwd(mode, I, pool=2, stride=2, padding="same"):
    I = _f(I)
    N, C, IH, IW = I.shape
    OH, OW, PL, PT = pool_out(IH, IW, pool, stride, padding)
    O = np.empty((N, C, OH, OW), np.float32)
    lib().lnn_o_pool2d_fwd(INT(POOL[mode]), _p(O), _p(I), I64(N), I64(C), INT(IH), INT(IW), INT(OH), INT(OW),
                           INT(pool), INT(stride), INT(PL), INT(PT))
    return O


def pool2d_bwd(mode, dI, I, dO, O, pool=2, stride=2, padding="same"):
    dI, I, dO, O = _f(dI).copy(), _f(I), _f(dO), _f(O)
    N, C, IH, IW = I.shape
    OH, OW, PL, PT = pool_out(IH, IW, pool, stride, padding)
    lib().lnn_o_pool2d_bwd(INT(POOL[mode]), _p(dI), _p(I), _p(dO), _p(O), I64(N), I64(C), INT(IH), INT(IW),
                           INT(OH), INT(OW), INT(pool), INT(stride), INT(PL), INT(PT))
    return dI


def reduce5(op, I, outer, r0, mid, r1, inner, out=None):
    I = _f(I)
    acc = out is not None
    O = _f(out).copy().reshape(-1) if acc else np.empty(outer * mid * inner, np.float32)
    lib().lnn_o_reduce(INT(RED[op]), _p(O), _p(I), I64(outer), I64(r0), I64(mid), I64(r1), I64(inner), INT(acc))
    return O


def reduce(op, I, axes=None, keepdims=False):
    """General axes: move the reduced axes last (the reference's own first step), then rows x cols."""
    I = _f(I)
    axes = tuple(range(I.ndim)) if axes is None else tuple(sorted(a % I.ndim for a in (axes if hasattr(axes, "__iter__") else (axes,))))
    keep = tuple(a for a in range(I.ndim) if a not in axes)
    T = np.ascontiguousarray(I.transpose(keep + axes))
    cols = int(np.prod([I.shape[a] for a in axes])) if axes else 1
    rows = T.size // cols
    O = reduce5(op, T, rows, 1, 1, cols, 1)
    shape = tuple(I.shape[a] for a in keep) or (1,)
    if keepdims:
        shape = tuple(1 if a in axes else I.shape[a] for a in range(I.ndim))
    return O.reshape(shape)


def reduce_bwd5(op, dI, I, dO, O, outer, r0, mid, r1, inner):
    dI, I, dO, O = _f(dI).copy(), _f(I), _f(dO), _f(O)
    lib().lnn_o_reduce_bwd(INT(RED[op]), _p(dI), _p(I), _p(dO), _p(O), I64(outer), I64(r0), I64(mid), I64(r1), I64(inner))
    return dI


def transpose(I, axes, out=None):
    I = _f(I)
    acc = out is not None
    oshape = tuple(I.shape[a] for a in axes)
    O = _f(out).copy() if acc else np.empty(oshape, np.float32)
    ax = (ctypes.c_int * len(axes))(*axes)
    lib().lnn_o_transpose(_p(O), _p(I), INT(I.ndim), _i64(I.shape), ax, INT(acc))
    return O.reshape(oshape)


def slice_fwd(I, out_shape_krn, begin, step, out=None):
    I = _f(I)
    acc = out is not None
    O = _f(out).copy() if acc else np.empty(out_shape_krn, np.float32)
    lib().lnn_o_slice(_p(O), _p(I), INT(I.ndim), _i64(I.shape), _i64(out_shape_krn), _i64(begin), _i64(step), INT(acc), INT(0))
    return O


def slice_bwd(dI, dO, out_shape_krn, begin, step):
    dI, dO = _f(dI).copy(), _f(dO)
    lib().lnn_o_slice(_p(dO), _p(dI), INT(dI.ndim), _i64(dI.shape), _i64(out_shape_krn), _i64(begin), _i64(step), INT(0), INT(1))
    return dI


def gemm(A, B, bias=None, trans_a=False, trans_b=False, out=None, accum64=False):
    A, B = _f(A), _f(B)
    batch = int(np.prod(A.shape[:-2])) if A.ndim > 2 else 1
    m = A.shape[-1] if trans_a else A.shape[-2]
    k = A.shape[-2] if trans_a else A.shape[-1]
    n = B.shape[-2] if trans_b else B.shape[-1]
    acc = out is not None
    C = _f(out).copy() if acc else np.empty(A.shape[:-2] + (m, n), np.float32)
    bias = _f(bias) if bias is not None else None
    lib().lnn_o_gemm(_p(C), _p(A), _p(B), _p(bias), I64(batch), I64(m), I64(n), I64(k), INT(trans_a), INT(trans_b),
                     INT(acc), INT(accum64))
    return C


def conv_geom(x_shape, w_shape, stride=1, dilation=1, padding="same"):
    N, IC, IH, IW = x_shape
    OC, _, KH, KW = w_shape
    ekh, ekw = (KH - 1) * dilation + 1, (KW - 1) * dilation + 1
    if padding == "same":
        pl, pt = (ekw - 1) // 2, (ekh - 1) // 2
        pr, pb = ekw - 1 - pl, ekh - 1 - pt
    elif padding == "valid":
        pl = pt = pr = pb = 0
    elif isinstance(padding, int):
        pl = pt = pr = pb = padding
    else:
        pl, pt, pr, pb = padding
    oh = max(1, int((IH + pt + pb - ekh) / stride + 1))
    ow = max(1, int((IW + pl + pr - ekw) / stride + 1))
    return ConvGeom(N, IC, IH, IW, OC, KH, KW, oh, ow, stride, dilation, pl, pt)


def conv2d_fwd(X, W, stride=1, dilation=1, padding="same", bias=None, act=0, alpha=0.1, accum64=False):
    X, W = _f(X), _f(W)
    g = conv_geom(X.shape, W.shape, stride, dilation, padding)
    Y = np.empty((g.n, g.oc, g.oh, g.ow), np.float32)
    bias = _f(bias) if bias is not None else None
    lib().lnn_o_conv2d_fwd(ctypes.byref(g), _p(Y), _p(X), _p(W), _p(bias), INT(act), F32(alpha), INT(0), INT(accum64))
    return Y


def conv2d_dx(dX, dY, W, x_shape, stride=1, dilation=1, padding="same", accum64=False):
    dX, dY, W = _f(dX).copy(), _f(dY), _f(W)
    g = conv_geom(x_shape, W.shape, stride, dilation, padding)
    lib().lnn_o_conv2d_dx(ctypes.byref(g), _p(dX), _p(dY), _p(W), INT(accum64))
    return dX


def conv2d_dw(dW, dY, X, stride=1, dilation=1, padding="same", accum64=False):
    dW, dY, X = _f(dW).copy(), _f(dY), _f(X)
    g = conv_geom(X.shape, dW.shape, stride, dilation, padding)
    lib().lnn_o_conv2d_dw(ctypes.byref(g), _p(dW), _p(dY), _p(X), INT(accum64))
    return dW


def convt_geom(x_shape, k_shape, stride=2, dilation=1, padding="same"):
    """Geometry of conv2DTranspose: output size as info/InfoConv2D.py:41-77 (OH_T, OW_T)."""
    N, IC, IH, IW = x_shape
    OC, _, KH, KW = k_shape
    ekh, ekw = (KH - 1) * dilation + 1, (KW - 1) * dilation + 1
    if padding == "same":
        pl, pt = (ekw - 1) // 2, (ekh - 1) // 2
        oh, ow = IH * stride, IW * stride
    elif padding == "valid":
        pl = pt = 0
        oh, ow = IH * stride + max(ekh - stride, 0), IW * stride + max(ekw - stride, 0)
    else:
        raise ValueError("only valid or same")
    return ConvGeom(N, IC, IH, IW, OC, KH, KW, oh, ow, stride, dilation, pl, pt)


def conv2d_transpose_fwd(X, K, stride=2, dilation=1, padding="same", accum64=False):
    X, K = _f(X), _f(K)
    g = convt_geom(X.shape, K.shape, stride, dilation, padding)
    Y = np.empty((g.n, g.oc, g.oh, g.ow), np.float32)
    lib().lnn_o_convt_fwd(ctypes.byref(g), _p(Y), _p(X), _p(K), INT(accum64))
    return Y


def conv2d_transpose_dx(dX, dY, K, stride=2, dilation=1, padding="same", accum64=False):
    dX, dY, K = _f(dX).copy(), _f(dY), _f(K)
    g = convt_geom(dX.shape, K.shape, stride, dilation, padding)
    lib().lnn_o_convt_dx(ctypes.byref(g), _p(dX), _p(dY), _p(K), INT(accum64))
    return dX


def conv2d_transpose_dk(dK, dY, X, stride=2, dilation=1, padding="same", accum64=False):
    dK, dY, X = _f(dK).copy(), _f(dY), _f(X)
    g = convt_geom(X.shape, dK.shape, stride, dilation, padding)
    lib().lnn_o_convt_dk(ctypes.byref(g), _p(dK), _p(dY), _p(X), INT(accum64))
    return dK


def _dw_geom(x_shape, k_shape, stride, dilation, padding):
    C, KH, KW = k_shape
    return conv_geom(x_shape, (C, C, KH, KW), stride, dilation, padding)


def depthwise_fwd(X, K, stride=1, dilation=1, padding="same"):
    X, K = _f(X), _f(K)
    g = _dw_geom(X.shape, K.shape, stride, dilation, padding)
    Y = np.empty((g.n, g.ic, g.oh, g.ow), np.float32)
    lib().lnn_o_depthwise_fwd(ctypes.byref(g), _p(Y), _p(X), _p(K))
    return Y


def depthwise_dx(dX, dY, K, stride=1, dilation=1, padding="same"):
    dX, dY, K = _f(dX).copy(), _f(dY), _f(K)
    g = _dw_geom(dX.shape, K.shape, stride, dilation, padding)
    lib().lnn_o_depthwise_dx(ctypes.byref(g), _p(dX), _p(K), _p(dY))
    return dX


def depthwise_dk(dK, dY, X, stride=1, dilation=1, padding="same"):
    """Products, then the tree-ordered row sums added to dK (depthwise_conv2D.py:45-50)."""
    dK, dY, X = _f(dK).copy(), _f(dY), _f(X)
    g = _dw_geom(X.shape, dK.shape, stride, dilation, padding)
    rows, cols = dK.size, g.n * g.oh * g.ow
    P = np.empty((rows, cols), np.float32)
    lib().lnn_o_depthwise_dk_products(ctypes.byref(g), _p(P), _p(X), _p(dY))
    return reduce5("sum", P, rows, 1, 1, cols, 1, out=dK.reshape(-1)).reshape(dK.shape)


def sgd(V, G, lr, gscale=1.0):
    V, G = _f(V).copy(), _f(G)
    lib().lnn_o_sgd(_p(V), _p(G), I64(V.size), F32(lr), F32(gscale))
    return V


def init_uniform(shape, seed, low=0.0, high=1.0):
    """RandomUniform as the reference's device kernel fills it (RandomUniform.py:12-28)."""
    out = np.empty(shape, np.float32)
    lib().lnn_o_init_uniform(_p(out), I64(out.size), ctypes.c_uint32(seed), F32(low), F32(high))
    return out


def init_normal(shape, seed, mean=0.0, stddev=1.0):
    """RandomNormal (Box-Muller on the 2-D PCG hash, RandomNormal.py:10-30)."""
    out = np.empty(shape, np.float32)
    lib().lnn_o_init_normal(_p(out), I64(out.size), ctypes.c_uint32(seed), F32(mean), F32(stddev))
    return out


def he_uniform_limits(gain, fan_in):
    """(low, high) of HeUniform: a = sqrt(3) * gain * sqrt(2 / fan_in)  (He.py:23-27)."""
    a = np.sqrt(3.0) * (gain * np.sqrt(2.0 / fan_in))
    return -a, a


def glorot_std(gain, fan_in, fan_out):
    """stddev of GlorotNormal: gain * sqrt(2 / (fan_in + fan_out))  (Glorot.py:25)."""
    return gain * np.sqrt(2.0 / (fan_in + fan_out))


def set_threads(n):
    """OpenMP threads used by the oracle's loops (the environment may have pinned it to 1)."""
    lib().lnn_o_set_threads(INT(n))
    return int(lib().lnn_o_get_max_threads())
