"""CPU: the oracle (oracle/lnn_oracle.c) against the golden vectors produced by the reference
itself (tests/golden/make_golden.py).  This is what pins the oracle."""
import numpy as np
import pytest

import cases
import oracle as o
from conftest import assert_bit_exact, assert_contraction_close, load_golden, ulp_diff

EW_PARAMS = {"add_const": (1.25, 0), "clip": (-0.5, 0.75), "div_const": (1.0 / 3.0, 0), "leaky_relu": (0.1, 0),
             "mul_const": (-1.7, 0), "rdiv_const": (2.5, 0), "rsub_const": (0.3, 0), "sub_const": (-0.6, 0)}
EW_ALIAS = {"div_const": "mul_const", "sub_const": "add_const"}


def _cases(family):
    return [(n, p) for n, f, p in cases.all_cases() if f == family]


@pytest.mark.parametrize("name,p", _cases("eltwise"))
def test_eltwise(name, p):
    ins, outs = load_golden("eltwise")[name]
    op = EW_ALIAS.get(p["op"], p["op"])
    p0, p1 = EW_PARAMS.get(p["op"], (0.0, 0.0))
    y = o.eltwise_fwd(op, ins["x"], p0, p1)
    dx = o.eltwise_bwd(op, np.ones_like(ins["x"]), ins["x"], y, ins["dy"], p0, p1)
    assert_bit_exact(y, outs["y"], name + " y")
    assert_bit_exact(dx, outs["dx"], name + " dx")


def _reduce_to(full, shape):
    """reduce_sum over the broadcast axes, the way dual_wise_op.py:110-130 does it."""
    rank = full.ndim
    br = (1,) * (rank - len(shape)) + tuple(shape)
    axes = tuple(i for i in range(rank) if br[i] == 1 and full.shape[i] != 1)
    if not axes:
        return full.reshape(shape)
    return o.reduce("sum", full, axes).reshape(shape)


@pytest.mark.parametrize("name,p", _cases("binary"))
def test_binary(name, p):
    ins, outs = load_golden("binary")[name]
    a, b, dy = ins["a"], ins["b"], ins["dy"]
    y = o.binary_fwd(p["op"], a, b)
    assert_bit_exact(y, outs["y"], name + " y")
    for which, key, src in ((0, "da", a), (1, "db", b)):
        full = o.binary_bwd(p["op"], which, np.zeros_like(y) if y.shape != src.shape else np.ones_like(y), a, b, y, dy)
        g = full if y.shape == src.shape else np.float32(1.0) + _reduce_to(full, src.shape)
        assert_bit_exact(g, outs[key], name + " " + key)


@pytest.mark.parametrize("name,p", _cases("pool"))
def test_pool(name, p):
    ins, outs = load_golden("pool")[name]
    y = o.pool2d_fwd(p["mode"], ins["x"], p["pool"], p["stride"], p["padding"])
    assert_bit_exact(y, outs["y"], name + " y")
    dy = cases._dy_like(ins["seed_dy"], y.shape)
    dx = o.pool2d_bwd(p["mode"], np.ones_like(ins["x"]), ins["x"], dy, y, p["pool"], p["stride"], p["padding"])
    assert_bit_exact(dx, outs["dx"], name + " dx")


@pytest.mark.parametrize("name,p", _cases("reduce"))
def test_reduce(name, p):
    ins, outs = load_golden("reduce")[name]
    x = ins["x"]
    y = o.reduce(p["op"], x, p["axes"], p["keepdims"])
    assert_bit_exact(y, outs["y"], name + " y")
    # backward through the [rows][cols] view
    axes = tuple(range(x.ndim)) if p["axes"] is None else tuple(sorted(a % x.ndim for a in p["axes"]))
    keep = tuple(a for a in range(x.ndim) if a not in axes)
    perm = keep + axes
    xt = np.ascontiguousarray(x.transpose(perm))
    cols = int(np.prod([x.shape[a] for a in axes]))
    rows = x.size // cols
    dy = cases._dy_like(ins["seed_dy"], y.shape)
    dxt = o.reduce_bwd5(p["op"], np.zeros_like(xt), xt, dy.reshape(-1), y.reshape(-1), rows, 1, 1, cols, 1)
    inv = np.argsort(perm)
    dx = np.float32(1.0) + dxt.reshape(xt.shape).transpose(inv)
    assert_bit_exact(dx, outs["dx"], name + " dx")


@pytest.mark.parametrize("name,p", _cases("transpose"))
def test_transpose(name, p):
    ins, outs = load_golden("transpose")[name]
    y = o.transpose(ins["x"], p["axes"])
    assert_bit_exact(y, outs["y"], name)
    assert_bit_exact(y, ins["x"].transpose(p["axes"]), name + " vs numpy")
    dy = cases._dy_like(ins["seed_dy"], y.shape)
    dx = o.transpose(dy, tuple(np.argsort(p["axes"])), out=np.ones_like(ins["x"]))
    assert_bit_exact(dx, outs["dx"], name + " dx")


@pytest.mark.parametrize("name,p", _cases("slice"))
def test_slice(name, p):
    from litenn_b200.info import InfoSlice
    from litenn_b200.ops import _hashable_slices
    from litenn_b200.shape import TensorShape
    ins, outs = load_golden("slice")[name]
    x = ins["x"]
    info = InfoSlice(TensorShape(x.shape), _hashable_slices(cases.SLICE_CASES[p["index"]][1]))
    begin, step = [b for b, _ in info.begin_step], [s for _, s in info.begin_step]
    y = o.slice_fwd(x, info.output_shape_krn.shape, begin, step).reshape(info.output_shape.shape)
    assert_bit_exact(y, outs["y"], name)
    dy = cases._dy_like(ins["seed_dy"], y.shape)
    dx = o.slice_bwd(np.ones_like(x), dy, info.output_shape_krn.shape, begin, step)
    assert_bit_exact(dx, outs["dx"], name + " dx")


@pytest.mark.parametrize("name,p", _cases("matmul"))
def test_matmul(name, p):
    ins, outs = load_golden("matmul")[name]
    a, b = ins["a"], ins["b"]
    y = o.gemm(a, b)
    dy = cases._dy_like(ins["seed_dy"], y.shape, p["integer"])
    da = o.gemm(dy, b, trans_b=True, out=np.ones_like(a))
    db = o.gemm(a, dy, trans_a=True, out=np.ones_like(b))
    check = assert_bit_exact if p["integer"] else (lambda g, w, what: assert_contraction_close(g, w, a.shape[-1], what))
    check(y, outs["y"], name + " y")
    check(da, outs["da"], name + " da")
    check(db, outs["db"], name + " db")
    # the sequential-k fp32 accumulation is the reference's: forward is bit-exact either way
    assert_bit_exact(y, outs["y"], name + " y (fp32 sequential k)")


@pytest.mark.parametrize("name,p", _cases("conv"))
def test_conv(name, p):
    ins, outs = load_golden("conv")[name]
    x, w = ins["x"], ins["w"]
    y = o.conv2d_fwd(x, w, p["stride"], p["dilation"], p["padding"])
    dy = cases._dy_like(ins["seed_dy"], y.shape, p["integer"])
    dx = o.conv2d_dx(np.ones_like(x), dy, w, x.shape, p["stride"], p["dilation"], p["padding"])
    dw = o.conv2d_dw(np.ones_like(w), dy, x, p["stride"], p["dilation"], p["padding"])
    assert_bit_exact(y, outs["y"], name + " y")
    assert_bit_exact(dx, outs["dx"], name + " dx")
    assert_bit_exact(dw, outs["dw"], name + " dw")


@pytest.mark.parametrize("name,p", _cases("conv_transpose"))
def test_conv_transpose(name, p):
    ins, outs = load_golden("conv_transpose")[name]
    x, k = ins["x"], ins["w"]
    args = (p["stride"], p["dilation"], p["padding"])
    y = o.conv2d_transpose_fwd(x, k, *args)
    dy = cases._dy_like(ins["seed_dy"], y.shape, p["integer"])
    assert_bit_exact(y, outs["y"], name + " y")
    assert_bit_exact(o.conv2d_transpose_dx(np.ones_like(x), dy, k, *args), outs["dx"], name + " dx")
    assert_bit_exact(o.conv2d_transpose_dk(np.ones_like(k), dy, x, *args), outs["dw"], name + " dk")


@pytest.mark.parametrize("name,p", _cases("depthwise"))
def test_depthwise(name, p):
    ins, outs = load_golden("depthwise")[name]
    x, k = ins["x"], ins["w"]
    args = (p["stride"], p["dilation"], p["padding"])
    y = o.depthwise_fwd(x, k, *args)
    dy = cases._dy_like(ins["seed_dy"], y.shape, p["integer"])
    assert_bit_exact(y, outs["y"], name + " y")
    assert_bit_exact(o.depthwise_dx(np.ones_like(x), dy, k, *args), outs["dx"], name + " dx")
    assert_bit_exact(o.depthwise_dk(np.ones_like(k), dy, x, *args), outs["dw"], name + " dk")


def _init_oracle(p, hash_seed):
    kind, a = p["kind"], p["args"]
    if kind == "uniform":
        return o.init_uniform(p["shape"], hash_seed, a[0], a[1])
    if kind == "normal":
        return o.init_normal(p["shape"], hash_seed, a[0], a[1])
    if kind == "he_uniform":
        lo, hi = o.he_uniform_limits(a[0], a[1])
        return o.init_uniform(p["shape"], hash_seed, lo, hi)
    return o.init_normal(p["shape"], hash_seed, 0.0, o.glorot_std(a[0], a[1], a[2]))


@pytest.mark.parametrize("name,p", _cases("init"))
def test_init(name, p):
    """Random initializers: the oracle's restatement of the PCG hashes against tensors the
    unmodified reference initialised (bit-exact: log / cos are the double functions rounded once
    in both)."""
    ins, outs = load_golden("init")[name]
    assert int(ins["hash_seed"][0]) == cases.init_seed(p["np_seed"])
    assert_bit_exact(_init_oracle(p, int(ins["hash_seed"][0])), outs["v"], name)


def test_conv_config1():
    ins, outs = load_golden("conv_config1")["conv_config1"]
    y = o.conv2d_fwd(ins["x"], ins["w"], 1, 1, "same", bias=ins["b"])
    assert_bit_exact(y, outs["y"], "config 1 conv + bias")
    y64 = o.conv2d_fwd(ins["x"], ins["w"], 1, 1, "same", bias=ins["b"], accum64=True)
    assert_contraction_close(y, y64, 144, "fp32 vs fp64 accumulation")


def test_chain():
    ins, outs = load_golden("chain")["chain"]
    assert_bit_exact(o.scale_bias_lrelu(ins["x"], ins["g"], ins["b"], 0.1), outs["y"], "leaky_relu(x*g+b)")


def test_sgd_matches_cnn_step_update():
    ins, outs = load_golden("cnn_step")["cnn_step"]
    for name in ("k0", "k1", "kb0", "kb1", "dw", "db"):
        assert_bit_exact(o.sgd(ins[name], outs["grad_" + name], 1e-3), outs["new_" + name], "sgd " + name)


def test_transcendental_restatement_is_double_rounded():
    # the golden values for exp/log/... were produced by the same "double libm, one rounding"
    # definition; this guards the definition against libm changes by a loose ulp bound
    ins, outs = load_golden("eltwise")["ew_exp"]
    assert ulp_diff(np.exp(ins["x"].astype(np.float64)).astype(np.float32), outs["y"]).max() <= 1
