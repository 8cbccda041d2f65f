"""Seeded parity cases, written against the `nn` namespace only, so the same code runs on the
reference (make_golden.py, producing the committed .npz fixtures) and on litenn_b200 (the GPU
parity tests).  Each case is (name, family, params, input builder); `run_case` returns a dict
of float32 arrays.  The procedures follow the reference's own self-tests (forward, then
backward into gradients PRE-FILLED with a constant to prove "+=" semantics:
litenn/core/op/conv2D.py:76-126, matmul.py:167-234, pool2D.py:232-282, reduce.py:303-367,
dual_wise_op.py:314-399, element_wise_op.py:367-403) with fixed seeds instead of np.random.
"""
import numpy as np

EW_OPS = {
    # name: (call(nn, x), needs_positive)
    "abs": (lambda nn, x: nn.abs(x), False),
    "add_const": (lambda nn, x: nn.add_const(x, 1.25), False),
    "clip": (lambda nn, x: nn.clip(x, -0.5, 0.75), False),
    "cos": (lambda nn, x: nn.cos(x), False),
    "div_const": (lambda nn, x: nn.div_const(x, 3.0), False),
    "exp": (lambda nn, x: nn.exp(x), False),
    "leaky_relu": (lambda nn, x: nn.leaky_relu(x, 0.1), False),
    "log": (lambda nn, x: nn.log(x), True),
    "mul_const": (lambda nn, x: nn.mul_const(x, -1.7), False),
    "rdiv_const": (lambda nn, x: nn.rdiv_const(x, 2.5), True),
    "rsub_const": (lambda nn, x: nn.rsub_const(x, 0.3), False),
    "relu": (lambda nn, x: nn.relu(x), False),
    "sigmoid": (lambda nn, x: nn.sigmoid(x), False),
    "sin": (lambda nn, x: nn.sin(x), False),
    "sqrt": (lambda nn, x: nn.sqrt(x), True),
    "square": (lambda nn, x: nn.square(x), False),
    "sub_const": (lambda nn, x: nn.sub_const(x, 0.6), False),
    "tanh": (lambda nn, x: nn.tanh(x), False),
}
# transcendental ops are delegated to the device math library by the reference: compared
# to a few ulp, everything else bit-exactly
EW_TRANSCENDENTAL = {"cos", "exp", "log", "sigmoid", "sin", "tanh"}

BIN_OPS = ["add", "sub", "mul", "div", "max", "min", "binary_crossentropy"]
BIN_SHAPES = [((4, 5), (4, 5)), ((3, 1, 5), (4, 1)), ((6,), (2, 3, 6)), ((2, 8, 3, 3), (1, 8, 1, 1)),
              ((1,), (3, 4)), ((5, 1), (1, 7))]

POOL_CASES = [  # (shape, pool, stride, padding)
    ((2, 3, 8, 8), 2, 2, "same"), ((1, 2, 7, 9), 2, 2, "same"), ((2, 2, 9, 7), 3, 2, "same"),
    ((1, 3, 8, 8), 3, 1, "valid"), ((2, 1, 6, 6), 2, 2, "valid"), ((1, 2, 5, 5), 3, 3, 1),
    ((1, 4, 12, 16), 2, 2, "same"),
]

REDUCE_CASES = [  # (shape, axes, keepdims)
    ((3, 4, 5, 6), None, False), ((3, 4, 5, 6), (1,), False), ((3, 4, 5, 6), (2, 3), True),
    ((3, 4, 5, 6), (0, 2, 3), False), ((3, 4, 5, 6), (0, 2), False), ((3, 4, 5, 6), (1, 3), True),
    ((4, 37), (1,), False), ((257, 3), (0,), False), ((2, 100, 3), (1,), False), ((1000,), None, False),
    ((2, 8, 16, 16), (2, 3), False), ((5, 1, 7), (-1,), False), ((64, 128), (1,), False),
    ((70000,), None, False),
]

TRANSPOSE_CASES = [((3, 5), (1, 0)), ((2, 3, 4), (2, 0, 1)), ((2, 3, 4, 5), (0, 3, 1, 2)),
                   ((2, 3, 4, 5), (1, 0, 2, 3)), ((4, 3, 2, 5, 2), (4, 2, 0, 3, 1)), ((7, 40, 33), (0, 2, 1))]

SLICE_CASES = [((5, 6, 7), (slice(1, 4), slice(None), slice(None, None, 2))),
               ((5, 6, 7), (2, Ellipsis, slice(None, None, -1))),
               ((4, 5), (slice(None, None, -2), 3)),
               ((3, 4, 5, 6), (Ellipsis, None, slice(1, 5, 3))),
               ((8,), (slice(6, 1, -2),))]

MATMUL_CASES = [  # (a_shape, b_shape, integer_valued)
    ((5, 7), (7, 3), True), ((16, 32), (32, 48), True), ((2, 3, 9, 13), (2, 3, 13, 6), True),
    ((33, 65), (65, 17), False), ((130, 100), (100, 260), False), ((4, 40, 24), (4, 24, 56), False),
]

CONV_CASES = [  # (x_shape, w_shape, stride, dilation, padding, integer_valued)
    ((2, 3, 8, 8), (4, 3, 3, 3), 1, 1, "same", True),
    ((1, 4, 9, 7), (6, 4, 3, 3), 2, 1, "same", True),
    ((2, 2, 10, 10), (3, 2, 5, 5), 1, 1, "valid", True),
    ((1, 3, 12, 12), (5, 3, 3, 3), 1, 2, "same", True),
    ((2, 8, 6, 6), (16, 8, 1, 1), 1, 1, "same", True),
    ((1, 5, 11, 13), (7, 5, 3, 3), 2, 2, 2, True),
    ((2, 16, 14, 14), (32, 16, 3, 3), 1, 1, "same", False),
    ((2, 12, 15, 15), (20, 12, 3, 3), 2, 1, "same", False),
    ((1, 40, 9, 9), (24, 40, 1, 1), 1, 1, "valid", False),
    ((3, 3, 16, 16), (8, 3, 3, 3), 1, 1, (1, 0, 2, 1), False),
]

# conv2DTranspose (op/conv2DTranspose.py:8-46): kernel (out_ch, in_ch, KH, KW), padding 'same' / 'valid'
CONVT_CASES = [  # (x_shape, k_shape, stride, dilation, padding, integer_valued)
    ((2, 3, 5, 6), (4, 3, 3, 3), 2, 1, "same", True),
    ((1, 4, 7, 5), (6, 4, 3, 3), 1, 1, "same", True),
    ((2, 2, 4, 4), (3, 2, 2, 2), 3, 1, "valid", True),      # kernel smaller than the stride: untouched pixels
    ((1, 3, 6, 6), (5, 3, 3, 3), 2, 2, "valid", True),
    ((2, 8, 6, 6), (16, 8, 1, 1), 2, 1, "same", True),
    ((2, 16, 9, 9), (24, 16, 3, 3), 2, 1, "same", False),
    ((1, 40, 8, 8), (12, 40, 4, 4), 2, 1, "same", False),
    ((2, 12, 10, 7), (20, 12, 3, 3), 1, 1, "valid", False),
]

# depthwise_conv2D (op/depthwise_conv2D.py:9-123): kernel (in_ch, KH, KW)
DEPTHWISE_CASES = [  # (x_shape, k_shape, stride, dilation, padding, integer_valued)
    ((2, 3, 8, 8), (3, 3, 3), 1, 1, "same", True),
    ((1, 4, 9, 7), (4, 3, 3), 2, 1, "same", True),
    ((2, 2, 10, 10), (2, 5, 5), 1, 2, "valid", True),
    ((1, 5, 11, 13), (5, 3, 3), 3, 1, 2, True),
    ((2, 16, 14, 14), (16, 3, 3), 1, 1, "same", False),
    ((3, 6, 16, 12), (6, 7, 7), 2, 1, (1, 0, 2, 1), False),
    ((2, 32, 20, 20), (32, 1, 1), 1, 1, "valid", False),
]


# random initializers (initializer/RandomUniform.py, RandomNormal.py, He.py, Glorot.py): the seed
# of the device-side hash is np.random.randint(2**31) drawn at initialisation time, so a case
# fixes numpy's legacy generator with np_seed first
INIT_CASES = [
    {"kind": "uniform", "args": (-0.5, 0.75), "shape": (5000,), "np_seed": 11},
    {"kind": "uniform", "args": (0.0, 1.0), "shape": (3, 7, 49), "np_seed": 12},
    {"kind": "normal", "args": (0.0, 1.0), "shape": (4096,), "np_seed": 13},
    {"kind": "normal", "args": (0.5, 0.02), "shape": (777,), "np_seed": 14},
    {"kind": "he_uniform", "args": (2.0, 36), "shape": (8, 4, 3, 3), "np_seed": 15},
    {"kind": "glorot_normal", "args": (1.0, 64, 10), "shape": (64, 10), "np_seed": 16},
]


def init_seed(np_seed):
    """The hash seed an initializer draws after np.random.seed(np_seed)."""
    np.random.seed(np_seed)
    return int(np.random.randint(2147483648))


def _rng(name):
    seed = int.from_bytes(name.encode(), "little") % (2**32)
    return np.random.default_rng(seed)


def all_cases():
    """(case name, family, params) for every parity case."""
    cases = []
    for op in EW_OPS:
        cases.append((f"ew_{op}", "eltwise", {"op": op}))
    for op in BIN_OPS:
        for i, (sa, sb) in enumerate(BIN_SHAPES):
            cases.append((f"bin_{op}_{i}", "binary", {"op": op, "a_shape": sa, "b_shape": sb}))
    for i, (shape, pool, stride, pad) in enumerate(POOL_CASES):
        for mode in ("avg", "max", "min"):
            cases.append((f"pool_{mode}_{i}", "pool", {"mode": mode, "shape": shape, "pool": pool, "stride": stride, "padding": pad}))
    for i, (shape, axes, keep) in enumerate(REDUCE_CASES):
        for op in ("sum", "mean", "max", "min"):
            cases.append((f"reduce_{op}_{i}", "reduce", {"op": op, "shape": shape, "axes": axes, "keepdims": keep}))
    for i, (shape, axes) in enumerate(TRANSPOSE_CASES):
        cases.append((f"transpose_{i}", "transpose", {"shape": shape, "axes": axes}))
    for i, (shape, sl) in enumerate(SLICE_CASES):
        cases.append((f"slice_{i}", "slice", {"shape": shape, "index": i}))
    for i, (sa, sb, integer) in enumerate(MATMUL_CASES):
        cases.append((f"matmul_{i}", "matmul", {"a_shape": sa, "b_shape": sb, "integer": integer}))
    for i, (sx, sw, s, d, p, integer) in enumerate(CONV_CASES):
        cases.append((f"conv_{i}", "conv", {"x_shape": sx, "w_shape": sw, "stride": s, "dilation": d, "padding": p, "integer": integer}))
    for i, (sx, sw, s, d, p, integer) in enumerate(CONVT_CASES):
        cases.append((f"convt_{i}", "conv_transpose", {"x_shape": sx, "w_shape": sw, "stride": s, "dilation": d, "padding": p, "integer": integer}))
    for i, (sx, sw, s, d, p, integer) in enumerate(DEPTHWISE_CASES):
        cases.append((f"depthwise_{i}", "depthwise", {"x_shape": sx, "w_shape": sw, "stride": s, "dilation": d, "padding": p, "integer": integer}))
    for i, p in enumerate(INIT_CASES):
        cases.append((f"init_{p['kind']}_{i}", "init", p))
    cases.append(("conv_config1", "conv_config1", {}))
    cases.append(("chain", "chain", {}))
    cases.append(("softmax_ce", "softmax_ce", {}))
    cases.append(("cnn_step", "cnn_step", {}))
    return cases


def make_inputs(name, family, p):
    """Deterministic float32 inputs of a case."""
    r = _rng(name)
    f32 = np.float32
    if family == "eltwise":
        x = r.uniform(-2.0, 2.0, (3, 5, 7)).astype(f32)
        if EW_OPS[p["op"]][1]:
            x = np.abs(x) + f32(0.25)
        return {"x": x, "dy": r.standard_normal((3, 5, 7)).astype(f32)}
    if family == "binary":
        a = r.uniform(0.1, 0.9, p["a_shape"]).astype(f32)
        b = r.uniform(0.1, 0.9, p["b_shape"]).astype(f32)
        if p["op"] not in ("binary_crossentropy", "div"):
            a, b = (a - f32(0.5)) * f32(4), (b - f32(0.5)) * f32(4)
        oshape = np.broadcast_shapes(p["a_shape"], p["b_shape"])
        return {"a": a, "b": b, "dy": r.standard_normal(oshape).astype(f32)}
    if family == "pool":
        n = int(np.prod(p["shape"]))
        x = (r.permutation(n).astype(f32) / f32(8.0) - f32(n / 16.0)).reshape(p["shape"])   # tie-free
        return {"x": x, "seed_dy": np.array([r.integers(1 << 30)], np.int64)}
    if family == "reduce":
        n = int(np.prod(p["shape"]))
        if p["op"] in ("max", "min"):
            x = (r.permutation(n).astype(f32) / f32(4.0) - f32(n / 8.0)).reshape(p["shape"])
        else:
            x = r.uniform(-1.0, 1.0, p["shape"]).astype(f32)
        return {"x": x, "seed_dy": np.array([r.integers(1 << 30)], np.int64)}
    if family in ("transpose", "slice"):
        return {"x": r.standard_normal(p["shape"]).astype(f32), "seed_dy": np.array([r.integers(1 << 30)], np.int64)}
    if family == "matmul":
        if p["integer"]:
            a = r.integers(0, 16, p["a_shape"]).astype(f32)
            b = r.integers(0, 16, p["b_shape"]).astype(f32)
        else:
            a = r.standard_normal(p["a_shape"]).astype(f32)
            b = r.standard_normal(p["b_shape"]).astype(f32)
        return {"a": a, "b": b, "seed_dy": np.array([r.integers(1 << 30)], np.int64)}
    if family in ("conv", "conv_transpose", "depthwise"):
        if p["integer"]:
            x = r.integers(0, 16, p["x_shape"]).astype(f32)
            w = r.integers(0, 16, p["w_shape"]).astype(f32)
        else:
            x = r.standard_normal(p["x_shape"]).astype(f32)
            fan = int(np.prod(p["w_shape"][1:]))
            w = (r.standard_normal(p["w_shape"]) * np.sqrt(2.0 / fan)).astype(f32)
        return {"x": x, "w": w, "seed_dy": np.array([r.integers(1 << 30)], np.int64), "integer": np.array([int(p["integer"])])}
    if family == "conv_config1":
        # single nn.conv2D forward: fp32 NCHW [8,16,32,32] ~N(0,1), weight [32,16,3,3] He-normal
        # (std sqrt(2/144)), stride 1, pad 'same', bias ~U(-0.1,0.1), seed 0
        r0 = np.random.default_rng(0)
        return {"x": r0.standard_normal((8, 16, 32, 32)).astype(f32),
                "w": (r0.standard_normal((32, 16, 3, 3)) * np.sqrt(2.0 / 144)).astype(f32),
                "b": r0.uniform(-0.1, 0.1, (32,)).astype(f32)}
    if family == "init":
        return {"np_seed": np.array([p["np_seed"]], np.int64), "hash_seed": np.array([init_seed(p["np_seed"])], np.int64)}
    if family == "chain":
        return {"x": r.standard_normal((3, 8, 6, 10)).astype(f32), "g": r.uniform(0.5, 1.5, (1, 8, 1, 1)).astype(f32),
                "b": r.uniform(-0.5, 0.5, (1, 8, 1, 1)).astype(f32)}
    if family == "softmax_ce":
        t = np.zeros((6, 10), f32)
        t[np.arange(6), r.integers(0, 10, 6)] = 1
        return {"logits": r.standard_normal((6, 10)).astype(f32), "target": t}
    if family == "cnn_step":
        d = {"x": r.uniform(0, 1, (4, 3, 16, 16)).astype(f32)}
        t = np.zeros((4, 10), f32)
        t[np.arange(4), r.integers(0, 10, 4)] = 1
        d["target"] = t
        chans = [3, 8, 16]
        for i in range(2):
            fan = chans[i] * 9
            d[f"k{i}"] = (r.standard_normal((chans[i + 1], chans[i], 3, 3)) * np.sqrt(2.0 / fan)).astype(f32)
            d[f"kb{i}"] = r.uniform(-0.1, 0.1, (chans[i + 1],)).astype(f32)
        d["dw"] = (r.standard_normal((16, 10)) * np.sqrt(2.0 / 16)).astype(f32)
        d["db"] = r.uniform(-0.1, 0.1, (10,)).astype(f32)
        return d
    raise KeyError(family)


def _dy_like(seed_arr, shape, integer=False):
    r = np.random.default_rng(int(seed_arr[0]))
    if integer:
        return r.integers(0, 8, shape).astype(np.float32)
    return r.standard_normal(shape).astype(np.float32)


def _prefill(t, value):
    t.get_grad().fill(value)


def run_case(nn, family, p, inp):
    """Run one case on the namespace `nn`; returns {output name: ndarray}."""
    T = nn.Tensor_from_value
    out = {}
    if family == "eltwise":
        x = T(inp["x"])
        _prefill(x, 1.0)
        y = EW_OPS[p["op"]][0](nn, x)
        out["y"] = y.np()
        nn.backward({y: inp["dy"]}, grad_for_non_trainables=True)
        out["dx"] = x.get_grad().np()
    elif family == "binary":
        a, b = T(inp["a"]), T(inp["b"])
        _prefill(a, 1.0)
        _prefill(b, 1.0)
        y = getattr(nn, p["op"])(a, b)
        out["y"] = y.np()
        nn.backward({y: inp["dy"]}, grad_for_non_trainables=True)
        out["da"], out["db"] = a.get_grad().np(), b.get_grad().np()
    elif family == "pool":
        x = T(inp["x"])
        _prefill(x, 1.0)
        y = getattr(nn, p["mode"] + "_pool2D")(x, p["pool"], p["stride"], p["padding"])
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape)}, grad_for_non_trainables=True)
        out["dx"] = x.get_grad().np()
    elif family == "reduce":
        x = T(inp["x"])
        _prefill(x, 1.0)
        y = getattr(nn, "reduce_" + p["op"])(x, p["axes"], p["keepdims"])
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape)}, grad_for_non_trainables=True)
        out["dx"] = x.get_grad().np()
    elif family == "transpose":
        x = T(inp["x"])
        _prefill(x, 1.0)
        y = nn.transpose(x, p["axes"])
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape)}, grad_for_non_trainables=True)
        out["dx"] = x.get_grad().np()
    elif family == "slice":
        x = T(inp["x"])
        _prefill(x, 1.0)
        y = x[SLICE_CASES[p["index"]][1]]
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape)}, grad_for_non_trainables=True)
        out["dx"] = x.get_grad().np()
    elif family == "matmul":
        a, b = T(inp["a"]), T(inp["b"])
        _prefill(a, 1.0)
        _prefill(b, 1.0)
        y = nn.matmul(a, b)
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape, p["integer"])}, grad_for_non_trainables=True)
        out["da"], out["db"] = a.get_grad().np(), b.get_grad().np()
    elif family == "conv":
        x, w = T(inp["x"]), T(inp["w"])
        _prefill(x, 1.0)
        _prefill(w, 1.0)
        y = nn.conv2D(x, w, stride=p["stride"], dilation=p["dilation"], padding=p["padding"])
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape, p["integer"])}, grad_for_non_trainables=True)
        out["dx"], out["dw"] = x.get_grad().np(), w.get_grad().np()
    elif family in ("conv_transpose", "depthwise"):
        x, w = T(inp["x"]), T(inp["w"])
        _prefill(x, 1.0)
        _prefill(w, 1.0)
        fn = nn.conv2DTranspose if family == "conv_transpose" else nn.depthwise_conv2D
        y = fn(x, w, stride=p["stride"], dilation=p["dilation"], padding=p["padding"])
        out["y"] = y.np()
        nn.backward({y: _dy_like(inp["seed_dy"], y.shape, p["integer"])}, grad_for_non_trainables=True)
        out["dx"], out["dw"] = x.get_grad().np(), w.get_grad().np()
    elif family == "conv_config1":
        x, w, b = T(inp["x"]), T(inp["w"]), T(inp["b"])
        y = nn.conv2D(x, w, stride=1, dilation=1, padding="same") + b.reshape((1, -1, 1, 1))
        out["y"] = y.np()
    elif family == "init":
        ini = nn.initializer
        make = {"uniform": lambda a: ini.RandomUniform(*a), "normal": lambda a: ini.RandomNormal(*a),
                "he_uniform": lambda a: ini.HeUniform(gain=a[0], fan_in=a[1]),
                "glorot_normal": lambda a: ini.GlorotNormal(gain=a[0], fan_in=a[1], fan_out=a[2])}[p["kind"]]
        np.random.seed(int(inp["np_seed"][0]))
        out["v"] = nn.Tensor(p["shape"], init=make(p["args"])).np()
    elif family == "chain":
        x, g, b = T(inp["x"]), T(inp["g"]), T(inp["b"])
        out["y"] = nn.leaky_relu(x * g + b, 0.1).np()
    elif family == "softmax_ce":
        lg, tg = T(inp["logits"]), T(inp["target"])
        prob = nn.softmax(lg)
        loss = nn.categorical_crossentropy(prob, tg).mean()
        out["prob"], out["loss"] = prob.np(), loss.np()
        loss.backward(grad_for_non_trainables=True)
        out["dlogits"] = lg.get_grad().np()
    elif family == "cnn_step":
        out.update(_cnn_step(nn, inp))
    else:
        raise KeyError(family)
    return {k: np.asarray(v, np.float32) for k, v in out.items()}


def _cnn_step(nn, inp):
    """conv3x3+lrelu+maxpool twice, global average, Dense, softmax-CE, one SGD(lr=1e-3) step:
    the structure of the small-CNN workload at a size the reference finishes in seconds."""
    T = nn.Tensor_from_value
    ks = [T(inp["k0"]), T(inp["k1"])]
    kbs = [T(inp["kb0"]), T(inp["kb1"])]
    dw, db = T(inp["dw"]), T(inp["db"])
    params = ks + kbs + [dw, db]
    opt = nn.optimizer.SGD(params, lr=1e-3)
    x = T(inp["x"])
    for k, kb in zip(ks, kbs):
        x = nn.conv2D(x, k, 1, 1, "same") + kb.reshape((1, -1, 1, 1))
        x = nn.leaky_relu(x, 0.1)
        x = nn.max_pool2D(x, 2, 2, "same")
    x = nn.flatten(nn.reduce_mean(x, (2, 3)))
    logits = nn.matmul(x, dw) + db
    loss = nn.categorical_crossentropy(nn.softmax(logits), T(inp["target"])).mean()
    out = {"logits": logits.np(), "loss": loss.np()}
    loss.backward()
    for name, t in zip(["k0", "k1", "kb0", "kb1", "dw", "db"], params):
        out["grad_" + name] = t.get_grad().np()
    opt.step()
    for name, t in zip(["k0", "k1", "kb0", "kb1", "dw", "db"], params):
        out["new_" + name] = t.np()
    return out
