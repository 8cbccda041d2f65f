"""GPU: litenn_b200 (CUDA kernels through the C ABI) against the reference's golden vectors
and the CPU oracle on the same seeded inputs.  Bit-exact for element-wise algebra, broadcast
binary, pooling, reductions (same summation tree), transpose/slice and integer-valued
contractions; a few ulp for the transcendental functions (the reference leaves them to the
device math library); the stated contraction tolerance (rel 1e-4 per element or 1e-3 max-abs
after dividing by sqrt(K)) for real-valued conv/matmul."""
import numpy as np
import pytest

import cases
from conftest import assert_bit_exact, assert_contraction_close, load_golden, ulp_diff

pytestmark = pytest.mark.gpu

TRANSCENDENTAL_ULP = 4   # OpenCL 1.2 allows exp/log <= 3 ulp, sin/cos <= 4 ulp


def _cases(*families):
    return [pytest.param(n, f, p, id=n) for n, f, p in cases.all_cases() if f in families]


def _check_ulp(got, want, max_ulp, what, atol=0.0):
    d = ulp_diff(got, want)
    bad = (d > max_ulp) & (np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)) > atol)
    assert not bad.any(), f"{what}: max ulp distance {int(d.max())} > {max_ulp}"


@pytest.mark.parametrize("name,family,p", _cases("eltwise"))
def test_eltwise(nn_gpu, name, family, p):
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    if p["op"] in cases.EW_TRANSCENDENTAL:
        # tanh is written 2/(1+exp(-2x)) - 1: the final subtraction amplifies exp's last-bit
        # differences near 0, so it gets an absolute allowance of a few ulp of 1.0
        _check_ulp(got["y"], outs["y"], TRANSCENDENTAL_ULP, name + " y", atol=1e-6 if p["op"] == "tanh" else 1e-7)
        # gradients combine the function value with dO and the pre-filled 1.0
        np.testing.assert_allclose(got["dx"], outs["dx"], rtol=2e-6, atol=2e-6, err_msg=name + " dx")
    else:
        assert_bit_exact(got["y"], outs["y"], name + " y")
        assert_bit_exact(got["dx"], outs["dx"], name + " dx")


@pytest.mark.parametrize("name,family,p", _cases("binary"))
def test_binary(nn_gpu, name, family, p):
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    if p["op"] == "binary_crossentropy":      # contains log()
        for k in ("y", "da", "db"):
            np.testing.assert_allclose(got[k], outs[k], rtol=3e-6, atol=3e-6, err_msg=f"{name} {k}")
    else:
        for k in ("y", "da", "db"):
            assert_bit_exact(got[k], outs[k], f"{name} {k}")


@pytest.mark.parametrize("name,family,p", _cases("pool", "reduce", "transpose", "slice", "chain"))
def test_exact_families(nn_gpu, name, family, p):
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    for k in outs:
        assert_bit_exact(got[k], outs[k], f"{name} {k}")


@pytest.mark.parametrize("name,family,p", _cases("matmul"))
def test_matmul(nn_gpu, name, family, p):
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    a_shape, b_shape = p["a_shape"], p["b_shape"]
    ks = {"y": a_shape[-1], "da": b_shape[-1], "db": a_shape[-2]}
    for k in outs:
        if p["integer"]:
            assert_bit_exact(got[k], outs[k], f"{name} {k}")
        else:
            assert_contraction_close(got[k], outs[k], ks[k], f"{name} {k}")


@pytest.mark.parametrize("name,family,p", _cases("conv"))
def test_conv(nn_gpu, name, family, p):
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    (N, IC, IH, IW), (OC, _, KH, KW) = p["x_shape"], p["w_shape"]
    OH, OW = outs["y"].shape[2:]
    ks = {"y": IC * KH * KW, "dx": OC * KH * KW, "dw": N * OH * OW}
    for k in outs:
        if p["integer"]:
            assert_bit_exact(got[k], outs[k], f"{name} {k}")
        else:
            assert_contraction_close(got[k], outs[k], ks[k], f"{name} {k}")


@pytest.mark.parametrize("name,family,p", _cases("conv_transpose"))
def test_conv_transpose(nn_gpu, name, family, p):
    """conv2DTranspose forward, dI and dK on the tile engine against the unmodified reference
    (gradients accumulated into tensors pre-filled with 1); integer cases bit for bit."""
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    (N, IC, IH, IW), (OC, _, KH, KW) = p["x_shape"], p["w_shape"]
    OH, OW = outs["y"].shape[2:]
    ks = {"y": IC * KH * KW, "dx": OC * KH * KW, "dw": N * OH * OW}
    for k in outs:
        if p["integer"]:
            assert_bit_exact(got[k], outs[k], f"{name} {k}")
        else:
            assert_contraction_close(got[k], outs[k], ks[k], f"{name} {k}")
    nn_gpu.devices.check_status()


@pytest.mark.parametrize("name,family,p", _cases("depthwise"))
def test_depthwise(nn_gpu, name, family, p):
    """depthwise_conv2D: forward, dI and dK bit for bit (same products, same order of additions)."""
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)
    for k in outs:
        assert_bit_exact(got[k], outs[k], f"{name} {k}")


def test_conv_config1(nn_gpu):
    """The single-conv configuration: x[8,16,32,32], w[32,16,3,3] He-normal, bias, 'same'."""
    import oracle as o
    ins, outs = load_golden("conv_config1")["conv_config1"]
    got = cases.run_case(nn_gpu, "conv_config1", {}, ins)
    assert_contraction_close(got["y"], outs["y"], 144, "config 1 vs reference")
    y64 = o.conv2d_fwd(ins["x"], ins["w"], 1, 1, "same", bias=ins["b"], accum64=True)
    assert_contraction_close(got["y"], y64, 144, "config 1 vs fp64 oracle")
    # split-TF32 should be at least as close to the fp64 result as fp32 sequential accumulation
    err_gpu = np.abs(got["y"].astype(np.float64) - y64).max()
    err_ref = np.abs(outs["y"].astype(np.float64) - y64).max()
    assert err_gpu <= 4 * err_ref + 1e-6, (err_gpu, err_ref)


def test_fused_conv_bias_lrelu_equals_unfused(nn_gpu):
    nn = nn_gpu
    ins, _ = load_golden("conv_config1")["conv_config1"]
    x, w, b = (nn.Tensor_from_value(ins[k]) for k in ("x", "w", "b"))
    with nn.deferred.disabled():          # one kernel per operator, as the reference runs the chain
        unfused = nn.leaky_relu(nn.conv2D(x, w) + b.reshape((1, -1, 1, 1)), 0.1).np()
    fused = nn.conv2D(x, w, bias_t=b, activation="leaky_relu", alpha=0.1).np()
    assert_bit_exact(fused, unfused, "conv epilogue fusion")
    # non-finite pre-activations must take the reference's literal form (0 * inf = NaN)
    bs = ins["b"].copy()
    bs[:4] = [np.inf, -np.inf, np.nan, 3e38]
    b2 = nn.Tensor_from_value(bs)
    with nn.deferred.disabled():
        unfused = nn.leaky_relu(nn.conv2D(x, w) + b2.reshape((1, -1, 1, 1)), 0.1).np()
    fused = nn.conv2D(x, w, bias_t=b2, activation="leaky_relu", alpha=0.1).np()
    assert_bit_exact(fused, unfused, "conv epilogue fusion, non-finite bias")


@pytest.mark.parametrize("xs,ws", [((2, 3, 17, 13), (8, 3, 3, 3)), ((2, 3, 32, 32), (32, 3, 3, 3)),
                                   ((2, 16, 12, 12), (24, 16, 3, 3)), ((1, 4, 9, 9), (5, 4, 5, 5))])
def test_conv_pool_fusion_equals_chain(nn_gpu, xs, ws):
    """conv2D_pool (direct FP32 kernel for IC <= 4, tile engine + pooling otherwise) against
    the unfused chain and the oracle."""
    import oracle as o
    nn = nn_gpu
    rng = np.random.default_rng(12)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.2).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (ws[0],)).astype(np.float32)
    xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(b)
    with nn.deferred.disabled():
        chain = nn.max_pool2D(nn.conv2D(xt, wt, bias_t=bt, activation="leaky_relu", alpha=0.1), 2, 2, "same").np()
    fused = nn.conv2D_pool(xt, wt, bias_t=bt, activation="leaky_relu", alpha=0.1).np()
    assert_bit_exact(fused, chain, "conv2D_pool vs chain")
    want = o.pool2d_fwd("max", o.conv2d_fwd(x, w, 1, 1, "same", bias=b, act=1, alpha=0.1, accum64=True), 2, 2, "same")
    assert_contraction_close(fused, want, ws[1] * ws[2] * ws[3], "conv2D_pool vs oracle")


@pytest.mark.parametrize("xs,ws,dil", [((3, 32, 64, 64), (64, 32, 3, 3), 1), ((2, 64, 32, 32), (128, 64, 3, 3), 1),
                                       ((2, 128, 16, 16), (200, 128, 3, 3), 1), ((2, 32, 30, 27), (48, 32, 3, 3), 1),
                                       ((2, 32, 40, 40), (64, 32, 3, 3), 2), ((2, 64, 28, 28), (96, 64, 5, 5), 1),
                                       ((2, 64, 21, 64), (24, 64, 3, 3), 1)])
def test_conv_halo_kernel(nn_gpu, monkeypatch, xs, ws, dil):
    """The unit-stride kernel with a halo-resident pixel patch (forced on, then forced off):
    forward with fused bias + leaky_relu, and the input gradient, against the fp64 oracle."""
    import oracle as o
    nn = nn_gpu
    rng = np.random.default_rng(5)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (ws[0],)).astype(np.float32)
    want = o.conv2d_fwd(x, w, 1, dil, "same", bias=b, act=1, alpha=0.1, accum64=True)
    dy = rng.standard_normal(want.shape).astype(np.float32)
    want_dx = o.conv2d_dx(np.zeros(xs, np.float32), dy, w, xs, 1, dil, "same", accum64=True)
    results = {}
    for mode in ("2", "0"):
        monkeypatch.setenv("LNN_TC_HALO", mode)
        xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(b)
        y = nn.conv2D(xt, wt, dilation=dil, bias_t=bt, activation="leaky_relu", alpha=0.1)
        assert_contraction_close(y.np(), want, ws[1] * ws[2] * ws[3], f"halo={mode} forward")
        assert np.abs(y.np() - want).max() <= 2e-5 * np.abs(want).max(), "split-TF32 accuracy"
        lin = nn.conv2D(xt, wt, dilation=dil)
        nn.backward({lin: dy}, grad_for_non_trainables=True)
        assert_contraction_close(xt.get_grad().np(), want_dx, ws[0] * ws[2] * ws[3], f"halo={mode} dX")
        results[mode] = y.np()
    nn.devices.check_status()
    assert_contraction_close(results["2"], results["0"], ws[1] * ws[2] * ws[3], "halo kernel vs per-tap kernel")


@pytest.mark.parametrize("xs,ws,stride,dil", [((8, 3, 33, 31), (20, 3, 3, 3), 1, 1), ((4, 3, 40, 44), (40, 3, 3, 3), 2, 1),
                                              ((4, 1, 24, 24), (8, 1, 3, 3), 1, 2), ((3, 4, 128, 128), (32, 4, 3, 3), 1, 1),
                                              ((2, 2, 7, 300), (33, 2, 3, 3), 1, 1)])
def test_conv_direct_dw(nn_gpu, monkeypatch, xs, ws, stride, dil):
    """Kernel gradient of few-input-channel layers on the FP32 pipes (IC <= 4, 3x3), against the
    fp64 oracle and against the tile-engine path; a second call must add into dW."""
    import oracle as o
    nn = nn_gpu
    rng = np.random.default_rng(6)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    y_shape = o.conv2d_fwd(x, w, stride, dil, "same").shape
    dy = rng.standard_normal(y_shape).astype(np.float32)
    want = o.conv2d_dw(np.zeros(ws, np.float32), dy, x, stride, dil, "same", accum64=True)
    K = xs[0] * y_shape[2] * y_shape[3]
    got = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("LNN_CONV_DIRECT", mode)
        xt, wt = nn.Tensor_from_value(x), nn.Tensor_from_value(w)
        y = nn.conv2D(xt, wt, stride=stride, dilation=dil)
        nn.backward({y: dy}, grad_for_non_trainables=True)
        got[mode] = wt.get_grad().np()
        assert_contraction_close(got[mode], want, K, f"direct={mode} dW")
        if mode == "1":
            y2 = nn.conv2D(xt, wt, stride=stride, dilation=dil)
            nn.backward({y2: dy}, grad_for_non_trainables=True)
            assert_contraction_close(wt.get_grad().np(), 2 * want, K, "dW accumulates")
    nn.devices.check_status()


@pytest.mark.parametrize("xs,ws", [((2, 3, 32, 32), (16, 3, 3, 3)), ((2, 32, 16, 24), (40, 32, 3, 3)),
                                   ((2, 8, 10, 10), (8, 8, 3, 3)), ((3, 32, 64, 64), (64, 32, 3, 3)),
                                   ((2, 64, 32, 32), (128, 64, 3, 3)), ((2, 16, 12, 12), (24, 16, 3, 3)),
                                   ((2, 8, 8, 12), (8, 8, 5, 5)), ((2, 3, 32, 64), (32, 3, 3, 3)),
                                   ((3, 4, 14, 128), (40, 4, 3, 3)), ((2, 1, 64, 64), (8, 1, 3, 3))])
def test_conv_block_equals_chain(nn_gpu, xs, ws):
    """conv2D_block (one trainable op: pool in the convolution's epilogue with the map of winning
    positions, fused pooling + leaky_relu gradient) against the chain conv2D(+bias, leaky_relu) ->
    max_pool2D: values, dX and dW bit for bit; the bias gradient sums the same terms in another
    order.  Ties inside a window (values repeated on purpose) must route the gradient to the first
    position, as the chain does."""
    nn = nn_gpu
    rng = np.random.default_rng(31)
    x = rng.standard_normal(xs).astype(np.float32)
    x[0, :, : xs[2] // 2] = 0.5                    # a constant region: every window there is a four-way tie
    w = (rng.standard_normal(ws) * 0.2).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (ws[0],)).astype(np.float32)
    dp = rng.standard_normal((xs[0], ws[0], (xs[2] + 1) // 2, (xs[3] + 1) // 2)).astype(np.float32)
    res = {}
    for kind in ("chain", "block"):
        xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(b)
        if kind == "chain":
            y = nn.max_pool2D(nn.conv2D(xt, wt, bias_t=bt, activation="leaky_relu", alpha=0.1), 2, 2, "same")
        else:
            y = nn.conv2D_block(xt, wt, bias_t=bt, activation="leaky_relu", alpha=0.1)
        nn.backward({y: dp}, grad_for_non_trainables=True)
        res[kind] = (y.np(), xt.get_grad().np(), wt.get_grad().np(), bt.get_grad().np())
    # a pooled first layer (at most 4 input channels, width a multiple of 64) sums the kernel
    # gradient over the winners of the pooling windows: the chain's non-zero terms, another order
    winners = xs[1] <= 4 and ws[2] == 3 and xs[3] % 64 == 0
    for name, a, c in zip(("y", "dx", "dw"), res["block"], res["chain"]):
        if name == "dw" and winners:
            assert_contraction_close(a, c, xs[0] * xs[2] * xs[3], "conv2D_block dw (winners)")
            assert float(np.abs(a - c).max()) <= 2e-5 * float(np.abs(c).max()) + 1e-6
        else:
            assert_bit_exact(a, c, f"conv2D_block {name}")
    np.testing.assert_allclose(res["block"][3], res["chain"][3], rtol=1e-5, atol=1e-5, err_msg="conv2D_block db")
    nn.devices.check_status()


def test_training_steps_do_not_accumulate_memory(nn_gpu):
    """Tensors of a finished step must be released by reference counting alone (no reference
    cycle through the grad functions): with the cycle collector off, device memory in use after
    step 6 equals that after step 3."""
    import ctypes
    import gc
    from litenn_b200 import _lib
    nn = nn_gpu
    lib = _lib.get_lib()
    dev = nn.devices.get_current()[0]
    rng = np.random.default_rng(3)

    class Net(nn.Module):
        def __init__(self):
            self.c1 = nn.Conv2D(3, 8, 3)
            self.c2 = nn.Conv2D(8, 16, 3)
            self.dense = nn.Dense(16, 5)

    net = Net()
    c1, c2, dense = net.c1, net.c2, net.dense
    x = nn.Tensor_from_value(rng.standard_normal((4, 3, 16, 16)).astype(np.float32))
    onehot = nn.Tensor_from_value(np.eye(5, dtype=np.float32)[rng.integers(0, 5, 4)])
    opt = nn.optimizer.SGD(net.trainables(), lr=1e-3)

    def step():
        h = nn.conv2D_block(x, c1.kernel, bias_t=c1.bias, activation="leaky_relu", alpha=0.1)
        h = nn.conv2D(h, c2.kernel, bias_t=c2.bias, activation="leaky_relu", alpha=0.1)
        logits = dense(nn.flatten(nn.reduce_mean(h, (2, 3))))
        loss = nn.categorical_crossentropy(nn.softmax(logits), onehot).mean()
        loss.backward()
        opt.step()
        opt.zero_grad()

    def live_bytes():
        a, p = ctypes.c_uint64(), ctypes.c_uint64()
        lib.lnn_mem_stats(dev.index, ctypes.byref(a), ctypes.byref(p))
        return a.value - p.value

    gc.collect()
    gc.disable()
    try:
        for _ in range(3):
            step()
        after3 = live_bytes()
        for _ in range(3):
            step()
        after6 = live_bytes()
    finally:
        gc.enable()
    assert after6 == after3, f"live device memory grew from {after3} to {after6} bytes over three steps"


def _tf32_rna(x):
    """cvt.rna.tf32.f32 on the host: nearest, ties away from zero, 10 mantissa bits kept."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x1000) & 0xFFFFE000).astype(np.uint32).view(np.float32)


def _expected_split(x, precision, e=None):
    """hi, lo and scale exponent the packed operand format must hold for the fp32 array x (e: the
    scale exponent the writer chose, when it derives it from a bound rather than from x)."""
    x = np.ascontiguousarray(x, np.float32)
    if precision != 2:
        hi = _tf32_rna(x)
        return hi, _tf32_rna(x - hi), 0
    from litenn_b200.ops import scale_exponent_of
    if e is None:
        e = scale_exponent_of(int(np.abs(x).max().astype(np.float32).view(np.uint32)))
    xs = np.ldexp(x, -e).astype(np.float32)          # exact: a power of two
    hi = xs.astype(np.float16)                       # round to nearest even, as cvt.rn.f16.f32
    return hi, (xs - hi.astype(np.float32)).astype(np.float16), e


@pytest.mark.parametrize("xs,ws", [((2, 3, 32, 32), (32, 3, 3, 3)), ((3, 32, 64, 64), (64, 32, 3, 3)),
                                   ((2, 64, 32, 32), (128, 64, 3, 3)), ((2, 32, 64, 64), (40, 32, 3, 3)),
                                   ((2, 16, 12, 12), (24, 16, 3, 3)), ((2, 64, 30, 34), (64, 64, 3, 3)),
                                   ((2, 64, 64, 32), (200, 64, 3, 3))])
def test_conv_infer_fused_and_packed(nn_gpu, xs, ws):
    """conv2D_infer: pooled NCHW output, packed output and packed input against the un-fused
    chain (bit-exact: the fused epilogues apply the same roundings in the same order)."""
    nn = nn_gpu
    rng = np.random.default_rng(21)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (ws[0],)).astype(np.float32)
    xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(b)
    kw = dict(bias_t=bt, activation="leaky_relu", alpha=0.1)
    with nn.deferred.disabled():
        chain = nn.max_pool2D(nn.conv2D(xt, wt, **kw), 2, 2, "same").np()
    pooled = nn.conv2D_infer(xt, wt, pool=True, **kw).np()
    assert_bit_exact(pooled, chain, "pool fused into the epilogue")
    packed = nn.conv2D_infer(xt, wt, pool=True, packed_output=True, **kw)
    oc = ws[0]
    hi, lo = packed.hi_np(), packed.lo_np()
    # a convolution scales its packed output by a bound of the result (never below the measured
    # maximum, and for these weights within 2**7 of it) and records the measured maximum beside it
    tight_e = _expected_split(chain, packed.precision)[2]
    if packed.precision == 2:
        assert tight_e <= packed.scale_exponent() <= tight_e + 7, (packed.scale_exponent(), tight_e)
        assert packed.largest_magnitude() == float(np.abs(chain).max())
    want_hi, want_lo, want_e = _expected_split(chain, packed.precision, packed.scale_exponent())
    assert_bit_exact(hi[..., :oc].transpose(0, 3, 1, 2), want_hi, "packed hi")
    assert_bit_exact(lo[..., :oc].transpose(0, 3, 1, 2), want_lo, "packed lo")
    assert not hi[..., oc:].any() and not lo[..., oc:].any(), "pad channels must be zero"
    # packed input: same result as the NCHW input, with and without the fused pool
    xp = nn.pack_activation(xt)
    got_pool = nn.conv2D_infer(xp, wt, pool=True, **kw).np()
    got_plain = nn.conv2D_infer(xp, wt, **kw).np()
    if xs[1] <= 4:
        # an NCHW input with so few channels takes the FP32-pipe kernel, a packed one the tensor cores
        K = ws[1] * ws[2] * ws[3]
        assert_contraction_close(got_pool, chain, K, "packed input, pooled")
        assert_contraction_close(got_plain, nn.conv2D(xt, wt, **kw).np(), K, "packed input, plain")
    else:
        assert_bit_exact(got_pool, chain, "packed input, pooled")
        assert_bit_exact(got_plain, nn.conv2D(xt, wt, **kw).np(), "packed input, plain")
    nn.devices.check_status()


@pytest.mark.parametrize("xs,ws", [((2, 3, 32, 32), (32, 3, 3, 3)), ((2, 32, 64, 64), (64, 32, 3, 3)),
                                   ((2, 64, 32, 32), (128, 64, 3, 3))])
def test_fused_pool_epilogue_non_finite(nn_gpu, xs, ws):
    """The fused epilogues reduce the 2x2 window before bias and activation (same bits on finite
    values); windows with inf / NaN must fall back to the literal order of the chain."""
    nn = nn_gpu
    rng = np.random.default_rng(41)
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (ws[0],)).astype(np.float32)
    b[:6] = [np.inf, -np.inf, np.nan, 3e38, -3e38, 0.0]
    x[0, 0, 5, 5] = np.inf          # a few windows with non-finite convolution results
    x[1, 1, 9, 4] = np.nan
    xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(b)
    kw = dict(bias_t=bt, activation="leaky_relu", alpha=0.1)
    with nn.deferred.disabled():
        chain = nn.max_pool2D(nn.conv2D(xt, wt, **kw), 2, 2, "same").np()
    fused = nn.conv2D_infer(xt, wt, pool=True, **kw).np()
    assert_bit_exact(fused, chain, "fused pool epilogue with non-finite values")
    nn.devices.check_status()


@pytest.mark.parametrize("name,family,p", _cases("init"))
def test_random_initializers(nn_gpu, name, family, p):
    """Device-side random initializers against tensors the unmodified reference initialised
    after the same np.random.seed: the uniform family bit for bit (integer hash times 2^-32),
    the normal family to the rounding of the device's logf / cosf."""
    ins, outs = load_golden(family)[name]
    got = cases.run_case(nn_gpu, family, p, ins)["v"]
    if p["kind"] in ("uniform", "he_uniform"):
        assert_bit_exact(got, outs["v"], name)
    else:
        std = p["args"][1] if p["kind"] == "normal" else float(np.std(outs["v"]))
        np.testing.assert_allclose(got, outs["v"], rtol=2e-5, atol=1e-5 * std, err_msg=name)


def _random_conv_geometries(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(count):
        k = int(rng.choice([1, 3, 3, 5]))
        out.append((int(rng.integers(1, 4)), int(rng.choice([3, 8, 16, 32, 40, 64])), int(rng.integers(k + 2, 41)),
                    int(rng.integers(k + 2, 41)), int(rng.choice([8, 24, 64, 100, 130])), k,
                    int(rng.choice([1, 1, 2])), int(rng.choice([1, 1, 2]))))
    return out


@pytest.mark.parametrize("n,ic,h,w,oc,k,stride,dil", _random_conv_geometries(24, 2024))
def test_conv_random_geometries(nn_gpu, n, ic, h, w, oc, k, stride, dil):
    """Seeded random geometries (channel counts off the 8/32 grid, odd sizes, strides, dilations,
    1x1 to 5x5 taps): forward with fused bias + leaky_relu, dX and dW against the fp64 oracle,
    and the inference entry with fused pool and packed output against the un-fused chain."""
    import oracle as o
    nn = nn_gpu
    rng = np.random.default_rng(n * 1000003 + ic * 10007 + h * 101 + w)
    x = rng.standard_normal((n, ic, h, w)).astype(np.float32)
    wt_np = (rng.standard_normal((oc, ic, k, k)) * 0.1).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (oc,)).astype(np.float32)
    want = o.conv2d_fwd(x, wt_np, stride, dil, "same", bias=b, act=1, alpha=0.1, accum64=True)
    lin = o.conv2d_fwd(x, wt_np, stride, dil, "same", accum64=True)
    dy = rng.standard_normal(lin.shape).astype(np.float32)
    want_dx = o.conv2d_dx(np.zeros_like(x), dy, wt_np, x.shape, stride, dil, "same", accum64=True)
    want_dw = o.conv2d_dw(np.zeros_like(wt_np), dy, x, stride, dil, "same", accum64=True)
    xt, wt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(wt_np), nn.Tensor_from_value(b)
    kw = dict(stride=stride, dilation=dil, bias_t=bt, activation="leaky_relu", alpha=0.1)
    y = nn.conv2D(xt, wt, **kw)
    assert_contraction_close(y.np(), want, ic * k * k, "forward")
    z = nn.conv2D(xt, wt, stride=stride, dilation=dil)
    nn.backward({z: dy}, grad_for_non_trainables=True)
    assert_contraction_close(xt.get_grad().np(), want_dx, oc * k * k, "dX")
    assert_contraction_close(wt.get_grad().np(), want_dw, n * lin.shape[2] * lin.shape[3], "dW")
    chain = nn.max_pool2D(y, 2, 2, "same").np()
    assert_bit_exact(nn.conv2D_infer(xt, wt, pool=True, **kw).np(), chain, "fused pool")
    packed = nn.conv2D_infer(xt, wt, pool=True, packed_output=True, **kw)
    assert_bit_exact(packed.hi_np()[..., :oc].transpose(0, 3, 1, 2),
                     _expected_split(chain, packed.precision, packed.scale_exponent())[0], "packed hi")
    nn.devices.check_status()


def test_softmax_ce(nn_gpu):
    """Fused softmax / categorical cross-entropy (one kernel each way) and the reference's
    composition of nine operators, both against what the unmodified reference produced."""
    ins, outs = load_golden("softmax_ce")["softmax_ce"]
    got = cases.run_case(nn_gpu, "softmax_ce", {}, ins)
    for k in outs:
        np.testing.assert_allclose(got[k], outs[k], rtol=1e-5, atol=1e-6, err_msg=f"fused {k}")
    with nn_gpu.deferred.disabled():
        comp = cases.run_case(nn_gpu, "softmax_ce", {}, ins)
    for k in outs:
        np.testing.assert_allclose(comp[k], outs[k], rtol=1e-5, atol=1e-6, err_msg=f"composition {k}")
    # forward values of the fused kernels are those of the composition, bit for bit
    assert_bit_exact(got["prob"], comp["prob"], "softmax")
    assert_bit_exact(got["loss"], comp["loss"], "cross-entropy")
    np.testing.assert_allclose(got["dlogits"], comp["dlogits"], rtol=2e-6, atol=1e-8)


def test_softmax_ce_classifier_size(nn_gpu):
    """[1024, 1000] logits (the classifier's micro-batch), one-hot targets and a shared target
    row: fused kernels against the composition."""
    nn = nn_gpu
    rng = np.random.default_rng(41)
    lg = (rng.standard_normal((1024, 1000)) * 3).astype(np.float32)
    onehot = np.zeros((1024, 1000), np.float32)
    onehot[np.arange(1024), rng.integers(0, 1000, 1024)] = 1
    shared = rng.dirichlet(np.ones(1000)).astype(np.float32)
    launches = {}
    for tg in (onehot, shared):
        res = {}
        for mode in ("fused", "composed"):
            lt, tt = nn.Tensor_from_value(lg), nn.Tensor_from_value(tg)
            dev = nn.devices.get_current()[0]
            n0 = dev.launch_count()
            if mode == "composed":
                with nn.deferred.disabled():
                    p = nn.softmax(lt)
                    loss = nn.categorical_crossentropy(p, tt).mean()
                    loss.backward(grad_for_non_trainables=True)
            else:
                p = nn.softmax(lt)
                loss = nn.categorical_crossentropy(p, tt).mean()
                loss.backward(grad_for_non_trainables=True)
            launches[mode] = dev.launch_count() - n0
            res[mode] = (p.np(), loss.np(), lt.get_grad().np())
        assert_bit_exact(res["fused"][0], res["composed"][0], "softmax")
        assert_bit_exact(res["fused"][1], res["composed"][1], "mean cross-entropy")
        np.testing.assert_allclose(res["fused"][2], res["composed"][2], rtol=1e-5, atol=1e-9)
    assert launches["fused"] * 2 <= launches["composed"], launches
    nn.devices.check_status()


def test_cnn_training_step(nn_gpu):
    """Forward, loss, backward and one SGD step of the small CNN against the reference."""
    ins, outs = load_golden("cnn_step")["cnn_step"]
    got = cases.run_case(nn_gpu, "cnn_step", {}, ins)
    np.testing.assert_allclose(got["logits"], outs["logits"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(got["loss"], outs["loss"], rtol=1e-5)
    for k in outs:
        if k.startswith("grad_"):
            scale = np.abs(outs[k]).max()
            np.testing.assert_allclose(got[k], outs[k], rtol=1e-3, atol=1e-4 * scale, err_msg=k)
        if k.startswith("new_"):
            np.testing.assert_allclose(got[k], outs[k], rtol=1e-6, atol=1e-7, err_msg=k)


def test_output_t_and_accumulate(nn_gpu):
    """The `output_t=` / `is_add_to_output=` convention (e.g. element_wise_op.py:48-76)."""
    nn = nn_gpu
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 6)).astype(np.float32)
    base = rng.standard_normal((24,)).astype(np.float32)
    xt, out = nn.Tensor_from_value(x), nn.Tensor_from_value(base)
    nn.op.square_op(xt, output_t=out, is_add_to_output=True)
    assert_bit_exact(out.np(), base + (x * x).reshape(-1), "square += into other shape")
    with pytest.raises(ValueError):
        nn.op.square_op(xt, output_t=nn.Tensor((5,)))
    a = nn.Tensor_from_value(rng.integers(0, 8, (6, 5)).astype(np.float32))
    b = nn.Tensor_from_value(rng.integers(0, 8, (5, 7)).astype(np.float32))
    c0 = rng.integers(0, 8, (6, 7)).astype(np.float32)
    c = nn.Tensor_from_value(c0)
    nn.op.matmul_op(a, b, output_t=c, is_add_to_output=True)
    assert_bit_exact(c.np(), c0 + a.np() @ b.np(), "matmul +=")


def test_device_status_clean(nn_gpu):
    """No bounded device-side wait may have expired during the parity run."""
    nn_gpu.devices.check_status()


@pytest.mark.parametrize("precision", ["3"])
def test_fused_paths_in_split_tf32(nn_gpu, monkeypatch, precision):
    """The fused epilogues, the packed operand format and the pooled block have separate code for
    the tf32 split (no scale, fp32 hi / lo, FP32-pipe first layer): the same bit-exact claims hold."""
    monkeypatch.setenv("LNN_PRECISION", precision)
    for xs, ws in [((2, 3, 32, 32), (16, 3, 3, 3)), ((3, 32, 64, 64), (64, 32, 3, 3)), ((2, 16, 12, 12), (24, 16, 3, 3))]:
        test_conv_block_equals_chain(nn_gpu, xs, ws)
    for xs, ws in [((2, 3, 32, 32), (32, 3, 3, 3)), ((2, 64, 32, 32), (128, 64, 3, 3))]:
        test_conv_infer_fused_and_packed(nn_gpu, xs, ws)
