"""The operand split must deliver fp32-level accuracy on every contraction, not just pass the
loose parity tolerance: a dropped hi*lo or lo*hi term (about 5e-4 relative per product) would
still sit inside `1e-3 * sqrt(K)`.  Each result is therefore compared with a float64 reference
and its error bounded by a small multiple of the error an fp32 computation of the same sums
makes; precision 1 (plain TF32) must FAIL that bound, which shows the bound has teeth.
Covers matmul forward / dA / dB and conv forward / dX / dW for both split formats."""
import numpy as np
import pytest

import oracle as o

pytestmark = pytest.mark.gpu


def _err(got, want64):
    return float(np.abs(np.asarray(got, np.float64) - want64).max())


def _matmul_errors(nn, rng):
    m, k, n = 256, 512, 384
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    a64, b64, dy64 = a.astype(np.float64), b.astype(np.float64), dy.astype(np.float64)
    want = {"y": a64 @ b64, "da": dy64 @ b64.T, "db": a64.T @ dy64}
    # the fp32 yardstick: the reference's own sequential-k fp32 GEMM on the same operands
    fp32 = {"y": _err(o.gemm(a, b), want["y"]), "da": _err(o.gemm(dy, b, trans_b=True), want["da"]),
            "db": _err(o.gemm(a, dy, trans_a=True), want["db"])}
    at, bt = nn.Tensor_from_value(a), nn.Tensor_from_value(b)
    y = nn.matmul(at, bt)
    nn.backward({y: dy}, grad_for_non_trainables=True)
    got = {"y": _err(y.np(), want["y"]), "da": _err(at.get_grad().np(), want["da"]),
           "db": _err(bt.get_grad().np(), want["db"])}
    return got, fp32


def _conv_errors(nn, rng, xs, ws, stride):
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    want_y = o.conv2d_fwd(x, w, stride, 1, "same", accum64=True)
    dy = rng.standard_normal(want_y.shape).astype(np.float32)
    want = {"y": want_y.astype(np.float64),
            "dx": o.conv2d_dx(np.zeros_like(x), dy, w, x.shape, stride, 1, "same", accum64=True).astype(np.float64),
            "dw": o.conv2d_dw(np.zeros_like(w), dy, x, stride, 1, "same", accum64=True).astype(np.float64)}
    # the fp32 yardstick: the oracle's sequential fp32 sums of the same products
    fp32 = {"y": _err(o.conv2d_fwd(x, w, stride, 1, "same"), want["y"]),
            "dx": _err(o.conv2d_dx(np.zeros_like(x), dy, w, x.shape, stride, 1, "same"), want["dx"]),
            "dw": _err(o.conv2d_dw(np.zeros_like(w), dy, x, stride, 1, "same"), want["dw"])}
    xt, wt = nn.Tensor_from_value(x), nn.Tensor_from_value(w)
    y = nn.conv2D(xt, wt, stride=stride)
    nn.backward({y: dy}, grad_for_non_trainables=True)
    got = {"y": _err(y.np(), want["y"]), "dx": _err(xt.get_grad().np(), want["dx"]),
           "dw": _err(wt.get_grad().np(), want["dw"])}
    return got, fp32


# The tensor cores add every 32-byte K step into the fp32 accumulator with truncation, so the
# error grows with the number of instructions per product: split TF32 issues twice as many as
# split FP16 and gets twice the allowance.  The accum64 oracle rounds its result to fp32 once:
# that half-ulp is part of every comparison.
def _bound(fp32_err, scale, precision=2):
    return (8.0 if precision == 3 else 4.0) * fp32_err + 2e-7 * scale


@pytest.mark.parametrize("precision", [2, 3])
def test_matmul_split_reaches_fp32_accuracy(nn_gpu, monkeypatch, precision):
    monkeypatch.setenv("LNN_PRECISION", str(precision))
    got, fp32 = _matmul_errors(nn_gpu, np.random.default_rng(5))
    for k in got:
        assert got[k] <= _bound(fp32[k], 100.0, precision), f"{k}: error {got[k]:.3e}, fp32 sums make {fp32[k]:.3e}"
    nn_gpu.devices.check_status()


@pytest.mark.parametrize("precision", [2, 3])
@pytest.mark.parametrize("xs,ws,stride", [((2, 64, 20, 24), (96, 64, 3, 3), 1), ((2, 32, 32, 32), (64, 32, 3, 3), 1),
                                          ((3, 24, 17, 19), (40, 24, 3, 3), 2)])
def test_conv_split_reaches_fp32_accuracy(nn_gpu, monkeypatch, precision, xs, ws, stride):
    monkeypatch.setenv("LNN_PRECISION", str(precision))
    got, fp32 = _conv_errors(nn_gpu, np.random.default_rng(6), xs, ws, stride)
    for k in got:
        assert got[k] <= _bound(fp32[k], 100.0, precision), f"{k}: error {got[k]:.3e}, fp32 sums make {fp32[k]:.3e}"
    nn_gpu.devices.check_status()


def test_single_pass_tf32_fails_the_bound(nn_gpu, monkeypatch):
    """Plain TF32 is ~100x less accurate: if it passed, the bound above would prove nothing."""
    monkeypatch.setenv("LNN_PRECISION", "1")
    got, fp32 = _matmul_errors(nn_gpu, np.random.default_rng(5))
    for k in got:
        assert got[k] > 10.0 * _bound(fp32[k], 100.0, 3), f"{k}: plain TF32 error {got[k]:.3e} is inside the bound"
    got, fp32 = _conv_errors(nn_gpu, np.random.default_rng(6), (2, 64, 20, 24), (96, 64, 3, 3), 1)
    for k in got:
        assert got[k] > 10.0 * _bound(fp32[k], 100.0, 3), f"{k}: plain TF32 error {got[k]:.3e} is inside the bound"


def test_split_fp16_wide_dynamic_range(nn_gpu, monkeypatch):
    """Split FP16 scales each operand by a power of two taken from its largest magnitude, so tiny
    and huge tensors must come out as accurately as O(1) ones, and an outlier must cost the other
    elements no more than the format's absolute error bound."""
    monkeypatch.setenv("LNN_PRECISION", "2")
    nn = nn_gpu
    rng = np.random.default_rng(7)
    a0 = rng.standard_normal((128, 256)).astype(np.float32)
    b0 = rng.standard_normal((256, 192)).astype(np.float32)
    for sa, sb in [(1e-30, 1e10), (3e20, 2e-25), (1e-38, 1.0), (7e17, 3e17)]:
        a, b = (a0 * np.float32(sa)).astype(np.float32), (b0 * np.float32(sb)).astype(np.float32)
        want = a.astype(np.float64) @ b.astype(np.float64)
        got = nn.matmul(nn.Tensor_from_value(a), nn.Tensor_from_value(b)).np()
        scale = float(np.abs(want).max())
        fp32 = _err((a.astype(np.float64) @ b.astype(np.float64)).astype(np.float32), want)
        assert np.isfinite(got).all()
        assert _err(got, want) <= 8e-6 * scale + 4 * fp32, f"scales {sa:g} x {sb:g}: {_err(got, want):.3e} vs {scale:.3e}"
    # one outlier: elements within 2**17 of it keep 22 significant bits, smaller ones an absolute
    # error of 2**-40 of the largest magnitude (the documented bound of the format)
    for big in (4096.0, 2.0 ** 20):
        a = a0.copy()
        a[3, 5] = big
        want = a.astype(np.float64) @ b0.astype(np.float64)
        got = nn.matmul(nn.Tensor_from_value(a), nn.Tensor_from_value(b0)).np()
        rows = np.arange(128) != 3
        fmt = 256 * 2.0 ** -40 * big * float(np.abs(b0).max())
        assert _err(got[rows], want[rows]) <= 4 * _err(o.gemm(a, b0)[rows], want[rows]) + 2e-5 + fmt, big
    # zeros and non-finite inputs: no scale is derived, values pass through
    z = nn.matmul(nn.Tensor_from_value(np.zeros((128, 64), np.float32)), nn.Tensor_from_value(b0[:64])).np()
    assert not z.any()
    a = a0.copy()
    a[0, 0] = np.inf
    got = nn.matmul(nn.Tensor_from_value(a), nn.Tensor_from_value(b0)).np()
    assert not np.isfinite(got[0]).any() and np.isfinite(got[1:]).all()
    nn.devices.check_status()


@pytest.mark.parametrize("spread", [1e-2, 1e-5])
def test_packed_chain_with_a_loose_scale_bound(nn_gpu, monkeypatch, spread):
    """A convolution that hands its result on in the packed format scales it by an upper bound
    of the result, not by the measured maximum.  Weights that cancel (a zero-sum high-pass
    filter on a nearly constant image) make that bound loose by the factor 1 / spread: the second
    convolution of the chain must still come out with the accuracy of the chain that passes fp32
    tensors, because the format has 17 bits of headroom below its largest element."""
    monkeypatch.setenv("LNN_PRECISION", "2")
    nn = nn_gpu
    rng = np.random.default_rng(11)
    n, c, h, w = 2, 32, 32, 32
    x = (1.0 + spread * rng.standard_normal((n, c, h, w))).astype(np.float32)
    w1 = rng.standard_normal((64, c, 3, 3)).astype(np.float32)
    w1 -= w1.mean(axis=(1, 2, 3), keepdims=True)                # every output channel sums to zero
    w1 = w1.astype(np.float32)
    w2 = (rng.standard_normal((64, 64, 3, 3)) * 0.1).astype(np.float32)
    xt, w1t, w2t = nn.Tensor_from_value(x), nn.Tensor_from_value(w1), nn.Tensor_from_value(w2)
    # interior pixels only see the noise: the border (zero padding) sees the constant and is cropped
    y1 = o.conv2d_fwd(x, w1, 1, 1, "same", accum64=True)
    p1 = y1.reshape(n, 64, h // 2, 2, w // 2, 2).max(axis=(3, 5))
    want = o.conv2d_fwd(p1, w2, 1, 1, "same", accum64=True).astype(np.float64)
    packed = nn.conv2D_infer(xt, w1t, pool=True, packed_output=True)
    loose = packed.scale_exponent() - nn.ops.scale_exponent_of(
        int(np.float32(packed.largest_magnitude()).view(np.uint32)))
    assert loose >= 0
    got = nn.conv2D_infer(packed, w2t).np()
    with nn.deferred.disabled():
        chain = nn.conv2D(nn.max_pool2D(nn.conv2D(xt, w1t), 2, 2, "same"), w2t).np()
    scale = float(np.abs(want).max())
    e_packed, e_chain = _err(got, want), _err(chain, want)
    assert e_packed <= 2 * e_chain + 1e-6 * scale, (e_packed, e_chain, scale, loose)
    nn.devices.check_status()
