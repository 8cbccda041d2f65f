"""GPU: the full-size configurations, checked through size-independent properties and sampled
float64 references (the oracle needs minutes at these sizes): exact power-of-two linearity of
the contractions, sampled outputs against float64 dot products, and bit-exact numpy float32
emulations of the pooling order, the halving reduction tree and the fused chain."""
import ctypes

import numpy as np
import pytest

from conftest import assert_bit_exact, assert_contraction_close

pytestmark = pytest.mark.gpu


def _tree_reduce(x, op):
    """The reference's ceil-halving tree along the last axis, in float32 (reduce.py:279-293)."""
    x = np.array(x, np.float32)
    n = x.shape[-1]
    while n > 1:
        h = (n + 1) // 2
        lo, hi = x[..., :n - h], x[..., h:n]
        if op == "max":
            x[..., :n - h] = np.maximum(lo, hi)
        else:
            x[..., :n - h] = lo + hi
        n = h
    return x[..., 0]


def test_matmul_4096_and_dense(nn_gpu):
    nn = nn_gpu
    rng = np.random.default_rng(0)
    n = 4096
    a = (rng.standard_normal((n, n)) / 64).astype(np.float32)
    b = (rng.standard_normal((n, n)) / 64).astype(np.float32)
    at, bt = nn.Tensor_from_value(a), nn.Tensor_from_value(b)
    c = nn.matmul(at, bt)
    got = c.np()
    rows = rng.choice(n, 48, replace=False)
    want = a[rows].astype(np.float64) @ b.astype(np.float64)
    assert_contraction_close(got[rows], want, n, "matmul 4096 forward (sampled rows)")
    # scaling an operand by a power of two scales every product and partial sum exactly
    c2 = nn.matmul(nn.Tensor_from_value(a * np.float32(4.0)), bt).np()
    assert_bit_exact(c2, got * np.float32(4.0), "matmul linearity under x4")
    # gradients: dA = dO.B^T, dB = A^T.dO, accumulated into grads pre-filled with 1
    do = np.random.default_rng(1).standard_normal((n, n)).astype(np.float32)
    at.get_grad().fill(1.0)
    bt.get_grad().fill(1.0)
    nn.backward({c: do}, grad_for_non_trainables=True)
    da, db = at.get_grad().np(), bt.get_grad().np()
    want_da = 1.0 + do[rows].astype(np.float64) @ b.astype(np.float64).T
    assert_contraction_close(da[rows], want_da, n, "matmul dA (sampled rows)")
    want_db = 1.0 + a.astype(np.float64).T[rows] @ do.astype(np.float64)
    assert_contraction_close(db[rows], want_db, n, "matmul dB (sampled rows)")
    del at, bt, c
    # Dense batch [8192,1024] -> [1024,4096] with bias
    x = rng.standard_normal((8192, 1024)).astype(np.float32)
    w = (rng.standard_normal((1024, 4096)) / 32).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, (4096,)).astype(np.float32)
    xt, wt, bt2 = nn.Tensor_from_value(x), nn.Tensor_from_value(w), nn.Tensor_from_value(bias)
    yt = nn.dense(xt, wt, bt2)
    y = yt.np()
    rows = rng.choice(8192, 32, replace=False)
    want = x[rows].astype(np.float64) @ w.astype(np.float64) + bias
    assert_contraction_close(y[rows], want, 1024, "Dense forward (sampled rows)")
    # Dense backward at the same size: dX = dY.W^T, dW = X^T.dY, db = sum over the batch, each
    # accumulated into a gradient pre-filled with 1 (module/Dense.py:44-48, op/matmul.py:64-72,
    # op/dual_wise_op.py:110-130)
    dy = np.random.default_rng(1).standard_normal((8192, 4096)).astype(np.float32)
    for t in (xt, wt, bt2):
        t.get_grad().fill(1.0)
    nn.backward({yt: dy}, grad_for_non_trainables=True)
    dx, dw, dbias = xt.get_grad().np(), wt.get_grad().np(), bt2.get_grad().np()
    want_dx = 1.0 + dy[rows].astype(np.float64) @ w.astype(np.float64).T
    assert_contraction_close(dx[rows], want_dx, 4096, "Dense dX (sampled rows)")
    wrows = rng.choice(1024, 32, replace=False)
    want_dw = 1.0 + x.astype(np.float64).T[wrows] @ dy.astype(np.float64)
    assert_contraction_close(dw[wrows], want_dw, 8192, "Dense dW (sampled rows)")
    want_db = 1.0 + dy.astype(np.float64).sum(0)
    np.testing.assert_allclose(dbias, want_db, rtol=1e-5, atol=2e-3, err_msg="Dense db")


CONV_STAGES = [((256, 64, 56, 56), (64, 64, 3, 3), 1, 1), ((256, 128, 56, 56), (256, 128, 3, 3), 2, 1),
               ((256, 256, 28, 28), (1024, 256, 1, 1), 1, 0)]


@pytest.mark.parametrize("xs,ws,stride,pad", CONV_STAGES)
def test_conv_stage(nn_gpu, xs, ws, stride, pad):
    nn = nn_gpu
    rng = np.random.default_rng(3)
    fan = ws[1] * ws[2] * ws[3]
    x = rng.standard_normal(xs).astype(np.float32)
    w = (rng.standard_normal(ws) * np.sqrt(2.0 / fan)).astype(np.float32)
    xt, wt = nn.Tensor_from_value(x), nn.Tensor_from_value(w)
    y = nn.conv2D(xt, wt, stride=stride, padding=pad)
    got = y.np()
    N, OC, OH, OW = got.shape
    KH, KW = ws[2], ws[3]
    xp = np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad))).astype(np.float64)
    w64 = w.astype(np.float64)
    # forward: sampled output pixels, all output channels
    for _ in range(40):
        n, oh, ow = rng.integers(N), rng.integers(OH), rng.integers(OW)
        patch = xp[n, :, oh * stride:oh * stride + KH, ow * stride:ow * stride + KW]
        want = np.tensordot(w64, patch, axes=([1, 2, 3], [0, 1, 2]))
        assert_contraction_close(got[n, :, oh, ow], want, fan, "conv forward sample")
    dy = np.random.default_rng(4).standard_normal(got.shape).astype(np.float32)
    nn.backward({y: dy}, grad_for_non_trainables=True)
    dx, dw = xt.get_grad().np(), wt.get_grad().np()
    dyp = dy.astype(np.float64)
    # dW: a few complete kernel entries (contraction over every output pixel)
    for _ in range(6):
        oc, ic, kh, kw = rng.integers(OC), rng.integers(ws[1]), rng.integers(KH), rng.integers(KW)
        xs_ = xp[:, ic, kh:kh + (OH - 1) * stride + 1:stride, kw:kw + (OW - 1) * stride + 1:stride]
        want = np.sum(dyp[:, oc] * xs_)
        assert_contraction_close(np.array([dw[oc, ic, kh, kw]]), np.array([want]), N * OH * OW, "conv dW sample")
    # dX: sampled input pixels, all input channels
    for _ in range(24):
        n, ih, iw = rng.integers(N), rng.integers(xs[2]), rng.integers(xs[3])
        want = np.zeros(xs[1])
        for kh in range(KH):
            for kw in range(KW):
                ny, nx = ih + pad - kh, iw + pad - kw
                if ny % stride or nx % stride:
                    continue
                oh, ow = ny // stride, nx // stride
                if 0 <= oh < OH and 0 <= ow < OW:
                    want += dyp[n, :, oh, ow] @ w64[:, :, kh, kw]
        assert_contraction_close(dx[n, :, ih, iw], want, OC * KH * KW, "conv dX sample")
    nn.devices.check_status()


def test_pools_full_size(nn_gpu):
    nn = nn_gpu
    x = np.random.default_rng(5).uniform(-1, 1, (256, 128, 112, 112)).astype(np.float32)
    xt = nn.Tensor_from_value(x)
    t00, t01, t10, t11 = x[:, :, 0::2, 0::2], x[:, :, 0::2, 1::2], x[:, :, 1::2, 0::2], x[:, :, 1::2, 1::2]
    assert_bit_exact(nn.max_pool2D(xt).np(), np.maximum(np.maximum(t00, t01), np.maximum(t10, t11)), "max_pool2D")
    avg = (((np.float32(0) + t00) + t01) + t10 + t11) / np.float32(4)     # row-major tap order, then / count
    assert_bit_exact(nn.avg_pool2D(xt).np(), avg, "avg_pool2D")
    # backward of avg: dO / 4 to every tap, added to a gradient pre-filled with 1
    y = nn.avg_pool2D(xt)
    dy = np.random.default_rng(6).standard_normal(y.shape.shape).astype(np.float32)
    xt.get_grad().fill(1.0)
    nn.backward({y: dy}, grad_for_non_trainables=True)
    want = np.float32(1.0) + np.repeat(np.repeat(dy / np.float32(4), 2, axis=2), 2, axis=3)
    assert_bit_exact(xt.get_grad().np(), want, "avg_pool2D backward")
    # backward of max: dO goes to the first maximum of each window in row-major order
    # (op/pool2D.py:181-230)
    xt.get_grad().fill(1.0)
    ym = nn.max_pool2D(xt)
    nn.backward({ym: dy}, grad_for_non_trainables=True)
    m = np.maximum(np.maximum(t00, t01), np.maximum(t10, t11))
    want = np.ones_like(x)
    taken = np.zeros(m.shape, bool)                     # the first tap that equals the maximum takes it
    for (r, c), tap in (((0, 0), t00), ((0, 1), t01), ((1, 0), t10), ((1, 1), t11)):
        hit = (tap == m) & ~taken
        want[:, :, r::2, c::2] += np.where(hit, dy, np.float32(0))
        taken |= hit
    assert_bit_exact(xt.get_grad().np(), want, "max_pool2D backward")


def test_reductions_full_size(nn_gpu):
    nn = nn_gpu
    x = np.random.default_rng(7).uniform(-1, 1, (256, 512, 1024)).astype(np.float32)
    xt = nn.Tensor_from_value(x)
    xa = np.ascontiguousarray(x.transpose(0, 2, 1))          # axis 1 moved last
    assert_bit_exact(nn.reduce_sum(xt, (1,)).np(), _tree_reduce(xa, "sum"), "reduce_sum axis 1")
    assert_bit_exact(nn.reduce_max(xt, (1,)).np(), _tree_reduce(xa, "max"), "reduce_max axis 1")
    assert_bit_exact(nn.reduce_mean(xt, (1,)).np(), _tree_reduce(xa, "sum") / np.float32(512), "reduce_mean axis 1")
    # backward over axis 1, accumulated into a gradient pre-filled with 1 (op/reduce.py:207-216,250-276)
    do = np.random.default_rng(8).standard_normal((256, 1024)).astype(np.float32)
    xt.get_grad().fill(1.0)
    ys = nn.reduce_sum(xt, (1,))
    nn.backward({ys: do}, grad_for_non_trainables=True)
    assert_bit_exact(xt.get_grad().np(), np.float32(1.0) + np.broadcast_to(do[:, None, :], x.shape), "reduce_sum backward")
    xt.get_grad().fill(1.0)
    ym = nn.reduce_max(xt, (1,))
    nn.backward({ym: do}, grad_for_non_trainables=True)
    want = np.ones_like(x)
    first = np.argmax(x, axis=1)                         # ties: the lowest index takes the gradient
    np.add.at(want, (np.arange(256)[:, None], first, np.arange(1024)[None, :]), do)
    assert_bit_exact(xt.get_grad().np(), want, "reduce_max backward")
    del want
    xt.free_grad()
    del xa
    flat = x.reshape(1, -1)
    assert_bit_exact(nn.reduce_sum(xt).np(), _tree_reduce(flat, "sum"), "reduce_sum all axes")
    assert_bit_exact(nn.reduce_max(xt).np(), _tree_reduce(flat, "max"), "reduce_max all axes")
    assert_bit_exact(nn.reduce_mean(xt).np(), _tree_reduce(flat, "sum") / np.float32(flat.size), "reduce_mean all")
    # "(2,3)": invalid on the rank-3 tensor in the reference; run on the [256,512,32,32] view
    with pytest.raises(ValueError):
        nn.reduce_sum(xt, (2, 3))
    x4 = xt.reshape((256, 512, 32, 32))
    assert_bit_exact(nn.reduce_sum(x4, (2, 3)).np(), _tree_reduce(x.reshape(256, 512, 1024), "sum"), "reduce_sum (2,3) view")
    assert_bit_exact(nn.reduce_sum(xt, (1, 2)).np(), _tree_reduce(x.reshape(256, -1), "sum"), "reduce_sum (1,2)")
    # sum is independent of how the rows are grouped: a checksum of checksums
    total = nn.reduce_sum(nn.reduce_sum(xt, (1, 2))).np()[0]
    np.testing.assert_allclose(total, x.astype(np.float64).sum(), rtol=1e-5)


def test_fused_chain_full_size(nn_gpu):
    nn = nn_gpu
    rng = np.random.default_rng(8)
    x = rng.standard_normal((256, 256, 56, 56)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, (1, 256, 1, 1)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, (1, 256, 1, 1)).astype(np.float32)
    t = x * g + b                                  # two float32 roundings, as two reference kernels
    want = t * (t >= 0) + (np.float32(0.1) * t) * (t < 0)
    xt, gt, bt = nn.Tensor_from_value(x), nn.Tensor_from_value(g), nn.Tensor_from_value(b)
    assert_bit_exact(nn.scale_bias_leaky_relu(xt, gt, bt, 0.1).np(), want, "fused chain")
    assert_bit_exact(nn.leaky_relu(xt * gt + bt, 0.1).np(), want, "three-op chain")


def test_cnn_micro_batch_against_oracle(nn_gpu):
    """The benchmark's network at its micro-batch size; a sample of images through the oracle."""
    import bench
    import oracle as o
    nn = nn_gpu
    w = bench.cnn_weights()
    x = np.random.default_rng(9).uniform(0, 1, (bench.MICRO_BATCH,) + bench.IMG).astype(np.float32)
    xt = nn.Tensor_from_value(x)
    logits = bench.make_cnn(nn, w).forward(xt).np()
    idx = [0, 17, 255, 511, bench.MICRO_BATCH - 1]
    want = bench.cnn_forward_oracle(o, w, x[idx])
    np.testing.assert_allclose(logits[idx], want, rtol=2e-4, atol=2e-4)
    # the same network written with the reference's namespace only: same kernels, same values
    stock = bench.make_cnn(nn, w, stock=True).forward(xt).np()
    assert_bit_exact(stock, logits, "stock-namespace model vs the explicit fused entries")
    nn.devices.check_status()
