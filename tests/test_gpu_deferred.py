"""The stock operator chain (nn.Conv2D, nn.leaky_relu, nn.max_pool2D, written as in the
reference's user guide) must give the values of one kernel per operator bit for bit while it runs
through the fused kernels, whatever the user does with the intermediate tensors."""
import numpy as np
import pytest

from conftest import assert_bit_exact, assert_contraction_close

pytestmark = pytest.mark.gpu


def _stock_model(nn, rng, chans=(3, 16, 32, 64), classes=10):
    class Net(nn.Module):
        def __init__(self):
            self.convs = [nn.Conv2D(chans[i], chans[i + 1], 3, fused=False) for i in range(len(chans) - 1)]
            self.dense = nn.Dense(chans[-1], classes)

        def forward(self, x):
            for i, c in enumerate(self.convs):
                x = nn.leaky_relu(c(x), 0.1)
                if i + 1 < len(self.convs):
                    x = nn.max_pool2D(x)
            x = nn.flatten(nn.reduce_mean(x, (2, 3)))
            return self.dense(x)

    net = Net()
    for t in net.trainables():
        t.set((rng.standard_normal(tuple(t.shape)) * 0.2).astype(np.float32))
    return net


def test_stock_chain_equals_eager_chain(nn_gpu):
    nn = nn_gpu
    rng = np.random.default_rng(31)
    net = _stock_model(nn, rng)
    x = nn.Tensor_from_value(rng.uniform(0, 1, (4, 3, 64, 48)).astype(np.float32))
    dev = nn.devices.get_current()[0]
    with nn.deferred.disabled():
        n0 = dev.launch_count()
        want = net(x).np()
        eager_launches = dev.launch_count() - n0
    n0 = dev.launch_count()
    got = net(x).np()
    lazy_launches = dev.launch_count() - n0
    assert_bit_exact(got, want, "stock chain through the fused kernels")
    assert lazy_launches < eager_launches, (lazy_launches, eager_launches)
    nn.devices.check_status()


def test_intermediates_of_a_deferred_chain_stay_usable(nn_gpu):
    nn = nn_gpu
    rng = np.random.default_rng(32)
    x = nn.Tensor_from_value(rng.standard_normal((2, 8, 20, 24)).astype(np.float32))
    w = nn.Tensor_from_value((rng.standard_normal((16, 8, 3, 3)) * 0.1).astype(np.float32))
    b = nn.Tensor_from_value(rng.uniform(-0.1, 0.1, (16,)).astype(np.float32))
    w2 = nn.Tensor_from_value((rng.standard_normal((24, 16, 3, 3)) * 0.1).astype(np.float32))
    with nn.deferred.disabled():
        e_y = nn.conv2D(x, w)
        e_z = e_y + b.reshape((1, -1, 1, 1))
        e_a = nn.leaky_relu(e_z, 0.1)
        e_p = nn.max_pool2D(e_a)
        e_c = nn.conv2D(e_p, w2)
        e_skip = e_a * e_y
        want = {k: v.np() for k, v in dict(y=e_y, z=e_z, a=e_a, p=e_p, c=e_c, skip=e_skip).items()}
    y = nn.conv2D(x, w)
    z = y + b.reshape((1, -1, 1, 1))
    a = nn.leaky_relu(z, 0.1)
    p = nn.max_pool2D(a)
    c = nn.conv2D(p, w2)
    assert nn.deferred.is_deferred(c) and nn.deferred.is_deferred(y)
    # the end of the chain first, then every intermediate, then an operator on two of them
    assert_bit_exact(c.np(), want["c"], "second convolution, fed in the packed format")
    assert_bit_exact(p.np(), want["p"], "pooled block")
    assert_bit_exact(a.np(), want["a"], "activation")
    assert_bit_exact(z.np(), want["z"], "convolution + bias")
    assert_bit_exact(y.np(), want["y"], "convolution")
    assert_bit_exact((a * y).np(), want["skip"], "operator on two intermediates")
    # shapes that no fused epilogue covers still work (odd sizes, pooling other than 2x2)
    x2 = nn.Tensor_from_value(rng.standard_normal((1, 8, 9, 7)).astype(np.float32))
    with nn.deferred.disabled():
        w_odd = nn.max_pool2D(nn.leaky_relu(nn.conv2D(x2, w), 0.2)).np()
        w_p3 = nn.max_pool2D(nn.conv2D(x2, w), 3, 2, "same").np()
        w_avg = nn.avg_pool2D(nn.conv2D(x2, w)).np()
    assert_bit_exact(nn.max_pool2D(nn.leaky_relu(nn.conv2D(x2, w), 0.2)).np(), w_odd, "odd sizes")
    assert_bit_exact(nn.max_pool2D(nn.conv2D(x2, w), 3, 2, "same").np(), w_p3, "3x3 pooling is not absorbed")
    assert_bit_exact(nn.avg_pool2D(nn.conv2D(x2, w)).np(), w_avg, "average pooling is not absorbed")
    nn.devices.check_status()


def test_gradients_through_a_deferred_chain(nn_gpu):
    """Nothing trainable upstream: the chain is deferred.  A gradient asked for anyway
    (grad_for_non_trainables) must equal the eager chain's."""
    nn = nn_gpu
    rng = np.random.default_rng(33)
    xs, ws = (2, 8, 16, 16), (16, 8, 3, 3)
    x_np = rng.standard_normal(xs).astype(np.float32)
    w_np = (rng.standard_normal(ws) * 0.1).astype(np.float32)
    b_np = rng.uniform(-0.1, 0.1, (16,)).astype(np.float32)
    dy = rng.standard_normal((2, 16, 8, 8)).astype(np.float32)

    def run(deferred):
        x, w, b = nn.Tensor_from_value(x_np), nn.Tensor_from_value(w_np), nn.Tensor_from_value(b_np)
        ctx = nn.deferred.disabled() if not deferred else _null()
        with ctx:
            y = nn.max_pool2D(nn.leaky_relu(nn.conv2D(x, w) + b.reshape((1, -1, 1, 1)), 0.1))
            if deferred:
                assert nn.deferred.is_deferred(y)
            out = y.np()
            nn.backward({y: dy}, grad_for_non_trainables=True)
        return out, x.get_grad().np(), w.get_grad().np(), b.get_grad().np()

    want, got = run(False), run(True)
    assert_bit_exact(got[0], want[0], "values")
    k = ws[1] * 9
    assert_contraction_close(got[1], want[1], k, "dX")
    assert_contraction_close(got[2], want[2], 2 * 16 * 16, "dW")
    np.testing.assert_allclose(got[3], want[3], rtol=1e-5, atol=1e-5, err_msg="db")
    nn.devices.check_status()


def test_trainable_weights_take_the_eager_path(nn_gpu):
    nn = nn_gpu
    rng = np.random.default_rng(34)
    x = nn.Tensor_from_value(rng.standard_normal((2, 4, 8, 8)).astype(np.float32))
    w = nn.Tensor_from_value((rng.standard_normal((8, 4, 3, 3)) * 0.1).astype(np.float32))
    opt = nn.optimizer.SGD([w])
    y = nn.conv2D(x, w)
    assert not nn.deferred.is_deferred(y)
    with nn.optimizer.freeze():
        assert nn.deferred.is_deferred(nn.conv2D(x, w)), "inside freeze() no gradient can be asked for"
    loss = nn.leaky_relu(y, 0.1).mean()
    loss.backward()
    assert w.has_grad()
    opt.step()


def test_leaky_relu_with_non_positive_slope_gradient(nn_gpu):
    """The fused epilogue takes leaky_relu' from the sign of the output, which is only valid for
    alpha > 0; alpha <= 0 must run the separate operators and give the reference's gradient."""
    nn = nn_gpu
    rng = np.random.default_rng(35)
    x_np = rng.standard_normal((2, 8, 8, 8)).astype(np.float32)
    w_np = (rng.standard_normal((8, 8, 3, 3)) * 0.2).astype(np.float32)
    dy = rng.standard_normal((2, 8, 8, 8)).astype(np.float32)
    for alpha in (0.0, -0.5):
        x, w = nn.Tensor_from_value(x_np), nn.Tensor_from_value(w_np)
        opt = nn.optimizer.SGD([w])
        y = nn.conv2D(x, w, activation="leaky_relu", alpha=alpha)
        nn.backward({y: dy}, grad_for_non_trainables=True)
        x2, w2 = nn.Tensor_from_value(x_np), nn.Tensor_from_value(w_np)
        opt2 = nn.optimizer.SGD([w2])
        y2 = nn.leaky_relu(nn.conv2D(x2, w2), alpha)
        nn.backward({y2: dy}, grad_for_non_trainables=True)
        assert_bit_exact(y.np(), y2.np(), f"values, alpha {alpha}")
        assert_bit_exact(w.get_grad().np(), w2.get_grad().np(), f"dW, alpha {alpha}")
        assert_bit_exact(x.get_grad().np(), x2.get_grad().np(), f"dX, alpha {alpha}")
        del opt, opt2


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
