"""Modules, checkpoints, optimizers and the tape's behaviours, against a checkpoint and update
results produced by the unmodified reference (tests/golden/module_ckpt.pkl, written by
make_golden_modules.py) and following the procedures of its own tests
(litenn/core/test/test.py:42-195)."""
import os
import pickle

import numpy as np
import pytest

import module_cases
from conftest import ROOT, assert_bit_exact

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "module_ckpt.pkl"), "rb") as f:
        return pickle.load(f)


def _assert_state_equal(got, want, exact=True, tol=0.0):
    assert list(got.keys()) == list(want.keys()), "state dict keys (and their order) differ"
    for k, w in want.items():
        g = got[k]
        if isinstance(w, tuple) and w[0] == "np.ndarray":
            assert g[0] == "np.ndarray" and g[1].shape == w[1].shape, k
            if exact:
                assert_bit_exact(g[1], w[1], k)
            else:
                np.testing.assert_allclose(g[1], w[1], rtol=tol, atol=tol, err_msg=k)
        else:
            assert g == w, f"{k}: {g!r} != {w!r}"


def test_tensor_names_follow_the_module_tree(nn_gpu, golden):
    trainer = module_cases.build(nn_gpu)
    assert [t.get_name() for t in trainer.mod1.trainables()] == golden["names"]
    assert trainer.mod1.mod.conv1.kernel.get_name() == "Trainer.mod1.mod.conv1.kernel"
    assert trainer.mod1.mod.list_of_convs[0].kernel.get_name() == "Trainer.mod1.mod.list_of_convs[0].kernel"
    assert trainer.mod1.mod.dict_of_layers["asd"].weight.get_name() == "Trainer.mod1.mod.dict_of_layers[asd].weight"
    assert trainer.mod1.mod.get_name(trainer) == "mod1.mod" and trainer.get_name(trainer) == ""


def test_reference_checkpoint_loads_and_round_trips(nn_gpu, golden, tmp_path):
    nn = nn_gpu
    ref_state = pickle.loads(golden["file_bytes"])
    trainer = module_cases.build(nn)
    module_cases.fill(trainer, seed=99)                 # different contents before loading
    path = tmp_path / "ref.bin"
    path.write_bytes(golden["file_bytes"])
    assert trainer.load(path) is True
    assert trainer.load(tmp_path / "missing.bin") is False
    # every tensor, python variable and optimizer state arrives bit for bit
    assert trainer.mod1.a == 3 and trainer.mod1.mod.l == [1, 9] and trainer.mod1.mod.tag == "second"
    assert trainer.mod1.scale == 0.25 and trainer.mod1.mod.scale == 0.5
    assert trainer.opt1.iteration == 2
    _assert_state_equal(trainer.dump_state(), ref_state)
    # a file written here has the reference's keys, order and entry forms
    out = tmp_path / "ours.bin"
    trainer.save(out)
    _assert_state_equal(pickle.loads(out.read_bytes()), ref_state)
    # sub-module state can be moved on its own (test.py:122-131)
    other = module_cases.build(nn)
    other.opt1.load_state(trainer.opt1.dump_state())
    _assert_state_equal(other.opt1.dump_state(), trainer.opt1.dump_state())


def test_training_continues_from_a_reference_checkpoint(nn_gpu, golden, tmp_path):
    """Load the reference's checkpoint (weights, momentum accumulators, iteration), take the step
    the reference took next, and land on its weights."""
    nn = nn_gpu
    trainer = module_cases.build(nn)
    path = tmp_path / "ref.bin"
    path.write_bytes(golden["file_bytes"])
    trainer.load(path)
    loss = module_cases.train_step(nn, trainer, golden["input"])
    np.testing.assert_allclose(loss, golden["losses"][2], rtol=1e-5, atol=1e-6)
    _assert_state_equal(trainer.dump_state(), golden["after_step3"], exact=False, tol=2e-6)
    nn.devices.check_status()


def test_load_skips_what_does_not_match(nn_gpu, golden):
    nn = nn_gpu
    trainer = module_cases.build(nn)
    module_cases.fill(trainer, seed=5)
    before = trainer.mod1.conv1.kernel.np()
    state = pickle.loads(golden["file_bytes"])
    state["mod1.conv1.kernel"] = ("np.ndarray", np.zeros((1, 2, 3), np.float32))     # wrong shape
    state["mod1.a"] = ("python-var", ("str", "x"))                                  # wrong class
    del state["mod1.conv1.bias"]                                                    # missing
    state["mod1.l__len"] = 5                                                        # wrong length
    bias_before = trainer.mod1.conv1.bias.np()
    trainer.load_state(state)
    assert_bit_exact(trainer.mod1.conv1.kernel.np(), before, "kernel with a wrong stored shape")
    assert_bit_exact(trainer.mod1.conv1.bias.np(), bias_before, "bias without stored data")
    assert trainer.mod1.a == 1 and trainer.mod1.l == [1, 1]
    assert trainer.mod1.mod.l == [1, 9]                                             # the rest still loads


def test_module_assignment_rules(nn_gpu):
    nn = nn_gpu

    class M(nn.Module):
        pass

    m = M()
    with pytest.raises(Exception):
        m.layers = []
    with pytest.raises(Exception):
        m.table = {}
    with pytest.raises(Exception):
        m.s = {1, 2}
    m._scratch = []                                     # underscore names are not managed
    t = nn.Tensor((2, 2))
    m.w = t
    with pytest.raises(Exception):
        M().w = t                                       # already owned by another module
    with pytest.raises(Exception):
        m.v = t + t                                     # produced by an operator
    with pytest.raises(ValueError):
        nn.optimizer.SGD([t, t])
    opt = nn.optimizer.SGD([t])
    with pytest.raises(ValueError):
        nn.optimizer.SGD([t])                           # already trained by another optimizer
    assert opt.get_trainable_tensors() == [t]


@pytest.mark.parametrize("name", list(module_cases.OPTIMIZERS))
def test_optimizer_updates_match_the_reference(nn_gpu, golden, name):
    """SGD (momentum, nesterov), RMSprop and Adam with learning-rate decay, dropout and gradient
    clipping: three steps give the reference's tensors and state bit for bit (one fused kernel
    here, the same roundings in the same order)."""
    got = module_cases.run_optimizer(nn_gpu, name)
    want = golden["optimizers"][name]
    assert list(got.keys()) == list(want.keys())
    for k in want:
        assert_bit_exact(got[k], want[k], f"{name}/{k}")
    nn_gpu.devices.check_status()


def test_freeze_and_stop_grad(nn_gpu):
    """test.py:166-195: a tensor used inside optimizer.freeze() gets no gradient; outside it does,
    and the step changes it.  backward(stop_grad=...) stops the walk at the named tensor."""
    nn = nn_gpu
    inp_t = nn.Tensor((2, 2, 8, 8), init=nn.initializer.Scalar(1.0))
    kernel_t = nn.Tensor((4, 2, 3, 3), init=nn.initializer.Scalar(0.0))
    kernel_2_t = nn.Tensor((4, 2, 3, 3), init=nn.initializer.Scalar(0.0))
    opt = nn.optimizer.RMSprop([inp_t, kernel_t, kernel_2_t])
    opt.zero_grad()
    with nn.optimizer.freeze():
        r = nn.conv2D(inp_t, kernel_2_t)
    r.backward()
    assert not kernel_2_t.has_grad(), "used inside freeze(), must not receive a gradient"
    r = nn.conv2D(inp_t, kernel_t)
    r.backward()
    assert kernel_t.has_grad()
    assert kernel_t.get_grad().np().any()
    opt.step()
    assert kernel_t.np().any(), "the optimisation step must change the kernel"
    assert not kernel_2_t.np().any(), "the frozen kernel must stay as it was"

    x = nn.Tensor((2, 3), init=nn.initializer.Scalar(2.0))
    w = nn.Tensor((3, 4), init=nn.initializer.Scalar(0.5))
    opt2 = nn.optimizer.SGD([x, w])
    opt2.zero_grad()
    h = nn.matmul(x, w)
    y = nn.square(h)
    nn.backward(y, stop_grad=[h])
    assert not x.has_grad() and not w.has_grad(), "stop_grad must cut everything below h"
    opt2.zero_grad()
    y = nn.square(nn.matmul(x, w))
    nn.backward(y)
    assert x.has_grad() and w.has_grad()
    np.testing.assert_allclose(w.get_grad().np(), np.full((3, 4), 2 * 3.0 * 2.0 * 2), rtol=1e-6)
    nn.devices.check_status()


def test_shallow_forward_allocates_nothing(nn_gpu):
    """test.py:147-164: shape inference through shallow_forward touches no device memory."""
    nn = nn_gpu

    class Module1(nn.Module):
        def __init__(self):
            self.conv = nn.Conv2D(1, 1, 3, stride=2)

        def forward(self, x):
            return self.conv(x)

    dev = nn.devices.get_current()[0]
    before = dev.get_used_memory()
    launches = dev.launch_count() if hasattr(dev, "launch_count") else None
    m = Module1()
    m.set_training(True)
    assert m.is_training() and m.conv.is_training()
    out = m.shallow_forward(nn.Tensor((1, 1, 16, 16)))
    assert tuple(out.shape) == (1, 1, 8, 8)
    assert dev.get_used_memory() == before, "memory was allocated in shallow_forward"
    if launches is not None:
        assert dev.launch_count() == launches, "kernels were launched in shallow_forward"


def test_expired_wait_is_reported_by_the_next_read(nn_gpu):
    """A bounded wait that expired leaves a status word on the device; tile kernels launched
    after it return at once.  The next host read (np(), wait()) must raise instead of handing
    out whatever the output buffer held, and must clear the word so that work can continue.
    The word is written from the host here: no kernel waits on anything."""
    nn = nn_gpu
    from litenn_b200 import _lib
    lib = _lib.get_lib()
    dev = nn.devices.get_current()[0]
    a = nn.Tensor_from_value(np.ones((128, 64), np.float32))
    b = nn.Tensor_from_value(np.ones((64, 32), np.float32))
    good = nn.matmul(a, b).np()
    assert (good == 64).all()
    lib.lnn_debug_set_status(dev.index, _lib.E_TIMEOUT, 1, 7, 3)
    y = nn.matmul(a, b)                       # the kernel sees the word and returns at once
    with pytest.raises(_lib.LnnError) as e:
        y.np()
    assert e.value.code == _lib.E_TIMEOUT and "role 1, tile 7, step 3" in str(e.value)
    assert (nn.matmul(a, b).np() == 64).all(), "the status must be cleared by the report"
    lib.lnn_debug_set_status(dev.index, _lib.E_TIMEOUT, 2, 0, 0)
    with pytest.raises(_lib.LnnError):
        nn.devices.wait()
    nn.devices.check_status()


_ALLOC_CHILD = r"""
import ctypes, sys
import numpy as np
import litenn_b200 as nn
from litenn_b200 import _lib
nn.devices.set_current(nn.devices.get_all()[0])
lib = _lib.get_lib()
dev = nn.devices.get_current()[0]
dev._ensure()
mode = sys.argv[1]
def stats():
    a, p = ctypes.c_uint64(), ctypes.c_uint64()
    lib.lnn_mem_stats(dev.index, ctypes.byref(a), ctypes.byref(p))
    return a.value, p.value
def alloc(n):
    p = ctypes.c_uint64()
    lib.lnn_alloc(dev.index, n, ctypes.byref(p))
    return p.value
if mode == "evict":
    # the injected failure hits the first fresh allocation below; the pool then holds two
    # buffers, the largest of which is released before the retry succeeds
    small, big = alloc(1 << 16), alloc(1 << 20)
    lib.lnn_free(dev.index, small, 1 << 16); lib.lnn_free(dev.index, big, 1 << 20)
    a0, p0 = stats()
    fresh = alloc(1 << 18)
    a1, p1 = stats()
    assert fresh and p0 - p1 == (1 << 20) and a1 == a0 - (1 << 20) + (1 << 18), (a0, p0, a1, p1)
    assert alloc(1 << 16) == small, "the smaller pooled buffer must still be there"
    print("EVICT-OK")
else:
    lib.lnn_pool_trim(dev.index)
    try:
        alloc(1 << 18)
    except _lib.LnnError as e:
        assert e.code == _lib.E_NOMEM, e
        print("NOMEM-OK")
"""


@pytest.mark.parametrize("mode", ["evict", "nomem"])
def test_allocation_failure_paths(mode):
    """Evict-largest-and-retry (minicl/CLDevice.py:134-164) and LNN_E_NOMEM, driven by failures
    injected on the host side of cudaMalloc in a child process; the GPU sees nothing unusual."""
    import subprocess
    import sys
    # only buffers taken through lnn_alloc count: two succeed before the failure in 'evict'
    env = dict(os.environ, PYTHONPATH=ROOT, LNN_FAIL_ALLOC_AFTER="2" if mode == "evict" else "0")
    if mode == "evict":
        env["LNN_FAIL_ALLOC_TIMES"] = "1"
    r = subprocess.run([sys.executable, "-c", _ALLOC_CHILD, mode], env=env, capture_output=True, text=True, timeout=300)
    assert ("EVICT-OK" if mode == "evict" else "NOMEM-OK") in r.stdout, f"{r.stdout[-400:]}\n{r.stderr[-1500:]}"


def test_transposed_and_depthwise_conv_modules(nn_gpu):
    """nn.Conv2DTranspose / nn.DepthwiseConv2D: the reference's constructor arguments, kernel shapes
    and saveables (module/Conv2DTranspose.py:22-58, module/DepthwiseConv2D.py:24-56); forward is
    the operator plus a broadcast bias, and both parameters receive gradients."""
    nn = nn_gpu
    rng = np.random.default_rng(51)

    class Net(nn.Module):
        def __init__(self):
            self.up = nn.Conv2DTranspose(4, 8, 3)
            self.dw = nn.DepthwiseConv2D(8, 3, use_bias=True)
            self.plain = nn.DepthwiseConv2D(8, 3, use_bias=False)

        def forward(self, x):
            return self.plain(self.dw(self.up(x)))

    net = Net()
    assert tuple(net.up.kernel.shape) == (8, 4, 3, 3) and tuple(net.up.bias.shape) == (8,)
    assert tuple(net.dw.kernel.shape) == (8, 3, 3) and net.plain.bias is None
    names = sorted(t.get_name() for t in net.trainables())
    assert names == ["Net.dw.bias", "Net.dw.kernel", "Net.plain.kernel", "Net.up.bias", "Net.up.kernel"], names
    net.up.bias.set(rng.uniform(-1, 1, (8,)).astype(np.float32))
    net.dw.bias.set(rng.uniform(-1, 1, (8,)).astype(np.float32))
    x = nn.Tensor_from_value(rng.standard_normal((2, 4, 8, 8)).astype(np.float32))
    up = net.up(x)
    assert tuple(up.shape) == (2, 8, 16, 16)
    want_up = nn.conv2DTranspose(x, net.up.kernel, 2, 1, "same").np() + net.up.bias.np().reshape(1, -1, 1, 1)
    np.testing.assert_array_equal(up.np(), want_up.astype(np.float32))
    y = net.dw(up)
    want_dw = nn.depthwise_conv2D(up, net.dw.kernel, 1, 1, "same").np() + net.dw.bias.np().reshape(1, -1, 1, 1)
    np.testing.assert_array_equal(y.np(), want_dw.astype(np.float32))
    opt = nn.optimizer.SGD(net.trainables(), lr=1e-2)
    before = {t.get_name(): t.np().copy() for t in net.trainables()}
    net(x).mean().backward()
    opt.step()
    for t in net.trainables():
        assert not np.array_equal(t.np(), before[t.get_name()]), f"{t.get_name()} was not updated"
    state = net.dump_state()
    assert any(k.endswith("up.kernel") for k in state) and any(k.endswith("dw.bias") for k in state)
    nn.devices.check_status()
