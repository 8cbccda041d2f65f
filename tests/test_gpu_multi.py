"""Two-GPU behaviour, run as child processes so that the session's single-device state is left
alone; skipped on a box with one GPU.  NCCL runs without NVLS (plain ring / tree over NVLink)."""
import os
import subprocess
import sys
import tempfile

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _gpu_count():
    import litenn_b200 as nn
    return len(nn.devices.get_all())


def _run(code, *argv, env=None, timeout=600):
    e = dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    e.update(env or {})
    return subprocess.run([sys.executable, "-c", code, *argv], env=e, capture_output=True, text=True, timeout=timeout)


_SINGLE_PROCESS = r"""
import numpy as np
import litenn_b200 as nn
devs = nn.devices.get_all()[:2]
nn.devices.set_current(devs)
n = len(nn.devices.get_current())
assert n == 2

# a tensor holds one buffer per current device; slicing a value over them and reading it back
v = np.arange(8, dtype=np.float32).reshape(4, 2)
t = nn.Tensor_sliced_from_value(v)
assert t.np_count() == 2 and tuple(t.shape) == (2, 2)
assert (t.np(0) == v[:2]).all() and (t.np(1) == v[2:]).all() and (t.np_combined() == v).all()
assert ((t * 2.0 + 1.0).np_combined() == v * 2 + 1).all(), "every op runs on every device"

# the reference's multi-device check (litenn/core/test/test.py:197-218): a different gradient on
# each device makes the replicas drift apart, unless the step is asked to keep them together
x = nn.Tensor_sliced_from_value(np.arange(0, n, dtype=np.float32).reshape((n,)))
w = nn.Tensor((1,), init=nn.initializer.Scalar(0.0))
w.get_grad().set(x)
nn.optimizer.RMSprop([w], rho=1).step()
assert w.np(0)[0] != w.np(1)[0], "without multi_gpu_step the replicas must differ"
w = nn.Tensor((1,), init=nn.initializer.Scalar(0.0))
w.get_grad().set(x)
nn.optimizer.RMSprop([w], rho=1).step(multi_gpu_step=True)      # creates the communicators itself
assert w.np(0)[0] == w.np(1)[0], "with multi_gpu_step the replicas must be equal"
assert nn.parallel.world_size() == 2

# a small training step, batch sharded over the two devices
rng = np.random.default_rng(0)
class Net(nn.Module):
    def __init__(self):
        self.conv = nn.Conv2D(3, 8, 3)
        self.dense = nn.Dense(8, 5)
    def forward(self, x):
        x = nn.max_pool2D(nn.leaky_relu(self.conv(x), 0.1))
        return self.dense(nn.flatten(nn.reduce_mean(x, (2, 3))))
net = Net()
for p in net.trainables():
    p.set((rng.standard_normal(tuple(p.shape)) * 0.2).astype(np.float32))
opt = nn.optimizer.SGD(net.trainables(), lr=0.1)
xb = nn.Tensor_sliced_from_value(rng.standard_normal((8, 3, 16, 16)).astype(np.float32))
oh = np.zeros((8, 5), np.float32); oh[np.arange(8), rng.integers(0, 5, 8)] = 1
tb = nn.Tensor_sliced_from_value(oh)
for _ in range(2):
    opt.zero_grad()
    loss = nn.categorical_crossentropy(nn.softmax(net(xb)), tb).mean()
    loss.backward()
    opt.step(multi_gpu_step=True)
for p in net.trainables():
    assert (p.np(0) == p.np(1)).all(), p.get_name()
    assert np.isfinite(p.np(0)).all()
nn.devices.check_status()
print("SINGLE-PROCESS-OK")
"""


_RANK = r"""
import os, sys, time
import numpy as np
import litenn_b200 as nn
from litenn_b200 import _lib, parallel
rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
nn.devices.set_current(nn.devices.get_all()[rank])
if rank == 0:
    uid = parallel.new_unique_id()
    with open(path + ".tmp", "wb") as f:
        f.write(uid)
    os.replace(path + ".tmp", path)
else:
    for _ in range(600):
        if os.path.exists(path):
            break
        time.sleep(0.1)
    uid = open(path, "rb").read()
parallel.init_process_rank(world, rank, uid)
lib = _lib.get_lib()
dev = nn.devices.get_current()[0]
# known per-rank buffers against the analytic sum, several sizes in one group
sizes = [1, 1000, 645416]
ts = [nn.Tensor_from_value(np.full((s,), rank + 1, np.float32) * (np.arange(s, dtype=np.float32) % 7 + 1)) for s in sizes]
lib.lnn_nccl_group_start()
for t in ts:
    lib.lnn_nccl_allreduce_sum(dev.index, t._ptr(0), t.shape.size)
lib.lnn_nccl_group_end()
tot = sum(range(1, world + 1))
for s, t in zip(sizes, ts):
    assert (t.np() == tot * (np.arange(s, dtype=np.float32) % 7 + 1)).all(), s
# gradient averaging through the optimizer: different gradients, equal weights afterwards
w = nn.Tensor((4,), init=nn.initializer.Scalar(1.0))
opt = nn.optimizer.SGD([w], lr=0.5)
w.get_grad().set(np.full((4,), float(rank), np.float32))
opt.step(multi_gpu_step=True)
want = 1.0 - 0.5 * (sum(range(world)) / world)
assert np.allclose(w.np(), want), (w.np(), want)
nn.devices.check_status()
print("RANK-OK", rank)
"""


def test_single_process_two_devices():
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run(_SINGLE_PROCESS)
    assert "SINGLE-PROCESS-OK" in r.stdout, f"{r.stdout[-600:]}\n{r.stderr[-2500:]}"


def test_nccl_allreduce_two_ranks():
    if _gpu_count() < 2:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "nccl_id")
        procs = [subprocess.Popen([sys.executable, "-c", _RANK, str(r), "2", path],
                                  env=dict(os.environ, PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0"),
                                  stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
        outs = []
        for p in procs:
            try:
                outs.append(p.communicate(timeout=300))
            except subprocess.TimeoutExpired:
                p.kill()                         # the exact child started above
                outs.append(p.communicate())
        for r, (so, se) in enumerate(outs):
            assert f"RANK-OK {r}" in so, f"rank {r}:\n{so[-400:]}\n{se[-2000:]}"
