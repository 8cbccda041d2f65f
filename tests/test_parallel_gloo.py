"""CPU, two gloo ranks: the host-side logic of the one-process-per-GPU layout -- rendezvous,
shard bounds, hand-over of the 128-byte communicator id, max-over-ranks timing, and the claim
that an all-reduce of gradients with 1/world folded into SGD equals the reference's averaging
of replica weights (litenn/core/optimizer/Optimizer.py:149-153) for plain SGD."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, {root!r}); sys.path.insert(0, os.path.join({root!r}, "oracle"))
    import torch, torch.distributed as td
    import bench, oracle as o
    from litenn_b200 import parallel
    d = bench.Dist()
    assert d.world == 2
    b, e = parallel.shard_bounds(bench.TOTAL_BATCH, d.world, d.rank)
    assert (e - b) == 2048 and b == d.rank * 2048
    uid = bytes(range(128)) if d.rank == 0 else None
    uid = d.bcast_bytes(uid, 128)
    assert uid == bytes(range(128))
    assert d.max(10.0 + d.rank) == 11.0 and d.sum(1.0) == 2.0
    # replicas start from identical weights and see different gradients
    rng = np.random.default_rng(0)
    w0 = rng.standard_normal(1000).astype(np.float32)
    g = np.random.default_rng(1 + d.rank).standard_normal(1000).astype(np.float32)
    # (a) reference: every replica steps on its own gradient, then weights are averaged
    local = o.sgd(w0, g, 1e-3)
    t = torch.from_numpy(local.astype(np.float64)); td.all_reduce(t); avg_w = (t / 2).numpy()
    # (b) here: gradients are summed across ranks, SGD applies lr * g / world
    tg = torch.from_numpy(g.copy()); td.all_reduce(tg)
    mine = o.sgd(w0, tg.numpy(), 1e-3, gscale=0.5)
    assert np.allclose(mine, avg_w, rtol=0, atol=2e-7), np.abs(mine - avg_w).max()
    d.barrier(); d.close()
    print("rank", d.rank, "ok")
""")


def test_two_rank_host_logic(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    procs = []
    for rank in range(2):
        env = dict(os.environ, WORLD_SIZE="2", RANK=str(rank), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT="29611", OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    for rank, p in enumerate(procs):
        out, _ = p.communicate(timeout=240)
        assert p.returncode == 0, f"rank {rank} failed:\\n{out}"
        assert f"rank {rank} ok" in out
