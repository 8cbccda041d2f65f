"""Batch-sharded data parallelism: replica bookkeeping and the gradient all-reduce.

Two layouts are supported.  (1) One process per GPU (the benchmark's layout): rank and world
size come from the launcher, the NCCL unique id is produced on rank 0 and handed to the
other ranks by the caller's own channel (bench.py uses a torch.distributed gloo group).
(2) One process driving several devices, the reference's layout (litenn/core/minicl/
CLKernel.py:58-62): one communicator per device via ncclCommInitAll and grouped calls.
"""
import ctypes

from . import _lib
from .devices import devices

_state = {"world": 1, "rank": 0, "mode": None}


def world_size():
    return _state["world"]


def rank():
    return _state["rank"]


def shard_bounds(total, nshards, index):
    """[begin, end) of shard `index` when `total` items are split evenly over `nshards`."""
    if total % nshards != 0:
        raise ValueError(f"Unable to evenly slice {total} items over {nshards} replicas.")
    per = total // nshards
    return index * per, (index + 1) * per


def new_unique_id():
    buf = ctypes.create_string_buffer(128)
    _lib.get_lib().lnn_nccl_unique_id(buf)
    return buf.raw


def init_process_rank(world, rank_, unique_id):
    """One process per GPU: join the communicator described by `unique_id` (128 bytes)."""
    devs = devices.get_current()
    if len(devs) != 1:
        raise ValueError("init_process_rank expects exactly one current device per process")
    devs[0]._ensure()
    _lib.get_lib().lnn_nccl_init_rank(devs[0].index, int(world), int(rank_), ctypes.c_char_p(unique_id))
    _state.update(world=int(world), rank=int(rank_), mode="rank")


def init_single_process():
    """One process, all current devices: one communicator per device."""
    devs = devices.get_current()
    for d in devs:
        d._ensure()
    arr = (ctypes.c_int * len(devs))(*[d.index for d in devs])
    _lib.get_lib().lnn_nccl_init_all(arr, len(devs))
    _state.update(world=len(devs), rank=0, mode="all")


def shutdown():
    if _state["mode"] is not None:
        for d in devices.get_current():
            _lib.get_lib().lnn_nccl_destroy(d.index)
    _state.update(world=1, rank=0, mode=None)


def allreduce_grads(tensors):
    """Sum the gradient of every tensor across replicas, in place, on the device stream."""
    if _state["mode"] is None:
        raise RuntimeError("parallel.init_process_rank / init_single_process has not been called")
    lib = _lib.get_lib()
    devs = devices.get_current()
    lib.lnn_nccl_group_start()
    try:
        for t in tensors:
            g = t.get_grad()
            for i, d in enumerate(devs):
                lib.lnn_nccl_allreduce_sum(d.index, g._ptr(i), t.shape.size)
    finally:
        lib.lnn_nccl_group_end()
