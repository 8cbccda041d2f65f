"""GPU: lnn_reduce_noalloc, the reduction entry point for callers that may not allocate device
memory (serving loops, hosts that own the whole GPU heap).  It must give the bits lnn_reduce
gives, on two calls in a row (the static scratch keeps the first call's contents), without the
library's allocation counter moving, and must refuse reductions whose partials exceed the
fixed 1 MiB scratch.  Collected last on purpose: a failure here stops nothing else."""
import ctypes

import numpy as np
import pytest

from conftest import assert_bit_exact

pytestmark = pytest.mark.gpu


def _reduce(lib, fn, dev, op, x_t, out_t, dims, acc=0):
    getattr(lib, fn)(dev, op, out_t._ptr(0), x_t._ptr(0), *dims, acc)


@pytest.mark.parametrize("shape,dims", [
    ((1 << 22,), (1, 1, 1, 1 << 22, 1)),              # one long row split over 65536 threads
    ((3, 300000), (3, 1, 1, 300000, 1)),              # non power of two columns, three rows
    ((50000, 48), (1, 1, 1, 50000, 48)),              # reduce the leading axis: three chained passes
    ((64, 4096), (64, 1, 1, 4096, 1)),                # no split at all: no scratch needed
])
def test_noalloc_matches_pooled_reduce_twice(nn_gpu, shape, dims):
    nn = nn_gpu
    from litenn_b200 import _lib
    lib = _lib.get_lib()
    dev = nn.devices.get_current()[0]
    rng = np.random.default_rng(11)
    outer, r0, mid, r1, inner = dims
    n_out = outer * mid * inner
    for op_name in ("sum", "mean", "max"):
        op = _lib.RED[op_name]
        results = []
        for call in range(2):
            x = nn.Tensor_from_value(rng.uniform(-1, 1, shape).astype(np.float32))
            want_t, got_t = nn.Tensor((n_out,)), nn.Tensor((n_out,))
            want_t.fill(0.0)
            got_t.fill(0.0)
            _reduce(lib, "lnn_reduce", dev.index, op, x, want_t, dims)
            before = dev.get_total_allocated_memory()
            _reduce(lib, "lnn_reduce_noalloc", dev.index, op, x, got_t, dims)
            assert dev.get_total_allocated_memory() == before, "the no-alloc entry point allocated"
            assert_bit_exact(got_t.np(), want_t.np(), f"{op_name} {shape} call {call}")
            results.append(got_t.np())
        assert not np.array_equal(results[0], results[1])   # two different inputs were reduced
    # "+=" convention
    x = nn.Tensor_from_value(rng.uniform(-1, 1, shape).astype(np.float32))
    a, b = nn.Tensor((n_out,)), nn.Tensor((n_out,))
    a.fill(2.5)
    b.fill(2.5)
    _reduce(lib, "lnn_reduce", dev.index, _lib.RED["sum"], x, a, dims, acc=1)
    _reduce(lib, "lnn_reduce_noalloc", dev.index, _lib.RED["sum"], x, b, dims, acc=1)
    assert_bit_exact(b.np(), a.np(), "accumulate")


def test_noalloc_refuses_oversized_scratch(nn_gpu):
    nn = nn_gpu
    from litenn_b200 import _lib
    lib = _lib.get_lib()
    dev = nn.devices.get_current()[0]
    # the planner shrinks the partial count to what the static array holds, but a power-of-two row
    # is split into subtrees of at most 2^9 leaves: 600 rows of 2^19 columns need 600 * 1024
    # partials, more than the 2^18 floats of the static scratch
    rows, cols = 600, 1 << 19
    x = nn.Tensor((rows, cols))
    out = nn.Tensor((rows,))
    with pytest.raises(_lib.LnnError) as ei:
        lib.lnn_reduce_noalloc(dev.index, _lib.RED["sum"], out._ptr(0), x._ptr(0), rows, 1, 1, cols, 1, 0)
    assert ei.value.code == _lib.E_UNSUPPORTED and "static scratch" in str(ei.value)
    nn.devices.check_status()
