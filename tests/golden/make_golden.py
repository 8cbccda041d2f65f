"""Generates the golden fixtures (tests/golden/<family>.npz) by running the UNMODIFIED
reference (iperov/litenn) on the cases of cases.py.  The reference's Python op layer and its
own generated kernel text are used as they are; only the OpenCL binding is replaced by the
host-C executor of cl_on_cpu.py because no OpenCL device exists where this runs.

    python tests/golden/make_golden.py /path/to/litenn/checkout [family ...]

Without family names every fixture is regenerated; with them only the named ones.

The fixtures hold inputs and outputs, so the tests never need the reference.
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/litenn/checkout [family ...]")
REF = sys.argv[1]
ONLY = set(sys.argv[2:])
sys.path.insert(0, REF)

import cl_on_cpu  # noqa: E402

cl_on_cpu.install()
import litenn as nn  # noqa: E402

import cases  # noqa: E402


def main():
    nn.devices.set_current(nn.devices.get_all()[0])
    by_family = {}
    t0 = time.time()
    for name, family, params in cases.all_cases():
        if ONLY and family not in ONLY:
            continue
        inp = cases.make_inputs(name, family, params)
        out = cases.run_case(nn, family, params, inp)
        store = by_family.setdefault(family, {})
        for k, v in inp.items():
            store[f"{name}/in/{k}"] = v
        for k, v in out.items():
            store[f"{name}/out/{k}"] = v
        print(f"{name:28s} {time.time() - t0:7.1f}s", flush=True)
    for family, store in by_family.items():
        path = os.path.join(HERE, f"{family}.npz")
        np.savez_compressed(path, **store)
        print(f"wrote {path} ({os.path.getsize(path) / 1024:.0f} KB, {len(store)} arrays)")


if __name__ == "__main__":
    main()
