"""Writes tests/golden/module_ckpt.pkl: a checkpoint saved by the UNMODIFIED reference
(iperov/litenn) for the scenario of module_cases.py, plus what the reference reports around it.

    python tests/golden/make_golden_modules.py /path/to/litenn/checkout

The reference's Python runs as it is; only its OpenCL binding is replaced by the host-C executor
of cl_on_cpu.py (no OpenCL device exists where this runs).  Contents of the pickle:
    file_bytes    the bytes Trainer.save() wrote (pickle protocol 4 of dump_state())
    names         get_name() of every trainable tensor, in trainables() order
    losses        the loss of each of the three training steps (two before the save, one after)
    after_step3   dump_state() of the trainer after a third step taken after saving
    input         the training input
    optimizers    {case: tensors and state after three steps} for module_cases.OPTIMIZERS
"""
import os
import pickle
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
if len(sys.argv) < 2:
    sys.exit("usage: make_golden_modules.py /path/to/litenn/checkout")
sys.path.insert(0, sys.argv[1])

import cl_on_cpu  # noqa: E402

cl_on_cpu.install()
import litenn as nn  # noqa: E402

import module_cases  # noqa: E402


def main():
    nn.devices.set_current(nn.devices.get_all()[0])
    trainer = module_cases.build(nn)
    module_cases.fill(trainer)
    x = module_cases.train_input()
    losses = [module_cases.train_step(nn, trainer, x) for _ in range(2)]
    trainer.mod1.a = 3
    trainer.mod1.mod.l[1] = 9
    trainer.mod1.mod.tag = "second"
    trainer.mod1.scale = 0.25
    path = os.path.join(tempfile.gettempdir(), "lnn_module_ckpt.bin")
    trainer.save(path)
    with open(path, "rb") as f:
        file_bytes = f.read()
    os.unlink(path)
    names = [t.get_name() for t in trainer.mod1.trainables()]
    losses.append(module_cases.train_step(nn, trainer, x))
    out = {"file_bytes": file_bytes, "names": names, "losses": [np.asarray(v) for v in losses],
           "after_step3": trainer.dump_state(), "input": x,
           "optimizers": {name: module_cases.run_optimizer(nn, name) for name in module_cases.OPTIMIZERS}}
    dst = os.path.join(HERE, "module_ckpt.pkl")
    with open(dst, "wb") as f:
        pickle.dump(out, f, protocol=4)
    state = pickle.loads(file_bytes)
    print(f"wrote {dst} ({os.path.getsize(dst)} bytes); {len(state)} keys in the checkpoint:")
    for k, v in state.items():
        desc = v if not (isinstance(v, tuple) and v[0] == "np.ndarray") else f"ndarray{v[1].shape}"
        print("   ", repr(k), desc)


if __name__ == "__main__":
    main()
