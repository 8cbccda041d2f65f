"""Benchmark of the LiteNN op-layer hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--no-ops] [--no-train]

Headline workload (the one quoted at 1/2/4/8 GPUs): inference of the small CNN classifier
(conv3x3 3->32 +leaky_relu, maxpool2; 32->64; 64->128; 128->256 +leaky_relu, global average;
Dense 256->1000), random He-init fp32 weights, input [4096,3,128,128] ~U(0,1) sharded over the
GPUs by batch index (no collective on the data path).  One step = one pass of a rank over its
whole shard, in micro-batches of 1024 images.  `value` times the pass with inputs resident in
HBM; `e2e` times the same pass through the public API from pinned HOST buffers, host->device
copy of the images and device->host copy of the logits inside the timed region.  Timing is
by CUDA events on the stream the kernels run on, max over ranks.

`stock_api` repeats both measurements for the same network written with nothing but the
reference's namespace (nn.Conv2D, nn.leaky_relu, nn.max_pool2D, ...): the library defers each
convolution until its consumer is known, so that chain runs through the same fused kernels.
`e2e.h2d_ceiling_gbs` is a copy-only run of the same uploads (no kernels): what the host side
can deliver to this rank while all ranks upload at once.

With N = 1 the line also carries `ops`: the single-op configurations (matmul / Dense / conv
stages in TFLOP/s, the memory-bound sweep in GB/s, forward and backward) and `train`: one
training step (softmax-CE, SGD lr 1e-3, NCCL gradient all-reduce when N > 1) in images/s.

`--impl reference` times the CPU path on the host cores: the C oracle (oracle/lnn_oracle.c,
a restatement of the reference's kernels, OpenMP over all host threads) on a bounded sample
of the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOTAL_BATCH = 4096
MICRO_BATCH = 1024
NCU_TRAFFIC_RATIO = 750.6 / 805.3     # dram bytes / (operand + output bytes) in an ncu capture of the same kernel on 512 images
IMG = (3, 128, 128)
CHANS = [3, 32, 64, 128, 256]
NCLASS = 1000
FWD_FLOP_PER_IMAGE = (2 * 32 * 27 * 128 * 128 + 2 * 64 * 288 * 64 * 64 + 2 * 128 * 576 * 32 * 32 +
                      2 * 256 * 1152 * 16 * 16 + 2 * 256 * 1000)


# ---------------------------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.lines, self.thread = gpu_index, None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def mark(self):
        return len(self.lines)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()        # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin=0, end=None):
        sm, mx, reasons = [], [], set()
        for line in self.lines[begin:end]:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


class Dist:
    """Rendezvous, barrier and max-over-ranks for one-process-per-GPU runs (gloo, CPU
    tensors): plumbing only -- the data path never goes through it."""

    def __init__(self):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.td = None
        if self.world > 1:
            import torch.distributed as td
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            td.init_process_group("gloo", rank=self.rank, world_size=self.world)
            self.td = td

    def barrier(self):
        if self.td is not None:
            self.td.barrier()

    def max(self, value):
        if self.td is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.MAX)
        return float(t.item())

    def sum(self, value):
        if self.td is None:
            return float(value)
        import torch
        t = torch.tensor([float(value)], dtype=torch.float64)
        self.td.all_reduce(t, op=self.td.ReduceOp.SUM)
        return float(t.item())

    def bcast_bytes(self, data, n):
        if self.td is None:
            return data
        import torch
        t = torch.zeros(n, dtype=torch.uint8)
        if self.rank == 0:
            t = torch.frombuffer(bytearray(data), dtype=torch.uint8).clone()
        self.td.broadcast(t, src=0)
        return bytes(t.numpy().tobytes())

    def close(self):
        if self.td is not None:
            self.td.destroy_process_group()


class DevTimer:
    """CUDA events on the library's stream."""

    def __init__(self, nn, dev):
        from litenn_b200 import _lib
        dev._ensure()
        self.lib, self.dev = _lib.get_lib(), dev.index
        self.e0, self.e1 = ctypes.c_uint64(), ctypes.c_uint64()
        self.lib.lnn_event_create(self.dev, ctypes.byref(self.e0))
        self.lib.lnn_event_create(self.dev, ctypes.byref(self.e1))

    def start(self):
        self.lib.lnn_event_record(self.dev, self.e0.value)

    def stop_ms(self):
        self.lib.lnn_event_record(self.dev, self.e1.value)
        ms = ctypes.c_float()
        self.lib.lnn_event_elapsed_ms(self.dev, self.e0.value, self.e1.value, ctypes.byref(ms))
        return float(ms.value)


# ---------------------------------------------------------------------------------------------
# the CNN
# ---------------------------------------------------------------------------------------------
def cnn_weights(seed=0):
    """He-normal convolution kernels and Dense weight, U(-0.1, 0.1) biases (host arrays)."""
    rng = np.random.default_rng(seed)
    w = {}
    for i in range(4):
        fan = CHANS[i] * 9
        w[f"k{i}"] = (rng.standard_normal((CHANS[i + 1], CHANS[i], 3, 3)) * np.sqrt(2.0 / fan)).astype(np.float32)
        w[f"b{i}"] = rng.uniform(-0.1, 0.1, (CHANS[i + 1],)).astype(np.float32)
    w["dw"] = (rng.standard_normal((256, NCLASS)) * np.sqrt(2.0 / 256)).astype(np.float32)
    w["db"] = rng.uniform(-0.1, 0.1, (NCLASS,)).astype(np.float32)
    return w


def make_cnn(nn, weights, stock=False):
    """The classifier as an nn.Module (tensor names come from the module tree, as the optimizer
    requires).

    stock=False: the library's explicit entries -- conv2D_infer with bias, leaky_relu and the
    max-pool in the convolution's epilogue and the activation between two convolutions kept in
    the tensor-core operand format (inference), conv2D_block (training).
    stock=True: the model as a LiteNN user writes it -- nn.Conv2D modules (conv2D, then + bias),
    nn.leaky_relu, nn.max_pool2D, nn.reduce_mean, nn.flatten, nn.Dense -- nothing that the
    reference's namespace does not have."""

    class CNN(nn.Module):
        def __init__(self):
            self._training_path = False
            self._packed = os.environ.get("LNN_BENCH_PACKED", "1") != "0"
            self._block = os.environ.get("LNN_BENCH_BLOCK", "1") != "0"
            self.convs = [nn.Conv2D(CHANS[i], CHANS[i + 1], 3, padding="same",
                                    kernel_initializer=nn.initializer.NumpyArray(weights[f"k{i}"]),
                                    bias_initializer=nn.initializer.NumpyArray(weights[f"b{i}"])) for i in range(4)]
            self.dense = nn.Dense(256, NCLASS, weight_initializer=nn.initializer.NumpyArray(weights["dw"]),
                                  bias_initializer=nn.initializer.NumpyArray(weights["db"]))

        def forward(self, x):
            for i, c in enumerate(self.convs):
                if not self._training_path:
                    x = nn.conv2D_infer(x, c.kernel, 1, 1, "same", bias_t=c.bias, activation="leaky_relu", alpha=0.1,
                                        pool=i < 3, packed_output=(i < 3 and self._packed))
                    continue
                if i < 3 and self._block:
                    # trainable fused block: same values and gradients as conv2D -> leaky_relu -> max_pool2D
                    x = nn.conv2D_block(x, c.kernel, 1, 1, "same", bias_t=c.bias, activation="leaky_relu", alpha=0.1)
                else:
                    x = nn.conv2D(x, c.kernel, 1, 1, "same", bias_t=c.bias, activation="leaky_relu", alpha=0.1)
                    if i < 3:
                        x = nn.max_pool2D(x, 2, 2, "same")
            x = nn.flatten(nn.reduce_mean(x, (2, 3)))
            return self.dense(x)

        def loss(self, logits, onehot):
            return nn.categorical_crossentropy(nn.softmax(logits), onehot).mean()

    class StockCNN(nn.Module):
        def __init__(self):
            self.conv1 = nn.Conv2D(3, 32, 3, kernel_initializer=nn.initializer.NumpyArray(weights["k0"]),
                                   bias_initializer=nn.initializer.NumpyArray(weights["b0"]))
            self.conv2 = nn.Conv2D(32, 64, 3, kernel_initializer=nn.initializer.NumpyArray(weights["k1"]),
                                   bias_initializer=nn.initializer.NumpyArray(weights["b1"]))
            self.conv3 = nn.Conv2D(64, 128, 3, kernel_initializer=nn.initializer.NumpyArray(weights["k2"]),
                                   bias_initializer=nn.initializer.NumpyArray(weights["b2"]))
            self.conv4 = nn.Conv2D(128, 256, 3, kernel_initializer=nn.initializer.NumpyArray(weights["k3"]),
                                   bias_initializer=nn.initializer.NumpyArray(weights["b3"]))
            self.dense = nn.Dense(256, NCLASS, weight_initializer=nn.initializer.NumpyArray(weights["dw"]),
                                  bias_initializer=nn.initializer.NumpyArray(weights["db"]))

        def forward(self, x):
            x = nn.max_pool2D(nn.leaky_relu(self.conv1(x), 0.1))
            x = nn.max_pool2D(nn.leaky_relu(self.conv2(x), 0.1))
            x = nn.max_pool2D(nn.leaky_relu(self.conv3(x), 0.1))
            x = nn.leaky_relu(self.conv4(x), 0.1)
            x = nn.flatten(nn.reduce_mean(x, (2, 3)))
            return self.dense(x)

        def loss(self, logits, onehot):
            return nn.categorical_crossentropy(nn.softmax(logits), onehot).mean()

    return StockCNN() if stock else CNN()


def cnn_forward_oracle(o, w, x):
    """The same network on the CPU oracle (one rounding per reference operator)."""
    for i in range(4):
        x = o.conv2d_fwd(x, w[f"k{i}"], 1, 1, "same", bias=w[f"b{i}"], act=1, alpha=0.1)
        if i < 3:
            x = o.pool2d_fwd("max", x, 2, 2, "same")
    x = o.reduce("mean", x, (2, 3))
    return o.gemm(x, w["dw"], bias=w["db"])


# ---------------------------------------------------------------------------------------------
# reference arm: the CPU path
# ---------------------------------------------------------------------------------------------
def cpu_cnn_images_per_s(target_seconds, seed=1):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as o
    o.build()
    cores = len(os.sched_getaffinity(0))
    cores = o.set_threads(cores)          # torchrun exports OMP_NUM_THREADS=1
    w = cnn_weights()
    rng = np.random.default_rng(seed)
    n = 2
    x = rng.uniform(0, 1, (n,) + IMG).astype(np.float32)
    t0 = time.perf_counter()
    cnn_forward_oracle(o, w, x)
    per_img = (time.perf_counter() - t0) / n
    n = int(max(2, min(256, target_seconds / max(per_img, 1e-6))))
    x = rng.uniform(0, 1, (n,) + IMG).astype(np.float32)
    t0 = time.perf_counter()
    cnn_forward_oracle(o, w, x)
    dt = time.perf_counter() - t0
    return n / dt, cores, f"{n} of {TOTAL_BATCH} images, forward pass, C oracle with OpenMP on {cores} threads", dt


def cpu_single_ops():
    """The reference's CPU path on configurations 1 and 2 at full size (one run each): the C
    oracle's sequential-k GEMM and direct convolution with OpenMP over all host threads."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as o
    o.build()
    cores = o.set_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(0)
    out = {}
    x = rng.standard_normal((8, 16, 32, 32)).astype(np.float32)
    w = (rng.standard_normal((32, 16, 3, 3)) * np.sqrt(2.0 / 144)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, (32,)).astype(np.float32)
    o.conv2d_fwd(x, w, 1, 1, "same", bias=b)
    t0 = time.perf_counter()
    for _ in range(5):
        o.conv2d_fwd(x, w, 1, 1, "same", bias=b)
    dt = (time.perf_counter() - t0) / 5
    out["conv_config1_8x16x32x32_k3_fwd"] = {"ms": round(dt * 1e3, 3), "gflops": round(75497472 / dt / 1e9, 2)}
    a = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    bm = (rng.standard_normal((4096, 4096)) / 64).astype(np.float32)
    t0 = time.perf_counter()
    o.gemm(a, bm)
    dt = time.perf_counter() - t0
    out["matmul_4096_fwd"] = {"ms": round(dt * 1e3, 1), "gflops": round(2.0 * 4096 ** 3 / dt / 1e9, 2)}
    xd = rng.standard_normal((8192, 1024)).astype(np.float32)
    wd = (rng.standard_normal((1024, 4096)) / 32).astype(np.float32)
    bd = rng.uniform(-0.1, 0.1, (4096,)).astype(np.float32)
    t0 = time.perf_counter()
    o.gemm(xd, wd, bias=bd)
    dt = time.perf_counter() - t0
    out["dense_8192x1024x4096_fwd"] = {"ms": round(dt * 1e3, 1), "gflops": round(2.0 * 8192 * 1024 * 4096 / dt / 1e9, 2)}
    return {"cores": cores, "kind": "port", "what": "C oracle (the reference's kernels restated), OpenMP, one full-size run each",
            "ops": out}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, sample, cores, t_total = [], "", 1, 0.0
    per_step = max(2.0, min(20.0, 90.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, cores, sample, dt = cpu_cnn_images_per_s(per_step)
        if i >= args.warmup:
            vals.append(v)
            t_total += dt
    value = float(np.mean(vals))
    line = {"impl": "reference", "metric": "cnn_inference_images_per_s", "value": value, "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * t_total / max(1, args.steps),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "small CNN classifier inference, fp32, input [4096,3,128,128] ~U(0,1), batch sharded over the GPUs",
            "global_batch": TOTAL_BATCH, "micro_batch": MICRO_BATCH, "parallelism": f"dp{n_gpus}",
            "precision": {1: "tf32", 2: "split fp16 (hi*hi + hi*lo + lo*hi, kind::f16)", 3: "split tf32"}[int(os.environ.get("LNN_PRECISION", "2"))],
            "l2": "every micro-batch streams > 2 GB of activations through HBM, far beyond the 126 MB L2; no explicit flush"}


# ---------------------------------------------------------------------------------------------
# single-op configurations (N = 1)
# ---------------------------------------------------------------------------------------------
def _time_calls(timer, nn, fn, warmup, iters):
    for _ in range(warmup):
        fn()
    nn.devices.wait()
    timer.start()
    for _ in range(iters):
        fn()
    ms = timer.stop_ms()
    return ms / iters


def op_cases(nn, dev, lib, passes):
    """(name, setup) pairs of the single-op configurations; setup() allocates the operands and
    returns (callable, flop or None, bytes or None, note or None)."""
    rng = np.random.default_rng(0)

    def T(a):
        return nn.Tensor_from_value(a)

    def gemm(o_t, a_t, b_t, bias, m, n_, k, ta, tb, acc):
        lib.lnn_gemm_f32(dev.index, o_t._ptr(0), a_t._ptr(0), b_t._ptr(0), bias, 1, m, n_, k, ta, tb, acc, passes)

    cases = []
    n = 4096

    def mm(kind):
        def setup():
            a = T(rng.standard_normal((n, n)).astype(np.float32) / 64)
            b = T(rng.standard_normal((n, n)).astype(np.float32) / 64)
            do = T(np.random.default_rng(1).standard_normal((n, n)).astype(np.float32))
            c = nn.Tensor((n, n))
            fn = {"fwd": lambda: gemm(c, a, b, 0, n, n, n, 0, 0, 0),
                  "dA": lambda: gemm(c, do, b, 0, n, n, n, 0, 1, 1),
                  "dB": lambda: gemm(c, a, do, 0, n, n, n, 1, 0, 1)}[kind]
            return fn, 2.0 * n ** 3, None, None
        return setup

    for kind in ("fwd", "dA", "dB"):
        cases.append((f"matmul_4096_{kind}", mm(kind)))

    def dense_setup():
        x = T(rng.standard_normal((8192, 1024)).astype(np.float32))
        w = T(rng.standard_normal((1024, 4096)).astype(np.float32) / 32)
        bias = T(rng.uniform(-0.1, 0.1, (4096,)).astype(np.float32))
        y = nn.Tensor((8192, 4096))
        return (lambda: gemm(y, x, w, bias._ptr(0), 8192, 4096, 1024, 0, 0, 0)), 2.0 * 8192 * 1024 * 4096, None, None

    cases.append(("dense_8192x1024x4096_fwd", dense_setup))

    def dense_bwd(kind):
        def setup():
            x = T(rng.standard_normal((8192, 1024)).astype(np.float32))
            w = T(rng.standard_normal((1024, 4096)).astype(np.float32) / 32)
            dy = T(np.random.default_rng(1).standard_normal((8192, 4096)).astype(np.float32))
            if kind == "dX":      # dX += dY . W^T
                dx = nn.Tensor((8192, 1024))
                return (lambda: gemm(dx, dy, w, 0, 8192, 1024, 4096, 0, 1, 1)), 2.0 * 8192 * 1024 * 4096, None, None
            if kind == "dW":      # dW += X^T . dY
                dw = nn.Tensor((1024, 4096))
                return (lambda: gemm(dw, x, dy, 0, 1024, 4096, 8192, 1, 0, 1)), 2.0 * 8192 * 1024 * 4096, None, None
            db = nn.Tensor((4096,))   # db += reduce_sum(dY, 0)
            return (lambda: nn.ops.reduce_sum_op(dy, 0, output_t=db, is_add_to_output=True)), None, 8192 * 4096 * 4, None
        return setup

    for kind in ("dX", "dW", "db"):
        cases.append((f"dense_8192x1024x4096_{kind}", dense_bwd(kind)))

    def tape_bwd(forward, shape, nbytes, note, lo=-1.0, hi=1.0, extra=()):
        """Backward of a single operator: its grad functions, called as backward() calls them
        (gradients are accumulated, "+=", into a gradient tensor that already exists)."""
        def setup():
            x = T(rng.uniform(lo, hi, shape).astype(np.float32))
            others = [T(a) for a in extra]
            y = forward(x, *others)
            y._ptr(0)
            dy = T(np.random.default_rng(2).standard_normal(tuple(y.shape)).astype(np.float32))
            fns = [f for inp, fl in y._get_gradfns().items() if inp is x for f in fl]
            x.get_grad()._ptr(0)
            keep = (x, y, dy, others)
            return (lambda: [f(y, dy) for f in fns] and keep and None), None, nbytes, note
        return setup

    convs = [("conv3a_256x64x56x56_k3s1", (256, 64, 56, 56), (64, 64, 3, 3), 1, 1),
             ("conv3b_256x128x56x56_k3s2", (256, 128, 56, 56), (256, 128, 3, 3), 2, 1),
             ("conv3c_256x256x28x28_k1", (256, 256, 28, 28), (1024, 256, 1, 1), 1, 0),
             ("conv_config1_8x16x32x32_k3", (8, 16, 32, 32), (32, 16, 3, 3), 1, 1)]

    def conv(xs, ws, stride, pad, kind):
        def setup():
            fan = ws[1] * ws[2] * ws[3]
            xt = T(rng.standard_normal(xs).astype(np.float32))
            wt = T((rng.standard_normal(ws) * np.sqrt(2.0 / fan)).astype(np.float32))
            g, oshape = nn.ops._conv_geom(xt.shape, wt.shape, stride, 1, pad)
            flop = 2.0 * oshape.size * fan
            if kind == "fwd":
                yt = nn.Tensor(oshape)
                return (lambda: lib.lnn_conv2d_fwd(dev.index, ctypes.byref(g), yt._ptr(0), xt._ptr(0), wt._ptr(0), 0, 0, 0.0, 0, passes)), flop, None, None
            dyt = T(np.random.default_rng(2).standard_normal(oshape.shape).astype(np.float32))
            if kind == "dX":
                dxt = nn.Tensor(xs)
                return (lambda: lib.lnn_conv2d_dx(dev.index, ctypes.byref(g), dxt._ptr(0), dyt._ptr(0), wt._ptr(0), passes)), flop, None, None
            dwt = nn.Tensor(ws)
            return (lambda: lib.lnn_conv2d_dw(dev.index, ctypes.byref(g), dwt._ptr(0), dyt._ptr(0), xt._ptr(0), passes)), flop, None, None
        return setup

    for name, xs, ws, stride, pad in convs:
        for kind in ("fwd", "dX", "dW"):
            cases.append((f"{name}_{kind}", conv(xs, ws, stride, pad, kind)))

    pool_bytes = (256 * 128 * 112 * 112 + 256 * 128 * 56 * 56) * 4

    def pool(fn_name):
        def setup():
            xp = T(rng.uniform(-1, 1, (256, 128, 112, 112)).astype(np.float32))
            fn = getattr(nn, fn_name)
            return (lambda: fn(xp)), None, pool_bytes, None
        return setup

    cases.append(("max_pool2D_256x128x112x112", pool("max_pool2D")))
    cases.append(("avg_pool2D_256x128x112x112", pool("avg_pool2D")))
    pin, pout = 256 * 128 * 112 * 112 * 4, 256 * 128 * 56 * 56 * 4
    cases.append(("max_pool2D_256x128x112x112_bwd", tape_bwd(lambda x: nn.max_pool2D(x), (256, 128, 112, 112), 3 * pin + 2 * pout,
                                                             "dI += dO at the first maximum of each window: reads I, O, dO, dI; writes dI")))
    cases.append(("avg_pool2D_256x128x112x112_bwd", tape_bwd(lambda x: nn.avg_pool2D(x), (256, 128, 112, 112), 2 * pin + pout,
                                                             "dI += dO / count: reads dO, dI; writes dI")))

    rb = 256 * 512 * 1024 * 4

    def red(opname, mode):
        def setup():
            xr = T(rng.uniform(-1, 1, (256, 512, 1024)).astype(np.float32))
            fn = getattr(nn, "reduce_" + opname)
            if mode == "axis1":
                return (lambda: fn(xr, (1,))), None, rb + 256 * 1024 * 4, None
            if mode == "all":
                return (lambda: fn(xr)), None, rb, None
            x4 = xr.reshape((256, 512, 32, 32))
            return (lambda: fn(x4, (2, 3))), None, rb + 256 * 512 * 4, \
                "axes (2,3) of the [256,512,32,32] view: (2,3) is invalid on the rank-3 tensor in the reference"
        return setup

    for opname in ("sum", "mean", "max"):
        cases.append((f"reduce_{opname}_axis1", red(opname, "axis1")))
        cases.append((f"reduce_{opname}_all", red(opname, "all")))
        cases.append((f"reduce_{opname}_axes23_view", red(opname, "view")))

    cases.append(("reduce_sum_axis1_bwd", tape_bwd(lambda x: nn.reduce_sum(x, (1,)), (256, 512, 1024), 2 * rb + 256 * 1024 * 4,
                                                   "dI += broadcast(dO): reads dO, dI; writes dI")))
    cases.append(("reduce_max_axis1_bwd", tape_bwd(lambda x: nn.reduce_max(x, (1,)), (256, 512, 1024), 3 * rb + 2 * 256 * 1024 * 4,
                                                   "dI += dO at the maximum: reads I, O, dO, dI; writes dI")))
    cb = 2 * 256 * 256 * 56 * 56 * 4

    def chain(fused):
        def setup():
            xc = T(rng.standard_normal((256, 256, 56, 56)).astype(np.float32))
            gc = T(rng.uniform(0.5, 1.5, (1, 256, 1, 1)).astype(np.float32))
            bc = T(rng.uniform(-0.5, 0.5, (1, 256, 1, 1)).astype(np.float32))
            if fused:
                yc = nn.Tensor(xc.shape)
                return (lambda: nn.scale_bias_leaky_relu(xc, gc, bc, 0.1, output_t=yc)), None, cb, None
            return (lambda: nn.leaky_relu(xc * gc + bc, 0.1)), None, cb, \
                "the reference's three kernels; GB/s counts algorithmic bytes (x in, y out) only"
        return setup

    cases.append(("chain_lrelu_xg_b_fused", chain(True)))
    cases.append(("chain_lrelu_xg_b_3ops", chain(False)))

    def chain_bwd():
        xc = T(rng.standard_normal((256, 256, 56, 56)).astype(np.float32))
        gc = T(rng.uniform(0.5, 1.5, (1, 256, 1, 1)).astype(np.float32))
        bc = T(rng.uniform(-0.5, 0.5, (1, 256, 1, 1)).astype(np.float32))
        dy = T(np.random.default_rng(2).standard_normal((256, 256, 56, 56)).astype(np.float32))
        xc.get_grad()._ptr(0)

        def run():
            y = nn.leaky_relu(xc * gc + bc, 0.1)
            nn.backward({y: dy}, grad_for_non_trainables=True)
        return run, None, 2 * cb, "forward and backward of the three-operator chain through the tape (dx, dg, db); GB/s " \
                                  "counts x, y, dy, dx once each"

    cases.append(("chain_lrelu_xg_b_3ops_fwd_bwd", chain_bwd))
    return cases


def bench_ops(nn, dev, peaks, quick, only=None):
    from litenn_b200 import _lib
    lib = _lib.get_lib()
    timer = DevTimer(nn, dev)
    passes = _lib.precision()
    out = {}
    iters = 3 if quick else 10
    tf32_peak = peaks["bf16_tflops"] / 2.0
    for name, setup in op_cases(nn, dev, lib, passes):
        if only and not any(o in name for o in only.split(",")):
            continue
        fn, flop, nbytes, note = setup()
        ms = _time_calls(timer, nn, fn, 3, iters)
        e = {"ms": round(ms, 4)}
        if flop is not None:
            e["tflops"] = round(flop / ms / 1e9, 2)
            e["frac_of_tf32_peak"] = round(e["tflops"] / tf32_peak, 4)
            e["tensor_pipe_frac"] = round(passes * e["tflops"] / tf32_peak, 4)
        if nbytes is not None:
            e["gbs"] = round(nbytes / ms / 1e6, 1)
            e["frac_of_hbm"] = round(e["gbs"] / peaks["hbm_gbs"], 4)
        if note:
            e["note"] = note
        out[name] = e
        del fn
    nn.devices.check_status()
    return out


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
def run_ours(args):
    dist = Dist()
    world, rank = dist.world, dist.rank
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    import litenn_b200 as nn
    from litenn_b200 import _lib, parallel
    devs = nn.devices.get_all()
    if not devs:
        raise SystemExit("no CUDA device: this benchmark has no CPU fallback")
    dev = devs[dist.local_rank % len(devs)]
    nn.devices.set_current(dev)
    lib = _lib.get_lib()
    peaks = load_peaks()
    passes = _lib.precision()

    local_batch = TOTAL_BATCH // world
    mb = min(MICRO_BATCH, local_batch)
    n_mb = local_batch // mb
    begin, end = parallel.shard_bounds(TOTAL_BATCH, world, rank)
    weights = cnn_weights()
    model = make_cnn(nn, weights)
    stock_model = make_cnn(nn, weights, stock=True)

    # synthetic input shard in PINNED host memory + resident device copies
    img_elems = int(np.prod(IMG))
    host_ptr = ctypes.c_void_p()
    lib.lnn_host_alloc(local_batch * img_elems * 4, ctypes.byref(host_ptr))
    host_x = np.ctypeslib.as_array(ctypes.cast(host_ptr, ctypes.POINTER(ctypes.c_float)), shape=(local_batch,) + IMG)
    rng = np.random.default_rng(1000 + rank)
    for i in range(0, local_batch, 256):
        host_x[i:i + 256] = rng.uniform(0, 1, (min(256, local_batch - i),) + IMG).astype(np.float32)
    host_out_ptr = ctypes.c_void_p()
    lib.lnn_host_alloc(local_batch * NCLASS * 4, ctypes.byref(host_out_ptr))
    resident = []
    for j in range(n_mb):
        t = nn.Tensor((mb,) + IMG)
        lib.lnn_h2d(dev.index, t._ptr(0), host_ptr.value + j * mb * img_elems * 4, mb * img_elems * 4)
        resident.append(t)

    def step_resident(m=None):
        m = m or model
        last = None
        for t in resident:
            last = m.forward(t)
        return last

    stages = [nn.Tensor((mb,) + IMG), nn.Tensor((mb,) + IMG)]
    for st in stages:
        st._ptr(0)
    done_ev = [ctypes.c_uint64(), ctypes.c_uint64()]
    for ev in done_ev:
        lib.lnn_event_create(dev.index, ctypes.byref(ev))
        lib.lnn_event_record(dev.index, ev.value)

    e2e_state = {"slot": 0, "primed": False}
    in_flight = []

    def upload(j, slot):
        mb_bytes = mb * img_elems * 4
        lib.lnn_h2d_prefetch(dev.index, stages[slot]._ptr(0), host_ptr.value + j * mb_bytes, mb_bytes, done_ev[slot].value)

    def step_e2e(more_steps_follow, m=None):
        """Host images in, logits out.  Every micro-batch of the step is uploaded from pinned host
        memory on the copy stream while the previous one computes; the step's first upload overlaps
        the tail of the previous step (a serving loop with two staging buffers), and is exposed
        only for the very first step."""
        if not e2e_state["primed"]:
            upload(0, e2e_state["slot"])
        for j in range(n_mb):
            slot = e2e_state["slot"]
            lib.lnn_wait_prefetch(dev.index)
            if j + 1 < n_mb:
                upload(j + 1, slot ^ 1)
            elif more_steps_follow:
                upload(0, slot ^ 1)               # first micro-batch of the next step
            logits = (m or model).forward(stages[slot])
            logits._ptr(0)                            # a deferred chain is launched here
            lib.lnn_event_record(dev.index, done_ev[slot].value)
            # the logits travel to pinned host memory on the read-back stream while the next
            # micro-batch computes; the tensors stay alive until the copies have finished
            lib.lnn_d2h_readback(dev.index, host_out_ptr.value + j * mb * NCLASS * 4, logits._ptr(0), mb * NCLASS * 4)
            in_flight.append(logits)
            e2e_state["slot"] = slot ^ 1
        e2e_state["primed"] = more_steps_follow
        lib.lnn_wait_readback(dev.index)          # the step's logits are in host memory
        del in_flight[:]

    sampler = ClockSampler(dev.index)
    sampler.start()
    timer = DevTimer(nn, dev)

    def timed_blocks(step_fn, steps):
        """The K-step block, repeated until 0.5 s have been timed (at most 40 blocks); every rank
        times its own blocks with CUDA events between barriers.  Returns the per-block maxima over
        the ranks."""
        blocks = []
        total = 0.0
        while True:
            nn.devices.wait()
            dist.barrier()
            timer.start()
            step_fn(steps)
            ms_b = timer.stop_ms()
            nn.devices.wait()
            dist.barrier()
            ms_b = dist.max(ms_b)
            blocks.append(ms_b)
            total += ms_b
            if total >= 500.0 or len(blocks) >= 40:
                return blocks

    def resident_block(m):
        def run(steps):
            for _ in range(steps):
                out = step_resident(m)
                out._ptr(0)                           # a deferred chain is launched here
        return run

    def e2e_block(m):
        def run(steps):
            for i in range(steps):
                step_e2e(i + 1 < steps, m)
        return run

    # ---- value: inputs resident in HBM --------------------------------------------------------
    resident_block(model)(args.warmup)
    nn.devices.wait()
    dist.barrier()
    launches0 = dev.launch_count()
    m0 = sampler.mark()
    blocks = timed_blocks(resident_block(model), args.steps)
    m1 = sampler.mark()
    launches = (dev.launch_count() - launches0) // len(blocks)
    ms_max = float(np.median(blocks))
    value = TOTAL_BATCH * args.steps / (ms_max / 1000.0)

    # ---- e2e: host buffers in, logits out -----------------------------------------------------
    e2e_block(model)(max(1, args.warmup // 2))
    e_blocks = timed_blocks(e2e_block(model), args.steps)
    ms_e_max = float(np.median(e_blocks))
    e2e_value = TOTAL_BATCH * args.steps / (ms_e_max / 1000.0)

    # ---- the same two measurements on the model written with the reference's namespace only -----
    resident_block(stock_model)(args.warmup)
    s_blocks = timed_blocks(resident_block(stock_model), args.steps)
    e2e_block(stock_model)(max(1, args.warmup // 2))
    se_blocks = timed_blocks(e2e_block(stock_model), args.steps)
    stock = {"value": round(TOTAL_BATCH * args.steps / (float(np.median(s_blocks)) / 1000.0), 1),
             "e2e": round(TOTAL_BATCH * args.steps / (float(np.median(se_blocks)) / 1000.0), 1), "unit": "images/s",
             "what": "the same network built from nn.Conv2D / nn.leaky_relu / nn.max_pool2D / nn.reduce_mean / "
                     "nn.flatten / nn.Dense only; value = inputs resident, e2e = host buffers in, logits out"}

    # ---- copy-only ceiling of the uploads: same pinned buffers, same calls, all ranks at once ----
    def copy_block(steps):
        for _ in range(steps):
            for j in range(n_mb):
                slot = j & 1
                lib.lnn_event_record(dev.index, done_ev[slot].value)
                upload(j, slot)
                lib.lnn_wait_prefetch(dev.index)
    copy_block(1)
    c_blocks = timed_blocks(copy_block, args.steps)
    copy_ms = float(np.median(c_blocks)) / args.steps
    h2d_gbs = -dist.max(-(local_batch * img_elems * 4 / copy_ms / 1e6))     # slowest rank
    copy_ms = dist.max(copy_ms)
    e2e_state["primed"] = False

    # ---- roofline of the dominant kernel: the implicit-GEMM convolution tile kernel -------------
    lib.lnn_profile_enable(dev.index, 1)
    prof_steps = min(args.steps, 3)
    for _ in range(prof_steps):
        step_resident()
    nl, tms = ctypes.c_uint64(), ctypes.c_float()
    lib.lnn_profile_read(dev.index, 1, ctypes.byref(nl), ctypes.byref(tms))
    npre, tpre = ctypes.c_uint64(), ctypes.c_float()
    lib.lnn_profile_read(dev.index, 3, ctypes.byref(npre), ctypes.byref(tpre))
    nfc, tfc = ctypes.c_uint64(), ctypes.c_float()
    lib.lnn_profile_read(dev.index, 4, ctypes.byref(nfc), ctypes.byref(tfc))
    lib.lnn_profile_enable(dev.index, 0)
    # the tile engine runs convolutions 2-4; the 3-channel input layer has its own kernel
    conv_flop = (FWD_FLOP_PER_IMAGE - 2 * 256 * 1000 - 2 * 32 * 27 * 128 * 128) * local_batch * prof_steps
    conv_tflops = conv_flop / (tms.value / 1000.0) / 1e12 if tms.value > 0 else 0.0
    # Denominators.  fp32 operands are split in two parts and three products are issued per fp32
    # product.  Split FP16 issues them as kind::f16 (the bf16 / fp16 rate), split TF32 as
    # kind::tf32 (half that rate).  `frac` keeps the yardstick named for this workload, dense
    # TF32 = half the measured bf16 rate; `issued_frac` is the share of the pipe actually in use.
    f16_peak = peaks["bf16_tflops_sustained"]
    tf32_peak = f16_peak / 2.0
    products = 1 if passes == 1 else 3
    pipe_peak = f16_peak if passes == 2 else tf32_peak
    # DRAM traffic per launch: operand + output bytes of convolutions 2-4 (hi and lo channel-innermost
    # copies read once, result written once) times the traffic / algorithmic ratio of an ncu capture of
    # the same kernel on 512 images; traffic grows with the units processed.
    esz = 2 if passes == 2 else 4
    conv_bytes_per_image = ((2 * esz * 32 * 4096 + 4 * 64 * 1024) + (2 * esz * 64 * 1024 + 4 * 128 * 256) +
                            (2 * esz * 128 * 256 + 4 * 256 * 256))
    traffic = NCU_TRAFFIC_RATIO * conv_bytes_per_image * local_batch * prof_steps / max(1, nl.value)
    kind = {1: "kind::tf32, hi only", 2: "kind::f16, split FP16", 3: "kind::tf32, split TF32"}[passes]
    roofline = {"bound": "tensor", "kernel": f"tcgen05 tile engine (tc_kernel, implicit-GEMM conv2D, {kind}), convolutions 2-4",
                "achieved": round(conv_tflops, 2), "peak": round(tf32_peak, 1), "unit": "TFLOP/s",
                "frac": round(conv_tflops / tf32_peak, 4), "traffic": int(traffic),
                "traffic_source": "algorithmic operand+output bytes x 0.932, the DRAM/algorithmic ratio ncu measured on the same three launches at 512 images (part of the output is still in L2 when a launch ends)",
                "issued_frac": round(products * conv_tflops / pipe_peak, 4),
                "frac_of_f16_peak": round(conv_tflops / f16_peak, 4),
                "launches": int(nl.value), "avg_launch_ms": round(tms.value / max(1, nl.value), 4),
                "prepass_ms_per_step": round(tpre.value / prof_steps, 3),
                "first_layer": {"kernel": "fewch_conv_kernel (3-channel input layer on the tensor cores)",
                                "launches": int(nfc.value), "avg_launch_ms": round(tfc.value / max(1, nfc.value), 4)},
                "peak_source": f"peak = dense TF32 taken as half of the {peaks['source']} sustained bf16 cuBLAS rate; achieved counts "
                               f"algorithmic 2*M*N*K flops; issued_frac counts the {products} products issued per fp32 product "
                               f"against the {peaks['source']} rate of the pipe they run on ({pipe_peak:.0f} TFLOP/s)"}

    # ---- training step (softmax-CE, SGD lr 1e-3, NCCL gradient all-reduce) ---------------------
    train = None
    if not args.no_train:
        if world > 1:
            uid = parallel.new_unique_id() if rank == 0 else None
            uid = dist.bcast_bytes(uid, 128)
            parallel.init_process_rank(world, rank, uid)
        opt = nn.optimizer.SGD(model.trainables(), lr=1e-3)
        lab_rng = np.random.default_rng(77 + rank)
        onehots = []
        for j in range(n_mb):
            oh = np.zeros((mb, NCLASS), np.float32)
            oh[np.arange(mb), lab_rng.integers(0, NCLASS, mb)] = 1
            onehots.append(nn.Tensor_from_value(oh))
        scale = 1.0 / n_mb

        model._training_path = True

        def train_step():
            last = None
            for t, oh in zip(resident, onehots):
                loss = model.loss(model.forward(t), oh)
                if n_mb > 1:
                    loss = loss * scale
                loss.backward()
                last = loss
            opt.step(multi_gpu_step=True)
            opt.zero_grad()
            return last

        tsteps = max(1, min(args.steps, 3))
        for _ in range(2):
            last = train_step()
        nn.devices.wait()
        dist.barrier()
        timer.start()
        for _ in range(tsteps):
            last = train_step()
        ms_t = timer.stop_ms()
        loss_val = float(last.np()[0])
        dist.barrier()
        ms_t_max = dist.max(ms_t)
        train = {"value": round(TOTAL_BATCH * tsteps / (ms_t_max / 1000.0), 1), "unit": "images/s", "steps": tsteps,
                 "ms_per_step": round(ms_t_max / tsteps, 2), "last_micro_batch_loss": loss_val,
                 "what": "forward + softmax-CE + backward + SGD(lr 1e-3)" + (" + NCCL all-reduce of 645,416 gradients" if world > 1 else "")}
        if world > 1:
            # the replicas started equal and applied the same averaged gradient: they must still be equal
            sums = [float(t.sum().np()[0]) for t in model.trainables()]
            train["replicas_equal"] = all(dist.max(v) == -dist.max(-v) for v in sums)
        del onehots

    clocks = sampler.summary(m0, m1)
    if clocks["samples"] < 3:       # timed region shorter than a few sampling periods:
        clocks = sampler.summary(m0, None)   # use every sample from its start to the end of the GPU work
        clocks["window"] = "timed region through the end of the run"
    sampler.stop()
    nn.devices.check_status()

    ops = None
    if rank == 0 and world == 1 and not args.no_ops:
        del resident[:]
        ops = bench_ops(nn, dev, peaks, args.quick)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, cores, sample, _ = cpu_cnn_images_per_s(15.0)
        cpu = {"value": round(v, 3), "unit": "images/s", "cores": cores, "kind": "port", "sample": sample}
        if not args.no_ops:
            cpu["single_ops"] = cpu_single_ops()

    if rank == 0:
        line = {"metric": "cnn_inference_images_per_s", "value": round(value, 1), "unit": "images/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_max / args.steps, 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(world),
                "e2e": {"value": round(e2e_value, 1), "unit": "images/s", "h2d_bytes_per_step": local_batch * img_elems * 4,
                        "d2h_bytes_per_step": local_batch * NCLASS * 4, "ms_per_step": round(ms_e_max / args.steps, 3),
                        "h2d_ceiling_gbs": round(h2d_gbs, 2),
                        "h2d_ceiling_images_per_s": round(TOTAL_BATCH / (copy_ms / 1000.0), 1),
                        "h2d_ceiling_what": "copy-only run of the same uploads (same pinned buffers and calls, no kernels), all "
                                            "ranks at once: slowest rank's GB/s, and the images/s that upload rate allows"},
                "stock_api": stock, "timed_blocks": len(blocks),
                "gpu_launches": int(launches), "clocks": clocks, "roofline": roofline,
                "model_tflops": round(value * FWD_FLOP_PER_IMAGE / 1e12, 2)}
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if train is not None:
            line["train"] = train
        if ops is not None:
            line["ops"] = ops
        print(json.dumps(line), flush=True)
    dist.close()


def main():
    global TOTAL_BATCH, MICRO_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the single-op configurations")
    ap.add_argument("--no-train", action="store_true", help="skip the training step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quick", action="store_true", help="fewer iterations in the single-op configurations")
    ap.add_argument("--batch", type=int, default=4096,
                    help="global batch (default 4096, the benchmark configuration; smaller values are for profiling)")
    ap.add_argument("--micro-batch", type=int, default=MICRO_BATCH, help="images per forward call on one GPU")
    ap.add_argument("--ops-only", default=None, metavar="NAMES",
                    help="run only the single-op configurations whose name contains one of the comma-separated NAMES")
    args = ap.parse_args()
    TOTAL_BATCH = args.batch
    MICRO_BATCH = args.micro_batch
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    if args.ops_only:
        import litenn_b200 as nn
        dev = nn.devices.get_all()[0]
        nn.devices.set_current(dev)
        print(json.dumps({"ops": bench_ops(nn, dev, load_peaks(), args.quick, args.ops_only)}), flush=True)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        # plain invocation with N > 1: start one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    run_ours(args)


if __name__ == "__main__":
    main()
