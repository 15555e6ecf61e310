#!/usr/bin/env python
"""Benchmark of the spectral hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload = "net_b30_10_6"``): forward pass of the three-stage equivariant
classifier  S2Conv(1->20, b 30->10) -> ReLU -> SO3Conv(20->40, b 10->6) -> ReLU -> so3_integrate ->
Linear(40->10)  on synthetic batches of 256 N(0,1) signals on the 60x60 sphere grid per GPU,
random-init weights, float32, written as plain module calls and rewritten into the fused kernels by
``s2cnn_b200.fuse``.  One step = ``batches_per_step`` forward passes, each over one batch taken in
turn from a pool of resident batches larger than L2 (a single pass lasts 0.3 ms; a step is sized so
that the timed region lasts about half a second).  Successive batches are independent, so
``--lanes`` (default 4) captured copies of the pass replay on their own streams with successive
batches on successive streams: the blocks of one pass fill the SMs that the partly filled last
waves of another leave idle (``--lanes 1``: one stream, one pass at a time).  The headline metric
is samples/s; ``value`` is measured with the batches resident in HBM, ``e2e`` through the public
module API from pinned host memory (host->device copy of every batch and device->host read of its
logits inside the timed interval; uploads run on a copy stream ahead of the passes, results return
on another stream - ``serial_ms_per_batch`` gives the same one after another on one stream).

Further objects on the same line:
  ``so3_fft_b64``     (rank 0, N = 1) the standalone SO(3) FFT round trip at b = 64 (real
                      [64,128,128,128] -> spectrum -> signal) in GB/s of algorithmic bytes;
  ``so3_mm_tensor``   (rank 0, N = 1) the tensor-core spectral product at a GEMM-sized case;
  ``train_step_c4``   (every N) training step of the deep model, batch 32 per rank, with the
                      per-layer gradient all-reduce launched from autograd hooks when N > 1;
  ``strong_scaling``  (N > 1) the same classifier with a FIXED global batch of 256 split over the
                      ranks (256 / N samples per GPU).

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N``;
every rank runs the same per-GPU batch (weak scaling, no data-path collective), the time is the max
over ranks and ``value`` the whole-job samples/s.

``--impl reference`` times the reference's own CPU implementation of the same network on the host
cores: the unmodified package from ``oracle/_ref`` when that copy exists (made by
``oracle/make_ref.py`` where a reference checkout is present), else the CPU oracle port
(oracle/s2cnn_oracle.py).
"""
import argparse
import json
import os
import re
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH_PER_GPU = 256
NET = dict(b0=30, b1=10, b2=6, f0=1, f1=20, f2=40, nclass=10)
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 << 20
TRAFFIC_PROFILE = os.path.join(ROOT, "profiles", "net_b30_10_6_dram_traffic.md")


def grids():
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    return g2, g3


def n3(b):
    return b * (4 * b * b - 1) // 3


def workload_config(world, batches_per_step):
    """The `config` object, identical for both arms."""
    return {"workload": "net_b30_10_6", "batch_per_gpu": BATCH_PER_GPU,
            "global_batch": BATCH_PER_GPU * world, "batches_per_step": batches_per_step,
            "layers": "S2Conv(1->20,b30->10) ReLU SO3Conv(20->40,b10->6) ReLU so3_integrate "
                      "Linear(40->10)"}


# ------------------------------------------------------------------------------------------------
# workload definitions
# ------------------------------------------------------------------------------------------------
def make_net(device, seed=0, fused=True):
    """The classifier written exactly as a user of the reference writes it (plain modules in a
    Sequential, examples/mnist/run.py:55-98); ``s2cnn_b200.fuse`` then routes the chain through the
    fused kernels.  Same values as the plain chain."""
    import s2cnn_b200 as S
    g2, g3 = grids()
    torch.manual_seed(seed)

    class Integrate(torch.nn.Module):
        def forward(self, x):
            return S.so3_integrate(x)

    net = torch.nn.Sequential(
        S.S2Convolution(NET["f0"], NET["f1"], NET["b0"], NET["b1"], g2),
        torch.nn.ReLU(),
        S.SO3Convolution(NET["f1"], NET["f2"], NET["b1"], NET["b2"], g3),
        torch.nn.ReLU(),
        Integrate(),
        torch.nn.Linear(NET["f2"], NET["nclass"]),
    ).to(device).eval()
    return S.fuse(net) if fused else net


def oracle_net_forward(x, params):
    from oracle import s2cnn_oracle as O
    g2, g3 = grids()
    h = torch.relu(O.s2_convolution(x, params["k1"], params["b1"], NET["b0"], NET["b1"], g2))
    h = torch.relu(O.so3_convolution(h, params["k2"], params["b2"], NET["b1"], NET["b2"], g3))
    return torch.nn.functional.linear(O.so3_integrate(h), params["w"], params["b"])


def oracle_params(seed=0):
    g2, g3 = grids()
    torch.manual_seed(seed)
    k1 = torch.empty(NET["f0"], NET["f1"], len(g2)).uniform_(-1, 1)
    k2 = torch.empty(NET["f1"], NET["f2"], len(g3)).uniform_(-1, 1)
    lin = torch.nn.Linear(NET["f2"], NET["nclass"])
    return dict(k1=k1, b1=torch.zeros(1, NET["f1"], 1, 1, 1), k2=k2,
                b2=torch.zeros(1, NET["f2"], 1, 1, 1), w=lin.weight.detach(), b=lin.bias.detach())


def reference_net(seed=0):
    """The same classifier built from the UNMODIFIED reference package (CPU), or None when no copy
    of it is available next to the oracle."""
    from oracle import ref_import
    path = ref_import.local_copy()
    if path is None:
        return None
    R = ref_import.load(path)
    g2, g3 = grids()
    torch.manual_seed(seed)
    c1 = R.S2Convolution(NET["f0"], NET["f1"], NET["b0"], NET["b1"], g2)
    c2 = R.SO3Convolution(NET["f1"], NET["f2"], NET["b1"], NET["b2"], g3)
    lin = torch.nn.Linear(NET["f2"], NET["nclass"])

    def forward(x):
        with ref_import.in_scratch():
            h = torch.relu(c2(torch.relu(c1(x))))
            return lin(R.so3_integrate(h))

    return forward


def kernel_bytes(B):
    """Per forward pass, per kernel name: bytes the kernel has to move once - its own inputs and
    outputs, constant tables excluded - summed over its launches in the pass.  Fused kernels are
    charged the bytes of the module boundaries they cover - the tensor each reference module writes
    once and the next one reads once (the per-sample figure of the workload: 14,400 + 2 * 640,000 +
    2 * 276,480 B) - although they keep those tensors on chip; `traffic` in the roofline object is
    what actually crosses DRAM."""
    b0, b1, b2, f0, f1, f2 = (NET[k] for k in ("b0", "b1", "b2", "f0", "f1", "f2"))
    c = 8  # bytes per complex
    sig1 = B * f1 * (2 * b1) ** 3 * 4   # conv1 output / conv2 input signal
    out = {}
    N0 = 2 * b0
    out["s2_fwd_fused"] = B * f0 * N0 * N0 * 4 + b1 * b1 * B * f0 * c
    out["rft_forward"] = (f0 * f1 * 24 * 4 + b1 * b1 * f0 * f1 * c) + (f1 * f2 * 192 * 4 + n3(b2) * f1 * f2 * c)
    out["so3_relay_fused<%d>" % (2 * b1)] = (b1 * b1 * (B * f0 + f0 * f1) * c + 2 * sig1 +
                                               n3(b2) * B * f1 * c)
    sig2 = B * f2 * (2 * b2) ** 3 * 4
    out["so3_inv_fused<%d>" % (2 * b2)] = n3(b2) * B * f2 * c + 2 * sig2 + B * f2 * 4
    out["so3_mm_tc_kernel"] = n3(b2) * (B * f1 + f1 * f2 + B * f2) * c
    return out


def net_flops(B):
    b1, b2, f0, f1, f2 = (NET[k] for k in ("b1", "b2", "f0", "f1", "f2"))
    c3 = b2 * b2 * (2 * b2 * b2 - 1)
    return dict(so3_mm=8 * c3 * B * f1 * f2, s2_mm=8 * n3(b1) * B * f0 * f1)


def measured_traffic():
    """DRAM bytes per launch, per kernel, from the committed ncu summary of this workload (table rows
    ``| `kernel` | launches | dram read MB | dram write MB |``); {} when the file is missing."""
    out = {}
    try:
        with open(TRAFFIC_PROFILE) as f:
            for ln in f:
                m = re.match(r"\|\s*`([^`]+)`\s*\|\s*(\d+)\s*\|\s*([\d.]+)\s*\|\s*([\d.]+)\s*\|", ln)
                if m:
                    out[m.group(1)] = (float(m.group(3)) + float(m.group(4))) * 1e6
    except OSError:
        pass
    return out


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        self.lines = []
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(self.index)], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, 1590.0, "fallback"


def numa_pin(local_rank):
    """Keep this rank's threads (and so the pinned host buffers it allocates next) on the CPUs of
    the NUMA node its GPU hangs off, when the platform tells; returns a short description."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = [i for i in range(os.cpu_count()) if (mask[i // 64] >> (i % 64)) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return "threads bound to the %d CPUs nearest GPU %d" % (len(allowed), local_rank)
    except Exception as e:  # noqa: BLE001
        return "not bound (%s)" % type(e).__name__
    return "not bound"


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("nccl", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", local))
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def timed_repeats(fn, repeats, warmup=3):
    """Per-call CUDA-event times (ms) of `repeats` calls after `warmup` untimed ones."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeats):
        a, e = event_pair()
        a.record()
        fn()
        e.record()
        e.synchronize()
        ts.append(a.elapsed_time(e))
    return ts


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU code (or the oracle port) on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_forward_fn():
    """(callable(x) -> logits, kind): the unmodified reference when a copy is present, else the
    oracle port."""
    ref = None
    try:
        ref = reference_net()
    except Exception:  # noqa: BLE001  (a broken copy must not take the bench down)
        ref = None
    if ref is not None:
        return ref, "reference"
    params = oracle_params()
    return (lambda x: oracle_net_forward(x, params)), "port"


def cpu_baseline(budget_s=20.0):
    """Bounded sample of the workload on the host cores: full batches until `budget_s` is used up
    (at least one), best batch time."""
    torch.set_num_threads(os.cpu_count() or 1)
    fwd, kind = cpu_forward_fn()
    batch = BATCH_PER_GPU
    x = torch.randn(batch, NET["f0"], 2 * NET["b0"], 2 * NET["b0"],
                    generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        fwd(x[:2])     # fills the table caches
        t_all = time.perf_counter()
        fwd(x)         # warm-up at full size
        best, n = float("inf"), 0
        while n < 1 or (time.perf_counter() - t_all < budget_s and n < 8):
            t0 = time.perf_counter()
            fwd(x)
            best = min(best, time.perf_counter() - t0)
            n += 1
    return {"value": batch / best, "unit": "samples/s", "cores": torch.get_num_threads(),
            "kind": kind, "sample": "%d full batches of %d, best (%.2f s)" % (n, batch, best)}


def run_reference(args):
    world, rank, _ = dist_setup(args.gpus)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    fwd, kind = cpu_forward_fn()
    batch = BATCH_PER_GPU
    x = torch.randn(batch, NET["f0"], 2 * NET["b0"], 2 * NET["b0"],
                    generator=torch.Generator().manual_seed(1))
    # one step of this arm = ONE batch (a bounded sample of the repo arm's step of
    # `batches_per_step` batches); the metric is samples/s either way
    with torch.no_grad():
        fwd(x[:2])
        for _ in range(max(1, min(args.warmup, 2))):
            fwd(x)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fwd(x)
        dt = (time.perf_counter() - t0) / args.steps
    value = batch / dt
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "samples_per_sec_fwd", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": workload_config(args.gpus, args.batches_per_step),
        "note": ("the reference's own CPU code path (unmodified package, three API shims, lie_learn "
                 "stand-in)" if kind == "reference" else
                 "CPU oracle port (no copy of the reference package next to the oracle)") +
                "; rank 0 only; each step of this arm is one batch of %d" % batch,
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": kind,
                         "sample": "%d steps of one full batch of %d" % (args.steps, batch)},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# extra measurements
# ------------------------------------------------------------------------------------------------
def so3_fft_b64(device, hbm_gbs, repeats=50):
    from s2cnn_b200.soft.so3_fft import so3_rfft, so3_rifft
    b, nb = 64, 64
    x = torch.randn(nb, 2 * b, 2 * b, 2 * b, device=device)
    t_build = time.perf_counter()
    s = so3_rfft(x)
    y = so3_rifft(s)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    res = {}
    for name, fn in (("rfft", lambda: so3_rfft(x)), ("rifft", lambda: so3_rifft(s))):
        ts = timed_repeats(fn, repeats)
        res[name + "_ms"] = float(np.median(ts))
        res[name + "_ms_min"] = float(np.min(ts))
    bytes_dir = nb * (2 * b) ** 3 * 4 + n3(b) * nb * 8
    # idempotence of the round trip (the reference's own test, tests/so3_fft.py:34-44)
    y2 = so3_rifft(so3_rfft(y))
    err = ((y - y2).norm() / y2.norm()).item()
    gbs = 2 * bytes_dir / ((res["rfft_ms"] + res["rifft_ms"]) * 1e-3) / 1e9
    res.update({"workload": "so3_rfft+so3_rifft b=64 batch=64 (inputs 537 MB > L2)",
                "repeats": repeats, "algorithmic_bytes_per_direction": bytes_dir,
                "roundtrip_GBps": gbs, "frac_of_hbm": gbs / hbm_gbs,
                "rfft_GBps": bytes_dir / (res["rfft_ms"] * 1e-3) / 1e9,
                "rifft_GBps": bytes_dir / (res["rifft_ms"] * 1e-3) / 1e9,
                "idempotence_rel_l2": err, "first_call_s_incl_tables": t_build})
    return res


def so3_mm_tensor(device, bf16_tf, repeats=50):
    """The spectral product of the widest layer of the deep model among the reference's
    configurations (SO3Conv 100 -> 100 at b_out = 10, batch 32): time of so3_mm on the tcgen05 path,
    algorithmic flops (8 per complex multiply-add) and the TF32 flops actually issued (three TF32
    products per FP32 product), against half of the measured bf16 GEMM peak (TF32 runs at half the
    bf16 rate)."""
    from s2cnn_b200 import so3_mm
    nl, nb, fi, fo = 10, 32, 100, 100
    x = torch.randn(n3(nl), nb, fi, 2, device=device)
    y = torch.randn(n3(nl), fi, fo, 2, device=device)
    ts = timed_repeats(lambda: so3_mm(x, y), repeats)
    ms = float(np.median(ts))
    flops = 8.0 * sum((2 * l + 1) ** 3 for l in range(nl)) * nb * fi * fo
    issued = 3.0 * flops / (ms * 1e-3) / 1e12
    alg = flops / (ms * 1e-3) / 1e12
    peak = bf16_tf / 2.0
    return {"workload": "so3_mm nl=10 batch=32 f_in=100 f_out=100 (operands L2-resident)",
            "repeats": repeats, "ms": ms, "ms_min": float(np.min(ts)),
            "algorithmic_TFLOPs": alg, "algorithmic_frac": alg / peak,
            "issued_tf32_TFLOPs": issued, "peak_tf32_TFLOPs": peak,
            "peak_source": "half of the measured bf16 GEMM peak", "frac": issued / peak}


def deep_model(device):
    """The deep model among the reference's configurations: S2Conv(6->100, b 64->16, max_beta pi/32)
    -> ReLU -> SO3Conv(100->100, b 16->10) -> ReLU -> SO3Conv(100->255, b 10->5) -> ReLU ->
    so3_integrate -> Linear(255->55)."""
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 32, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    torch.manual_seed(4)   # same weights on every rank

    class Deep(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.c1 = S.S2Convolution(6, 100, 64, 16, g2)
            self.c2 = S.SO3Convolution(100, 100, 16, 10, g3)
            self.c3 = S.SO3Convolution(100, 255, 10, 5, g3)
            self.lin = torch.nn.Linear(255, 55)

        def forward(self, x):
            x = torch.relu(self.c1(x))
            x = torch.relu(self.c2(x))
            x = torch.relu(self.c3(x))
            return self.lin(S.so3_integrate(x))

    # written with plain calls; fuse() folds every ReLU into the kernel that consumes it (in a
    # training step the activations are still stored - only the separate ReLU passes disappear)
    return S.fuse(Deep().to(device))


def train_step_c4(device, world, rank, batch=32, steps=60):
    """Training step (forward, cross-entropy on uniform random labels, backward, gradient
    all-reduce) of the deep model, batch 32 per rank, synthetic input.  With several ranks every
    layer's gradients are summed over the ranks by one NCCL all-reduce launched from an autograd
    hook as soon as that layer's backward is done (s2cnn_b200.parallel.GradientReducer), so the
    reduction of the last layers overlaps the backward pass of the first.  Times are CUDA-event
    times, max over ranks."""
    from s2cnn_b200 import parallel
    net = deep_model(device)
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(batch, 6, 128, 128, generator=gen).to(device)
    labels = torch.randint(0, 55, (batch,), generator=gen).to(device)
    reducer = parallel.GradientReducer(net)
    grad_bytes = sum(f.numel() * f.element_size() for f in reducer.flat)

    def step(reduce):
        reducer.zero_grad()
        loss = torch.nn.functional.cross_entropy(net(x), labels)
        if not reduce:
            reducer.suspended = True
        loss.backward()
        reducer.suspended = False
        if reduce:
            reducer.finish()
        return loss

    def timed(reduce):
        for _ in range(3):
            step(reduce)
        torch.cuda.synchronize()
        barrier(world)
        a, e = event_pair()
        a.record()
        for _ in range(steps):
            loss = step(reduce)
        e.record()
        e.synchronize()
        return max_over_ranks(a.elapsed_time(e) / steps, world, device), loss

    ms_local, loss = timed(False)
    # one more step with a CUDA-event pair around every launch of the library: where the step goes
    import ctypes
    from s2cnn_b200 import _lib
    lib = _lib.cuda_lib()
    lib.s2c_timing_begin()
    step(False)
    torch.cuda.synchronize()
    cbuf = ctypes.create_string_buffer(1 << 16)
    lib.call("s2c_timing_end", cbuf, len(cbuf))
    rows = [ln.split() for ln in cbuf.value.decode().splitlines() if ln.strip()]
    rows.sort(key=lambda r: -float(r[2]))
    kernels = {r[0]: {"launches": int(r[1]), "ms": round(float(r[2]), 4)} for r in rows[:10]}
    kernels_ms = sum(float(r[2]) for r in rows)
    out = {"workload": "deep model 6->100->100->255->55, b 64->16->10->5, batch %d per rank, "
                       "fwd+bwd" % batch,
           "steps": steps, "n_ranks": world, "global_batch": batch * world,
           "ms_per_step_no_allreduce": ms_local, "grad_bytes": grad_bytes,
           "library_kernels_ms": round(kernels_ms, 4), "kernels": kernels,
           "loss_finite": bool(torch.isfinite(loss))}
    if world > 1:
        import torch.distributed as dist
        ms, loss = timed(True)
        # the same buckets reduced with nothing else running: what the all-reduce costs by itself
        for _ in range(3):
            for f in reducer.flat:
                dist.all_reduce(f)
        torch.cuda.synchronize()
        barrier(world)
        a, e = event_pair()
        a.record()
        for _ in range(20):
            for f in reducer.flat:
                dist.all_reduce(f)
        e.record()
        e.synchronize()
        alone = max_over_ranks(a.elapsed_time(e) / 20, world, device)
        out.update({"ms_per_step": ms, "allreduce_ms": alone,
                    "allreduce_exposed_ms": ms - ms_local,
                    "allreduce": "one NCCL all-reduce per layer (%d buckets), launched from autograd "
                                 "hooks during backward" % len(reducer.flat),
                    "samples_per_s": batch * world / (ms * 1e-3),
                    "loss_finite": bool(torch.isfinite(loss))})
    else:
        out.update({"ms_per_step": ms_local, "allreduce_ms": 0.0, "allreduce_exposed_ms": 0.0,
                    "samples_per_s": batch / (ms_local * 1e-3)})
    reducer.remove()
    return out


def strong_scaling(device, world, rank, net, flush, steps, batches_per_step, lanes=1):
    """BASELINE config 3 as written: a FIXED global batch of 256 split over the ranks (successive
    global batches on `lanes` alternating streams, as in the headline measurement)."""
    from s2cnn_b200 import parallel
    from s2cnn_b200.graph import GraphedForward, InterleavedForward
    lo, hi = parallel.shard_range(BATCH_PER_GPU, rank, world)
    b = hi - lo
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(BATCH_PER_GPU, NET["f0"], 2 * NET["b0"], 2 * NET["b0"], generator=gen)[lo:hi]
    x = x.to(device)
    g = InterleavedForward(net, x, lanes=lanes) if lanes > 1 else GraphedForward(net, x)

    def run_batches(n):
        if lanes > 1:
            g.fork()
            for _ in range(n):
                g.submit(x)
            g.join()
        else:
            for _ in range(n):
                g(x)

    run_batches(2 * lanes + 1)
    torch.cuda.synchronize()
    barrier(world)
    total = 0.0
    for _ in range(steps):
        flush.zero_()
        a, e = event_pair()
        a.record()
        run_batches(batches_per_step)
        e.record()
        e.synchronize()
        total += a.elapsed_time(e)
    ms = max_over_ranks(total, world, device) / (steps * batches_per_step)
    return {"workload": "net_b30_10_6, global batch 256 split over the ranks",
            "batch_per_gpu": b, "ms_per_batch": ms, "samples_per_s": BATCH_PER_GPU / (ms * 1e-3),
            "passes_in_flight": lanes,
            "limiter": "at %d samples per GPU the kernels of one pass have fewer blocks than the "
                       "GPU has SM slots and launch latency shows; several passes in flight "
                       "(passes_in_flight) fill the SMs" % b}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    world, rank, local = dist_setup(args.gpus)
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback exists)"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = numa_pin(local)
    from s2cnn_b200 import _lib
    lib = _lib.cuda_lib()
    hbm_gbs, bf16_tf, peak_kind = measured_peaks()

    net = make_net(device)
    B = BATCH_PER_GPU
    M = args.batches_per_step
    gen = torch.Generator().manual_seed(1 + rank)
    in_bytes = B * NET["f0"] * (2 * NET["b0"]) ** 2 * 4
    pool_n = L2_BYTES // in_bytes + 4            # resident batches: more bytes than L2 holds
    host_n = 4
    x_host = [torch.randn(B, NET["f0"], 2 * NET["b0"], 2 * NET["b0"], generator=gen).pin_memory()
              for _ in range(host_n)]
    pool = [x_host[i % host_n].to(device) + 0.001 * i for i in range(pool_n)]
    out_host = torch.empty(B, NET["nclass"]).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    from s2cnn_b200.graph import GraphedForward, InterleavedForward, PipelinedForward
    use_graph = not args.no_graph
    graphed = GraphedForward(net, pool[0]) if use_graph else None
    lanes = InterleavedForward(net, pool[0], lanes=args.lanes) if use_graph and args.lanes > 1 else None

    def forward_resident(i):
        if use_graph:
            return graphed(pool[i % pool_n])
        with torch.no_grad():
            return net(pool[i % pool_n])

    def step_resident():
        if lanes is not None:      # successive batches on alternating streams, two passes in flight
            lanes.fork()
            for i in range(M):
                lanes.submit(pool[i % pool_n])
            lanes.join()
            return
        for i in range(M):
            forward_resident(i)

    def forward_eager():
        with torch.no_grad():
            return net(pool[0])

    def step_serial():
        # host -> device copy of each batch, forward, device -> host read of the logits, in turn
        for i in range(M):
            if use_graph:
                out_host.copy_(graphed(x_host[i % host_n]), non_blocking=True)
            else:
                with torch.no_grad():
                    xd = x_host[i % host_n].to(device, non_blocking=True)
                    out_host.copy_(net(xd), non_blocking=True)

    for _ in range(max(args.warmup, 3)):
        step_resident()
    step_serial()
    torch.cuda.synchronize()

    def time_steps(fn):
        """Sum of per-step CUDA-event times; L2 is flushed (256 MB write) between steps, outside
        the timed intervals."""
        total = 0.0
        for _ in range(args.steps):
            flush.zero_()
            a, e = event_pair()
            a.record()
            fn()
            e.record()
            e.synchronize()
            total += a.elapsed_time(e)
        return total

    # ---- resident-input throughput (headline `value`) ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier(world)
    torch.cuda.synchronize()
    total_ms = time_steps(step_resident)
    torch.cuda.synchronize()
    # kernels of this library per forward pass, counted on an eager pass (a graph replay launches
    # the same kernels without going through the library's launch counter)
    n0 = lib.s2c_launch_count()
    forward_eager()
    torch.cuda.synchronize()
    launches = (lib.s2c_launch_count() - n0) * args.steps * M
    barrier(world)
    total_ms = max_over_ranks(total_ms, world, device)
    ms_per_step = total_ms / args.steps
    value = B * M * world / (ms_per_step * 1e-3)

    # ---- end to end through the module API from pinned host memory ----
    barrier(world)
    torch.cuda.synchronize()
    serial_ms = time_steps(step_serial) / args.steps
    torch.cuda.synchronize()
    if use_graph:
        # the same batches with the upload of batch i + 1 running behind the forward pass of batch i
        # (s2cnn_b200.graph.PipelinedForward): every timed interval holds M forward passes, M result
        # read-backs and M uploads; the L2 flush stays between intervals
        # one slot more than passes in flight, so that an upload never waits for a running pass
        pipe = PipelinedForward(net, pool[0], depth=max(2, args.lanes + 1))
        for i in range(3):
            pipe.submit(x_host[i % host_n], out_host)
        pipe.wait()
        pipe.prefetch(x_host[0])
        torch.cuda.synchronize()
        barrier(world)
        e2e_ms = 0.0
        for _ in range(args.steps):
            flush.zero_()
            a, e = event_pair()
            a.record()
            for i in range(M):
                pipe.prefetch(x_host[(i + 1) % host_n])   # batch i + 1 -> the idle input buffer
                pipe.run(out_host)                        # batch i: replay + logits to host memory
            pipe.join_uploads()        # the interval ends when the last upload has landed, too,
            pipe.join_results()        # and the last result has reached the host
            e.record()
            e.synchronize()
            e2e_ms += a.elapsed_time(e)
        pipe.run(out_host)
        torch.cuda.synchronize()
    else:
        e2e_ms = serial_ms * args.steps
    barrier(world)
    e2e_ms = max_over_ranks(e2e_ms, world, device) / args.steps
    clocks = sampler.stop() if rank == 0 else None   # sampled over both timed legs
    e2e = {"value": B * M * world / (e2e_ms * 1e-3), "unit": "samples/s",
           "h2d_bytes_per_step": in_bytes * M, "d2h_bytes_per_step": out_host.numel() * 4 * M,
           "ms_per_step": e2e_ms, "ms_per_batch": e2e_ms / M,
           "how": ("uploads overlapped with the forward passes (%d input buffers, copy stream; each "
                   "buffer's pass replays on its own stream; results return on another stream); "
                   "every batch is uploaded, run and read back inside the interval"
                   % max(2, args.lanes + 1))
                  if use_graph else "upload, forward, read-back one after another",
           "serial_ms_per_batch": serial_ms / M, "host_buffers": numa}

    # ---- per-kernel CUDA-event times over K more eager passes (roofline) ----
    lib.s2c_timing_begin()
    for _ in range(args.steps):
        flush.zero_()
        forward_eager()
    import ctypes
    cbuf = ctypes.create_string_buffer(1 << 16)
    lib.call("s2c_timing_end", cbuf, len(cbuf))
    per_kernel = {}
    for ln in cbuf.value.decode().splitlines():
        name, cnt, ms = ln.split()
        per_kernel[name] = (int(cnt), float(ms))
    kb = kernel_bytes(B)
    kernels = []
    for name, (cnt, ms) in per_kernel.items():
        per_pass_bytes = kb.get(name, 0)
        kernels.append({"kernel": name, "launches_per_batch": cnt / args.steps,
                        "ms_per_batch": ms / args.steps, "avg_launch_ms": ms / cnt,
                        "alg_bytes_per_batch": per_pass_bytes,
                        "GBps": per_pass_bytes / (ms / args.steps * 1e-3) / 1e9 if ms > 0 else None})
    kernels.sort(key=lambda k: -k["ms_per_batch"])
    top = kernels[0]
    flops = net_flops(B)
    traffic_tab = measured_traffic() if B == 256 else {}
    if top["kernel"] == "so3_mm_tc_kernel":
        # dominant kernel is the spectral product: tensor roofline, TF32 dense = 1/2 bf16
        fl = flops["so3_mm"]
        ach = fl / (top["ms_per_batch"] * 1e-3) / 1e12
        peak = bf16_tf / 2
        roofline = {"kernel": "so3_mm_tc_kernel", "bound": "tensor", "achieved": ach,
                    "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                    "traffic": traffic_tab.get(top["kernel"]),
                    "peak_source": peak_kind + " bf16 / 2 (TF32 dense)"}
    else:
        ach = top["GBps"]
        traffic = traffic_tab.get(top["kernel"])
        roofline = {"kernel": top["kernel"], "bound": "hbm", "achieved": ach, "peak": hbm_gbs,
                    "unit": "GB/s", "frac": ach / hbm_gbs, "traffic": traffic,
                    "peak_source": peak_kind,
                    "alg_bytes_per_launch": top["alg_bytes_per_batch"] / max(top["launches_per_batch"], 1),
                    "launches_per_batch": top["launches_per_batch"],
                    "note": "algorithmic bytes of a fused kernel are those of the module boundaries "
                            "it covers (tensors it keeps on chip); `traffic` is what crosses DRAM "
                            "per launch in the committed ncu summary, `dram_frac` that figure over "
                            "the launch time and the peak - the kernel is bound by instruction "
                            "issue, not by HBM"}
        if traffic:
            roofline["dram_frac"] = traffic / (top["avg_launch_ms"] * 1e-3) / 1e9 / hbm_gbs
            roofline["traffic_source"] = os.path.relpath(TRAFFIC_PROFILE, ROOT)
    step_bytes = 1847360 * B    # module-boundary bytes per sample of the whole pass
    whole = step_bytes / (ms_per_step / M * 1e-3) / 1e9
    roofline["whole_pass"] = {"alg_bytes_per_batch": step_bytes, "GBps": whole,
                              "frac": whole / hbm_gbs}
    roofline["timing"] = "per-launch CUDA events on the launching stream over %d passes run right " \
                         "after the timed region (launched op by op)" % args.steps

    launches_total = int(sum_over_ranks(launches, world, device))

    cfg = workload_config(world, M)
    cfg.update({
        "fusion": "s2_mm + conv1 synthesis + ReLU + conv2 analysis in one kernel; second ReLU and "
                  "so3_integrate inside conv2's synthesis kernel (s2cnn_b200.fuse on a plain Sequential)",
        "launch": "eager" if args.no_graph else (
            "CUDA graph replay (s2cnn_b200.graph.GraphedForward)" if args.lanes < 2 else
            "CUDA graph replays on %d streams, successive batches on alternating streams "
            "(s2cnn_b200.graph.InterleavedForward)" % args.lanes),
        "sharding": "batch over ranks, no collective in forward",
        "l2": "inputs rotate through a pool of %d resident batches (%d MB > L2); 256 MB flush "
              "write between timed steps" % (pool_n, pool_n * in_bytes >> 20)})
    line = {
        "metric": "samples_per_sec_fwd", "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "ms_per_batch": ms_per_step / M,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": cfg,
        "e2e": e2e, "gpu_launches": launches_total, "roofline": roofline,
        "kernels": kernels[:8],
    }
    extras = {}
    if not args.skip_train:
        extras["train_step_c4"] = train_step_c4(device, world, rank)
    if world > 1 and not args.skip_train:
        extras["strong_scaling"] = strong_scaling(device, world, rank, net, flush, args.steps, M,
                                                  lanes=args.lanes if use_graph else 1)
    if rank == 0:
        line["clocks"] = clocks
        line.update(extras)
        if world == 1 and not args.skip_cpu:
            line["cpu_baseline"] = cpu_baseline()
        if world == 1 and not args.skip_fft64:
            line["so3_fft_b64"] = so3_fft_b64(device, hbm_gbs)
            line["so3_mm_tensor"] = so3_mm_tensor(device, bf16_tf)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batches-per-step", type=int, default=80,
                    help="forward passes (batches) inside one timed step")
    ap.add_argument("--lanes", type=int, default=4,
                    help="forward passes in flight on separate streams (1 = one stream)")
    ap.add_argument("--skip-fft64", action="store_true")
    ap.add_argument("--skip-train", action="store_true",
                    help="omit the training-step and strong-scaling legs")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU-baseline leg")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the forward op by op instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
