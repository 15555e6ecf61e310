#!/usr/bin/env python
"""Benchmark of the spectral hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload = "net_b30_10_6"``): forward pass of the three-stage equivariant
classifier  S2Conv(1->20, b 30->10) -> ReLU -> SO3Conv(20->40, b 10->6) -> ReLU -> so3_integrate ->
Linear(40->10)  on a synthetic batch of 256 N(0,1) signals on the 60x60 sphere grid per GPU,
random-init weights, float32.  One step = one forward pass over one batch.  The headline metric is
samples/s; ``value`` is measured with the batch resident in HBM, ``e2e`` through the public module
API from pinned host memory (host->device copy of a batch and device->host read of the logits
inside every timed interval; the copy is that of the NEXT batch, overlapped with the forward pass
on a copy stream - ``serial_ms_per_step`` gives the same without the overlap).  Further objects on
the same line (rank 0, one GPU): ``so3_fft_b64`` - the standalone SO(3) FFT round trip at b = 64
(real [64,128,128,128] -> spectrum -> signal) in GB/s of algorithmic bytes; ``so3_mm_tensor`` - the
tensor-core spectral product at a GEMM-sized case; ``train_step_c4`` - the training step of the deep
model among the reference's configurations.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N bench.py --gpus N``;
every rank runs the same per-GPU batch (weak scaling, no data-path collective), the time is the max
over ranks and ``value`` the whole-job samples/s.

``--impl reference`` times the CPU oracle (a torch-CPU restatement of the reference's own CPU code
path, oracle/s2cnn_oracle.py) on the host cores for the same workload.
"""
import argparse
import json
import os
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


def grids():
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 16, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    return g2, g3


def n3(b):
    return b * (4 * b * b - 1) // 3


# ------------------------------------------------------------------------------------------------
# workload definitions
# ------------------------------------------------------------------------------------------------
def make_net(device, seed=0):
    import s2cnn_b200 as S
    g2, g3 = grids()
    torch.manual_seed(seed)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = S.S2Convolution(NET["f0"], NET["f1"], NET["b0"], NET["b1"], g2)
            self.conv2 = S.SO3Convolution(NET["f1"], NET["f2"], NET["b1"], NET["b2"], g3)
            self.linear = torch.nn.Linear(NET["f2"], NET["nclass"])

        def forward(self, x):
            # relu(conv1) -> conv2 -> relu -> integrate -> linear.  conv1's synthesis, the first ReLU
            # and conv2's analysis run as one kernel (the 20^3 signal between the layers is never
            # written); the second ReLU and the integration run in the last pass of conv2's
            # synthesis (its output signal is never written either).  Same values as the plain chain.
            x = self.conv1(x, relu_so3_fft=self.conv2.b_out)          # conv2's input spectrum
            x = self.conv2(x, input_spectrum=True, relu_integrate=True)   # [batch, f2]
            return self.linear(x)

    return Net().to(device).eval()


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


# algorithmic bytes per launch of each kernel of the net forward at batch B (what the kernel must
# read and write once: its own inputs and outputs, constant tables excluded)
def kernel_bytes(B):
    """Per forward pass, per kernel name: bytes the kernel has to move once - its own inputs and
    outputs, constant tables excluded - summed over its launches in the step."""
    b0, b1, b2, f0, f1, f2 = (NET[k] for k in ("b0", "b1", "b2", "f0", "f1", "f2"))
    c = 8  # bytes per complex
    sig1 = B * f1 * (2 * b1) ** 3 * 4   # conv1 output / conv2 input signal
    out = {}
    # S2 analysis of the real input in one kernel: reads the signal, writes the S2 spectrum
    N0 = 2 * b0
    out["s2_fwd_fused"] = B * f0 * N0 * N0 * 4 + b1 * b1 * B * f0 * c
    # kernel-grid -> spectrum transforms of both layers
    out["rft_forward"] = (f0 * f1 * 24 * 4 + b1 * b1 * f0 * f1 * c) + (f1 * f2 * 192 * 4 + n3(b2) * f1 * f2 * c)
    # Fused kernels are charged the bytes of the module boundaries they cover - the tensor each
    # reference module writes once and the next one reads once (the per-sample figure of the
    # workload: 14,400 + 2 * 640,000 + 2 * 276,480 B) - although they keep those tensors on chip;
    # `traffic` in the roofline object is what actually crosses DRAM.
    # conv1 tail + ReLU + conv2 head in one kernel: conv1's output written + read as conv2's input
    out["so3_relay_fused<%d>" % (2 * b1)] = (b1 * b1 * (B * f0 + f0 * f1) * c + 2 * sig1 +
                                               n3(b2) * B * f1 * c)
    # conv2 synthesis with its ReLU + integration tail: conv2's output written + read by so3_integrate
    sig2 = B * f2 * (2 * b2) ** 3 * 4
    out["so3_inv_fused<%d>" % (2 * b2)] = n3(b2) * B * f2 * c + 2 * sig2 + B * f2 * 4
    out["so3_mm_tc_kernel"] = n3(b2) * (B * f1 + f1 * f2 + B * f2) * c
    return out


def net_flops(B):
    b1, b2, f0, f1, f2 = (NET[k] for k in ("b1", "b2", "f0", "f1", "f2"))
    c3 = b2 * b2 * (2 * b2 * b2 - 1)
    return dict(so3_mm=8 * c3 * B * f1 * f2, s2_mm=8 * n3(b1) * B * f0 * f1)


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


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU oracle on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_baseline(batch, repeats=3):
    torch.set_num_threads(os.cpu_count() or 1)
    params = oracle_params()
    x = torch.randn(batch, NET["f0"], 2 * NET["b0"], 2 * NET["b0"],
                    generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        oracle_net_forward(x[:2], params)  # fills the table caches
        oracle_net_forward(x, params)      # warm-up at full size
        best = float("inf")
        for _ in range(repeats):
            t0 = time.perf_counter()
            oracle_net_forward(x, params)
            best = min(best, time.perf_counter() - t0)
    return batch / best, best


def run_reference(args):
    world, rank, _ = dist_setup(args.gpus)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    params = oracle_params()
    batch = BATCH_PER_GPU
    x = torch.randn(batch, NET["f0"], 2 * NET["b0"], 2 * NET["b0"],
                    generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        oracle_net_forward(x[:2], params)
        for _ in range(max(1, min(args.warmup, 2))):
            oracle_net_forward(x, params)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            oracle_net_forward(x, params)
        dt = (time.perf_counter() - t0) / args.steps
    value = batch / dt
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "samples_per_sec_fwd", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "net_b30_10_6", "batch_per_step": batch,
                   "note": "CPU oracle (torch-CPU restatement of the reference's CPU branches; "
                           "the Python reference itself cannot travel to the GPU box); rank 0 only"},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": "port",
                         "sample": "%d steps of the full batch of %d" % (args.steps, batch)},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def time_steps(fn, steps, flush_buf, stream_sync):
    """Sum of per-step CUDA-event times; L2 is flushed (256 MB write) between steps, outside the
    timed intervals."""
    total = 0.0
    for _ in range(steps):
        flush_buf.zero_()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        total += a.elapsed_time(b)
    return total


def so3_fft_b64(device, hbm_gbs):
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
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a = torch.cuda.Event(enable_timing=True)
            e = torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            e.record()
            e.synchronize()
            ts.append(a.elapsed_time(e))
        res[name + "_ms"] = float(np.median(ts))
    bytes_dir = nb * (2 * b) ** 3 * 4 + n3(b) * nb * 8
    # idempotence of the round trip (the reference's own test, tests/so3_fft.py:34-44)
    y2 = so3_rifft(so3_rfft(y))
    err = ((y - y2).norm() / y2.norm()).item()
    gbs = 2 * bytes_dir / ((res["rfft_ms"] + res["rifft_ms"]) * 1e-3) / 1e9
    res.update({"workload": "so3_rfft+so3_rifft b=64 batch=64 (inputs 537 MB > L2)",
                "algorithmic_bytes_per_direction": bytes_dir,
                "roundtrip_GBps": gbs, "frac_of_hbm": gbs / hbm_gbs,
                "rfft_GBps": bytes_dir / (res["rfft_ms"] * 1e-3) / 1e9,
                "rifft_GBps": bytes_dir / (res["rifft_ms"] * 1e-3) / 1e9,
                "idempotence_rel_l2": err, "first_call_s_incl_tables": t_build})
    return res


def so3_mm_tensor(device, bf16_tf):
    """The spectral product of the widest layer of the deep model among the reference's
    configurations (SO3Conv 100 -> 100 at b_out = 10, batch 32): time of so3_mm on the tcgen05 path, algorithmic flops (8 per complex
    multiply-add) and the TF32 flops actually issued (three TF32 products per FP32 product),
    against half of the measured bf16 GEMM peak (TF32 runs at half the bf16 rate)."""
    from s2cnn_b200 import so3_mm
    nl, nb, fi, fo = 10, 32, 100, 100
    x = torch.randn(n3(nl), nb, fi, 2, device=device)
    y = torch.randn(n3(nl), fi, fo, 2, device=device)
    for _ in range(3):
        so3_mm(x, y)
    torch.cuda.synchronize()
    ts = []
    for _ in range(10):
        a = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        a.record()
        so3_mm(x, y)
        e.record()
        e.synchronize()
        ts.append(a.elapsed_time(e))
    ms = float(np.median(ts))
    flops = 8.0 * sum((2 * l + 1) ** 3 for l in range(nl)) * nb * fi * fo
    issued = 3.0 * flops / (ms * 1e-3) / 1e12
    peak = bf16_tf / 2.0
    return {"workload": "so3_mm nl=10 batch=32 f_in=100 f_out=100 (operands L2-resident)",
            "ms": ms, "algorithmic_TFLOPs": flops / (ms * 1e-3) / 1e12,
            "issued_tf32_TFLOPs": issued, "peak_tf32_TFLOPs": peak,
            "peak_source": "half of the measured bf16 GEMM peak", "frac": issued / peak}


def train_step_c4(device, batch=32, steps=5):
    """Training step (forward, cross-entropy on uniform random labels, backward) of the deep model
    among the reference's configurations, batch 32 on one GPU, synthetic input: S2Conv(6->100,
    b 64->16, max_beta pi/32) -> ReLU -> SO3Conv(100->100, b 16->10) -> ReLU -> SO3Conv(100->255,
    b 10->5) -> ReLU -> so3_integrate -> Linear(255->55).  (With several ranks the gradients would
    additionally be summed by s2cnn_b200.parallel.allreduce_gradients; not timed here.)"""
    import s2cnn_b200 as S
    g2 = S.s2_near_identity_grid(max_beta=np.pi / 32, n_alpha=8, n_beta=3)
    g3 = S.so3_near_identity_grid(max_beta=np.pi / 8, max_gamma=2 * np.pi, n_alpha=8, n_beta=3,
                                  n_gamma=8)
    torch.manual_seed(4)

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

    net = Deep().to(device)
    x = torch.randn(batch, 6, 128, 128, device=device)
    labels = torch.randint(0, 55, (batch,), device=device)

    def step():
        net.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(net(x), labels)
        loss.backward()
        return loss

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True)
    e = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step()
    e.record()
    e.synchronize()
    ms = a.elapsed_time(e) / steps
    return {"workload": "deep model 6->100->100->255->55, b 64->16->10->5, batch %d, fwd+bwd" % batch,
            "ms_per_step": ms, "samples_per_s": batch / (ms * 1e-3), "loss_finite": bool(torch.isfinite(loss))}


def run_ours(args):
    world, rank, local = dist_setup(args.gpus)
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback exists)"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    from s2cnn_b200 import _lib
    lib = _lib.cuda_lib()
    hbm_gbs, bf16_tf, peak_kind = measured_peaks()

    net = make_net(device)
    B = BATCH_PER_GPU
    gen = torch.Generator().manual_seed(1 + rank)
    x_host = torch.randn(B, NET["f0"], 2 * NET["b0"], 2 * NET["b0"], generator=gen).pin_memory()
    x_dev = x_host.to(device)
    out_host = torch.empty(B, NET["nclass"]).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    from s2cnn_b200.graph import GraphedForward
    use_graph = not args.no_graph
    graphed = GraphedForward(net, x_dev) if use_graph else None

    def step_resident():
        if use_graph:
            return graphed(x_dev)
        with torch.no_grad():
            return net(x_dev)

    def step_e2e():
        # host -> device copy of the batch, forward, device -> host read of the logits
        if use_graph:
            out_host.copy_(graphed(x_host), non_blocking=True)
            return
        with torch.no_grad():
            xd = x_host.to(device, non_blocking=True)
            out_host.copy_(net(xd), non_blocking=True)

    def step_eager():
        with torch.no_grad():
            return net(x_dev)

    for _ in range(max(args.warmup, 3)):
        step_resident()
        step_e2e()
    torch.cuda.synchronize()

    # ---- resident-input throughput (headline `value`) ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier(world)
    torch.cuda.synchronize()
    total_ms = time_steps(step_resident, args.steps, flush, None)
    torch.cuda.synchronize()
    # kernels of this library per forward pass, counted on an eager pass (a graph replay launches
    # the same kernels without going through the library's launch counter)
    n0 = lib.s2c_launch_count()
    step_eager()
    torch.cuda.synchronize()
    launches = (lib.s2c_launch_count() - n0) * args.steps
    barrier(world)
    total_ms = max_over_ranks(total_ms, world, device)
    ms_per_step = total_ms / args.steps
    value = B * world / (ms_per_step * 1e-3)

    # ---- end to end through the module API from pinned host memory ----
    barrier(world)
    torch.cuda.synchronize()
    serial_ms = time_steps(step_e2e, args.steps, flush, None) / args.steps
    torch.cuda.synchronize()
    if use_graph:
        # the same steps with the upload of batch i + 1 running behind the forward pass of batch i
        # (s2cnn_b200.graph.PipelinedForward): each timed interval holds one forward pass, one
        # result read-back and one upload (of the next batch); the L2 flush stays between intervals
        from s2cnn_b200.graph import PipelinedForward
        pipe = PipelinedForward(net, x_dev)
        for _ in range(3):
            pipe.submit(x_host, out_host)
        pipe.wait()
        pipe.prefetch(x_host)
        torch.cuda.synchronize()
        barrier(world)
        e2e_ms = 0.0
        for _ in range(args.steps):
            flush.zero_()
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
            pipe.prefetch(x_host)      # batch i + 1 -> the idle input buffer, on the copy stream
            pipe.run(out_host)         # batch i: graph replay + logits to pinned host memory
            pipe.join_uploads()        # the interval ends when the upload has landed, too
            b.record()
            b.synchronize()
            e2e_ms += a.elapsed_time(b)
        pipe.run(out_host)
        torch.cuda.synchronize()
    else:
        e2e_ms = serial_ms * args.steps
    barrier(world)
    e2e_ms = max_over_ranks(e2e_ms, world, device) / args.steps
    clocks = sampler.stop() if rank == 0 else None   # sampled over both timed legs
    e2e = {"value": B * world / (e2e_ms * 1e-3), "unit": "samples/s",
           "h2d_bytes_per_step": x_host.numel() * 4, "d2h_bytes_per_step": out_host.numel() * 4,
           "ms_per_step": e2e_ms,
           "how": ("upload of the next batch overlapped with the forward pass (two input buffers, "
                   "copy stream); every interval holds one upload, one forward, one read-back")
                  if use_graph else "upload, forward, read-back one after another",
           "serial_ms_per_step": serial_ms}

    # ---- per-kernel CUDA-event times over K more identical steps (roofline) ----
    lib.s2c_timing_begin()
    for _ in range(args.steps):
        flush.zero_()
        step_eager()
    buf = torch.zeros(1, dtype=torch.uint8)  # keep torch import used
    import ctypes
    cbuf = ctypes.create_string_buffer(1 << 16)
    lib.call("s2c_timing_end", cbuf, len(cbuf))
    per_kernel = {}
    for ln in cbuf.value.decode().splitlines():
        name, cnt, ms = ln.split()
        per_kernel[name] = (int(cnt), float(ms))
    # launch order of the FFT kernels inside one forward disambiguates conv1 / conv2 instances:
    # the bytes table lists both; time is split in proportion to algorithmic bytes.
    kb = kernel_bytes(B)
    kernels = []
    for name, (cnt, ms) in per_kernel.items():
        per_step_bytes = kb.get(name, 0)
        kernels.append({"kernel": name, "launches_per_step": cnt / args.steps,
                        "ms_per_step": ms / args.steps, "avg_launch_ms": ms / cnt,
                        "alg_bytes_per_step": per_step_bytes,
                        "GBps": per_step_bytes / (ms / args.steps * 1e-3) / 1e9 if ms > 0 else None})
    kernels.sort(key=lambda k: -k["ms_per_step"])
    top = kernels[0]
    flops = net_flops(B)
    if top["kernel"] == "so3_mm_tc_kernel":
        # dominant kernel is the spectral product: tensor roofline, TF32 dense = 1/2 bf16
        fl = flops["so3_mm"]
        ach = fl / (top["ms_per_step"] * 1e-3) / 1e12
        peak = bf16_tf / 2
        roofline = {"kernel": "so3_mm_tc_kernel", "bound": "tensor", "achieved": ach,
                    "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                    "peak_source": peak_kind + " bf16 / 2 (TF32 dense)"}
    else:
        ach = top["GBps"]
        # DRAM bytes per step of this kernel's launches from one ncu capture of this same command
        # (profiles/net_b30_10_6_launch_list.md); far below the algorithmic bytes for the fused
        # kernels, which keep the tensors at the module boundaries on chip
        traffic = {"so3_relay_fused<20>": 9.0e6 + 0.02e6, "so3_inv_fused<12>": 23.5e6,
                   "so3_inv_fused<20>": 1.5e6 + 104.7e6,
                   "so3_fwd_fused<20>": 163.9e6 + 3.8e6}.get(top["kernel"]) if B == 256 else None
        roofline = {"kernel": top["kernel"], "bound": "hbm", "achieved": ach, "peak": hbm_gbs,
                    "unit": "GB/s", "frac": ach / hbm_gbs, "traffic": traffic,
                    "peak_source": peak_kind,
                    "alg_bytes_per_step": top["alg_bytes_per_step"],
                    "launches_per_step": top["launches_per_step"]}
    roofline["timing"] = "per-launch CUDA events on the launching stream over %d steps run right " \
                         "after the timed region (launched op by op)" % args.steps

    launches_total = int(sum_over_ranks(launches, world, device))

    line = {
        "metric": "samples_per_sec_fwd", "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "net_b30_10_6", "batch_per_gpu": B, "global_batch": B * world,
                   "layers": "S2Conv(1->20,b30->10) ReLU SO3Conv(20->40,b10->6) ReLU "
                             "so3_integrate Linear(40->10)",
                   "fusion": "s2_mm + conv1 synthesis + ReLU + conv2 analysis in one kernel; second ReLU and so3_integrate inside conv2's synthesis kernel",
                   "launch": "eager" if args.no_graph else "CUDA graph replay (s2cnn_b200.graph.GraphedForward)",
                   "sharding": "batch over ranks, no collective in forward",
                   "l2": "256 MB flush write between timed steps"},
        "e2e": e2e, "gpu_launches": launches_total, "roofline": roofline,
        "kernels": kernels[:8],
    }
    if rank == 0:
        line["clocks"] = clocks
        if world == 1 and not args.skip_cpu:
            v, best = cpu_baseline(B)
            line["cpu_baseline"] = {"value": v, "unit": "samples/s",
                                    "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": "full batch of %d, best of 3 (%.2f s each)" % (B, best)}
        if world == 1 and not args.skip_fft64:
            line["so3_fft_b64"] = so3_fft_b64(device, hbm_gbs)
            line["so3_mm_tensor"] = so3_mm_tensor(device, bf16_tf)
            line["train_step_c4"] = train_step_c4(device)
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
    ap.add_argument("--skip-fft64", action="store_true")
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
