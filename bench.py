"""Benchmark of the logic-gate hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

Workload ``c2`` (default; the configuration the headline metric is quoted on): one fused ConvLogic
block, forward + backward, fp32, batch 256 per GPU, 9 binary input channels 32x32 (Bernoulli 0.5),
256 output kernels, 3x3 window, padding 1, N(0,1) gate logits, N(0,1) upstream gradient.
One "step" = soft forward, input gradient and gate-logit gradient of one batch; with N > 1 every
rank runs its own batch (weak scaling) and the logit gradients are all-reduced over NCCL.

Printed JSON (one line, rank 0):
  value      images/s over all GPUs with inputs resident in HBM, public module API
             (``layer(x)`` + ``backward``), CUDA-event timed, max over ranks.
  e2e        the same step fed from pinned host memory: x and the upstream gradient are copied
             host->device and the input/logit gradients device->host inside the timed region
             (copies run on a second stream, double-buffered against compute).
  roofline   dominant kernel of the step, algorithmic bytes / measured duration vs the measured
             HBM copy bandwidth.
  cpu_baseline  the CPU oracle (a port of the reference's ``implementation="python"`` path) timed on
             this host on a bounded sample.
``--impl reference`` times that CPU port alone as the reference arm (the reference's CPU path is
Python that cannot travel to the GPU box; the port follows it line by line, see oracle/).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

C2 = dict(batch=256, cin=9, cout=256, size=32)


# ------------------------------------------------------------------------------------------ utils
def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                return float(json.load(f)["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


# ------------------------------------------------------------------------------------ workload c2
def make_c2_inputs(seed, device, sets):
    g = torch.Generator().manual_seed(seed)
    b, ci, c, s = C2["batch"], C2["cin"], C2["cout"], C2["size"]
    xs = [(torch.rand(b, ci, s, s, generator=g) < 0.5).float() for _ in range(sets)]
    gys = [torch.randn(b, c, s // 2, s // 2, generator=g) for _ in range(sets)]
    return xs, gys


def c2_layer(device):
    import convlogic_b200 as cb

    torch.manual_seed(0)
    layer = cb.ConvLogicLayer(C2["cin"], C2["cout"], padding=1, complete=True)
    layer.weights.data = torch.randn(C2["cout"], 7, 16, generator=torch.Generator().manual_seed(1))
    return layer.to(device).train()


def c2_algorithmic_bytes():
    b, ci, c, s = C2["batch"], C2["cin"], C2["cout"], C2["size"]
    x = b * ci * s * s * 4
    y = b * c * (s // 2) ** 2 * 4
    w, sel = c * 7 * 16 * 4, c * 8 * 4
    return {"fwd": x + y + w + sel, "bwd": y + x + x + 2 * w + sel, "step": (x + y + w + sel) + (y + x + x + 2 * w + sel)}


def run_ours(args):
    import torch.distributed as dist

    from convlogic_b200 import _lib, ops
    from convlogic_b200._lib import W_SOFTMAX

    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    layer = c2_layer(dev)
    sets = 3  # rotating input sets: ~150 MB each, so every step streams from HBM, not from the 126 MB L2
    xs_h, gys_h = make_c2_inputs(100 + rank, dev, sets)
    xs = [x.to(dev) for x in xs_h]
    gys = [g.to(dev) for g in gys_h]
    lib = _lib.lib()

    def step(i, sync_grads=True):
        x = xs[i % sets].requires_grad_(True)
        x.grad = None
        layer.weights.grad = None
        y = layer(x)
        y.backward(gys[i % sets])
        if world > 1 and sync_grads:
            dist.all_reduce(layer.weights.grad)
        return x.grad, layer.weights.grad

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    # ---- device-resident timing (value) ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = lib.clb_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches = lib.clb_kernel_launches() - launches0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- per-kernel timing on the same stream (roofline) ----
    geom = (1, 1, 1, 1, 3, 3)
    w = layer.weights.detach()
    sel = layer.selection
    kern_ms = {}
    reps = max(args.steps, 10)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    y, amax, _, _, _ = ops.convtree_fwd(xs[0], w, sel, geom, W_SOFTMAX)
    amaxes = []
    for i in range(sets):
        amaxes.append(ops.convtree_fwd(xs[i].detach(), w, sel, geom, W_SOFTMAX)[1])
    torch.cuda.synchronize()
    for name, fn in (
        ("fwd", lambda i: ops.convtree_fwd(xs[i % sets].detach(), w, sel, geom, W_SOFTMAX)),
        ("bwd", lambda i: ops.convtree_bwd(gys[i % sets], xs[i % sets].detach(), w, sel, amaxes[i % sets], geom, W_SOFTMAX)),
    ):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        ev[0].record()
        for i in range(reps):
            fn(i)
        ev[1].record()
        torch.cuda.synchronize()
        kern_ms[name] = ev[0].elapsed_time(ev[1]) / reps
    clocks = sampler.stop() if rank == 0 else None

    # ---- end-to-end: host buffers in, gradients out, copies inside the timed region ----
    xs_p = [x.pin_memory() for x in xs_h]
    gys_p = [g.pin_memory() for g in gys_h]
    gx_host = [torch.empty_like(xs_h[0]).pin_memory() for _ in range(2)]
    gw_host = [torch.empty(C2["cout"], 7, 16).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()
    x_dev = [torch.empty_like(xs[0]) for _ in range(2)]
    gy_dev = [torch.empty_like(gys[0]) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        s = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[s])
            x_dev[s].copy_(xs_p[i % sets], non_blocking=True)
            gy_dev[s].copy_(gys_p[i % sets], non_blocking=True)
            ready[s].record(copy_stream)

    def e2e_loop(n):
        for s in range(2):
            consumed[s].record(main)
        upload(0)
        for i in range(n):
            s = i % 2
            if i + 1 < n:
                upload(i + 1)
            main.wait_event(ready[s])
            x = x_dev[s].requires_grad_(True)
            x.grad = None
            layer.weights.grad = None
            layer(x).backward(gy_dev[s])
            if world > 1:
                dist.all_reduce(layer.weights.grad)
            gx_host[s].copy_(x.grad, non_blocking=True)
            gw_host[s].copy_(layer.weights.grad, non_blocking=True)
            consumed[s].record(main)
            x_dev[s].requires_grad_(False)

    e2e_loop(max(3, args.warmup))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    e2e_loop(args.steps)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = measured_peaks()
    alg = c2_algorithmic_bytes()
    top = max(kern_ms, key=kern_ms.get)
    achieved = alg[top] / (kern_ms[top] * 1e-3) / 1e9
    imgs = C2["batch"] * world * args.steps
    h2d = xs_h[0].numel() * 4 + gys_h[0].numel() * 4
    d2h = xs_h[0].numel() * 4 + C2["cout"] * 7 * 16 * 4
    out = {
        "metric": "train imgs/sec (fwd+bwd), single ConvLogic block", "value": imgs / (ms * 1e-3), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c2: ConvLogicLayer(9->256, 3x3, pad 1, complete) fwd+bwd, batch 256 per GPU, 32x32 Bernoulli(0.5) input",
                   "l2": f"{sets} rotating input sets of ~153 MB each (> 126 MB L2)",
                   "parallelism": f"dp{world}, all-reduce of gate-logit gradients" if world > 1 else "single GPU"},
        "e2e": {"value": imgs / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches),
        "kernel_ms": {k: round(v, 5) for k, v in kern_ms.items()},
        "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "algorithmic_bytes": alg[top], "traffic": None,
                     "step_frac": alg["step"] / (ms / args.steps * 1e-3) / 1e9 / peak},
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_c2(sample_batch=args.cpu_sample, passes=1)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------- CPU baseline
def cpu_baseline_c2(sample_batch, passes):
    """The CPU oracle (port of the reference's Python path) on `sample_batch` images of workload c2."""
    import oracle

    torch.manual_seed(0)
    import convlogic_b200 as cb

    layer = cb.ConvLogicLayer(C2["cin"], C2["cout"], padding=1, complete=True)
    sel = layer.selection
    g = torch.Generator().manual_seed(1)
    w = torch.randn(C2["cout"], 7, 16, generator=g).requires_grad_(True)
    best = None
    for _ in range(passes + 1):  # first pass warms the allocator
        x = (torch.rand(sample_batch, C2["cin"], C2["size"], C2["size"], generator=g) < 0.5).float().requires_grad_(True)
        gy = torch.randn(sample_batch, C2["cout"], C2["size"] // 2, C2["size"] // 2, generator=g)
        t0 = time.perf_counter()
        y = oracle.full_convlogic(x, oracle.gate_probabilities(w, True), sel)[0]
        torch.autograd.grad((y * gy).sum(), (x, w))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": sample_batch / best, "unit": "images/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_batch} of the 256 images per step, forward + autograd backward, torch CPU tensors, "
                      f"{os.cpu_count()} logical CPUs"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, args.steps)
    sample = args.cpu_sample
    t_all = []
    base = None
    for _ in range(min(steps, 5)):
        base = cpu_baseline_c2(sample_batch=sample, passes=1)
        t_all.append(sample / base["value"])
    sec = statistics.median(t_all)
    value = sample / sec
    out = {
        "impl": "reference", "metric": "train imgs/sec (fwd+bwd), single ConvLogic block", "value": value, "unit": "images/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": len(t_all), "warmup": 1, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c2: ConvLogicLayer(9->256, 3x3, pad 1, complete) fwd+bwd, batch 256 per GPU, 32x32 Bernoulli(0.5) input",
                   "note": "CPU port of the reference's implementation='python' path; each step is a bounded sample"},
        "cpu_baseline": dict(base, value=value),
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2"])
    ap.add_argument("--cpu-sample", type=int, default=32)
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
