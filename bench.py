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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the two c2 kernels, from the ncu captures
# summarised in profiles/convtree_fwd_pair_c2.md and profiles/convtree_bwd_cls_c2.md
NCU_TRAFFIC = {"fwd": 38.0e6, "bwd": 105.5e6}


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
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
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

    # ---- the reference's own CUDA kernels on this GPU, when oracle/build_ref.py has built them ----
    ref_cuda = None
    if world == 1:
        try:
            from oracle.build_ref import load_ref

            rc = load_ref("convlogic_cuda")
        except Exception:
            rc = None
        if rc is not None:
            wp = torch.softmax(w, -1)
            t_f = t_b = 0.0
            nrep = 5
            for i in range(nrep + 1):
                xi, gi = xs[i % sets].detach(), gys[i % sets]
                ev[0].record()
                y_r, x2_r, x3_r, idx_r = rc.full_convlogic_forward(xi, wp, sel, 1, 1, 1, 1, 3, 3)
                ev[1].record()
                gx_r, gx2_r, gx3_r = rc.full_convlogic_backward_x(gi, xi, x2_r, x3_r, wp, idx_r, sel, 1, 1, 1, 1)
                rc.full_convlogic_backward_weight(gx2_r, gx3_r, gi, xi, x2_r, x3_r, idx_r, sel, 1, 1, 1, 1)
                ev[2].record()
                torch.cuda.synchronize()
                if i:  # first pass warms the allocator
                    t_f += ev[0].elapsed_time(ev[1])
                    t_b += ev[1].elapsed_time(ev[2])
            del y_r, x2_r, x3_r, idx_r, gx_r, gx2_r, gx3_r
            ref_cuda = {"fwd_ms": t_f / nrep, "bwd_ms": t_b / nrep, "images_per_s": C2["batch"] / ((t_f + t_b) / nrep * 1e-3),
                        "what": "lkorinek/convlogic full_convlogic_forward + backward_x + backward_weight (its CUDA extension "
                                "compiled unmodified for sm_100a), same inputs, mixture given as probabilities"}

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
    clocks = sampler.stop() if rank == 0 else None  # sampled over the device-resident, per-kernel and end-to-end regions

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
                     "peak_kind": f"of {peak_kind}", "algorithmic_bytes": alg[top], "traffic": NCU_TRAFFIC.get(top),
                     "step_frac": alg["step"] / (ms / args.steps * 1e-3) / 1e9 / peak},
        "clocks": clocks,
    }
    if ref_cuda is not None:
        out["reference_cuda_same_gpu"] = ref_cuda
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_c2(sample_batch=args.cpu_sample, passes=1)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------- secondary workloads
def _timed(fn, steps, warmup, world, dev):
    """CUDA-event time of `steps` calls of fn(i) after `warmup` calls; max over ranks; returns ms."""
    import torch.distributed as dist

    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def _finish(out, world):
    import torch.distributed as dist

    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def run_c1(args):
    """mnist_s-shaped stack (k = 16, tau 6.5) in eval mode at batch 256: the correctness configuration, timed for
    completeness -- float eval forward, packed forward and the compiled network, which must agree."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib

    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    model = cb.ConvLogicMnistModel(k_param=16, tau=6.5)
    g = torch.Generator().manual_seed(1)
    for prm in model.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    model = model.to(dev).eval()
    gi = torch.Generator().manual_seed(100 + rank)
    xb = (torch.rand(256, 1, 28, 28, generator=gi) < 0.2).to(dev)
    xf = xb.float()
    cnet = cb.CompiledLogicNet(model.network, input_shape=(1, 28, 28)).compile()
    with torch.no_grad():
        counts = model(cb.PackBitsTensor(xb, 64))
        agree = bool(torch.equal(counts, cnet(xb))) and bool(torch.equal((model(xf) * 6.5).round().int(), counts))
    lib = _lib.lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    def fwd_float(i):
        with torch.no_grad():
            model(xf)

    def fwd_packed(i):
        with torch.no_grad():
            model(cb.PackBitsTensor(xb, 64))

    l0 = lib.clb_kernel_launches()
    ms = _timed(fwd_float, args.steps, args.warmup, world, dev)
    launches = (lib.clb_kernel_launches() - l0) * args.steps // (args.steps + args.warmup)
    ms_p = _timed(fwd_packed, args.steps, 3, world, dev)
    ms_c = _timed(lambda i: cnet(xb), args.steps, 3, world, dev)
    replay = cnet.capture(xb)
    graph_ok = bool(torch.equal(replay(xb), counts))
    ms_g = _timed(lambda i: replay(xb), args.steps, 3, world, dev)
    clocks = sampler.stop() if rank == 0 else None
    _finish({
        "metric": "eval imgs/sec, mnist_s-shaped LogicTreeNet (float eval forward)", "value": 256 * world * args.steps / (ms * 1e-3),
        "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c1: mnist_s-shaped stack (k=16, tau=6.5), eval mode, batch 256 of 1x28x28 Bernoulli(0.2) bits",
                   "l2": "launch-bound: every tensor fits the L2", "parallelism": f"{world} independent replicas"},
        "packed_ms": ms_p / args.steps, "compiled_net_ms": ms_c / args.steps, "compiled_net_graph_ms": ms_g / args.steps,
        "paths_agree": agree and graph_ok,
        "gpu_launches": int(launches), "clocks": clocks}, world)


def run_c3(args):
    """cifar10_m-shaped full training step: soft forward, cross-entropy, backward, Adam(lr 0.01); batch 256
    per GPU; data-parallel with one all-reduce of the flat gate-logit gradient bucket."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib, dp

    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    net = cb.ConvLogicCifarModel(k_param=256, input_channels=9, input_size=32, tau=40).network
    g = torch.Generator().manual_seed(1)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    net = cb.fuse_logic_layers(net.to(dev)).train()  # the three flat layers run as one gate tree per output neuron (same parameters)
    bucket = dp.GradBucket(net).overlap(average=True)  # a layer's slice is all-reduced while the layers in front of it run backward
    opt = torch.optim.Adam(net.parameters(), lr=0.01, fused=True)
    sets = 4
    gi = torch.Generator().manual_seed(100 + rank)
    xs_h = [(torch.rand(256, 9, 32, 32, generator=gi) < 0.5).float().pin_memory() for _ in range(sets)]
    ls_h = [torch.randint(0, 10, (256,), generator=gi).pin_memory() for _ in range(sets)]
    xs, ls = [x.to(dev) for x in xs_h], [l.to(dev) for l in ls_h]
    loss_host = torch.zeros(1).pin_memory()

    def step(i, host=False):
        x = xs_h[i % sets].to(dev, non_blocking=True) if host else xs[i % sets]
        lab = ls_h[i % sets].to(dev, non_blocking=True) if host else ls[i % sets]
        bucket.zero()
        loss = torch.nn.functional.cross_entropy(net(x), lab)
        loss.backward()
        bucket.finish()
        opt.step()
        if host:
            loss_host.copy_(loss.detach().reshape(1), non_blocking=True)

    lib = _lib.lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = lib.clb_kernel_launches()
    ms = _timed(step, args.steps, args.warmup, world, dev)
    launches = (lib.clb_kernel_launches() - l0) * args.steps // (args.steps + args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = _timed(lambda i: step(i, host=True), args.steps, 3, world, dev)
    imgs = 256 * world * args.steps
    peak, kind = measured_peaks()
    step_bytes = 15.80e6 * 256 + 0.47e9  # algorithmic bytes of one step (activations + parameter/Adam traffic)
    _finish({
        "metric": "train imgs/sec (fwd+bwd+Adam), cifar10_m-shaped LogicTreeNet", "value": imgs / (ms * 1e-3), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c3: cifar10_m-shaped stack (k=256, tau=40), 9x32x32 Bernoulli(0.5) bits, batch 256 per GPU, Adam lr 0.01",
                   "l2": "activations of one step (~1.5 GB) exceed the 126 MB L2", "parameters": bucket.numel,
                   "parallelism": f"dp{world}, per-layer all-reduces of the gate-logit gradients ({bucket.numel * 4 / 1e6:.1f} MB per step) overlapped with backward" if world > 1 else "single GPU"},
        "e2e": {"value": imgs / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": 256 * 9 * 32 * 32 * 4 + 256 * 8,
                "d2h_bytes_per_step": 4},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": step_bytes / (ms / args.steps * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": step_bytes / (ms / args.steps * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}", "traffic": None,
                     "note": "whole step, algorithmic bytes 4.52 GB"},
        "clocks": clocks}, world)


def run_c4(args):
    """cifar10_l-shaped discretised inference on bit-packed activations (64 images per word), the batch of
    2^20 images sharded over the ranks and streamed in chunks; no collective."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib, dp, ops

    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    net = cb.ConvLogicCifarModel(k_param=1024, input_channels=93, input_size=32, tau=340).network
    g = torch.Generator().manual_seed(1)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    net = net.to(dev).eval()
    total = args.images
    lo, hi = dp.shard_range(total, rank, world)
    chunk = args.chunk
    n_chunks = (hi - lo + chunk - 1) // chunk
    resident = min(n_chunks, 16)
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    th = torch.arange(1, 32, device=dev, dtype=torch.float32) / 32  # channel 3*(i-1)+c holds pixel[c] > i/32
    # resident inputs: uint8 pixel chunks (16 x 25 MB, beyond the L2); the thermometer + pack stage is part of the pipeline
    hgen = torch.Generator().manual_seed(2000 + rank)
    host_px = [torch.randint(0, 256, (chunk, 3, 32, 32), dtype=torch.uint8, generator=hgen).pin_memory() for _ in range(2)]
    pixels = [torch.randint(0, 256, (chunk, 3, 32, 32), dtype=torch.uint8, device=dev, generator=gen) for _ in range(resident)]
    # the public call: the stack serialised once and run by the library's runtime, one C call per chunk
    cnet = cb.CompiledLogicNet(net, input_shape=(93, 32, 32)).compile()
    # end to end: uint8 pixels in pinned host memory -> device (copy stream, double-buffered) -> the compiled network
    # -> class index -> pinned host memory
    dev_px = [torch.empty((chunk, 3, 32, 32), dtype=torch.uint8, device=dev) for _ in range(2)]
    host_out = torch.empty((n_chunks, chunk), dtype=torch.int64).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def step(i):
        for j in range(n_chunks):
            cnet.forward_pixels(pixels[(i * n_chunks + j) % resident], th).argmax(-1)

    def fetch(j):
        b = j % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[b])
            dev_px[b].copy_(host_px[b], non_blocking=True)
            arrived[b].record(copy_stream)

    def step_e2e(i):
        cur = torch.cuda.current_stream(dev)
        for b in range(2):
            consumed[b].record(cur)
        fetch(0)
        for j in range(n_chunks):
            if j + 1 < n_chunks:
                fetch(j + 1)
            b = j % 2
            cur.wait_event(arrived[b])
            counts = cnet.forward_pixels(dev_px[b], th)
            consumed[b].record(cur)
            host_out[j].copy_(counts.argmax(-1), non_blocking=True)
        cur.synchronize()

    lib = _lib.lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = lib.clb_kernel_launches()
    steps = max(1, min(args.steps, 5))
    ms = _timed(step, steps, 1, world, dev)
    launches = (lib.clb_kernel_launches() - l0) * steps // (steps + 1)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = _timed(step_e2e, 1, 1, world, dev)
    # beside it: the same stack layer by layer through the nn.Modules (PackBitsTensor path), per-layer times of one chunk
    layer_ms, module_path = [], None
    if rank == 0:
        with torch.no_grad():
            p0 = cb.PackBitsTensor.from_pixels(pixels[0], th)
            same = bool(torch.equal(cnet.forward_pixels(pixels[0], th), net(p0)))
            ms_m = _timed(lambda i: net(cb.PackBitsTensor.from_pixels(pixels[i % resident], th)), 3, 1, 1, dev) / 3
            h = p0
            for m in net:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                o = m(h)
                e1.record()
                torch.cuda.synchronize()
                layer_ms.append(round(e0.elapsed_time(e1), 4))
                h = o
        module_path = {"ms_per_chunk": round(ms_m, 4), "images_per_s": chunk / (ms_m * 1e-3), "equals_compiled_net": same,
                       "layer_ms_per_chunk": layer_ms, "what": "nn.Sequential of ConvLogicLayer / LogicLayer / GroupSum on PackBitsTensor"}
    imgs = total * steps
    peak, kind = measured_peaks()
    alg = 1388200.0 * total / world  # layer-by-layer algorithmic bytes per image, per rank and step
    _finish({
        "metric": "packed-inference imgs/sec, cifar10_l-shaped LogicTreeNet", "value": imgs / (ms * 1e-3), "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": 1, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": {"workload": f"c4: cifar10_l-shaped stack (k=1024), {total} images of 93x32x32 thermometer bits, 64 per word, "
                               f"chunks of {chunk}, CompiledLogicNet.forward_pixels on uint8 pixels",
                   "l2": f"{resident} resident uint8 pixel chunks (~{resident * 3072 * chunk / 1e9:.2f} GB); every chunk's activations exceed the L2",
                   "parallelism": f"batch sharded over {world} ranks, no collective"},
        "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": 3 * 1024 * (hi - lo),
                "d2h_bytes_per_step": (hi - lo) * 8,
                "what": "uint8 pixels from pinned host memory, the compiled network on the GPU, class indices back to the host"},
        "gpu_launches": int(launches), "blob_bytes": len(cnet.blob), "module_path": module_path,
        "roofline": {"bound": "hbm", "achieved": alg / (ms / steps * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / (ms / steps * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}", "traffic": None,
                     "note": "whole pipeline, 1 388 200 algorithmic bytes per image"},
        "clocks": clocks}, world)


def run_c5(args):
    """Flat difflogic stack: 3072 -> 8 x 256000 LogicLayers -> GroupSum(10, tau=100), batch 1024, fwd + bwd."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib

    world, rank, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    dims = [3072] + [256000] * 8
    net = torch.nn.Sequential(*[cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])], cb.GroupSum(10, 100.0)).to(dev).train()
    gi = torch.Generator().manual_seed(100 + rank)
    x = (torch.rand(1024, 3072, generator=gi) < 0.5).float().to(dev)
    gy = torch.randn(1024, 10, generator=gi).to(dev)

    def step(i):
        for prm in net.parameters():
            prm.grad = None
        net(x).backward(gy)
        if world > 1:
            from convlogic_b200 import dp
            dp.allreduce_gate_gradients(net)

    lib = _lib.lib()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    steps = max(1, min(args.steps, 20))
    l0 = lib.clb_kernel_launches()
    ms = _timed(step, steps, 3, world, dev)
    launches = (lib.clb_kernel_launches() - l0) * steps // (steps + 3)
    clocks = sampler.stop() if rank == 0 else None
    # one 256000 -> 256000 layer, ours and (when built) the reference's CUDA kernels, same tensors
    layer_cmp = None
    if world == 1:
        from convlogic_b200 import ops
        from convlogic_b200._lib import W_PROB

        lay = net[1]
        xf = torch.rand(256000, 1024, device=dev)
        gyf = torch.randn(256000, 1024, device=dev)
        wp = torch.softmax(lay.weights.detach(), -1)
        a_, b_, st_, cs_ = lay.indices_0, lay.indices_1, lay.given_x_indices_of_y_start, lay.given_x_indices_of_y

        def t3(fwd, bw, bx):
            out = []
            for fn in (fwd, bw, bx):
                fn()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(3):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                out.append(round(e0.elapsed_time(e1) / 3, 4))
            return out

        layer_cmp = {"ours_ms_fwd_bwdw_bwdx": t3(lambda: ops.logic_fwd(xf, a_, b_, wp, W_PROB), lambda: ops.logic_bwd_w(xf, a_, b_, wp, gyf, W_PROB),
                                                  lambda: ops.logic_bwd_x(xf, a_, b_, wp, gyf, st_, cs_, W_PROB))}
        try:
            from oracle.build_ref import load_ref

            rf = load_ref("difflogic_cuda")
        except Exception:
            rf = None
        if rf is not None:
            layer_cmp["reference_cuda_ms_fwd_bwdw_bwdx"] = t3(lambda: rf.forward(xf, a_, b_, wp), lambda: rf.backward_w(xf, a_, b_, gyf),
                                                              lambda: rf.backward_x(xf, a_, b_, wp, gyf, st_, cs_))
        del xf, gyf
    peak, kind = measured_peaks()
    alg = 39.9e9
    _finish({
        "metric": "train samples/sec (fwd+bwd), flat difflogic stack", "value": 1024 * world * steps / (ms * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c5: 8 LogicLayers 3072->256000x8 + GroupSum(10, tau=100), batch 1024, fwd+bwd",
                   "l2": "every activation is 1.05 GB (> 126 MB L2)"},
        "gpu_launches": int(launches),
        "roofline": {"bound": "hbm", "achieved": alg / (ms / steps * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": alg / (ms / steps * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}", "traffic": None,
                     "note": "whole step, 39.9 GB algorithmic"},
        "one_layer_256000x1024": layer_cmp,
        "clocks": clocks}, world)


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
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--images", type=int, default=1 << 20, help="c4: total images")
    ap.add_argument("--chunk", type=int, default=8192, help="c4: images per streamed chunk")
    ap.add_argument("--cpu-sample", type=int, default=32)
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        {"c1": run_c1, "c2": run_ours, "c3": run_c3, "c4": run_c4, "c5": run_c5}[args.workload](args)


if __name__ == "__main__":
    main()
