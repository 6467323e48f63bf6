"""Benchmark of the logic-gate hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c1|c2|c3|c4|c5] [--impl ours|reference]

The printed line (one JSON object, rank 0) is the record of workload c3, the configuration the training half of
the headline metric is quoted on: the cifar10_m-shaped LogicTreeNet, one full training step (soft forward,
cross-entropy, backward, Adam lr 0.01) at batch 256 per GPU, data-parallel with an all-reduce of the gate-logit
gradients.  With ``--workload all`` (the default) the same line carries three nested records:

  packed_inference  workload c4, the other half of the metric: the cifar10_l-shaped stack, discretised, bit-packed
                    64 images per word, 2^20 images sharded over the ranks with no collective;
  microbench_c2     one fused ConvLogic block 9 -> 256 at 32x32, forward + backward, batch 256;
  flat_c5           eight flat LogicLayers of 256 000 neurons + GroupSum, forward + backward, batch 1024.

Keys of every record:
  value      whole-job throughput with the inputs resident in HBM, through the public module API, CUDA-event
             timed, maximum over ranks.
  e2e        the same work fed from pinned host memory, the host->device copies of the inputs and the
             device->host read of the result inside the timed region.
  roofline   the step's slowest kernel: algorithmic bytes / its CUDA-event time (events recorded by the library
             around each of its launches, on the launching stream) against the measured HBM copy bandwidth;
             ``kernels`` lists the five slowest the same way, ``step_frac`` does it for the whole step.
  cpu_baseline  the CPU oracle (a port of the reference's ``implementation="python"`` path) on this host's cores,
             on a bounded sample of the same step.
``--impl reference`` times that CPU port alone as the reference arm: every step is a bounded sample of the c3
training step (the reference's own CPU path is Python that needs the reference checkout; the port follows it
function by function, see oracle/).
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


def host_cores():
    """Cores this process may run on (the cgroup / affinity count, not the machine's)."""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, active=True):
        self.index, self.proc, self.lines, self.active = index, None, [], active

    def start(self):
        if not self.active:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.active:
            return None
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


class Ctx:
    """One process per GPU: rank, device and the NCCL group (world > 1), set up once for all workloads."""

    def __init__(self):
        import torch.distributed as dist

        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # The gradient exchange (42.8 MB per step at c3) runs under the backward kernels: on 2 and 4 GPUs NCCL's default
            # number of blocks takes SMs from them for longer than the transfer needs.  Measured c3 ms/step, default / 16 / 8 / 4
            # blocks: 2.46 / 2.42 / 2.42 / 2.52 on 2 GPUs, 2.47 / 2.46 / 2.43 / - on 4.  On 8 GPUs the ring is longer and 8
            # blocks are too few: default / 32 / 16 / 12 / 8 blocks 2.366 / 2.365 / 2.365 / 2.356 / 2.439 ms (2.27 on one GPU).
            # A value the caller set wins.
            os.environ.setdefault("NCCL_MAX_CTAS", "8" if self.world <= 4 else "12")
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        else:
            torch.cuda.set_device(0)
        self.dev = torch.device("cuda", self.local)
        self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, ms):
        if self.world > 1:
            t = torch.tensor([ms], device=self.dev, dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def timed(self, fn, steps, warmup):
        """CUDA-event time (ms) of `steps` calls of fn(i) after `warmup` untimed calls, bracketed by a barrier and a
        device synchronisation on both sides; maximum over ranks."""
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        self.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t0 = time.perf_counter()
        for i in range(steps):
            fn(i)
        self.host_ms = (time.perf_counter() - t0) * 1e3   # host time to enqueue the timed steps (no device wait unless fn has one)
        e1.record()
        torch.cuda.synchronize()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1))

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def traced(fn, steps):
    """Runs fn(i) `steps` times with the library's launch tracing on; {kernel: (launches per step, ms per step)}."""
    from convlogic_b200 import _lib

    torch.cuda.synchronize()
    _lib.trace(True)
    for i in range(steps):
        fn(i)
    torch.cuda.synchronize()
    rep = _lib.trace_report()
    _lib.trace(False)
    return {k: (n / steps, ms / steps) for k, (n, ms) in rep.items()}


# DRAM bytes (read + write) ncu counted for each kernel, summed over the kernel's launches in ONE step (c3, c2, c5) or
# one 8192-image chunk (c4) of the default workload sizes: dram__bytes.sum over one capture of the same bench command
# per workload (c5: the 64 000-neuron case of the same kernels, scaled by 4 to 256 000 neurons; its traffic grows with
# the neuron count).  Other sizes report null.
NCU_TRAFFIC = {
    "c3": {"convtree_bwd_plane_kernel": 1930.7e6, "plane_sum_kernel": 1526.9e6, "logic_tree_bwd_kernel": 954.8e6,
           "row_segment_sum_kernel": 706.5e6, "convtree_fwd_plane_kernel": 383.1e6, "adam_step_kernel": 245.7e6,
           "logic_tree_fwd_sum_kernel": 92.1e6, "convtree_bwd_w_plane32_kernel": 97.8e6, "convtree_fwd_pair_kernel": 37.7e6},
    "c4": {"packed_convtree_slab_kernel": 2317.2e6, "packed_tree_kernel": 1639.4e6, "group_popcount_kernel": 676.1e6,
           "packed_rows_to_slab_kernel": 223.9e6, "thermometer_pack_kernel": 65.1e6},
    "c2": {"convtree_fwd_pair_kernel": 37.3e6, "convtree_bwd_cls_kernel": 105.4e6, "convtree_bwd_post_kernel": 33.1e6},
    "c5": {"logic_bwd_x_kernel": 7 * 4 * 1254.0e6, "logic_bwd_w_kernel": 7 * 4 * 741.0e6 + 4 * 288.5e6,
           "logic_fwd_kernel": 7 * 4 * 707.5e6 + 4 * 227.0e6},
}


def kernel_table(trace, alg_bytes, peak, top=5, traffic=None):
    """The `top` slowest kernels of a traced step with their algorithmic bytes, HBM fraction and measured DRAM traffic."""
    rows = []
    for name, (launches, ms) in sorted(trace.items(), key=lambda kv: -kv[1][1])[:top]:
        b = alg_bytes.get(name)
        row = {"kernel": name, "launches_per_step": round(launches, 2), "ms_per_step": round(ms, 5), "algorithmic_bytes": b,
               "traffic": (traffic or {}).get(name)}
        if b:
            row["achieved_gbs"] = b / (ms * 1e-3) / 1e9
            row["frac"] = row["achieved_gbs"] / peak
        rows.append(row)
    return rows


# ------------------------------------------------------------------------------------ workload c3
C3_BATCH = 256
C3_WORKLOAD = ("c3: cifar10_m-shaped LogicTreeNet (k=256, tau=40: ConvLogic blocks 9->256->1024->4096->8192 on 32x32..4x4, "
               "LogicLayers 32768->327680->163840->81920, GroupSum 10), full training step (soft fwd + cross-entropy + bwd + "
               "Adam lr 0.01), fp32, batch 256 per GPU, 9x32x32 Bernoulli(0.5) bits, uniform labels")


def c3_config(world):
    return {"workload": C3_WORKLOAD,
            "l2": "4 rotating input sets; one step's activations (~1.5 GB) exceed the 126 MB L2",
            "parallelism": f"dp{world}: batch-sharded replicas, per-layer NCCL all-reduces of the gate-logit gradients "
                           f"(42.8 MB per step) overlapped with the backward pass, NCCL_MAX_CTAS={os.environ.get('NCCL_MAX_CTAS')}"
                           if world > 1 else "single GPU"}


def c3_algorithmic_bytes(batch):
    """Per step and kernel: every distinct input read once + every output written once (fp32), no intermediates."""
    x1, y1, y2, y3, y4 = 9 * 32 * 32 * 4, 256 * 16 * 16 * 4, 1024 * 8 * 8 * 4, 4096 * 4 * 4 * 4, 8192 * 2 * 2 * 4
    fin, fout = 32768 * 4, 81920 * 4
    per_image = {
        "convtree_fwd_pair_kernel": x1 + y1,
        "convtree_fwd_tile_kernel": x1 + y1,
        "convtree_fwd_chan_pair_kernel": (y1 + y2) + (y2 + y3) + (y3 + y4),
        "convtree_fwd_chan_kernel": (y1 + y2) + (y2 + y3) + (y3 + y4),
        "convtree_bwd_cls_kernel": y1 + x1,
        "convtree_bwd_w_plane32_kernel": y1 + x1,
        "convtree_fwd_plane_kernel": (y1 + y2) + (y2 + y3) + (y3 + y4),
        "convtree_bwd_plane_kernel": (y2 + y1) + (y3 + y2) + (y4 + y3),            # upstream gradient + input
        "plane_sum_kernel": y1 + y2 + y3,                                           # the input gradients
        "convtree_bwd_w_win_kernel<tapgrad>": (y2 + y1) + (y3 + y2) + (y4 + y3),   # upstream gradient + input
        "convtree_bwd_x_scatter_kernel": y1 + y2 + y3,                              # the input gradients
        "adam_step_kernel": 7 * 4 * 10694656 // batch,   # p, g, m, v read; p, m, v written (per step, not per image)
        "logic_tree_fwd_kernel": fin + fout,
        "logic_tree_fwd_sum_kernel": fin,          # class sums instead of the activation: only the input is moved
        "logic_tree_bwd_kernel": fout + fin,
        "row_segment_sum_kernel": fin,
        "transpose_f32_kernel": 4 * fin,   # [batch, features] <-> [features, batch] in front of the flat part: two copies, read + write
    }
    out = {k: v * batch for k, v in per_image.items()}
    out["step"] = 15.80e6 * batch + 0.47e9   # activations + parameter / Adam traffic
    return out


def build_c3(dev):
    import convlogic_b200 as cb

    torch.manual_seed(0)
    net = cb.ConvLogicCifarModel(k_param=256, input_channels=9, input_size=32, tau=40).network
    g = torch.Generator().manual_seed(1)
    for prm in net.parameters():
        prm.data = torch.randn(*prm.shape, generator=g)
    return net.to(dev)


def run_c3(ctx, args, with_cpu=True):
    """cifar10_m-shaped full training step; data-parallel with the overlapped all-reduce of the flat logit-gradient bucket."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib, dp

    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    net = cb.fuse_logic_layers(build_c3(dev), feature_major_blocks=not args.no_feature_major).train()   # the three flat layers run as one gate tree per output neuron
    if args.torch_tail:   # torch's cross-entropy, gradient accumulation and fused Adam behind the library's layers
        bucket = dp.GradBucket(net).overlap(average=True)
        opt = torch.optim.Adam(net.parameters(), lr=0.01, fused=True)
    else:                 # the library's own tail: GroupSum + cross-entropy kernel, gradients written into the bucket, flat Adam
        if isinstance(net[-2], cb.FusedLogicLayers) and not args.separate_head:
            # the fused flat layers and the loss head as one autograd node (the gradient tensor between them is never written)
            body, trees, gs = net[:-2], net[-2], net[-1]
            head = lambda feats, lab: trees.cross_entropy(feats, lab, gs.k, gs.tau)  # noqa: E731
        else:
            body, head = net[:-1], cb.GroupSumCrossEntropy(net[-1].k, net[-1].tau)
        bucket = dp.GradBucket(net).direct().overlap(average=True)
        opt = cb.FlatAdam(bucket, lr=0.01)
    sets = 4
    gi = torch.Generator().manual_seed(100 + rank)
    bits_h = [(torch.rand(C3_BATCH, 9, 32, 32, generator=gi) < 0.5).to(torch.uint8).pin_memory() for _ in range(sets)]
    labs_h = [torch.randint(0, 10, (C3_BATCH,), generator=gi).pin_memory() for _ in range(sets)]
    xs, labs = [b.to(dev).float() for b in bits_h], [l.to(dev) for l in labs_h]
    loss_host = torch.zeros(1).pin_memory()

    def train_step(x, lab):
        if args.torch_tail:
            bucket.zero()
            loss = torch.nn.functional.cross_entropy(net(x), lab)
        else:
            loss = head(body(x), lab)
        loss.backward()
        if args.torch_tail:
            bucket.finish()
            opt.step()
        else:
            opt.finish_and_step()   # the update of all but the last-exchanged slice runs under that exchange
        return loss

    def step(i):
        train_step(xs[i % sets], labs[i % sets])

    # end to end: the binary input travels as uint8 (9 KB per image) from pinned host memory on a copy stream, one step
    # ahead of the compute; the loss goes back to the host every step
    copy_stream = torch.cuda.Stream(device=dev)
    stage = [(torch.empty((C3_BATCH, 9, 32, 32), dtype=torch.uint8, device=dev), torch.empty(C3_BATCH, dtype=torch.int64, device=dev))
             for _ in range(2)]
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def upload(i):
        s = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[s])
            stage[s][0].copy_(bits_h[i % sets], non_blocking=True)
            stage[s][1].copy_(labs_h[i % sets], non_blocking=True)
            arrived[s].record(copy_stream)

    state = {"k": None}

    def step_e2e(_):
        cur = torch.cuda.current_stream(dev)
        if state["k"] is None:      # first call: nothing is in flight yet
            for s in range(2):
                consumed[s].record(cur)
            upload(0)
            state["k"] = 0
        k = state["k"]
        upload(k + 1)               # the next step's input travels while this step computes
        s = k % 2
        cur.wait_event(arrived[s])
        loss = train_step(stage[s][0].float(), stage[s][1])
        consumed[s].record(cur)
        loss_host.copy_(loss.detach().reshape(1), non_blocking=True)
        state["k"] = k + 1

    lib = _lib.lib()
    sampler = ClockSampler(ctx.local, rank == 0).start()
    ms = ctx.timed(step, args.steps, args.warmup)
    host_ms = ctx.host_ms
    l0 = lib.clb_kernel_launches()
    step(0)
    launches = lib.clb_kernel_launches() - l0
    trace = traced(step, max(3, min(args.steps, 10)))
    ms_e2e = ctx.timed(step_e2e, args.steps, 3)
    clocks = sampler.stop()
    torch.cuda.synchronize()

    imgs = C3_BATCH * world * args.steps
    peak, kind = measured_peaks()
    alg = c3_algorithmic_bytes(C3_BATCH)
    kernels = kernel_table(trace, alg, peak, top=12, traffic=NCU_TRAFFIC["c3"])
    top = kernels[0] if kernels else {}
    traced_ms = sum(v[1] for v in trace.values())
    rec = {
        "metric": "train imgs/sec (fwd+bwd+Adam), cifar10_m-shaped LogicTreeNet", "value": imgs / (ms * 1e-3), "unit": "images/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": c3_config(world),
        "e2e": {"value": imgs / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": C3_BATCH * 9 * 32 * 32 + C3_BATCH * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps,
                "what": "uint8 bits + int64 labels from pinned host memory (copy stream, one step ahead), expanded to fp32 on the "
                        "device, the loss read back every step"},
        "gpu_launches": int(launches) * args.steps,
        "gpu_launches_per_step": int(launches),
        "host_enqueue_ms_per_step": host_ms / args.steps,   # Python + ctypes + torch time to enqueue a step; below ms_per_step = the GPU binds
        "parameters": bucket.numel,
        "roofline": {"bound": "hbm", "kernel": top.get("kernel"), "achieved": top.get("achieved_gbs"), "peak": peak, "unit": "GB/s",
                     "frac": top.get("frac"), "peak_kind": f"of {kind}", "algorithmic_bytes": top.get("algorithmic_bytes"), "traffic": top.get("traffic"),
                     "step_frac": alg["step"] / (ms / args.steps * 1e-3) / 1e9 / peak, "step_algorithmic_bytes": alg["step"],
                     "kernels": kernels, "traced_library_ms_per_step": round(traced_ms, 5),
                     "note": "kernel times: CUDA events the library records around each launch on the launching stream, in a "
                             "separate pass of the same step right after the timed region; the many-channel conv kernels are bound "
                             "by shared-memory gathers and instruction issue, not HBM"},
        "clocks": clocks,
    }
    bucket.remove_overlap()
    del net, opt, bucket, xs, labs, stage
    torch.cuda.empty_cache()
    if with_cpu and rank == 0 and world == 1 and not args.no_cpu:
        rec["cpu_baseline"] = cpu_baseline_c3(args.cpu_sample, passes=1)
    return rec


# ------------------------------------------------------------------------------------ workload c4
def run_c4(ctx, args):
    """cifar10_l-shaped discretised inference on bit-packed activations (64 images per word): 2^20 images sharded
    over the ranks, streamed in chunks through the compiled network; no collective."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib, dp

    dev, world, rank = ctx.dev, ctx.world, ctx.rank
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
    cnet = cb.CompiledLogicNet(net, input_shape=(93, 32, 32)).compile()  # the public call: one C call per chunk
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

    # parity on a 256-image subsample: compiled network == modules on packed activations == tau x float eval scores
    with torch.no_grad():
        sub = pixels[0][:256].contiguous()
        c_sub = cnet.forward_pixels(sub, th)
        bits = torch.cat([(sub.float() / 255 > t) for t in th.tolist()], dim=1)
        equals_modules = bool(torch.equal(c_sub, net(cb.PackBitsTensor.from_pixels(sub, th))))
        equals_float = bool(torch.equal(c_sub, (net(bits.float()).double() * 340).round().to(torch.int32)))
        del bits
    torch.cuda.empty_cache()

    lib = _lib.lib()
    sampler = ClockSampler(ctx.local, rank == 0).start()
    steps = max(1, min(args.steps, 3))
    ms = ctx.timed(step, steps, 1)
    l0 = lib.clb_kernel_launches()
    cnet.forward_pixels(pixels[0], th)
    launches_chunk = lib.clb_kernel_launches() - l0
    trace = traced(lambda i: cnet.forward_pixels(pixels[i % resident], th), 8)   # per chunk
    ms_e2e = ctx.timed(step_e2e, 1, 1)
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    per_image = {"packed_convtree_slab_kernel": 44672 + 65536 + 65536 + 49152, "packed_tree_kernel": 16384 + 81920,
                 "group_popcount_kernel": 81920 + 40, "thermometer_pack_kernel": 3072 + 11904}
    kernels = kernel_table(trace, {k: v * chunk for k, v in per_image.items()}, peak, traffic=NCU_TRAFFIC["c4"] if chunk == 8192 else None)
    top = kernels[0] if kernels else {}
    alg = 1388200.0 * (hi - lo)   # layer-by-layer algorithmic bytes of this rank's shard
    rec = {
        "metric": "packed-inference imgs/sec, cifar10_l-shaped LogicTreeNet", "value": total * steps / (ms * 1e-3), "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": 1, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u64", "data": "synthetic",
        "config": {"workload": f"c4: cifar10_l-shaped stack (k=1024, 4 ConvLogic blocks + 3 LogicLayers + GroupSum), discretised, {total} images "
                               f"of 93x32x32 thermometer bits (31 thresholds x RGB), 64 per word, chunks of {chunk}, "
                               "CompiledLogicNet.forward_pixels on uint8 pixels",
                   "l2": f"{resident} resident uint8 pixel chunks (~{resident * 3072 * chunk / 1e9:.2f} GB); every chunk's activations exceed the L2",
                   "parallelism": f"batch sharded over {world} ranks, no collective"},
        "e2e": {"value": total / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": 3 * 1024 * (hi - lo),
                "d2h_bytes_per_step": (hi - lo) * 8,
                "what": "uint8 pixels from pinned host memory, the compiled network on the GPU, class indices back to the host"},
        "gpu_launches": int(launches_chunk) * n_chunks * steps, "gpu_launches_per_chunk": int(launches_chunk), "blob_bytes": len(cnet.blob),
        "equals_float_eval": equals_float, "equals_module_path": equals_modules,
        "roofline": {"bound": "hbm", "kernel": top.get("kernel"), "achieved": top.get("achieved_gbs"), "peak": peak, "unit": "GB/s",
                     "frac": top.get("frac"), "peak_kind": f"of {kind}", "algorithmic_bytes": top.get("algorithmic_bytes"), "traffic": top.get("traffic"),
                     "step_frac": alg / (ms / steps * 1e-3) / 1e9 / peak, "kernels": kernels,
                     "note": "kernels per chunk; step_frac: 1 388 200 layer-by-layer algorithmic bytes per image over the whole pipeline"},
        "clocks": clocks}
    del cnet, net, pixels, dev_px
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------ workload c2
C2 = dict(batch=256, cin=9, cout=256, size=32)


def c2_algorithmic_bytes():
    b, ci, c, s = C2["batch"], C2["cin"], C2["cout"], C2["size"]
    x = b * ci * s * s * 4
    y = b * c * (s // 2) ** 2 * 4
    w, sel = c * 7 * 16 * 4, c * 8 * 4
    return {"fwd": x + y + w + sel, "bwd": y + x + x + 2 * w + sel, "step": (x + y + w + sel) + (y + x + x + 2 * w + sel)}


def run_c2(ctx, args):
    """One fused ConvLogic block 9 -> 256, 32x32, batch 256 per GPU: soft forward, input gradient, gate-logit gradient."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib

    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    dist = ctx.dist
    torch.manual_seed(0)
    layer = cb.ConvLogicLayer(C2["cin"], C2["cout"], padding=1, complete=True)
    layer.weights.data = torch.randn(C2["cout"], 7, 16, generator=torch.Generator().manual_seed(1))
    layer = layer.to(dev).train()
    sets = 3  # rotating input sets: ~150 MB each, so every step streams from HBM, not from the 126 MB L2
    g = torch.Generator().manual_seed(100 + rank)
    b, ci, c, s = C2["batch"], C2["cin"], C2["cout"], C2["size"]
    xs_h = [(torch.rand(b, ci, s, s, generator=g) < 0.5).float().pin_memory() for _ in range(sets)]
    gys_h = [torch.randn(b, c, s // 2, s // 2, generator=g).pin_memory() for _ in range(sets)]
    xs, gys = [x.to(dev) for x in xs_h], [t.to(dev) for t in gys_h]

    def block_step(x, gy):
        x.requires_grad_(True)
        x.grad = None
        layer.weights.grad = None
        layer(x).backward(gy)
        if world > 1:
            dist.all_reduce(layer.weights.grad)
        gx = x.grad
        x.requires_grad_(False)
        return gx, layer.weights.grad

    def step(i):
        block_step(xs[i % sets], gys[i % sets])

    gx_host = [torch.empty(b, ci, s, s).pin_memory() for _ in range(2)]
    gw_host = [torch.empty(c, 7, 16).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    x_dev = [torch.empty_like(xs[0]) for _ in range(2)]
    gy_dev = [torch.empty_like(gys[0]) for _ in range(2)]
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    state = {"k": None}

    def upload(k):
        sl = k % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[sl])
            x_dev[sl].copy_(xs_h[k % sets], non_blocking=True)
            gy_dev[sl].copy_(gys_h[k % sets], non_blocking=True)
            arrived[sl].record(copy_stream)

    def step_e2e(_):
        cur = torch.cuda.current_stream(dev)
        if state["k"] is None:
            for sl in range(2):
                consumed[sl].record(cur)
            upload(0)
            state["k"] = 0
        k = state["k"]
        upload(k + 1)
        sl = k % 2
        cur.wait_event(arrived[sl])
        gx, gw = block_step(x_dev[sl], gy_dev[sl])
        gx_host[sl].copy_(gx, non_blocking=True)
        gw_host[sl].copy_(gw, non_blocking=True)
        consumed[sl].record(cur)
        state["k"] = k + 1

    lib = _lib.lib()
    steps = max(args.steps, 20)
    sampler = ClockSampler(ctx.local, rank == 0).start()
    ms = ctx.timed(step, steps, args.warmup)
    l0 = lib.clb_kernel_launches()
    step(0)
    launches = lib.clb_kernel_launches() - l0
    trace = traced(step, 10)
    ms_e2e = ctx.timed(step_e2e, steps, 3)
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    alg = c2_algorithmic_bytes()
    names = {"convtree_fwd_pair_kernel": alg["fwd"], "convtree_fwd_tile_kernel": alg["fwd"], "convtree_bwd_cls_kernel": alg["bwd"]}
    kernels = kernel_table(trace, names, peak, traffic=NCU_TRAFFIC["c2"])
    top = kernels[0] if kernels else {}
    imgs = b * world * steps
    rec = {
        "metric": "train imgs/sec (fwd+bwd), single ConvLogic block", "value": imgs / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c2: ConvLogicLayer(9->256, 3x3, pad 1, complete) fwd+bwd, batch 256 per GPU, 32x32 Bernoulli(0.5) input",
                   "l2": f"{sets} rotating input sets of ~153 MB each (> 126 MB L2)",
                   "parallelism": f"dp{world}, all-reduce of gate-logit gradients" if world > 1 else "single GPU"},
        "e2e": {"value": imgs / (ms_e2e * 1e-3), "unit": "images/s", "h2d_bytes_per_step": xs_h[0].numel() * 4 + gys_h[0].numel() * 4,
                "d2h_bytes_per_step": xs_h[0].numel() * 4 + c * 7 * 16 * 4, "ms_per_step": ms_e2e / steps},
        "gpu_launches": int(launches) * steps,
        "kernel_ms": {k: round(v[1], 5) for k, v in trace.items()},
        "roofline": {"bound": "hbm", "kernel": top.get("kernel"), "achieved": top.get("achieved_gbs"), "peak": peak, "unit": "GB/s",
                     "frac": top.get("frac"), "peak_kind": f"of {kind}", "algorithmic_bytes": top.get("algorithmic_bytes"), "traffic": top.get("traffic"),
                     "step_frac": alg["step"] / (ms / steps * 1e-3) / 1e9 / peak, "kernels": kernels,
                     "note": "not HBM-bound: shared-memory gathers and instruction issue bind both kernels"},
        "clocks": clocks}
    # the reference's own CUDA kernels on this GPU and these inputs, when oracle/build_ref.py has built them (outside every timed region)
    if world == 1:
        try:
            from oracle.build_ref import load_ref

            rc = load_ref("convlogic_cuda")
        except Exception:
            rc = None
        if rc is not None:
            w, sel = layer.weights.detach(), layer.selection
            wp = torch.softmax(w, -1)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            t_f = t_b = 0.0
            nrep = 5
            for i in range(nrep + 1):
                xi, gi = xs[i % sets], gys[i % sets]
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
            rec["reference_cuda_same_gpu"] = {
                "fwd_ms": t_f / nrep, "bwd_ms": t_b / nrep, "images_per_s": b / ((t_f + t_b) / nrep * 1e-3),
                "what": "lkorinek/convlogic full_convlogic_forward + backward_x + backward_weight (its CUDA extension compiled unmodified "
                        "for sm_100a), same inputs, mixture given as probabilities"}
    del layer, xs, gys, x_dev, gy_dev
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------ workload c5
def run_c5(ctx, args):
    """Flat difflogic stack: 3072 -> 8 x 256000 LogicLayers -> GroupSum(10, tau=100), batch 1024, fwd + bwd."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib, dp, ops
    from convlogic_b200._lib import W_PROB

    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    torch.manual_seed(0)
    width, depth, batch = args.flat_width, args.flat_layers, 1024   # 256000 x 8 is the configuration; smaller ones are for profiling
    dims = [3072] + [width] * depth
    net = torch.nn.Sequential(*[cb.LogicLayer(i, o) for i, o in zip(dims[:-1], dims[1:])], cb.GroupSum(10, 100.0)).to(dev).train()
    gi = torch.Generator().manual_seed(100 + rank)
    x = (torch.rand(batch, 3072, generator=gi) < 0.5).float().to(dev)
    gy = torch.randn(batch, 10, generator=gi).to(dev)

    def step(i):
        for prm in net.parameters():
            prm.grad = None
        net(x).backward(gy)
        if world > 1:
            dp.allreduce_gate_gradients(net)

    lib = _lib.lib()
    sampler = ClockSampler(ctx.local, rank == 0).start()
    steps = max(1, min(args.steps, 10))
    ms = ctx.timed(step, steps, 3)
    l0 = lib.clb_kernel_launches()
    step(0)
    launches = lib.clb_kernel_launches() - l0
    trace = traced(step, 3)
    clocks = sampler.stop()
    peak, kind = measured_peaks()
    row = width * batch * 4          # one activation [width, batch] fp32
    xin = 3072 * batch * 4
    names = {
        "logic_fwd_kernel": (xin + row) + (depth - 1) * 2 * row,    # layer 1: x + y; the others: x + y
        "logic_bwd_w_kernel": (xin + row) + (depth - 1) * 2 * row,  # gy + x per layer
        "logic_bwd_x_kernel": (depth - 1) * 3 * row,                # all but the first layer: gy + x + gx
        "group_sum_partial_kernel": row, "group_sum_bwd_kernel": row,
    }
    kernels = kernel_table(trace, names, peak, traffic=NCU_TRAFFIC["c5"] if (width, depth, batch) == (256000, 8, 1024) else None)
    top = kernels[0] if kernels else {}
    # forward: layer 1 in + out, the others 2 rows each, GroupSum read; backward: 3 rows per layer, the first gy + x
    # (the GroupSum gradient counted as fused into the last layer): 39.9 GB at 256000 x 8
    alg = (xin + row) + (depth - 1) * 2 * row + row + (depth - 1) * 3 * row + (row + xin)
    rec = {
        "metric": "train samples/sec (fwd+bwd), flat difflogic stack", "value": 1024 * world * steps / (ms * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": steps, "warmup": 3, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"c5: {depth} LogicLayers 3072->{width}x{depth} + GroupSum(10, tau=100), batch {batch}, fwd+bwd",
                   "l2": f"every activation is {row / 1e9:.2f} GB (> 126 MB L2)"},
        "gpu_launches": int(launches) * steps,
        "roofline": {"bound": "hbm", "kernel": top.get("kernel"), "achieved": top.get("achieved_gbs"), "peak": peak, "unit": "GB/s",
                     "frac": top.get("frac"), "peak_kind": f"of {kind}", "algorithmic_bytes": top.get("algorithmic_bytes"), "traffic": top.get("traffic"),
                     "step_frac": alg / (ms / steps * 1e-3) / 1e9 / peak, "kernels": kernels,
                     "note": f"whole step {alg / 1e9:.1f} GB algorithmic; per kernel: gathered rows counted once per use (12 B in + 4 B out per "
                             "neuron and sample in the forward)"},
        "clocks": clocks}
    # one 256000 -> 256000 layer, ours and (when built) the reference's CUDA kernels, same tensors
    if world == 1 and width == 256000 and depth > 1:
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

        cmp = {"ours_ms_fwd_bwdw_bwdx": t3(lambda: ops.logic_fwd(xf, a_, b_, wp, W_PROB), lambda: ops.logic_bwd_w(xf, a_, b_, wp, gyf, W_PROB),
                                           lambda: ops.logic_bwd_x(xf, a_, b_, wp, gyf, st_, cs_, W_PROB))}
        try:
            from oracle.build_ref import load_ref

            rf = load_ref("difflogic_cuda")
        except Exception:
            rf = None
        if rf is not None:
            cmp["reference_cuda_ms_fwd_bwdw_bwdx"] = t3(lambda: rf.forward(xf, a_, b_, wp), lambda: rf.backward_w(xf, a_, b_, gyf),
                                                        lambda: rf.backward_x(xf, a_, b_, wp, gyf, st_, cs_))
        rec["one_layer_256000x1024"] = cmp
        del xf, gyf
    del net, x, gy
    torch.cuda.empty_cache()
    return rec


# ------------------------------------------------------------------------------------ workload c1
def run_c1(ctx, args):
    """mnist_s-shaped stack (k = 16, tau 6.5) in eval mode at batch 256: the correctness configuration, timed for
    completeness -- float eval forward, packed forward and the compiled network, which must agree."""
    import convlogic_b200 as cb
    from convlogic_b200 import _lib

    dev, world, rank = ctx.dev, ctx.world, ctx.rank
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
    sampler = ClockSampler(ctx.local, rank == 0).start()

    def fwd_float(i):
        with torch.no_grad():
            model(xf)

    def fwd_packed(i):
        with torch.no_grad():
            model(cb.PackBitsTensor(xb, 64))

    ms = ctx.timed(fwd_float, args.steps, args.warmup)
    l0 = lib.clb_kernel_launches()
    fwd_float(0)
    launches = lib.clb_kernel_launches() - l0
    ms_p = ctx.timed(fwd_packed, args.steps, 3)
    ms_c = ctx.timed(lambda i: cnet(xb), args.steps, 3)
    replay = cnet.capture(xb)
    graph_ok = bool(torch.equal(replay(xb), counts))
    ms_g = ctx.timed(lambda i: replay(xb), args.steps, 3)
    clocks = sampler.stop()
    return {
        "metric": "eval imgs/sec, mnist_s-shaped LogicTreeNet (float eval forward)", "value": 256 * world * args.steps / (ms * 1e-3),
        "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c1: mnist_s-shaped stack (k=16, tau=6.5), eval mode, batch 256 of 1x28x28 Bernoulli(0.2) bits",
                   "l2": "launch-bound: every tensor fits the L2", "parallelism": f"{world} independent replicas"},
        "packed_ms": ms_p / args.steps, "compiled_net_ms": ms_c / args.steps, "compiled_net_graph_ms": ms_g / args.steps,
        "paths_agree": agree and graph_ok, "gpu_launches": int(launches) * args.steps, "clocks": clocks}


# ---------------------------------------------------------------------------------- CPU baseline
class OracleC3:
    """The c3 training step on the CPU oracle: the same stack (same seeds, hence same connections and logits as
    build_c3), soft forward through oracle.full_convlogic / logic_layer / group_sum, cross-entropy, autograd
    backward and torch's Adam -- what the reference's ``implementation="python"`` path does, vectorised."""

    def __init__(self):
        import convlogic_b200 as cb

        torch.manual_seed(0)
        net = cb.ConvLogicCifarModel(k_param=256, input_channels=9, input_size=32, tau=40).network
        g = torch.Generator().manual_seed(1)
        self.params, self.blocks, self.flats = [], [], []
        for m in net:
            if hasattr(m, "weights"):
                w = torch.randn(*m.weights.shape, generator=g).requires_grad_(True)
                self.params.append(w)
                if isinstance(m, cb.ConvLogicLayer):
                    self.blocks.append((w, m.selection.clone()))
                else:
                    self.flats.append((w, m.indices_0.clone(), m.indices_1.clone()))
        self.opt = torch.optim.Adam(self.params, lr=0.01)

    def step(self, x, labels):
        import oracle

        self.opt.zero_grad(set_to_none=True)
        h = x
        for w, sel in self.blocks:
            h = oracle.full_convlogic(h, oracle.gate_probabilities(w, True), sel)[0]
        h = h.flatten(1)
        for w, a, b in self.flats:
            h = oracle.logic_layer(h, a, b, oracle.gate_probabilities(w, True))
        loss = torch.nn.functional.cross_entropy(oracle.group_sum(h, 10, 40.0), labels)
        loss.backward()
        self.opt.step()
        return float(loss.detach())


def cpu_baseline_c3(sample_batch, passes, model=None):
    """Times the oracle's c3 training step on `sample_batch` images with all the host cores this process may use."""
    cores = host_cores()
    torch.set_num_threads(cores)   # torchrun exports OMP_NUM_THREADS=1: do not inherit that
    model = model or OracleC3()
    g = torch.Generator().manual_seed(7)
    best = None
    for _ in range(passes + 1):  # the first pass warms the allocator
        x = (torch.rand(sample_batch, 9, 32, 32, generator=g) < 0.5).float()
        lab = torch.randint(0, 10, (sample_batch,), generator=g)
        t0 = time.perf_counter()
        model.step(x, lab)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": sample_batch / best, "unit": "images/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_batch} of the 256 images of a step: soft forward, cross-entropy, autograd backward, Adam over all "
                      f"10.7 M logits; torch CPU tensors on {cores} cores ({os.cpu_count()} logical CPUs on the host)"}


def run_reference(args):
    """Reference arm: the CPU port of the reference's Python path on the c3 training step.  Each of the K timed steps
    (after W warm-up steps) is the full step on a bounded sample of `--cpu-sample` images.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cores = host_cores()
    torch.set_num_threads(cores)
    model = OracleC3()
    sample = args.cpu_sample
    g = torch.Generator().manual_seed(7)
    times = []
    budget_s, t_start = 240.0, time.perf_counter()
    for i in range(args.warmup + args.steps):
        x = (torch.rand(sample, 9, 32, 32, generator=g) < 0.5).float()
        lab = torch.randint(0, 10, (sample,), generator=g)
        t0 = time.perf_counter()
        model.step(x, lab)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s and len(times) >= 3:
            break   # bounded: never more than a few minutes
    sec = statistics.median(times)
    value = sample / sec
    base = {"value": value, "unit": "images/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"each step = the full c3 training step on {sample} of the 256 images (soft forward, cross-entropy, autograd "
                      f"backward, Adam over all 10.7 M logits), torch CPU tensors on {cores} cores; median of {len(times)} steps"}
    print(json.dumps({
        "impl": "reference", "metric": "train imgs/sec (fwd+bwd+Adam), cifar10_m-shaped LogicTreeNet", "value": value, "unit": "images/s",
        "n_gpus": world, "steps": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": c3_config(world),
        "cpu_baseline": base, "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU port of the reference's implementation='python' path (oracle/); the reference's own Python needs its checkout, "
                "which is not on this machine"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--images", type=int, default=1 << 20, help="c4: total images")
    ap.add_argument("--chunk", type=int, default=8192, help="c4: images per streamed chunk")
    ap.add_argument("--flat-width", type=int, default=256000, help="c5: neurons per layer (smaller values: profiling cases)")
    ap.add_argument("--flat-layers", type=int, default=8, help="c5: number of LogicLayers")
    ap.add_argument("--cpu-sample", type=int, default=8, help="images per step of the CPU port")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--tapgrad-slice-mb", type=int, default=None,
                    help="override the library's slice size of the two-pass conv backward (0 = whole batch in one slice)")
    ap.add_argument("--plane-kernels", type=int, default=None, choices=[0, 1],
                    help="override the library's choice of the TMA-staged many-channel conv kernels (0 = the older staged kernels)")
    ap.add_argument("--no-feature-major", action="store_true", help="c3: the last block hands [N, C, h, w] to the flat layers (two transposed copies per step)")
    ap.add_argument("--separate-head", action="store_true", help="c3: GroupSumCrossEntropy as its own autograd node behind the fused flat layers")
    ap.add_argument("--torch-tail", action="store_true",
                    help="c3: torch's cross-entropy, .grad accumulation and fused Adam instead of the library's fused tail")
    ap.add_argument("--slab-mux", type=int, default=None, choices=[0, 1], help="override how the packed slab kernel applies gates")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    ctx = Ctx()
    if args.tapgrad_slice_mb is not None:
        from convlogic_b200 import _lib

        _lib.check(_lib.lib().clb_tune(_lib.TUNE_TAPGRAD_SLICE_BYTES, args.tapgrad_slice_mb << 20))
    if args.plane_kernels is not None:
        from convlogic_b200 import _lib

        _lib.check(_lib.lib().clb_tune(_lib.TUNE_PLANE_KERNELS, args.plane_kernels))
    if args.slab_mux is not None:
        from convlogic_b200 import _lib

        _lib.check(_lib.lib().clb_tune(_lib.TUNE_SLAB_MUX, args.slab_mux))
    if args.workload == "all":
        rec = run_c3(ctx, args)
        rec["packed_inference"] = run_c4(ctx, args)
        rec["microbench_c2"] = run_c2(ctx, args)
        rec["flat_c5"] = run_c5(ctx, args)
    else:
        rec = {"c1": run_c1, "c2": run_c2, "c3": run_c3, "c4": run_c4, "c5": run_c5}[args.workload](ctx, args)
    if ctx.rank == 0:
        print(json.dumps(rec))
    ctx.close()


if __name__ == "__main__":
    main()
