"""Data-parallel plumbing for the logic-gate layers: one process per GPU, batch-sharded replicas.

The only tensors that differ between ranks after a backward pass are the gate-logit gradients
(``weights.grad`` of every layer); connections (``selection``, ``indices_*``) are buffers and equal
on all ranks.  So a training step exchanges exactly one flat fp32 bucket, and inference exchanges
nothing.  The reference gets the same effect implicitly from Lightning's DDP strategy
(configs/config.yaml:20, src/convlogic/model.py:149-176).
"""

import torch
import torch.distributed as dist


def gate_parameters(model):
    """The ``weights`` parameters of every logic layer, in module order."""
    return [p for name, p in model.named_parameters() if name.split(".")[-1] == "weights"]


class GradBucket:
    """Keeps all gate-logit gradients in ONE flat buffer (each ``weights.grad`` is a view into it),
    so that the data-parallel exchange is a single all-reduce with no packing copies.

    ``zero()`` replaces ``optimizer.zero_grad()``.  If something drops the views all the same
    (``zero_grad(set_to_none=True)`` is torch's default and makes autograd allocate fresh ``.grad`` tensors),
    the bucket notices before it exchanges anything: the stray gradient is copied into its slice and
    ``.grad`` is bound to the slice again, so ranks never exchange a stale buffer."""

    def __init__(self, model):
        self.params = gate_parameters(model)
        if not self.params:
            raise ValueError("model has no logic-gate parameters")
        p0 = self.params[0]
        self.numel = sum(p.numel() for p in self.params)
        self.flat = torch.zeros(self.numel, dtype=p0.dtype, device=p0.device)
        off = 0
        self.ranges = []
        for p in self.params:
            p.grad = self.flat[off:off + p.numel()].view_as(p)
            self.ranges.append((off, off + p.numel()))
            off += p.numel()
        self._works, self._work_ranges, self._hooks, self._group, self._average = [], [], [], None, True
        self.rebinds = 0
        self._direct = False

    def zero(self):
        self._rebind_all(copy=False)
        self.flat.zero_()

    def _rebind(self, p, lo, hi, copy=True):
        """Make ``p.grad`` the bucket's slice again if it is not (any longer); returns True when it had to."""
        view = self.flat[lo:hi].view_as(p)
        g = p.grad
        if g is not None and g.data_ptr() == view.data_ptr() and g.shape == view.shape:
            return False
        if g is not None and copy:
            view.copy_(g)
        elif g is None and copy:
            view.zero_()  # no gradient arrived for this layer in this step
        p.grad = view
        self.rebinds += 1
        return True

    def _rebind_all(self, copy=True):
        for p, (lo, hi) in zip(self.params, self.ranges):
            self._rebind(p, lo, hi, copy)

    # ---- all-reduce overlapped with the rest of the backward pass
    def overlap(self, group=None, average=True):
        """From now on every layer's slice of the bucket is all-reduced (asynchronously) the moment autograd has
        accumulated that layer's gradient, i.e. while the layers in front of it are still in their backward
        kernels; call ``finish()`` after ``backward()`` and before the optimizer step.  The last layers' slices
        (the large flat layers) go first, as they are ready first."""
        self.remove_overlap()
        self._group, self._average = group, average
        for p, (lo, hi) in zip(self.params, self.ranges):
            self._hooks.append(p.register_post_accumulate_grad_hook(lambda _p, lo=lo, hi=hi: self._slice_ready(lo, hi, _p)))
        return self

    def remove_overlap(self):
        for h in self._hooks:
            h.remove()
        self._hooks, self._works, self._work_ranges = [], [], []

    def _slice_ready(self, lo, hi, p=None):
        if p is not None:
            if self._direct:
                return  # direct mode: the kernels' own ready() calls drive the exchange, not autograd's hooks
            self._rebind(p, lo, hi)
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self._group) == 1:
            return
        # NCCL averages inside the collective; other backends (gloo on CPU ranks) sum, finish() then divides
        self._in_op_average = self._average and dist.get_backend(self._group) == "nccl"
        op = dist.ReduceOp.AVG if self._in_op_average else dist.ReduceOp.SUM
        self._works.append(dist.all_reduce(self.flat[lo:hi], op=op, group=self._group, async_op=True))
        self._work_ranges.append((lo, hi))

    def _ranges_ready(self, ranges):
        """Several slices written by one backward kernel: neighbours in the bucket are exchanged as one piece."""
        if not self._hooks:
            return
        merged = []
        for lo, hi in sorted(ranges):
            if merged and merged[-1][1] == lo:
                merged[-1][1] = hi
            else:
                merged.append([lo, hi])
        for lo, hi in merged:
            self._slice_ready(lo, hi)

    # ---- kernels write their gate gradients straight into the bucket
    def direct(self, on=True):
        """From now on the backward kernels of this library write each layer's gate gradient straight into its slice
        of the bucket (no ``.grad`` accumulation kernels, no clearing between steps): every parameter carries a
        ``(slice, ready)`` pair the autograd Functions look for.  A parameter must then be used ONCE per backward pass
        (its slice is overwritten, not added to) -- true of the layer stacks this library models.  With ``overlap()``
        active the slice is all-reduced the moment its kernel has been enqueued, as the hooks would do."""
        for p, (lo, hi) in zip(self.params, self.ranges):
            if on:
                p._clb_grad_sink = (self.flat[lo:hi].view_as(p), lambda lo=lo, hi=hi: self._slice_ready(lo, hi) if self._hooks else None,
                                    self._ranges_ready, (lo, hi))
            elif hasattr(p, "_clb_grad_sink"):
                del p._clb_grad_sink
        self._direct = bool(on)
        return self

    def finish(self):
        """Waits for the slices in flight (the waits are stream-side for NCCL) and applies the averaging."""
        works, self._works, self._work_ranges = self._works, [], []
        for w in works:
            w.wait()
        if works and self._average and not getattr(self, "_in_op_average", False):
            self.flat.div_(dist.get_world_size(self._group))
        return len(works)

    def finish_but_last(self):
        """Waits for every exchange in flight except the one issued last (the first layer's small gradient, which the
        backward pass produces at its very end) and returns that one's element range [lo, hi), or None when nothing stays
        in flight.  Only with averaging inside the collective (NCCL): otherwise the same as ``finish()``."""
        if len(self._works) < 2 or (self._average and not getattr(self, "_in_op_average", False)):
            self.finish()
            return None
        for w in self._works[:-1]:
            w.wait()
        self._works, self._work_ranges = self._works[-1:], self._work_ranges[-1:]
        return self._work_ranges[0]

    def allreduce(self, group=None, average=True, async_op=False):
        """Sum (or mean) over ranks.  A no-op without an initialised process group."""
        self._rebind_all()
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return None
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if average:
            if async_op:
                work.wait()
            self.flat.div_(dist.get_world_size(group))
        return work


def allreduce_gate_gradients(model, group=None, average=True):
    """One-shot variant: flattens the existing ``weights.grad`` tensors, all-reduces, copies back."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    grads = [p.grad for p in gate_parameters(model) if p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat.div_(dist.get_world_size(group))
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


def broadcast_state(model, src=0, group=None):
    """Make parameters and connection buffers identical on all ranks (rank `src` wins)."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    for t in list(model.parameters()) + list(model.buffers()):
        dist.broadcast(t.data, src=src, group=group)


def shard_range(n_items, rank=None, world=None):
    """[lo, hi) of the items rank `rank` owns when `n_items` are split as evenly as possible."""
    if rank is None:
        rank = dist.get_rank() if dist.is_initialized() else 0
    if world is None:
        world = dist.get_world_size() if dist.is_initialized() else 1
    return n_items * rank // world, n_items * (rank + 1) // world


class FlatAdam:
    """Adam / AdamW over ALL gate logits of a model in one kernel launch (``clb_adam_step``).

    The parameters become views into one flat buffer (their names, shapes and values are unchanged, so state dicts
    interchange), the gradients are the flat buffer of a ``GradBucket``; ``step()`` is one launch over both.  Matches
    ``torch.optim.Adam(lr, betas, eps, weight_decay)`` / ``torch.optim.AdamW`` (``decoupled=True``, what the reference
    trains with: src/convlogic/model.py:179-180) to fp32 rounding."""

    def __init__(self, bucket, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled=False):
        from . import ops  # noqa: F401  (needs the CUDA library)

        self.bucket, self.lr, self.betas, self.eps, self.weight_decay, self.decoupled = bucket, lr, betas, eps, weight_decay, decoupled
        self.params = torch.empty_like(bucket.flat)
        for p, (lo, hi) in zip(bucket.params, bucket.ranges):
            self.params[lo:hi].copy_(p.data.reshape(-1))
            p.data = self.params[lo:hi].view_as(p)
        self.exp_avg = torch.zeros_like(bucket.flat)
        self.exp_avg_sq = torch.zeros_like(bucket.flat)
        self.steps = 0

    def zero_grad(self, set_to_none=False):
        """Clears the bucket (the gradients are views of it and stay bound)."""
        del set_to_none
        self.bucket.zero()

    def _update(self, lo, hi):
        from . import ops

        if hi > lo:
            ops.adam_step(self.params[lo:hi], self.bucket.flat[lo:hi], self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], self.lr, self.betas[0],
                          self.betas[1], self.eps, self.weight_decay, self.steps, self.decoupled)

    def step(self):
        if not self.bucket._direct:
            self.bucket._rebind_all()  # gradients that autograd re-allocated are copied into the bucket first
        self.steps += 1
        self._update(0, self.bucket.numel)

    def finish_and_step(self):
        """``bucket.finish()`` + ``step()`` for data-parallel runs with the overlapped exchange: the update of everything
        but the slice whose exchange was issued last runs while that exchange is still in flight, the update of that
        slice after it.  Same result as the two calls."""
        left = self.bucket.finish_but_last()
        if left is None:
            return self.step()
        if not self.bucket._direct:
            self.bucket._rebind_all()
        self.steps += 1
        self._update(0, left[0])
        self._update(left[1], self.bucket.numel)
        self.bucket.finish()
        self._update(left[0], left[1])
