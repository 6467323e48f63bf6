"""Data-parallel helpers on CPU ranks (gloo, world size 2): the N > 1 host logic of training and
of batch-sharded inference, without a GPU."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import convlogic_b200 as cb
        from convlogic_b200 import dp

        torch.manual_seed(100 + rank)  # deliberately different: broadcast_state must fix it
        model = torch.nn.Sequential(cb.ConvLogicLayer(3, 4, complete=True), torch.nn.Flatten(), cb.LogicLayer(16, 40),
                                    cb.GroupSum(10, 2.0))
        dp.broadcast_state(model)
        ref = [t.clone() for t in list(model.parameters()) + list(model.buffers())]
        gathered = [None] * world
        dist.all_gather_object(gathered, [t.tolist() for t in ref[:2]] + [ref[2].tolist()])
        assert gathered[0] == gathered[1], "state differs after broadcast"

        # flat bucket: gradients are views, one all-reduce averages them
        bucket = dp.GradBucket(model)
        params = dp.gate_parameters(model)
        assert [tuple(p.shape) for p in params] == [(4, 7, 16), (40, 16)]
        assert bucket.numel == 4 * 7 * 16 + 40 * 16
        for p in params:
            p.grad.fill_(float(rank + 1))
        assert float(bucket.flat.min()) == rank + 1  # views share storage
        bucket.allreduce(average=True)
        assert torch.allclose(bucket.flat, torch.full_like(bucket.flat, 1.5))
        assert all(torch.allclose(p.grad, torch.full_like(p, 1.5)) for p in params)
        bucket.zero()
        assert float(params[1].grad.abs().max()) == 0.0

        # overlapped variant: a slice is all-reduced from a hook as soon as autograd has accumulated into it
        bucket.overlap(average=True)
        bucket.zero()
        loss = sum((p * float(rank + 1)).sum() for p in params)   # d loss / d p = rank + 1 everywhere
        loss.backward()
        assert bucket.finish() == len(params)
        assert torch.allclose(bucket.flat, torch.full_like(bucket.flat, 1.5))
        assert all(p.grad.data_ptr() == bucket.flat[lo:hi].data_ptr() for p, (lo, hi) in zip(params, bucket.ranges))
        bucket.remove_overlap()
        bucket.zero()
        sum((p * 2.0).sum() for p in params).backward()
        assert bucket.finish() == 0 and torch.allclose(bucket.flat, torch.full_like(bucket.flat, 2.0))

        # zero_grad(set_to_none=True), torch's default, drops the views: the bucket must notice and exchange the
        # real gradients, in the overlapped variant (hooks) and in the one-call variant
        bucket.overlap(average=True)
        opt = torch.optim.SGD(params, lr=0.0)
        opt.zero_grad(set_to_none=True)
        assert all(p.grad is None for p in params)
        sum((p * float(rank + 1)).sum() for p in params).backward()      # autograd allocates fresh .grad tensors
        assert bucket.finish() == len(params)
        assert torch.allclose(bucket.flat, torch.full_like(bucket.flat, 1.5)), "stale bucket was exchanged"
        assert all(torch.allclose(p.grad, torch.full_like(p, 1.5)) for p in params)
        assert all(p.grad.data_ptr() == bucket.flat[lo:hi].data_ptr() for p, (lo, hi) in zip(params, bucket.ranges))
        assert bucket.rebinds >= len(params)
        bucket.remove_overlap()
        model.zero_grad(set_to_none=True)
        sum((p * float(3 * (rank + 1))).sum() for p in params).backward()
        bucket.allreduce(average=True)
        assert torch.allclose(bucket.flat, torch.full_like(bucket.flat, 4.5))
        assert all(torch.allclose(p.grad, torch.full_like(p, 4.5)) for p in params)
        bucket.zero()   # also re-binds (nothing to copy)
        assert all(p.grad.data_ptr() == bucket.flat[lo:hi].data_ptr() for p, (lo, hi) in zip(params, bucket.ranges))

        # direct mode: a backward kernel writes a layer's gradient into its bucket slice and reports it ready (the
        # library's autograd Functions do this on the GPU; here a stand-in Function follows the same protocol)
        from convlogic_b200.functional import _grad_sink

        class WritesIntoSink(torch.autograd.Function):
            @staticmethod
            def forward(ctx, w, scale):
                ctx.save_for_backward(w)
                ctx.scale = scale
                return (w * scale).sum()

            @staticmethod
            def backward(ctx, g):
                (w,) = ctx.saved_tensors
                sink = _grad_sink(w)
                assert sink is not None and w is params[0] or w is params[1]
                sink[0].copy_(torch.full_like(w, ctx.scale) * g)
                sink[1]()
                return None, None

        bucket.direct().overlap(average=True)
        bucket.flat.fill_(-7.0)            # stale values: direct mode overwrites, nothing clears the bucket
        sum(WritesIntoSink.apply(p, float(rank + 1)) for p in params).backward()
        assert bucket.finish() == len(params)
        assert torch.allclose(bucket.flat, torch.full_like(bucket.flat, 1.5))
        assert all(p.grad.data_ptr() == bucket.flat[lo:hi].data_ptr() for p, (lo, hi) in zip(params, bucket.ranges))
        # a kernel that writes several neighbouring slices (the fused flat layers) reports them together: one exchange
        bucket.flat.fill_(float(rank + 1))
        sinks = [_grad_sink(p) for p in params]
        assert all(len(s) == 4 and s[2] == sinks[0][2] for s in sinks)
        sinks[0][2]([s[3] for s in sinks])
        assert bucket.finish() == 1 and torch.allclose(bucket.flat, torch.full_like(bucket.flat, 1.5))
        # all exchanges but the last-issued one: gloo sums and finish() divides, so the call degrades to finish()
        for s in sinks:
            s[1]()
        assert bucket.finish_but_last() is None and not bucket._works
        bucket.remove_overlap()
        bucket.direct(False)
        assert all(_grad_sink(p) is None for p in params)

        # one-shot variant on ordinary .grad tensors
        for p in params:
            p.grad = torch.full_like(p, float(10 * (rank + 1)))
        dp.allreduce_gate_gradients(model, average=False)
        assert all(torch.allclose(p.grad, torch.full_like(p, 30.0)) for p in params)

        # inference shards: disjoint, exhaustive, no collective needed
        lo, hi = dp.shard_range(1001)
        spans = [None] * world
        dist.all_gather_object(spans, (lo, hi))
        assert spans[0][0] == 0 and spans[-1][1] == 1001 and spans[0][1] == spans[1][0]

        # a rank that fails on the host before the collective: the others see it through the store
        # (no collective is entered, nothing hangs)
        flags = [None] * world
        dist.all_gather_object(flags, "error" if rank == fail_rank else "ok")
        if "error" in flags:
            raise RuntimeError("peer failure reported before the collective")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_gradient_bucket_and_sharding():
    mp.spawn(_worker, args=(2, _free_port(), -1), nprocs=2, join=True)


@pytest.mark.timeout(300)
def test_host_side_failure_is_reported_not_hung():
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, _free_port(), 1), nprocs=2, join=True)
