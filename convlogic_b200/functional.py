"""Autograd Functions with the reference's names and argument lists.

``FullConvLogicFunction``, ``ConvLogicFunction`` (src/convlogic/convlogic_layer.py:16-82),
``TreeLogicFunction`` (src/convlogic/treelogic_layer.py:15-30), ``LogicLayerCudaFunction``
(src/difflogic/difflogic.py:214-230) and ``GradFactor`` (src/difflogic/functional.py:131-139).

As in the reference the gate argument is a MIXTURE over the 16 gates (soft-max already taken,
or one-hot) and the returned gradient is w.r.t. that mixture.  Each Function accepts one extra,
optional trailing argument ``wmode``; the layer modules pass W_SOFTMAX / W_ARGMAX together with
the raw logits so that the soft-max (and its Jacobian in backward) runs inside the kernels.

Unlike the reference, nothing but the input and an 8-bit arg-max per pooled output is saved for
backward: the gate tree is recomputed at the arg-max position.
"""

import torch
from torch.autograd import Function

from . import ops
from ._lib import W_ARGMAX, W_PROB, W_SOFTMAX  # noqa: F401


def _grad_sink(w):
    """(slice, ready-callback) when a gradient bucket (``dp.GradBucket.direct``) wants this parameter's gradient written
    straight into its slice of the flat buffer, else None.  Backward passes then hand the slice to the kernel as its
    output, call ``ready()`` and return no gradient for the parameter: no ``.grad`` accumulation kernel runs."""
    return getattr(w, "_clb_grad_sink", None)


class GradFactor(Function):
    @staticmethod
    def forward(ctx, x, f):
        ctx.f = f
        return x

    @staticmethod
    def backward(ctx, grad_y):
        return grad_y * ctx.f, None


class FullConvLogicFunction(Function):
    @staticmethod
    def forward(ctx, x, w_prob, selection, stride_h, stride_w, pad_h, pad_w, kernel_h, kernel_w,
                return_intermediate=False, return_indices=False, wmode=W_PROB, y_feature_major=False):
        x = x.contiguous()
        w_prob = w_prob.contiguous()
        geom = (stride_h, stride_w, pad_h, pad_w, kernel_h, kernel_w)
        need_bwd = any(ctx.needs_input_grad[:2])
        y, amax, x2, x3, idx = ops.convtree_fwd(x, w_prob, selection, geom, wmode, want_amax=need_bwd,
                                                want_intermediate=return_intermediate, want_indices=return_indices,
                                                y_feature_major=y_feature_major)
        ctx.save_for_backward(x, w_prob, selection, amax)
        ctx.geom, ctx.wmode = geom, wmode
        extra = []
        if return_intermediate:
            extra += [x2, x3]
        if return_indices:
            extra.append(idx)
        if extra:
            ctx.mark_non_differentiable(*extra)
            return (y, *extra)
        return y

    @staticmethod
    def backward(ctx, grad_y, *unused):
        x, w, sel, amax = ctx.saved_tensors
        if not ops._is_feature_major(grad_y):   # a feature-major gradient (from flat layers behind this block) is read as it is
            grad_y = grad_y.contiguous()
        need_gx = ctx.needs_input_grad[0]
        need_gw = ctx.needs_input_grad[1] and ctx.wmode != W_ARGMAX
        gx = gw = None
        if need_gx or need_gw:
            sink = _grad_sink(w) if need_gw else None
            gx, gw = ops.convtree_bwd(grad_y, x, w, sel, amax, ctx.geom, ctx.wmode, need_gx, need_gw,
                                      gw_out=None if sink is None else sink[0])
            if sink is not None:
                sink[1]()
                gw = None
        return (gx, gw) + (None,) * 11


class ConvLogicFunction(Function):
    @staticmethod
    def forward(ctx, x, w_prob, selection, stride_h, stride_w, pad_h, pad_w, kernel_h, kernel_w, wmode=W_PROB):
        x = x.contiguous()
        w_prob = w_prob.contiguous()
        geom = (stride_h, stride_w, pad_h, pad_w, kernel_h, kernel_w)
        y = ops.conv_fwd(x, w_prob, selection, geom, wmode)
        ctx.save_for_backward(x, w_prob, selection)
        ctx.geom, ctx.wmode = geom, wmode
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, w, sel = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = ops.conv_bwd_x(grad_y, x, w, sel, ctx.geom, ctx.wmode)
        if ctx.needs_input_grad[1] and ctx.wmode != W_ARGMAX:
            gw = ops.conv_bwd_w(grad_y, x, w, sel, ctx.geom, ctx.wmode)
        return (gx, gw) + (None,) * 8


class TreeLogicFunction(Function):
    @staticmethod
    def forward(ctx, x, w_prob, wmode=W_PROB):
        x = x.contiguous()
        w_prob = w_prob.contiguous()
        y = ops.tree_fwd(x, w_prob, wmode)
        ctx.save_for_backward(x, w_prob)
        ctx.wmode = wmode
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, w = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = ops.tree_bwd_x(grad_y, x, w, ctx.wmode)
        if ctx.needs_input_grad[1] and ctx.wmode != W_ARGMAX:
            gw = ops.tree_bwd_w(grad_y, x, w, ctx.wmode)
        return gx, gw, None


class LogicLayerCudaFunction(Function):
    """x is feature-major [in_dim, batch]; returns [out_dim, batch]."""

    @staticmethod
    def forward(ctx, x, a, b, w, given_x_indices_of_y_start, given_x_indices_of_y, wmode=W_PROB):
        x = x.contiguous()
        w = w.contiguous()
        ctx.save_for_backward(x, a, b, w, given_x_indices_of_y_start, given_x_indices_of_y)
        ctx.wmode = wmode
        return ops.logic_fwd(x, a, b, w, wmode)

    @staticmethod
    def backward(ctx, grad_y):
        x, a, b, w, start, cons = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = ops.logic_bwd_x(x, a, b, w, grad_y, start, cons, ctx.wmode)
        if ctx.needs_input_grad[3] and ctx.wmode != W_ARGMAX:
            sink = _grad_sink(w)
            gw = ops.logic_bwd_w(x, a, b, w, grad_y, ctx.wmode, gw_out=None if sink is None else sink[0])
            if sink is not None:
                sink[1]()
                gw = None
        return gx, None, None, gw, None, None, None


class GroupSumFunction(torch.autograd.Function):
    """GroupSum on the feature-major [F, B] storage a LogicLayer's output is a view of (no transposed copy)."""

    @staticmethod
    def forward(ctx, y_fm, k, tau):
        ctx.meta = (y_fm.shape[0], k, tau)
        return ops.group_sum_fwd(y_fm, k, tau)

    @staticmethod
    def backward(ctx, gout):
        f, k, tau = ctx.meta
        return ops.group_sum_bwd(gout.contiguous(), f, k, tau), None, None


class LogicTreeFunction(torch.autograd.Function):
    """Three flat layers fused into one gate tree per neuron of the last one (feature-major in and out)."""

    @staticmethod
    def forward(ctx, x_fm, w0, w1, w2, leaf, node, start, slots, wmode, covers_all=False):
        x_fm, w0, w1, w2 = x_fm.contiguous(), w0.contiguous(), w1.contiguous(), w2.contiguous()
        ctx.save_for_backward(x_fm, w0, w1, w2, leaf, node, start, slots)
        ctx.wmode, ctx.covers_all = wmode, covers_all
        return ops.logic_tree_fwd(x_fm, leaf, node, w0, w1, w2, wmode)

    @staticmethod
    def backward(ctx, gy):
        x_fm, w0, w1, w2, leaf, node, start, slots = ctx.saved_tensors
        sinks = [_grad_sink(w) for w in (w0, w1, w2)]
        direct = ctx.wmode != W_ARGMAX and all(s is not None for s in sinks)
        gx, g0, g1, g2 = ops.logic_tree_bwd(x_fm, leaf, node, w0, w1, w2, gy.contiguous(), start, slots, ctx.wmode,
                                            need_gx=ctx.needs_input_grad[0], gw_out=[s[0] for s in sinks] if direct else None,
                                            clear_gw=not ctx.covers_all)
        if direct:
            if all(len(s) > 2 and s[2] == sinks[0][2] for s in sinks):
                sinks[0][2]([s[3] for s in sinks])   # one bucket: neighbouring slices go out as one exchange
            else:
                for s in sinks:
                    s[1]()
        if ctx.wmode == W_ARGMAX or direct:
            g0 = g1 = g2 = None
        return gx, g0, g1, g2, None, None, None, None, None, None


class GroupSumCrossEntropyFunction(torch.autograd.Function):
    """GroupSum(k, tau) followed by the mean cross-entropy, on the feature-major [F, B] storage of a LogicLayer's output:
    the scores are never materialised for autograd, and the backward is one broadcast kernel."""

    @staticmethod
    def forward(ctx, y_fm, labels, k, tau):
        loss, dscore, _ = ops.group_sum_ce(y_fm.contiguous(), labels.contiguous(), k, tau)
        ctx.save_for_backward(dscore)
        ctx.meta = (y_fm.shape[0], k, tau)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, gloss):
        (dscore,) = ctx.saved_tensors
        f, k, tau = ctx.meta
        return ops.group_sum_bwd(dscore, f, k, tau, scale=gloss.reshape(1).to(dscore.dtype).contiguous()), None, None, None


class LogicTreeCrossEntropyFunction(torch.autograd.Function):
    """The fused flat layers followed by GroupSum(k, tau) and the mean cross-entropy as ONE autograd node: the backward
    pass derives the trees' upstream gradient from the head's score gradient inside the tree kernel, so the [T, B]
    gradient tensor between the two is neither written (the GroupSum backward kernel is not launched) nor read."""

    @staticmethod
    def forward(ctx, x_fm, w0, w1, w2, leaf, node, start, slots, labels, k, tau, covers_all=False):
        x_fm, w0, w1, w2 = x_fm.contiguous(), w0.contiguous(), w1.contiguous(), w2.contiguous()
        labels = labels.contiguous()
        out = ops.logic_tree_fwd_ce(x_fm, leaf, node, w0, w1, w2, labels, k, tau, W_SOFTMAX)   # class sums without the activation
        if out is None:
            out = ops.group_sum_ce(ops.logic_tree_fwd(x_fm, leaf, node, w0, w1, w2, W_SOFTMAX), labels, k, tau)[:2]
        loss, dscore = out
        ctx.save_for_backward(x_fm, w0, w1, w2, leaf, node, start, slots, dscore)
        ctx.meta = (k, tau, covers_all)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, gloss):
        x_fm, w0, w1, w2, leaf, node, start, slots, dscore = ctx.saved_tensors
        k, tau, covers_all = ctx.meta
        sinks = [_grad_sink(w) for w in (w0, w1, w2)]
        direct = all(s is not None for s in sinks)
        head = (dscore, gloss.reshape(1).to(torch.float32).contiguous(), k, tau)
        gx, g0, g1, g2 = ops.logic_tree_bwd(x_fm, leaf, node, w0, w1, w2, None, start, slots, W_SOFTMAX, need_gx=ctx.needs_input_grad[0],
                                            gw_out=[s[0] for s in sinks] if direct else None, clear_gw=not covers_all, head=head)
        if direct:
            if all(len(s) > 2 and s[2] == sinks[0][2] for s in sinks):
                sinks[0][2]([s[3] for s in sinks])
            else:
                for s in sinks:
                    s[1]()
            g0 = g1 = g2 = None
        return (gx, g0, g1, g2) + (None,) * 8


class FeatureMajorFunction(torch.autograd.Function):
    """[batch, features] -> contiguous [features, batch] (and the same copy back for the gradient) with the library's
    tiled transpose instead of a strided torch copy: the layout change in front of the flat layers."""

    @staticmethod
    def forward(ctx, x):
        return ops.transpose2d(x)

    @staticmethod
    def backward(ctx, g):
        return ops.transpose2d(g.contiguous())


def to_feature_major(x):
    """Feature-major copy of a 2-D activation; free (a view) when x is the transposed view a flat layer returned."""
    xt = x.transpose(0, 1)
    if xt.is_contiguous() or not (x.is_cuda and x.dtype == torch.float32 and x.is_contiguous() and x.numel()):
        return xt.contiguous()
    return FeatureMajorFunction.apply(x)
