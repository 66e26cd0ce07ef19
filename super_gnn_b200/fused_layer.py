"""One hidden GraphSAGE layer as a single autograd node:

    y = relu(LayerNorm(dropout(lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias)))

the composition of DistSAGEConvGrad.forward (super_gnn/layers/sageconv.py:62-89) with the
dropout / LayerNorm / relu that follow it in DistSAGE.forward
(examples/graphsage/sage.py:189-196).  Same parameters, same math; what changes is the
number of passes over the [n, hidden] activations and where the dense products run: the two
linear maps run as ONE fp32-accurate tensor-core GEMM over the [aggregated input | input] buffer with the
concatenated weights (``ops.gemm_nt``), their weight gradients as one reduction over the nodes
(``ops.gemm_tn``) and their input gradients as one GEMM onto a [., .] buffer of the same shape, the four
elementwise / normalisation ops run as one kernel each way, and the backward aggregation accumulates into
the self-path gradient in place.  Saved for the backward: the aggregated input, the GEMM output
h and two numbers per row (mean, reciprocal standard deviation); the normalised values, the
sign of the output and the dropout mask are recomputed from those.
"""
from __future__ import annotations

import torch

from . import supergnn_ops as ops
from .aggregator import _spmm_overwrite, _world, aggregate_backward, aggregate_forward


class _AggCtx:
    """Stand-in for the autograd context the Aggregator's static methods write to."""


# [n, 2K] buffers whose right half is a layer's input x: the layer that produced x puts it there, the
# aggregation writes the left half, and one GEMM with the concatenated weights
# [W_neigh | W_self] then replaces two GEMMs and a pass that re-reads and re-writes their sum.  Keyed by the
# address of the right half; cleared by the model at the start of every forward pass.
_AX = {}


# Addresses of the input gradients the layers below handed to autograd during the current backward pass: a
# layer that receives one of them as its incoming gradient is its only reader and may overwrite it.
_OWN_GRADS = set()


def reset_layer_buffers():
    _AX.clear()
    _OWN_GRADS.clear()


def _own(gx):
    if gx is not None:
        _OWN_GRADS.add(gx.data_ptr())
    return gx


def _concat_buffer(x):
    """The registered [n, 2K] buffer whose right half IS ``x`` (same memory), or None."""
    n, K = x.shape
    buf = _AX.get(x.data_ptr())
    if (buf is not None and tuple(buf.shape) == (n, 2 * K) and x.stride() == (2 * K, 1) and buf.device == x.device
            and x.data_ptr() == buf.data_ptr() + 4 * K):
        return buf
    return None


class FusedSAGELayer(torch.autograd.Function):
    """``feeds_fused_layer``: the output goes to another layer of this kind, so it is written into the right half
    of that layer's [aggregated input | input] buffer (no copy later).  A layer whose own input is not in such a
    buffer (the first one: the caller's features) runs its two linear maps as two GEMMs, the second one adding
    onto the first one's output, instead of copying the input."""

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, gamma, beta, graph, layer, num_bits, is_pre_delay, training, p, eps,
                seed, mask, feeds_fused_layer=False):
        n, K = x.shape
        H = w_neigh.size(0)
        actx = _AggCtx()
        ax = _concat_buffer(x)  # [agg | x], or None
        if ax is not None:
            aggregate_forward(actx, graph, x, layer, num_bits, is_pre_delay, training, out=ax[:, :K])
            agg = ax[:, :K]
        else:
            agg = aggregate_forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        if ax is not None:
            w_cat = torch.cat([w_neigh, w_self], dim=1)  # [H, 2K]
            h = ops.gemm_nt(ax, w_cat)
            keep = [ax, w_cat]
        else:
            h = ops.gemm_nt(agg, w_neigh)
            ops.gemm_nt(x, w_self, out=h, beta=1.0)
            keep = [x, agg, w_neigh, w_self]
        if feeds_fused_layer:
            nxt = x.new_empty((n, 2 * H))  # the next layer's [agg | x] buffer: this layer's output is its right half
            y, stats = ops.sage_epilogue_forward(h, bias, gamma, beta, p, training, seed, eps, mask, out=nxt[:, H:])
            _AX[y.data_ptr()] = nxt
        else:
            y, stats = ops.sage_epilogue_forward(h, bias, gamma, beta, p, training, seed, eps, mask)
        ctx.actx, ctx.graph = actx, graph
        ctx.cfg = (training, p, seed)
        ctx.has_mask = mask is not None
        ctx.K, ctx.concat = K, ax is not None
        saved = [h, stats, bias, gamma, beta] + keep + ([mask] if mask is not None else [])
        ctx.save_for_backward(*saved)
        return y

    @staticmethod
    def backward(ctx, gy):
        saved = ctx.saved_tensors
        h, stats, bias, gamma, beta = saved[:5]
        mask = saved[-1] if ctx.has_mask else None
        training, p, seed = ctx.cfg
        K = ctx.K
        gy = gy if gy.stride(-1) == 1 else gy.contiguous()
        mine = gy.data_ptr() in _OWN_GRADS and gy.stride(0) % 4 == 0  # produced by the layer above for this one alone
        _OWN_GRADS.discard(gy.data_ptr())
        gh, g_bias, g_gamma, g_beta = ops.sage_epilogue_backward(gy, h, stats, bias, gamma, beta, p, training, seed,
                                                                 mask, in_place=mine)
        gx = None
        if ctx.concat:
            ax, w_cat = saved[5:7]
            gw = ops.gemm_tn(gh, ax)  # [H, 2K] = [grad W_neigh | grad W_self]
            gw_neigh, gw_self = gw[:, :K], gw[:, K:]
            if ctx.needs_input_grad[0]:
                # [gh W_neigh | gh W_self] in one GEMM; the backward aggregation reads the left half and adds onto
                # the right half, which then is grad_x = Aggregator^T(gh W_neigh / in_degrees) + gh W_self
                g_cat = ops.gemm_nt(gh, w_cat.t().contiguous())
                if not getattr(ctx.graph, "fold_mean", False):
                    g_cat[:, :K].div_(ctx.graph.in_degrees)
                gx = aggregate_backward(ctx.actx, g_cat[:, :K], out=g_cat[:, K:], accumulate=True)
        else:
            x, agg, w_neigh, w_self = saved[5:9]
            gw_neigh = ops.gemm_tn(gh, agg)
            gw_self = ops.gemm_tn(gh, x)
            if ctx.needs_input_grad[0]:
                g_agg = ops.gemm_nt(gh, w_neigh.t().contiguous())
                if not getattr(ctx.graph, "fold_mean", False):
                    g_agg.div_(ctx.graph.in_degrees)
                gx = ops.gemm_nt(gh, w_self.t().contiguous())
                gx = aggregate_backward(ctx.actx, g_agg, out=gx, accumulate=True)
        return (_own(gx), gw_neigh, gw_self, g_bias, g_gamma, g_beta) + (None,) * 10


def _pad_rows(w, rows):
    """[rows, K] copy of the [C, K] weight with zero rows appended (C is rounded up to a multiple of 4 so that the
    class dimension meets the GEMM's 16-byte row rule)."""
    if w.size(0) == rows:
        return w
    out = w.new_zeros((rows, w.size(1)))
    out[:w.size(0)] = w
    return out


def narrow_local_applies(graph, w_neigh) -> bool:
    """Several partitions, mean folded into the aggregation, fewer classes (rounded up to 4) than input channels."""
    C, K = w_neigh.shape
    return (FusedSAGEOutputLayer.narrow_local and _world()[1] > 1 and getattr(graph, "fold_mean", False)
            and (C + 3) // 4 * 4 < K)


def _narrow_local_forward(x, w_neigh, w_self, graph, layer, num_bits, is_pre_delay, training):
    """Logits (without bias) of the last layer with the reference's boundary exchange: local edges aggregate the
    projected rows while the boundary rows of x are in flight, the remote edges' share of the aggregation is
    projected afterwards.  Returns (actx, w_cat, agg_remote, logits [n, C] view, (C, Cp))."""
    C, K = w_neigh.shape
    Cp = (C + 3) // 4 * 4
    w_cat = x.new_zeros((2 * Cp, K))
    w_cat[:C] = w_neigh
    w_cat[Cp:Cp + C] = w_self
    holder = {}

    def local_work():  # runs while the boundary rows are in flight
        zs = holder["zs"] = ops.gemm_nt(x, w_cat)  # [n, 2 Cp] = [x W_neigh^T | x W_self^T]
        _spmm_overwrite(graph.local_adj_t, zs[:, :Cp], zs[:, Cp:], transpose=False, row_scale=graph.inv_in_degrees,
                        accumulate=True)
        return x.new_zeros((x.size(0), K))  # receives the remote edges' share of the aggregation

    actx = _AggCtx()
    agg_remote = aggregate_forward(actx, graph, x, layer, num_bits, is_pre_delay, training, local_work=local_work)
    zs = holder["zs"]
    ops.gemm_nt(agg_remote, w_cat[:Cp], out=zs[:, Cp:], beta=1.0)
    return actx, w_cat, agg_remote, zs[:, Cp:Cp + C], (C, Cp)


def _narrow_local_backward(ctx, G, x, agg_remote, w_cat):
    """G = [. | g] with the gradient of the logits in the right half (padding columns zero): returns
    (grad_x, grad_W_neigh, grad_W_self); the exchanged rows are those of A_remote^T (g W_neigh), as in the
    reference."""
    C, Cp = ctx.dims
    graph = ctx.graph
    g_right = G[:, Cp:]
    g_agg = ops.gemm_nt(g_right, w_cat[:Cp].t().contiguous())  # what the transposed remote aggregation consumes

    def local_work():  # runs while the boundary gradients are in flight
        _spmm_overwrite(graph.local_adj_t, g_right, G[:, :Cp], transpose=True, col_scale=graph.inv_in_degrees)
        # (A_local^T g) W_neigh + g W_self, written over g_agg: its only readers, the transposed remote
        # aggregations, were enqueued on this stream before this call, and a gradient buffer of the input width
        # less is alive at what is the memory peak of the step
        return ops.gemm_nt(G, w_cat.t().contiguous(), out=g_agg)

    gx = _own(aggregate_backward(ctx.actx, g_agg, local_work=local_work))
    gw = ops.gemm_tn(G, x)  # rows [0, Cp): local share of grad W_neigh; rows [Cp, 2 Cp): grad W_self
    ops.gemm_tn(g_right, agg_remote, out=gw[:Cp], beta=1.0)  # + g^T (remote share of the aggregation)
    return gx, gw[:C], gw[Cp:Cp + C]


class FusedSAGEOutputLayer(torch.autograd.Function):
    """The last layer, ``lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias`` (no normalisation,
    dropout or relu follows it), with the reference's boundary exchange (the rows of ``x`` cross the partition
    boundary, at the configured bit width) as one autograd node: the same tensor-core GEMMs and in-place
    accumulations as the hidden layers, with the class dimension padded to a multiple of 4 inside the node.

    ``narrow_local`` (several partitions, mean folded into the aggregation): only the contribution of the REMOTE
    edges is aggregated at the input width and then projected; the local edges aggregate the already projected
    rows, ``A_local (x W_neigh^T)``, one fifth as wide at 47 classes against 256 channels.  The exchanged bytes are
    the reference's (same rows of ``x`` forward, same rows of ``A_remote^T (g W_neigh)`` backward), the result
    differs from aggregate-then-project by fp32 rounding only."""

    narrow_local = True

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training):
        C, K = w_neigh.shape
        Cp = (C + 3) // 4 * 4
        actx = _AggCtx()
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.dims = (C, Cp)
        ctx.hybrid = narrow_local_applies(graph, w_neigh)
        if ctx.hybrid:
            ctx.actx, w_cat, agg_remote, logits, _ = _narrow_local_forward(x, w_neigh, w_self, graph, layer, num_bits,
                                                                           is_pre_delay, training)
            out = logits + bias if bias is not None else logits.contiguous()
            ctx.save_for_backward(x, agg_remote, w_cat)
            return out
        agg = aggregate_forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        wn, ws = _pad_rows(w_neigh, Cp), _pad_rows(w_self, Cp)
        out = ops.gemm_nt(agg, wn)
        ops.gemm_nt(x, ws, out=out, beta=1.0)
        out = out[:, :C] + bias if bias is not None else out[:, :C].contiguous()
        ctx.save_for_backward(x, agg, wn, ws)
        return out

    @staticmethod
    def backward(ctx, g):
        C, Cp = ctx.dims
        g_bias = g.sum(0) if ctx.has_bias else None
        if ctx.hybrid:
            x, agg_remote, w_cat = ctx.saved_tensors
            G = g.new_empty((g.size(0), 2 * Cp))  # [A_local^T (g / in_degrees) | g], zero in the padding columns
            G[:, Cp:Cp + C] = g
            if Cp > C:
                G[:, Cp + C:] = 0
            gx, gw_neigh, gw_self = _narrow_local_backward(ctx, G, x, agg_remote, w_cat)
            return (gx, gw_neigh, gw_self, g_bias) + (None,) * 5
        x, agg, wn, ws = ctx.saved_tensors
        if Cp != C:
            gp = g.new_zeros((g.size(0), Cp))
            gp[:, :C] = g
        else:
            gp = g.contiguous()
        gw_neigh = ops.gemm_tn(gp, agg)[:C]
        gw_self = ops.gemm_tn(gp, x)[:C]
        gx = None
        if ctx.needs_input_grad[0]:
            g_agg = ops.gemm_nt(gp, wn.t().contiguous())
            if not getattr(ctx.graph, "fold_mean", False):
                g_agg.div_(ctx.graph.in_degrees)
            gx = ops.gemm_nt(gp, ws.t().contiguous())
            gx = _own(aggregate_backward(ctx.actx, g_agg, out=gx, accumulate=True))
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 5


def _project_first_forward(x, w_neigh, w_self, graph, layer, num_bits, is_pre_delay, training):
    """[x W_neigh^T | x W_self^T] in one GEMM, then the aggregation of the left half added onto the right half.
    Returns (actx, w_cat, logits without bias as a [n, C] view, (C, Cp))."""
    C, K = w_neigh.shape
    Cp = (C + 3) // 4 * 4
    w_cat = x.new_zeros((2 * Cp, K))
    w_cat[:C] = w_neigh
    w_cat[Cp:Cp + C] = w_self
    zs = ops.gemm_nt(x, w_cat)  # [n, 2 Cp]
    actx = _AggCtx()
    if getattr(graph, "fold_mean", False):
        aggregate_forward(actx, graph, zs[:, :Cp], layer, num_bits, is_pre_delay, training, out=zs[:, Cp:],
                           accumulate=True)
        logits = zs[:, Cp:Cp + C]
    else:
        agg = aggregate_forward(actx, graph, zs[:, :Cp], layer, num_bits, is_pre_delay, training)
        logits = agg.div_(graph.in_degrees)[:, :C].add_(zs[:, Cp:Cp + C])
    return actx, w_cat, logits, (C, Cp)


def _project_first_backward(ctx, G, x, w_cat, need_gx: bool):
    """G = [. | g] with the gradient of the logits in the right half (padding columns zero): fills the left half
    with A^T (g / in_degrees) and returns (grad_x, grad_W_neigh, grad_W_self)."""
    C, Cp = ctx.dims
    g_in = G[:, Cp:]
    if not getattr(ctx.graph, "fold_mean", False):
        g_in = g_in / ctx.graph.in_degrees
    aggregate_backward(ctx.actx, g_in, out=G[:, :Cp], accumulate=False)
    gw = ops.gemm_tn(G, x)  # [2 Cp, K]: rows of grad W_neigh, then of grad W_self
    gx = _own(ops.gemm_nt(G, w_cat.t().contiguous())) if need_gx else None
    return gx, gw[:C], gw[Cp:Cp + C]


class FusedSAGEOutputLayerProjectFirst(torch.autograd.Function):
    """The last layer with the projection moved in front of the aggregation:

        out = Aggregator(x W_neigh^T) / in_degrees + x W_self^T + bias

    which is the same function of the same parameters as ``lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) +
    bias`` (super_gnn/layers/sageconv.py:62-89) because the mean aggregation is linear; the results differ by
    fp32 rounding only.  With 47 classes against 256 hidden channels the two aggregations of the layer (forward
    and backward) then move 48-wide rows instead of 256-wide ones.  Both projections of x run as ONE GEMM onto
    [n, 2 Cp] (Cp = classes rounded up to 4), the aggregation reads the left half of that buffer and adds onto
    the right half, and the backward mirrors it: one buffer [A^T g | g], one GEMM for both weight gradients, one
    for grad_x.

    What crosses the partition boundary is x W_neigh^T instead of x, so with a quantised boundary exchange the
    quantisation noise would enter at a different place than in the reference: DistSAGE picks this node only
    when the exchange is exact (one partition, or 32-bit rows).
    """

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training):
        actx, w_cat, logits, ctx.dims = _project_first_forward(x, w_neigh, w_self, graph, layer, num_bits,
                                                               is_pre_delay, training)
        out = logits + bias if bias is not None else logits.contiguous()
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, w_cat)
        return out

    @staticmethod
    def backward(ctx, g):
        x, w_cat = ctx.saved_tensors
        C, Cp = ctx.dims
        G = g.new_empty((g.size(0), 2 * Cp))  # [A^T (g / in_degrees) | g], zero in the padding columns
        G[:, Cp:Cp + C] = g
        if Cp > C:
            G[:, Cp + C:] = 0
        g_bias = g.sum(0) if ctx.has_bias else None
        gx, gw_neigh, gw_self = _project_first_backward(ctx, G, x, w_cat, ctx.needs_input_grad[0])
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 5


class FusedSAGELossProjectFirst(torch.autograd.Function):
    """``FusedSAGEOutputLayerProjectFirst`` followed by the training loss, as one node:

        loss = nll_loss(log_softmax(out)[mask], labels[mask], reduction="sum") * inv_count

    (examples/graphsage/sage.py:211 and examples/graphsage/train.py:41-44).  The logits are read once: the loss
    and its gradient with respect to the logits come out of the same kernel, written straight into the buffer
    the backward aggregation and the weight-gradient GEMM read.  ``unit_grad``: the caller promises to start the
    backward pass from this loss with a gradient of exactly 1 (``loss.backward()``), which saves scaling the
    stored gradient."""

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training, labels, mask,
                inv_count, unit_grad):
        actx, w_cat, logits, ctx.dims = _project_first_forward(x, w_neigh, w_self, graph, layer, num_bits,
                                                               is_pre_delay, training)
        C, Cp = ctx.dims
        G = x.new_empty((x.size(0), 2 * Cp))
        loss, _ = ops.softmax_nll_loss(logits, bias, labels, mask, inv_count, grad=G[:, Cp:])
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.unit_grad = bool(unit_grad)
        ctx.save_for_backward(x, w_cat, G)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, g_loss):
        x, w_cat, G = ctx.saved_tensors
        C, Cp = ctx.dims
        if not ctx.unit_grad:
            G[:, Cp:].mul_(g_loss)
        g_bias = G[:, Cp:Cp + C].sum(0) if ctx.has_bias else None
        gx, gw_neigh, gw_self = _project_first_backward(ctx, G, x, w_cat, ctx.needs_input_grad[0])
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 9


class FusedSAGELossNarrowLocal(torch.autograd.Function):
    """The last layer with the reference's (possibly quantised) boundary exchange, ``FusedSAGEOutputLayer`` in its
    ``narrow_local`` form, followed by the training loss as one node: see ``FusedSAGELossProjectFirst``."""

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training, labels, mask,
                inv_count, unit_grad):
        ctx.actx, w_cat, agg_remote, logits, ctx.dims = _narrow_local_forward(x, w_neigh, w_self, graph, layer,
                                                                              num_bits, is_pre_delay, training)
        C, Cp = ctx.dims
        G = x.new_empty((x.size(0), 2 * Cp))
        loss, _ = ops.softmax_nll_loss(logits, bias, labels, mask, inv_count, grad=G[:, Cp:])
        ctx.graph = graph
        ctx.has_bias = bias is not None
        ctx.unit_grad = bool(unit_grad)
        ctx.save_for_backward(x, agg_remote, w_cat, G)
        return loss.reshape(())

    @staticmethod
    def backward(ctx, g_loss):
        x, agg_remote, w_cat, G = ctx.saved_tensors
        C, Cp = ctx.dims
        if not ctx.unit_grad:
            G[:, Cp:].mul_(g_loss)
        g_bias = G[:, Cp:Cp + C].sum(0) if ctx.has_bias else None
        gx, gw_neigh, gw_self = _narrow_local_backward(ctx, G, x, agg_remote, w_cat)
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 9
