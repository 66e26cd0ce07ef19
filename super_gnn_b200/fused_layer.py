"""One hidden GraphSAGE layer as a single autograd node:

    y = relu(LayerNorm(dropout(lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias)))

the composition of DistSAGEConvGrad.forward (super_gnn/layers/sageconv.py:62-89) with the
dropout / LayerNorm / relu that follow it in DistSAGE.forward
(examples/graphsage/sage.py:189-196).  Same parameters, same math; what changes is the
number of passes over the [n, hidden] activations and where the dense products run: the two
linear maps and their gradients are fp32-accurate tensor-core GEMMs (``ops.gemm_nt`` /
``ops.gemm_tn``), the second map accumulates into the first one's output (beta = 1), the four
elementwise / normalisation ops run as one kernel each way, and the backward aggregation accumulates into
the self-path gradient in place.  Saved for the backward: the aggregated input, the GEMM output
h and two numbers per row (mean, reciprocal standard deviation); the normalised values, the
sign of the output and the dropout mask are recomputed from those.
"""
from __future__ import annotations

import torch

from . import supergnn_ops as ops
from .aggregator import Aggregator


class _AggCtx:
    """Stand-in for the autograd context the Aggregator's static methods write to."""


def _input_grad(ctx, g, w_neigh, w_self):
    """grad_x = Aggregator^T(g W_neigh / in_degrees) + g W_self: the self path is written first and the backward
    aggregation adds onto it."""
    g_agg = ops.gemm_nt(g, w_neigh.t().contiguous())
    if not getattr(ctx.graph, "fold_mean", False):
        g_agg.div_(ctx.graph.in_degrees)
    gx = ops.gemm_nt(g, w_self.t().contiguous())
    return Aggregator.backward(ctx.actx, g_agg, out=gx, accumulate=True)[1]


class FusedSAGELayer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, gamma, beta, graph, layer, num_bits, is_pre_delay, training, p, eps,
                seed, mask):
        actx = _AggCtx()
        agg = Aggregator.forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        h = ops.gemm_nt(agg, w_neigh)
        ops.gemm_nt(x, w_self, out=h, beta=1.0)
        y, stats = ops.sage_epilogue_forward(h, bias, gamma, beta, p, training, seed, eps, mask)
        ctx.actx, ctx.graph = actx, graph
        ctx.cfg = (training, p, seed)
        ctx.has_mask = mask is not None
        saved = [x, agg, h, stats, w_neigh, w_self, bias, gamma, beta] + ([mask] if mask is not None else [])
        ctx.save_for_backward(*saved)
        return y

    @staticmethod
    def backward(ctx, gy):
        saved = ctx.saved_tensors
        x, agg, h, stats, w_neigh, w_self, bias, gamma, beta = saved[:9]
        mask = saved[9] if ctx.has_mask else None
        training, p, seed = ctx.cfg
        gy = gy if gy.stride(-1) == 1 else gy.contiguous()
        gh, g_bias, g_gamma, g_beta = ops.sage_epilogue_backward(gy, h, stats, bias, gamma, beta, p, training, seed,
                                                                 mask)
        gw_neigh = ops.gemm_tn(gh, agg)
        gw_self = ops.gemm_tn(gh, x)
        gx = None
        if ctx.needs_input_grad[0]:
            gx = _input_grad(ctx, gh, w_neigh, w_self)
        return (gx, gw_neigh, gw_self, g_bias, g_gamma, g_beta) + (None,) * 9


def _pad_rows(w, rows):
    """[rows, K] copy of the [C, K] weight with zero rows appended (C is rounded up to a multiple of 4 so that the
    class dimension meets the GEMM's 16-byte row rule)."""
    if w.size(0) == rows:
        return w
    out = w.new_zeros((rows, w.size(1)))
    out[:w.size(0)] = w
    return out


class FusedSAGEOutputLayer(torch.autograd.Function):
    """The last layer, ``lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias`` (no normalisation,
    dropout or relu follows it), in the reference's order (aggregate, then project) as one autograd node: the
    same tensor-core GEMMs and in-place accumulations as the hidden layers, with the class dimension padded to
    a multiple of 4 inside the node."""

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training):
        actx = _AggCtx()
        agg = Aggregator.forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        C = w_neigh.size(0)
        Cp = (C + 3) // 4 * 4
        wn, ws = _pad_rows(w_neigh, Cp), _pad_rows(w_self, Cp)
        out = ops.gemm_nt(agg, wn)
        ops.gemm_nt(x, ws, out=out, beta=1.0)
        out = out[:, :C] + bias if bias is not None else out[:, :C].contiguous()
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.dims = (C, Cp)
        ctx.save_for_backward(x, agg, wn, ws)
        return out

    @staticmethod
    def backward(ctx, g):
        x, agg, wn, ws = ctx.saved_tensors
        C, Cp = ctx.dims
        g_bias = g.sum(0) if ctx.has_bias else None
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
            gx = Aggregator.backward(ctx.actx, g_agg, out=gx, accumulate=True)[1]
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 5


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
        C, K = w_neigh.shape
        Cp = (C + 3) // 4 * 4
        w_cat = x.new_zeros((2 * Cp, K))
        w_cat[:C] = w_neigh
        w_cat[Cp:Cp + C] = w_self
        zs = ops.gemm_nt(x, w_cat)  # [n, 2 Cp] = [x W_neigh^T | x W_self^T]
        actx = _AggCtx()
        fold = getattr(graph, "fold_mean", False)
        if fold:
            Aggregator.forward(actx, graph, zs[:, :Cp], layer, num_bits, is_pre_delay, training, out=zs[:, Cp:],
                               accumulate=True)
            out = zs[:, Cp:Cp + C]
        else:
            agg = Aggregator.forward(actx, graph, zs[:, :Cp], layer, num_bits, is_pre_delay, training)
            out = agg.div_(graph.in_degrees)[:, :C] + zs[:, Cp:Cp + C]
        out = out + bias if bias is not None else out.contiguous()
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.dims = (C, Cp)
        ctx.save_for_backward(x, w_cat)
        return out

    @staticmethod
    def backward(ctx, g):
        x, w_cat = ctx.saved_tensors
        C, Cp = ctx.dims
        n = g.size(0)
        G = g.new_empty((n, 2 * Cp))  # [A^T (g / in_degrees) | g], zero in the padding columns
        G[:, Cp:Cp + C] = g
        if Cp > C:
            G[:, Cp + C:] = 0
        g_bias = g.sum(0) if ctx.has_bias else None
        g_in = G[:, Cp:]
        if not getattr(ctx.graph, "fold_mean", False):
            g_in = g_in / ctx.graph.in_degrees
        Aggregator.backward(ctx.actx, g_in, out=G[:, :Cp], accumulate=False)
        gw = ops.gemm_tn(G, x)  # [2 Cp, K]: rows of grad W_neigh, then of grad W_self
        gx = ops.gemm_nt(G, w_cat.t().contiguous()) if ctx.needs_input_grad[0] else None
        return (gx, gw[:C], gw[Cp:Cp + C], g_bias) + (None,) * 5
