"""One hidden GraphSAGE layer as a single autograd node:

    y = relu(LayerNorm(dropout(lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias)))

the composition of DistSAGEConvGrad.forward (super_gnn/layers/sageconv.py:62-89) with the
dropout / LayerNorm / relu that follow it in DistSAGE.forward
(examples/graphsage/sage.py:189-196).  Same parameters, same math; what changes is the
number of passes over the [n, hidden] activations and where the dense products run: the two
linear maps and their gradients are fp32-accurate tensor-core GEMMs (``ops.gemm_nt`` /
``ops.gemm_tn``), their sum is taken inside the epilogue kernel, the four elementwise /
normalisation ops run as one kernel each way, and the backward aggregation accumulates into
the self-path gradient in place.  Saved for the backward: the aggregated input, x_hat (stored
over the GEMM output), y (which the next layer needs anyway) and one reciprocal standard
deviation per row; the dropout mask is regenerated from its seed.
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
    return Aggregator.backward(ctx.actx, g_agg, accumulate_into=gx)[1]


class FusedSAGELayer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, gamma, beta, graph, layer, num_bits, is_pre_delay, training, p, eps,
                seed, mask):
        actx = _AggCtx()
        agg = Aggregator.forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        h = ops.gemm_nt(agg, w_neigh)
        h_self = ops.gemm_nt(x, w_self)
        y, rstd = ops.sage_epilogue_forward(h, bias, gamma, beta, p, training, seed, eps, mask, h2=h_self)
        del h_self
        ctx.actx, ctx.graph = actx, graph
        ctx.cfg = (training, p, seed)
        ctx.has_mask = mask is not None
        saved = [x, agg, h, y, rstd, w_neigh, w_self, gamma] + ([mask] if mask is not None else [])
        ctx.save_for_backward(*saved)
        return y

    @staticmethod
    def backward(ctx, gy):
        saved = ctx.saved_tensors
        x, agg, xhat, y, rstd, w_neigh, w_self, gamma = saved[:8]
        mask = saved[8] if ctx.has_mask else None
        training, p, seed = ctx.cfg
        gy = gy if gy.stride(-1) == 1 else gy.contiguous()
        gh, g_bias, g_gamma, g_beta = ops.sage_epilogue_backward(gy, y, xhat, rstd, gamma, p, training, seed, mask)
        gw_neigh = ops.gemm_tn(gh, agg)
        gw_self = ops.gemm_tn(gh, x)
        gx = None
        if ctx.needs_input_grad[0]:
            gx = _input_grad(ctx, gh, w_neigh, w_self)
        return (gx, gw_neigh, gw_self, g_bias, g_gamma, g_beta) + (None,) * 9


class FusedSAGEOutputLayer(torch.autograd.Function):
    """The last layer, ``lin_neigh(Aggregator(x) / in_degrees) + lin_self(x) + bias`` (no normalisation,
    dropout or relu follows it), as one autograd node: same in-place accumulations as the hidden layers, so
    the [n, hidden] gradient is not summed from two separately materialised parts."""

    @staticmethod
    def forward(ctx, x, w_neigh, w_self, bias, graph, layer, num_bits, is_pre_delay, training):
        actx = _AggCtx()
        agg = Aggregator.forward(actx, graph, x, layer, num_bits, is_pre_delay, training)
        if not getattr(graph, "fold_mean", False):
            agg.div_(graph.in_degrees)
        out = torch.mm(agg, w_neigh.t())
        out.addmm_(x, w_self.t())
        if bias is not None:
            out.add_(bias)
        ctx.actx, ctx.graph = actx, graph
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, agg, w_neigh, w_self)
        return out

    @staticmethod
    def backward(ctx, g):
        x, agg, w_neigh, w_self = ctx.saved_tensors
        g = g.contiguous()
        gw_neigh = torch.mm(g.t(), agg)
        gw_self = torch.mm(g.t(), x)
        g_bias = g.sum(0) if ctx.has_bias else None
        gx = None
        if ctx.needs_input_grad[0]:
            g_agg = torch.mm(g, w_neigh)
            if not getattr(ctx.graph, "fold_mean", False):
                g_agg.div_(ctx.graph.in_degrees)
            gx = Aggregator.backward(ctx.actx, g_agg)[1]
            gx.addmm_(g, w_self)
        return (gx, gw_neigh, gw_self, g_bias) + (None,) * 5
