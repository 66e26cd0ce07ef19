"""CPU restatement of one full-batch GraphSAGE training step ("epoch") of the
reference, single process — TEST INFRASTRUCTURE AND TIMED CPU BASELINE ONLY.

The aggregation runs on the reference's own compiled ``supergnn_ops.spmm``
(``oracle/_ref``, built by build_ref.py) when it is present and this host can
run it, otherwise on the C oracle; the rest is stock PyTorch on the CPU, layer
for layer as in the reference:

* Aggregator, world_size 1: out = A x, grad = A^T g   (super_gnn/aggregator.py:62-65, 145-148)
  with the nnz-balanced per-thread row split            (super_gnn/ops/spmm_kernel.py:8-29)
* DistSAGEConvGrad: out /= in_degrees; lin_neigh(out) + lin_self(x) + bias
                                                         (super_gnn/layers/sageconv.py:62-89)
* DistSAGE: conv -> dropout -> LayerNorm -> relu ... -> log_softmax
                                                         (examples/graphsage/sage.py:179-211)
* train_step: summed NLL / #train nodes, backward, Adam  (examples/graphsage/train.py:21-54)
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))
if _HERE not in sys.path:
    sys.path.insert(0, _HERE)
if os.path.dirname(_HERE) not in sys.path:
    sys.path.insert(0, os.path.dirname(_HERE))


def load_backend(prefer_reference: bool = True):
    """Returns (kind, spmm_fn): kind is "reference" (the compiled reference op) or "port"."""
    import oracle as port

    if prefer_reference:
        try:
            import build_ref

            ref = build_ref.load()

            def spmm_ref(csr, x, out):
                ref.spmm(csr["rowptr"], csr["col"], csr["val"], x, out, csr["rowptr"].numel() - 1, csr["splits"],
                         torch.tensor([0, x.size(1)], dtype=torch.int32))

            return "reference", spmm_ref
        except Exception:  # not built, or the host lacks the ISA the build enables
            pass

    def spmm_port(csr, x, out):
        port.spmm(csr["rowptr"].numpy(), csr["col"].numpy(), csr["val"].numpy(), x.detach().numpy(), out.numpy())

    return "port", spmm_port


def make_csr(rowptr: torch.Tensor, col: torch.Tensor, num_threads: int) -> dict:
    """Reference layout: int64 rowptr/col, explicit fp32 ones, one row range per thread."""
    import oracle as port

    rowptr = rowptr.to(torch.int64).contiguous()
    col = col.to(torch.int64).contiguous()
    val = torch.ones(col.numel(), dtype=torch.float32)
    splits = torch.from_numpy(port.distribute_work_for_row(rowptr.numpy(), val.numpy(), num_threads))
    return dict(rowptr=rowptr, col=col, val=val, splits=splits)


def transpose_csr(rowptr: torch.Tensor, col: torch.Tensor, num_cols: int):
    col = col.to(torch.int64)
    M = rowptr.numel() - 1
    row = torch.repeat_interleave(torch.arange(M, dtype=torch.int64), rowptr[1:] - rowptr[:-1])
    order = torch.sort(col, stable=True).indices
    colptr = torch.zeros(num_cols + 1, dtype=torch.int64)
    torch.cumsum(torch.bincount(col, minlength=num_cols), 0, out=colptr[1:])
    return colptr, row[order]


class CpuGraph:
    def __init__(self, rowptr, col, num_nodes, num_threads):
        self.n = num_nodes
        self.fwd = make_csr(rowptr, col, num_threads)
        colptr, row_T = transpose_csr(rowptr.to(torch.int64), col, num_nodes)
        self.bwd = make_csr(colptr, row_T, num_threads)
        self.in_degrees = (rowptr[1:] - rowptr[:-1]).to(torch.float32).clamp(min=1).unsqueeze(-1)


class CpuAggregator(torch.autograd.Function):
    spmm = None

    @staticmethod
    def forward(ctx, graph, x):
        ctx.graph = graph
        out = torch.zeros((graph.n, x.size(1)), dtype=torch.float32)
        CpuAggregator.spmm(graph.fwd, x.contiguous(), out)
        return out

    @staticmethod
    def backward(ctx, g):
        graph = ctx.graph
        out = torch.zeros((graph.n, g.size(1)), dtype=torch.float32)
        CpuAggregator.spmm(graph.bwd, g.contiguous(), out)
        return None, out


class CpuSAGE(torch.nn.Module):
    def __init__(self, in_channels, hidden, out_channels, num_layers=3, dropout=0.5):
        super().__init__()
        dims = [in_channels] + [hidden] * (num_layers - 1) + [out_channels]
        self.lin_neigh = torch.nn.ModuleList([torch.nn.Linear(dims[i], dims[i + 1], bias=False) for i in range(num_layers)])
        self.lin_self = torch.nn.ModuleList([torch.nn.Linear(dims[i], dims[i + 1], bias=False) for i in range(num_layers)])
        self.bias = torch.nn.ParameterList([torch.nn.Parameter(torch.zeros(dims[i + 1])) for i in range(num_layers)])
        self.norms = torch.nn.ModuleList([torch.nn.LayerNorm(hidden) for _ in range(num_layers - 1)])
        self.dropout = dropout
        self.dropout_masks = None
        gain = torch.nn.init.calculate_gain("relu")
        for l in list(self.lin_neigh) + list(self.lin_self):
            torch.nn.init.xavier_uniform_(l.weight, gain=gain)

    def load_from(self, state: dict):
        """Copy the weights of a ``super_gnn_b200.graphsage.DistSAGE`` state dict."""
        with torch.no_grad():
            for i in range(len(self.lin_neigh)):
                self.lin_neigh[i].weight.copy_(state[f"convs.{i}.lin_neigh.weight"])
                self.lin_self[i].weight.copy_(state[f"convs.{i}.lin_self.weight"])
                self.bias[i].copy_(state[f"convs.{i}.bias"])
            for i in range(len(self.norms)):
                self.norms[i].weight.copy_(state[f"norms.{i}.weight"])
                self.norms[i].bias.copy_(state[f"norms.{i}.bias"])

    def conv(self, i, graph, x):
        out = CpuAggregator.apply(graph, x)
        out = out / graph.in_degrees
        out = self.lin_neigh[i](out)
        out = out + self.lin_self[i](x)
        return out + self.bias[i]

    def forward(self, graph, x):
        L = len(self.lin_neigh)
        for i in range(L - 1):
            x = self.conv(i, graph, x)
            if self.training and self.dropout_masks is not None:
                x = x * self.dropout_masks[i]
            else:
                x = F.dropout(x, p=self.dropout, training=self.training)
            x = self.norms[i](x)
            x = F.relu(x)
        return F.log_softmax(self.conv(L - 1, graph, x), dim=1)


def train_step(model, graph, feats, labels, train_mask, optimizer, num_train_nodes):
    model.train()
    optimizer.zero_grad()
    out = model(graph, feats)
    loss = F.nll_loss(out[train_mask], labels[train_mask], reduction="sum") / num_train_nodes
    loss.backward()
    optimizer.step()
    return loss
