"""The driver-side pieces of full-batch GraphSAGE training that sit directly on
the hot path: the ``DistSAGE`` model (examples/graphsage/sage.py:129-211), model /
optimiser construction with the sum-allreduce DDP hook
(examples/graphsage/utils.py:9-54) and one training step = one "epoch"
(examples/graphsage/train.py:21-54).  Everything here is stock PyTorch on CUDA;
the aggregation inside every conv goes through ``Aggregator``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.nn import LayerNorm

from .fused_layer import (FusedSAGELayer, FusedSAGELossNarrowLocal, FusedSAGELossProjectFirst, FusedSAGEOutputLayer,
                          FusedSAGEOutputLayerProjectFirst, narrow_local_applies, reset_layer_buffers)
from .layers import DistSAGEConvGrad


class DistSAGE(torch.nn.Module):
    def __init__(self, in_channels, hidden_channels, out_channels, num_layers=3, dropout=0.5, num_bits=32,
                 is_pre_delay=False, norm_type="LayerNorm"):
        super().__init__()
        self.convs = torch.nn.ModuleList()
        self.norms = torch.nn.ModuleList()
        dims = [in_channels] + [hidden_channels] * (num_layers - 1) + [out_channels]
        for i in range(num_layers):
            self.convs.append(DistSAGEConvGrad(dims[i], dims[i + 1], num_bits, is_pre_delay))
            if i < num_layers - 1 and norm_type == "LayerNorm":
                self.norms.append(LayerNorm(hidden_channels))
        if norm_type not in (None, "LayerNorm"):
            raise ValueError("only norm_type=None or 'LayerNorm' is provided on this path")
        self.dropout = dropout
        self.norm_type = norm_type
        # optional fixed dropout masks (one per hidden layer) for runs that must be
        # reproducible against a CPU reference; None = native dropout
        self.dropout_masks = None
        # hidden layers as one fused autograd node (conv + dropout + LayerNorm + relu); the unfused
        # chain of framework ops is kept for comparison (fused = False) and for CPU tensors
        self.fused = True
        # last layer: project to the classes before aggregating (same function, narrower aggregation).
        # "auto" = whenever the boundary exchange is exact (one partition or 32-bit rows), so that quantised
        # runs keep the reference's place for the quantisation noise; True / False force it.
        self.project_first = "auto"
        self._dropout_calls = 0

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        for norm in self.norms:
            norm.reset_parameters()

    def _fused_ok(self, x):
        """The fused path as a whole is available (CUDA fp32 input, LayerNorm variant); each layer is then fused
        or not on its own, see ``_layer_fusable``."""
        return (self.fused and self.norm_type == "LayerNorm" and x.is_cuda and x.dtype == torch.float32
                and self.convs[0].bias is not None and self.convs[0].normalize)

    @staticmethod
    def _layer_fusable(conv, hidden: bool) -> bool:
        """The tensor-core GEMMs read rows through TMA, which wants 16-byte rows: the layer's input width must be a
        multiple of 4 (reddit's 602 input channels are not), and a hidden layer's output at most 512 wide and a
        multiple of 4 for the fused epilogue.  Other layers run as the unfused chain of framework ops."""
        if conv.in_channels % 4 != 0 or conv.bias is None or not conv.normalize:
            return False
        return (conv.out_channels % 4 == 0 and conv.out_channels <= 512) if hidden else True

    def _project_first(self, conv):
        if self.project_first != "auto":
            return bool(self.project_first)
        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        return (world == 1 or conv.num_bits == 32) and conv.out_channels < conv.in_channels and conv.in_channels % 4 == 0

    def can_fuse_loss(self, nodes_feats, graph=None) -> bool:
        """True when ``forward(..., loss_mask=, loss_inv_count=)`` returns the training loss from a fused node: fused
        CUDA path, at most 256 classes, and a last layer that either projects before it aggregates or (given the
        graph) aggregates only the remote edges at the input width."""
        last = self.convs[-1]
        if not (self._fused_ok(nodes_feats) and self._layer_fusable(last, hidden=False) and last.out_channels <= 256):
            return False
        return self._project_first(last) or (fuse_loss_narrow_local and graph is not None
                                             and narrow_local_applies(graph, last.lin_neigh.weight))

    def forward(self, graph, nodes_feats, labels=None, label_mask=None, loss_mask=None, loss_inv_count=None,
                loss_unit_grad=False):
        """Log-probabilities per node (examples/graphsage/sage.py:179-211).  With ``loss_mask`` and
        ``loss_inv_count`` (and ``can_fuse_loss``) the summed negative log-likelihood of ``labels`` over the masked
        nodes times ``loss_inv_count`` is returned instead, computed together with the last layer."""
        if self._fused_ok(nodes_feats):
            reset_layer_buffers()
            for i, conv in enumerate(self.convs[:-1]):
                mask = self.dropout_masks[i] if (self.training and self.dropout_masks is not None) else None
                if not self._layer_fusable(conv, hidden=True):
                    nodes_feats = self._unfused_hidden(graph, nodes_feats, i)
                    continue
                self._dropout_calls += 1
                rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
                seed = (torch.initial_seed() * 1_000_003 + self._dropout_calls * 8191 + rank) % (1 << 62)
                norm = self.norms[i]
                nodes_feats = FusedSAGELayer.apply(nodes_feats, conv.lin_neigh.weight,
                                                   conv.lin_self.weight, conv.bias, norm.weight, norm.bias, graph, i,
                                                   conv.num_bits, conv.is_pre_delay, self.training, float(self.dropout),
                                                   float(norm.eps), seed, mask,
                                                   i + 1 < len(self.convs) - 1
                                                   and self._layer_fusable(self.convs[i + 1], hidden=True))
            last = self.convs[-1]
            if not self._layer_fusable(last, hidden=False):
                nodes_feats = last(graph, nodes_feats, len(self.convs) - 1)
                return F.log_softmax(nodes_feats, dim=1)
            if loss_mask is not None and loss_inv_count is not None and self.can_fuse_loss(nodes_feats, graph):
                node = FusedSAGELossProjectFirst if self._project_first(last) else FusedSAGELossNarrowLocal
                return node.apply(nodes_feats, last.lin_neigh.weight,
                                  last.lin_self.weight, last.bias, graph, len(self.convs) - 1,
                                  last.num_bits, last.is_pre_delay, self.training, labels,
                                  loss_mask, float(loss_inv_count), bool(loss_unit_grad))
            node = FusedSAGEOutputLayerProjectFirst if self._project_first(last) else FusedSAGEOutputLayer
            nodes_feats = node.apply(nodes_feats, last.lin_neigh.weight,
                                     last.lin_self.weight, last.bias, graph, len(self.convs) - 1,
                                     last.num_bits, last.is_pre_delay, self.training)
            return F.log_softmax(nodes_feats, dim=1)
        for i in range(len(self.convs) - 1):
            nodes_feats = self._unfused_hidden(graph, nodes_feats, i)
        nodes_feats = self.convs[-1](graph, nodes_feats, len(self.convs) - 1)
        return F.log_softmax(nodes_feats, dim=1)

    def _unfused_hidden(self, graph, nodes_feats, i):
        """One hidden layer as the reference's chain of ops (examples/graphsage/sage.py:189-196)."""
        nodes_feats = self.convs[i](graph, nodes_feats, i)
        if self.training and self.dropout_masks is not None:
            nodes_feats = nodes_feats * self.dropout_masks[i]
        else:
            nodes_feats = F.dropout(nodes_feats, p=self.dropout, training=self.training)
        if self.norm_type is not None:
            nodes_feats = self.norms[i](nodes_feats)
        return F.relu(nodes_feats)


def allreduce_hook(process_group, bucket):
    """Sum (not mean) of the weight gradients across ranks (utils.py:9-16)."""
    group = process_group if process_group is not None else dist.group.WORLD
    return dist.all_reduce(bucket.buffer(), group=group, async_op=True).get_future().then(lambda f: f.value()[0])


def create_model_and_optimizer(config: dict, device=None):
    model = DistSAGE(config["in_channels"], config["hidden_channels"], config["out_channels"],
                     config.get("num_layers", 3), config.get("dropout", 0.5), config.get("num_bits", 32),
                     config.get("is_pre_delay", False), config.get("norm_type", "LayerNorm"))
    model.reset_parameters()
    if device is not None:
        model = model.to(device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        model = torch.nn.parallel.DistributedDataParallel(model)
        model.register_comm_hook(state=None, hook=allreduce_hook)
    optimizer = torch.optim.Adam(model.parameters(), lr=config.get("lr", 0.01),
                                 weight_decay=config.get("weight_decay", 0.0))
    return model, optimizer


def index_to_mask(index: torch.Tensor, size: int) -> torch.Tensor:
    """Boolean mask of length ``size`` that is set at ``index`` (what the reference's driver does with the node
    index lists ``load_data`` returns, examples/graphsage/train.py:125-127, through torch_geometric.utils)."""
    mask = torch.zeros(int(size), dtype=torch.bool, device=index.device)
    mask[index] = True
    return mask


def _train_mask(data) -> torch.Tensor:
    """``nodes_train_masks`` as a boolean mask; an index tensor (the form ``load_data`` returns) is converted once
    and the result kept beside it."""
    mask = data["nodes_train_masks"]
    if mask.dtype in (torch.bool, torch.uint8):
        return mask
    cached = data.get("_train_mask_from_index")
    if cached is None or cached[0] is not mask:
        cached = data["_train_mask_from_index"] = (mask, index_to_mask(mask, data["nodes_labels"].numel()))
    return cached[1]


fuse_loss = True  # module switch: False keeps log_softmax / nll_loss as framework ops after the model
fuse_loss_narrow_local = True  # the same for several partitions with the reference's boundary exchange


def train_step(model, data, optimizer, num_train_nodes: float):
    """One full-batch training step (train.py:21-54): forward, summed NLL over the
    training nodes divided by the global count, backward, Adam."""
    model.train()
    optimizer.zero_grad()
    mask = _train_mask(data)
    labels = data["nodes_labels"]
    core = model.module if hasattr(model, "module") else model
    if fuse_loss and core.can_fuse_loss(data["nodes_features"], data["graph"]):
        # log_softmax, the masked NLL sum and their gradient computed with the last layer, in one pass over the logits
        loss = model(data["graph"], data["nodes_features"], labels, None, loss_mask=mask,
                     loss_inv_count=1.0 / num_train_nodes, loss_unit_grad=True)
        loss.backward()
        optimizer.step()
        return loss
    out = model(data["graph"], data["nodes_features"], labels, None)
    mask = mask.bool() & (labels >= 0) & (labels < out.size(1))  # an unlabelled node (-1) is out of the loss
    if out.is_cuda:
        # same sum as nll_loss(out[mask], labels[mask], "sum"), without compacting the masked rows: boolean
        # indexing costs a device->host synchronisation and two passes over the [n, classes] logits each way
        per_node = F.nll_loss(out, torch.where(mask, labels, torch.zeros_like(labels)), reduction="none")
        loss = (per_node * mask).sum() / num_train_nodes
    else:
        loss = F.nll_loss(out[mask], labels[mask], reduction="sum") / num_train_nodes
    loss.backward()
    optimizer.step()
    return loss
