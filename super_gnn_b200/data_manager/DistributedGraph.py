"""Per-rank graph containers read by the Aggregator
(super_gnn/data_manager/DistributedGraph.py:9-89)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from ..sparse import SparseTensor
from .CommBuffer import CommBuffer, CommBufferForQuantization
from .CommSplits import CommSplits


def _in_degrees_of(adjs, num_local_nodes, device, clamp: bool):
    degs = torch.zeros(num_local_nodes, dtype=torch.float32, device=device)
    for adj in adjs:
        rowptr = adj.storage.rowptr()
        degs += (rowptr[1:] - rowptr[:-1]).to(torch.float32)
    if clamp:
        degs = degs.clamp(min=1)
    return degs.unsqueeze(-1)


class _MeanFolding:
    """``fold_mean = True`` asks the Aggregator to return the MEAN over the in-neighbours
    (sum x 1/in_degree, applied inside the SpMM kernels) instead of the sum; the layer
    then skips its own division (super_gnn/layers/sageconv.py:76-78)."""

    fold_mean = False

    def set_fold_mean(self, flag: bool = True):
        self.fold_mean = bool(flag)
        self.inv_in_degrees = (1.0 / self.in_degrees).reshape(-1).contiguous() if flag else None
        return self


class DistributedGraph(_MeanFolding):
    def __init__(self, local_adj_t: SparseTensor, remote_adj_t: SparseTensor, idx_nodes_send_to_others: Tensor,
                 num_nodes_send_to_others: list, num_nodes_recv_from_others: list, in_degrees: Tensor,
                 comm_splits: CommSplits, comm_buf: CommBuffer,
                 comm_buf_for_quantization: Optional[CommBufferForQuantization]) -> None:
        self.local_adj_t = local_adj_t
        self.remote_adj_t = remote_adj_t
        self.idx_nodes_send_to_others = idx_nodes_send_to_others
        self.num_nodes_send_to_others = num_nodes_send_to_others
        self.num_nodes_recv_from_others = num_nodes_recv_from_others
        self.in_degrees = in_degrees
        self.comm_splits = comm_splits
        self.comm_buf = comm_buf
        self.comm_buf_for_quantization = comm_buf_for_quantization

    def get_in_degrees(self):
        """Unclamped in-degrees over local and remote edges (DistributedGraph.py:36-49)."""
        n = self.local_adj_t.sparse_sizes()[0]
        self.in_degrees = _in_degrees_of([self.local_adj_t, self.remote_adj_t], n, self.local_adj_t.device, False)
        return self.in_degrees


class DistributedGraphForPre(_MeanFolding):
    def __init__(self, local_adj_t: SparseTensor, adj_t_pre_post_aggr_from: SparseTensor,
                 adj_t_pre_post_aggr_to: SparseTensor, pre_post_aggr_from_splits: list,
                 pre_post_aggr_to_splits: list, in_degrees: Tensor, comm_splits: CommSplits, comm_buf: CommBuffer,
                 comm_buf_for_quantization: Optional[CommBufferForQuantization]) -> None:
        self.local_adj_t = local_adj_t
        self.adj_t_pre_post_aggr_from = adj_t_pre_post_aggr_from
        self.adj_t_pre_post_aggr_to = adj_t_pre_post_aggr_to
        self.pre_post_aggr_from_splits = pre_post_aggr_from_splits
        self.pre_post_aggr_to_splits = pre_post_aggr_to_splits
        self.in_degrees = in_degrees
        self.comm_splits = comm_splits
        self.comm_buf = comm_buf
        self.comm_buf_for_quantization = comm_buf_for_quantization
