"""Pre/post-aggregation planner and graph builder (``is_pre_delay=True``).

For receiver rank r and source rank i, each cross edge (src on i -> dst on r) is
classified by a minimum vertex cover of the bipartite cross-edge graph
(super_gnn/data_manager/DataProcessor.py:259-281): src in the cover => **post**
(the raw src row is shipped once and aggregated on r); otherwise => **pre** (rank
i sums its src rows per dst and ships one partial-sum row per dst).  The rows
shipped per pair then number |cover|, the minimum possible.

Same outputs as the reference's DataProcessorForPreAggresive
(DataProcessor.py:138-541) + DataLoader.get_distributed_graph_for_pre_aggressive
(DataLoader.py:131-212), without its per-edge Python loops and its Python
Hopcroft-Karp: the cover is computed by the native
``sgnn_bipartite_min_vertex_cover`` and everything else is sort / unique on
tensors.  Ordering contract (both ends sort the same key set): within a peer,
rows on the wire are in ascending key order, key = global src id for a post row,
global dst id for a pre row.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import _cabi
from ..sparse import SparseTensor
from .CommBuffer import CommBuffer, CommBufferForQuantization, default_device
from .CommSplits import CommSplits
from .DistributedGraph import DistributedGraphForPre
from .graph_builder import _exchange, _world


def min_vertex_cover(src: torch.Tensor, dst: torch.Tensor):
    """Minimum vertex cover of the bipartite graph with edges (src[e], dst[e]).

    Returns ``(src_in_cover bool[E], cover_size)``: the per-edge flag "source is in
    the cover" (=> post aggregation).  König's construction from the unmatched
    sources, so the cover does not depend on the matching found."""
    E = src.numel()
    if E == 0:
        return torch.zeros(0, dtype=torch.bool), 0
    src = src.cpu()
    dst = dst.cpu()
    us, inv_s = torch.unique(src, sorted=True, return_inverse=True)
    ud, inv_d = torch.unique(dst, sorted=True, return_inverse=True)
    order = torch.sort(inv_s * ud.numel() + inv_d).indices  # by (left, right): deterministic adjacency order
    rowptr = torch.zeros(us.numel() + 1, dtype=torch.int64)
    torch.cumsum(torch.bincount(inv_s, minlength=us.numel()), 0, out=rowptr[1:])
    col = inv_d[order].to(torch.int32).contiguous()
    cover_l = torch.zeros(us.numel(), dtype=torch.uint8)
    cover_r = torch.zeros(ud.numel(), dtype=torch.uint8)
    size = ctypes.c_int64(0)
    rc = _cabi.lib().sgnn_bipartite_min_vertex_cover(us.numel(), ud.numel(), rowptr.data_ptr(), col.data_ptr(),
                                                     cover_l.data_ptr(), cover_r.data_ptr(), ctypes.addressof(size))
    _cabi.check(rc, "bipartite_min_vertex_cover")
    return cover_l.bool()[inv_s], int(size.value)


def decide_pre_or_post_aggr(src: torch.Tensor, dst: torch.Tensor):
    """(pre_aggr_edge_idx, post_aggr_edge_idx) like DataProcessor.decide_pre_or_post_aggr_v2."""
    post, _ = min_vertex_cover(src, dst)
    idx = torch.arange(src.numel(), dtype=torch.int64)
    return idx[~post], idx[post]


def _dense_rank(peer: torch.Tensor, key: torch.Tensor, num_nodes_total: int, world: int):
    """Rank of every (peer, key) pair in the ascending list of distinct pairs, and the
    number of distinct keys per peer."""
    comp = peer * num_nodes_total + key
    uniq, inv = torch.unique(comp, sorted=True, return_inverse=True)
    per_peer = torch.bincount(uniq // num_nodes_total, minlength=world)
    return inv, per_peer.tolist()


def _first_occurrence(comp: torch.Tensor) -> torch.Tensor:
    """Mask that keeps the first element of every distinct value of ``comp``."""
    if comp.numel() == 0:
        return torch.zeros(0, dtype=torch.bool)
    _, inv = torch.unique(comp, return_inverse=True)
    firsts = torch.zeros(int(inv.max()) + 1, dtype=torch.int64).scatter_reduce(
        0, inv, torch.arange(inv.numel()), "amin", include_self=False)
    mask = torch.zeros(inv.numel(), dtype=torch.bool)
    mask[firsts] = True
    return mask


def rows_to_request(src, dst, post, peer=None, num_nodes_total: int = 1 << 40):
    """What the source ranks must produce, as (peer, src, key) in ascending (peer, key) order:
    every pre edge as (src, key = dst) and every post source once as (src, key = src)
    (DataProcessor.collect_edges_sent_to_other_subgraphs, DataProcessor.py:285-312)."""
    peer = torch.zeros_like(src) if peer is None else peer
    pre = ~post
    post_once = _first_occurrence(peer[post] * num_nodes_total + src[post])
    req_peer = torch.cat([peer[pre], peer[post][post_once]])
    req_src = torch.cat([src[pre], src[post][post_once]])
    req_key = torch.cat([dst[pre], src[post][post_once]])
    order = torch.sort(req_peer * num_nodes_total + req_key, stable=True).indices
    return req_peer[order], req_src[order], req_key[order]


def rows_to_aggregate(src, dst, post, peer=None, num_nodes_total: int = 1 << 40):
    """What the receiver aggregates, as (peer, key, dst) in ascending (peer, key) order: post edges
    (key = src -> dst) and ONE identity edge per pre-summed destination (key = dst -> dst)
    (DataProcessor.collect_edges_for_aggregation, DataProcessor.py:316-359)."""
    peer = torch.zeros_like(src) if peer is None else peer
    pre = ~post
    pre_once = _first_occurrence(peer[pre] * num_nodes_total + dst[pre])
    from_peer = torch.cat([peer[post], peer[pre][pre_once]])
    from_key = torch.cat([src[post], dst[pre][pre_once]])
    from_dst = torch.cat([dst[post], dst[pre][pre_once]])
    order = torch.sort(from_peer * num_nodes_total + from_key, stable=True).indices
    return from_peer[order], from_key[order], from_dst[order]


def build_distributed_graph_pre_post(local_edges: torch.Tensor, remote_edges: torch.Tensor, begins: Sequence[int],
                                     max_feat_len: int, bits: int, device: Optional[torch.device] = None,
                                     with_values: bool = False) -> DistributedGraphForPre:
    """This rank's :class:`DistributedGraphForPre` (collective when world_size > 1).
    Edge lists as for ``build_distributed_graph``: ``[2,E]``, row 0 = source (local id
    for local edges, global id for remote edges), row 1 = local destination id."""
    device = device or default_device()
    rank, world = _world()
    n_total = int(begins[-1])
    lo = int(begins[rank])
    n = int(begins[rank + 1]) - lo
    begins_t = torch.as_tensor(list(begins), dtype=torch.int64)
    local_edges = local_edges.to(device)
    r_src = remote_edges[0].cpu()
    r_dst = remote_edges[1].cpu() + lo  # global destination ids, as the reference restores them

    deg = torch.bincount(local_edges[1], minlength=n).cpu() + torch.bincount(remote_edges[1].cpu(), minlength=n)
    in_degrees = deg.to(torch.float32).clamp(min=1).unsqueeze(-1).to(device)

    owner = torch.searchsorted(begins_t, r_src, right=True) - 1  # source rank of every remote edge
    post = torch.zeros(r_src.numel(), dtype=torch.bool)
    for i in range(world):
        sel = (owner == i).nonzero(as_tuple=True)[0]
        if sel.numel():
            post[sel], _ = min_vertex_cover(r_src[sel], r_dst[sel])

    from_peer, from_key, from_dst = rows_to_aggregate(r_src, r_dst, post, owner, n_total)
    from_col, recv_splits = _dense_rank(from_peer, from_key, n_total, world)
    from_dst = from_dst - lo
    R = sum(recv_splits)

    req_peer, req_src, req_key = rows_to_request(r_src, r_dst, post, owner, n_total)
    send_counts = torch.bincount(req_peer, minlength=world).tolist()  # pairs requested from every source rank

    if world > 1:
        dev_comm = device
        counts = _exchange(torch.tensor(send_counts, dtype=torch.int64, device=dev_comm), [1] * world, [1] * world)
        recv_counts = counts.tolist()
        got_src = _exchange(req_src.to(dev_comm), send_counts, recv_counts).cpu()
        got_key = _exchange(req_key.to(dev_comm), send_counts, recv_counts).cpu()
    else:
        recv_counts = [0] * world
        got_src = torch.empty(0, dtype=torch.int64)
        got_key = torch.empty(0, dtype=torch.int64)
    got_peer = torch.repeat_interleave(torch.arange(world), torch.tensor(recv_counts, dtype=torch.int64))
    to_row, send_splits = _dense_rank(got_peer, got_key, n_total, world)
    S = sum(send_splits)

    ones = (lambda e: torch.ones(e, dtype=torch.float32, device=device)) if with_values else (lambda e: None)
    local_adj_t = SparseTensor(row=local_edges[1], col=local_edges[0], value=ones(local_edges.size(1)),
                               sparse_sizes=(n, n))
    adj_from = SparseTensor(row=from_dst.to(device), col=from_col.to(device), value=ones(from_dst.numel()),
                            sparse_sizes=(n, R))
    adj_to = SparseTensor(row=to_row.to(device), col=(got_src - lo).to(device), value=ones(to_row.numel()),
                          sparse_sizes=(S, n))

    comm_splits = CommSplits(recv_splits, send_splits, world, bits)
    comm_buf = CommBuffer(comm_splits, max_feat_len, bits, device=device)
    qbuf = CommBufferForQuantization(comm_splits, max_feat_len, bits, device=device) if bits in (2, 4, 8) else None
    return DistributedGraphForPre(local_adj_t, adj_from, adj_to, recv_splits, send_splits, in_degrees, comm_splits,
                                  comm_buf, qbuf)
