"""Reader (and a writer, for tests and synthetic data) of the reference's on-disk
partition format, and ``load_data`` with the reference's signature
(super_gnn/data_manager/DataLoader.py:17-68, 215-278; files written by
graph_partition/postprocess_graph_multi_proc.py:110-136, 284-293):

    p{rank:03d}-{graph}_nodes.npy            int64 [n,2]  (new id, original id)
    p{rank:03d}-{graph}_local_edges.npy      int64 [2,E]  row 0 = src, row 1 = dst, local ids
    p{rank:03d}-{graph}_remote_edges.npy     int64 [2,E]  src global id, dst local id
    p{rank:03d}-{graph}_nodes_feat.npy       fp32 / fp16 [n,F]
    p{rank:03d}-{graph}_nodes_label.npy      int64 [n]
    p{rank:03d}-{graph}_nodes_{train,valid,test}_idx.npy   int64 local ids
    begin_node_on_each_partition.txt         world+1 integers on one line

``load_data`` returns the reference's dict, with every tensor on the GPU of this rank.
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist

from .CommBuffer import default_device
from .graph_builder import build_distributed_graph, order_nodes_by_degree
from .pre_post import build_distributed_graph_pre_post


def _name(input_dir, rank, graph_name, what):
    return os.path.join(input_dir, "p{:0>3d}-{}_{}.npy".format(rank, graph_name, what))


def load_graph_structures(input_dir, graph_name, rank):
    local_nodes_list = np.load(_name(input_dir, rank, graph_name, "nodes"))
    num_local_nodes = int(local_nodes_list[-1][0] - local_nodes_list[0][0] + 1)
    local_edges_list = np.load(_name(input_dir, rank, graph_name, "local_edges"))
    remote_edges_list = np.load(_name(input_dir, rank, graph_name, "remote_edges"))
    nodes_range = np.loadtxt(os.path.join(input_dir, "begin_node_on_each_partition.txt"), dtype=np.int64,
                             delimiter=" ").reshape(-1)
    return (torch.from_numpy(local_nodes_list), torch.from_numpy(local_edges_list),
            torch.from_numpy(remote_edges_list), torch.from_numpy(nodes_range), num_local_nodes)


def load_nodes_labels(input_dir, graph_name, rank):
    return torch.from_numpy(np.load(_name(input_dir, rank, graph_name, "nodes_label")))


def load_nodes_features(input_dir, graph_name, rank):
    feats = np.load(_name(input_dir, rank, graph_name, "nodes_feat"))
    if feats.dtype == np.float16:
        feats = feats.astype(np.float32)
    return torch.from_numpy(feats)


def load_dataset_mask(input_dir, graph_name, rank):
    return tuple(torch.from_numpy(np.load(_name(input_dir, rank, graph_name, f"nodes_{k}_idx")))
                 for k in ("train", "valid", "test"))


def save_partition(output_dir, graph_name, rank, begins, local_edges, remote_edges, feats, labels, train_idx,
                   valid_idx, test_idx):
    """Write one rank's files in the layout above (``begin_node_on_each_partition.txt`` by rank 0)."""
    os.makedirs(output_dir, exist_ok=True)
    lo, hi = int(begins[rank]), int(begins[rank + 1])
    ids = np.arange(lo, hi, dtype=np.int64)
    np.save(_name(output_dir, rank, graph_name, "nodes"), np.stack([ids, ids], axis=1))
    np.save(_name(output_dir, rank, graph_name, "local_edges"), np.asarray(local_edges, dtype=np.int64))
    np.save(_name(output_dir, rank, graph_name, "remote_edges"), np.asarray(remote_edges, dtype=np.int64))
    np.save(_name(output_dir, rank, graph_name, "nodes_feat"), np.asarray(feats))
    np.save(_name(output_dir, rank, graph_name, "nodes_label"), np.asarray(labels, dtype=np.int64))
    for k, v in (("train", train_idx), ("valid", valid_idx), ("test", test_idx)):
        np.save(_name(output_dir, rank, graph_name, f"nodes_{k}_idx"), np.asarray(v, dtype=np.int64))
    if rank == 0:
        np.savetxt(os.path.join(output_dir, "begin_node_on_each_partition.txt"),
                   np.asarray(list(begins), dtype=np.int64).reshape(1, -1), fmt="%d", delimiter=" ")


def load_data(config, device=None):
    """Same keys as the reference's ``load_data`` (DataLoader.py:215-278).

    ``config["node_order"] = "degree"`` (not in the reference; default: the files' numbering) renumbers this rank's
    nodes by ascending in-degree while loading (``order_nodes_by_degree``): features, labels and the train / valid /
    test index lists are returned in the new numbering, and ``"node_order"`` in the result maps new local ids to the
    files' (``order[new] = old``), for anything else that is stored per node."""
    device = device or default_device()
    input_dir = config["input_dir"]
    graph_name = config["graph_name"]
    num_bits = config["num_bits"]
    is_pre_delay = config["is_pre_delay"]
    rank = dist.get_rank() if dist.is_initialized() else 0
    max_feat_len = max(config["in_channels"], config["hidden_channels"], config["out_channels"])
    _, local_edges, remote_edges, nodes_range, _ = load_graph_structures(input_dir, graph_name, rank)
    order = None
    node_order = config.get("node_order", "file")
    if node_order == "degree":
        local_edges, remote_edges, order = order_nodes_by_degree(local_edges.to(device), remote_edges.to(device),
                                                                 nodes_range.tolist())
    elif node_order != "file":
        raise ValueError(f"node_order must be 'file' or 'degree', not {node_order!r}")
    build = build_distributed_graph_pre_post if is_pre_delay else build_distributed_graph
    graph = build(local_edges, remote_edges, nodes_range.tolist(), max_feat_len, num_bits, device=device)
    train_idx, valid_idx, test_idx = (t.to(device) for t in load_dataset_mask(input_dir, graph_name, rank))
    feats = load_nodes_features(input_dir, graph_name, rank).to(device)
    labels = load_nodes_labels(input_dir, graph_name, rank).to(device)
    out = {}
    if order is not None:
        new_of_old = torch.empty_like(order)
        new_of_old[order] = torch.arange(order.numel(), dtype=order.dtype, device=order.device)
        feats, labels = feats[order], labels[order]
        train_idx, valid_idx, test_idx = new_of_old[train_idx], new_of_old[valid_idx], new_of_old[test_idx]
        out["node_order"] = order
    out.update({
        "graph": graph,
        "nodes_features": feats,
        "nodes_labels": labels,
        "nodes_train_masks": train_idx,
        "nodes_valid_masks": valid_idx,
        "nodes_test_masks": test_idx,
    })
    return out
