"""On-disk partition format: write a 2-rank partition of a small graph, read it back with
``load_data`` (world_size 1 view of rank 0) and check the graph fields against the
hand-derived expectations of the reference's tests/test_data_preprocessor.py style."""
import torch

from super_gnn_b200 import synthetic
from super_gnn_b200.data_manager import load_data, partition_edges, save_partition
from super_gnn_b200.data_manager.DataLoader import load_graph_structures
from super_gnn_b200.quantizer import Quantizer_for_all_procs


def test_round_trip_and_graph_fields(tmp_path):
    n, W = 10, 2
    src = torch.tensor([0, 1, 2, 7, 8, 9, 5, 6, 3, 3])
    dst = torch.tensor([1, 2, 0, 0, 0, 4, 6, 5, 8, 9])
    begins = synthetic.even_ranges(n, W)
    feats = torch.arange(n * 3, dtype=torch.float32).reshape(n, 3)
    labels = torch.arange(n) % 4
    for r in range(W):
        le, re = partition_edges(src, dst, begins, r)
        lo, hi = begins[r], begins[r + 1]
        save_partition(str(tmp_path), "toy", r, begins, le.numpy(), re.numpy(), feats[lo:hi].numpy().astype("float16"),
                       labels[lo:hi].numpy(), [0, 1], [2], [3, 4])
    nodes, le, re, rng, n_local = load_graph_structures(str(tmp_path), "toy", 0)
    assert n_local == 5 and rng.tolist() == [0, 5, 10]
    assert le.tolist() == [[0, 1, 2], [1, 2, 0]]            # local edges of rank 0, local ids
    assert re.tolist() == [[7, 8, 9], [0, 0, 4]]            # remote sources keep their global id
    Quantizer_for_all_procs(1, 32)
    cfg = dict(input_dir=str(tmp_path), graph_name="toy", num_bits=32, is_pre_delay=False, in_channels=3,
               hidden_channels=4, out_channels=2)
    data = load_data(cfg, device=torch.device("cpu"))
    g = data["graph"]
    assert data["nodes_features"].dtype == torch.float32 and data["nodes_features"].shape == (5, 3)
    assert data["nodes_train_masks"].tolist() == [0, 1]
    assert g.local_adj_t.sparse_sizes() == (5, 5) and g.remote_adj_t.sparse_sizes() == (5, 3)
    assert g.in_degrees.squeeze(1).tolist() == [3.0, 1.0, 1.0, 1.0, 1.0]   # clamped to >= 1
    rowptr, col, _ = g.remote_adj_t.csr()
    assert rowptr.tolist() == [0, 2, 2, 2, 2, 3] and col.tolist() == [0, 1, 2]   # remote ids in ascending global order
    assert g.comm_splits.recv_splits == [0, 3]  # rows wanted from partition 0 (itself) and from partition 1
