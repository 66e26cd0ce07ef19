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


def test_loaded_partition_trains_with_index_lists_and_unlabelled_nodes(tmp_path):
    """``load_data`` returns the train / valid / test node INDEX lists, as the reference's does; ``train_step`` takes
    them as they are, and a node without a label (-1 in the files) that is listed for training stays out of the
    loss.  (CPU tensors over the oracle-backed op stand-ins.)"""
    import cpu_ops_emulation
    from super_gnn_b200 import graphsage
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.time_recorder import TimeRecorder

    cpu_ops_emulation.install()
    try:
        n = 40
        g = torch.Generator().manual_seed(0)
        src, dst = torch.randint(0, n, (200,), generator=g), torch.randint(0, n, (200,), generator=g)
        le, re = partition_edges(src, dst, [0, n], 0)
        labels = torch.randint(0, 3, (n,), generator=g)
        labels[5] = -1
        save_partition(str(tmp_path), "toy", 0, [0, n], le.numpy(), re.numpy(),
                       torch.randn(n, 8, generator=g).numpy(), labels.numpy(), [1, 5, 7, 9, 20], [2], [3])
        Quantizer_for_all_procs(1, 32)
        Communicator(32)
        TimeRecorder(3, 1)
        cfg = dict(input_dir=str(tmp_path), graph_name="toy", num_bits=32, is_pre_delay=False, in_channels=8,
                   hidden_channels=16, out_channels=3, num_layers=3, dropout=0.0)
        data = load_data(cfg, device=torch.device("cpu"))
        assert data["nodes_train_masks"].tolist() == [1, 5, 7, 9, 20]
        torch.manual_seed(0)
        model, opt = graphsage.create_model_and_optimizer(cfg)
        l0 = float(graphsage.train_step(model, data, opt, 4.0))
        # the same step with the unlabelled node removed from the list gives the same loss
        torch.manual_seed(0)
        model2, opt2 = graphsage.create_model_and_optimizer(cfg)
        data2 = dict(data, nodes_train_masks=torch.tensor([1, 7, 9, 20]))
        assert abs(float(graphsage.train_step(model2, data2, opt2, 4.0)) - l0) < 1e-6
        assert torch.isfinite(torch.tensor(l0))
    finally:
        cpu_ops_emulation.uninstall()


def test_loading_with_the_nodes_renumbered_by_degree_trains_to_the_same_loss(tmp_path):
    """``node_order="degree"``: features, labels and index lists follow the renumbering, so a training step gives
    the loss of the files' numbering (summation order aside), and the result says which node went where."""
    import cpu_ops_emulation
    from super_gnn_b200 import graphsage
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.time_recorder import TimeRecorder

    cpu_ops_emulation.install()
    try:
        n = 60
        g = torch.Generator().manual_seed(1)
        src, dst = torch.randint(0, n, (400,), generator=g), torch.randint(0, n, (400,), generator=g)
        le, re = partition_edges(src, dst, [0, n], 0)
        feats = torch.randn(n, 8, generator=g)
        labels = torch.randint(0, 3, (n,), generator=g)
        train = [1, 5, 7, 9, 20, 33, 41]
        save_partition(str(tmp_path), "toy", 0, [0, n], le.numpy(), re.numpy(), feats.numpy(), labels.numpy(), train,
                       [2], [3])
        Quantizer_for_all_procs(1, 32)
        Communicator(32)
        TimeRecorder(3, 1)
        cfg = dict(input_dir=str(tmp_path), graph_name="toy", num_bits=32, is_pre_delay=False, in_channels=8,
                   hidden_channels=16, out_channels=3, num_layers=3, dropout=0.0)
        losses = []
        for order in ("file", "degree"):
            data = load_data(dict(cfg, node_order=order), device=torch.device("cpu"))
            if order == "degree":
                o = data["node_order"]
                assert sorted(o.tolist()) == list(range(n))
                assert torch.equal(data["nodes_features"], feats[o]) and torch.equal(data["nodes_labels"], labels[o])
                assert sorted(o[data["nodes_train_masks"]].tolist()) == train  # the same nodes, under their new ids
                deg = data["graph"].in_degrees.squeeze(1)
                assert bool((deg[1:] >= deg[:-1]).all())
            else:
                assert "node_order" not in data
            torch.manual_seed(0)
            model, opt = graphsage.create_model_and_optimizer(cfg)
            losses.append(float(graphsage.train_step(model, data, opt, float(len(train)))))
        assert abs(losses[0] - losses[1]) < 1e-5 * max(1.0, abs(losses[0]))
        with __import__("pytest").raises(ValueError):
            load_data(dict(cfg, node_order="bfs"), device=torch.device("cpu"))
    finally:
        cpu_ops_emulation.uninstall()
