"""Graph construction against the reference's own known answers for its DataProcessor steps
(tests/test_data_preprocessor.py:10-26 and :41-100 of the reference: inputs and expected outputs are those
tests', re-typed), and the one-call device builder against the composition of the steps."""
import torch

from super_gnn_b200.data_manager import graph_builder as gb
from super_gnn_b200.data_manager import build_distributed_graph


def test_sort_remote_edges_by_source_known_answer():
    edges = torch.tensor([[3, 2, 1, 4, 0, 0], [6, 5, 8, 7, 9, 10]])
    got = gb.sort_remote_edges_list_based_on_remote_nodes(edges)
    assert torch.equal(got, torch.tensor([[0, 0, 1, 2, 3, 4], [9, 10, 8, 5, 6, 7]]))


def test_remote_nodes_list_known_answer():
    edges = torch.tensor([[2, 5, 5, 4, 4, 4, 1], [6, 5, 7, 8, 9, 10, 8]])
    srt = gb.sort_remote_edges_list_based_on_remote_nodes(edges)
    relabelled, remote_nodes, rng, counts = gb.obtain_remote_nodes_list(srt, 2, torch.tensor([0, 3, 6, 9]), 3)
    assert torch.equal(relabelled, torch.tensor([[2, 3, 4, 4, 4, 5, 5], [8, 6, 8, 9, 10, 5, 7]]))
    assert torch.equal(remote_nodes, torch.tensor([1, 2, 4, 5]))
    assert torch.equal(rng, torch.tensor([0, 2, 4, 4]))
    assert torch.equal(counts, torch.tensor([2, 2, 0]))


def test_edge_index_to_sparse_tensors_known_answers():
    local = [torch.tensor([1, 2, 3]), torch.tensor([2, 3, 4])]
    remote = [torch.tensor([7, 7, 7]), torch.tensor([2, 0, 1])]
    la, ra = gb.transform_edge_index_to_sparse_tensor(local, remote, 5, 3)
    want_l = torch.sparse_coo_tensor(torch.tensor([[2, 3, 4], [1, 2, 3]]), torch.ones(3), size=(5, 5)).to_dense()
    want_r = torch.sparse_coo_tensor(torch.tensor([[2, 0, 1], [2, 2, 2]]), torch.ones(3), size=(5, 3)).to_dense()
    assert torch.equal(la.to_dense(), want_l) and torch.equal(ra.to_dense(), want_r)

    local = torch.tensor([[0, 1, 1], [0, 0, 1]])
    remote = torch.tensor([[2, 5, 5, 4, 4, 4, 2], [0, 0, 0, 1, 0, 1, 0]])
    remote = gb.sort_remote_edges_list_based_on_remote_nodes(remote)
    relabelled, remote_nodes, _, _ = gb.obtain_remote_nodes_list(remote, 2, torch.tensor([0, 3, 6, 9]), 3)
    assert torch.equal(relabelled, torch.tensor([[2, 2, 3, 3, 3, 4, 4], [0, 0, 1, 0, 1, 0, 0]]))
    la, ra = gb.transform_edge_index_to_sparse_tensor(local, relabelled, 2, 3)
    want_l = torch.sparse_coo_tensor(torch.tensor([[0, 0, 1], [0, 1, 1]]), torch.ones(3), size=(2, 2)).to_dense()
    want_r = torch.sparse_coo_tensor(torch.tensor([[0, 0, 1, 0], [0, 1, 1, 2]]), torch.ones(4), size=(2, 3)).to_dense()
    assert torch.equal(la.to_dense(), want_l)
    assert torch.equal(ra.to_dense(), want_r)  # repeated edges land on one entry, as in the reference's container


def test_in_degrees_known_answer():
    local = [torch.tensor([1, 2, 3]), torch.tensor([0, 0, 1])]
    remote = [torch.tensor([2, 3, 4]), torch.tensor([2, 3, 3])]
    assert torch.equal(gb.get_in_degrees(local, remote, 5), torch.tensor([[2.], [1.], [1.], [2.], [1.]]))


def test_device_builder_is_the_composition_of_the_steps():
    g = torch.Generator().manual_seed(5)
    n, R0, begins = 40, 100, [0, 40, 100]
    local = torch.randint(0, n, (2, 300), generator=g)
    remote = torch.stack([torch.randint(n, R0, (200,), generator=g), torch.randint(0, n, (200,), generator=g)])
    graph = build_distributed_graph(local, remote, begins, 8, 32, device=torch.device("cpu"), with_values=True)
    srt = gb.sort_remote_edges_list_based_on_remote_nodes(remote)
    relabelled, remote_nodes, rng, counts = gb.obtain_remote_nodes_list(srt, n, begins, 2)
    la, ra = gb.transform_edge_index_to_sparse_tensor(local, relabelled, n, remote_nodes.numel())
    assert torch.equal(graph.in_degrees, gb.get_in_degrees(local, remote, n))
    assert graph.comm_splits.recv_splits == counts.tolist()
    # the builder keeps repeated edges as repeated entries (they add up in the aggregation, as in the reference)
    for mine, theirs in ((graph.local_adj_t, la), (graph.remote_adj_t, ra)):
        assert mine.sparse_sizes() == theirs.sparse_sizes()
        for a, b in zip(mine.csr(), theirs.csr()):
            assert torch.equal(a, b)
