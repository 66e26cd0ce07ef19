"""Partition-parallel generators of the large benchmark graphs and the memory model (CPU).

The generators draw from a stream whose chunks depend only on (seed, chunk id), so the graph must not depend on how
many ranks generate it; every rank keeps the edges whose destination it owns."""
import pytest
import torch

from super_gnn_b200 import workloads


def union(parts, begins):
    """Global (source, destination) keys of the edges the ranks hold."""
    n = begins[-1]
    keys = []
    for r, (le, re) in enumerate(parts):
        lo = begins[r]
        keys.append((le[1] + lo) * n + le[0] + lo)
        keys.append((re[1] + lo) * n + re[0])
    return torch.sort(torch.cat(keys))[0]


def check_simple_symmetric(keys, n):
    assert torch.unique(keys).numel() == keys.numel()  # no duplicates
    dst, src = keys // n, keys % n
    assert bool((dst != src).all())  # no self loops
    assert torch.equal(torch.sort(src * n + dst)[0], keys)  # every edge has its reverse


@pytest.mark.parametrize("worlds", [(1, 3), (1, 4)])
def test_rmat_stream_is_the_same_graph_at_every_rank_count(worlds, monkeypatch):
    monkeypatch.setattr(workloads, "CHUNK", 1 << 12)  # several chunks at this size
    n, pairs = 5000, 30000
    got = []
    for W in worlds:
        parts, begins = [], None
        for r in range(W):
            le, re, begins = workloads.rmat_partition(n, pairs, r, W, seed=11, device="cpu")
            lo, hi = begins[r], begins[r + 1]
            assert le.numel() == 0 or (int(le.min()) >= 0 and int(le.max()) < hi - lo)
            assert re.numel() == 0 or bool(((re[0] < lo) | (re[0] >= hi)).all())  # remote sources are global ids
            parts.append((le, re))
        got.append(union(parts, begins))
    assert torch.equal(got[0], got[1])
    check_simple_symmetric(got[0], n)
    assert got[0].numel() > pairs  # both directions of (most of) the generated pairs


def test_sbm_blocks_are_the_same_graph_at_every_rank_count_and_mostly_internal():
    blocks, size, pairs = 8, 300, 20000
    n = blocks * size
    got = []
    for W in (1, 2, 8):
        parts, begins = [], None
        for r in range(W):
            le, re, begins = workloads.sbm_partition(blocks, size, pairs, 0.9, r, W, seed=5, device="cpu")
            parts.append((le, re))
        assert begins == [r * (blocks // W) * size for r in range(W + 1)]
        got.append(union(parts, begins))
    assert torch.equal(got[0], got[1]) and torch.equal(got[0], got[2])
    check_simple_symmetric(got[0], n)
    dst, src = got[0] // n, got[0] % n
    inside = float(((dst // size) == (src // size)).float().mean())
    assert 0.85 < inside < 0.95
    with pytest.raises(AssertionError):
        workloads.sbm_partition(blocks, size, pairs, 0.9, 0, 3, seed=5, device="cpu")  # 8 blocks over 3 ranks


def test_memory_model_against_the_measured_points():
    # 12 M nodes / 169.4 M directed edges on one GPU: 115.7 GB allocated at the peak of a measured run
    one = workloads.step_memory_bytes(12_000_000, 169_438_684, 0, 0, 0, 128, 256, 172, 2, 1)
    assert one["boundary"] == 0 and 0.95 * 115.7e9 < one["total"] < 1.12 * 115.7e9
    # 80 M nodes on 8 ranks, 12.56 M boundary rows each way: measured 123.2 GB with one more input-width buffer
    # alive at the peak than the code has now (1 KB per node)
    rank = workloads.step_memory_bytes(10_000_000, 1_139_832_562 // 64, 1_139_832_562 // 8 * 7 // 8, 12_555_531,
                                       12_496_409, 128, 256, 172, 2, 8, chunks=7)
    assert 0.93 * (123.2e9 - 10.24e9) < rank["total"] < 1.1 * (123.2e9 - 10.24e9)
    # fewer bits, less boundary memory; the rest does not move
    wide = workloads.step_memory_bytes(10_000_000, 10 ** 8, 10 ** 8, 12_000_000, 12_000_000, 128, 256, 172, 32, 8)
    mid = workloads.step_memory_bytes(10_000_000, 10 ** 8, 10 ** 8, 12_000_000, 12_000_000, 128, 256, 172, 8, 8)
    low = workloads.step_memory_bytes(10_000_000, 10 ** 8, 10 ** 8, 12_000_000, 12_000_000, 128, 256, 172, 2, 8)
    assert wide["boundary"] > mid["boundary"] > low["boundary"] > 0
    assert wide["activations"] == mid["activations"] == low["activations"]
    # the bound used before a graph exists is never below what a run showed
    remote, rows, _ = workloads.rmat_boundary_estimate(111_000_000, 1_582_153_606, 8)
    assert rows >= 16_838_162 and remote <= 1_582_153_606 // 8
