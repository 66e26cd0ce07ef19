"""Pre/post-aggregation planner (CPU): the native minimum vertex cover and the row
bookkeeping, pinned to the known answers of the reference's
tests/test_data_preprocessor_pre_aggr.py."""
import numpy as np
import pytest
import torch

from super_gnn_b200.data_manager.pre_post import (decide_pre_or_post_aggr, min_vertex_cover, rows_to_aggregate,
                                                  rows_to_request)

T = lambda *a: torch.tensor(a, dtype=torch.int64)  # noqa: E731


@pytest.mark.parametrize("src,dst,expected_is_pre", [
    # tests/test_data_preprocessor_pre_aggr.py:60-92 (1 = pre, 0 = post)
    ([1, 3, 1, 1], [12, 11, 12, 13], [0, 0, 0, 0]),
    ([2, 1, 2, 1, 0], [11, 14, 11, 11, 11], [1, 0, 1, 0, 1]),
    ([0, 2, 2, 2, 4, 4, 5, 5], [11, 11, 12, 14, 14, 13, 16, 13], [0] * 8),
    ([], [], []),
])
def test_vertex_cover_reference_known_answers(src, dst, expected_is_pre):
    post, size = min_vertex_cover(T(*src), T(*dst))
    assert (~post).int().tolist() == expected_is_pre
    pre_idx, post_idx = decide_pre_or_post_aggr(T(*src), T(*dst))
    assert pre_idx.tolist() == [i for i, p in enumerate(expected_is_pre) if p == 1]
    assert post_idx.tolist() == [i for i, p in enumerate(expected_is_pre) if p == 0]


def test_vertex_cover_is_minimum_and_valid_on_random_graphs():
    sp = pytest.importorskip("scipy.sparse")
    from scipy.sparse.csgraph import maximum_bipartite_matching

    rng = np.random.default_rng(0)
    for _ in range(40):
        nl, nr, E = int(rng.integers(1, 80)), int(rng.integers(1, 80)), int(rng.integers(1, 400))
        s = rng.integers(0, nl, E)
        d = rng.integers(0, nr, E)
        post, size = min_vertex_cover(torch.from_numpy(s), torch.from_numpy(d) + 10_000)
        m = maximum_bipartite_matching(sp.csr_matrix((np.ones(E), (s, d)), shape=(nl, nr)), perm_type="column")
        post = post.numpy()
        cover_src = set(s[post].tolist())
        cover_dst = set(d[~post].tolist())     # a pre edge must be covered by its destination
        assert size == int((m >= 0).sum())     # Koenig: |minimum cover| = |maximum matching|
        assert len(cover_src) + len(cover_dst) == size
        assert not (set(s[~post].tolist()) & cover_src)  # the flag is a property of the source vertex


def test_rows_to_request_reference_known_answers():
    """tests/test_data_preprocessor_pre_aggr.py:94-139."""
    src, dst = T(0, 2, 2, 2, 4, 4, 5, 5), T(1, 1, 2, 4, 4, 3, 6, 3)
    post = torch.zeros(8, dtype=torch.bool)
    post[[1, 2, 3, 6]] = True
    _, s, k = rows_to_request(src, dst, post)
    assert s.tolist() == [0, 2, 4, 5, 4, 5] and k.tolist() == [1, 2, 3, 3, 4, 5]
    _, s, k = rows_to_request(src, dst, torch.zeros(8, dtype=torch.bool))            # pre only
    assert s.tolist() == [0, 2, 2, 4, 5, 2, 4, 5] and k.tolist() == [1, 1, 2, 3, 3, 4, 4, 6]
    _, s, k = rows_to_request(T(0, 2, 9, 3, 4, 1, 5, 3), dst, torch.ones(8, dtype=torch.bool))  # post only
    assert s.tolist() == [0, 1, 2, 3, 4, 5, 9] and k.tolist() == [0, 1, 2, 3, 4, 5, 9]


def test_rows_to_aggregate_matches_the_reference_rule():
    """DataProcessor.collect_edges_for_aggregation: post edges keep (src -> dst); every pre-summed
    destination appears once as (dst -> dst); sorted by key; #distinct keys = rows received."""
    src, dst = T(0, 2, 2, 2, 4, 4, 5, 5), T(11, 11, 12, 14, 14, 13, 16, 13)
    post = torch.zeros(8, dtype=torch.bool)
    post[[1, 2, 3, 6]] = True
    _, key, d = rows_to_aggregate(src, dst, post)
    assert key.tolist() == [2, 2, 2, 5, 11, 13, 14] and d.tolist() == [11, 12, 14, 16, 11, 13, 14]
    assert torch.unique(key).numel() == 5
