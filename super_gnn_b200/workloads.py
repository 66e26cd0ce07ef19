"""Partition-parallel generators of the multi-GPU benchmark graphs, and the memory model that says which
(GPU count, bit width) cells of a scaling sweep fit.

The reference loads graphs that ParMETIS partitioned offline, one set of ``.npy`` files per rank
(super_gnn/data_manager/DataLoader.py:215-278; node ranges from ``begin_node_on_each_partition.txt``).  The
synthetic stand-ins here produce the same per-rank inputs — ``local_edges`` / ``remote_edges`` as ``[2, E]``
int64 tensors (row 0 = source, row 1 = destination; local ids except for remote sources) and the range
begins — WITHOUT any rank ever holding the global edge list: the edge stream is cut into chunks whose random
draws depend only on (seed, chunk id), every rank walks the stream on its own GPU and keeps the edges whose
destination it owns.  The same seed therefore gives the same graph at every rank count.

* ``sbm``: stochastic block model with equal blocks (the 8-GPU pre/post-aggregation configuration: 8 blocks,
  10 M nodes, 200 M directed edges, 90 % of them inside a block; block b belongs to rank b * ranks / blocks).
* ``rmat``: R-MAT (a, b, c, d) = (0.57, 0.19, 0.19, 0.05), node ids randomly relabelled, contiguous ranges (the
  large scaling-sweep configuration: 111 M nodes, 1.6 B directed edges).

Both are symmetrised (each generated pair yields both directions), self loops are dropped and duplicate
edges removed, as the reference's preprocessing does (graph_partition/preprocess_graph.py:96-127).
"""
from __future__ import annotations

import math
from typing import List, Sequence, Tuple

import torch

CHUNK = 1 << 24  # generated pairs per chunk of the R-MAT stream


def _gen(device, *key) -> torch.Generator:
    """Generator seeded by a tuple of small integers (a counter-based stream: same key, same draws)."""
    seed = 0x9E3779B97F4A7C15
    for k in key:
        seed = (seed ^ (int(k) + 0x632BE59BD9B4E019)) * 0xBF58476D1CE4E5B9 % (1 << 63)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def even_ranges(num_nodes: int, parts: int) -> List[int]:
    base, rem = divmod(num_nodes, parts)
    out = [0]
    for p in range(parts):
        out.append(out[-1] + base + (1 if p < rem else 0))
    return out


def _keep_mine(s: torch.Tensor, t: torch.Tensor, lo: int, hi: int, n: int) -> torch.Tensor:
    """Both directions of the pairs (s, t), reduced to the edges whose destination lies in [lo, hi) and packed
    as one int64 key per edge: (destination - lo) * n + source.  Self loops are dropped."""
    keys = []
    for src, dst in ((s, t), (t, s)):
        m = (dst >= lo) & (dst < hi) & (src != dst)
        keys.append((dst[m] - lo) * n + src[m])
    return torch.cat(keys)


def _finish(keys: List[torch.Tensor], lo: int, hi: int, n: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Unique edge keys -> (local_edges, remote_edges) of the rank that owns [lo, hi)."""
    key = torch.unique(torch.cat(keys)) if keys else torch.empty(0, dtype=torch.int64)
    dst, src = key // n, key % n
    is_local = (src >= lo) & (src < hi)
    local_edges = torch.stack([src[is_local] - lo, dst[is_local]])
    remote_edges = torch.stack([src[~is_local], dst[~is_local]])
    return local_edges, remote_edges


def rmat_partition(num_nodes: int, num_pairs: int, rank: int, world: int, seed: int, device,
                   abcd: Sequence[float] = (0.57, 0.19, 0.19, 0.05), relabel: bool = True):
    """This rank's edges of the symmetrised R-MAT graph with ``num_pairs`` generated pairs.
    Returns ``(local_edges, remote_edges, begins)``."""
    a, b, c, _ = abcd
    begins = even_ranges(num_nodes, world)
    lo, hi = begins[rank], begins[rank + 1]
    scale = max(1, math.ceil(math.log2(max(2, num_nodes))))
    full = 1 << scale
    perm = None
    if relabel:  # the same permutation on every rank (same seed, same device type)
        perm = torch.randperm(num_nodes, generator=_gen(device, seed, 1), device=device)
    keys = []
    for chunk_id, start in enumerate(range(0, num_pairs, CHUNK)):
        m = min(CHUNK, num_pairs - start)
        g = _gen(device, seed, 2, chunk_id)
        s = torch.zeros(m, dtype=torch.int64, device=device)
        t = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):  # one quadrant draw per bit level
            r = torch.rand(m, generator=g, device=device)
            s = (s << 1) | (r >= (a + b)).to(torch.int64)
            t = (t << 1) | (((r >= a) & (r < a + b)) | (r >= (a + b + c))).to(torch.int64)
        if full != num_nodes:
            s = (s * num_nodes) // full
            t = (t * num_nodes) // full
        if perm is not None:
            s, t = perm[s], perm[t]
        keys.append(_keep_mine(s, t, lo, hi, num_nodes))
        del s, t, r
    del perm
    local_edges, remote_edges = _finish(keys, lo, hi, num_nodes)
    return local_edges, remote_edges, begins


def sbm_partition(num_blocks: int, block_size: int, num_pairs: int, intra_fraction: float, rank: int, world: int,
                  seed: int, device):
    """This rank's edges of the symmetrised stochastic block model: ``intra_fraction`` of the generated pairs
    have both endpoints uniform inside one block (the same number in every block), the rest have their
    endpoints uniform in two different blocks (the same number for every unordered pair of blocks).  Ranks own
    ``num_blocks / world`` consecutive blocks.  Returns ``(local_edges, remote_edges, begins)``."""
    assert num_blocks % world == 0, "the blocks must divide evenly over the ranks"
    n = num_blocks * block_size
    per_rank = num_blocks // world
    begins = [r * per_rank * block_size for r in range(world + 1)]
    lo, hi = begins[rank], begins[rank + 1]
    mine = range(rank * per_rank, (rank + 1) * per_rank)
    n_intra = int(round(num_pairs * intra_fraction)) // num_blocks
    pairs = num_blocks * (num_blocks - 1) // 2
    n_inter = (num_pairs - n_intra * num_blocks) // max(pairs, 1)
    keys = []

    def draw(g, count, block):
        return block * block_size + torch.randint(0, block_size, (count,), generator=g, device=device)

    for b in mine:  # pairs inside my blocks
        for start in range(0, n_intra, CHUNK):
            m = min(CHUNK, n_intra - start)
            g = _gen(device, seed, 3, b, start // CHUNK)
            keys.append(_keep_mine(draw(g, m, b), draw(g, m, b), lo, hi, n))
    for b1 in range(num_blocks):  # pairs between two blocks, at least one of them mine
        for b2 in range(b1 + 1, num_blocks):
            if b1 not in mine and b2 not in mine:
                continue
            g = _gen(device, seed, 4, b1, b2)
            keys.append(_keep_mine(draw(g, n_inter, b1), draw(g, n_inter, b2), lo, hi, n))
    local_edges, remote_edges = _finish(keys, lo, hi, n)
    return local_edges, remote_edges, begins


# ---------------------------------------------------------------------------
# memory model
# ---------------------------------------------------------------------------
def step_memory_bytes(n_local: int, nnz_local: int, nnz_remote: int, rows_recv: int, rows_send: int, in_channels: int,
                      hidden: int, classes: int, bits: int, world: int, chunks: int = 1) -> dict:
    """Device bytes one rank needs for a training step of the 3-layer model as the fused path runs it (fp32).

    Activations kept for the backward pass, per node: the input x, and per hidden layer the aggregated input,
    the pre-normalisation output h and the layer output (two statistics per row are negligible); for the last
    layer the aggregated remote share (input width) and the [A^T g | g] buffer (2 x classes rounded up to 4).
    Transients: the widest forward scratch (the last layer's [x W_n^T | x W_s^T]) and, in the backward pass of
    the second hidden layer, four hidden-width buffers (the incoming gradient's buffer, overwritten by the
    gradient of h, and the [g W_n | g W_s] buffer) less what the last layer kept and has released by then; with
    several ranks the last layer's backward instead: the logits, their gradient and the gradient of the layer's
    input (the gradient of the remote share is overwritten by it).
    Checked against a measured run: 12 M nodes on one GPU peaked at 119.6 GB allocated, the model says 121.
    Graph: int32 column + int64 row pointers for the matrices and their transposes, plus 1/in_degree edge
    values of the transposed matrices.  Boundary: with 2/4/8 bits the codes and bf16 parameters of the rows
    received (forward) and sent (backward direction) plus one fp32 chunk of the largest per-peer share of the
    remote gradient rows (``chunks`` = peers the backward pass walks one at a time); with 32 bits the fp32
    send and receive buffers at the hidden width."""
    cp = (classes + 3) // 4 * 4
    F = 4
    act = n_local * F * (in_channels + (in_channels + 2 * hidden) + 3 * hidden + (hidden + 2 * cp))
    fwd_peak = n_local * F * (2 * cp)
    bwd_peak = max(0, n_local * F * (4 * hidden - (hidden + 2 * cp)))
    if world > 1:  # last layer's backward: logits, their gradient and the gradient of the layer's input
        bwd_peak = max(bwd_peak, n_local * F * (2 * classes + hidden))
    nnz = nnz_local + nnz_remote
    graph = nnz * (4 + 4 + 4) + (4 * n_local + 2 * rows_recv) * 8
    if world == 1:
        boundary = 0
    elif bits in (2, 4, 8):
        per_row = hidden * bits // 8 + 4
        boundary = (rows_recv + rows_send) * per_row + (rows_recv // max(chunks, 1) + 1) * hidden * F
        boundary += rows_send * 8  # send index
    else:
        boundary = (rows_recv + rows_send) * hidden * F * (2 if bits == 16 else 1) + rows_send * 8
    total = act + max(fwd_peak, bwd_peak) + graph + boundary
    return dict(activations=act, transient=max(fwd_peak, bwd_peak), graph=graph, boundary=boundary, total=total)


def rmat_boundary_estimate(num_nodes: int, directed_edges: int, world: int) -> Tuple[int, int, int]:
    """(remote nonzeros, rows received, rows sent) per rank for a randomly relabelled graph cut into ``world``
    contiguous ranges, before it is built: (world-1)/world of a rank's in-edges have a remote source, and the
    rows received are bounded by both that count and the nodes other ranks own.  R-MAT's skew (many edges
    share a few hub sources) makes the true figure smaller; the bound is what a fits / does-not-fit decision
    may rely on."""
    if world == 1:
        return 0, 0, 0
    nnz_rank = directed_edges // world
    remote = nnz_rank * (world - 1) // world
    rows = min(remote, num_nodes - num_nodes // world)
    return remote, rows, rows
