"""Seeded synthetic inputs with the shapes and distributions of the benchmark
configurations (the public datasets the reference trains on are not available
offline): Poisson-degree CSR, R-MAT and stochastic-block-model edge lists,
symmetrisation / de-duplication / random relabelling, row-scaled feature blocks.

Every generator draws from one ``torch.Generator`` on the requested device, so a
(seed, device) pair reproduces its input exactly; checks against the CPU oracle
copy the generated tensors instead of regenerating them.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def poisson_csr(num_rows: int, num_cols: int, mean_degree: float, seed: int, device="cpu", mean_values: bool = True):
    """Square-ish CSR with Poisson row lengths and uniform random columns (duplicates
    allowed).  Values are 1/deg(row) (mean aggregation) or None.
    Returns (rowptr int64, col int32, value fp32 | None)."""
    g = _gen(seed, device)
    deg = torch.poisson(torch.full((num_rows,), float(mean_degree), device=device), generator=g).to(torch.int64)
    rowptr = torch.zeros(num_rows + 1, dtype=torch.int64, device=device)
    torch.cumsum(deg, 0, out=rowptr[1:])
    nnz = int(rowptr[-1])
    col = torch.randint(0, num_cols, (nnz,), generator=g, device=device, dtype=torch.int64).to(torch.int32)
    value = None
    if mean_values:
        value = torch.repeat_interleave(1.0 / deg.clamp(min=1).to(torch.float32), deg)
    return rowptr, col, value


def rmat_edges(num_nodes: int, num_edges: int, a: float, b: float, c: float, d: float, seed: int, device="cpu",
               chunk: int = 1 << 24) -> Tuple[torch.Tensor, torch.Tensor]:
    """R-MAT edge list (src, dst): one quadrant draw per bit level on a 2^scale grid,
    ids scaled down to ``num_nodes``.  Duplicates and self loops are left in."""
    g = _gen(seed, device)
    scale = max(1, math.ceil(math.log2(max(2, num_nodes))))
    srcs, dsts = [], []
    for start in range(0, num_edges, chunk):
        m = min(chunk, num_edges - start)
        s = torch.zeros(m, dtype=torch.int64, device=device)
        t = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(m, generator=g, device=device)
            sbit = r >= (a + b)
            tbit = ((r >= a) & (r < a + b)) | (r >= (a + b + c))
            s = (s << 1) | sbit.to(torch.int64)
            t = (t << 1) | tbit.to(torch.int64)
        srcs.append(s)
        dsts.append(t)
    s = torch.cat(srcs)
    t = torch.cat(dsts)
    full = 1 << scale
    if full != num_nodes:
        s = (s * num_nodes) // full
        t = (t * num_nodes) // full
    return s, t


def sbm_edges(num_blocks: int, block_size: int, num_edges: int, intra_fraction: float, seed: int, device="cpu"):
    """Stochastic block model with equal blocks: ``intra_fraction`` of the edges have
    both endpoints uniform inside one (uniformly chosen) block, the rest have
    endpoints uniform in two different blocks."""
    g = _gen(seed, device)
    n_intra = int(round(num_edges * intra_fraction))
    n_inter = num_edges - n_intra
    blk = torch.randint(0, num_blocks, (n_intra,), generator=g, device=device)
    s1 = blk * block_size + torch.randint(0, block_size, (n_intra,), generator=g, device=device)
    t1 = blk * block_size + torch.randint(0, block_size, (n_intra,), generator=g, device=device)
    b1 = torch.randint(0, num_blocks, (n_inter,), generator=g, device=device)
    off = torch.randint(1, max(2, num_blocks), (n_inter,), generator=g, device=device)
    b2 = (b1 + off) % num_blocks
    s2 = b1 * block_size + torch.randint(0, block_size, (n_inter,), generator=g, device=device)
    t2 = b2 * block_size + torch.randint(0, block_size, (n_inter,), generator=g, device=device)
    return torch.cat([s1, s2]), torch.cat([t1, t2])


def symmetrize_dedup(src: torch.Tensor, dst: torch.Tensor, num_nodes: int, drop_self_loops: bool = True):
    """Both directions of every edge, duplicates (and self loops) removed; sorted by (dst, src)."""
    s = torch.cat([src, dst])
    t = torch.cat([dst, src])
    if drop_self_loops:
        keep = s != t
        s, t = s[keep], t[keep]
    key = torch.unique(t * num_nodes + s)
    return key % num_nodes, key // num_nodes


def random_relabel(src: torch.Tensor, dst: torch.Tensor, num_nodes: int, seed: int):
    g = _gen(seed, src.device)
    perm = torch.randperm(num_nodes, generator=g, device=src.device)
    return perm[src], perm[dst]


def even_ranges(num_nodes: int, parts: int):
    """Contiguous node ranges of (almost) equal size: begin of every partition, plus the end."""
    base, rem = divmod(num_nodes, parts)
    out = [0]
    for p in range(parts):
        out.append(out[-1] + base + (1 if p < rem else 0))
    return out


def scaled_features(rows: int, cols: int, seed: int, device="cpu", lognormal_scale: bool = True):
    """N(0,1) rows times a per-row LogNormal(0,1) scale (the quantiser's test input)."""
    g = _gen(seed, device)
    x = torch.randn(rows, cols, generator=g, device=device)
    if lognormal_scale:
        x = x * torch.exp(torch.randn(rows, 1, generator=g, device=device))
    return x
