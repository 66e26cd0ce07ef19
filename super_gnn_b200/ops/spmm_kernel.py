"""``SPMM_forward`` / ``SPMM_backward`` with the reference's names and signatures
(super_gnn/ops/spmm_kernel.py:46-68, 72-91): ``out += A @ other`` and
``out += A^T @ other`` in place, return value unused.

The reference caches a per-thread row split on the SparseTensor
(``get/set_work_range``); on the GPU the same slots cache the degree statistics
that choose the kernel: near-uniform degrees take the deterministic row-split
kernel (a warp or sub-warp per row), skewed ones the nnz-split (merge-path)
kernel.
"""
from __future__ import annotations

import torch

from .. import supergnn_ops
from ..supergnn_ops import spmm  # noqa: F401  (same import the reference makes)

# a row this many times longer than the mean makes a straggler worth avoiding
_SKEW_RATIO = 8.0
_SKEW_MIN_LEN = 512


def choose_algo(rowptr: torch.Tensor, nnz: int) -> int:
    """Pick the SpMM work split from the row-length statistics (one device sync)."""
    M = rowptr.numel() - 1
    if M <= 0 or nnz == 0:
        return supergnn_ops.SPMM_ROW_SPLIT
    max_len, _ = supergnn_ops.csr_row_stats(rowptr)
    mean = nnz / M
    if max_len >= _SKEW_MIN_LEN and max_len > _SKEW_RATIO * max(mean, 1.0):
        return supergnn_ops.SPMM_NNZ_SPLIT
    return supergnn_ops.SPMM_ROW_SPLIT


def distribute_work_for_row(rowptr: torch.Tensor, value: torch.Tensor, num_threads_on_row: int) -> torch.Tensor:
    """Greedy nnz-balanced row split (spmm_kernel.py:8-29), vectorised.  Only the
    CPU ops consume it; the GPU kernels ignore it."""
    if value is None:
        csum = rowptr.to(torch.float64)
    else:
        ex = torch.cat([torch.zeros(1, dtype=torch.float64, device=value.device), torch.cumsum(value.to(torch.float64), 0)])
        csum = ex[rowptr]  # csum[i] = sum of the values of rows < i
    M = rowptr.numel() - 1
    target = float(torch.floor(csum[-1] / num_threads_on_row))
    splits = [0]
    base = 0.0
    for _ in range(num_threads_on_row):
        # first row whose inclusive prefix exceeds base + target
        i = int(torch.searchsorted(csum[1:], torch.tensor(base + target, dtype=torch.float64, device=csum.device),
                                   right=True))
        if i >= M:
            break
        splits.append(i)
        base = float(csum[i])
    out = torch.full((num_threads_on_row + 1,), M, dtype=torch.int32)
    out[: len(splits)] = torch.tensor(splits, dtype=torch.int32)
    out[-1] = M
    return out


def disribute_work_for_col(other: torch.Tensor, num_threads_on_col: int) -> torch.Tensor:
    """Even column split (spmm_kernel.py:31-44); kept for interface parity."""
    num_cols = other.shape[-1]
    step = num_cols // num_threads_on_col
    col_splits = torch.full((num_threads_on_col + 1,), num_cols, dtype=torch.int32)
    for i in range(num_threads_on_col):
        col_splits[i] = i * step
    return col_splits


def _algo_from_slot(slot) -> int:
    row_splits, _ = slot
    if isinstance(row_splits, torch.Tensor) and row_splits.numel() == 1:
        return int(row_splits.item())
    return -1


def SPMM_forward(src, other: torch.Tensor, out: torch.Tensor, row_scale=None, col_scale=None):
    rowptr, col, value = src.csr()
    algo = _algo_from_slot(src.get_work_range())
    if algo < 0:
        algo = choose_algo(rowptr, col.numel())
        src.set_work_range(torch.tensor([algo], dtype=torch.int32), torch.empty(0, dtype=torch.int32))
    if value is not None:
        value = value.to(other.dtype)
    sparse_row = rowptr.shape[0] - 1
    spmm(rowptr, col, value, other, out, sparse_row, None, None, algo=algo, row_scale=row_scale, col_scale=col_scale)
    return None


def SPMM_backward(src, other: torch.Tensor, out: torch.Tensor, row_scale=None, col_scale=None):
    colptr = src.storage.colptr()
    row_T = src.storage.row_T()
    value_T = src.storage.value_T()
    algo = _algo_from_slot(src.get_work_range_for_transpose())
    if algo < 0:
        algo = choose_algo(colptr, row_T.numel())
        src.set_work_range_for_transpose(torch.tensor([algo], dtype=torch.int32), torch.empty(0, dtype=torch.int32))
    sparse_row = colptr.shape[0] - 1
    spmm(colptr, row_T, value_T, other, out, sparse_row, None, None, algo=algo, row_scale=row_scale, col_scale=col_scale)
    return None
