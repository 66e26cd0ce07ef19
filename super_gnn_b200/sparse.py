"""Minimal CSR container with the ``torch_sparse.SparseTensor`` surface the hot
path touches (the reference depends on an un-vendored fork of torch_sparse).

Call sites mirrored: construction from COO (data_manager/DataProcessor.py:109-121),
``csr()`` (ops/spmm_kernel.py:47), ``storage.colptr()/row_T()/value_T()`` — the
cached CSR of the transpose (:77-79), the opaque cached work-range slots
``get/set_work_range[_for_transpose]`` (:49-58, :81-88), ``sparse_size(s)``
(aggregator.py:62,146), ``coo()`` (DistributedGraph.py:37-38), ``to_dense()``.

Differences, on purpose: column indices are kept as int32 (what the kernels
read), ``value`` may be ``None`` for an all-ones matrix, and the transpose is
built on the device by ``sgnn_csr_transpose``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


class _Storage:
    """``SparseTensor.storage``: owns the arrays and the cached transpose."""

    def __init__(self, rowptr, col, value, sparse_sizes):
        self._rowptr = rowptr
        self._col = col
        self._value = value
        self._sparse_sizes = tuple(int(s) for s in sparse_sizes)
        self._colptr = None
        self._row_T = None
        self._value_T = None
        self._row = None

    def rowptr(self):
        return self._rowptr

    def col(self):
        return self._col

    def value(self):
        return self._value

    def sparse_sizes(self):
        return self._sparse_sizes

    def row(self):
        if self._row is None:
            counts = self._rowptr[1:] - self._rowptr[:-1]
            self._row = torch.repeat_interleave(
                torch.arange(self._sparse_sizes[0], device=self._rowptr.device, dtype=torch.int64), counts)
        return self._row

    def _build_transpose(self):
        if self._colptr is not None:
            return
        if self._rowptr.is_cuda:
            from . import supergnn_ops

            self._colptr, self._row_T, self._value_T = supergnn_ops.csr_transpose(
                self._rowptr, self._col, self._value, self._sparse_sizes[1])
        else:  # host containers exist only for set-up code and CPU tests of the host logic
            col = self._col.to(torch.int64)
            order = torch.sort(col, stable=True).indices
            self._row_T = self.row()[order].to(torch.int32)
            self._value_T = None if self._value is None else self._value[order]
            counts = torch.bincount(col, minlength=self._sparse_sizes[1])
            self._colptr = torch.zeros(self._sparse_sizes[1] + 1, dtype=torch.int64)
            torch.cumsum(counts, 0, out=self._colptr[1:])

    def colptr(self):
        self._build_transpose()
        return self._colptr

    def row_T(self):
        self._build_transpose()
        return self._row_T

    def value_T(self):
        self._build_transpose()
        return self._value_T


class SparseTensor:
    def __init__(self, row: Optional[torch.Tensor] = None, rowptr: Optional[torch.Tensor] = None,
                 col: Optional[torch.Tensor] = None, value: Optional[torch.Tensor] = None,
                 sparse_sizes: Optional[Tuple[int, int]] = None, is_sorted: bool = False):
        assert col is not None and sparse_sizes is not None, "col and sparse_sizes are required"
        M, K = int(sparse_sizes[0]), int(sparse_sizes[1])
        dev = col.device
        if rowptr is None:
            assert row is not None, "give row or rowptr"
            row = row.to(torch.int64)
            col64 = col.to(torch.int64)
            if not is_sorted and row.numel() > 0:
                key = row * K + col64  # sort by (row, col) like torch_sparse
                order = torch.sort(key, stable=True).indices
                row, col64 = row[order], col64[order]
                if value is not None:
                    value = value[order]
            counts = torch.bincount(row, minlength=M) if row.numel() > 0 else torch.zeros(M, dtype=torch.int64, device=dev)
            rowptr = torch.zeros(M + 1, dtype=torch.int64, device=dev)
            torch.cumsum(counts, 0, out=rowptr[1:])
            col = col64
        assert rowptr.numel() == M + 1
        assert K <= 2**31 - 1, "column count must fit int32"
        if value is not None:
            value = value.to(torch.float32).contiguous()
        self.storage = _Storage(rowptr.to(torch.int64).contiguous(), col.to(torch.int32).contiguous(), value, (M, K))
        empty = torch.empty(0, dtype=torch.int32)
        self._work_range = (empty, empty)
        self._work_range_T = (empty, empty)

    # --- torch_sparse surface ------------------------------------------------
    def csr(self):
        s = self.storage
        return s.rowptr(), s.col(), s.value()

    def coo(self):
        s = self.storage
        return s.row(), s.col().to(torch.int64), s.value()

    def sparse_sizes(self):
        return self.storage.sparse_sizes()

    def sparse_size(self, dim: int) -> int:
        return self.storage.sparse_sizes()[dim]

    def size(self, dim: int) -> int:
        return self.sparse_size(dim)

    def nnz(self) -> int:
        return self.storage.col().numel()

    @property
    def device(self):
        return self.storage.col().device

    def get_work_range(self):
        return self._work_range

    def set_work_range(self, row_splits, col_splits):
        self._work_range = (row_splits, col_splits)

    def get_work_range_for_transpose(self):
        return self._work_range_T

    def set_work_range_for_transpose(self, row_splits, col_splits):
        self._work_range_T = (row_splits, col_splits)

    def to(self, device):
        s = self.storage
        out = SparseTensor(rowptr=s.rowptr().to(device), col=s.col().to(device),
                           value=None if s.value() is None else s.value().to(device),
                           sparse_sizes=s.sparse_sizes(), is_sorted=True)
        return out

    def cuda(self):
        return self.to(torch.device("cuda", torch.cuda.current_device()))

    def t(self):
        s = self.storage
        return SparseTensor(rowptr=s.colptr(), col=s.row_T(), value=s.value_T(),
                            sparse_sizes=(s.sparse_sizes()[1], s.sparse_sizes()[0]), is_sorted=True)

    def to_dense(self):
        M, K = self.sparse_sizes()
        row, col, val = self.coo()
        out = torch.zeros(M, K, dtype=torch.float32, device=self.device)
        v = val if val is not None else torch.ones(row.numel(), dtype=torch.float32, device=self.device)
        out[row, col] = v  # an entry stored twice shows its value once, as in torch_sparse's to_dense
        return out

    def set_value(self, value):
        s = self.storage
        return SparseTensor(rowptr=s.rowptr(), col=s.col(), value=value, sparse_sizes=s.sparse_sizes(), is_sorted=True)

    def fill_diag(self, fill_value: float = 1.0):
        """Set the main diagonal to ``fill_value`` (used by the GCN driver, train.py:253)."""
        M, K = self.sparse_sizes()
        row, col, val = self.coo()
        v = val if val is not None else torch.ones(row.numel(), dtype=torch.float32, device=self.device)
        keep = row != col
        d = torch.arange(min(M, K), device=self.device, dtype=torch.int64)
        return SparseTensor(row=torch.cat([row[keep], d]), col=torch.cat([col[keep], d]),
                            value=torch.cat([v[keep], torch.full((d.numel(),), float(fill_value), device=self.device)]),
                            sparse_sizes=(M, K))

    def __repr__(self):
        return f"SparseTensor(sparse_sizes={self.sparse_sizes()}, nnz={self.nnz()}, device={self.device})"
