"""GPU drop-in for the reference's ``supergnn_ops`` extension module.

Same function names and argument orders as the pybind11 module of
super_gnn/ops/csrc/ops.cpp:12-27 (both the x86 export list and the SVE one):
outputs are caller-allocated and written in place, every function returns
``None``, bad arguments raise ``RuntimeError``.  All tensors must live on a CUDA
device; the work is enqueued on the current stream of that device through the
C ABI (``include/supergnn_b200.h``) and the call returns without synchronising.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _cabi

SPMM_AUTO, SPMM_ROW_SPLIT, SPMM_NNZ_SPLIT, SPMM_NNZ_SPLIT_STAGED = 0, 1, 2, 3

# Optional launch log for benchmarks: when set to a list, every op appends
# (kind, info, start_event, end_event) with CUDA events recorded on the launching stream.
LAUNCH_LOG = None
# Number of C-ABI calls that enqueued kernels since import (each call launches our kernels only).
LAUNCH_COUNT = 0


class _Logged:
    """Context manager that counts a launch and, if enabled, brackets it with CUDA events."""

    __slots__ = ("kind", "info", "dev", "start")

    def __init__(self, kind, dev, **info):
        self.kind, self.info, self.dev = kind, info, dev

    def __enter__(self):
        global LAUNCH_COUNT
        LAUNCH_COUNT += 1
        self.start = None
        if LAUNCH_LOG is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.dev))
        return self

    def __exit__(self, *exc):
        if self.start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.dev))
            LAUNCH_LOG.append((self.kind, self.info, self.start, end))
        return False


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _cuda(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    _need(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _need(t.is_cuda, f"{name} must be a CUDA tensor (supergnn_b200 has no CPU path)")
    if dtype is not None:
        _need(t.dtype == dtype, f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None:
        _need(t.dim() == dim, f"{name} must have {dim} dimensions, got {t.dim()}")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _same_device(*ts) -> None:
    dev = None
    for t in ts:
        if t is None:
            continue
        if dev is None:
            dev = t.device
        _need(t.device == dev, "all tensors must be on the same CUDA device")


def _i32_col(col: torch.Tensor) -> torch.Tensor:
    """The kernels take int32 column indices; an int64 tensor (the reference's
    layout) is narrowed here — keep int32 in the container to avoid the copy."""
    if col.dtype == torch.int32:
        return col.contiguous()
    _need(col.dtype == torch.int64, "col must be int32 or int64")
    return col.to(torch.int32)


# ---------------------------------------------------------------------------
# SpMM
# ---------------------------------------------------------------------------
def _scale(t, n, name, device):
    if t is None:
        return None
    _cuda(t, name, torch.float32, None)
    _need(t.numel() == n and t.is_contiguous() and t.device == device, f"{name} must be a contiguous fp32 tensor of {n} entries")
    return t


def spmm(rowptr, col, value, mat, out, sparse_rows, row_split=None, col_split=None, algo: int = SPMM_AUTO,
         accumulate: bool = True, row_scale=None, col_scale=None, nnz_range=None):
    """``out += A @ mat`` — supergnn_ops.spmm (super_gnn/ops/csrc/spmm.h:3-6).

    ``row_split`` / ``col_split`` (the reference's per-thread work ranges) are
    accepted and ignored; ``algo`` chooses the GPU work split instead.  The op
    always accumulates unless ``accumulate=False`` is passed explicitly.
    ``row_scale`` ([M]) / ``col_scale`` ([K]) turn the product into
    ``diag(row_scale) A diag(col_scale) mat`` (mean normalisation folded in).
    ``nnz_range = (begin, count)``: ``rowptr`` is a slice of a larger matrix's row pointers (``sparse_rows + 1``
    entries that still hold positions in the whole ``col`` / ``value`` arrays), ``begin`` the value of its first
    entry and ``count`` the nonzeros of those rows; the product then covers that range of rows only.
    """
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", None, 1)
    _cuda(mat, "mat", torch.float32, 2)
    _cuda(out, "out", torch.float32, 2)
    if value is not None:
        _cuda(value, "value", torch.float32, 1)
        _need(value.numel() == col.numel(), "value and col must have the same length")
        value = value.contiguous()
    _same_device(rowptr, col, value, mat, out)
    M = int(sparse_rows)
    _need(rowptr.numel() == M + 1, f"rowptr must have sparse_rows + 1 = {M + 1} entries")
    _need(out.size(0) == M and out.size(1) == mat.size(1), "out must be [sparse_rows, mat.size(1)]")
    _need(out.stride(1) == 1 or out.size(1) <= 1, "out must have contiguous rows (it is written in place)")
    if mat.stride(1) != 1 and mat.size(1) > 1:
        mat = mat.contiguous()  # column slices of a wider row-major buffer pass through with their row stride
    rowptr = rowptr.contiguous()
    col = _i32_col(col)
    K, N = mat.shape
    if _DEBUG and nnz_range is None:  # debugging aid: the kernels themselves trust the indices
        rep = check_csr(rowptr, col, K)
        _need(rep["rows_ending_before_start"] == 0 and rep["columns_out_of_range"] == 0 and rep["rowptr_starts_at_zero"]
              and rep["rowptr_ends_at_nnz"], f"spmm: malformed CSR matrix: {rep}")
    row_scale = _scale(row_scale, M, "row_scale", out.device)
    col_scale = _scale(col_scale, K, "col_scale", out.device)
    if nnz_range is not None:
        begin, count = int(nnz_range[0]), int(nnz_range[1])
        _need(0 <= begin and 0 <= count and begin + count <= col.numel(), "nnz_range outside the col array")
        with torch.cuda.device(out.device), _Logged("spmm", out.device, M=M, K=K, N=N, nnz=count,
                                                    has_val=value is not None, acc=bool(accumulate), algo=int(algo)):
            rc = _cabi.lib().sgnn_spmm_csr_rows_f32(_ptr(rowptr), _ptr(col), _ptr(value), begin, count, _ptr(mat),
                                                    max(mat.stride(0), N), _ptr(out), max(out.stride(0), N), M, K, N,
                                                    1 if accumulate else 0, int(algo), _ptr(row_scale),
                                                    _ptr(col_scale), _stream(out))
        _cabi.check(rc, "spmm")
        return None
    with torch.cuda.device(out.device), _Logged("spmm", out.device, M=M, K=K, N=N, nnz=col.numel(),
                                                has_val=value is not None, acc=bool(accumulate), algo=int(algo)):
        rc = _cabi.lib().sgnn_spmm_csr_f32(_ptr(rowptr), _ptr(col), _ptr(value), col.numel(), _ptr(mat),
                                           max(mat.stride(0), N), _ptr(out), max(out.stride(0), N), M, K, N,
                                           1 if accumulate else 0, int(algo),
                                           _ptr(row_scale), _ptr(col_scale), _stream(out))
    _cabi.check(rc, "spmm")
    return None


def spmm_dequant(rowptr, col, value, packed, params, work_range, num_procs, bits, out, sparse_rows,
                 algo: int = SPMM_AUTO, row_scale=None):
    """``out += A @ dequantize(packed)`` without materialising the fp32 rows.

    ``params`` is fp32 ``[R,2]`` or bf16 ``[R,2]`` (zero_point, scale) as received.
    Fuses dequantize_tensor_for_all_procs with the spmm that follows it
    (super_gnn/aggregator.py:74-79, 88-92)."""
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", None, 1)
    _cuda(packed, "packed", torch.uint8, 2)
    _cuda(params, "params", None, 2)
    _cuda(out, "out", torch.float32, 2)
    _need(params.dtype in (torch.float32, torch.bfloat16), "params must be float32 or bfloat16")
    _need(params.size(1) == 2 and params.is_contiguous(), "params must be a contiguous [R,2] tensor")
    if value is not None:
        _cuda(value, "value", torch.float32, 1)
        value = value.contiguous()
    M = int(sparse_rows)
    F = packed.size(1)
    R = params.size(0)
    bits = _check_bits(bits)
    host_range = _work_range_host(work_range) if isinstance(work_range, torch.Tensor) else ()
    work_range = _work_range(work_range, num_procs, out.device)
    _need(host_range[-1] <= R, "params has fewer rows than the work range covers")
    _need(packed.size(0) >= _packed_rows(host_range, bits), "packed has fewer rows than the work range needs")
    _same_device(rowptr, col, value, packed, params, out)
    _need(rowptr.numel() == M + 1, "rowptr must have sparse_rows + 1 entries")
    _need(out.size(0) == M and out.size(1) == F and (out.stride(1) == 1 or F <= 1),
          "out must be [sparse_rows, F] with contiguous rows")
    _need(packed.is_contiguous(), "packed must be contiguous")
    col = _i32_col(col)
    p32 = params if params.dtype == torch.float32 else None
    p16 = params if params.dtype == torch.bfloat16 else None
    with torch.cuda.device(out.device), _Logged("spmm_dequant", out.device, M=M, R=R, N=F, nnz=col.numel(),
                                                has_val=value is not None, bits=int(bits), algo=int(algo)):
        rc = _cabi.lib().sgnn_spmm_csr_dequant_f32(_ptr(rowptr.contiguous()), _ptr(col), _ptr(value), col.numel(),
                                                   _ptr(packed), _ptr(p32), _ptr(p16), R, F, _ptr(work_range),
                                                   int(num_procs), int(bits), _ptr(out), max(out.stride(0), F), M,
                                                   int(algo),
                                                   _ptr(_scale(row_scale, M, "row_scale", out.device)), _stream(out))
    _cabi.check(rc, "spmm_dequant")
    return None


def check_csr(rowptr, col, num_cols: int) -> dict:
    """Structural check of a CSR matrix on the device (synchronises): counts of rows that end before they start,
    of column indices outside ``[0, num_cols)``, and whether ``rowptr[0] == 0`` and ``rowptr[-1] == len(col)``.
    The kernels trust these; with ``SGNN_DEBUG=1`` in the environment ``spmm`` runs this check first and raises."""
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", None, 1)
    col = _i32_col(col)
    flags = torch.zeros(4, dtype=torch.int64, device=rowptr.device)
    with torch.cuda.device(rowptr.device):
        rc = _cabi.lib().sgnn_csr_check(_ptr(rowptr.contiguous()), _ptr(col), rowptr.numel() - 1, int(num_cols),
                                        col.numel(), _ptr(flags), _stream(rowptr))
    _cabi.check(rc, "csr_check")
    bad_rows, bad_cols, bad_first, bad_last = flags.tolist()
    return dict(rows_ending_before_start=int(bad_rows), columns_out_of_range=int(bad_cols),
                rowptr_starts_at_zero=not bad_first, rowptr_ends_at_nnz=not bad_last)


_DEBUG = bool(int(__import__("os").environ.get("SGNN_DEBUG", "0") or 0))


def csr_row_stats(rowptr):
    """(max row length, number of empty rows) of a CSR matrix; synchronises once."""
    _cuda(rowptr, "rowptr", torch.int64, 1)
    stats = torch.zeros(2, dtype=torch.int64, device=rowptr.device)
    with torch.cuda.device(rowptr.device):
        rc = _cabi.lib().sgnn_csr_row_stats(_ptr(rowptr.contiguous()), rowptr.numel() - 1, _ptr(stats), _stream(rowptr))
    _cabi.check(rc, "csr_row_stats")
    mx, empty = stats.tolist()
    return int(mx), int(empty)


def csr_transpose(rowptr, col, value, num_cols: int):
    """CSR of the transpose (rows ascending inside each column): returns
    ``(colptr int64[K+1], row_T int32[nnz], value_T fp32[nnz] | None)``."""
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", None, 1)
    col = _i32_col(col)
    if value is not None:
        _cuda(value, "value", torch.float32, 1)
        value = value.contiguous()
    _same_device(rowptr, col, value)
    dev = rowptr.device
    M, K, nnz = rowptr.numel() - 1, int(num_cols), col.numel()
    colptr = torch.empty(K + 1, dtype=torch.int64, device=dev)
    row_T = torch.empty(nnz, dtype=torch.int32, device=dev)
    value_T = torch.empty(nnz, dtype=torch.float32, device=dev) if value is not None else None
    l = _cabi.lib()
    nbytes = int(l.sgnn_csr_transpose_workspace_bytes(M, K, nnz))
    _need(nbytes > 0, "csr_transpose: sizes out of range (M, K, nnz must fit int32)")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = l.sgnn_csr_transpose(_ptr(rowptr.contiguous()), _ptr(col), _ptr(value), M, K, nnz, _ptr(colptr),
                                  _ptr(row_T), _ptr(value_T), _ptr(ws), nbytes, _stream(rowptr))
    _cabi.check(rc, "csr_transpose")
    # the workspace must outlive the enqueued work on this stream
    ws.record_stream(torch.cuda.current_stream(dev))
    return colptr, row_T, value_T


def csr_transpose_noalloc(rowptr, col, value, num_cols: int, colptr, row_T, value_T=None):
    """``csr_transpose`` into caller-provided outputs with the library's static
    scratch: no device allocation happens in the call (see the limits in the
    header; sizes beyond them raise ``RuntimeError``)."""
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", torch.int32, 1)
    _cuda(colptr, "colptr", torch.int64, 1)
    _cuda(row_T, "row_T", torch.int32, 1)
    M, K, nnz = rowptr.numel() - 1, int(num_cols), col.numel()
    _need(colptr.numel() == K + 1 and row_T.numel() == nnz, "colptr must be [K+1] and row_T [nnz]")
    _need(rowptr.is_contiguous() and col.is_contiguous() and colptr.is_contiguous() and row_T.is_contiguous(),
          "all arrays must be contiguous")
    if value is not None:
        _cuda(value, "value", torch.float32, 1)
        _need(value_T is not None and value_T.numel() == nnz and value.is_contiguous() and value_T.is_contiguous(),
              "value_T must be a contiguous fp32 [nnz] tensor when value is given")
    _same_device(rowptr, col, value, colptr, row_T, value_T)
    with torch.cuda.device(rowptr.device):
        rc = _cabi.lib().sgnn_csr_transpose_noalloc(_ptr(rowptr), _ptr(col), _ptr(value), M, K, nnz, _ptr(colptr),
                                                    _ptr(row_T), _ptr(value_T), _stream(rowptr))
    _cabi.check(rc, "csr_transpose_noalloc")
    return None


# ---------------------------------------------------------------------------
# quantisation
# ---------------------------------------------------------------------------
def _work_range_host(work_range: torch.Tensor) -> tuple:
    """Host copy of a work range, read back once per tensor (and again after an in-place change): the kernels
    trust these numbers for their row counts and buffer offsets, so the sizes are checked against them on the
    host before anything is launched.  The copy is kept on the tensor object itself, so it cannot outlive it."""
    if not work_range.is_cuda:
        return tuple(int(v) for v in work_range.tolist())
    hit = getattr(work_range, "_sgnn_host_copy", None)
    if hit is not None and hit[0] == work_range._version:
        return hit[1]
    host = tuple(int(v) for v in work_range.tolist())
    work_range._sgnn_host_copy = (work_range._version, host)
    return host


def _packed_rows(host_range, bits: int) -> int:
    epb = 8 // bits
    return sum(-(-(b - a) // epb) for a, b in zip(host_range[:-1], host_range[1:]))


def _work_range(work_range, num_procs, device, rows=None) -> torch.Tensor:
    """Validated device copy of ``work_range_per_proc``; ``rows`` (if given) must equal its last entry."""
    _need(isinstance(work_range, torch.Tensor) and work_range.dtype == torch.int32,
          "work_range_per_proc must be an int32 tensor")
    _need(work_range.numel() == int(num_procs) + 1, "work_range_per_proc must have num_procs + 1 entries")
    host = _work_range_host(work_range)
    _need(host[0] == 0 and all(a <= b for a, b in zip(host[:-1], host[1:])),
          "work_range_per_proc must start at 0 and be non-decreasing")
    if rows is not None:
        _need(host[-1] == int(rows), f"work_range_per_proc ends at {host[-1]} but there are {int(rows)} rows")
    if not work_range.is_cuda:
        work_range = work_range.to(device)
    return work_range.contiguous()


def _single_range(S: int, device) -> torch.Tensor:
    return torch.tensor([0, S], dtype=torch.int32, device=device)


def _check_bits(bits) -> int:
    bits = int(bits)
    _need(bits in (2, 4, 8), f"bits must be 2, 4 or 8 (8 % bits == 0), got {bits}")
    return bits


def quant_pack_rows(src, row_index, work_range, num_procs, bits, packed, params=None, params_bf16=None):
    """Fused (optional row gather) + per-row min-max quantise + per-peer pack.

    ``row_index`` (int64 ``[S]`` or None) selects the rows of ``src``; None means
    rows ``0..S-1``.  Writes ``packed`` and whichever of ``params`` (fp32 ``[S,2]``)
    and ``params_bf16`` (``[S,2]``) is given."""
    bits = _check_bits(bits)
    _cuda(src, "input", torch.float32, 2)
    _cuda(packed, "output", torch.uint8, None)
    _need(src.stride(1) == 1, "input rows must be contiguous")
    _need(packed.is_contiguous(), "output must be contiguous")
    F = src.size(1)
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = src.size(0)
    host_range = _work_range_host(work_range) if isinstance(work_range, torch.Tensor) else ()
    work_range = _work_range(work_range, num_procs, src.device, rows=S)
    if params is not None:
        _cuda(params, "params", torch.float32, 2)
        _need(params.is_contiguous() and params.size(0) >= S and params.size(1) == 2, "params must be contiguous [S,2]")
    if params_bf16 is not None:
        _cuda(params_bf16, "params_bf16", torch.bfloat16, 2)
        _need(params_bf16.is_contiguous() and params_bf16.size(0) >= S and params_bf16.size(1) == 2,
              "params_bf16 must be contiguous [S,2]")
    # every peer's segment is rounded up to whole packed rows: sum_p ceil(n_p / EPB) rows of F bytes are written
    _need(packed.numel() >= _packed_rows(host_range, bits) * F, "output buffer too small for the packed rows")
    _same_device(src, row_index, packed, params, params_bf16)
    with torch.cuda.device(src.device), _Logged("quant_pack", src.device, S=S, F=F, bits=bits,
                                                gather=row_index is not None):
        rc = _cabi.lib().sgnn_quant_pack_rows(_ptr(src), src.stride(0), _ptr(row_index), S, F, _ptr(work_range),
                                              int(num_procs), bits, _ptr(packed), _ptr(params), _ptr(params_bf16),
                                              _stream(src))
    _cabi.check(rc, "quant_pack_rows")
    return None


def quant_pack_rows_p2p(src, row_index, work_range, num_procs, bits, peer_tables, params=None):
    """Quantise + pack + store into the peers' receive buffers (one-sided exchange).
    ``peer_tables`` = (packed_ptrs, packed_row0, params_ptrs, params_row0): int64 device
    tensors of length ``num_procs`` (see ``sgnn_quant_pack_rows_p2p``)."""
    bits = _check_bits(bits)
    _cuda(src, "input", torch.float32, 2)
    _need(src.stride(1) == 1, "input rows must be contiguous")
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = src.size(0)
    work_range = _work_range(work_range, num_procs, src.device, rows=S)
    for t in peer_tables:
        _cuda(t, "peer table", torch.int64, 1)
        _need(t.numel() == int(num_procs) and t.is_contiguous(), "peer tables must be contiguous [num_procs] int64")
    if params is not None:
        _cuda(params, "params", torch.float32, 2)
        _need(params.is_contiguous() and params.size(0) >= S and params.size(1) == 2, "params must be contiguous [S,2]")
    pk, pk0, pp, pp0 = peer_tables
    with torch.cuda.device(src.device), _Logged("quant_pack_p2p", src.device, S=S, F=src.size(1), bits=bits,
                                                gather=row_index is not None):
        rc = _cabi.lib().sgnn_quant_pack_rows_p2p(_ptr(src), src.stride(0), _ptr(row_index), S, src.size(1),
                                                  _ptr(work_range), int(num_procs), bits, _ptr(pk), _ptr(pk0),
                                                  _ptr(pp), _ptr(pp0), _ptr(params), _stream(src))
    _cabi.check(rc, "quant_pack_rows_p2p")
    return None


# ---------------------------------------------------------------------------
# the same quantised rows in the row-codes layout (every row owns F*bits/8 contiguous bytes)
# ---------------------------------------------------------------------------
def rowcodes_supported(feat_len: int) -> bool:
    """Row widths the row-codes layout covers: a multiple of 4 up to 128, or 256, or 512."""
    F = int(feat_len)
    return F > 0 and F % 4 == 0 and (F <= 128 or F in (256, 512))


def rowcodes_view(buf: torch.Tensor, rows: int, feat_len: int, bits: int) -> torch.Tensor:
    """``[rows, F*bits/8]`` uint8 view of the start of a (contiguous) packed buffer.  The row-codes form of
    ``rows`` rows never needs more bytes than their row-group form, so the reference's buffers can hold it."""
    pitch = int(feat_len) * int(bits) // 8
    flat = buf.view(-1) if buf.is_contiguous() else buf.reshape(-1)
    _need(flat.numel() >= rows * pitch, "packed buffer too small for the row codes")
    return flat[: rows * pitch].view(rows, pitch)


def _codes_arg(codes, rows, F, bits, name="codes"):
    _cuda(codes, name, torch.uint8, 2)
    _need(codes.is_contiguous() and codes.size(0) >= rows and codes.size(1) == F * bits // 8,
          f"{name} must be a contiguous uint8 [rows, F*bits/8] tensor")


def quant_pack_rowcodes(src, row_index, bits, codes, params=None, params_bf16=None):
    """Per-row min-max quantise of ``src[row_index]`` (or ``src``) into row codes: same codes and parameters as
    ``quant_pack_rows``, every row in its own ``F*bits/8`` bytes of ``codes``."""
    bits = _check_bits(bits)
    _cuda(src, "input", torch.float32, 2)
    _need(src.stride(1) == 1, "input rows must be contiguous")
    F = src.size(1)
    _need(rowcodes_supported(F), f"the row-codes layout does not cover rows of {F} values")
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = src.size(0)
    _codes_arg(codes, S, F, bits)
    if params is not None:
        _cuda(params, "params", torch.float32, 2)
        _need(params.is_contiguous() and params.size(0) >= S and params.size(1) == 2, "params must be contiguous [S,2]")
    if params_bf16 is not None:
        _cuda(params_bf16, "params_bf16", torch.bfloat16, 2)
        _need(params_bf16.is_contiguous() and params_bf16.size(0) >= S and params_bf16.size(1) == 2,
              "params_bf16 must be contiguous [S,2]")
    _same_device(src, row_index, codes, params, params_bf16)
    with torch.cuda.device(src.device), _Logged("quant_pack_rowcodes", src.device, S=S, F=F, bits=bits,
                                                gather=row_index is not None):
        rc = _cabi.lib().sgnn_quant_pack_rowcodes(_ptr(src), src.stride(0), _ptr(row_index), S, F, bits, _ptr(codes),
                                                  _ptr(params), _ptr(params_bf16), _stream(src))
    _cabi.check(rc, "quant_pack_rowcodes")
    return None


def peer_barrier(flag_ptrs, rank: int, world: int, epoch: int, timeout_us: int, status, device=None):
    """Barrier number ``epoch`` (1, 2, ...) among the ``world`` ranks of a one-sided exchange, on the current
    stream of ``flag_ptrs``' device.  ``flag_ptrs``: int64 device tensor with the address of every rank's flag array
    (uint32 [world], zeroed once, mapped by all ranks).  ``status``: int32 [world] tensor, zeroed once, in pinned
    host memory or on the device; a wait that exceeds ``timeout_us`` writes ``epoch`` into ``status[p]`` for the
    missing peer ``p`` and the kernel returns (no trap; the caller reads ``status``)."""
    _cuda(flag_ptrs, "flag_ptrs", torch.int64, 1)
    _need(flag_ptrs.numel() == int(world) and flag_ptrs.is_contiguous(), "flag_ptrs must be a contiguous [world] int64")
    _need(status.dtype == torch.int32 and status.numel() >= int(world) and status.is_contiguous(),
          "status must be a contiguous int32 [world]")
    _need(status.is_cuda or status.is_pinned(), "status must live in pinned host memory or on the device")
    dev = flag_ptrs.device
    with torch.cuda.device(dev), _Logged("peer_barrier", dev, world=int(world)):
        rc = _cabi.lib().sgnn_peer_barrier(_ptr(flag_ptrs), int(rank), int(world), int(epoch) & 0xFFFFFFFF,
                                           int(timeout_us), status.data_ptr(), _stream(flag_ptrs))
    _cabi.check(rc, "peer_barrier")


def quant_pack_rowcodes_p2p(src, row_index, work_range, num_procs, bits, peer_tables, params=None):
    """``quant_pack_rowcodes`` that stores every row into the receive buffers of the peer that owns its segment.
    ``peer_tables`` = (code buffer addresses, bf16 parameter buffer addresses, first row of this rank's segment
    there): int64 device tensors of length ``num_procs``."""
    bits = _check_bits(bits)
    _cuda(src, "input", torch.float32, 2)
    _need(src.stride(1) == 1, "input rows must be contiguous")
    F = src.size(1)
    _need(rowcodes_supported(F), f"the row-codes layout does not cover rows of {F} values")
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = src.size(0)
    work_range = _work_range(work_range, num_procs, src.device, rows=S)
    for t in peer_tables:
        _cuda(t, "peer table", torch.int64, 1)
        _need(t.numel() == int(num_procs) and t.is_contiguous(), "peer tables must be contiguous [num_procs] int64")
    if params is not None:
        _cuda(params, "params", torch.float32, 2)
        _need(params.is_contiguous() and params.size(0) >= S and params.size(1) == 2, "params must be contiguous [S,2]")
    pc, pp, row0 = peer_tables
    with torch.cuda.device(src.device), _Logged("quant_pack_rowcodes_p2p", src.device, S=S, F=F, bits=bits,
                                                gather=row_index is not None):
        rc = _cabi.lib().sgnn_quant_pack_rowcodes_p2p(_ptr(src), src.stride(0), _ptr(row_index), S, F, _ptr(work_range),
                                                      int(num_procs), bits, _ptr(pc), _ptr(pp), _ptr(row0),
                                                      _ptr(params), _stream(src))
    _cabi.check(rc, "quant_pack_rowcodes_p2p")
    return None


def unpack_dequant_rowcodes(codes, output, params, bits, row_index=None):
    """``output[r] = zero_point + code * scale`` from row codes; with ``row_index`` the rows are added into
    ``output[row_index[r]]`` instead.  ``params``: fp32 or bf16 ``[S,2]``."""
    bits = _check_bits(bits)
    _cuda(output, "output", torch.float32, 2)
    _cuda(params, "params", None, 2)
    _need(params.dtype in (torch.float32, torch.bfloat16), "params must be float32 or bfloat16")
    _need(params.is_contiguous() and params.size(1) == 2, "params must be contiguous [S,2]")
    _need(output.stride(1) == 1, "output rows must be contiguous")
    F = output.size(1)
    _need(rowcodes_supported(F), f"the row-codes layout does not cover rows of {F} values")
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = output.size(0)
    _codes_arg(codes, S, F, bits)
    _need(params.size(0) >= S, "params has fewer rows than the data")
    _same_device(codes, output, params, row_index)
    p32 = params if params.dtype == torch.float32 else None
    p16 = params if params.dtype == torch.bfloat16 else None
    with torch.cuda.device(output.device), _Logged("unpack_dequant_rowcodes", output.device, S=S, F=F, bits=bits,
                                                   scatter=row_index is not None):
        rc = _cabi.lib().sgnn_unpack_dequant_rowcodes(_ptr(codes), _ptr(p32), _ptr(p16), S, F, bits, _ptr(output),
                                                      output.stride(0), _ptr(row_index), _stream(output))
    _cabi.check(rc, "unpack_dequant_rowcodes")
    return None


def spmm_dequant_rowcodes(rowptr, col, value, codes, params, bits, out, sparse_rows, algo: int = SPMM_AUTO,
                          row_scale=None):
    """``out += A @ dequantize(codes)`` with the operand rows in the row-codes layout: a gathered row costs
    ``F*bits/8`` bytes (the row-group form costs ``F`` at every bit width)."""
    bits = _check_bits(bits)
    _cuda(rowptr, "rowptr", torch.int64, 1)
    _cuda(col, "col", None, 1)
    _cuda(params, "params", None, 2)
    _cuda(out, "out", torch.float32, 2)
    _need(params.dtype in (torch.float32, torch.bfloat16), "params must be float32 or bfloat16")
    _need(params.size(1) == 2 and params.is_contiguous(), "params must be a contiguous [R,2] tensor")
    if value is not None:
        _cuda(value, "value", torch.float32, 1)
        value = value.contiguous()
    M = int(sparse_rows)
    F = out.size(1)
    R = params.size(0)
    _need(rowcodes_supported(F), f"the row-codes layout does not cover rows of {F} values")
    _codes_arg(codes, R, F, bits)
    _need(rowptr.numel() == M + 1, "rowptr must have sparse_rows + 1 entries")
    _need(out.size(0) == M and (out.stride(1) == 1 or F <= 1), "out must be [sparse_rows, F] with contiguous rows")
    _same_device(rowptr, col, value, codes, params, out)
    col = _i32_col(col)
    p32 = params if params.dtype == torch.float32 else None
    p16 = params if params.dtype == torch.bfloat16 else None
    with torch.cuda.device(out.device), _Logged("spmm_dequant_rowcodes", out.device, M=M, R=R, N=F, nnz=col.numel(),
                                                has_val=value is not None, bits=bits, algo=int(algo)):
        rc = _cabi.lib().sgnn_spmm_csr_dequant_rowcodes_f32(
            _ptr(rowptr.contiguous()), _ptr(col), _ptr(value), col.numel(), _ptr(codes), _ptr(p32), _ptr(p16), R, F,
            bits, _ptr(out), max(out.stride(0), F), M, int(algo), _ptr(_scale(row_scale, M, "row_scale", out.device)),
            _stream(out))
    _cabi.check(rc, "spmm_dequant_rowcodes")
    return None


def quantize_tensor_for_all_procs(input, output, params, work_range_per_proc, num_procs, bits):
    """supergnn_ops.quantize_tensor_for_all_procs (quantization_arm.cpp:496-578)."""
    _need(input.dim() == 2 and input.is_contiguous(), "input must be a contiguous 2-D tensor")
    quant_pack_rows(input, None, work_range_per_proc, num_procs, bits, output, params=params)
    return None


def dequantize_tensor_for_all_procs(input, output, params, work_range_per_proc, num_procs, bits,
                                    row_index=None):
    """supergnn_ops.dequantize_tensor_for_all_procs (quantization_arm.cpp:580-633).

    ``params`` may be fp32 or bf16 ``[S,2]``.  With ``row_index`` the rows are
    added into ``output[row_index[r]]`` instead of stored to ``output[r]``."""
    bits = _check_bits(bits)
    _cuda(input, "input", torch.uint8, 2)
    _cuda(output, "output", torch.float32, 2)
    _cuda(params, "params", None, 2)
    _need(params.dtype in (torch.float32, torch.bfloat16), "params must be float32 or bfloat16")
    _need(params.is_contiguous() and params.size(1) == 2, "params must be contiguous [S,2]")
    _need(input.is_contiguous() and output.stride(1) == 1, "input must be contiguous and output rows contiguous")
    F = output.size(1)
    _need(input.size(1) == F, "input and output feature lengths differ")
    if row_index is not None:
        _cuda(row_index, "row_index", torch.int64, 1)
        S = row_index.numel()
        row_index = row_index.contiguous()
    else:
        S = output.size(0)
    host_range = _work_range_host(work_range_per_proc) if isinstance(work_range_per_proc, torch.Tensor) else ()
    work_range = _work_range(work_range_per_proc, num_procs, output.device, rows=S)
    _need(params.size(0) >= S, "params has fewer rows than the data")
    _need(input.size(0) >= _packed_rows(host_range, bits), "input has fewer packed rows than the work range needs")
    _same_device(input, output, params, row_index)
    p32 = params if params.dtype == torch.float32 else None
    p16 = params if params.dtype == torch.bfloat16 else None
    with torch.cuda.device(output.device), _Logged("unpack_dequant", output.device, S=S, F=F, bits=bits,
                                                   scatter=row_index is not None):
        rc = _cabi.lib().sgnn_unpack_dequant_rows(_ptr(input), _ptr(p32), _ptr(p16), S, F, _ptr(work_range),
                                                  int(num_procs), bits, _ptr(output), output.stride(0),
                                                  _ptr(row_index), _stream(output))
    _cabi.check(rc, "dequantize_tensor_for_all_procs")
    return None


def quantize_tensor(input, output, *args):
    """Both reference forms: x86 ``(input, output, min, scale, bits)``
    (quantization_x86.cpp:17-102) and SVE ``(input, output, params, bits)``
    (quantization_arm.cpp:433-494, single segment, params computed)."""
    _cuda(input, "input", torch.float32, 2)
    _cuda(output, "output", torch.uint8, None)
    _need(input.is_contiguous() and output.is_contiguous(), "input and output must be contiguous")
    S, F = input.shape
    if len(args) == 3:
        mn, scale, bits = args
        bits = _check_bits(bits)
        _cuda(mn, "min", torch.float32, None)
        _cuda(scale, "scale", torch.float32, None)
        mn, scale = mn.contiguous(), scale.contiguous()
        _need(mn.numel() >= S and scale.numel() >= S, "min and scale need one entry per row")
        _need(output.numel() >= -(-S // (8 // bits)) * F, "output buffer too small")
        _same_device(input, output, mn, scale)
        with torch.cuda.device(input.device):
            rc = _cabi.lib().sgnn_quantize_tensor(_ptr(input), S, F, _ptr(mn), _ptr(scale), bits, _ptr(output),
                                                  _stream(input))
        _cabi.check(rc, "quantize_tensor")
    elif len(args) == 2:
        params, bits = args
        quant_pack_rows(input, None, _single_range(S, input.device), 1, bits, output, params=params)
    else:
        raise RuntimeError("quantize_tensor takes (input, output, min, scale, bits) or (input, output, params, bits)")
    return None


def dequantize_tensor(input, output, *args):
    """x86 ``(input, output, min, scale, bits)`` (quantization_x86.cpp:104-168) or
    SVE ``(input, output, params, bits)``."""
    _cuda(input, "input", torch.uint8, None)
    _cuda(output, "output", torch.float32, 2)
    _need(input.is_contiguous() and output.is_contiguous(), "input and output must be contiguous")
    S, F = output.shape
    if len(args) == 3:
        mn, scale, bits = args
        bits = _check_bits(bits)
        _cuda(mn, "min", torch.float32, None)
        _cuda(scale, "scale", torch.float32, None)
        mn, scale = mn.contiguous(), scale.contiguous()
        _need(mn.numel() >= S and scale.numel() >= S, "min and scale need one entry per row")
        _need(input.numel() >= -(-S // (8 // bits)) * F, "input buffer too small")
        _same_device(input, output, mn, scale)
        with torch.cuda.device(output.device):
            rc = _cabi.lib().sgnn_dequantize_tensor(_ptr(input), S, F, _ptr(mn), _ptr(scale), bits, _ptr(output),
                                                    _stream(output))
        _cabi.check(rc, "dequantize_tensor")
    elif len(args) == 2:
        params, bits = args
        dequantize_tensor_for_all_procs(input.view(-1, F), output, params, _single_range(S, output.device), 1, bits)
    else:
        raise RuntimeError("dequantize_tensor takes (input, output, min, scale, bits) or (input, output, params, bits)")
    return None


def quantize_tensor_v1(input, output, quantized_nodes_feat_range, quantized_params):
    """supergnn_ops.quantize_tensor_v1 (quantization_x86.cpp:170-253)."""
    _cuda(input, "input", torch.float32, 2)
    _cuda(output, "output", torch.uint8, None)
    _cuda(quantized_nodes_feat_range, "quantized_nodes_feat_range", torch.int64, 1)
    _cuda(quantized_params, "quantized_params", torch.float32, 2)
    S, F = input.shape
    _need(input.is_contiguous() and output.is_contiguous() and quantized_params.is_contiguous(),
          "input, output and quantized_params must be contiguous")
    _need(quantized_params.size(0) == S and quantized_params.size(1) == 3, "quantized_params must be [rows,3]")
    _need(quantized_nodes_feat_range.numel() == S + 1, "quantized_nodes_feat_range must have rows + 1 entries")
    _same_device(input, output, quantized_nodes_feat_range, quantized_params)
    with torch.cuda.device(input.device):
        rc = _cabi.lib().sgnn_quantize_rows_v1(_ptr(input), S, F, _ptr(quantized_nodes_feat_range.contiguous()),
                                               _ptr(quantized_params), _ptr(output), _stream(input))
    _cabi.check(rc, "quantize_tensor_v1")
    return None


def dequantize_tensor_v1(input, output, quantized_nodes_feat_range, quantized_params):
    """supergnn_ops.dequantize_tensor_v1 (quantization_x86.cpp:255-312)."""
    _cuda(input, "input", torch.uint8, None)
    _cuda(output, "output", torch.float32, 2)
    _cuda(quantized_nodes_feat_range, "quantized_nodes_feat_range", torch.int64, 1)
    _cuda(quantized_params, "quantized_params", torch.float32, 2)
    S, F = output.shape
    _need(input.is_contiguous() and output.is_contiguous() and quantized_params.is_contiguous(),
          "input, output and quantized_params must be contiguous")
    _need(quantized_params.size(0) == S and quantized_params.size(1) == 3, "quantized_params must be [rows,3]")
    _need(quantized_nodes_feat_range.numel() == S + 1, "quantized_nodes_feat_range must have rows + 1 entries")
    _same_device(input, output, quantized_nodes_feat_range, quantized_params)
    with torch.cuda.device(output.device):
        rc = _cabi.lib().sgnn_dequantize_rows_v1(_ptr(input), S, F, _ptr(quantized_nodes_feat_range.contiguous()),
                                                 _ptr(quantized_params), _ptr(output), _stream(output))
    _cabi.check(rc, "dequantize_tensor_v1")
    return None


def _v2_args(data, packed, quantized_nodes_feat_range, zero_points, scales, num_bits, S):
    bits = _check_bits(num_bits)
    _cuda(quantized_nodes_feat_range, "quantized_nodes_feat_range", torch.int64, 1)
    _need(quantized_nodes_feat_range.numel() == S + 1, "quantized_nodes_feat_range must have rows + 1 entries")
    for t, name in ((zero_points, "zero_points"), (scales, "scales")):
        _cuda(t, name, torch.float32, None)
        _need(t.numel() >= S, f"{name} needs one entry per row")
    _need(data.is_contiguous() and packed.is_contiguous(), "input and output must be contiguous")
    _same_device(data, packed, quantized_nodes_feat_range, zero_points, scales)
    return bits, quantized_nodes_feat_range.contiguous(), zero_points.contiguous(), scales.contiguous()


def quantize_tensor_v2_torch(input, output, quantized_nodes_feat_range, zero_points, scales, num_bits):
    """supergnn_ops.quantize_tensor_v2_torch (quantization_x86.cpp:314-388): ``rne(x / scale + zero_point)`` in
    torch.quantize_per_channel's convention, first element of a byte in the low bits."""
    _cuda(input, "input", torch.float32, 2)
    _cuda(output, "output", torch.uint8, None)
    S, F = input.shape
    bits, rng, zp, sc = _v2_args(input, output, quantized_nodes_feat_range, zero_points, scales, num_bits, S)
    _need(output.numel() >= S * -(-F // (8 // bits)), "output buffer too small")
    with torch.cuda.device(input.device):
        rc = _cabi.lib().sgnn_quantize_rows_v2(_ptr(input), S, F, _ptr(rng), _ptr(zp), _ptr(sc), bits, _ptr(output),
                                               _stream(input))
    _cabi.check(rc, "quantize_tensor_v2_torch")
    return None


def dequantize_tensor_v2_torch(input, output, quantized_nodes_feat_range, zero_points, scales, num_bits):
    """supergnn_ops.dequantize_tensor_v2_torch (quantization_x86.cpp:390-459): ``(code - zero_point) * scale``."""
    _cuda(input, "input", torch.uint8, None)
    _cuda(output, "output", torch.float32, 2)
    S, F = output.shape
    bits, rng, zp, sc = _v2_args(output, input, quantized_nodes_feat_range, zero_points, scales, num_bits, S)
    _need(input.numel() >= S * -(-F // (8 // bits)), "input buffer too small")
    with torch.cuda.device(output.device):
        rc = _cabi.lib().sgnn_dequantize_rows_v2(_ptr(input), S, F, _ptr(rng), _ptr(zp), _ptr(sc), bits, _ptr(output),
                                                 _stream(output))
    _cabi.check(rc, "dequantize_tensor_v2_torch")
    return None


# ---------------------------------------------------------------------------
# boundary-row gather / scatter-add
# ---------------------------------------------------------------------------
def gather_rows(src, index, out):
    """``out[r] = src[index[r]]`` — torch.index_select(src, 0, index, out=out)
    as used at super_gnn/aggregator.py:48."""
    _cuda(src, "src", torch.float32, 2)
    _cuda(index, "index", torch.int64, 1)
    _cuda(out, "out", torch.float32, 2)
    _need(src.stride(1) == 1 and out.stride(1) == 1, "rows must be contiguous")
    _need(out.size(0) == index.numel() and out.size(1) == src.size(1), "out must be [len(index), F]")
    _same_device(src, index, out)
    with torch.cuda.device(out.device), _Logged("gather_rows", out.device, S=index.numel(), F=src.size(1)):
        rc = _cabi.lib().sgnn_gather_rows(_ptr(src), src.stride(0), _ptr(index.contiguous()), index.numel(),
                                          src.size(1), _ptr(out), out.stride(0), _stream(out))
    _cabi.check(rc, "gather_rows")
    return None


def scatter_add_rows(src, index, out):
    """``out[index[r]] += src[r]`` — out.index_add_(0, index, src) as used at
    super_gnn/aggregator.py:173-175."""
    _cuda(src, "src", torch.float32, 2)
    _cuda(index, "index", torch.int64, 1)
    _cuda(out, "out", torch.float32, 2)
    _need(src.stride(1) == 1 and out.stride(1) == 1, "rows must be contiguous")
    _need(src.size(0) == index.numel() and out.size(1) == src.size(1), "src must be [len(index), F]")
    _same_device(src, index, out)
    with torch.cuda.device(out.device), _Logged("scatter_add_rows", out.device, S=index.numel(), F=src.size(1)):
        rc = _cabi.lib().sgnn_scatter_add_rows(_ptr(src), src.stride(0), _ptr(index.contiguous()), index.numel(),
                                               src.size(1), _ptr(out), out.stride(0), _stream(out))
    _cabi.check(rc, "scatter_add_rows")
    return None


# ---------------------------------------------------------------------------
# fused layer epilogue
# ---------------------------------------------------------------------------
def _mode_of(training: bool, p: float, mask) -> int:
    if not training:
        return 0
    if mask is not None:
        return 2
    return 1 if p > 0.0 else 0


_GEMM_WORKSPACE = {}
GEMM_SIX_PRODUCTS = 16  # or-ed into the op code: leave out the three smallest of the nine bf16 cross products
# Cross products the fp32 GEMM computes when a call does not say: 9 (every one) or 6.  SGNN_GEMM_PRODUCTS sets it.
GEMM_PRODUCTS = int(os.environ.get("SGNN_GEMM_PRODUCTS", "9"))


def _gemm_op(base: int, products) -> int:
    products = GEMM_PRODUCTS if products is None else int(products)
    _need(products in (6, 9), "gemm: products must be 6 or 9")
    return base | (GEMM_SIX_PRODUCTS if products == 6 else 0)


def _gemm_workspace(dev, nbytes: int):
    """One scratch buffer per (device, stream), grown on demand: calls on one stream are ordered, calls on
    different streams may overlap and must not share it."""
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    ws = _GEMM_WORKSPACE.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _GEMM_WORKSPACE[key] = ws
    return ws


def _gemm(op: int, a, b, out, beta: float, M: int, N: int, K: int, kind: str):
    lib = _cabi.lib()
    dev = a.device
    need = ctypes.c_size_t(0)
    _cabi.check(lib.sgnn_gemm_f32_workspace_bytes(op, M, N, K, ctypes.byref(need)), kind)
    ws = _gemm_workspace(dev, need.value) if need.value else None
    with torch.cuda.device(dev), _Logged(kind, dev, M=M, N=N, K=K):
        rc = lib.sgnn_gemm_f32(op, _ptr(a), a.stride(0), _ptr(b), b.stride(0), _ptr(out), out.stride(0), M, N, K,
                               float(beta), _ptr(ws), ws.numel() if ws is not None else 0, _stream(a))
    _cabi.check(rc, kind)
    return out


def _gemm_operands(a, b, out, names):
    for t, name in zip((a, b), names):
        _cuda(t, name, torch.float32, 2)
        _need(t.stride(1) == 1, f"{name} must have contiguous rows")
    if out is not None:
        _cuda(out, "out", torch.float32, 2)
        _need(out.stride(1) == 1, "out must have contiguous rows")
    _same_device(a, b, out)


def gemm_nt(a, b, out=None, beta: float = 0.0, products=None):
    """``out = a @ b.T (+ beta * out)`` for ``a`` [M, K] and ``b`` [N, K] (a linear map ``x W^T``; with
    ``b = W^T`` the input gradient ``g W``).  fp32 in, fp32 out, fp32 accuracy on the tensor cores.
    ``products``: 9 or 6 bf16 cross products per element pair (default: ``GEMM_PRODUCTS``)."""
    _gemm_operands(a, b, out, ("a", "b"))
    M, K = a.shape
    N = b.size(0)
    _need(b.size(1) == K, "gemm_nt: a is [M, K] and b must be [N, K]")
    if out is None:
        _need(beta == 0.0, "gemm_nt: beta needs an existing out")
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(tuple(out.shape) == (M, N), "gemm_nt: out must be [M, N]")
    if M == 0 or N == 0:
        return out
    return _gemm(_gemm_op(0, products), a, b, out, beta, M, N, K, "gemm_nt")


def gemm_tn(a, b, out=None, beta: float = 0.0, products=None):
    """``out = a.T @ b (+ beta * out)`` for ``a`` [K, M] and ``b`` [K, N]: the weight gradient ``g^T x`` of a
    linear map, reduced over the K rows (nodes) with the K range split over the SMs."""
    _gemm_operands(a, b, out, ("a", "b"))
    K, M = a.shape
    N = b.size(1)
    _need(b.size(0) == K, "gemm_tn: a is [K, M] and b must be [K, N]")
    if out is None:
        _need(beta == 0.0, "gemm_tn: beta needs an existing out")
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(tuple(out.shape) == (M, N), "gemm_tn: out must be [M, N]")
    if M == 0 or N == 0:
        return out
    if K == 0:
        return out.zero_() if beta == 0.0 else out.mul_(beta)
    return _gemm(_gemm_op(1, products), a, b, out, beta, M, N, K, "gemm_tn")


def sage_epilogue_forward(h, bias, gamma, beta, p: float, training: bool, seed: int, eps: float = 1e-5, mask=None,
                          out=None):
    """``y = relu(LayerNorm(dropout(h + bias)))``.  Returns ``(y, stats)`` with ``stats`` [n, 2] = (mean, reciprocal
    standard deviation) per row; ``h`` is left as it is (the backward recomputes everything else from it).
    ``out`` (optional): an [n, H] buffer with contiguous rows that receives ``y`` (a column slice of a wider
    buffer, for instance)."""
    _cuda(h, "h", torch.float32, 2)
    _need(h.stride(1) == 1, "h must have contiguous rows")
    n, H = h.shape
    for t, name in ((gamma, "gamma"), (beta, "beta")):
        _cuda(t, name, torch.float32, 1)
        _need(t.numel() == H and t.is_contiguous(), f"{name} must be a contiguous [H] tensor")
    if bias is not None:
        _cuda(bias, "bias", torch.float32, 1)
        _need(bias.numel() == H and bias.is_contiguous(), "bias must be a contiguous [H] tensor")
    mode = _mode_of(training, p, mask)
    if mode == 2:
        _cuda(mask, "mask", torch.float32, 2)
        _need(mask.shape == h.shape and mask.stride(1) == 1, "mask must be [n, H] with contiguous rows")
    if out is None:
        y = torch.empty((n, H), dtype=torch.float32, device=h.device)
    else:
        y = out
        _cuda(y, "out", torch.float32, 2)
        _need(tuple(y.shape) == (n, H) and y.stride(1) == 1 and y.stride(0) % 4 == 0 and y.data_ptr() % 16 == 0,
              "out must be [n, H] with contiguous, 16-byte aligned rows")
    stats = torch.empty((n, 2), dtype=torch.float32, device=h.device)
    _same_device(h, bias, gamma, beta, mask, y)
    with torch.cuda.device(h.device), _Logged("sage_epilogue_fwd", h.device, n=n, H=H):
        rc = _cabi.lib().sgnn_sage_epilogue_forward(_ptr(h), h.stride(0), _ptr(bias), _ptr(gamma), _ptr(beta),
                                                    _ptr(mask) if mode == 2 else None,
                                                    mask.stride(0) if mode == 2 else 0, mode, int(seed), float(p),
                                                    float(eps), _ptr(y), max(y.stride(0), H), _ptr(stats), n, H,
                                                    _stream(h))
    _cabi.check(rc, "sage_epilogue_forward")
    return y, stats


def sage_epilogue_backward(gy, h, stats, bias, gamma, beta, p: float, training: bool, seed: int, mask=None,
                           in_place: bool = False):
    """Backward of :func:`sage_epilogue_forward` from the same ``h``, ``stats`` and parameters the forward saw:
    returns ``(grad_h, grad_bias, grad_gamma, grad_beta)``.  ``in_place``: ``grad_h`` overwrites ``gy`` (every row
    is read completely before it is written), for a caller that owns ``gy`` and has no further use for it."""
    for t, name in ((gy, "gy"), (h, "h")):
        _cuda(t, name, torch.float32, 2)
        _need(t.stride(1) == 1, f"{name} must have contiguous rows")
    n, H = h.shape
    _cuda(stats, "stats", torch.float32, 2)
    _need(gy.shape == h.shape and tuple(stats.shape) == (n, 2) and stats.is_contiguous(), "shape mismatch")
    for t, name in ((gamma, "gamma"), (beta, "beta")) + (((bias, "bias"),) if bias is not None else ()):
        _cuda(t, name, torch.float32, 1)
        _need(t.numel() == H and t.is_contiguous(), f"{name} must be a contiguous [H] tensor")
    mode = _mode_of(training, p, mask)
    if mode == 2:
        _cuda(mask, "mask", torch.float32, 2)
        _need(mask.shape == h.shape and mask.stride(1) == 1, "mask must be [n, H] with contiguous rows")
    gh = gy if in_place else torch.empty((n, H), dtype=torch.float32, device=h.device)
    lib = _cabi.lib()
    partials = torch.empty((int(lib.sgnn_epilogue_blocks()), 3, H), dtype=torch.float32, device=h.device)
    grads = torch.empty((3, H), dtype=torch.float32, device=h.device)
    _same_device(gy, h, stats, bias, gamma, beta, mask)
    with torch.cuda.device(h.device), _Logged("sage_epilogue_bwd", h.device, n=n, H=H):
        rc = lib.sgnn_sage_epilogue_backward(_ptr(gy), gy.stride(0), _ptr(h), h.stride(0), _ptr(stats), _ptr(bias),
                                             _ptr(gamma), _ptr(beta), _ptr(mask) if mode == 2 else None,
                                             mask.stride(0) if mode == 2 else 0, mode, int(seed), float(p), _ptr(gh),
                                             max(gh.stride(0), H), _ptr(partials), _ptr(grads), n, H, _stream(h))
    _cabi.check(rc, "sage_epilogue_backward")
    return gh, grads[0], grads[1], grads[2]


def softmax_nll_loss(logits, bias, labels, mask, inv_count: float, grad=None):
    """``loss = -sum_{mask} log_softmax(logits + bias)[r, labels[r]] * inv_count`` and its gradient with respect to
    the logits, in one pass.  ``grad`` (optional): a [n, Cg >= C] buffer with contiguous rows that receives the
    gradient (columns beyond C are zeroed).  Returns ``(loss [1], grad)``."""
    _cuda(logits, "logits", torch.float32, 2)
    _need(logits.stride(1) == 1, "logits must have contiguous rows")
    n, C = logits.shape
    _cuda(labels, "labels", torch.int64, 1)
    _need(labels.numel() == n and labels.is_contiguous(), "labels must be a contiguous int64 [n] tensor")
    if bias is not None:
        _cuda(bias, "bias", torch.float32, 1)
        _need(bias.numel() == C and bias.is_contiguous(), "bias must be a contiguous [C] tensor")
    if mask is not None:
        _cuda(mask, "mask", None, 1)
        _need(mask.dtype in (torch.bool, torch.uint8) and mask.numel() == n and mask.is_contiguous(),
              "mask must be a contiguous bool / uint8 [n] tensor")
    if grad is None:
        grad = torch.empty((n, C), dtype=torch.float32, device=logits.device)
    _cuda(grad, "grad", torch.float32, 2)
    _need(grad.size(0) == n and grad.size(1) >= C and grad.stride(1) == 1, "grad must be [n, >= C] with contiguous rows")
    _same_device(logits, bias, labels, mask, grad)
    lib = _cabi.lib()
    partials = torch.empty(int(lib.sgnn_softmax_nll_blocks()), dtype=torch.float32, device=logits.device)
    loss = torch.empty(1, dtype=torch.float32, device=logits.device)
    with torch.cuda.device(logits.device), _Logged("softmax_nll_loss", logits.device, n=n, C=C):
        rc = lib.sgnn_softmax_nll_loss(_ptr(logits), logits.stride(0), _ptr(bias), _ptr(labels), _ptr(mask),
                                       float(inv_count), n, C, _ptr(grad), grad.stride(0), grad.size(1), _ptr(partials),
                                       _ptr(loss), _stream(logits))
    _cabi.check(rc, "softmax_nll_loss")
    return loss, grad


def dropout_mask(seed: int, p: float, n: int, H: int, device) -> torch.Tensor:
    """The scaled keep mask the counter-based dropout applies for ``(seed, p)``."""
    out = torch.empty((n, H), dtype=torch.float32, device=device)
    with torch.cuda.device(out.device):
        rc = _cabi.lib().sgnn_dropout_mask(int(seed), float(p), n, H, _ptr(out), _stream(out))
    _cabi.check(rc, "dropout_mask")
    return out


def find_vertex_cover(*args, **kwargs):
    """Present in the reference's export list (ops.cpp:26) but unreachable from
    its own call graph (VertexCoverFinder.py:629-632); not part of this path."""
    raise RuntimeError("find_vertex_cover is not part of the GraphSAGE hot path and is not provided")
