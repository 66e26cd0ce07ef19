"""Oracle-backed CPU stand-ins for the CUDA ops — TEST INFRASTRUCTURE ONLY.

``install()`` replaces the functions of ``super_gnn_b200.supergnn_ops`` with
versions that run the CPU oracle on host tensors.  It exists so that the
host-side orchestration (Aggregator, Communicator, graph builder) can be
exercised on gloo CPU ranks, where no CUDA device exists.  The product never
imports this module; without it, every op raises on a CPU tensor.
"""
from __future__ import annotations

import numpy as np
import torch

import oracle
from super_gnn_b200 import supergnn_ops as ops

_saved = {}


def _np(t):
    return None if t is None else t.detach().cpu().contiguous().numpy()


def _params_f32(params):
    return params.float() if params.dtype == torch.bfloat16 else params


def spmm(rowptr, col, value, mat, out, sparse_rows, row_split=None, col_split=None, algo=0, accumulate=True,
         row_scale=None, col_scale=None, nnz_range=None):
    if nnz_range is not None:  # a range of rows of a larger matrix: re-base it to a matrix of its own
        begin, count = int(nnz_range[0]), int(nnz_range[1])
        rowptr = rowptr - begin
        col = col[begin:begin + count]
        value = None if value is None else value[begin:begin + count]
    base = _np(out).copy() if accumulate else np.zeros(tuple(out.shape), np.float32)
    m = _np(mat)
    if col_scale is not None:
        m = m * _np(col_scale)[:, None]
    if row_scale is None:
        res = oracle.spmm(_np(rowptr), _np(col).astype(np.int64), _np(value), m, base)
    else:
        part = oracle.spmm(_np(rowptr), _np(col).astype(np.int64), _np(value), m, np.zeros_like(base))
        res = base + part * _np(row_scale)[:, None]
    out.copy_(torch.from_numpy(res.astype(np.float32)))


def spmm_dequant(rowptr, col, value, packed, params, work_range, num_procs, bits, out, sparse_rows, algo=0,
                 row_scale=None):
    x = oracle.dequantize_for_all_procs(_np(packed), _np(_params_f32(params)), _np(work_range), int(bits))
    spmm(rowptr, col, value, torch.from_numpy(x), out, sparse_rows, row_scale=row_scale)


def csr_row_stats(rowptr):
    d = (rowptr[1:] - rowptr[:-1])
    return (int(d.max()) if d.numel() else 0), int((d == 0).sum())


def quant_pack_rows(src, row_index, work_range, num_procs, bits, packed, params=None, params_bf16=None):
    x = _np(src) if row_index is None else _np(src)[_np(row_index)]
    if x.shape[0] == 0:
        return
    q, p = oracle.quantize_for_all_procs(x, _np(work_range), int(bits))
    packed.view(-1)[: q.size].copy_(torch.from_numpy(q).view(-1))
    if params is not None:
        params[: p.shape[0]].copy_(torch.from_numpy(p))
    if params_bf16 is not None:
        params_bf16[: p.shape[0]].copy_(torch.from_numpy(p).to(torch.bfloat16))


def quantize_tensor_for_all_procs(input, output, params, work_range_per_proc, num_procs, bits):
    quant_pack_rows(input, None, work_range_per_proc, num_procs, bits, output, params=params)


def dequantize_tensor_for_all_procs(input, output, params, work_range_per_proc, num_procs, bits, row_index=None):
    S = int(work_range_per_proc[-1])
    if S == 0:
        return
    x = oracle.dequantize_for_all_procs(_np(input), _np(_params_f32(params))[:S], _np(work_range_per_proc), int(bits))
    if row_index is None:
        output.copy_(torch.from_numpy(x))
    else:
        output.index_add_(0, row_index, torch.from_numpy(x))


def _single(S):
    return np.array([0, S], np.int32)


def quant_pack_rowcodes(src, row_index, bits, codes, params=None, params_bf16=None):
    x = _np(src) if row_index is None else _np(src)[_np(row_index)]
    S = x.shape[0]
    if S == 0:
        return
    q, p = oracle.quantize_for_all_procs(x, _single(S), int(bits))
    rc = oracle.row_codes_of(oracle.codes_of_row_groups(q, _single(S), int(bits)), int(bits))
    codes[:S].copy_(torch.from_numpy(rc))
    if params is not None:
        params[:S].copy_(torch.from_numpy(p))
    if params_bf16 is not None:
        params_bf16[:S].copy_(torch.from_numpy(p).to(torch.bfloat16))


def _rowcodes_values(codes, params, S, F, bits):
    c = oracle.codes_of_row_codes(_np(codes)[:S], F, int(bits))
    q = oracle.row_groups_of(c, _single(S), int(bits))
    return oracle.dequantize_for_all_procs(q, _np(_params_f32(params))[:S], _single(S), int(bits))


def unpack_dequant_rowcodes(codes, output, params, bits, row_index=None):
    S = output.size(0) if row_index is None else row_index.numel()
    if S == 0:
        return
    x = torch.from_numpy(_rowcodes_values(codes, params, S, output.size(1), bits))
    if row_index is None:
        output.copy_(x)
    else:
        output.index_add_(0, row_index, x)


def spmm_dequant_rowcodes(rowptr, col, value, codes, params, bits, out, sparse_rows, algo=0, row_scale=None):
    R = params.size(0)
    x = _rowcodes_values(codes, params, R, out.size(1), bits)
    spmm(rowptr, col, value, torch.from_numpy(x), out, sparse_rows, row_scale=row_scale)


def gather_rows(src, index, out):
    torch.index_select(src, 0, index, out=out)


def scatter_add_rows(src, index, out):
    out.index_add_(0, index, src)


def csr_transpose(rowptr, col, value, num_cols):
    raise RuntimeError("host containers build their transpose in sparse.py")


_REPLACEMENTS = dict(spmm=spmm, spmm_dequant=spmm_dequant, csr_row_stats=csr_row_stats,
                     quant_pack_rows=quant_pack_rows, quantize_tensor_for_all_procs=quantize_tensor_for_all_procs,
                     dequantize_tensor_for_all_procs=dequantize_tensor_for_all_procs, gather_rows=gather_rows,
                     scatter_add_rows=scatter_add_rows, quant_pack_rowcodes=quant_pack_rowcodes,
                     unpack_dequant_rowcodes=unpack_dequant_rowcodes, spmm_dequant_rowcodes=spmm_dequant_rowcodes)


def install():
    import super_gnn_b200.ops.spmm_kernel as sk

    oracle.build()
    for name, fn in _REPLACEMENTS.items():
        _saved.setdefault(name, getattr(ops, name))
        setattr(ops, name, fn)
    _saved.setdefault("sk.spmm", sk.spmm)
    sk.spmm = spmm


def uninstall():
    import super_gnn_b200.ops.spmm_kernel as sk

    for name in _REPLACEMENTS:
        if name in _saved:
            setattr(ops, name, _saved[name])
    if "sk.spmm" in _saved:
        sk.spmm = _saved["sk.spmm"]
