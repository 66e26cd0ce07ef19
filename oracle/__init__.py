"""numpy front end of the CPU oracle (``sgnn_oracle.c``) — TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline legs may
import this package; the product package never does.  Each wrapper names the
reference function it restates; the C file carries the file:line citations.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "sgnn_oracle.c")
_LIB = os.path.join(_HERE, "libsgnn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile ``sgnn_oracle.c`` with gcc (no-op when the library is current)."""
    if not force and os.path.exists(_LIB) and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC):
        return _LIB
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    subprocess.check_call([cc, "-O2", "-fopenmp", "-ffp-contract=off", "-mfma", "-shared", "-fPIC",
                           "-fvisibility=hidden", _SRC, "-o", _LIB, "-lm"])
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        _lib = ctypes.CDLL(_LIB)
        _lib.oracle_packed_rows.restype = ctypes.c_int64
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=dtype)


I64 = ctypes.c_int64


def spmm(rowptr, col, value, mat, out) -> np.ndarray:
    """``out += A @ mat`` in place (supergnn_ops.spmm, optimized path)."""
    rowptr = _c(rowptr, np.int64); col = _c(col, np.int64)
    value = None if value is None else _c(value, np.float32)
    mat = _c(mat, np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    M, N = out.shape
    lib().oracle_spmm_csr_f32(_p(rowptr), _p(col), _p(value), _p(mat), _p(out), I64(M), I64(N))
    return out


def distribute_work_for_row(rowptr, value, num_threads: int) -> np.ndarray:
    """Greedy row split of super_gnn/ops/spmm_kernel.py:8-29."""
    rowptr = _c(rowptr, np.int64); value = _c(value, np.float32)
    out = np.empty(num_threads + 1, np.int32)
    lib().oracle_distribute_work_for_row(_p(rowptr), _p(value), I64(len(rowptr) - 1), int(num_threads), _p(out))
    return out


def row_params(x, bits: int) -> np.ndarray:
    x = _c(x, np.float32); S, F = x.shape
    params = np.empty((S, 2), np.float32)
    lib().oracle_row_params(_p(x), I64(S), I64(F), int(bits), _p(params))
    return params


def quantize_tensor(x, mn, scale, bits: int) -> np.ndarray:
    """x86 5-argument ``quantize_tensor`` (caller-supplied min/scale)."""
    x = _c(x, np.float32); mn = _c(mn, np.float32); scale = _c(scale, np.float32)
    S, F = x.shape
    epb = 8 // bits
    out = np.zeros(((S + epb - 1) // epb, F), np.uint8)
    rc = lib().oracle_quantize_tensor(_p(x), I64(S), I64(F), _p(mn), _p(scale), int(bits), _p(out))
    assert rc == 0
    return out


def dequantize_tensor(q, S: int, mn, scale, bits: int) -> np.ndarray:
    q = _c(q, np.uint8); mn = _c(mn, np.float32); scale = _c(scale, np.float32)
    F = q.shape[1]
    out = np.empty((S, F), np.float32)
    rc = lib().oracle_dequantize_tensor(_p(q), I64(S), I64(F), _p(mn), _p(scale), int(bits), _p(out))
    assert rc == 0
    return out


def packed_rows(work_range, bits: int) -> int:
    wr = _c(work_range, np.int32)
    return int(lib().oracle_packed_rows(_p(wr), len(wr) - 1, int(bits)))


def quantize_for_all_procs(x, work_range, bits: int):
    """``quantize_tensor_for_all_procs``: returns (packed uint8 [rows,F], params fp32 [S,2])."""
    x = _c(x, np.float32); wr = _c(work_range, np.int32)
    S, F = x.shape
    assert wr[-1] == S and wr[0] == 0
    out = np.zeros((packed_rows(wr, bits), F), np.uint8)
    params = np.zeros((S, 2), np.float32)
    rc = lib().oracle_quantize_for_all_procs(_p(x), I64(F), _p(wr), len(wr) - 1, int(bits), _p(out), _p(params))
    assert rc == 0
    return out, params


def dequantize_for_all_procs(q, params, work_range, bits: int) -> np.ndarray:
    q = _c(q, np.uint8); params = _c(params, np.float32); wr = _c(work_range, np.int32)
    F = q.shape[1]; S = int(wr[-1])
    out = np.zeros((S, F), np.float32)
    rc = lib().oracle_dequantize_for_all_procs(_p(q), _p(params), I64(F), _p(wr), len(wr) - 1, int(bits), _p(out))
    assert rc == 0
    return out


def codes_of_row_groups(q, work_range, bits: int) -> np.ndarray:
    """The code of every (row, feature) recovered from the reference's row-group bytes
    (quantization_arm.cpp:177-185: row i of a peer's segment sits in packed row off_p + i // EPB at
    shift (EPB - 1 - i % EPB) * bits).  Returns uint8 [S, F]."""
    work_range = np.asarray(work_range, np.int64)
    epb = 8 // bits
    q = np.asarray(q, np.uint8)
    F = q.shape[1] if q.ndim == 2 else 0
    S = int(work_range[-1])
    out = np.zeros((S, F), np.uint8)
    off = 0
    for p in range(len(work_range) - 1):
        a, b = int(work_range[p]), int(work_range[p + 1])
        i = np.arange(b - a)
        rows = q[off + i // epb]
        shift = ((epb - 1 - i % epb) * bits).astype(np.uint8)
        out[a:b] = (rows >> shift[:, None]) & ((1 << bits) - 1)
        off += -(-(b - a) // epb)
    return out


def row_codes_of(codes, bits: int) -> np.ndarray:
    """Row-codes bytes (include/supergnn_b200.h, "Row codes") of a uint8 [S, F] matrix of codes: quad q =
    features 4q..4q+3 as one little-endian field of 4*bits bits, feature j at bit j*bits; quad q at position q
    for F <= 128, else (q % 32) * NV + q // 32 with NV = F // 128.  Returns uint8 [S, F*bits/8]."""
    codes = np.asarray(codes, np.uint8)
    S, F = codes.shape
    assert F % 4 == 0 and (F <= 128 or F in (256, 512))
    Q, nv, qb = F // 4, (1 if F <= 128 else F // 128), bits // 2
    quads = codes.reshape(S, Q, 4).astype(np.uint32)
    field = quads[:, :, 0] | (quads[:, :, 1] << bits) | (quads[:, :, 2] << (2 * bits)) | (quads[:, :, 3] << (3 * bits))
    qi = np.arange(Q)
    pos = qi if nv == 1 else (qi % 32) * nv + qi // 32
    out = np.zeros((S, Q * qb), np.uint8)
    for k in range(qb):
        out[:, pos * qb + k] = ((field >> (8 * k)) & 0xFF).astype(np.uint8)
    return out


def codes_of_row_codes(rc, F: int, bits: int) -> np.ndarray:
    """Inverse of :func:`row_codes_of`: uint8 [S, F] codes from row-codes bytes."""
    rc = np.asarray(rc, np.uint8)
    S = rc.shape[0]
    Q, nv, qb = F // 4, (1 if F <= 128 else F // 128), bits // 2
    qi = np.arange(Q)
    pos = qi if nv == 1 else (qi % 32) * nv + qi // 32
    field = np.zeros((S, Q), np.uint32)
    for k in range(qb):
        field |= rc[:, pos * qb + k].astype(np.uint32) << (8 * k)
    out = np.zeros((S, Q, 4), np.uint8)
    for j in range(4):
        out[:, :, j] = ((field >> (j * bits)) & ((1 << bits) - 1)).astype(np.uint8)
    return out.reshape(S, F)


def row_groups_of(codes, work_range, bits: int) -> np.ndarray:
    """The reference's row-group bytes of a uint8 [S, F] matrix of codes (inverse of
    :func:`codes_of_row_groups`)."""
    work_range = np.asarray(work_range, np.int64)
    codes = np.asarray(codes, np.uint8)
    epb = 8 // bits
    F = codes.shape[1]
    out = np.zeros((packed_rows(work_range, bits), F), np.uint8)
    off = 0
    for p in range(len(work_range) - 1):
        a, b = int(work_range[p]), int(work_range[p + 1])
        for i in range(b - a):
            out[off + i // epb] |= (codes[a + i] << ((epb - 1 - i % epb) * bits)).astype(np.uint8)
        off += -(-(b - a) // epb)
    return out


def quantized_nodes_feat_range(feat_len: int, bits_per_row) -> np.ndarray:
    """super_gnn/quantizer.py:66-73."""
    b = np.asarray(bits_per_row, np.float64)
    lens = np.ceil(b * feat_len / 8.0).astype(np.int64)
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)


def quantize_v1(x, bits_per_row):
    """``quantize_tensor_v1``: returns (bytes, params [S,3], range [S+1])."""
    x = _c(x, np.float32); S, F = x.shape
    rng = quantized_nodes_feat_range(F, bits_per_row)
    params = np.zeros((S, 3), np.float32); params[:, 0] = np.asarray(bits_per_row, np.float32)
    out = np.zeros(int(rng[-1]), np.uint8)
    rc = lib().oracle_quantize_v1(_p(x), I64(S), I64(F), _p(rng), _p(params), _p(out))
    assert rc == 0
    return out, params, rng


def dequantize_v1(q, params, F: int) -> np.ndarray:
    q = _c(q, np.uint8); params = _c(params, np.float32)
    S = params.shape[0]
    rng = quantized_nodes_feat_range(F, params[:, 0])
    out = np.zeros((S, F), np.float32)
    rc = lib().oracle_dequantize_v1(_p(q), I64(S), I64(F), _p(rng), _p(params), _p(out))
    assert rc == 0
    return out


def quantize_v2_torch(x, zero_points, scales, bits: int):
    x = _c(x, np.float32); S, F = x.shape
    zp = _c(zero_points, np.float32); sc = _c(scales, np.float32)
    rng = quantized_nodes_feat_range(F, np.full(S, bits))
    out = np.zeros(int(rng[-1]), np.uint8)
    rc = lib().oracle_quantize_v2_torch(_p(x), I64(S), I64(F), _p(rng), _p(zp), _p(sc), int(bits), _p(out))
    assert rc == 0
    return out, rng


def dequantize_v2_torch(q, S: int, F: int, zero_points, scales, bits: int) -> np.ndarray:
    q = _c(q, np.uint8); zp = _c(zero_points, np.float32); sc = _c(scales, np.float32)
    rng = quantized_nodes_feat_range(F, np.full(S, bits))
    out = np.zeros((S, F), np.float32)
    rc = lib().oracle_dequantize_v2_torch(_p(q), I64(S), I64(F), _p(rng), _p(zp), _p(sc), int(bits), _p(out))
    assert rc == 0
    return out


def round_bf16(a) -> np.ndarray:
    """fp32 -> bf16 (round to nearest even) -> fp32, as the params travel."""
    a = _c(a, np.float32)
    out = np.empty_like(a)
    lib().oracle_round_bf16(_p(a), I64(a.size), _p(out))
    return out


def quantized_splits(splits, bits: int) -> list:
    """Packed rows per peer: super_gnn/quantizer.py:91-92, data_manager/CommSplits.py:13-18."""
    epb = 8 // bits
    return [-(-int(s) // epb) for s in splits]


def splits_for_comm_quantized_data(recv_splits, send_splits, dequantized_range, quantized_range):
    """super_gnn/communicator.py:308-342 (byte counts per peer for the v1 layout)."""
    rb = np.concatenate([[0], np.cumsum(np.asarray(recv_splits, np.int64))])
    sb = np.concatenate([[0], np.cumsum(np.asarray(send_splits, np.int64))])
    dr = np.asarray(dequantized_range, np.int64); qr = np.asarray(quantized_range, np.int64)
    return ([int(dr[rb[i + 1]] - dr[rb[i]]) for i in range(len(recv_splits))],
            [int(qr[sb[i + 1]] - qr[sb[i]]) for i in range(len(send_splits))])
