"""ctypes binding of ``libsupergnn_b200.so`` (declarations: ``include/supergnn_b200.h``).

There is no CPU fallback: if the library is missing it is built with nvcc, and
if that is impossible the import fails loudly.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_size_t, c_uint32, c_uint64, c_void_p

from . import build as _build

_lib = None

_P = c_void_p
_I = c_int
_L = c_int64

# name -> (restype, argtypes); one entry per declaration in include/supergnn_b200.h
SIGNATURES = {
    "sgnn_version": (_I, []),
    "sgnn_last_error_string": (ctypes.c_char_p, []),
    "sgnn_spmm_csr_f32": (_I, [_P, _P, _P, _L, _P, _L, _P, _L, _L, _L, _L, _I, _I, _P, _P, _P]),
    "sgnn_spmm_csr_rows_f32": (_I, [_P, _P, _P, _L, _L, _P, _L, _P, _L, _L, _L, _L, _I, _I, _P, _P, _P]),
    "sgnn_csr_check": (_I, [_P, _P, _L, _L, _L, _P, _P]),
    "sgnn_csr_row_stats": (_I, [_P, _L, _P, _P]),
    "sgnn_csr_transpose_workspace_bytes": (c_size_t, [_L, _L, _L]),
    "sgnn_csr_transpose": (_I, [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P, c_size_t, _P]),
    "sgnn_csr_transpose_noalloc": (_I, [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P]),
    "sgnn_quant_pack_rows": (_I, [_P, _L, _P, _L, _L, _P, _I, _I, _P, _P, _P, _P]),
    "sgnn_quant_pack_rows_p2p": (_I, [_P, _L, _P, _L, _L, _P, _I, _I, _P, _P, _P, _P, _P, _P]),
    "sgnn_unpack_dequant_rows": (_I, [_P, _P, _P, _L, _L, _P, _I, _I, _P, _L, _P, _P]),
    "sgnn_spmm_csr_dequant_f32": (_I, [_P, _P, _P, _L, _P, _P, _P, _L, _L, _P, _I, _I, _P, _L, _L, _I, _P, _P]),
    "sgnn_rowcodes_width_supported": (_I, [_L]),
    "sgnn_quant_pack_rowcodes": (_I, [_P, _L, _P, _L, _L, _I, _P, _P, _P, _P]),
    "sgnn_quant_pack_rowcodes_p2p": (_I, [_P, _L, _P, _L, _L, _P, _I, _I, _P, _P, _P, _P, _P]),
    "sgnn_unpack_dequant_rowcodes": (_I, [_P, _P, _P, _L, _L, _I, _P, _L, _P, _P]),
    "sgnn_spmm_csr_dequant_rowcodes_f32": (_I, [_P, _P, _P, _L, _P, _P, _P, _L, _L, _I, _P, _L, _L, _I, _P, _P]),
    "sgnn_quantize_tensor": (_I, [_P, _L, _L, _P, _P, _I, _P, _P]),
    "sgnn_dequantize_tensor": (_I, [_P, _L, _L, _P, _P, _I, _P, _P]),
    "sgnn_quantize_rows_v1": (_I, [_P, _L, _L, _P, _P, _P, _P]),
    "sgnn_dequantize_rows_v1": (_I, [_P, _L, _L, _P, _P, _P, _P]),
    "sgnn_quantize_rows_v2": (_I, [_P, _L, _L, _P, _P, _P, _I, _P, _P]),
    "sgnn_dequantize_rows_v2": (_I, [_P, _L, _L, _P, _P, _P, _I, _P, _P]),
    "sgnn_epilogue_blocks": (_I, []),
    "sgnn_sage_epilogue_forward": (_I, [_P, _L, _P, _P, _P, _P, _L, _I, c_uint64, c_float, c_float, _P, _L, _P, _L, _L,
                                         _P]),
    "sgnn_sage_epilogue_backward": (_I, [_P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _I, c_uint64, c_float, _P, _L, _P, _P,
                                          _L, _L, _P]),
    "sgnn_softmax_nll_blocks": (_I, []),
    "sgnn_softmax_nll_loss": (_I, [_P, _L, _P, _P, _P, c_float, _L, _L, _P, _L, _L, _P, _P, _P]),
    "sgnn_gemm_f32_workspace_bytes": (_I, [_I, _L, _L, _L, _P]),
    "sgnn_gemm_f32": (_I, [_I, _P, _L, _P, _L, _P, _L, _L, _L, _L, c_float, _P, c_size_t, _P]),
    "sgnn_dropout_mask": (_I, [c_uint64, c_float, _L, _L, _P, _P]),
    "sgnn_bipartite_min_vertex_cover": (_I, [_L, _L, _P, _P, _P, _P, _P]),
    "sgnn_peer_barrier": (_I, [_P, c_int, c_int, c_uint32, _L, _P, _P]),
    "sgnn_gather_rows": (_I, [_P, _L, _P, _L, _L, _P, _L, _P]),
    "sgnn_scatter_add_rows": (_I, [_P, _L, _P, _L, _L, _P, _L, _P]),
}


def library_path() -> str:
    return _build.LIB


def lib() -> ctypes.CDLL:
    """Load (building first if needed) the C-ABI library."""
    global _lib
    if _lib is None:
        if not os.path.exists(_build.LIB):
            _build.build()
        if not os.path.exists(_build.LIB):
            raise RuntimeError("libsupergnn_b200.so is missing and could not be built; "
                               "supergnn_b200 has no CPU or PyTorch fallback")
        l = ctypes.CDLL(_build.LIB)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)  # AttributeError here = header and library out of sync
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def last_error() -> str:
    return lib().sgnn_last_error_string().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status (the reference raises RuntimeError
    from AT_ASSERTM / TORCH_CHECK, super_gnn/ops/csrc/utils.h:12-13)."""
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {last_error()}")
