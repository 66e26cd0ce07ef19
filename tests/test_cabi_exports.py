"""The C-ABI library loads on a machine without a GPU, exports every symbol the
header declares, and rejects malformed arguments on the host (no launch)."""
import os
import re

import pytest

from super_gnn_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "supergnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sgnn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 15
    lib = _cabi.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _cabi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_cabi.SIGNATURES) == names
    assert lib.sgnn_version() >= 100


@pytest.mark.parametrize("call,needle", [
    (lambda l: l.sgnn_spmm_csr_f32(None, None, None, -1, None, 0, None, 0, 0, 0, 0, 0, 0, None, None, None), "negative"),
    (lambda l: l.sgnn_spmm_csr_f32(None, None, None, 0, None, 0, None, 0, 1, 1, 4, 0, 0, None, None, None), "rowptr"),
    (lambda l: l.sgnn_spmm_csr_f32(8, None, None, 0, None, 2, 8, 4, 1, 1, 4, 0, 0, None, None, None), "ldx"),
    (lambda l: l.sgnn_spmm_csr_f32(8, None, None, 0, 8, 4, 8, 4, 1, 1, 4, 0, 7, None, None, None), "algo"),
    (lambda l: l.sgnn_quant_pack_rows(8, 4, None, 4, 4, 8, 1, 3, 8, None, None, None), "bits"),
    (lambda l: l.sgnn_quant_pack_rows(8, 4, None, 4, 4, None, 1, 2, 8, None, None, None), "work_range"),
    (lambda l: l.sgnn_quant_pack_rows(8, 4, None, 4, 4, 8, 5000, 2, 8, None, None, None), "P="),
    (lambda l: l.sgnn_unpack_dequant_rows(8, None, None, 4, 4, 8, 1, 2, 8, 4, None, None), "exactly one"),
    (lambda l: l.sgnn_spmm_csr_dequant_f32(8, 8, None, 1, 8, 8, 8, 4, 4, 8, 1, 2, 8, 4, 1, 0, None, None), "exactly one"),
    (lambda l: l.sgnn_csr_transpose(8, 8, None, 1, 1, 1, 8, 8, None, None, 0, None), "workspace"),
    (lambda l: l.sgnn_gather_rows(8, 2, 8, 1, 4, 8, 4, None), "leading dimension"),
    (lambda l: l.sgnn_quantize_tensor(8, 1, 4, 8, 8, 5, 8, None), "bits"),
])
def test_malformed_arguments_are_rejected_before_any_launch(call, needle):
    lib = _cabi.lib()
    rc = call(lib)
    assert rc != 0
    assert needle in _cabi.last_error()


def test_workspace_query_never_faults():
    # 0 means "cannot be served": sizes out of range, or (here) no CUDA device to size the sort for
    assert _cabi.lib().sgnn_csr_transpose_workspace_bytes(10, 10, 2 ** 31) == 0
    assert _cabi.lib().sgnn_csr_transpose_workspace_bytes(10, 10, 100) >= 0


def test_build_finds_a_cutlass_tree_with_the_sm100_emulated_fp32_mainloop():
    """The dense GEMM is compiled from CUTLASS templates: the build must locate a header tree that has them."""
    import os

    from super_gnn_b200 import build

    inc = build.cutlass_include()
    assert os.path.exists(os.path.join(inc, "cutlass", "gemm", "collective", "sm100_mma_warpspecialized_emulated.hpp"))
    assert os.path.exists(os.path.join(inc, "cute", "tensor.hpp"))


def test_gemm_entry_points_validate_on_the_host():
    """Bad arguments are rejected before any CUDA call (no GPU needed)."""
    import ctypes

    from super_gnn_b200 import _cabi

    lib = _cabi.lib()
    need = ctypes.c_size_t(123)
    assert lib.sgnn_gemm_f32_workspace_bytes(7, 4, 4, 4, ctypes.byref(need)) == 1       # unknown op
    assert lib.sgnn_gemm_f32_workspace_bytes(0, 4, 4, 0, ctypes.byref(need)) == 1       # K == 0
    assert lib.sgnn_gemm_f32_workspace_bytes(0, 1 << 31, 4, 4, ctypes.byref(need)) == 4  # too large
    assert lib.sgnn_gemm_f32_workspace_bytes(0, 0, 4, 4, ctypes.byref(need)) == 0 and need.value == 0
    assert lib.sgnn_gemm_f32(0, None, 4, None, 4, None, 4, 4, 4, 4, 0.0, None, 0, None) == 1  # null pointers
    assert b"null pointer" in lib.sgnn_last_error_string()
    buf = (ctypes.c_float * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.sgnn_gemm_f32(0, p, 3, p, 4, p, 4, 4, 4, 4, 0.0, None, 0, None) == 1      # lda < K
    assert lib.sgnn_gemm_f32(0, p, 6, p, 4, p, 4, 4, 4, 4, 0.0, None, 0, None) == 1      # lda not a multiple of 4


def test_layer_fusion_and_one_sided_exchange_decide_per_width():
    """Host-side decisions that keep unsupported widths off the vector kernels (no GPU involved)."""
    from super_gnn_b200.graphsage import DistSAGE
    from super_gnn_b200.peer_exchange import PeerExchange
    from super_gnn_b200 import supergnn_ops as ops

    m = DistSAGE(602, 256, 41, 3)   # reddit: 602 input channels
    assert not m._layer_fusable(m.convs[0], hidden=True)    # rows of 602 floats are not 16-byte multiples
    assert m._layer_fusable(m.convs[1], hidden=True) and m._layer_fusable(m.convs[2], hidden=False)
    assert not DistSAGE(100, 130, 10, 3)._layer_fusable(DistSAGE(100, 130, 10, 3).convs[0], hidden=True)
    assert PeerExchange.supports(256) and not PeerExchange.supports(602) and not PeerExchange.supports(1024)
    assert ops.rowcodes_supported(100) and ops.rowcodes_supported(512) and not ops.rowcodes_supported(768)
