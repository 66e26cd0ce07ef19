"""Operands with more than 2^31 elements: the reference indexes with 32-bit ints
(spmm.cpp:117-118, the quantisers' int rows) and overflows there; these kernels use 64-bit
offsets.  The big operands exist only on the device; expectations are computed on the host
from the few rows that matter."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _need_memory(gb):
    free, _ = torch.cuda.mem_get_info()
    if free < gb * (1 << 30):
        pytest.skip(f"needs {gb} GB of free device memory")


def test_spmm_gathers_rows_beyond_2_31_elements(oracle):
    _need_memory(14)
    K, N, M = 9_000_000, 256, 64          # K * N = 2.3e9 elements > 2^31
    rng = np.random.default_rng(0)
    X = torch.zeros((K, N), device=DEV)
    hot = np.unique(np.concatenate([rng.integers(K - 1000, K, 40), rng.integers(0, K, 40), [K - 1, 8_388_608, 8_388_607]]))
    Xh = rng.standard_normal((len(hot), N)).astype(np.float32)
    X[torch.from_numpy(hot).to(DEV)] = torch.from_numpy(Xh).to(DEV)
    deg = rng.integers(0, 9, M)
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    pick = rng.integers(0, len(hot), rowptr[-1])
    col = hot[pick].astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32)
    want = oracle.spmm(rowptr, pick.astype(np.int64), val, Xh, np.zeros((M, N), np.float32))  # same rows, compacted
    for algo in (ops.SPMM_ROW_SPLIT, ops.SPMM_NNZ_SPLIT):
        y = torch.empty((M, N), device=DEV)
        ops.spmm(torch.from_numpy(rowptr).to(DEV), torch.from_numpy(col).to(DEV).to(torch.int32),
                 torch.from_numpy(val).to(DEV), X, y, M, None, None, algo=algo, accumulate=False)
        assert np.allclose(y.cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    del X
    torch.cuda.empty_cache()


@pytest.mark.parametrize("bits", [8, 2])
def test_quantise_rows_beyond_2_31_elements(oracle, bits):
    _need_memory(48)
    S, F = 8_500_003, 256                  # S * F = 2.18e9 elements > 2^31; S not a multiple of 4
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn((S, F), generator=g, device=DEV)
    half = S // 2 + 1
    wr = torch.tensor([0, half, S], dtype=torch.int32, device=DEV)
    epb = 8 // bits
    rows = -(-half // epb) + -(-(S - half) // epb)
    packed = torch.empty((rows, F), dtype=torch.uint8, device=DEV)
    params = torch.empty((S, 2), device=DEV)
    ops.quantize_tensor_for_all_procs(x, packed, params, wr, 2, bits)
    # the last 4099 rows (second peer's tail, ragged last group) against the oracle
    tail = 4099
    start = S - tail
    start -= (start - half) % epb          # begin at a group boundary of the second peer
    xs = x[start:].cpu().numpy()
    q_want, p_want = oracle.quantize_for_all_procs(xs, np.array([0, len(xs)], np.int32), bits)
    assert np.array_equal(params[start:].cpu().numpy(), p_want)
    assert np.array_equal(packed[rows - q_want.shape[0]:].cpu().numpy(), q_want)
    out = torch.empty((S, F), device=DEV)
    ops.dequantize_tensor_for_all_procs(packed, out, params, wr, 2, bits)
    d_want = oracle.dequantize_for_all_procs(q_want, p_want, np.array([0, len(xs)], np.int32), bits)
    assert np.array_equal(out[start:].cpu().numpy(), d_want)
    assert ((out - x).abs() / params[:, 1:2]).max().item() <= 0.5 + 1e-3
    del x, out, packed
    torch.cuda.empty_cache()
