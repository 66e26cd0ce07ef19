"""Fused dequantise-SpMM, CSR transpose and the single-process Aggregator vs the CPU oracle."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops
from super_gnn_b200.aggregator import Aggregator
from super_gnn_b200.data_manager import build_distributed_graph
from super_gnn_b200.sparse import SparseTensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


def random_csr(M, K, mean_deg, seed):
    rng = np.random.default_rng(seed)
    deg = rng.poisson(mean_deg, M)
    deg[::5] = 0
    deg[1] = 900
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = rng.integers(0, K, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32)
    return rowptr, col, val


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("F", [256, 128, 100, 37])
@pytest.mark.parametrize("bf16_params", [False, True])
def test_spmm_dequant_equals_dequantise_then_spmm(oracle, bits, F, bf16_params):
    M, R, P = 400, 1211, 5
    rng = np.random.default_rng(F + bits)
    x = (rng.standard_normal((R, F)) * np.exp(rng.standard_normal((R, 1)))).astype(np.float32)
    wr = np.array([0, 300, 300, 707, 1210, 1211], np.int32)
    q, p = oracle.quantize_for_all_procs(x, wr, bits)
    p_used = oracle.round_bf16(p) if bf16_params else p
    xhat = oracle.dequantize_for_all_procs(q, p_used, wr, bits)
    rowptr, col, val = random_csr(M, R, 6, seed=bits)
    Y0 = rng.standard_normal((M, F)).astype(np.float32)
    want = oracle.spmm(rowptr, col, val, xhat, Y0.copy())
    mag = oracle.spmm(rowptr, col, np.abs(val), np.abs(xhat), np.abs(Y0))
    params_t = torch.from_numpy(p).to(DEV)
    if bf16_params:
        params_t = params_t.to(torch.bfloat16)
    for algo in (ops.SPMM_ROW_SPLIT, ops.SPMM_NNZ_SPLIT):
        y = torch.from_numpy(Y0.copy()).to(DEV)
        ops.spmm_dequant(torch.from_numpy(rowptr).to(DEV), torch.from_numpy(col).to(DEV).to(torch.int32),
                         torch.from_numpy(val).to(DEV), torch.from_numpy(q).to(DEV), params_t,
                         torch.from_numpy(wr).to(DEV), P, bits, y, M, algo=algo)
        err = np.abs(y.cpu().numpy() - want)
        assert np.all(err <= 1e-5 * (mag + np.abs(want)) + 1e-30), np.max(err / (mag + 1e-30))


@pytest.mark.parametrize("weighted", [True, False])
def test_csr_transpose_matches_host(weighted):
    M, K = 1500, 900
    rowptr, col, val = random_csr(M, K, 7, seed=2)
    A = SparseTensor(rowptr=torch.from_numpy(rowptr), col=torch.from_numpy(col),
                     value=torch.from_numpy(val) if weighted else None, sparse_sizes=(M, K), is_sorted=True)
    Ad = A.to(DEV)
    assert torch.equal(Ad.storage.colptr().cpu(), A.storage.colptr())
    assert torch.equal(Ad.storage.row_T().cpu(), A.storage.row_T())
    if weighted:
        assert torch.equal(Ad.storage.value_T().cpu(), A.storage.value_T())
    else:
        assert Ad.storage.value_T() is None
    mx, empty = ops.csr_row_stats(Ad.storage.rowptr())
    deg = np.diff(rowptr)
    assert mx == deg.max() and empty == int((deg == 0).sum())
    # empty matrix
    E = SparseTensor(rowptr=torch.zeros(4, dtype=torch.int64), col=torch.zeros(0, dtype=torch.int64),
                     sparse_sizes=(3, 5), is_sorted=True).to(DEV)
    assert E.storage.colptr().tolist() == [0] * 6 and E.storage.row_T().numel() == 0


def test_single_process_aggregator_forward_backward(oracle):
    """world_size == 1: Aggregator == A x and its gradient == A^T g."""
    n, F = 3000, 100
    rng = np.random.default_rng(0)
    E = 40000
    src = torch.from_numpy(rng.integers(0, n, E))
    dst = torch.from_numpy(rng.integers(0, n, E))
    graph = build_distributed_graph(torch.stack([src, dst]), torch.zeros((2, 0), dtype=torch.int64), [0, n], F, 32,
                                    device=torch.device(DEV))
    x = torch.randn(n, F, device=DEV, requires_grad=True)
    out = Aggregator.apply(graph, x, 0, 32, False, True)
    g = torch.randn_like(out)
    out.backward(g)
    rowptr, col, _ = graph.local_adj_t.csr()
    rowptr, col = rowptr.cpu().numpy(), col.cpu().numpy().astype(np.int64)
    want = oracle.spmm(rowptr, col, None, x.detach().cpu().numpy(), np.zeros((n, F), np.float32))
    mag = oracle.spmm(rowptr, col, None, x.detach().abs().cpu().numpy(), np.zeros((n, F), np.float32))
    assert np.all(np.abs(out.detach().cpu().numpy() - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30)
    At = torch.sparse_coo_tensor(torch.stack([src, dst]), torch.ones(E), (n, n)).coalesce()  # [src, dst] = A^T
    want_g = torch.sparse.mm(At, g.cpu())
    assert torch.allclose(x.grad.cpu(), want_g, rtol=1e-4, atol=1e-4)
    deg = torch.bincount(dst, minlength=n).clamp(min=1).float()
    assert torch.equal(graph.in_degrees.cpu().squeeze(1), deg)
