"""CUDA SpMM vs the CPU oracle on the same seeded inputs, through the C ABI.
Tolerance: 1e-5 relative to the row scale (fp32, summation order differs)."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops
from super_gnn_b200 import synthetic
from super_gnn_b200.ops.spmm_kernel import SPMM_backward, SPMM_forward
from super_gnn_b200.sparse import SparseTensor

pytestmark = pytest.mark.gpu
DEV = "cuda"
RTOL = 1e-5


def random_csr(M, K, mean_deg, seed, heavy=None, empty_every=0, weighted=True):
    rng = np.random.default_rng(seed)
    deg = rng.poisson(mean_deg, M)
    if empty_every:
        deg[::empty_every] = 0
    if heavy:
        for r, d in heavy.items():
            if r < M:
                deg[r] = d
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = rng.integers(0, K, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32) if weighted else None
    return rowptr, col, val


def assert_close(got, want, absx_rowsum):
    """|got - want| <= RTOL * (sum_e |w_e| |x_e| + |want|), elementwise."""
    err = np.abs(got - want)
    bound = RTOL * (absx_rowsum + np.abs(want)) + 1e-30
    assert np.all(err <= bound), f"max err/bound = {np.max(err / bound):.3f}"


# the two work splits, and the nnz split with its rows staged through shared memory
ALGOS = [ops.SPMM_ROW_SPLIT, ops.SPMM_NNZ_SPLIT, ops.SPMM_NNZ_SPLIT_STAGED]


def run_case(oracle, rowptr, col, val, K, N, algo, accumulate, seed=0):
    rng = np.random.default_rng(seed + 100)
    M = len(rowptr) - 1
    X = rng.standard_normal((K, N)).astype(np.float32)
    Y0 = rng.standard_normal((M, N)).astype(np.float32)
    base = Y0.copy() if accumulate else np.zeros_like(Y0)
    want = oracle.spmm(rowptr, col, val, X, base.copy())
    mag = oracle.spmm(rowptr, col, None if val is None else np.abs(val), np.abs(X), np.abs(base))
    y = torch.from_numpy(Y0.copy()).to(DEV)
    ops.spmm(torch.from_numpy(rowptr).to(DEV), torch.from_numpy(col).to(DEV).to(torch.int32),
             None if val is None else torch.from_numpy(val).to(DEV), torch.from_numpy(X).to(DEV), y, M, None, None,
             algo=algo, accumulate=accumulate)
    assert_close(y.cpu().numpy(), want, mag)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("N", [1, 3, 4, 16, 32, 47, 48, 64, 100, 128, 172, 256, 300, 640])
def test_widths(oracle, algo, N):
    rowptr, col, val = random_csr(517, 333, 9, seed=N, heavy={5: 700, 6: 129}, empty_every=7)
    run_case(oracle, rowptr, col, val, 333, N, algo, accumulate=True, seed=N)
    run_case(oracle, rowptr, col, val, 333, N, algo, accumulate=False, seed=N + 1)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("M", [1, 3, 4, 5, 33, 255])
def test_tiny_and_degenerate_shapes(oracle, algo, M):
    for mean_deg in (0.0, 0.5, 40.0):
        rowptr, col, val = random_csr(M, 7, mean_deg, seed=M)
        run_case(oracle, rowptr, col, val, 7, 8, algo, accumulate=True)
        run_case(oracle, rowptr, col, val, 7, 5, algo, accumulate=False)


@pytest.mark.parametrize("algo", ALGOS)
def test_unweighted_sum_aggregation(oracle, algo):
    rowptr, col, _ = random_csr(1000, 1000, 12, seed=3, weighted=False)
    run_case(oracle, rowptr, col, None, 1000, 128, algo, accumulate=False)


def test_long_rows_and_runs_of_empty_rows(oracle):
    # a row longer than many warp chunks, chunk boundaries falling on row boundaries, and
    # more than 32 consecutive empty rows inside a chunk
    deg = np.array([128, 0, 128, 5000] + [0] * 100 + [1, 127, 256, 0, 0, 3] + [0] * 40 + [2], np.int64)
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    rng = np.random.default_rng(9)
    col = rng.integers(0, 50, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32)
    for algo in ALGOS:
        run_case(oracle, rowptr, col, val, 50, 128, algo, accumulate=True)
        run_case(oracle, rowptr, col, val, 50, 100, algo, accumulate=False)


def test_matches_reference_golden(golden):
    for N in (7, 16, 100):
        y = torch.from_numpy(golden[f"spmm_Y0_{N}"].copy()).to(DEV)
        M = y.shape[0]
        for algo in ALGOS:
            yy = y.clone()
            ops.spmm(torch.from_numpy(golden["spmm_rowptr"]).to(DEV), torch.from_numpy(golden["spmm_col"]).to(DEV),
                     torch.from_numpy(golden["spmm_val"]).to(DEV), torch.from_numpy(golden[f"spmm_X_{N}"]).to(DEV), yy,
                     M, None, None, algo=algo)
            want = golden[f"spmm_Y_{N}"]
            assert np.allclose(yy.cpu().numpy(), want, rtol=1e-5, atol=1e-5)  # the reference test's atol


def test_config1_shape_forward_and_transposed(oracle):
    """200k x 200k, Poisson(12) degrees, values 1/deg, X 200k x 128 (seed 0), as SPMM_forward /
    SPMM_backward are called; the backward against the oracle on the transposed CSR."""
    n, N = 200_000, 128
    rowptr, col, val = synthetic.poisson_csr(n, n, 12.0, seed=0)
    g = torch.Generator().manual_seed(0)
    X = torch.randn(n, N, generator=g)
    A = SparseTensor(rowptr=rowptr.to(DEV), col=col.to(DEV), value=val.to(DEV), sparse_sizes=(n, n), is_sorted=True)
    out = torch.zeros(n, N, device=DEV)
    SPMM_forward(A, X.to(DEV), out)
    want = oracle.spmm(rowptr.numpy(), col.numpy(), val.numpy(), X.numpy(), np.zeros((n, N), np.float32))
    mag = oracle.spmm(rowptr.numpy(), col.numpy(), val.numpy(), X.abs().numpy(), np.zeros((n, N), np.float32))
    assert_close(out.cpu().numpy(), want, mag)
    # transposed: out_T = A^T X
    outT = torch.zeros(n, N, device=DEV)
    SPMM_backward(A, X.to(DEV), outT)
    colptr, row_T, val_T = A.storage.colptr().cpu().numpy(), A.storage.row_T().cpu().numpy(), A.storage.value_T().cpu().numpy()
    # the device-built transpose is the CSR of A^T with ascending rows
    dense_check = torch.sparse_csr_tensor(rowptr, col.to(torch.int64), val, size=(n, n)).to_sparse_coo().t().coalesce()
    wantT = oracle.spmm(colptr, row_T, val_T, X.numpy(), np.zeros((n, N), np.float32))
    magT = oracle.spmm(colptr, row_T, val_T, X.abs().numpy(), np.zeros((n, N), np.float32))
    assert_close(outT.cpu().numpy(), wantT, magT)
    ref = torch.sparse.mm(dense_check, X)
    assert torch.allclose(outT.cpu(), ref, rtol=1e-4, atol=1e-5)


def test_size_independent_properties_full_size():
    """Linearity and a row-sum identity at the full configuration-1 size on both kernels."""
    n, N = 200_000, 128
    rowptr, col, val = synthetic.poisson_csr(n, n, 12.0, seed=0, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(5)
    X1 = torch.randn(n, N, generator=g, device=DEV)
    X2 = torch.randn(n, N, generator=g, device=DEV)
    for algo in ALGOS:
        def mm(X):
            y = torch.empty(n, N, device=DEV)
            ops.spmm(rowptr, col, val, X, y, n, None, None, algo=algo, accumulate=False)
            return y
        y1, y2, y12 = mm(X1), mm(X2), mm(2.0 * X1 - 3.0 * X2)
        assert torch.allclose(y12, 2.0 * y1 - 3.0 * y2, rtol=1e-4, atol=1e-4)
        ones = mm(torch.ones(n, N, device=DEV))  # rows of a mean-aggregation matrix sum to 1 (0 if empty)
        deg = (rowptr[1:] - rowptr[:-1]).clamp(max=1).to(torch.float32)
        assert torch.allclose(ones, deg[:, None].expand(n, N), rtol=1e-5, atol=1e-5)


def test_rejects_bad_arguments():
    rowptr = torch.zeros(5, dtype=torch.int64, device=DEV)
    col = torch.zeros(0, dtype=torch.int32, device=DEV)
    X = torch.zeros(4, 8, device=DEV)
    with pytest.raises(RuntimeError):
        ops.spmm(rowptr, col, None, X, torch.zeros(3, 8, device=DEV), 4)  # out has the wrong row count
    with pytest.raises(RuntimeError):
        ops.spmm(rowptr, col, None, X.double(), torch.zeros(4, 8, device=DEV), 4)  # dtype
    with pytest.raises(RuntimeError):
        ops.spmm(rowptr.cpu(), col, None, X, torch.zeros(4, 8, device=DEV), 4)  # CPU tensor
    torch.cuda.synchronize()


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("weighted", [True, False])
def test_row_and_column_scales(oracle, algo, weighted):
    """Y (+)= diag(r) A diag(c) X, the folded mean normalisation (forward: r = 1/deg, backward: c = 1/deg)."""
    M, K, N = 700, 450, 256
    rowptr, col, val = random_csr(M, K, 11, seed=21, heavy={3: 1500}, empty_every=9, weighted=weighted)
    rng = np.random.default_rng(5)
    X = rng.standard_normal((K, N)).astype(np.float32)
    r = (1.0 / rng.integers(1, 40, M)).astype(np.float32)
    c = (1.0 / rng.integers(1, 40, K)).astype(np.float32)
    Y0 = rng.standard_normal((M, N)).astype(np.float32)
    for use_r, use_c, acc in ((True, False, False), (False, True, False), (True, True, True)):
        Xs = X * c[:, None] if use_c else X
        part = oracle.spmm(rowptr, col, val, Xs, np.zeros((M, N), np.float32))
        mag = oracle.spmm(rowptr, col, None if val is None else np.abs(val), np.abs(Xs), np.zeros((M, N), np.float32))
        if use_r:
            part, mag = part * r[:, None], mag * r[:, None]
        want = part + (Y0 if acc else 0)
        mag = mag + (np.abs(Y0) if acc else 0)
        y = torch.from_numpy(Y0.copy()).to(DEV)
        ops.spmm(torch.from_numpy(rowptr).to(DEV), torch.from_numpy(col).to(DEV).to(torch.int32),
                 None if val is None else torch.from_numpy(val).to(DEV), torch.from_numpy(X).to(DEV), y, M, None, None,
                 algo=algo, accumulate=acc, row_scale=torch.from_numpy(r).to(DEV) if use_r else None,
                 col_scale=torch.from_numpy(c).to(DEV) if use_c else None)
        assert_close(y.cpu().numpy(), want, mag)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("N", [48, 24, 128])
@pytest.mark.parametrize("accumulate", [True, False])
def test_column_slices_of_a_wider_buffer(oracle, algo, N, accumulate):
    """Operand = left N columns, result = right N columns of ONE row-major [., 2N] buffer each (how the last layer
    aggregates its projected rows): the row stride is passed through, nothing outside the slice is touched."""
    M = K = 600
    rowptr, col, val = random_csr(M, K, 11, seed=N, heavy={3: 900}, empty_every=9)
    rng = np.random.default_rng(N)
    buf = rng.standard_normal((M, 2 * N)).astype(np.float32)
    X, Y0 = buf[:, :N].copy(), buf[:, N:].copy()
    base = Y0.copy() if accumulate else np.zeros_like(Y0)
    want = oracle.spmm(rowptr, col, val, X, base.copy())
    mag = oracle.spmm(rowptr, col, np.abs(val), np.abs(X), np.abs(base))
    t = torch.from_numpy(buf.copy()).to(DEV)
    ops.spmm(torch.from_numpy(rowptr).to(DEV), torch.from_numpy(col).to(DEV).to(torch.int32),
             torch.from_numpy(val).to(DEV), t[:, :N], t[:, N:], M, None, None, algo=algo, accumulate=accumulate)
    got = t.cpu().numpy()
    assert np.array_equal(got[:, :N], X)  # the operand half is untouched
    assert_close(got[:, N:], want, mag)


@pytest.mark.parametrize("algo", ALGOS)
@pytest.mark.parametrize("N", [48, 128, 256])
def test_row_ranges_of_a_larger_matrix(oracle, algo, N):
    """The product over ranges of rows (row pointers sliced, column / value arrays whole, first nonzero given):
    the ranges together reproduce the whole product; empty ranges and ranges that end in empty rows included."""
    M, K = 700, 400
    rowptr, col, val = random_csr(M, K, 9, seed=N, heavy={350: 3000}, empty_every=5)
    rng = np.random.default_rng(N)
    X = rng.standard_normal((K, N)).astype(np.float32)
    want = oracle.spmm(rowptr, col, val, X, np.zeros((M, N), np.float32))
    mag = oracle.spmm(rowptr, col, np.abs(val), np.abs(X), np.zeros((M, N), np.float32))
    rp, c, v, x = (torch.from_numpy(a).to(DEV) for a in (rowptr, col.astype(np.int32), val, X))
    cuts = [0, 1, 1, 200, 351, 355, 699, 700]
    got = torch.full((M, N), float("nan"), device=DEV)
    for a, b in zip(cuts[:-1], cuts[1:]):
        if b == a:
            continue
        begin, count = int(rowptr[a]), int(rowptr[b] - rowptr[a])
        ops.spmm(rp[a:b + 1], c, v, x, got[a:b], b - a, None, None, algo=algo, accumulate=False, nnz_range=(begin, count))
    assert_close(got.cpu().numpy(), want, mag)


def test_structural_check_counts_what_the_kernels_would_trust():
    rowptr = torch.tensor([0, 2, 5, 4, 7], dtype=torch.int64, device=DEV)      # row 2 ends before it starts
    col = torch.tensor([0, 9, 3, -1, 2, 1, 7], dtype=torch.int32, device=DEV)  # 9 and -1 outside [0, 8)
    rep = ops.check_csr(rowptr, col, 8)
    assert rep == dict(rows_ending_before_start=1, columns_out_of_range=2, rowptr_starts_at_zero=True,
                       rowptr_ends_at_nnz=True)
    good_rp, good_col, _ = random_csr(300, 50, 6, seed=1)
    rep = ops.check_csr(torch.from_numpy(good_rp).to(DEV), torch.from_numpy(good_col.astype(np.int32)).to(DEV), 50)
    assert rep == dict(rows_ending_before_start=0, columns_out_of_range=0, rowptr_starts_at_zero=True,
                       rowptr_ends_at_nnz=True)
    rep = ops.check_csr(torch.tensor([1, 3], dtype=torch.int64, device=DEV),
                        torch.tensor([0, 0, 0, 0], dtype=torch.int32, device=DEV), 4)
    assert not rep["rowptr_starts_at_zero"] and not rep["rowptr_ends_at_nnz"]
