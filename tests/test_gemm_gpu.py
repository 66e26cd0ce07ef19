"""Dense fp32 GEMM (tensor cores, operands split into three bf16 terms, nine or the six leading cross
products) against an fp64 product of the same operands.

The contract is fp32 accuracy: the error relative to the largest entry of the exact result must stay
at the level of a plain fp32 GEMM (a few 1e-7 for K in the hundreds), far below what a single-pass
TF32 or bf16 product gives (1e-3 .. 1e-2).  The stock fp32 matmul of PyTorch is measured beside it."""
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_err(c, ref64):
    return ((c.double() - ref64).abs().max() / ref64.abs().max()).item()


def strided(rows, cols, ld, gen, scale=1.0):
    """[rows, cols] view with leading dimension ld >= cols; the padding holds NaN so that a kernel which
    reads it shows up in the result."""
    buf = torch.full((rows, ld), float("nan"), device=DEV)
    buf[:, :cols] = torch.randn(rows, cols, generator=gen, device=DEV) * scale
    return buf[:, :cols]


@pytest.mark.parametrize("M,N,K", [(4096, 256, 256), (4099, 256, 100), (1, 128, 256), (777, 48, 256), (5000, 256, 48),
                                   (130, 4, 4), (20000, 100, 256), (3000, 512, 1000)])
@pytest.mark.parametrize("products", [9, 6])
def test_gemm_nt_matches_fp64(M, N, K, products, monkeypatch):
    monkeypatch.setattr(ops, "GEMM_PRODUCTS", products)
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device=DEV).manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g, device=DEV)
    b = torch.randn(N, K, generator=g, device=DEV) * 0.1
    ref = a.double() @ b.double().t()
    c = ops.gemm_nt(a, b)
    e9, e32 = rel_err(c, ref), rel_err(a @ b.t(), ref)
    assert e9 <= 1e-6 and e9 <= 2 * e32 + 1e-7, (e9, e32)
    # beta: accumulate into an existing matrix
    c0 = torch.randn(M, N, generator=g, device=DEV)
    c1 = c0.clone()
    ops.gemm_nt(a, b, out=c1, beta=1.0)
    assert rel_err(c1, ref + c0.double()) <= 1e-6
    ops.gemm_nt(a, b, out=c1, beta=-0.5)
    assert rel_err(c1, ref - 0.5 * (ref + c0.double())) <= 2e-6


def test_gemm_nt_leading_dimensions():
    g = torch.Generator(device=DEV).manual_seed(7)
    M, N, K = 1500, 64, 100
    a, b = strided(M, K, 128, g), strided(N, K, 104, g, 0.1)
    out = torch.full((M, 72), float("nan"), device=DEV)
    c = ops.gemm_nt(a, b, out=out[:, :N])
    ref = a.double() @ b.double().t()
    assert rel_err(c, ref) <= 1e-6
    assert torch.isnan(out[:, N:]).all()  # nothing written beyond the N columns


@pytest.mark.parametrize("M,N,K", [(256, 256, 4096), (256, 100, 5001), (48, 256, 3000), (256, 48, 3000), (4, 4, 1),
                                   (100, 100, 70000), (512, 256, 9999)])
@pytest.mark.parametrize("products", [9, 6])
def test_gemm_tn_matches_fp64(M, N, K, products, monkeypatch):
    monkeypatch.setattr(ops, "GEMM_PRODUCTS", products)
    torch.backends.cuda.matmul.allow_tf32 = False
    g = torch.Generator(device=DEV).manual_seed(M * 3 + N + K)
    a = torch.randn(K, M, generator=g, device=DEV)
    b = torch.randn(K, N, generator=g, device=DEV)
    ref = a.double().t() @ b.double()
    c = ops.gemm_tn(a, b)
    e9, e32 = rel_err(c, ref), rel_err(a.t() @ b, ref)
    assert e9 <= 2e-6 and e9 <= 2 * e32 + 1e-7, (e9, e32)
    # the split along K is combined in a fixed order: a second run is bit-identical
    assert torch.equal(c, ops.gemm_tn(a, b))
    c0 = torch.randn(M, N, generator=g, device=DEV)
    c1 = c0.clone()
    ops.gemm_tn(a, b, out=c1, beta=1.0)
    assert rel_err(c1, ref + c0.double()) <= 2e-6


def test_gemm_tn_leading_dimensions_and_large_k():
    g = torch.Generator(device=DEV).manual_seed(11)
    K, M, N = 300000, 256, 100
    a, b = strided(K, M, 260, g), strided(K, N, 128, g)
    ref = torch.zeros(M, N, dtype=torch.float64, device=DEV)
    for i in range(0, K, 1 << 16):
        ref += a[i:i + (1 << 16)].double().t() @ b[i:i + (1 << 16)].double()
    assert rel_err(ops.gemm_tn(a, b), ref) <= 5e-6


def test_gemm_rejects_what_the_kernel_does_not_cover():
    a = torch.randn(64, 256, device=DEV)
    with pytest.raises(RuntimeError):  # 47 columns: rows of the result would not start on 16-byte boundaries
        ops.gemm_nt(a, torch.randn(47, 256, device=DEV))
    with pytest.raises(RuntimeError):  # K mismatch
        ops.gemm_nt(a, torch.randn(64, 128, device=DEV))
    with pytest.raises(RuntimeError):  # K = 102 is not a multiple of 4
        ops.gemm_nt(torch.randn(64, 102, device=DEV), torch.randn(64, 102, device=DEV))
    with pytest.raises(RuntimeError):  # operand on the host
        ops.gemm_nt(a.cpu(), torch.randn(64, 256))
    with pytest.raises(RuntimeError):  # transposed view: rows not contiguous
        ops.gemm_nt(a, torch.randn(256, 64, device=DEV).t())
    # empty problems are no-ops
    assert ops.gemm_nt(torch.empty(0, 256, device=DEV), torch.randn(64, 256, device=DEV)).shape == (0, 64)
    assert torch.equal(ops.gemm_tn(torch.empty(0, 8, device=DEV), torch.empty(0, 4, device=DEV)), torch.zeros(8, 4, device=DEV))
