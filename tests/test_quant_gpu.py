"""CUDA quantize-pack / unpack-dequantize vs the CPU oracle: packed bytes and
parameters bit-exact, dequantised values bit-exact (same fused multiply-add)."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops
from super_gnn_b200 import synthetic
from super_gnn_b200.quantizer import QuantizerForMixedBits, Quantizer_for_all_procs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rand_rows(S, F, seed):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((S, F)) * np.exp(rng.standard_normal((S, 1)))).astype(np.float32)
    if S > 3:
        x[2] = 1.5      # constant row -> scale 1
        x[3, :] = 0.0
    return x


def random_work_range(S, P, seed):
    rng = np.random.default_rng(seed)
    cuts = np.sort(rng.integers(0, S + 1, P - 1))
    wr = np.concatenate([[0], cuts, [S]]).astype(np.int32)
    if P > 3:
        wr[2] = wr[1]  # an empty peer
    return wr


def gpu_quantize(x, wr, bits, with_bf16=True, row_index=None, src=None):
    S, F = x.shape
    P = len(wr) - 1
    epb = 8 // bits
    rows = int(sum(-(-(int(wr[p + 1]) - int(wr[p])) // epb) for p in range(P)))
    packed = torch.full((rows, F), 0xAB, dtype=torch.uint8, device=DEV)
    params = torch.zeros((S, 2), device=DEV)
    p16 = torch.zeros((S, 2), dtype=torch.bfloat16, device=DEV) if with_bf16 else None
    wr_t = torch.from_numpy(wr).to(DEV)
    if row_index is None:
        ops.quant_pack_rows(torch.from_numpy(x).to(DEV), None, wr_t, P, bits, packed, params=params, params_bf16=p16)
    else:
        ops.quant_pack_rows(src, row_index, wr_t, P, bits, packed, params=params, params_bf16=p16)
    return packed, params, p16


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("S,F,P", [(1, 4, 1), (3, 16, 2), (5, 100, 3), (1000, 128, 8), (4333, 123, 16),
                                     (777, 256, 5), (513, 512, 4), (129, 516, 3), (64, 1, 2), (1001, 47, 7)])
def test_pack_and_params_bit_exact(oracle, bits, S, F, P):
    x = rand_rows(S, F, seed=S + F + bits)
    wr = random_work_range(S, P, seed=S + bits)
    want_q, want_p = oracle.quantize_for_all_procs(x, wr, bits)
    packed, params, p16 = gpu_quantize(x, wr, bits)
    assert np.array_equal(params.cpu().numpy(), want_p)
    assert np.array_equal(packed.cpu().numpy(), want_q)
    assert np.array_equal(p16.float().cpu().numpy(), oracle.round_bf16(want_p))
    # reference class front end
    Quantizer_for_all_procs(P, bits)
    q2 = torch.zeros_like(packed)
    p2 = torch.zeros_like(params)
    Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(torch.from_numpy(x).to(DEV), q2, p2, torch.from_numpy(wr))
    assert torch.equal(q2, packed) and torch.equal(p2, params)
    # unpack + dequantise (fp32 params and bf16 params)
    out = torch.empty((S, F), device=DEV)
    Quantizer_for_all_procs.ctx.dequantize_intX_to_fp32(packed, out, params, torch.from_numpy(wr).to(DEV))
    assert np.array_equal(out.cpu().numpy(), oracle.dequantize_for_all_procs(want_q, want_p, wr, bits))
    out16 = torch.empty((S, F), device=DEV)
    ops.dequantize_tensor_for_all_procs(packed, out16, p16, torch.from_numpy(wr).to(DEV), P, bits)
    assert np.array_equal(out16.cpu().numpy(),
                          oracle.dequantize_for_all_procs(want_q, oracle.round_bf16(want_p), wr, bits))


@pytest.mark.parametrize("bits", [8, 4, 2])
def test_fused_gather_quantise_and_dequantise_scatter_add(oracle, bits):
    n, F, S, P = 500, 256, 1203, 6
    rng = np.random.default_rng(bits)
    feats = rand_rows(n, F, seed=11)
    idx = rng.integers(0, n, S).astype(np.int64)  # repeated nodes, as when a node goes to several peers
    wr = random_work_range(S, P, seed=3)
    want_q, want_p = oracle.quantize_for_all_procs(feats[idx], wr, bits)
    packed, params, _ = gpu_quantize(feats[idx], wr, bits, row_index=torch.from_numpy(idx).to(DEV),
                                     src=torch.from_numpy(feats).to(DEV))
    assert np.array_equal(packed.cpu().numpy(), want_q) and np.array_equal(params.cpu().numpy(), want_p)
    # gather alone
    gathered = torch.empty((S, F), device=DEV)
    ops.gather_rows(torch.from_numpy(feats).to(DEV), torch.from_numpy(idx).to(DEV), gathered)
    assert np.array_equal(gathered.cpu().numpy(), feats[idx])
    # dequantise + scatter-add == index_add_ of the dequantised rows (order of additions differs)
    deq = oracle.dequantize_for_all_procs(want_q, want_p, wr, bits)
    base = rng.standard_normal((n, F)).astype(np.float32)
    want = base.astype(np.float64)
    np.add.at(want, idx, deq.astype(np.float64))
    mag = np.abs(base).astype(np.float64)
    np.add.at(mag, idx, np.abs(deq).astype(np.float64))
    acc = torch.from_numpy(base.copy()).to(DEV)
    ops.dequantize_tensor_for_all_procs(packed, acc, params, torch.from_numpy(wr).to(DEV), P, bits,
                                        row_index=torch.from_numpy(idx).to(DEV))
    assert np.all(np.abs(acc.cpu().numpy() - want) <= 1e-5 * mag + 1e-30)
    acc2 = torch.from_numpy(base.copy()).to(DEV)
    ops.scatter_add_rows(torch.from_numpy(deq).to(DEV), torch.from_numpy(idx).to(DEV), acc2)
    assert np.all(np.abs(acc2.cpu().numpy() - want) <= 1e-5 * mag + 1e-30)


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_x86_form_matches_reference_golden(golden, bits, tag):
    k = f"q{bits}{tag}"
    x, mn, sc = (torch.from_numpy(golden[k + s]).to(DEV) for s in ("_x", "_min", "_scale"))
    q = torch.zeros(golden[k + "_q"].shape, dtype=torch.uint8, device=DEV)
    ops.quantize_tensor(x, q, mn, sc, bits)
    assert np.array_equal(q.cpu().numpy(), golden[k + "_q"])
    d = torch.zeros_like(x)
    ops.dequantize_tensor(q, d, mn, sc, bits)
    assert np.array_equal(d.cpu().numpy(), golden[k + "_deq"])
    # SVE 4-argument form: parameters computed, one segment
    q4 = torch.zeros_like(q)
    p4 = torch.zeros((x.shape[0], 2), device=DEV)
    ops.quantize_tensor(x, q4, p4, bits)
    assert torch.equal(q4, q) and torch.equal(p4[:, 0], mn) and torch.equal(p4[:, 1], sc)


def test_v1_reference_known_answer_and_golden(golden):
    """tests/test_quantizer.py:57-114 of the reference, on the GPU."""
    x = torch.tensor([[0.2, 0.1, 0.3], [0.4, 0.5, 0.6], [0.7, 0.8, 0.9], [1.0, 1.1, 1.2], [0.3, 0.1, 0.7]], device=DEV)
    bits = torch.tensor([8, 4, 2, 4, 4], device=DEV)
    params = torch.empty((5, 3), device=DEV)
    params[:, 0] = bits
    rng = QuantizerForMixedBits.get_quantized_nodes_feat_range(5, 3, bits)
    assert rng.tolist() == [0, 3, 5, 6, 8, 10]
    q = torch.empty(int(rng[-1]), dtype=torch.uint8, device=DEV)
    QuantizerForMixedBits.quantize_fp32_to_intX(x, q, rng, params)
    assert q.tolist() == [127, 0, 255, 7, 240, 44, 8, 240, 80, 240]
    assert torch.allclose(params[:, 1], x.min(1)[0])
    assert torch.allclose(params[:, 2], (x.max(1)[0] - x.min(1)[0]) / (2 ** bits.float() - 1))
    d = torch.empty_like(x)
    QuantizerForMixedBits.dequantize_intX_to_fp32(q, d, rng, params)
    assert torch.all((d - x).abs() <= 0.5 * params[:, 2:3] * (1 + 1e-3) + 1e-6)
    # golden made by the reference ops
    gx = torch.from_numpy(golden["v1_x"]).to(DEV)
    gp = torch.zeros((gx.shape[0], 3), device=DEV)
    gp[:, 0] = torch.from_numpy(golden["v1_bits"]).to(DEV)
    gr = torch.from_numpy(golden["v1_range"]).to(DEV)
    gq = torch.zeros(int(gr[-1]), dtype=torch.uint8, device=DEV)
    ops.quantize_tensor_v1(gx, gq, gr, gp)
    assert np.array_equal(gq.cpu().numpy(), golden["v1_q"]) and np.array_equal(gp.cpu().numpy(), golden["v1_params"])
    gd = torch.zeros_like(gx)
    ops.dequantize_tensor_v1(gq, gd, gr, gp)
    assert np.array_equal(gd.cpu().numpy(), golden["v1_deq"])


@pytest.mark.parametrize("bits", [8, 4, 2])
def test_config2_full_size_round_trip(oracle, bits):
    """500k x 256, N(0,1) x LogNormal(0,1) row scale, seed 1: round-trip error <= half a step for every
    element (size-independent property), and the first 20k rows bit-exact against the oracle."""
    S, F = 500_000, 256
    x = synthetic.scaled_features(S, F, seed=1, device=DEV)
    wr = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    epb = 8 // bits
    packed = torch.empty((S // epb, F), dtype=torch.uint8, device=DEV)
    params = torch.empty((S, 2), device=DEV)
    ops.quantize_tensor_for_all_procs(x, packed, params, wr, 1, bits)
    out = torch.empty_like(x)
    ops.dequantize_tensor_for_all_procs(packed, out, params, wr, 1, bits)
    err = ((out - x).abs() / params[:, 1:2]).max().item()
    assert err <= 0.5 + 1e-3
    assert torch.equal(params[:, 0], x.min(1)[0])
    head = 20_000
    want_q, want_p = oracle.quantize_for_all_procs(x[:head].cpu().numpy(), np.array([0, head], np.int32), bits)
    assert np.array_equal(packed[: head // epb].cpu().numpy(), want_q)
    assert np.array_equal(params[:head].cpu().numpy(), want_p)


def test_rejects_bad_arguments():
    x = torch.zeros((8, 16), device=DEV)
    wr = torch.tensor([0, 8], dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):
        ops.quantize_tensor_for_all_procs(x, torch.zeros((8, 16), dtype=torch.uint8, device=DEV),
                                          torch.zeros((8, 2), device=DEV), wr, 1, 3)  # 8 % bits != 0
    with pytest.raises(RuntimeError):
        ops.quantize_tensor_for_all_procs(x, torch.zeros((1, 16), dtype=torch.uint8, device=DEV),
                                          torch.zeros((8, 2), device=DEV), wr, 1, 8)  # output too small
    with pytest.raises(RuntimeError):
        ops.quantize_tensor_for_all_procs(x.cpu(), torch.zeros((8, 16), dtype=torch.uint8, device=DEV),
                                          torch.zeros((8, 2), device=DEV), wr, 1, 8)  # CPU input
    torch.cuda.synchronize()


def test_v2_torch_layout_matches_reference_golden_and_oracle(golden, oracle):
    """quantize_tensor_v2_torch / dequantize_tensor_v2_torch: the reference's own outputs (golden vectors made by
    its compiled x86 ops) and the oracle on a larger ragged case, byte for byte."""
    for b in (8, 4, 2):
        x, zp, sc = golden[f"v2_{b}_x"], golden[f"v2_{b}_zp"], golden[f"v2_{b}_sc"]
        S, F = x.shape
        rng = oracle.quantized_nodes_feat_range(F, np.full(S, b))
        q = torch.zeros(int(rng[-1]), dtype=torch.uint8, device=DEV)
        args = (torch.from_numpy(rng).to(DEV), torch.from_numpy(zp).to(DEV), torch.from_numpy(sc).to(DEV), b)
        ops.quantize_tensor_v2_torch(torch.from_numpy(x).to(DEV), q, *args)
        assert np.array_equal(q.cpu().numpy(), golden[f"v2_{b}_q"])
        d = torch.zeros((S, F), device=DEV)
        ops.dequantize_tensor_v2_torch(q, d, *args)
        assert np.array_equal(d.cpu().numpy(), golden[f"v2_{b}_deq"])
    rng_ = np.random.default_rng(5)
    for b, (S, F) in ((8, (333, 101)), (4, (70, 47)), (2, (129, 258))):
        x = rng_.standard_normal((S, F)).astype(np.float32)
        sc = ((x.max(1) - x.min(1)) / (2 ** b - 1)).astype(np.float32)
        zp = np.round(-x.min(1) / sc).astype(np.float32)
        want_q, rng = oracle.quantize_v2_torch(x, zp, sc, b)
        q = torch.zeros(int(rng[-1]), dtype=torch.uint8, device=DEV)
        args = (torch.from_numpy(rng).to(DEV), torch.from_numpy(zp).to(DEV), torch.from_numpy(sc).to(DEV), b)
        ops.quantize_tensor_v2_torch(torch.from_numpy(x).to(DEV), q, *args)
        assert np.array_equal(q.cpu().numpy(), want_q)
        d = torch.zeros((S, F), device=DEV)
        ops.dequantize_tensor_v2_torch(q, d, *args)
        assert np.array_equal(d.cpu().numpy(), oracle.dequantize_v2_torch(want_q, S, F, zp, sc, b))
