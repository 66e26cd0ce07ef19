"""Pins of the CPU oracle (oracle/sgnn_oracle.c): against the golden vectors made
by the reference's own compiled ops, against the byte-exact vectors in the
reference's tests/test_quantizer.py, and — when oracle/_ref is present — against
the reference ops live on larger random inputs."""
import numpy as np
import pytest
import torch


def test_spmm_matches_reference_golden(golden, oracle):
    for N in (7, 16, 100):
        y = oracle.spmm(golden["spmm_rowptr"], golden["spmm_col"], golden["spmm_val"], golden[f"spmm_X_{N}"],
                        golden[f"spmm_Y0_{N}"].copy())
        assert np.array_equal(y, golden[f"spmm_Y_{N}"])  # same FMA order -> bit equal


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("tag", ["a", "b"])
def test_quantize_tensor_matches_reference_golden(golden, oracle, bits, tag):
    k = f"q{bits}{tag}"
    x, mn, sc = golden[k + "_x"], golden[k + "_min"], golden[k + "_scale"]
    q = oracle.quantize_tensor(x, mn, sc, bits)
    assert np.array_equal(q, golden[k + "_q"])
    d = oracle.dequantize_tensor(q, x.shape[0], mn, sc, bits)
    assert np.array_equal(d, golden[k + "_deq"])
    # the oracle's own per-row parameters are the min / scale the golden file was made with
    p = oracle.row_params(x, bits)
    assert np.array_equal(p[:, 0], mn) and np.array_equal(p[:, 1], sc)


@pytest.mark.parametrize("bits", [8, 4, 2])
def test_for_all_procs_equals_x86_per_segment(golden, oracle, bits):
    """The per-peer packing is the x86 single-segment packing applied to every peer's
    rows (what the reference's tests/test_quantization_ops.py:214-228 checks)."""
    rng = np.random.default_rng(5)
    S, F = 211, 37
    x = (rng.standard_normal((S, F)) * 3).astype(np.float32)
    wr = np.array([0, 0, 5, 5, 70, 71, 211], np.int32)  # empty peers and ragged groups
    q, params = oracle.quantize_for_all_procs(x, wr, bits)
    assert np.array_equal(params, oracle.row_params(x, bits))
    off = 0
    epb = 8 // bits
    for p in range(len(wr) - 1):
        seg = x[wr[p]:wr[p + 1]]
        g = -(-len(seg) // epb)
        if len(seg):
            qs = oracle.quantize_tensor(seg, params[wr[p]:wr[p + 1], 0], params[wr[p]:wr[p + 1], 1], bits)
            assert np.array_equal(qs, q[off:off + g])
        off += g
    assert off == q.shape[0] == oracle.packed_rows(wr, bits)
    d = oracle.dequantize_for_all_procs(q, params, wr, bits)
    assert np.max(np.abs(d - x) / params[:, 1:2]) <= 0.5 + 1e-3  # round to nearest


def test_v1_reference_known_answer(oracle):
    """Byte-exact vector of the reference's tests/test_quantizer.py:57-84 and its inverse :87-114."""
    x = np.array([[0.2, 0.1, 0.3], [0.4, 0.5, 0.6], [0.7, 0.8, 0.9], [1.0, 1.1, 1.2], [0.3, 0.1, 0.7]], np.float32)
    bits = [8, 4, 2, 4, 4]
    q, params, rng = oracle.quantize_v1(x, bits)
    assert rng.tolist() == [0, 3, 5, 6, 8, 10]
    assert q.tolist() == [127, 0, 255, 7, 240, 44, 8, 240, 80, 240]
    exp_scale = (x.max(1) - x.min(1)) / (2.0 ** np.array(bits, np.float32) - 1)
    assert np.allclose(params[:, 1], x.min(1)) and np.allclose(params[:, 2], exp_scale)
    deq_params = np.array([[8, 0.1, 7.8431e-04], [4, 0.4, 1.3333e-02], [2, 0.7, 6.6667e-02], [4, 1.0, 1.3333e-02],
                           [4, 0.1, 4.0000e-02]], np.float32)
    d = oracle.dequantize_v1(np.array([127, 0, 255, 7, 240, 44, 8, 240, 80, 240], np.uint8), deq_params, 3)
    # the reference asserts allclose at default tolerances, which lossy 2/4-bit codes cannot meet;
    # the bound that does hold is half a quantisation step per row
    assert np.all(np.abs(d - x) <= 0.5 * deq_params[:, 2:3] * (1 + 1e-3) + 1e-6)


def test_v1_v2_match_reference_golden(golden, oracle):
    q, params, rng = oracle.quantize_v1(golden["v1_x"], golden["v1_bits"])
    assert np.array_equal(rng, golden["v1_range"])
    assert np.array_equal(q, golden["v1_q"]) and np.array_equal(params, golden["v1_params"])
    assert np.array_equal(oracle.dequantize_v1(q, params, golden["v1_x"].shape[1]), golden["v1_deq"])
    for b in (8, 4, 2):
        x, zp, sc = golden[f"v2_{b}_x"], golden[f"v2_{b}_zp"], golden[f"v2_{b}_sc"]
        q2, _ = oracle.quantize_v2_torch(x, zp, sc, b)
        assert np.array_equal(q2, golden[f"v2_{b}_q"])
        assert np.array_equal(oracle.dequantize_v2_torch(q2, x.shape[0], x.shape[1], zp, sc, b), golden[f"v2_{b}_deq"])


def test_split_arithmetic_known_answers(oracle):
    """tests/test_quantizer.py:8-27 and :29-55 of the reference."""
    recv, send = oracle.splits_for_comm_quantized_data([2, 0, 4, 1], [0, 3, 0, 3], [0, 2, 4, 6, 8, 12, 13, 19],
                                                       [0, 1, 2, 5, 7, 11, 30])
    assert recv == [4, 0, 9, 6] and send == [0, 5, 0, 25]
    assert oracle.quantized_nodes_feat_range(4, [8, 4, 2, 8, 4, 2]).tolist() == [0, 4, 6, 7, 11, 13, 14]
    assert oracle.quantized_nodes_feat_range(1, [2, 2, 2]).tolist() == [0, 1, 2, 3]
    assert oracle.quantized_nodes_feat_range(3, [4, 4, 2]).tolist() == [0, 2, 4, 5]
    assert oracle.quantized_splits([5, 0, 8, 1], 2) == [2, 0, 2, 1]


def test_bf16_round_trip_matches_torch(oracle):
    a = (np.random.default_rng(0).standard_normal(4096) * 37).astype(np.float32)
    assert np.array_equal(oracle.round_bf16(a), torch.from_numpy(a).to(torch.bfloat16).float().numpy())


def test_oracle_equals_reference_live(ref_ops, oracle):
    """Larger random inputs, straight against the reference's compiled ops."""
    rng = np.random.default_rng(1)
    M, K, N = 3000, 2500, 128
    deg = rng.poisson(9, M)
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = rng.integers(0, K, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32)
    X = rng.standard_normal((K, N)).astype(np.float32)
    y = torch.zeros((M, N))
    T = torch.get_num_threads()
    splits = torch.from_numpy(oracle.distribute_work_for_row(rowptr, np.ones_like(val), T))
    ref_ops.spmm(torch.from_numpy(rowptr), torch.from_numpy(col), torch.from_numpy(val), torch.from_numpy(X), y, M,
                 splits, torch.tensor([0, N], dtype=torch.int32))
    assert np.array_equal(oracle.spmm(rowptr, col, val, X, np.zeros((M, N), np.float32)), y.numpy())
    for bits in (8, 4, 2):
        S, F = 4333, 123  # the shape of the reference's tests/test_quantization_ops.py
        x = rng.standard_normal((S, F)).astype(np.float32)
        p = oracle.row_params(x, bits)
        q = torch.zeros((-(-S // (8 // bits)), F), dtype=torch.uint8)
        ref_ops.quantize_tensor(torch.from_numpy(x), q, torch.from_numpy(p[:, 0].copy()), torch.from_numpy(p[:, 1].copy()), bits)
        assert np.array_equal(oracle.quantize_tensor(x, p[:, 0], p[:, 1], bits), q.numpy())
