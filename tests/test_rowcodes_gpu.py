"""The row-codes layout of quantised boundary rows (every row in its own F*bits/8 bytes) against the CPU
oracle: the codes are the reference's — undoing the layout permutation gives the oracle's row-group bytes
exactly — and the consumers (unpack-dequantise, fused dequantise-SpMM) give the oracle's values.  Also the
one-sided (peer-store) forms of both quantisers, run on ONE device with peer tables that point at local
buffers laid out as the peers' receive buffers would be."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops
from super_gnn_b200 import synthetic

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


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("S,F", [(1, 4), (5, 16), (3, 100), (1000, 128), (4333, 256), (513, 512), (777, 48), (64, 124)])
def test_row_codes_are_the_reference_codes_permuted(oracle, bits, S, F):
    x = rand_rows(S, F, seed=S + F + bits)
    wr = random_work_range(S, 5, seed=S + bits)
    want_q, want_p = oracle.quantize_for_all_procs(x, wr, bits)
    codes = torch.full((S, F * bits // 8), 0xAB, dtype=torch.uint8, device=DEV)
    params = torch.zeros((S, 2), device=DEV)
    p16 = torch.zeros((S, 2), dtype=torch.bfloat16, device=DEV)
    ops.quant_pack_rowcodes(torch.from_numpy(x).to(DEV), None, bits, codes, params=params, params_bf16=p16)
    assert np.array_equal(params.cpu().numpy(), want_p)
    assert np.array_equal(p16.float().cpu().numpy(), oracle.round_bf16(want_p))
    got_codes = oracle.codes_of_row_codes(codes.cpu().numpy(), F, bits)
    assert np.array_equal(oracle.row_groups_of(got_codes, wr, bits), want_q)  # the oracle's wire bytes, exactly
    assert np.array_equal(codes.cpu().numpy(), oracle.row_codes_of(oracle.codes_of_row_groups(want_q, wr, bits), bits))
    # unpack + dequantise, fp32 and bf16 parameters: bit-exact with the reference's dequantiser
    out = torch.empty((S, F), device=DEV)
    ops.unpack_dequant_rowcodes(codes, out, params, bits)
    assert np.array_equal(out.cpu().numpy(), oracle.dequantize_for_all_procs(want_q, want_p, wr, bits))
    ops.unpack_dequant_rowcodes(codes, out, p16, bits)
    assert np.array_equal(out.cpu().numpy(),
                          oracle.dequantize_for_all_procs(want_q, oracle.round_bf16(want_p), wr, bits))


@pytest.mark.parametrize("bits", [8, 4, 2])
def test_gather_quantise_and_dequantise_scatter_add(oracle, bits):
    n, F, S = 500, 256, 1203
    rng = np.random.default_rng(bits)
    feats = rand_rows(n, F, seed=11)
    idx = rng.integers(0, n, S).astype(np.int64)
    wr = np.array([0, S], np.int32)
    want_q, want_p = oracle.quantize_for_all_procs(feats[idx], wr, bits)
    codes = torch.zeros((S, F * bits // 8), dtype=torch.uint8, device=DEV)
    p16 = torch.zeros((S, 2), dtype=torch.bfloat16, device=DEV)
    ops.quant_pack_rowcodes(torch.from_numpy(feats).to(DEV), torch.from_numpy(idx).to(DEV), bits, codes, params_bf16=p16)
    assert np.array_equal(oracle.row_groups_of(oracle.codes_of_row_codes(codes.cpu().numpy(), F, bits), wr, bits), want_q)
    base = rng.standard_normal((n, F)).astype(np.float32)
    acc = torch.from_numpy(base.copy()).to(DEV)
    ops.unpack_dequant_rowcodes(codes, acc, p16, bits, row_index=torch.from_numpy(idx).to(DEV))
    rows = oracle.dequantize_for_all_procs(want_q, oracle.round_bf16(want_p), wr, bits)
    want = base.astype(np.float64)
    mag = np.abs(base).astype(np.float64)
    np.add.at(want, idx, rows.astype(np.float64))
    np.add.at(mag, idx, np.abs(rows).astype(np.float64))
    assert np.all(np.abs(acc.cpu().numpy() - want) <= 1e-5 * mag + 1e-30)


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("F", [32, 48, 100, 128, 256, 512])
@pytest.mark.parametrize("algo", [ops.SPMM_ROW_SPLIT, ops.SPMM_NNZ_SPLIT])
def test_spmm_on_row_codes_equals_dequantise_then_spmm(oracle, bits, F, algo):
    M, R = 3000, 4099
    x = rand_rows(R, F, seed=F + bits)
    wr = np.array([0, R], np.int32)
    q, p = oracle.quantize_for_all_procs(x, wr, bits)
    xhat = oracle.dequantize_for_all_procs(q, oracle.round_bf16(p), wr, bits)
    rp, c, v = synthetic.poisson_csr(M, R, 6.0, seed=2)
    rp[-1] = rp[-1]  # (kept: rows of very different lengths come from the Poisson draw)
    codes = torch.from_numpy(oracle.row_codes_of(oracle.codes_of_row_groups(q, wr, bits), bits)).to(DEV)
    p16 = torch.from_numpy(p).to(DEV).to(torch.bfloat16)
    scale = torch.rand(M, generator=torch.Generator().manual_seed(3)) + 0.5
    for value, row_scale in ((v, None), (None, None), (None, scale)):
        base = np.random.default_rng(5).standard_normal((M, F)).astype(np.float32)
        y = torch.from_numpy(base.copy()).to(DEV)
        ops.spmm_dequant_rowcodes(rp.to(DEV), c.to(DEV), None if value is None else value.to(DEV), codes, p16, bits, y, M,
                                  algo=algo, row_scale=None if row_scale is None else row_scale.to(DEV))
        vv = None if value is None else value.numpy()
        prod = oracle.spmm(rp.numpy(), c.numpy().astype(np.int64), vv, xhat, np.zeros((M, F), np.float32))
        mag = oracle.spmm(rp.numpy(), c.numpy().astype(np.int64), None if vv is None else np.abs(vv), np.abs(xhat),
                          np.zeros((M, F), np.float32))
        if row_scale is not None:
            prod, mag = prod * row_scale.numpy()[:, None], mag * row_scale.numpy()[:, None]
        want = base + prod
        assert np.all(np.abs(y.cpu().numpy() - want) <= 1e-5 * (mag + np.abs(base) + np.abs(want)) + 1e-30)


def test_spmm_on_row_codes_with_a_hub_row_and_empty_rows(oracle):
    bits, F, R = 2, 256, 5000
    x = rand_rows(R, F, seed=1)
    wr = np.array([0, R], np.int32)
    q, p = oracle.quantize_for_all_procs(x, wr, bits)
    xhat = oracle.dequantize_for_all_procs(q, oracle.round_bf16(p), wr, bits)
    rng = np.random.default_rng(0)
    deg = rng.poisson(3, 400)
    deg[::7] = 0
    deg[13] = 9000  # one row far longer than a warp's chunk of nonzeros
    rp = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    c = rng.integers(0, R, rp[-1]).astype(np.int32)
    codes = torch.from_numpy(oracle.row_codes_of(oracle.codes_of_row_groups(q, wr, bits), bits)).to(DEV)
    p16 = torch.from_numpy(p).to(DEV).to(torch.bfloat16)
    y = torch.zeros((400, F), device=DEV)
    ops.spmm_dequant_rowcodes(torch.from_numpy(rp).to(DEV), torch.from_numpy(c).to(DEV), None, codes, p16, bits, y, 400)
    want = oracle.spmm(rp, c.astype(np.int64), None, xhat, np.zeros((400, F), np.float32))
    mag = oracle.spmm(rp, c.astype(np.int64), None, np.abs(xhat), np.zeros((400, F), np.float32))
    assert np.all(np.abs(y.cpu().numpy() - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30)


def _peer_buffers(P, me, seg_rows, others_before, bytes_per_row, extra_rows=3):
    """Receive buffers of P peers as local tensors: peer p's buffer holds the segments of the ranks before `me`
    (others_before[p] rows), then ours (seg_rows[p] rows), then a few rows that must stay untouched."""
    bufs, row0 = [], []
    for p in range(P):
        rows = others_before[p] + seg_rows[p] + extra_rows
        bufs.append(torch.full((rows, bytes_per_row), 0xCD, dtype=torch.uint8, device=DEV))
        row0.append(others_before[p])
    return bufs, row0


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("F", [128, 256])
def test_one_sided_quantisers_store_the_oracle_bytes_into_each_peers_buffer(oracle, bits, F):
    """Both peer-store kernels on one device: the tables point at local tensors, one per destination peer."""
    P, S = 6, 1499
    epb = 8 // bits
    x = rand_rows(S, F, seed=bits + F)
    wr = random_work_range(S, P, seed=3)
    want_q, want_p = oracle.quantize_for_all_procs(x, wr, bits)
    want_p16 = oracle.round_bf16(want_p)
    n = [int(wr[p + 1] - wr[p]) for p in range(P)]
    before_rows = [7 * p + 1 for p in range(P)]          # rows other senders own in front of our segment
    table = lambda vals: torch.tensor(vals, dtype=torch.int64, device=DEV)  # noqa: E731
    xt, wrt = torch.from_numpy(x).to(DEV), torch.from_numpy(wr).to(DEV)

    # --- the reference's row-group bytes
    before_groups = [3 * p + 2 for p in range(P)]
    qbufs, qrow0 = _peer_buffers(P, 0, [-(-c // epb) for c in n], before_groups, F)
    pbufs, prow0 = _peer_buffers(P, 0, n, before_rows, 4)
    ops.quant_pack_rows_p2p(xt, None, wrt, P, bits, (table([b.data_ptr() for b in qbufs]), table(qrow0),
                                                     table([b.data_ptr() for b in pbufs]), table(prow0)))
    torch.cuda.synchronize()
    off = 0
    for p in range(P):
        g = -(-n[p] // epb)
        got = qbufs[p].cpu().numpy()
        assert np.array_equal(got[qrow0[p]:qrow0[p] + g], want_q[off:off + g]), f"packed rows for peer {p}"
        assert np.all(got[:qrow0[p]] == 0xCD) and np.all(got[qrow0[p] + g:] == 0xCD), "bytes outside the segment"
        gp = pbufs[p].cpu().view(torch.bfloat16).float().numpy()
        assert np.array_equal(gp[prow0[p]:prow0[p] + n[p]], want_p16[wr[p]:wr[p + 1]]), f"params for peer {p}"
        off += g

    # --- row codes
    pitch = F * bits // 8
    cbufs, crow0 = _peer_buffers(P, 0, n, before_rows, pitch)
    pbufs, prow0 = _peer_buffers(P, 0, n, before_rows, 4)
    p32 = torch.zeros((S, 2), device=DEV)
    idx = torch.arange(S, device=DEV)
    ops.quant_pack_rowcodes_p2p(xt, idx, wrt, P, bits, (table([b.data_ptr() for b in cbufs]),
                                                        table([b.data_ptr() for b in pbufs]), table(crow0)), params=p32)
    torch.cuda.synchronize()
    assert np.array_equal(p32.cpu().numpy(), want_p)
    want_codes = oracle.row_codes_of(oracle.codes_of_row_groups(want_q, wr, bits), bits)
    for p in range(P):
        got = cbufs[p].cpu().numpy()
        assert np.array_equal(got[crow0[p]:crow0[p] + n[p]], want_codes[wr[p]:wr[p + 1]]), f"row codes for peer {p}"
        assert np.all(got[:crow0[p]] == 0xCD) and np.all(got[crow0[p] + n[p]:] == 0xCD), "bytes outside the segment"
        gp = pbufs[p].cpu().view(torch.bfloat16).float().numpy()
        assert np.array_equal(gp[prow0[p]:prow0[p] + n[p]], want_p16[wr[p]:wr[p + 1]]), f"params for peer {p}"


def test_unsupported_widths_are_refused():
    x = torch.zeros((8, 192), device=DEV)
    with pytest.raises(RuntimeError):
        ops.quant_pack_rowcodes(x, None, 2, torch.zeros((8, 48), dtype=torch.uint8, device=DEV))
    assert ops.rowcodes_supported(100) and ops.rowcodes_supported(256) and not ops.rowcodes_supported(192)
    assert not ops.rowcodes_supported(102)
