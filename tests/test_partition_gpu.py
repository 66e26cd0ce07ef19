"""Partitioned aggregation on ONE device: the ranks of a W-way partition are run one
after another in this process and the boundary exchange is done by slicing the
ranks' send buffers (what all_to_all_single delivers), so the kernels, the wire
format and the partition bookkeeping are checked together against the
single-graph A x — fp32 exactly the same sum, 2/4/8-bit against the oracle's
quantise -> bf16 params -> dequantise pipeline."""
import numpy as np
import pytest
import torch

from super_gnn_b200 import supergnn_ops as ops
from super_gnn_b200 import synthetic
from super_gnn_b200.sparse import SparseTensor

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build_parts(src, dst, n, W):
    """Per-rank local/remote CSR + send index, by the same vectorised steps as
    data_manager.graph_builder (which needs a process group for W > 1)."""
    begins = synthetic.even_ranges(n, W)
    parts = []
    for r in range(W):
        lo, hi = begins[r], begins[r + 1]
        mine = (dst >= lo) & (dst < hi)
        s, d = src[mine], dst[mine] - lo
        loc = (s >= lo) & (s < hi)
        remote_nodes, inv = torch.unique(s[~loc], sorted=True, return_inverse=True)
        bounds = torch.searchsorted(remote_nodes, torch.tensor(begins))
        parts.append(dict(n=hi - lo, lo=lo,
                          local=SparseTensor(row=d[loc], col=s[loc] - lo, sparse_sizes=(hi - lo, hi - lo)).to(DEV),
                          remote=SparseTensor(row=d[~loc], col=inv, sparse_sizes=(hi - lo, remote_nodes.numel())).to(DEV),
                          remote_nodes=remote_nodes, recv_splits=(bounds[1:] - bounds[:-1]).tolist()))
    for r in range(W):
        # rows rank r must send to every peer p = the nodes p wants from r's range
        want = [parts[p]["remote_nodes"][sum(parts[p]["recv_splits"][:r]):sum(parts[p]["recv_splits"][:r + 1])] - begins[r]
                for p in range(W)]
        parts[r]["send_idx"] = torch.cat(want).to(DEV)
        parts[r]["send_splits"] = [w.numel() for w in want]
    return begins, parts


@pytest.mark.parametrize("W,family", [(2, "rmat"), (4, "rmat"), (8, "sbm")])
@pytest.mark.parametrize("bits", [32, 8, 4, 2])
def test_partitioned_aggregation_equals_single_graph(oracle, W, family, bits):
    n, F, E = 4000, 128, 60000
    if family == "rmat":   # power-law graph, random relabel, contiguous ranges (the scaling-sweep configuration)
        s, t = synthetic.rmat_edges(n, E, 0.57, 0.19, 0.19, 0.05, seed=4)
        s, t = synthetic.symmetrize_dedup(s, t, n)
        s, t = synthetic.random_relabel(s, t, n, seed=4)
    else:                  # stochastic block model, 90 % intra-block edges, block b = rank b (the 8-GPU configuration)
        s, t = synthetic.sbm_edges(W, n // W, E, 0.9, seed=3)
        s, t = synthetic.symmetrize_dedup(s, t, n)
    x = torch.randn(n, F, generator=torch.Generator().manual_seed(1))
    begins, parts = build_parts(s, t, n, W)
    A = SparseTensor(row=t, col=s, sparse_sizes=(n, n))
    rowptr, col, _ = A.csr()

    # what every rank sends (fp32 rows or wire format)
    sent = []
    for r, p in enumerate(parts):
        xr = x[begins[r]:begins[r + 1]].to(DEV)
        p["x"] = xr
        if bits == 32:
            buf = torch.empty((p["send_idx"].numel(), F), device=DEV)
            ops.gather_rows(xr, p["send_idx"], buf)
            sent.append(buf)
        else:
            wr = torch.tensor([0] + list(np.cumsum(p["send_splits"])), dtype=torch.int32, device=DEV)
            epb = 8 // bits
            rows = sum(-(-c // epb) for c in p["send_splits"])
            q = torch.zeros((rows, F), dtype=torch.uint8, device=DEV)
            p16 = torch.zeros((p["send_idx"].numel(), 2), dtype=torch.bfloat16, device=DEV)
            ops.quant_pack_rows(xr, p["send_idx"], wr, W, bits, q, params_bf16=p16)
            sent.append((q, p16))

    xhat = x.numpy().copy()  # what the receivers reconstruct for a remote row (per sender/receiver pair)
    outs = []
    for r, p in enumerate(parts):
        out = torch.empty((p["n"], F), device=DEV)
        rp, c, v = p["local"].csr()
        ops.spmm(rp, c, v, p["x"], out, p["n"], accumulate=False)
        if sum(p["recv_splits"]):
            rp, c, v = p["remote"].csr()
            if bits == 32:
                recv = torch.cat([sent[q][sum(parts[q]["send_splits"][:r]):sum(parts[q]["send_splits"][:r + 1])]
                                  for q in range(W)])
                ops.spmm(rp, c, v, recv, out, p["n"])
            else:
                epb = 8 // bits
                qs, ps = [], []
                for q in range(W):
                    ss = parts[q]["send_splits"]
                    r0 = sum(-(-cnt // epb) for cnt in ss[:r])
                    qs.append(sent[q][0][r0:r0 + -(-ss[r] // epb)])
                    ps.append(sent[q][1][sum(ss[:r]):sum(ss[:r + 1])])
                wr = torch.tensor([0] + list(np.cumsum(p["recv_splits"])), dtype=torch.int32, device=DEV)
                ops.spmm_dequant(rp, c, v, torch.cat(qs), torch.cat(ps), wr, W, bits, out, p["n"])
        outs.append(out.cpu())
    got = torch.cat(outs).numpy()

    if bits == 32:
        want = oracle.spmm(rowptr.numpy(), col.numpy().astype(np.int64), None, x.numpy(), np.zeros((n, F), np.float32))
        mag = oracle.spmm(rowptr.numpy(), col.numpy().astype(np.int64), None, x.abs().numpy(), np.zeros((n, F), np.float32))
        assert np.all(np.abs(got - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30)
    else:
        # oracle pipeline per receiving rank: local rows exact, remote rows quantised by their sender
        want = np.zeros((n, F), np.float32)
        mag = np.zeros((n, F), np.float32)
        for r, p in enumerate(parts):
            lo, hi = begins[r], begins[r + 1]
            rp, c, _ = p["local"].csr()
            want[lo:hi] = oracle.spmm(rp.cpu().numpy(), c.cpu().numpy().astype(np.int64), None, x[lo:hi].numpy(),
                                      np.zeros((hi - lo, F), np.float32))
            mag[lo:hi] = oracle.spmm(rp.cpu().numpy(), c.cpu().numpy().astype(np.int64), None, x[lo:hi].abs().numpy(),
                                     np.zeros((hi - lo, F), np.float32))
            if not sum(p["recv_splits"]):
                continue
            rows = []
            for q in range(W):
                ss = parts[q]["send_splits"]
                idx = parts[q]["send_idx"].cpu().numpy()
                xs = x[begins[q]:begins[q + 1]].numpy()[idx]
                wrq = np.array([0] + list(np.cumsum(ss)), np.int32)
                qq, pp = oracle.quantize_for_all_procs(xs, wrq, bits)
                deq = oracle.dequantize_for_all_procs(qq, oracle.round_bf16(pp), wrq, bits)
                rows.append(deq[sum(ss[:r]):sum(ss[:r + 1])])
            recv = np.concatenate(rows)
            rp, c, _ = p["remote"].csr()
            want[lo:hi] = oracle.spmm(rp.cpu().numpy(), c.cpu().numpy().astype(np.int64), None, recv, want[lo:hi].copy())
            mag[lo:hi] = oracle.spmm(rp.cpu().numpy(), c.cpu().numpy().astype(np.int64), None, np.abs(recv), mag[lo:hi].copy())
        assert np.all(np.abs(got - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30)
