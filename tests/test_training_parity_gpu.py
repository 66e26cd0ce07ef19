"""20-epoch loss curve of the GPU GraphSAGE step against the CPU restatement of the
reference's step (oracle/cpu_graphsage.py: reference/oracle SpMM + stock PyTorch CPU),
same initial weights and the same injected dropout masks.  Tolerance: |loss difference|
<= 1e-3 at every epoch."""
import os
import sys

import numpy as np
import pytest
import torch

from super_gnn_b200 import graphsage, synthetic
from super_gnn_b200.data_manager import build_distributed_graph

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_loss_curve_matches_cpu_reference_over_20_epochs(oracle):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_graphsage as cg

    dev = torch.device("cuda", 0)
    n, e, fin, hid, ncls, epochs = 20_000, 250_000, 100, 256, 47, 20
    s, t = synthetic.rmat_edges(n, e, 0.57, 0.19, 0.19, 0.05, seed=2)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    g = torch.Generator().manual_seed(2)
    feats = torch.randn(n, fin, generator=g)
    labels = torch.randint(0, ncls, (n,), generator=g)
    mask = torch.rand(n, generator=g) < 0.10
    num_train = float(mask.sum())

    # CPU side: CSR of the in-edges (row = destination), reference SpMM when available
    kind, spmm_fn = cg.load_backend(prefer_reference=True)
    cg.CpuAggregator.spmm = spmm_fn
    order = torch.argsort(t * n + s)
    rowptr = torch.zeros(n + 1, dtype=torch.int64)
    torch.cumsum(torch.bincount(t, minlength=n), 0, out=rowptr[1:])
    threads = torch.get_num_threads()
    if kind == "reference":
        import ctypes
        try:
            threads = int(ctypes.CDLL("libgomp.so.1").omp_get_max_threads())
        except OSError:
            pass
    cgraph = cg.CpuGraph(rowptr, s[order], n, threads)

    # GPU side
    graph = build_distributed_graph(torch.stack([s, t]), torch.zeros((2, 0), dtype=torch.int64), [0, n], hid, 32,
                                    device=dev)
    torch.manual_seed(2)
    cfg = dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=0.5, lr=0.01)
    model, opt = graphsage.create_model_and_optimizer(cfg, device=None)  # initialised on the CPU generator
    cmodel = cg.CpuSAGE(fin, hid, ncls, 3, 0.5)
    cmodel.load_from(model.state_dict())
    model = model.to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=0.01)
    copt = torch.optim.Adam(cmodel.parameters(), lr=0.01)
    data = dict(graph=graph, nodes_features=feats.to(dev), nodes_labels=labels.to(dev), nodes_train_masks=mask.to(dev))

    mg = torch.Generator().manual_seed(99)
    gpu_curve, cpu_curve = [], []
    for _ in range(epochs):
        masks = [(torch.rand(n, hid, generator=mg) >= 0.5).float() * 2.0 for _ in range(2)]
        model.dropout_masks = [m.to(dev) for m in masks]
        cmodel.dropout_masks = masks
        gpu_curve.append(float(graphsage.train_step(model, data, opt, num_train)))
        cpu_curve.append(float(cg.train_step(cmodel, cgraph, feats, labels, mask, copt, num_train)))
    diff = np.abs(np.array(gpu_curve) - np.array(cpu_curve))
    assert gpu_curve[-1] < gpu_curve[0]  # it trains
    assert diff.max() <= 1e-3, f"max |loss diff| {diff.max():.2e}; gpu {gpu_curve[:3]}..{gpu_curve[-1]}, cpu {cpu_curve[:3]}..{cpu_curve[-1]}"
