"""Worker of the drop-in test (launched by torch.distributed.run on gloo CPU ranks).

The package is registered under the reference's module names (``install_as_super_gnn``) and the reference's OWN
driver code is then imported from its tree, unmodified and read-only: ``examples/graphsage/sage.py`` (``DistSAGE``),
``utils.py`` (``create_model_and_optimizer`` with its DDP sum hook) and ``train.py`` (``train_step``).  Three
stand-in modules cover names the drivers import but this environment does not have and the GraphSAGE path does
not use: ``torch_geometric.utils.index_to_mask`` (train.py:17), ``super_gnn.layers.gcnconv`` (imported by the GCN
model that utils.py pulls in).

The reference's model and training step, running over this package's Aggregator / Communicator / layers with a
2-bit boundary exchange, must give the same losses and the same parameters after three epochs as this package's
own ``graphsage.DistSAGE`` / ``train_step`` (unfused path): same weights, same dropout draws, same kernels
underneath.  On these CPU ranks the kernels are the oracle-backed stand-ins of ``cpu_ops_emulation``.
"""
import argparse
import os
import sys
import types

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def install_stand_ins():
    tg = types.ModuleType("torch_geometric")
    tgu = types.ModuleType("torch_geometric.utils")

    def index_to_mask(index, size=None):
        size = int(index.max()) + 1 if size is None else size
        mask = index.new_zeros(size, dtype=torch.bool)
        mask[index] = True
        return mask

    tgu.index_to_mask = index_to_mask
    tg.utils = tgu
    sys.modules.setdefault("torch_geometric", tg)
    sys.modules.setdefault("torch_geometric.utils", tgu)
    gcn = types.ModuleType("super_gnn.layers.gcnconv")

    class DistGCNConvGrad(torch.nn.Module):  # the GCN driver is outside the GraphSAGE path
        def __init__(self, *a, **k):
            raise RuntimeError("GCN layers are not provided")

    gcn.DistGCNConvGrad = DistGCNConvGrad
    sys.modules.setdefault("super_gnn.layers.gcnconv", gcn)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()

    import cpu_ops_emulation
    import super_gnn_b200

    cpu_ops_emulation.install()
    torch.cuda.is_available = lambda: False
    super_gnn_b200.install_as_super_gnn()
    install_stand_ins()
    sys.path.insert(0, os.path.join(args.reference, "examples", "graphsage"))
    import sage as ref_sage  # noqa: E402  the reference's model, from its own tree
    import train as ref_train  # noqa: E402  the reference's training step
    import utils as ref_utils  # noqa: E402

    from super_gnn.assigner import Assigner
    from super_gnn.communicator import Communicator
    from super_gnn.data_manager import build_distributed_graph, partition_edges
    from super_gnn.quantizer import Quantizer_for_all_procs
    from super_gnn.time_recorder import TimeRecorder
    from super_gnn_b200 import graphsage, synthetic
    from torch_geometric.utils import index_to_mask

    assert ref_sage.DistSAGEConvGrad is sys.modules["super_gnn_b200.layers.sageconv"].DistSAGEConvGrad

    bits, fin, hid, ncls, layers = 2, 32, 64, 7, 3
    Communicator(bits, is_async=True)
    rank, W = Communicator.ctx.init_dist_group()
    Quantizer_for_all_procs(W, bits)
    TimeRecorder(layers, 3)
    n = 1500
    s, t = synthetic.rmat_edges(n, 15000, 0.57, 0.19, 0.19, 0.05, seed=21)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    s, t = synthetic.random_relabel(s, t, n, seed=21)
    begins = synthetic.even_ranges(n, W)
    lo, hi = begins[rank], begins[rank + 1]
    local_edges, remote_edges = partition_edges(s, t, begins, rank)
    gen = torch.Generator().manual_seed(22)
    x_all = torch.randn(n, fin, generator=gen)
    labels = torch.randint(0, ncls, (n,), generator=gen)
    train_idx_all = torch.nonzero(torch.rand(n, generator=gen) < 0.4).reshape(-1)
    mine = train_idx_all[(train_idx_all >= lo) & (train_idx_all < hi)] - lo
    num_train = float(train_idx_all.numel())
    cfg = dict(model_name="sage", in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=layers, dropout=0.5,
               num_bits=bits, is_pre_delay=False, norm_type="LayerNorm", is_label_augment=False, lr=0.01, weight_decay=0.0)

    def fresh_data():
        graph = build_distributed_graph(local_edges, remote_edges, begins, max(fin, hid), bits, device=torch.device("cpu"))
        Assigner(bits, layers, torch.tensor([0.0, 0.0, 1.0]), 1, sum(graph.comm_splits.send_splits),
                 sum(graph.comm_splits.recv_splits))
        train_mask = index_to_mask(mine, hi - lo)  # train.py:125 does the same conversion
        rest = torch.nonzero(~train_mask).reshape(-1)
        return dict(graph=graph, nodes_features=x_all[lo:hi].clone(), nodes_labels=labels[lo:hi].clone(),
                    nodes_train_masks=train_mask, nodes_valid_masks=index_to_mask(rest[::2], hi - lo),
                    nodes_test_masks=index_to_mask(rest[1::2], hi - lo))

    # --- the reference's model, optimiser and training step
    torch.manual_seed(5)
    ref_model, ref_opt = ref_utils.create_model_and_optimizer(cfg)
    init = {k: v.detach().clone() for k, v in ref_model.state_dict().items()}
    data = fresh_data()
    torch.manual_seed(77)  # dropout draws
    ref_losses = [float(ref_train.train_step(ref_model, data, ref_opt, epoch, num_train, 0.0)) for epoch in range(3)]
    ref_acc = ref_train.test_step(ref_model, data, False)  # the reference's evaluation pass (fp32 exchange: train.py:57-99)
    with torch.no_grad():
        ref_eval = ref_model(data["graph"], data["nodes_features"], data["nodes_labels"], None)

    # --- this package's model and step on the same weights and dropout draws
    torch.manual_seed(5)
    own_model, own_opt = graphsage.create_model_and_optimizer(cfg)
    own_model.load_state_dict(init)
    data = fresh_data()
    torch.manual_seed(77)
    own_losses = [float(graphsage.train_step(own_model, data, own_opt, num_train)) for _ in range(3)]
    own_acc = ref_train.test_step(own_model, data, False)  # the same evaluation pass over this package's model
    with torch.no_grad():
        own_eval = own_model(data["graph"], data["nodes_features"])

    fails = []
    for a, b in zip(ref_losses, own_losses):
        if abs(a - b) > 1e-6 * max(1.0, abs(a)):
            fails.append(f"loss {a} (reference driver) vs {b}")
    ref_state, own_state = ref_model.state_dict(), own_model.state_dict()
    if sorted(ref_state) != sorted(own_state):
        fails.append("parameter names differ")
    for k in ref_state:
        if not torch.allclose(ref_state[k], own_state[k], rtol=1e-5, atol=1e-7):
            fails.append(f"parameter {k} differs after three epochs")
    if not torch.allclose(ref_eval, own_eval, rtol=1e-5, atol=1e-6):
        fails.append("evaluation forward differs")
    if any(abs(a - b) > 1e-6 * max(1.0, abs(a)) for a, b in zip(ref_acc, own_acc)):
        fails.append(f"test_step results differ: {ref_acc} vs {own_acc}")
    if not (ref_losses[-1] < ref_losses[0]):
        fails.append(f"the reference driver does not train: {ref_losses}")
    everyone = [None] * W
    dist.all_gather_object(everyone, fails)
    fails = [f for fs in everyone for f in fs]
    if rank == 0:
        for f in fails:
            print("FAIL:", f, flush=True)
        print("drop_in_worker:", "ok" if not fails else f"{len(fails)} failure(s)", ref_losses, flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if not fails else 1)


if __name__ == "__main__":
    main()
