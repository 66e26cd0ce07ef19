"""Worker of the partitioned loss-curve parity test (launched by torch.distributed.run).

Every rank trains its partition of one seeded R-MAT graph for ``--epochs`` full-batch steps with a
QUANTISED boundary exchange (the reference's training mode of interest: super_gnn/communicator.py:221-306
under examples/graphsage/train.py:21-54), for every ``bits:pre`` pair of ``--cases``; rank 0 writes the summed
loss per epoch to ``--out`` as JSON.

Two pipelines produce the curves that the test compares (|difference| <= 1e-3 at every epoch):

* ``--emulate``: the CPU pipeline.  gloo CPU ranks, the reference's unfused chain of ops per layer
  (aggregate, divide by the in-degree, two linear maps, bias, dropout, LayerNorm, relu), the boundary rows
  through the oracle's quantise -> bf16 parameters -> dequantise.
* ``--gloo-gpu``: the CUDA path as the benchmark runs it (fused layers, mean folded into the SpMM, last layer
  aggregating only the remote edges at the input width, loss fused into the last layer, fused
  quantise-pack / dequantise-SpMM kernels), on ranks that share one GPU with the exchange staged through host
  memory; without the flag the ranks use NCCL, one GPU each.

Both start from the same weights (CPU generator) and use the same dropout masks (drawn per epoch for the whole
graph from one seeded generator; each rank takes its rows).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

DIMS = dict(fin=32, hid=64, ncls=7, p=0.5)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--emulate", action="store_true")
    ap.add_argument("--gloo-gpu", action="store_true")
    ap.add_argument("--cases", default="2:0,8:1", help="comma-separated bits:pre pairs")
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--nodes", type=int, default=6000)
    ap.add_argument("--edges", type=int, default=60000)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()

    if args.gloo_gpu:
        os.environ["SGNN_DIST_BACKEND"] = "gloo"
    from super_gnn_b200 import graphsage, synthetic
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.data_manager import (build_distributed_graph, build_distributed_graph_pre_post,
                                             partition_edges)
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    if args.emulate:
        import cpu_ops_emulation

        cpu_ops_emulation.install()
        torch.cuda.is_available = lambda: False
    Communicator(32, is_async=True)
    rank, W = Communicator.ctx.init_dist_group()
    device = torch.device("cpu") if args.emulate else torch.device("cuda", torch.cuda.current_device())
    if args.emulate:
        import oracle

        oracle.build()

    n = args.nodes
    fin, hid, ncls, p = DIMS["fin"], DIMS["hid"], DIMS["ncls"], DIMS["p"]
    s, t = synthetic.rmat_edges(n, args.edges, 0.57, 0.19, 0.19, 0.05, seed=11)
    s, t = synthetic.symmetrize_dedup(s, t, n)
    s, t = synthetic.random_relabel(s, t, n, seed=11)
    gen = torch.Generator().manual_seed(12)
    x_all = torch.randn(n, fin, generator=gen)
    labels = torch.randint(0, ncls, (n,), generator=gen)
    train = torch.rand(n, generator=gen) < 0.3
    num_train = float(train.sum())
    begins = synthetic.even_ranges(n, W)
    lo, hi = begins[rank], begins[rank + 1]
    local_edges, remote_edges = partition_edges(s, t, begins, rank)

    curves = {}
    for case in args.cases.split(","):
        bits, is_pre = int(case.split(":")[0]), bool(int(case.split(":")[1]))
        Communicator.ctx.num_bits = bits
        Quantizer_for_all_procs(W, bits)
        build = build_distributed_graph_pre_post if is_pre else build_distributed_graph
        graph = build(local_edges, remote_edges, begins, max(fin, hid), bits, device=device)
        if not args.emulate:
            graph.set_fold_mean(True)
        torch.manual_seed(2)  # CPU generator: the same initial weights in both pipelines and on every rank
        model = graphsage.DistSAGE(fin, hid, ncls, 3, p, bits, is_pre, "LayerNorm")
        model.reset_parameters()
        model = model.to(device)
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        ddp.register_comm_hook(state=None, hook=graphsage.allreduce_hook)
        opt = torch.optim.Adam(ddp.parameters(), lr=0.01)
        data = dict(graph=graph, nodes_features=x_all[lo:hi].to(device), nodes_labels=labels[lo:hi].to(device),
                    nodes_train_masks=train[lo:hi].to(device))
        mg = torch.Generator().manual_seed(99)
        curve = []
        for _ in range(args.epochs):
            masks = [(torch.rand(n, hid, generator=mg) >= p).float() / (1 - p) for _ in range(2)]
            model.dropout_masks = [m[lo:hi].to(device) for m in masks]
            loss = graphsage.train_step(ddp, data, opt, num_train).detach().clone().reshape(1)
            dist.all_reduce(loss)  # every rank holds its share of the summed NLL / global count
            curve.append(float(loss.item()))
        curves[case] = curve
        del ddp, opt
    Communicator.ctx.num_bits = 32
    if rank == 0:
        with open(args.out, "w") as f:
            json.dump({"world": W, "epochs": args.epochs, "nodes": n, "edges": args.edges, "curves": curves}, f)
        print("loss_curve_worker: ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
