"""Worker of the multi-rank Aggregator tests (launched by torch.distributed.run).

Every rank builds its partition of one seeded R-MAT graph, runs
``Aggregator`` forward and backward through the real ``Communicator`` for
32/16/8/4/2-bit boundary exchange, fused and unfused, and rank 0 checks the
gathered results against the CPU oracle:

* 32 bit: partitioned result == single-graph A x and A^T g (1e-5 relative);
* 2/4/8 bit: == the oracle's pipeline quantise -> bf16 params -> dequantise of the
  reference (codes bit-exact, so the same 1e-5 bound applies).  In the backward
  pass the rows that get quantised are themselves SpMM results, so the oracle
  quantises the ranks' own fp32 gradient rows (gathered), not a recomputation.

``--emulate``: gloo CPU ranks with the oracle-backed op stand-ins, which
exercises exactly the same host logic where no GPU exists.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--emulate", action="store_true")
    ap.add_argument("--p2p", action="store_true", help="2/4/8-bit modes through the one-sided NVLink exchange")
    ap.add_argument("--graph", default="rmat", choices=["rmat", "sbm8", "rmat-stream"],
                    help="rmat: a global edge list cut into ranges; sbm8 / rmat-stream: the partition-parallel generators")
    ap.add_argument("--row-groups", action="store_true",
                    help="keep the reference's row-group bytes on the wire (default: the row-codes layout)")
    ap.add_argument("--gloo-gpu", action="store_true",
                    help="CUDA kernels on every rank, exchange staged through host memory over gloo: the ranks may "
                         "share one GPU (no kernel of one rank waits for another's)")
    ap.add_argument("--nodes", type=int, default=3000)
    ap.add_argument("--edges", type=int, default=40000)
    ap.add_argument("--feat", type=int, default=128)
    ap.add_argument("--model", action="store_true", help="whole GraphSAGE model against a dense single-process reference")
    ap.add_argument("--degree-order", action="store_true",
                    help="renumber every rank's nodes by in-degree first (order_nodes_by_degree); the checks then run "
                         "on the renumbered graph put together from the ranks' edge lists")
    ap.add_argument("--absent-peer", action="store_true",
                    help="one-sided exchange: the last rank stays away from a barrier (on the host, between steps); "
                         "the others must get a PeerTimeout, not a trap, and carry on")
    args = ap.parse_args()

    import oracle
    from super_gnn_b200 import synthetic
    from super_gnn_b200.aggregator import Aggregator
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.data_manager import (build_distributed_graph, build_distributed_graph_pre_post,
                                             partition_edges)
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    if args.gloo_gpu:
        os.environ["SGNN_DIST_BACKEND"] = "gloo"
    if args.emulate:
        import cpu_ops_emulation

        cpu_ops_emulation.install()
        torch.cuda.is_available = lambda: False
    Communicator(32, is_async=True)
    if args.row_groups:
        Communicator.row_codes = False
    rank, W = Communicator.ctx.init_dist_group()
    device = torch.device("cpu") if args.emulate else torch.device("cuda", torch.cuda.current_device())
    oracle.build()

    n, F = args.nodes, args.feat
    if args.graph == "rmat":  # one global edge list, cut into contiguous ranges after a random relabel
        s, t = synthetic.rmat_edges(n, args.edges, 0.57, 0.19, 0.19, 0.05, seed=7)
        s, t = synthetic.symmetrize_dedup(s, t, n)
        s, t = synthetic.random_relabel(s, t, n, seed=7)
        begins = synthetic.even_ranges(n, W)
        local_edges, remote_edges = partition_edges(s, t, begins, rank)
    else:
        # the partition-parallel generators of the large benchmark workloads: every rank produces its own edges,
        # no rank holds the global list; it is put together here only so that rank 0 can check against the oracle
        from super_gnn_b200 import workloads

        if args.graph == "sbm8":  # 8 equal blocks, 90 % of the edges inside a block (the pre/post configuration)
            n = n // 8 * 8
            local_edges, remote_edges, begins = workloads.sbm_partition(8, n // 8, args.edges, 0.9, rank, W, 3, device)
        else:  # "rmat-stream": the chunked R-MAT stream with a random relabel (the large scaling sweep)
            local_edges, remote_edges, begins = workloads.rmat_partition(n, args.edges, rank, W, 4, device)
        local_edges, remote_edges = local_edges.cpu(), remote_edges.cpu()
    if args.degree_order:
        from super_gnn_b200.data_manager import order_nodes_by_degree

        before = (local_edges.size(1), remote_edges.size(1))
        local_edges, remote_edges, order = order_nodes_by_degree(local_edges.to(device), remote_edges.to(device), begins)
        local_edges, remote_edges = local_edges.cpu(), remote_edges.cpu()
        assert (local_edges.size(1), remote_edges.size(1)) == before
        assert sorted(order.tolist()) == list(range(begins[rank + 1] - begins[rank]))
        deg = torch.bincount(torch.cat([local_edges[1], remote_edges[1]]), minlength=order.numel())
        assert bool((deg[1:] >= deg[:-1]).all()), "in-degrees must ascend with the new ids"
    if args.graph != "rmat" or args.degree_order:
        old_edges = (s, t) if args.graph == "rmat" else None
        lo0 = begins[rank]
        mine = (torch.cat([local_edges[0] + lo0, remote_edges[0]]), torch.cat([local_edges[1], remote_edges[1]]) + lo0)
        everyone = [None] * W
        dist.all_gather_object(everyone, mine)
        s, t = torch.cat([e[0] for e in everyone]), torch.cat([e[1] for e in everyone])
        if args.degree_order and old_edges is not None:
            # the renumbered graph is the old one under the permutation the ranks report
            orders = [None] * W
            dist.all_gather_object(orders, order.cpu())
            new_of_old = torch.empty(n, dtype=torch.int64)
            for r, o in enumerate(orders):
                new_of_old[o + begins[r]] = torch.arange(o.numel()) + begins[r]
            want = torch.sort(new_of_old[old_edges[1]] * n + new_of_old[old_edges[0]])[0]
            assert torch.equal(want, torch.sort(t * n + s)[0]), "renumbered edges are not the old edges under `order`"
    gen = torch.Generator().manual_seed(3)
    x_all = torch.randn(n, F, generator=gen)
    g_all = torch.randn(n, F, generator=gen)
    lo, hi = begins[rank], begins[rank + 1]

    if args.model:
        failures = model_against_dense_reference(rank, W, device, s, t, n, begins, local_edges, remote_edges)
        finish(rank, failures)
        return
    if args.absent_peer:
        finish(rank, absent_peer(rank, W, device, begins, local_edges, remote_edges, F))
        return

    failures = []
    for is_pre in (False, True):
        for bits in (32, 16, 8, 4, 2):
            Communicator.ctx.num_bits = bits
            Quantizer_for_all_procs(W, bits)
            build = build_distributed_graph_pre_post if is_pre else build_distributed_graph
            graph = build(local_edges, remote_edges, begins, F, bits, device=device)
            if args.p2p and bits in (2, 4, 8):
                Communicator.ctx.enable_peer_exchange(graph, F)
            remote_adj = graph.adj_t_pre_post_aggr_from if is_pre else graph.remote_adj_t
            for fused, fold in ((True, False), (False, False), (True, True)):
                Aggregator.fused = fused
                graph.set_fold_mean(fold)
                x = x_all[lo:hi].to(device).requires_grad_(True)
                out = Aggregator.apply(graph, x, 0, bits, is_pre, True)
                if device.type == "cuda":
                    torch.cuda.synchronize()
                fwd_send_rows = graph.comm_buf.send_buf.detach().cpu().numpy().copy() if is_pre else None
                out.backward(g_all[lo:hi].to(device))
                if device.type == "cuda":
                    torch.cuda.synchronize()
                if fused:
                    failures += check_out_and_accumulate(Aggregator, graph, x.detach(), g_all[lo:hi].to(device),
                                                         out.detach(), x.grad, bits, is_pre, rank,
                                                         f"pre={is_pre} bits={bits} fold_mean={fold}")
                mine = dict(out=out.detach().cpu().numpy(), grad=x.grad.cpu().numpy(),
                            remote_grad_rows=graph.comm_buf.recv_buf.detach().cpu().numpy().copy(),
                            fwd_send_rows=fwd_send_rows, fold=fold,
                            inv_deg=(1.0 / graph.in_degrees).reshape(-1).cpu().numpy(),
                            send_splits=list(graph.comm_splits.send_splits),
                            recv_splits=list(graph.comm_splits.recv_splits),
                            local=tuple(a.cpu().numpy() for a in graph.local_adj_t.csr()[:2]),
                            remote=tuple(a.cpu().numpy() for a in remote_adj.csr()[:2]),
                            local_T=(graph.local_adj_t.storage.colptr().cpu().numpy(),
                                     graph.local_adj_t.storage.row_T().cpu().numpy()))
                if is_pre:
                    to = graph.adj_t_pre_post_aggr_to
                    mine["to"] = tuple(a.cpu().numpy() for a in to.csr()[:2])
                    mine["to_T"] = (to.storage.colptr().cpu().numpy(), to.storage.row_T().cpu().numpy())
                else:
                    mine["send_idx"] = graph.idx_nodes_send_to_others.cpu().numpy()
                parts = [None] * W
                dist.all_gather_object(parts, mine)
                if rank == 0:
                    failures += check(oracle, parts, begins, x_all.numpy(), g_all.numpy(), bits, fused, W, F, is_pre,
                                      (s.numpy(), t.numpy()))
            if bits in (2, 4, 8):
                failures += by_peer_matches_full(Aggregator, graph, remote_adj, x_all[lo:hi].to(device),
                                                 g_all[lo:hi].to(device), bits, is_pre, rank)
    Aggregator.fused = True
    failures += eval_mode_uses_exact_rows(Aggregator, rank, W, device, begins, local_edges, remote_edges, x_all, F,
                                          (s.numpy(), t.numpy()))
    finish(rank, failures)


def by_peer_matches_full(Aggregator, graph, remote_adj, x, g, bits, is_pre, rank):
    """Backward pass with the gradient rows for the peers produced, quantised and sent one peer at a time
    (row ranges of A_remote^T, the fp32 rows of one peer at a time) against the same pass over the full buffer.
    The transposed remote matrix is pinned to the row-split kernel, whose per-row sums do not depend on how the
    rows are grouped into launches, so both passes quantise identical rows and only the order of the final
    fp32 additions may differ."""
    from super_gnn_b200 import supergnn_ops

    Aggregator.fused = True
    graph.set_fold_mean(False)
    remote_adj.set_work_range_for_transpose(torch.tensor([supergnn_ops.SPMM_ROW_SPLIT], dtype=torch.int32),
                                            torch.empty(0, dtype=torch.int32))
    grads = {}
    for mode in (False, True):
        Aggregator.remote_gradient_by_peer = mode
        xx = x.clone().requires_grad_(True)
        Aggregator.apply(graph, xx, 0, bits, is_pre, True).backward(g)
        if x.is_cuda:
            torch.cuda.synchronize()
        grads[mode] = xx.grad.detach().clone()
    Aggregator.remote_gradient_by_peer = "auto"
    err = (grads[True] - grads[False]).abs().max().item()
    ok = err <= 2e-5 * (grads[False].abs().max().item() + 1.0)
    return [] if ok else [f"remote gradient by peer differs from the full pass: pre={is_pre} bits={bits} rank={rank} "
                          f"max |diff| {err:.3e}"]


def eval_mode_uses_exact_rows(Aggregator, rank, W, device, begins, local_edges, remote_edges, x_all, F, edges):
    """Outside training the boundary rows travel as fp32 whatever ``num_bits`` says
    (super_gnn/communicator.py:61, super_gnn/aggregator.py:74): with a 2- or 8-bit communicator the evaluation
    forward must equal the single-graph A x to fp32 rounding, in both aggregation modes."""
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.data_manager import build_distributed_graph, build_distributed_graph_pre_post
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    lo, hi = begins[rank], begins[rank + 1]
    src, dst = edges
    n = begins[-1]
    fails = []
    for is_pre in (False, True):
        for bits in (8, 2):
            Communicator.ctx.num_bits = bits
            Quantizer_for_all_procs(W, bits)
            build = build_distributed_graph_pre_post if is_pre else build_distributed_graph
            graph = build(local_edges, remote_edges, begins, F, bits, device=device)
            with torch.no_grad():
                out = Aggregator.apply(graph, x_all[lo:hi].to(device), 0, bits, is_pre, False)
            if device.type == "cuda":
                torch.cuda.synchronize()
            parts = [None] * W
            dist.all_gather_object(parts, out.cpu().numpy())
            if rank == 0:
                got = np.concatenate(parts)
                want = np.zeros((n, F), np.float64)
                np.add.at(want, dst, x_all.numpy()[src].astype(np.float64))
                mag = np.zeros((n, F), np.float64)
                np.add.at(mag, dst, np.abs(x_all.numpy()[src]).astype(np.float64))
                if not np.all(np.abs(got - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30):
                    fails.append(f"evaluation forward with a {bits}-bit communicator, pre={is_pre}: not the exact A x")
    Communicator.ctx.num_bits = 32
    return fails


def finish(rank, failures):
    everyone = [None] * dist.get_world_size()
    dist.all_gather_object(everyone, list(failures))  # some checks run on every rank
    failures = [f for fs in everyone for f in fs]
    if rank == 0:
        for f in failures:
            print("FAIL:", f, flush=True)
        print("dist_worker:", "ok" if not failures else f"{len(failures)} failure(s)", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if (rank != 0 or not failures) else 1)


def absent_peer(rank, W, device, begins, local_edges, remote_edges, F):
    """A rank that never joins a barrier of the one-sided exchange (a failure made on the host: it simply does not
    make the call, with none of its kernels in flight).  The ranks that do call wait for the short limit, their
    kernel returns, ``check()`` raises ``PeerTimeout`` naming the absent rank, and the context is still usable."""
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.data_manager import build_distributed_graph
    from super_gnn_b200.peer_exchange import PeerTimeout
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    failures = []
    Communicator.ctx.num_bits = 2
    Quantizer_for_all_procs(W, 2)
    graph = build_distributed_graph(local_edges, remote_edges, begins, F, 2, device=device)
    px = Communicator.ctx.enable_peer_exchange(graph, F, timeout_ms=300)
    cur = torch.cuda.current_stream()
    px.begin(cur)  # everybody arrives
    px.end(cur)
    torch.cuda.synchronize()
    try:
        px.check()
    except PeerTimeout as e:
        failures.append(f"rank {rank}: barrier with every rank present reported {e}")
    absent = W - 1
    if rank != absent:
        px.begin(cur)  # the last rank never makes this call
        torch.cuda.synchronize()
        try:
            px.check()
            failures.append(f"rank {rank}: no PeerTimeout although rank {absent} stayed away")
        except PeerTimeout as e:
            if f"peer(s) {absent} " not in str(e):
                failures.append(f"rank {rank}: PeerTimeout names the wrong peer: {e}")
        got = px.status.tolist()
        if [i for i, v in enumerate(got) if v] != [absent]:
            failures.append(f"rank {rank}: status {got}")
        if int(torch.arange(10, device=device).sum().item()) != 45:  # the context survived
            failures.append(f"rank {rank}: context unusable after the timeout")
    return failures


def model_against_dense_reference(rank, W, device, s, t, n, begins, local_edges, remote_edges):
    """One training-mode forward + backward of the 3-layer model over W partitions with an exact (32-bit)
    boundary exchange and injected dropout masks, against the same model evaluated by rank 0 on the whole graph
    with a dense adjacency matrix in fp64: loss and every (summed) parameter gradient.  On CUDA ranks this is the
    fused path (tensor-core GEMMs, fused epilogues, last layer projecting before it aggregates across the
    partition boundary); on CPU ranks the unfused chain over the emulated ops."""
    import torch.nn.functional as Fn

    from super_gnn_b200 import graphsage
    from super_gnn_b200.data_manager import build_distributed_graph, build_distributed_graph_pre_post

    fin, hid, ncls, p = 20, 64, 7, 0.5
    gen = torch.Generator().manual_seed(5)
    x_all = torch.randn(n, fin, generator=gen)
    labels = torch.randint(0, ncls, (n,), generator=gen)
    train = torch.rand(n, generator=gen) < 0.6
    masks = [(torch.rand(n, hid, generator=gen) >= p).float() / (1 - p) for _ in range(2)]
    lo, hi = begins[rank], begins[rank + 1]
    failures = []
    for is_pre in (False, True):
        build = build_distributed_graph_pre_post if is_pre else build_distributed_graph
        graph = build(local_edges, remote_edges, begins, hid, 32, device=device)
        # last layer: "auto" projects before it aggregates (the exchange is exact here); False keeps the reference's
        # order, which with a folded mean aggregates only the remote edges at the input width
        for fold, project_first in ((False, "auto"), (True, "auto"), (True, False), (False, False)):
            graph.set_fold_mean(fold)
            torch.manual_seed(0)
            model, _ = graphsage.create_model_and_optimizer(
                dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=p, num_bits=32,
                     is_pre_delay=is_pre), device=device)
            core = model.module if hasattr(model, "module") else model
            core.project_first = project_first
            core.dropout_masks = [m[lo:hi].to(device) for m in masks]
            model.train()
            model.zero_grad()
            out = model(graph, x_all[lo:hi].to(device))
            m = train[lo:hi].to(device)
            loss = Fn.nll_loss(out[m], labels[lo:hi].to(device)[m], reduction="sum") / float(train.sum())
            loss.backward()  # DDP sums the weight gradients over the ranks
            total = loss.detach().clone()
            dist.all_reduce(total)
            if rank != 0:
                continue
            # dense fp64 reference of the whole graph on rank 0
            A = torch.zeros(n, n, dtype=torch.float64)
            A[t, s] = 1.0  # row = destination
            A = A / A.sum(1).clamp(min=1).unsqueeze(1)
            params = {k: v.detach().cpu().double().requires_grad_(True) for k, v in core.named_parameters()}
            h = x_all.double()
            for i in range(3):
                z = (A @ h) @ params[f"convs.{i}.lin_neigh.weight"].t() + h @ params[f"convs.{i}.lin_self.weight"].t() \
                    + params[f"convs.{i}.bias"]
                if i < 2:
                    z = z * masks[i].double()
                    z = Fn.layer_norm(z, (hid,), params[f"norms.{i}.weight"], params[f"norms.{i}.bias"], 1e-5)
                    h = torch.relu(z)
            ref = Fn.nll_loss(Fn.log_softmax(z, 1)[train], labels[train], reduction="sum") / float(train.sum())
            ref.backward()
            tag = f"model pre={is_pre} fold_mean={fold} project_first={project_first}"
            if abs(total.item() - ref.item()) > 2e-5 * abs(ref.item()):
                failures.append(f"{tag}: loss {total.item()} vs {ref.item()}")
            for k, v in core.named_parameters():
                got, want = v.grad.detach().cpu().double(), params[k].grad
                if (got - want).abs().max() > 1e-4 * (want.abs().max() + 1e-12):
                    failures.append(f"{tag}: grad {k} off by {(got - want).abs().max().item():.3e} "
                                    f"(scale {want.abs().max().item():.3e})")
    if device.type == "cuda":
        failures += narrow_local_against_reference_order(rank, device, begins, local_edges, remote_edges, x_all, labels,
                                                         train, masks, (fin, hid, ncls, p))
    return failures


def narrow_local_against_reference_order(rank, device, begins, local_edges, remote_edges, x_all, labels, train, masks,
                                         dims):
    """Quantised boundary exchange: the last layer that aggregates only the remote edges at the input width must
    give what the plain aggregate-then-project order gives (the exchanged rows are the same, so the quantisation
    noise is the same; only fp32 rounding differs)."""
    import torch.nn.functional as Fn

    from super_gnn_b200 import graphsage
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.data_manager import build_distributed_graph, build_distributed_graph_pre_post
    from super_gnn_b200.fused_layer import FusedSAGEOutputLayer
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    fin, hid, ncls, p = dims
    lo, hi = begins[rank], begins[rank + 1]
    failures = []
    W = dist.get_world_size()
    for is_pre in (False, True):
        for bits in (2, 8):
            Communicator.ctx.num_bits = bits
            Quantizer_for_all_procs(W, bits)
            build = build_distributed_graph_pre_post if is_pre else build_distributed_graph
            graph = build(local_edges, remote_edges, begins, hid, bits, device=device)
            graph.set_fold_mean(True)
            results = {}
            for narrow in (True, False, "with-loss"):
                FusedSAGEOutputLayer.narrow_local = bool(narrow)
                torch.manual_seed(0)
                model, _ = graphsage.create_model_and_optimizer(
                    dict(in_channels=fin, hidden_channels=hid, out_channels=ncls, num_layers=3, dropout=p,
                         num_bits=bits, is_pre_delay=is_pre), device=device)
                core = model.module
                core.dropout_masks = [m[lo:hi].to(device) for m in masks]
                model.train()
                model.zero_grad()
                m = train[lo:hi].to(device)
                lab = labels[lo:hi].to(device)
                if narrow == "with-loss":  # the loss computed together with the last layer
                    graphsage.fuse_loss_narrow_local = True
                    assert core.can_fuse_loss(x_all[lo:hi].to(device), graph)
                    loss = model(graph, x_all[lo:hi].to(device), lab, None, loss_mask=m,
                                 loss_inv_count=1.0 / float(train.sum()), loss_unit_grad=True)
                else:
                    out = model(graph, x_all[lo:hi].to(device))
                    loss = Fn.nll_loss(out[m], lab[m], reduction="sum") / float(train.sum())
                loss.backward()
                total = loss.detach().clone()
                dist.all_reduce(total)
                results[narrow] = (total.item(), {k: v.grad.detach().clone() for k, v in core.named_parameters()})
            FusedSAGEOutputLayer.narrow_local = True
            for variant in (True, "with-loss"):
                tag = f"narrow-local last layer ({variant}), pre={is_pre} bits={bits}"
                if abs(results[variant][0] - results[False][0]) > 2e-5 * abs(results[False][0]):
                    failures.append(f"{tag}: loss {results[variant][0]} vs {results[False][0]}")
                for k, want in results[False][1].items():
                    got = results[variant][1][k]
                    if (got - want).abs().max() > 1e-4 * (want.abs().max() + 1e-12):
                        failures.append(f"{tag}: grad {k} off by {(got - want).abs().max().item():.3e} "
                                        f"(scale {want.abs().max().item():.3e})")
    Communicator.ctx.num_bits = 32
    return failures


def check_out_and_accumulate(Aggregator, graph, x, g, want_out, want_grad, bits, is_pre, rank, tag):
    """The entry the fused layers use: results written into (or added onto) a column slice of a wider row-major
    buffer must equal what the autograd path returned (same kernels, same exchanged bytes; only the order of the
    fp32 additions may differ)."""
    from super_gnn_b200.aggregator import aggregate_backward, aggregate_forward

    class Ctx:
        pass

    def near(a, b):
        return bool((a - b).abs().max() <= 2e-5 * (b.abs().max() + 1.0))

    fails = []
    n, F = x.shape
    gen = torch.Generator().manual_seed(11 + rank)
    wide = torch.randn(n, 2 * F + 4, generator=gen).to(x.device)
    left, right = wide[:, :F], wide[:, F + 4:]
    keep_mid = wide[:, F:F + 4].clone()
    base = right.clone()
    c = Ctx()
    with torch.no_grad():
        left.copy_(x)
        r1 = aggregate_forward(c, graph, left, 0, bits, is_pre, True, out=right, accumulate=True)
        if not (r1.data_ptr() == right.data_ptr() and near(right, base + want_out)):
            fails.append(f"forward accumulate into a slice: {tag}")
        aggregate_forward(c, graph, left, 0, bits, is_pre, True, out=right, accumulate=False)
        if not near(right, want_out):
            fails.append(f"forward overwrite of a slice: {tag}")
        left.copy_(g)
        base = right.clone()
        aggregate_backward(c, left, out=right, accumulate=True)
        if not near(right, base + want_grad):
            fails.append(f"backward accumulate into a slice: {tag}")
        aggregate_backward(c, left, out=right, accumulate=False)
        if not near(right, want_grad):
            fails.append(f"backward overwrite of a slice: {tag}")
        if not torch.equal(wide[:, F:F + 4], keep_mid) or not torch.equal(left, g):
            fails.append(f"bytes outside the result slice were touched: {tag}")
        # local_work: the caller aggregates over the local edges itself while the exchange is in flight and hands
        # back the buffer the remote contributions are added to
        from super_gnn_b200.aggregator import _mean_scale, _spmm_overwrite

        def local_forward():
            buf = torch.empty(n, F, device=x.device)
            _spmm_overwrite(graph.local_adj_t, x, buf, transpose=False, row_scale=_mean_scale(graph))
            return buf

        def local_backward():
            buf = torch.empty(n, F, device=x.device)
            _spmm_overwrite(graph.local_adj_t, g, buf, transpose=True, col_scale=_mean_scale(graph))
            return buf

        r2 = aggregate_forward(c, graph, x, 0, bits, is_pre, True, local_work=local_forward)
        if not near(r2, want_out):
            fails.append(f"forward with local_work: {tag}")
        r3 = aggregate_backward(c, g, local_work=local_backward)
        if not near(r3, want_grad):
            fails.append(f"backward with local_work: {tag}")
    return fails


def spmm64(oracle, rowptr, col, x, base=None, rows=None):
    rows = len(rowptr) - 1 if rows is None else rows
    out = np.zeros((rows, x.shape[1]), np.float32) if base is None else base.copy()
    return oracle.spmm(rowptr, col.astype(np.int64), None, x, out)


def through_the_wire(oracle, rows, splits, bits):
    """What the receiver reconstructs from fp32 rows grouped per peer."""
    if bits == 32 or rows.shape[0] == 0:
        return rows
    if bits == 16:  # bf16 on the wire, round to nearest even (communicator.py:101-133 of the reference)
        return oracle.round_bf16(rows)
    wr = np.concatenate([[0], np.cumsum(splits)]).astype(np.int32)
    q, p = oracle.quantize_for_all_procs(rows, wr, bits)
    return oracle.dequantize_for_all_procs(q, oracle.round_bf16(p), wr, bits)


def check(oracle, parts, begins, x_all, g_all, bits, fused, W, F, is_pre, edges):
    fails = []
    fold = parts[0]["fold"]
    tag = f"pre={is_pre} bits={bits} fused={fused} fold_mean={fold}"
    inv_deg = np.concatenate([p["inv_deg"] for p in parts]).astype(np.float32)
    if fold:
        # mean folded in: outputs are the sums times 1/in_degree, and the incoming gradient acts as g / in_degree
        g_all = g_all * inv_deg[:, None]
        for r, p in enumerate(parts):
            p["out"] = p["out"] / p["inv_deg"][:, None]

    def close(got, want, mag):
        return np.all(np.abs(got - want) <= 1e-5 * (mag + np.abs(want)) + 1e-30)

    # ---- forward: the fp32 rows every rank sends, grouped per destination
    if is_pre:  # partial sums / raw rows produced by adj_to @ x (checked here), then through the wire
        rows = []
        for q in range(W):
            xl = x_all[begins[q]:begins[q + 1]]
            S = sum(parts[q]["send_splits"])
            want = spmm64(oracle, *parts[q]["to"], xl, rows=S)
            mag = spmm64(oracle, *parts[q]["to"], np.abs(xl), rows=S)
            if not close(parts[q]["fwd_send_rows"], want, mag):
                fails.append(f"{tag} pre-aggregated send rows rank {q}")
            rows.append(parts[q]["fwd_send_rows"])
    else:
        rows = [x_all[begins[q]:begins[q + 1]][parts[q]["send_idx"]] for q in range(W)]
    sent = [through_the_wire(oracle, rows[q], parts[q]["send_splits"], bits) for q in range(W)]
    for r in range(W):
        p = parts[r]
        xl = x_all[begins[r]:begins[r + 1]]
        want = spmm64(oracle, *p["local"], xl)
        mag = spmm64(oracle, *p["local"], np.abs(xl))
        if sum(p["recv_splits"]):
            recv = np.concatenate([sent[q][sum(parts[q]["send_splits"][:r]):sum(parts[q]["send_splits"][:r + 1])]
                                   for q in range(W)])
            want = spmm64(oracle, *p["remote"], recv, base=want)
            mag = spmm64(oracle, *p["remote"], np.abs(recv), base=mag)
        if not close(p["out"], want, mag):
            fails.append(f"{tag} forward rank {r}")
    # ---- backward: every rank sends its remote-gradient rows (grouped per owner) through the wire
    back = [through_the_wire(oracle, parts[r]["remote_grad_rows"], parts[r]["recv_splits"], bits) for r in range(W)]
    for q in range(W):
        p = parts[q]
        gl = g_all[begins[q]:begins[q + 1]]
        want = spmm64(oracle, *p["local_T"], gl).astype(np.float64)
        mag = spmm64(oracle, *p["local_T"], np.abs(gl)).astype(np.float64)
        if sum(p["send_splits"]):
            got_rows = np.concatenate([back[r][sum(parts[r]["recv_splits"][:q]):sum(parts[r]["recv_splits"][:q + 1])]
                                       for r in range(W)])
            if is_pre:
                want = spmm64(oracle, *p["to_T"], got_rows, base=want.astype(np.float32)).astype(np.float64)
                mag = spmm64(oracle, *p["to_T"], np.abs(got_rows), base=mag.astype(np.float32)).astype(np.float64)
            else:
                np.add.at(want, p["send_idx"], got_rows.astype(np.float64))
                np.add.at(mag, p["send_idx"], np.abs(got_rows).astype(np.float64))
        if not close(p["grad"], want, mag):
            fails.append(f"{tag} backward rank {q}")
    # ---- the remote-gradient rows themselves: A_remote^T g
    for r in range(W):
        p = parts[r]
        if sum(p["recv_splits"]) == 0:
            continue
        rp, c = p["remote"]
        R = sum(p["recv_splits"])
        gl = g_all[begins[r]:begins[r + 1]]
        dense_rows = np.repeat(np.arange(len(rp) - 1), np.diff(rp))
        want = np.zeros((R, F), np.float64)
        np.add.at(want, c.astype(np.int64), gl[dense_rows].astype(np.float64))
        mag = np.zeros((R, F), np.float64)
        np.add.at(mag, c.astype(np.int64), np.abs(gl[dense_rows]).astype(np.float64))
        if not close(p["remote_grad_rows"], want, mag):
            fails.append(f"{tag} remote gradient rows rank {r}")
    # ---- fp32 exchange: the partitioned result is the single-graph A x and A^T g
    if bits == 32:
        src, dst = edges
        n = begins[-1]
        out_all = np.concatenate([p["out"] for p in parts])
        grad_all = np.concatenate([p["grad"] for p in parts])
        for name, got, rows_i, cols_i, dense in (("A x", out_all, dst, src, x_all), ("A^T g", grad_all, src, dst, g_all)):
            want = np.zeros((n, F), np.float64)
            np.add.at(want, rows_i, dense[cols_i].astype(np.float64))
            mag = np.zeros((n, F), np.float64)
            np.add.at(mag, rows_i, np.abs(dense[cols_i]).astype(np.float64))
            if not close(got, want, mag):
                fails.append(f"{tag} single-graph {name}")
    return fails


if __name__ == "__main__":
    main()
