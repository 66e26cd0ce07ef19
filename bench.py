"""Benchmark of the full-batch GraphSAGE hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` times K training steps
("epochs": forward + backward + Adam over the whole graph, the interval the
reference prints, examples/graphsage/train.py:135-141) on N GPUs of one node
and prints ONE JSON line on rank 0.

Workload: the single-GPU GraphSAGE configuration of the baseline — R-MAT
(0.57, 0.19, 0.19, 0.05), 2.4 M nodes, 62 M undirected edges symmetrised and
de-duplicated, features 2.4 M x 100 fp32, hidden 256, 47 classes, 10 % train
mask, dropout 0.5, 3 layers, seed 2 — generated on the device (synthetic
stand-in for ogbn-products).  With N > 1 the same graph is randomly relabelled
and split into N contiguous node ranges, one per GPU (strong scaling), and the
boundary rows are exchanged at ``--bits`` bits per value (default 2, the
reference's int2 mode; 32 = fp32).

``--impl reference`` times the reference's CPU implementation of the same step
on this box's host cores (rank 0 only), on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


_ARGV_REFERENCE = "--impl" in sys.argv and "reference" in sys.argv
if _ARGV_REFERENCE:
    # the CPU arm uses every host thread it may (torchrun defaults OMP_NUM_THREADS to 1)
    os.environ["OMP_NUM_THREADS"] = str(_host_threads())
else:
    os.environ.setdefault("OMP_NUM_THREADS", str(_host_threads()))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

WORKLOADS = {
    # the single-GPU configuration the headline metric is quoted on (default; strong scaling of it for N > 1)
    "rmat-2.4M": dict(name="graphsage-rmat-2.4M", kind="rmat-global", nodes=2_400_000, undirected_edges=62_000_000,
                      rmat=(0.57, 0.19, 0.19, 0.05), in_channels=100, hidden_channels=256, out_channels=47,
                      num_layers=3, dropout=0.5, train_fraction=0.10, lr=0.01, seed=2),
    # 8-GPU pre/post-aggregation configuration: stochastic block model, 8 blocks, 200 M directed edges, 90 % inside
    # a block, block b on rank b * ranks / 8; every rank generates its own blocks
    "sbm-10M": dict(name="graphsage-sbm-10M", kind="sbm", nodes=10_000_000, blocks=8, undirected_edges=100_000_000,
                    intra_fraction=0.9, in_channels=128, hidden_channels=256, out_channels=100, num_layers=3,
                    dropout=0.5, train_fraction=0.10, lr=0.01, seed=3),
    # large scaling-sweep configuration: R-MAT, random relabel, contiguous ranges, 14.4 directed edges per node
    # (111 M nodes / 1.6 B edges at full size; --nodes picks the size); every rank walks the edge stream itself
    "rmat-large": dict(name="graphsage-rmat-large", kind="rmat-stream", nodes=111_000_000, edges_per_node=14.4,
                       rmat=(0.57, 0.19, 0.19, 0.05), in_channels=128, hidden_channels=256, out_channels=172,
                       num_layers=3, dropout=0.5, train_fraction=0.01, lr=0.01, seed=4),
}
WORKLOAD = WORKLOADS["rmat-2.4M"]  # replaced in main() by the --workload choice
METRIC = "graphsage_epoch_time"
UNIT = "s"
# DRAM bytes (read + write) of one SpMM launch on the full-size single-GPU workload, by operand width, from a
# one-pass ncu capture (dram__bytes_read.sum + dram__bytes_write.sum) of this same command.  Only valid for
# --scale 1 on one GPU.
# Keyed by node order, then width (the average of the forward and the transposed launch where both exist).
SPMM_DRAM_TRAFFIC_BYTES = {"generated": {100: 15.15e9, 256: 52.1e9},
                           "degree": {48: 5.70e9, 100: 14.71e9, 256: 52.73e9}}


# ---------------------------------------------------------------------------
# algorithmic bytes (per launch) used for the roofline fractions
# ---------------------------------------------------------------------------
def spmm_bytes(info) -> float:
    """(M+1)*8 rowptr + nnz*(4 col [+4 val]) + nnz*N*4 gathered rows + M*N*4*(1 + accumulate) output."""
    M, N, nnz = info["M"], info["N"], info["nnz"]
    return (M + 1) * 8 + nnz * (4 + (4 if info["has_val"] else 0)) + nnz * N * 4 + M * N * 4 * (1 + (1 if info["acc"] else 0))


def spmm_dequant_bytes(info) -> float:
    """Gather of one packed row (N bytes: the row-group layout stores one byte per feature per group,
    whatever the bit width) + 8 B of params per nonzero, output read + written."""
    M, N, nnz = info["M"], info["N"], info["nnz"]
    return (M + 1) * 8 + nnz * (4 + (4 if info["has_val"] else 0)) + nnz * (N + 4) + M * N * 4 * 2


def rc_bytes_of(M, F, nnz, bits) -> float:
    """Fused dequantise-SpMM on row codes: F*bits/8 code bytes + 4 B of bf16 parameters + 4 B column index per
    nonzero, output read + written."""
    return (M + 1) * 8 + nnz * (F * bits // 8 + 8) + M * F * 4 * 2


def quant_bytes(S, F, bits, bf16=True) -> float:
    return S * F * 4 + S * F * bits / 8 + S * 8 + (S * 4 if bf16 else 0)


# ---------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.path = f"/tmp/sgnn_clocks_{os.getpid()}.csv"
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# workload construction (device side)
# ---------------------------------------------------------------------------
def scaled(v: int, scale: float) -> int:
    return max(64, int(round(v * scale)))


# Node numbering of the synthetic graphs: "degree" = every partition's nodes renumbered by ascending in-degree
# (data_manager.order_nodes_by_degree: a preprocessing step, the graph and the partition are unchanged);
# "generated" = the ids the generator produced.  --node-order sets it, both arms use it.
NODE_ORDER = "degree"
NODE_ORDER_TEXT = {"degree": "ascending in-degree within each partition (preprocessing)", "generated": "as generated"}

HOST_INPUT_LIMIT_BYTES = 16 << 30  # pinned host bytes over all ranks of the box: beyond this the node data is
#                                     generated on the device and no end-to-end leg is run


def workload_size(scale: float, nodes=None):
    """(nodes, generated undirected pairs) of the chosen workload."""
    w = WORKLOAD
    n = int(nodes) if nodes else scaled(w["nodes"], scale)
    if w["kind"] == "rmat-stream":
        return n, int(n * w["edges_per_node"] / 2)
    if w["kind"] == "sbm":
        n = n // w["blocks"] * w["blocks"]
        return n, int(w["undirected_edges"] * (n / w["nodes"]))
    return n, scaled(w["undirected_edges"], scale) if not nodes else int(w["undirected_edges"] * (n / w["nodes"]))


def build_workload(scale: float, rank: int, world: int, bits: int, device, pre: bool = False, nodes=None):
    from super_gnn_b200 import synthetic, workloads
    from super_gnn_b200.data_manager import (build_distributed_graph, build_distributed_graph_pre_post,
                                             partition_edges)

    w = WORKLOAD
    n, e = workload_size(scale, nodes)
    max_feat = max(w["in_channels"], w["hidden_channels"], w["out_channels"])
    if w["kind"] == "rmat-global":  # one edge list per rank (2.4 M nodes: small), then this rank's share of it
        a, b, c, d = w["rmat"]
        s, t = synthetic.rmat_edges(n, e, a, b, c, d, seed=w["seed"], device=device)
        s, t = synthetic.symmetrize_dedup(s, t, n)
        nnz_total = int(s.numel())
        if world > 1:
            s, t = synthetic.random_relabel(s, t, n, seed=w["seed"])
            begins = synthetic.even_ranges(n, world)
            local_edges, remote_edges = partition_edges(s, t, begins, rank)
        else:
            begins = [0, n]
            local_edges = torch.stack([s, t])
            remote_edges = torch.zeros((2, 0), dtype=torch.int64, device=device)
        del s, t
    else:  # partition-parallel: no rank ever holds the global edge list
        if w["kind"] == "sbm":
            local_edges, remote_edges, begins = workloads.sbm_partition(w["blocks"], n // w["blocks"], e,
                                                                        w["intra_fraction"], rank, world, w["seed"], device)
        else:
            local_edges, remote_edges, begins = workloads.rmat_partition(n, e, rank, world, w["seed"], device, w["rmat"],
                                                                         relabel=world > 1)
        cnt = torch.tensor([local_edges.size(1) + remote_edges.size(1)], dtype=torch.int64, device=device)
        if world > 1:
            dist.all_reduce(cnt)
        nnz_total = int(cnt.item())
    if NODE_ORDER == "degree":
        from super_gnn_b200.data_manager import order_nodes_by_degree

        local_edges, remote_edges, _ = order_nodes_by_degree(local_edges, remote_edges, begins)
    torch.cuda.empty_cache()
    build = build_distributed_graph_pre_post if (pre and world > 1) else build_distributed_graph
    graph = build(local_edges, remote_edges, begins, max_feat, bits, device=device)
    graph.set_fold_mean(True)  # the 1/in_degree of the mean aggregation is applied inside the SpMM kernels
    del local_edges, remote_edges
    n_local = begins[rank + 1] - begins[rank]
    host_bytes = n_local * (w["in_channels"] * 4 + 9)
    if host_bytes * world <= HOST_INPUT_LIMIT_BYTES:
        # node data of this rank, kept in pinned host memory (the end-to-end leg copies it every step)
        g = torch.Generator().manual_seed(w["seed"] * 1000 + rank)
        feats = torch.randn(n_local, w["in_channels"], generator=g).pin_memory()
        labels = torch.randint(0, w["out_channels"], (n_local,), generator=g).pin_memory()
        mask = (torch.rand(n_local, generator=g) < w["train_fraction"]).pin_memory()
    else:  # too large to stage through pinned host memory on every rank of one box: generated where it is used
        g = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + rank)
        feats = torch.randn(n_local, w["in_channels"], generator=g, device=device)
        labels = torch.randint(0, w["out_channels"], (n_local,), generator=g, device=device)
        mask = torch.rand(n_local, generator=g, device=device) < w["train_fraction"]
    torch.cuda.empty_cache()
    return graph, feats, labels, mask, n, nnz_total


def memory_table(nodes=None, hbm_bytes: float = 183_359 * 2 ** 20, headroom: float = 0.92):
    """Per (GPU count, boundary bits): modelled device bytes per rank of the chosen workload and whether they fit
    one B200 (``headroom`` of its memory: the caching allocator and the CUDA context need the rest).  Boundary
    rows are taken at their upper bound for a random partition (``workloads.rmat_boundary_estimate``)."""
    from super_gnn_b200 import workloads

    w = WORKLOAD
    n, pairs = workload_size(1.0, nodes)
    directed = 2 * pairs
    rows = []
    for world in (1, 2, 4, 8):
        for bits in (32, 8, 2):
            if world == 1 and bits != 32:
                continue
            if w["kind"] == "sbm":  # 10 % of the edges cross blocks; a rank's share of them, sources mostly distinct
                remote = int(directed * (1 - w["intra_fraction"]) / world) if world > 1 else 0
                recv = send = remote
            else:
                remote, recv, send = workloads.rmat_boundary_estimate(n, directed, world)
            m = workloads.step_memory_bytes(n // world, directed // world - remote, remote, recv, send, w["in_channels"],
                                            w["hidden_channels"], w["out_channels"], bits, world, chunks=world - 1)
            rows.append(dict(gpus=world, bits=bits, nodes_per_rank=n // world, gb={k: round(v / 1e9, 1) for k, v in m.items()},
                             fits=bool(m["total"] <= hbm_bytes * headroom)))
    return dict(workload=w["name"], nodes=n, directed_edges=directed, hbm_gb=round(hbm_bytes / 1e9, 1), headroom=headroom,
                cells=rows)


def make_model(bits: int, device, pre: bool = False):
    from super_gnn_b200 import graphsage

    w = WORKLOAD
    torch.manual_seed(w["seed"])
    cfg = dict(in_channels=w["in_channels"], hidden_channels=w["hidden_channels"], out_channels=w["out_channels"],
               num_layers=w["num_layers"], dropout=w["dropout"], num_bits=bits, is_pre_delay=pre,
               norm_type="LayerNorm", lr=w["lr"])
    return graphsage.create_model_and_optimizer(cfg, device=device)


# ---------------------------------------------------------------------------
# CPU arm: the reference's implementation of the step on the host cores
# ---------------------------------------------------------------------------
def host_memory_available_bytes() -> int:
    """Host memory this process may still use: the smaller of what the kernel reports as available and what the
    control group allows."""
    avail = None
    try:
        import psutil

        avail = int(psutil.virtual_memory().available)
    except Exception:
        pass
    for path, used_path in (("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory.current"),
                            ("/sys/fs/cgroup/memory/memory.limit_in_bytes", "/sys/fs/cgroup/memory/memory.usage_in_bytes")):
        try:
            limit = open(path).read().strip()
            if limit != "max":
                left = int(limit) - int(open(used_path).read().strip())
                avail = left if avail is None else min(avail, left)
        except (OSError, ValueError):
            pass
    return avail if avail is not None else 0


# host bytes the CPU step of the single-GPU configuration needs at full size (about twenty [nodes, hidden]
# activations and their gradients, the int64 graph in both orientations, the features), with a margin
CPU_FULL_SIZE_HOST_BYTES = 72 << 30


def cpu_epoch_baseline(steps: int, warmup: int, target_step_seconds, full_size: bool = False, scale: float = 1.0):
    """Times the reference's CPU training step.  ``full_size``: on the stated configuration itself (falling back to
    the largest power-of-two fraction of it that the host memory takes, and saying so); otherwise on a down-scaled
    graph of the same family chosen so that a step takes about ``target_step_seconds`` (the bounded sample the
    GPU arm reports beside its own number).  Returns (seconds per epoch of the stated size, description); the
    value is measured / fraction, and fraction == 1 means it is a plain measurement."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_graphsage as cg
    from super_gnn_b200 import synthetic

    w = WORKLOAD
    T = _host_threads()
    torch.set_num_threads(T)
    kind, spmm_fn = cg.load_backend(prefer_reference=True)
    if kind == "reference":
        import ctypes

        try:  # the compiled reference sizes its row split by its own OpenMP runtime
            T_omp = int(ctypes.CDLL("libgomp.so.1").omp_get_max_threads())
        except OSError:
            T_omp = T
    else:
        T_omp = T
    cg.CpuAggregator.spmm = spmm_fn

    gen_device = "cuda" if torch.cuda.is_available() else "cpu"  # set-up only: the timed step runs on the host

    def build(frac):
        n, e = scaled(w["nodes"], frac), scaled(w["undirected_edges"], frac)
        s, t = synthetic.rmat_edges(n, e, *w["rmat"], seed=w["seed"], device=gen_device)
        s, t = synthetic.symmetrize_dedup(s, t, n)  # sorted by (destination, source)
        if NODE_ORDER == "degree":  # the same renumbering as the GPU arm's
            from super_gnn_b200.data_manager import order_nodes_by_degree

            le, _, _ = order_nodes_by_degree(torch.stack([s, t]), torch.zeros((2, 0), dtype=torch.int64, device=s.device),
                                             [0, n])
            key = torch.sort(le[1] * n + le[0])[0]
            s, t = key % n, key // n
            del le, key
        s, t = s.cpu(), t.cpu()
        if gen_device == "cuda":
            torch.cuda.empty_cache()
        rowptr = torch.zeros(n + 1, dtype=torch.int64)
        torch.cumsum(torch.bincount(t, minlength=n), 0, out=rowptr[1:])
        graph = cg.CpuGraph(rowptr, s, n, T_omp)
        g = torch.Generator().manual_seed(w["seed"])
        feats = torch.randn(n, w["in_channels"], generator=g)
        labels = torch.randint(0, w["out_channels"], (n,), generator=g)
        mask = torch.rand(n, generator=g) < w["train_fraction"]
        torch.manual_seed(w["seed"])
        model = cg.CpuSAGE(w["in_channels"], w["hidden_channels"], w["out_channels"], w["num_layers"], w["dropout"])
        opt = torch.optim.Adam(model.parameters(), lr=w["lr"])
        return graph, feats, labels, mask, model, opt, n, int(s.numel())

    def one_step(state):
        graph, feats, labels, mask, model, opt = state[:6]
        t0 = time.perf_counter()
        cg.train_step(model, graph, feats, labels, mask, opt, float(mask.sum()))
        return time.perf_counter() - t0

    if full_size:
        frac = min(1.0, float(scale))  # --scale below 1 is a debugging aid; the line then says so
        have = host_memory_available_bytes()
        while frac > 1.0 / 64 and have and CPU_FULL_SIZE_HOST_BYTES * frac > have:
            frac /= 2
        state = build(frac)
    else:
        # probe at 1/64 of the size, then pick the largest power-of-two fraction within the time target
        probe = build(1.0 / 64)
        one_step(probe)
        t_probe = one_step(probe)
        frac = 1.0 / 64
        while frac < 1.0 and t_probe * (frac * 2 * 64) <= target_step_seconds:
            frac *= 2
        state = probe if frac == 1.0 / 64 else build(frac)
        del probe
    for _ in range(warmup):
        one_step(state)
    times = [one_step(state) for _ in range(steps)]
    mean = sum(times) / len(times)
    what = ("the stated configuration at full size" if frac == 1.0 else
            f"same R-MAT family at {frac:g} of the nodes and edges")
    desc = dict(kind=kind, cores=T, unit=UNIT,
                sample=(f"{what} ({state[6]} nodes, {state[7]} directed edges), full training step (fwd+bwd+Adam) on "
                        f"the host; {len(times)} steps after {warmup} warm-up, mean {mean:.3f} s, best {min(times):.3f} s"
                        + ("" if frac == 1.0 else f"; value = mean / {frac:g} (extrapolated, not measured at full size)")),
                fraction=frac, measured_s=mean, nodes=state[6], directed_edges=state[7], steps_timed=len(times),
                warmup_steps=warmup)
    return mean / frac, desc


def cpu_op_baselines():
    """The reference's own CPU ops on the two kernel configurations (SpMM configuration 1; quantise / dequantise
    configuration 2), all host threads, best of a few runs after a warm-up: the figures the `kernels` object of the
    GPU arm is to be read against.  Uses the compiled reference ops when they could be built on this host, else
    the C restatement (single thread for the quantiser)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cpu_graphsage as cg
    import oracle as port
    from super_gnn_b200 import synthetic

    T = _host_threads()
    torch.set_num_threads(T)
    out = {"threads": T}

    def best(fn, reps=4):
        fn()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts) * 1e3

    kind, spmm_fn = cg.load_backend(prefer_reference=True)
    T_omp = T
    if kind == "reference":
        import ctypes

        try:
            T_omp = int(ctypes.CDLL("libgomp.so.1").omp_get_max_threads())
        except OSError:
            pass
    n, N = 200_000, 128
    rowptr, col, val = synthetic.poisson_csr(n, n, 12.0, seed=0, device="cpu")
    csr = cg.make_csr(rowptr, col, T_omp)
    csr["val"] = val.contiguous()
    X = torch.randn(n, N)
    Y = torch.zeros(n, N)
    out["spmm_cfg1"] = dict(ms=best(lambda: spmm_fn(csr, X, Y)), kind=kind, nnz=int(col.numel()))
    del X, Y, csr

    S, F = 500_000, 256
    x = synthetic.scaled_features(S, F, seed=1, device="cpu")
    ref = None
    try:
        import build_ref

        ref = build_ref.load()
    except Exception:
        ref = None
    for bits in (8, 4, 2):
        epb = 8 // bits
        if ref is not None:
            q = torch.empty(((S + epb - 1) // epb) * F, dtype=torch.uint8)
            d = torch.empty(S, F)
            state = {}

            def quant():
                mn, mx = torch.aminmax(x, dim=1)
                sc = (mx - mn) / float(2 ** bits - 1)
                sc[sc == 0] = 1.0
                state["mn"], state["sc"] = mn.contiguous(), sc.contiguous()
                ref.quantize_tensor(x, q, state["mn"], state["sc"], bits)

            out[f"quantize_cfg2_{bits}bit"] = dict(ms=best(quant), kind="reference",
                                                  note="torch aminmax + reference quantize_tensor (x86 form)")
            out[f"dequantize_cfg2_{bits}bit"] = dict(
                ms=best(lambda: ref.dequantize_tensor(q, d, state["mn"], state["sc"], bits)), kind="reference")
        else:
            xn = x.numpy()
            wr = np.array([0, S], np.int32)
            res = {}

            def quant_port():
                res["q"], res["p"] = port.quantize_for_all_procs(xn, wr, bits)

            out[f"quantize_cfg2_{bits}bit"] = dict(ms=best(quant_port, 2), kind="port", note="one thread")
            out[f"dequantize_cfg2_{bits}bit"] = dict(
                ms=best(lambda: port.dequantize_for_all_procs(res["q"], res["p"], wr, bits), 2), kind="port")
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    # A CPU step of the stated configuration takes about 20 s: the run times at most 3 of them after 1 warm-up
    # (a true number on the stated size, inside a few minutes) however many GPU steps were asked for.
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    value, desc = cpu_epoch_baseline(steps, warmup, None, full_size=True, scale=args.scale)
    frac = desc["fraction"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": value * 1e3, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "nodes": desc["nodes"], "directed_edges": desc["directed_edges"],
                   "features": WORKLOAD["in_channels"], "hidden": WORKLOAD["hidden_channels"],
                   "classes": WORKLOAD["out_channels"], "layers": WORKLOAD["num_layers"], "dropout": WORKLOAD["dropout"],
                   "norm": "LayerNorm", "optimizer": "Adam", "node_order": NODE_ORDER_TEXT[NODE_ORDER], "scale": frac,
                   "note": ("CPU arm: single process, all host threads, the stated configuration at full size"
                            if frac == 1.0 else
                            f"CPU arm: {'--scale was given' if args.scale < 1.0 else 'the host memory did not take the full size'}"
                            f"; ran {frac:g} of it (nodes and edges above are those of the run) and value = measured / "
                            f"{frac:g}")},
        "cpu_baseline": dict(value=value, **desc),
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ---------------------------------------------------------------------------
# kernel micro-benchmarks (N = 1 only): SpMM and quantise-pack vs the HBM roofline
# ---------------------------------------------------------------------------
def flush_l2(buf):
    buf.add_(1)


def time_kernel(fn, iters, flush_buf):
    times = []
    for _ in range(iters):
        flush_l2(flush_buf)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e) * 1e-3)
    times.sort()
    return times[len(times) // 2], times[0]


def kernel_benchmarks(device, peak_gbs, sections=("spmm_cfg1", "remote", "remote_large", "quant_cfg2", "gemm")):
    from super_gnn_b200 import supergnn_ops as ops
    from super_gnn_b200 import synthetic

    out = {}
    flush_buf = torch.zeros(64 * 1024 * 1024, dtype=torch.float32, device=device)  # 256 MB > L2
    if "spmm_cfg1" in sections:
        # SpMM, configuration 1: 200k x 200k Poisson(12), values 1/deg, X 200k x 128
        n, N = 200_000, 128
        rowptr, col, val = synthetic.poisson_csr(n, n, 12.0, seed=0, device=device)
        X = torch.randn(n, N, device=device)
        Y = torch.empty(n, N, device=device)
        nnz = col.numel()
        info = dict(M=n, N=N, nnz=nnz, has_val=True, acc=False)
        for name, algo in (("row_split", ops.SPMM_ROW_SPLIT), ("nnz_split", ops.SPMM_NNZ_SPLIT)):
            fn = lambda: ops.spmm(rowptr, col, val, X, Y, n, None, None, algo=algo, accumulate=False)  # noqa: E731
            for _ in range(3):
                fn()
            med, best = time_kernel(fn, 20, flush_buf)
            b = spmm_bytes(info)
            out[f"spmm_cfg1_{name}"] = dict(ms=med * 1e3, best_ms=best * 1e3, gather_model_gbs=b / med / 1e9,
                                            geps=nnz / med / 1e9, frac_of_measured_peak=b / med / 1e9 / peak_gbs,
                                            compulsory_gbs=((n + 1) * 8 + nnz * 8 + 2 * n * N * 4) / med / 1e9)
        del X, Y, rowptr, col, val
    if "remote" in sections:
        # remote aggregation of one rank of an 8-way partition: 300k destination rows, 800k received rows from 8 peers,
        # 12.7 M nonzeros, F = 256: fused dequantise-SpMM on the 2-bit wire format vs the fp32 SpMM on materialised rows
        M, R, F, P, nnz_r = 300_000, 800_000, 256, 8, 12_700_000
        g = torch.Generator(device=device).manual_seed(7)
        rows = torch.randint(0, M, (nnz_r,), generator=g, device=device)
        rp = torch.zeros(M + 1, dtype=torch.int64, device=device)
        torch.cumsum(torch.bincount(rows, minlength=M), 0, out=rp[1:])
        cl = torch.randint(0, R, (nnz_r,), generator=g, device=device, dtype=torch.int64).to(torch.int32)
        xr = torch.randn(R, F, generator=g, device=device)
        wr = torch.tensor([R * p // P for p in range(P + 1)], dtype=torch.int32, device=device)
        pk = torch.empty((R // 4 + P, F), dtype=torch.uint8, device=device)
        p16 = torch.empty((R, 2), dtype=torch.bfloat16, device=device)
        ops.quant_pack_rows(xr, None, wr, P, 2, pk, params_bf16=p16)
        Yr = torch.zeros(M, F, device=device)
        ff = lambda: ops.spmm_dequant(rp, cl, None, pk, p16, wr, P, 2, Yr, M, algo=ops.SPMM_ROW_SPLIT)  # noqa: E731
        fd = lambda: ops.spmm(rp, cl, None, xr, Yr, M, None, None, algo=ops.SPMM_ROW_SPLIT)  # noqa: E731
        fn2 = lambda: ops.spmm_dequant(rp, cl, None, pk, p16, wr, P, 2, Yr, M, algo=ops.SPMM_NNZ_SPLIT)  # noqa: E731
        # the same rows in the row-codes layout: a gathered row costs F*bits/8 bytes
        rc = torch.empty((R, F * 2 // 8), dtype=torch.uint8, device=device)
        ops.quant_pack_rowcodes(xr, None, 2, rc, params_bf16=p16)
        frc = lambda: ops.spmm_dequant_rowcodes(rp, cl, None, rc, p16, 2, Yr, M, algo=ops.SPMM_ROW_SPLIT)  # noqa: E731
        frc2 = lambda: ops.spmm_dequant_rowcodes(rp, cl, None, rc, p16, 2, Yr, M, algo=ops.SPMM_NNZ_SPLIT)  # noqa: E731
        rc_bytes = rc_bytes_of(M, F, nnz_r, 2)
        for name, fn, byts in (("spmm_dequant_rowcodes_2bit_remote", frc, rc_bytes),
                               ("spmm_dequant_rowcodes_2bit_remote_nnz_split", frc2, rc_bytes),
                               ("spmm_dequant_2bit_remote_nnz_split", fn2, spmm_dequant_bytes(dict(M=M, N=F, nnz=nnz_r, has_val=False))),
                               ("spmm_dequant_2bit_remote", ff, spmm_dequant_bytes(dict(M=M, N=F, nnz=nnz_r, has_val=False))),
                               ("spmm_fp32_remote", fd, spmm_bytes(dict(M=M, N=F, nnz=nnz_r, has_val=False, acc=True)))):
            for _ in range(3):
                fn()
            med, _ = time_kernel(fn, 10, flush_buf)
            out[name] = dict(ms=med * 1e3, geps=nnz_r / med / 1e9, algorithmic_gbs=byts / med / 1e9)
        # boundary-row gather and scatter-add: 800k rows of 256 floats picked from 300k nodes
        idx = torch.randint(0, M, (R,), generator=g, device=device)
        feats = torch.randn(M, F, generator=g, device=device)
        fg = lambda: ops.gather_rows(feats, idx, xr)  # noqa: E731
        fs = lambda: ops.scatter_add_rows(xr, idx, Yr)  # noqa: E731
        for name, fn in (("gather_rows_800k", fg), ("scatter_add_rows_800k", fs)):
            for _ in range(3):
                fn()
            med, _ = time_kernel(fn, 10, flush_buf)
            b = 2.0 * R * F * 4 + R * 8
            out[name] = dict(ms=med * 1e3, gbs=b / med / 1e9, frac_of_measured_peak=b / med / 1e9 / peak_gbs)
        del rows, rp, cl, xr, pk, p16, Yr, idx, feats
    if "remote_large" in sections:
        # the same remote aggregation at the scale of a 10 M-node rank of the large sweep, where the received rows no
        # longer fit L2: 1.5 M destination rows, 8 M received rows (512 MB of 2-bit codes), 60 M nonzeros, F = 256;
        # codes and parameters are random bytes (the kernels' work does not depend on their values)
        M, R, F, P, nnz_r = 1_500_000, 8_000_000, 256, 8, 60_000_000
        g = torch.Generator(device=device).manual_seed(8)
        rows = torch.randint(0, M, (nnz_r,), generator=g, device=device)
        rp = torch.zeros(M + 1, dtype=torch.int64, device=device)
        torch.cumsum(torch.bincount(rows, minlength=M), 0, out=rp[1:])
        del rows
        cl = torch.randint(0, R, (nnz_r,), generator=g, device=device, dtype=torch.int64).to(torch.int32)
        wr = torch.tensor([R * p // P for p in range(P + 1)], dtype=torch.int32, device=device)
        p16 = (torch.rand((R, 2), generator=g, device=device) + 0.5).to(torch.bfloat16)
        Yr = torch.zeros(M, F, device=device)
        rc = torch.randint(0, 256, (R, F * 2 // 8), generator=g, device=device, dtype=torch.uint8)
        pk = torch.randint(0, 256, (R // 4 + P, F), generator=g, device=device, dtype=torch.uint8)
        cases = (("spmm_dequant_rowcodes_2bit_remote_large", rc_bytes_of(M, F, nnz_r, 2),
                  lambda: ops.spmm_dequant_rowcodes(rp, cl, None, rc, p16, 2, Yr, M, algo=ops.SPMM_NNZ_SPLIT)),
                 ("spmm_dequant_2bit_remote_large", spmm_dequant_bytes(dict(M=M, N=F, nnz=nnz_r, has_val=False)),
                  lambda: ops.spmm_dequant(rp, cl, None, pk, p16, wr, P, 2, Yr, M, algo=ops.SPMM_NNZ_SPLIT)))
        for name, byts, fn in cases:
            for _ in range(2):
                fn()
            med, _ = time_kernel(fn, 6, flush_buf)
            out[name] = dict(ms=med * 1e3, geps=nnz_r / med / 1e9, algorithmic_gbs=byts / med / 1e9,
                             frac_of_measured_peak=byts / med / 1e9 / peak_gbs)
        del rp, cl, p16, Yr, rc, pk
    if "quant_cfg2" in sections:
        # quantise-pack and unpack-dequantise, configuration 2: 500k x 256, row scale LogNormal(0,1)
        S, F = 500_000, 256
        x = synthetic.scaled_features(S, F, seed=1, device=device)
        wr = torch.tensor([0, S], dtype=torch.int32, device=device)
        params = torch.empty(S, 2, device=device)
        back = torch.empty_like(x)
        for bits in (8, 4, 2):
            packed = torch.empty((S // (8 // bits), F), dtype=torch.uint8, device=device)
            fq = lambda: ops.quantize_tensor_for_all_procs(x, packed, params, wr, 1, bits)  # noqa: E731
            fd = lambda: ops.dequantize_tensor_for_all_procs(packed, back, params, wr, 1, bits)  # noqa: E731
            for _ in range(3):
                fq()
                fd()
            mq, _ = time_kernel(fq, 20, flush_buf)
            md, _ = time_kernel(fd, 20, flush_buf)
            bq = quant_bytes(S, F, bits, bf16=False)
            out[f"quant_pack_cfg2_{bits}bit"] = dict(ms=mq * 1e3, gbs=bq / mq / 1e9, frac_of_measured_peak=bq / mq / 1e9 / peak_gbs,
                                                     frac_of_nominal_8tbs=bq / mq / 1e9 / 8000.0)
            out[f"unpack_dequant_cfg2_{bits}bit"] = dict(ms=md * 1e3, gbs=bq / md / 1e9, frac_of_measured_peak=bq / md / 1e9 / peak_gbs,
                                                        frac_of_nominal_8tbs=bq / md / 1e9 / 8000.0)
            codes = torch.empty((S, F * bits // 8), dtype=torch.uint8, device=device)
            fq2 = lambda: ops.quant_pack_rowcodes(x, None, bits, codes, params=params)  # noqa: E731
            fd2 = lambda: ops.unpack_dequant_rowcodes(codes, back, params, bits)  # noqa: E731
            for _ in range(3):
                fq2()
                fd2()
            mq, _ = time_kernel(fq2, 20, flush_buf)
            md, _ = time_kernel(fd2, 20, flush_buf)
            out[f"quant_pack_rowcodes_cfg2_{bits}bit"] = dict(ms=mq * 1e3, gbs=bq / mq / 1e9, frac_of_measured_peak=bq / mq / 1e9 / peak_gbs,
                                                              frac_of_nominal_8tbs=bq / mq / 1e9 / 8000.0)
            out[f"unpack_dequant_rowcodes_cfg2_{bits}bit"] = dict(ms=md * 1e3, gbs=bq / md / 1e9, frac_of_measured_peak=bq / md / 1e9 / peak_gbs,
                                                                 frac_of_nominal_8tbs=bq / md / 1e9 / 8000.0)
            # the one-sided form of the same kernel with eight "peers" whose tables point at this GPU's own buffers
            # (what the per-row destination lookup costs; NVLink itself is not in this number)
            P8 = 8
            wr8 = torch.tensor([S * p // P8 for p in range(P8 + 1)], dtype=torch.int32, device=device)
            p16 = torch.empty((S, 2), dtype=torch.bfloat16, device=device)
            tab = lambda v: torch.tensor(v, dtype=torch.int64, device=device)  # noqa: E731
            tabs = (tab([codes.data_ptr()] * P8), tab([p16.data_ptr()] * P8), tab([S * p // P8 for p in range(P8)]))
            fq3 = lambda: ops.quant_pack_rowcodes_p2p(x, None, wr8, P8, bits, tabs)  # noqa: E731
            for _ in range(3):
                fq3()
            mq, _ = time_kernel(fq3, 20, flush_buf)
            out[f"quant_pack_rowcodes_p2p_local_tables_cfg2_{bits}bit"] = dict(
                ms=mq * 1e3, gbs=bq / mq / 1e9, frac_of_measured_peak=bq / mq / 1e9 / peak_gbs,
                frac_of_nominal_8tbs=bq / mq / 1e9 / 8000.0)
            del codes, p16
        del x, back, params, packed
    if "gemm" in sections:
        # dense fp32 GEMMs of one hidden layer at the full node count, beside the stock fp32 matmul (TF32 off)
        torch.backends.cuda.matmul.allow_tf32 = False
        bf16_peak = measured_peak_bf16_tflops()
        M, H = WORKLOAD["nodes"], WORKLOAD["hidden_channels"]
        a = torch.randn(M, H, device=device)
        w = torch.randn(H, H, device=device) * 0.05
        c = torch.empty(M, H, device=device)
        gw = torch.empty(H, H, device=device)
        cases = (("gemm_nt_nodes_x_hidden_x_hidden", lambda: ops.gemm_nt(a, w, out=c), lambda: torch.mm(a, w.t(), out=c)),
                 ("gemm_tn_hidden_x_hidden_over_nodes", lambda: ops.gemm_tn(c, a, out=gw), lambda: torch.mm(c.t(), a, out=gw)))
        for name, ours, stock in cases:
            for _ in range(3):
                ours()
                stock()
            mo, _ = time_kernel(ours, 10, flush_buf)
            ms_, _ = time_kernel(stock, 10, flush_buf)
            tf = 2.0 * M * H * H / mo / 1e12
            out[name] = dict(ms=mo * 1e3, fp32_equivalent_tflops=tf, bf16_mma_tflops=9 * tf,
                             frac_of_measured_bf16_peak_sustained=9 * tf / bf16_peak, stock_fp32_matmul_ms=ms_ * 1e3)
            if name.startswith("gemm_nt"):  # the same product with the three smallest of the nine cross products left out
                m6, _ = time_kernel(lambda: ops.gemm_nt(a, w, out=c, products=6), 10, flush_buf)
                out[name]["six_products_ms"] = m6 * 1e3
    if "node_order" in sections:
        # SpMM (mean aggregation, forward form) on the benchmark graph under different node numberings: which part of
        # a renumbering by degree helps (the order the rows are processed in, or the layout of x), and what a
        # breadth-first numbering does.  Not part of the default sections.
        w_ = WORKLOADS["rmat-2.4M"]
        n, e = w_["nodes"], w_["undirected_edges"]
        s0, t0 = synthetic.rmat_edges(n, e, *w_["rmat"], seed=w_["seed"], device=device)
        s0, t0 = synthetic.symmetrize_dedup(s0, t0, n)
        sr, tr = synthetic.random_relabel(s0, t0, n, seed=w_["seed"])
        deg = torch.bincount(tr, minlength=n)

        def ranks_of(order):  # order[new] = old  ->  new id of every old id
            r = torch.empty_like(order)
            r[order] = torch.arange(n, device=device)
            return r

        asc, desc = ranks_of(torch.argsort(deg, stable=True)), ranks_of(torch.argsort(deg, stable=True, descending=True))
        # breadth-first levels from the best-connected node (nodes never reached go last)
        key = torch.sort(tr * n + sr)[0]
        dst_sorted, src_sorted = key // n, key % n
        level = torch.full((n,), -1, dtype=torch.int64, device=device)
        level[torch.argmax(deg)] = 0
        depth = 0
        while True:
            nb = src_sorted[level[dst_sorted] == depth]
            nb = nb[level[nb] < 0]
            if nb.numel() == 0:
                break
            depth += 1
            level[nb] = depth
        level[level < 0] = depth + 1
        bfs = ranks_of(torch.argsort(level, stable=True))
        del key, dst_sorted, src_sorted, level
        numberings = (("generated", s0, t0), ("random", sr, tr), ("degree_ascending", asc[sr], asc[tr]),
                      ("degree_descending", desc[sr], desc[tr]), ("degree_ascending_rows_only", sr, asc[tr]),
                      ("degree_ascending_columns_only", asc[sr], tr), ("breadth_first_levels", bfs[sr], bfs[tr]))
        for tag, s_, t_ in numberings:
            key = torch.sort(t_ * n + s_)[0]
            col = (key % n).to(torch.int32)
            rowptr = torch.zeros(n + 1, dtype=torch.int64, device=device)
            torch.cumsum(torch.bincount(key // n, minlength=n), 0, out=rowptr[1:])
            del key
            inv_deg = (rowptr[1:] - rowptr[:-1]).clamp(min=1).float().reciprocal()
            for N in (256, 100, 48):
                X, Y = torch.randn(n, N, device=device), torch.empty(n, N, device=device)
                fn = lambda: ops.spmm(rowptr, col, None, X, Y, n, inv_deg, None, algo=ops.SPMM_NNZ_SPLIT,  # noqa: E731
                                      accumulate=False)
                for _ in range(3):
                    fn()
                med, best = time_kernel(fn, 8, flush_buf)
                out[f"node_order_{tag}_N{N}"] = dict(ms=med * 1e3, best_ms=best * 1e3)
                del X, Y
            del col, rowptr, inv_deg
    return out


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def measured_peak_bf16_tflops():
    """Sustained dense bf16 GEMM rate measured on this pool (the figure for a kernel timed inside a long step)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"])
    except (OSError, KeyError, ValueError):
        return 1400.0  # earlier measurement on this pool, used only when the file is absent


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def run_ours(args):
    from super_gnn_b200 import graphsage
    from super_gnn_b200 import supergnn_ops as ops
    from super_gnn_b200.communicator import Communicator
    from super_gnn_b200.quantizer import Quantizer_for_all_procs

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    world = int(os.environ.get("WORLD_SIZE", 1))
    bits = args.bits if args.bits is not None else (2 if world > 1 else 32)
    Communicator(bits, is_async=True)
    if world > 1:
        rank, world = Communicator.ctx.init_dist_group()
    else:
        rank = 0
        torch.cuda.set_device(0)
    device = torch.device("cuda", torch.cuda.current_device())
    Quantizer_for_all_procs(world, bits)

    if args.row_groups:
        Communicator.row_codes = False
    if args.by_peer != "auto":
        from super_gnn_b200.aggregator import Aggregator

        Aggregator.remote_gradient_by_peer = args.by_peer == "on"
    torch.cuda.reset_peak_memory_stats()
    graph, feats_h, labels_h, mask_h, n_total, nnz_total = build_workload(args.scale, rank, world, bits, device,
                                                                          pre=args.pre, nodes=args.nodes)
    host_inputs = not feats_h.is_cuda
    exchange = "nccl" if dist.is_initialized() and dist.get_backend() == "nccl" else "gloo (staged through host memory)"
    if world > 1 and args.exchange == "p2p" and bits in (2, 4, 8) and exchange == "nccl":
        try:
            Communicator.ctx.enable_peer_exchange(graph, max(WORKLOAD["in_channels"], WORKLOAD["hidden_channels"],
                                                             WORKLOAD["out_channels"]))
            exchange = "p2p"
        except Exception as e:  # symmetric memory cannot be set up here: the collectives carry the same bytes
            exchange = f"nccl (one-sided set-up failed: {type(e).__name__})"
    model, opt = make_model(bits, device, pre=args.pre)
    data = dict(graph=graph, nodes_features=feats_h.to(device), nodes_labels=labels_h.to(device),
                nodes_train_masks=mask_h.to(device))
    nt = torch.tensor([float(mask_h.sum())], device=device)
    if world > 1:
        dist.all_reduce(nt)
    num_train = float(nt.item())

    def step():
        return graphsage.train_step(model, data, opt, num_train)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # started before the warm-up: nvidia-smi needs a few hundred ms before its first sample
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    for _ in range(args.warmup):
        step()
    sync()
    # ---- timed region 1: inputs resident in HBM ----
    ops.LAUNCH_LOG = []
    launches0 = ops.LAUNCH_COUNT
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    ev0.record()
    for _ in range(args.steps):
        loss = step()
    ev1.record()
    sync()
    launches = ops.LAUNCH_COUNT - launches0
    log, ops.LAUNCH_LOG = ops.LAUNCH_LOG, None
    dev_s = ev0.elapsed_time(ev1) * 1e-3
    t = torch.tensor([dev_s], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_s = t.item() / args.steps
    loss_sum = loss.detach().clone()
    if world > 1:
        dist.all_reduce(loss_sum)  # every rank holds its share of the summed NLL / global count
    final_loss = float(loss_sum.item())

    # ---- timed region 2: end to end, host buffers in and the loss out, every step ----
    # Every step's inputs (features, labels, mask) are copied from pinned host memory; the copy of step k+1
    # runs on a side stream while step k computes (two device buffers), and the loss is read back each step.
    h2d = feats_h.numel() * 4 + labels_h.numel() * 8 + mask_h.numel()
    e2e_step_s = loss_host = None
    copy_stream = torch.cuda.Stream() if host_inputs else None
    if not host_inputs:
        h2d = 0
    if host_inputs:
        bufs = [dict(f=torch.empty_like(data["nodes_features"]), l=torch.empty_like(data["nodes_labels"]),
                     m=torch.empty_like(data["nodes_train_masks"]), ready=torch.cuda.Event(), free=torch.cuda.Event())
                for _ in range(2)]

        def upload(b):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(b["free"])  # the step that last used this buffer has finished with it
                b["f"].copy_(feats_h, non_blocking=True)
                b["l"].copy_(labels_h, non_blocking=True)
                b["m"].copy_(mask_h, non_blocking=True)
                b["ready"].record(copy_stream)

        for b in bufs:
            b["free"].record()
        sync()
        t0 = time.perf_counter()
        upload(bufs[0])
        for k in range(args.steps):
            b = bufs[k % 2]
            if k + 1 < args.steps:
                upload(bufs[(k + 1) % 2])
            torch.cuda.current_stream().wait_event(b["ready"])
            data["nodes_features"], data["nodes_labels"], data["nodes_train_masks"] = b["f"], b["l"], b["m"]
            loss_t = step()
            b["free"].record()
            loss_host = loss_t.item()  # device -> host read of the result
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        t = torch.tensor([e2e_s], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_step_s = t.item() / args.steps
    clocks = sampler.stop() if sampler is not None else None

    phases = None
    if args.phases:  # two extra steps with CUDA-event timing of the Aggregator's phases (not part of any reported time)
        from super_gnn_b200.time_recorder import TimeRecorder

        rec = TimeRecorder(0, 0, enabled=True)
        rec.set_mode("training")
        rec.set_epoch(0)
        for _ in range(2):
            step()
        recs = rec.get_records()
        phases = {name: sum(v[0]) / 2 for name, v in recs.items()}
        TimeRecorder(0, 0)

    # device memory high-water mark of the run (build + steps), the largest over the ranks
    mem = torch.tensor([torch.cuda.max_memory_allocated(), torch.cuda.max_memory_reserved()], dtype=torch.float64,
                       device=device)
    recv_rows = torch.tensor([float(sum(graph.comm_splits.recv_splits)) if world > 1 else 0.0,
                              float(sum(graph.comm_splits.send_splits)) if world > 1 else 0.0], device=device,
                             dtype=torch.float64)
    if world > 1:
        dist.all_reduce(mem, op=dist.ReduceOp.MAX)
        dist.all_reduce(recv_rows, op=dist.ReduceOp.MAX)
    if rank != 0:
        if world > 1:
            dist.barrier()
        return

    # ---- roofline of the dominant kernel from the launch log of region 1: the CSR SpMM over the hidden width
    #      (the widest and longest launches; the narrower SpMM launches are listed beside it) ----
    peak, peak_kind = measured_peak_gbs()
    per_kind = {}
    spmm_by_width = {}
    gemm_flops = gemm_t = 0.0
    for kind, info, s, e in log:
        ms = s.elapsed_time(e)
        k = per_kind.setdefault(kind, [0, 0.0])
        k[0] += 1
        k[1] += ms
        if kind == "spmm":
            w = spmm_by_width.setdefault(info["N"], [0, 0.0, 0.0])
            w[0] += 1
            w[1] += ms * 1e-3
            w[2] += spmm_bytes(info)
        elif kind in ("gemm_nt", "gemm_tn"):
            gemm_flops += 2.0 * info["M"] * info["N"] * info["K"]
            gemm_t += ms * 1e-3
    roofline = {"bound": "hbm", "kernel": None, "achieved": None, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": None, "traffic": None}
    if spmm_by_width:
        wide = max(spmm_by_width, key=lambda n: spmm_by_width[n][1])  # width with the largest total time
        n_l, tot_t, tot_b = spmm_by_width[wide]
        default_cfg = world == 1 and args.scale == 1.0 and args.workload == "rmat-2.4M" and not args.nodes
        traffic = SPMM_DRAM_TRAFFIC_BYTES[NODE_ORDER].get(wide) if default_cfg else None
        gather_model = tot_b / tot_t / 1e9
        traffic_gbs = (traffic * n_l / tot_t / 1e9) if traffic else None
        # `achieved` / `frac` are the DRAM bytes the launch really moves over the live launch time wherever that
        # traffic is known (the default single-GPU workload); the gather model charges every nonzero a full row,
        # most of which L2 serves on a skewed graph, so its rate exceeds the HBM peak and is not a fraction of it
        achieved = traffic_gbs if traffic_gbs is not None else gather_model
        roofline.update({
            "kernel": f"spmm_nnz_split_kernel, N = {wide} (sgnn_spmm_csr_f32)", "achieved": achieved,
            "achieved_is": ("DRAM traffic (read + write) per launch / live launch time" if traffic_gbs is not None else
                            "gather-model algorithmic bytes / live launch time (DRAM traffic of this workload not captured)"),
            "frac": achieved / peak, "frac_of_nominal_8tbs": achieved / 8000.0, "traffic": traffic,
            "traffic_source": ("stored constant: dram__bytes_read.sum + dram__bytes_write.sum of one launch from a "
                               "one-pass ncu capture of this command at full size "
                               "(profiles/spmm_nnz_split_rmat2.4M_dram.md); not re-measured in this run"
                               if traffic else None),
            "gather_model_gbs": gather_model, "gather_model_over_peak": gather_model / peak,
            "launches": n_l, "avg_launch_ms": tot_t / n_l * 1e3, "algorithmic_bytes_per_launch": tot_b / n_l,
            "time_share_of_step": (tot_t / args.steps) / step_s if step_s > 0 else None,
            "all_spmm_widths": {str(n): {"launches": v[0], "avg_launch_ms": v[1] / v[0] * 1e3,
                                         "algorithmic_gbs": v[2] / v[1] / 1e9} for n, v in sorted(spmm_by_width.items())},
        })
    gemm = None
    if gemm_t > 0:  # fp32-accurate GEMM: each fp32 multiply-add is nine bf16 tensor-core multiply-adds
        bf16_peak = measured_peak_bf16_tflops()
        tf = gemm_flops / gemm_t / 1e12
        gemm = {"bound": "tensor", "fp32_equivalent_tflops": tf, "bf16_mma_tflops": 9 * tf,
                "peak_bf16_tflops_sustained": bf16_peak,
                "frac": (9 * tf / bf16_peak) if bf16_peak else None,
                "time_share_of_step": (gemm_t / args.steps) / step_s if step_s > 0 else None}

    line = {
        "metric": METRIC, "value": step_s, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_s * 1e3, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], "nodes": n_total, "directed_edges": nnz_total,
                   "features": WORKLOAD["in_channels"], "hidden": WORKLOAD["hidden_channels"],
                   "classes": WORKLOAD["out_channels"], "layers": WORKLOAD["num_layers"], "dropout": WORKLOAD["dropout"],
                   "norm": "LayerNorm", "optimizer": "Adam", "node_order": NODE_ORDER_TEXT[NODE_ORDER],
                   "boundary_bits": bits if world > 1 else None,
                   "partition": (("one block range per rank" if WORKLOAD["kind"] == "sbm" else
                                  f"{world} contiguous ranges after random relabel") if world > 1 else "single"),
                   "exchange": exchange if world > 1 else None,
                   "wire_layout": (("row codes" if Communicator.row_codes else "row groups (reference bytes)")
                                   if (world > 1 and bits in (2, 4, 8)) else None),
                   "pre_post_aggregation": bool(args.pre and world > 1),
                   "boundary_rows_recv_rank0": sum(graph.comm_splits.recv_splits) if world > 1 else 0,
                   "boundary_rows_recv_max": int(recv_rows[0].item()), "boundary_rows_send_max": int(recv_rows[1].item()),
                   "l2": "inputs larger than L2 (activations of gigabytes per layer), no flush", "scale": args.scale},
        "memory_high_water_gb_max_over_ranks": {"allocated": mem[0].item() / 1e9, "reserved": mem[1].item() / 1e9},
        "loss": final_loss,
        "roofline": roofline,
        "gemm": gemm,
        # both kernels that carry the step: the hot-path SpMM (HBM bound) and the dense GEMM of the layers around
        # it (tensor bound; the largest time share at one GPU)
        "rooflines": [roofline] + ([{"bound": "tensor", "kernel": "gemm_bf16x9 (sgnn_gemm_f32), all launches of the step",
                                     "achieved": gemm["bf16_mma_tflops"], "peak": gemm["peak_bf16_tflops_sustained"],
                                     "unit": "TFLOP/s", "frac": gemm["frac"], "traffic": None,
                                     "time_share_of_step": gemm["time_share_of_step"]}] if gemm else []),
        "kernel_time_ms_per_step": {k: v[1] / args.steps for k, v in per_kind.items()},
        "e2e": ({"value": e2e_step_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                 "loss": loss_host} if host_inputs else
                {"value": None, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                 "note": "node data of this workload is too large to stage through pinned host memory on every rank "
                         "of one box; it is generated on the device and no end-to-end leg is run"}),
        "gpu_launches": launches,
        "clocks": clocks,
    }
    if phases is not None:
        line["phases_ms_per_step"] = phases
    if world == 1 and not args.no_kernels:
        line["kernels"] = kernel_benchmarks(device, peak)
    if world == 1 and not args.no_cpu_baseline:
        del model, opt, data, graph
        torch.cuda.empty_cache()
        value, desc = cpu_epoch_baseline(steps=2, warmup=1, target_step_seconds=8.0)
        line["cpu_baseline"] = dict(value=value, **desc)
        if not args.no_kernels:
            line["cpu_baseline"]["ops"] = cpu_op_baselines()
    emit(line)
    if world > 1:
        dist.barrier()


_RESULT_FD = None


def keep_stdout_for_the_result():
    """Libraries write banners to file descriptor 1 (NCCL prints its version there): point descriptor 1 at stderr
    for the run and keep the original for the one JSON line."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict):
    text = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, text)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bits", type=int, default=None, choices=[32, 16, 8, 4, 2],
                    help="bits per boundary value on the wire (default: 2 with several GPUs)")
    ap.add_argument("--scale", type=float, default=1.0, help="scale nodes and edges (debugging only; 1.0 = the workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--exchange", default="p2p", choices=["nccl", "p2p"],
                    help="boundary exchange of the 2/4/8-bit modes: NCCL all_to_all, or the one-sided kernel that stores "
                         "packed rows into the peers' buffers over NVLink")
    ap.add_argument("--pre", action="store_true", help="pre/post-aggregation mode (minimum vertex cover per rank pair)")
    ap.add_argument("--phases", action="store_true", help="also report CUDA-event times of the Aggregator phases")
    ap.add_argument("--workload", default="rmat-2.4M", choices=sorted(WORKLOADS),
                    help="rmat-2.4M: the headline single-GPU configuration (default); sbm-10M: the 8-block pre/post "
                         "configuration; rmat-large: the large scaling-sweep configuration (size with --nodes)")
    ap.add_argument("--nodes", type=int, default=None, help="node count (sbm-10M, rmat-large); default: the full size")
    ap.add_argument("--row-groups", action="store_true",
                    help="2/4/8-bit exchange in the reference's row-group bytes instead of the row-codes layout")
    ap.add_argument("--by-peer", default="auto", choices=["auto", "on", "off"],
                    help="backward pass: produce the gradient rows for the peers one peer at a time (auto: when the fp32 "
                         "buffer for all of them would exceed 1 GiB)")
    ap.add_argument("--only-kernels", default=None, metavar="SECTIONS",
                    help="run only the kernel micro-benchmarks (comma-separated: spmm_cfg1, remote, remote_large, "
                         "quant_cfg2, gemm, and node_order = the SpMM under different node numberings) on one GPU and "
                         "print their JSON; the command to put under a profiler")
    ap.add_argument("--node-order", default="degree", choices=["degree", "generated"],
                    help="numbering of the synthetic graph's nodes: every partition's nodes by ascending in-degree "
                         "(order_nodes_by_degree, a preprocessing step), or the ids the generator produced")
    ap.add_argument("--memory-table", action="store_true",
                    help="print which (GPU count, bits) cells of the chosen workload fit one B200 per rank, and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    global WORKLOAD, NODE_ORDER
    WORKLOAD = WORKLOADS[args.workload]
    NODE_ORDER = args.node_order
    if args.memory_table:
        print(json.dumps(memory_table(args.nodes), indent=1))
        return
    keep_stdout_for_the_result()
    if args.only_kernels:
        torch.cuda.set_device(0)
        peak, _ = measured_peak_gbs()
        emit({"kernels": kernel_benchmarks(torch.device("cuda", 0), peak, tuple(args.only_kernels.split(",")))})
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
