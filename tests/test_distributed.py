"""Multi-rank Aggregator / Communicator / graph-builder tests.

* CPU (runs everywhere): world_size 2 and 3 on gloo with the oracle-backed op
  stand-ins — the host-side orchestration is identical to the GPU path.
* GPU (needs >= 2 devices): world_size 2 on NCCL with the CUDA kernels.
"""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(nproc: int, extra):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "dist_worker.py")] + extra
    env = dict(os.environ, OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + "\n" + res.stderr[-3000:]
    assert "dist_worker: ok" in res.stdout, res.stdout[-3000:]


@pytest.mark.parametrize("world", [2, 3])
def test_aggregator_on_gloo_cpu_ranks(world):
    launch(world, ["--emulate", "--nodes", "1200", "--edges", "12000", "--feat", "32"])


def test_aggregator_on_gloo_cpu_ranks_with_the_reference_wire_bytes():
    launch(2, ["--emulate", "--row-groups", "--nodes", "1200", "--edges", "12000", "--feat", "32"])


@pytest.mark.gpu
def test_aggregator_ranks_sharing_one_gpu_with_the_reference_wire_bytes():
    launch(2, ["--gloo-gpu", "--row-groups"])


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_aggregator_ranks_sharing_one_gpu(world):
    """The CUDA kernels, the real Aggregator / Communicator / graph builders and every exchange mode
    (32/16/8/4/2 bits, post and pre/post, fused and unfused, training and evaluation) on ``world`` ranks that
    share ONE device, the exchange staged through host memory over gloo."""
    launch(world, ["--gloo-gpu"])


@pytest.mark.parametrize("world,graph", [(4, "sbm8"), (3, "rmat-stream")])
def test_partition_parallel_generators_on_gloo_cpu_ranks(world, graph):
    """The generators of the large workloads (every rank produces its own edges) feeding the same checks."""
    if graph == "sbm8" and 8 % world:
        pytest.skip("the blocks must divide over the ranks")
    launch(world, ["--emulate", "--graph", graph, "--nodes", "1200", "--edges", "7000", "--feat", "32"])


@pytest.mark.parametrize("world", [1, 3])
def test_nodes_renumbered_by_degree_on_gloo_cpu_ranks(world):
    """``order_nodes_by_degree`` (every rank renumbers its own nodes, the remote sources follow through an exchange
    with their owners): same edge counts, a permutation, ascending degrees, and every Aggregator check passes on
    the renumbered graph."""
    launch(world, ["--emulate", "--degree-order", "--nodes", "1200", "--edges", "12000", "--feat", "32"])


@pytest.mark.gpu
def test_sbm_blocks_on_eight_ranks_sharing_one_gpu():
    """The 8-GPU pre/post configuration at a down-scaled size: 8 blocks on 8 ranks (one device), generated rank by
    rank, post and pre/post aggregation, every exchange mode, against the oracle."""
    launch(8, ["--gloo-gpu", "--graph", "sbm8", "--nodes", "4000", "--edges", "30000", "--feat", "128"])


@pytest.mark.gpu
def test_streamed_rmat_on_four_ranks_sharing_one_gpu():
    launch(4, ["--gloo-gpu", "--graph", "rmat-stream", "--nodes", "3000", "--edges", "20000", "--feat", "256"])


@pytest.mark.gpu
def test_fused_model_ranks_sharing_one_gpu_matches_dense_reference():
    launch(2, ["--gloo-gpu", "--model", "--nodes", "3000", "--edges", "40000"])


@pytest.mark.gpu
@pytest.mark.multigpu
def test_aggregator_on_nccl_two_gpus():
    launch(2, [])


@pytest.mark.gpu
@pytest.mark.multigpu
def test_aggregator_one_sided_exchange_two_gpus():
    """Same checks with the quantise-pack kernel storing straight into the peer's receive buffers."""
    launch(2, ["--p2p"])


@pytest.mark.gpu
@pytest.mark.multigpu
def test_absent_peer_ends_in_a_timeout_status_two_gpus():
    """A rank stays away from a barrier of the one-sided exchange (on the host, nothing of it in flight; NVLS off,
    plain peer loads and stores): the other rank's bounded wait runs out, it gets ``PeerTimeout`` and carries on."""
    launch(2, ["--absent-peer"])


@pytest.mark.parametrize("world", [2, 3])
def test_model_on_gloo_cpu_ranks_matches_dense_reference(world):
    launch(world, ["--emulate", "--model", "--nodes", "900", "--edges", "9000"])


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_model_on_nccl_two_gpus_matches_dense_reference():
    launch(2, ["--model", "--nodes", "3000", "--edges", "40000"])
