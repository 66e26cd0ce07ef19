"""The drop-in claim: with the package registered under the reference's module names, the reference's own
GraphSAGE driver code (``examples/graphsage/sage.py``, ``utils.py``, ``train.py``: imported from the reference tree,
unmodified) builds its model, trains three epochs with a 2-bit boundary exchange on two ranks and evaluates, and
lands on the same losses and parameters as this package's own driver.  Needs the reference tree (skipped where it is
not mounted) and no GPU: the ranks are gloo CPU ranks over the oracle-backed op stand-ins."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_reference_graphsage_driver_runs_unchanged_on_the_aliased_package():
    ref = build_ref.default_reference_dir()
    if not os.path.exists(os.path.join(ref, "examples", "graphsage", "sage.py")):
        pytest.skip("reference tree not mounted")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "drop_in_worker.py"), "--reference", ref]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"),
                         cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + "\n" + res.stderr[-3000:]
    assert "drop_in_worker: ok" in res.stdout, res.stdout[-3000:]
