"""Generate ``loss_curves_partitioned.json``: the 20-epoch loss curves of the CPU pipeline
(``tests/loss_curve_worker.py --emulate``: gloo CPU ranks, the reference's unfused op chain, boundary rows
through the oracle's quantise -> bf16 parameters -> dequantise) for 2 and 4 partitions.

Run from the repository root:  ``python tests/golden/make_loss_curves.py``.
The GPU test compares the CUDA path's curves with this file; a CPU test re-runs one world size and checks
that the file is still what the pipeline produces.
"""
import json
import os
import socket
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "loss_curves_partitioned.json")
# world size -> bits:pre cases; together they cover 2 and 8 bits in post and pre/post mode
CASES = {2: "2:0,8:1", 4: "2:1,8:0"}
SIZE = ["--nodes", "16000", "--edges", "160000", "--epochs", "20"]


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_worker(world: int, mode: str, cases: str) -> dict:
    """Launch the worker (``mode``: "--emulate" or "--gloo-gpu" or "" for NCCL ranks) and return its JSON."""
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "curves.json")
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
               os.path.join(ROOT, "tests", "loss_curve_worker.py"), "--cases", cases, "--out", out] + SIZE
        if mode:
            cmd.append(mode)
        env = dict(os.environ, OMP_NUM_THREADS="2", NCCL_NVLS_ENABLE="0")
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
        assert res.returncode == 0 and "loss_curve_worker: ok" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
        with open(out) as f:
            return json.load(f)


def main():
    golden = {str(w): run_worker(w, "--emulate", cases) for w, cases in CASES.items()}
    with open(OUT, "w") as f:
        json.dump(golden, f, indent=1)
    print("wrote", OUT)


if __name__ == "__main__":
    main()
