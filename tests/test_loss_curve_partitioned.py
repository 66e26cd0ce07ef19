"""20-epoch loss curves with a QUANTISED, partitioned boundary exchange: the CUDA path (fused layers and
kernels, real Aggregator / Communicator / graph builders) against the CPU pipeline (the reference's unfused op
chain with the oracle's quantise -> bf16 parameters -> dequantise on gloo CPU ranks), same initial weights and
dropout masks.  World sizes 2 and 4, 2 and 8 bits, post and pre/post aggregation.  Tolerance: |loss
difference| <= 1e-3 at every epoch (the stated end-to-end bound).

The CPU curves are the committed fixture ``tests/golden/loss_curves_partitioned.json`` (made by
``tests/golden/make_loss_curves.py``); the CPU test below re-runs one world size to keep the fixture honest.
The GPU ranks share one device (exchange staged through host memory over gloo), so one GPU is enough.
"""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
import make_loss_curves as mk  # noqa: E402


def golden():
    with open(mk.OUT) as f:
        return json.load(f)


def test_cpu_pipeline_reproduces_the_committed_curves():
    want = golden()["2"]["curves"]
    got = mk.run_worker(2, "--emulate", mk.CASES[2])["curves"]
    for case, curve in want.items():
        assert np.abs(np.array(got[case]) - np.array(curve)).max() <= 2e-4, case


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_cuda_path_matches_cpu_pipeline_over_20_epochs(world):
    want = golden()[str(world)]["curves"]
    got = mk.run_worker(world, "--gloo-gpu", mk.CASES[world])["curves"]
    for case, curve in want.items():
        g, w = np.array(got[case]), np.array(curve)
        assert g[-1] < g[0], f"bits:pre={case} does not train: {g}"
        assert np.abs(g - w).max() <= 1e-3, f"bits:pre={case}: max |loss diff| {np.abs(g - w).max():.2e}\n{g}\n{w}"
