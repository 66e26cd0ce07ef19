"""Host-side pieces of ``bench.py``: workload sizes, the algorithmic-byte models of the roofline figures and the
fits / does-not-fit table (no GPU, nothing timed)."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_byte_models(bench):
    info = dict(M=10, N=8, nnz=100, has_val=True, acc=False)
    assert bench.spmm_bytes(info) == 11 * 8 + 100 * 8 + 100 * 8 * 4 + 10 * 8 * 4
    assert bench.spmm_bytes(dict(info, has_val=False, acc=True)) == 11 * 8 + 100 * 4 + 100 * 8 * 4 + 10 * 8 * 4 * 2
    # a gathered quantised row: F bytes in the row-group layout at every width, F*bits/8 in row codes
    assert bench.spmm_dequant_bytes(dict(M=10, N=256, nnz=100, has_val=False)) == 11 * 8 + 100 * 4 + 100 * 260 + 10 * 256 * 8
    assert bench.rc_bytes_of(10, 256, 100, 2) == 11 * 8 + 100 * (64 + 8) + 10 * 256 * 8
    assert bench.quant_bytes(4, 256, 2, bf16=False) == 4 * 1024 + 4 * 64 + 32
    assert bench.quant_bytes(4, 256, 8) == 4 * 1024 + 4 * 256 + 32 + 16


def test_workload_sizes_and_memory_table(bench):
    bench.WORKLOAD = bench.WORKLOADS["rmat-2.4M"]
    assert bench.workload_size(1.0) == (2_400_000, bench.WORKLOADS["rmat-2.4M"]["undirected_edges"])
    bench.WORKLOAD = bench.WORKLOADS["sbm-10M"]
    n, e = bench.workload_size(1.0)
    assert n == 10_000_000 and n % 8 == 0 and e == bench.WORKLOADS["sbm-10M"]["undirected_edges"]
    bench.WORKLOAD = bench.WORKLOADS["rmat-large"]
    table = bench.memory_table()
    assert table["nodes"] == 111_000_000
    cells = {(c["gpus"], c["bits"]): c for c in table["cells"]}
    assert set(cells) == {(1, 32)} | {(w, b) for w in (2, 4, 8) for b in (32, 8, 2)}
    assert not cells[(1, 32)]["fits"] and not cells[(8, 32)]["fits"]  # 111 M nodes: nowhere near one GPU
    assert cells[(8, 2)]["gb"]["total"] < cells[(8, 8)]["gb"]["total"] < cells[(8, 32)]["gb"]["total"]
    small = {(c["gpus"], c["bits"]): c for c in bench.memory_table(12_000_000)["cells"]}
    assert all(c["fits"] for c in small.values())  # 12 M nodes fit everywhere, one GPU included
    mid = {(c["gpus"], c["bits"]): c for c in bench.memory_table(80_000_000)["cells"]}
    assert mid[(8, 2)]["fits"] and mid[(8, 8)]["fits"] and not mid[(8, 32)]["fits"] and not mid[(4, 2)]["fits"]
    bench.WORKLOAD = bench.WORKLOADS["rmat-2.4M"]
