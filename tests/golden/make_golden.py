"""Generate the golden vectors in this folder from the reference's own CPU ops.

Run where the reference tree is mounted:  ``python tests/golden/make_golden.py``.
It imports the unmodified reference ops compiled by ``oracle/build_ref.py``
(``oracle/_ref``), feeds them small seeded inputs and stores inputs and outputs
in ``golden_ops.npz``.  The tests read only the ``.npz``; neither the reference
tree nor ``oracle/_ref`` is needed to run them.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import build_ref  # noqa: E402


def main():
    build_ref.build()
    ref = build_ref.load()
    rng = np.random.default_rng(20240611)
    out = {}

    # --- spmm (accumulating), three widths incl. one that is not a multiple of 4
    M, K = 61, 45
    deg = rng.poisson(5, M)
    deg[7] = 0
    deg[8] = 0
    deg[20] = 70
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = rng.integers(0, K, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(rowptr[-1]).astype(np.float32)
    out["spmm_rowptr"], out["spmm_col"], out["spmm_val"] = rowptr, col, val
    for N in (7, 16, 100):
        X = rng.standard_normal((K, N)).astype(np.float32)
        Y0 = rng.standard_normal((M, N)).astype(np.float32)
        y = torch.from_numpy(Y0.copy())
        # one row range per OpenMP thread, as the reference's wrapper builds them
        T = torch.get_num_threads()
        splits = torch.tensor([M * t // T for t in range(T + 1)], dtype=torch.int32)
        ref.spmm(torch.from_numpy(rowptr), torch.from_numpy(col), torch.from_numpy(val), torch.from_numpy(X), y, M,
                 splits, torch.tensor([0, N], dtype=torch.int32))
        out[f"spmm_X_{N}"], out[f"spmm_Y0_{N}"], out[f"spmm_Y_{N}"] = X, Y0, y.numpy()

    # --- x86 quantize_tensor / dequantize_tensor (caller-supplied min, scale)
    for bits in (8, 4, 2):
        for tag, (S, F) in {"a": (13, 19), "b": (9, 32)}.items():
            x = (rng.standard_normal((S, F)) * np.exp(rng.standard_normal((S, 1)))).astype(np.float32)
            if tag == "b":
                x[3] = 0.25  # constant row: scale 0 -> 1
            mn = x.min(1)
            sc = ((x.max(1) - mn) / np.float32(2 ** bits - 1)).astype(np.float32)
            sc[sc == 0] = 1.0
            epb = 8 // bits
            q = torch.zeros((-(-S // epb), F), dtype=torch.uint8)
            ref.quantize_tensor(torch.from_numpy(x), q, torch.from_numpy(mn.copy()), torch.from_numpy(sc.copy()), bits)
            d = torch.zeros((S, F))
            ref.dequantize_tensor(q, d, torch.from_numpy(mn.copy()), torch.from_numpy(sc.copy()), bits)
            k = f"q{bits}{tag}"
            out[k + "_x"], out[k + "_min"], out[k + "_scale"], out[k + "_q"], out[k + "_deq"] = x, mn, sc, q.numpy(), d.numpy()

    # --- v1 (per-row bit width)
    S, F = 23, 11
    x = rng.standard_normal((S, F)).astype(np.float32)
    bits = rng.choice([2, 4, 8], S).astype(np.float32)
    lens = np.ceil(bits * F / 8.0).astype(np.int64)
    rng_ = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    params = torch.zeros((S, 3))
    params[:, 0] = torch.from_numpy(bits)
    q = torch.zeros(int(rng_[-1]), dtype=torch.uint8)
    ref.quantize_tensor_v1(torch.from_numpy(x), q, torch.from_numpy(rng_), params)
    d = torch.zeros((S, F))
    ref.dequantize_tensor_v1(q, d, torch.from_numpy(rng_), params)
    out["v1_x"], out["v1_bits"], out["v1_range"], out["v1_params"], out["v1_q"], out["v1_deq"] = (
        x, bits, rng_, params.numpy(), q.numpy(), d.numpy())

    # --- v2 (torch.quantize_per_channel compatible)
    for b in (8, 4, 2):
        S, F = 6, 10
        zp = rng.integers(0, 2 ** b, S).astype(np.float32)
        sc = (np.abs(rng.standard_normal(S)) + 0.1).astype(np.float32)
        x = ((rng.integers(0, 2 ** b, (S, F)) - zp[:, None]) * sc[:, None]).astype(np.float32)
        lens = np.ceil(np.full(S, b) * F / 8.0).astype(np.int64)
        r2 = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        q = torch.zeros(int(r2[-1]), dtype=torch.uint8)
        ref.quantize_tensor_v2_torch(torch.from_numpy(x), q, torch.from_numpy(r2), torch.from_numpy(zp), torch.from_numpy(sc), b)
        d = torch.zeros((S, F))
        ref.dequantize_tensor_v2_torch(q, d, torch.from_numpy(r2), torch.from_numpy(zp), torch.from_numpy(sc), b)
        out[f"v2_{b}_x"], out[f"v2_{b}_zp"], out[f"v2_{b}_sc"], out[f"v2_{b}_q"], out[f"v2_{b}_deq"] = x, zp, sc, q.numpy(), d.numpy()

    path = os.path.join(HERE, "golden_ops.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
