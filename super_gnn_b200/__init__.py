"""supergnn_b200: the full-batch GraphSAGE hot path of SuperGNN on B200 (sm_100a).

Host code mirrors the reference's Python interface for this path
(``super_gnn.aggregator``, ``.quantizer``, ``.communicator``, ``.ops`` and the
``supergnn_ops`` extension module); the arithmetic runs in hand-written CUDA
kernels behind a C ABI (``include/supergnn_b200.h``, ``libsupergnn_b200.so``).
There is no CPU path.

``install_as_super_gnn()`` registers this package under the reference's module
names so that code written against ``super_gnn`` imports it unchanged.
"""
from __future__ import annotations

import sys

__version__ = "0.1.0"


def install_as_super_gnn() -> None:
    """Alias this package as ``super_gnn`` / ``supergnn_ops`` in ``sys.modules``."""
    import importlib

    pkg = importlib.import_module(__name__)
    names = ["supergnn_ops", "sparse", "time_recorder", "quantizer", "data_manager", "communicator", "assigner",
             "ops", "ops.spmm_kernel", "aggregator", "layers", "layers.sageconv"]
    mods = {n: importlib.import_module(f"{__name__}.{n}") for n in names}
    sys.modules.setdefault("super_gnn", pkg)
    sys.modules.setdefault("supergnn_ops", mods["supergnn_ops"])
    for n, m in mods.items():
        if n != "supergnn_ops":
            sys.modules.setdefault("super_gnn." + n, m)
