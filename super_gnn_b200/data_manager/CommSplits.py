"""Rows exchanged with every peer (super_gnn/data_manager/CommSplits.py:6-18)."""
from __future__ import annotations

from ..quantizer import Quantizer_for_all_procs


class CommSplits(object):
    def __init__(self, recv_splits: list, send_splits: list, world_size: int, bits: int) -> None:
        self.recv_splits = [int(x) for x in recv_splits]
        self.send_splits = [int(x) for x in send_splits]
        if bits == 2 or bits == 4 or bits == 8:
            # packed rows per peer; the "int2" in the name is historical (used for 2, 4 and 8 bits)
            q = Quantizer_for_all_procs.ctx
            if q is None or q.num_bits != bits:
                q = Quantizer_for_all_procs(world_size, bits)
            self.recv_splits_int2 = [q.get_quantized_splits(self.recv_splits[r]) for r in range(world_size)]
            self.send_splits_int2 = [q.get_quantized_splits(self.send_splits[r]) for r in range(world_size)]
