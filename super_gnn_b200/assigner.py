"""``Assigner`` kept importable for drivers that construct it
(examples/graphsage/train.py:259-266 in the reference; class at
super_gnn/assigner.py:7-64).  Its mixed-bit branch is unreachable from
``Communicator.comm`` in the reference, so only the bookkeeping is kept."""
from __future__ import annotations

import torch

bits_idx = torch.tensor([8.0, 4.0, 2.0], dtype=torch.float32)


class Assigner(object):
    ctx = None

    def __init__(self, num_bits, num_layers, assign_weight, assign_period, num_send_nodes_on_forward,
                 num_send_nodes_on_backward):
        self.num_bits = num_bits
        self.num_layers = num_layers
        self.assign_weight = assign_weight
        self.assign_period = assign_period
        self.num_send_nodes_on_forward = num_send_nodes_on_forward
        self.num_send_nodes_on_backward = num_send_nodes_on_backward
        self.node_dataformat_dict = {}
        for layer in range(num_layers):
            fill = float(num_bits) if num_bits != -1 else 0.0
            self.node_dataformat_dict[f"forward{layer}"] = torch.full((num_send_nodes_on_forward,), fill)
            self.node_dataformat_dict[f"backward{layer}"] = torch.full((num_send_nodes_on_backward,), fill)
        Assigner.ctx = self

    def reassign_node_dataformat(self, epoch):
        if self.num_bits == -1 and epoch % self.assign_period == 0:
            for layer, t in self.node_dataformat_dict.items():
                pick = torch.multinomial(self.assign_weight, t.size(0), replacement=True)
                t.copy_(bits_idx[pick])

    def get_node_dataformat(self, layer):
        return self.node_dataformat_dict[layer]
