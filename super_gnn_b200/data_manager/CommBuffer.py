"""Communication buffers (super_gnn/data_manager/CommBuffer.py:5-48), allocated
on the device the exchange runs on (``device`` defaults to the current CUDA
device, or the CPU when there is none — host-logic tests only)."""
from __future__ import annotations

import torch

from .CommSplits import CommSplits


def default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class CommBuffer(object):
    def __init__(self, comm_splits: CommSplits, feat_len: int, bits: int, device=None) -> None:
        device = device or default_device()
        size_send_buf = (sum(comm_splits.send_splits), feat_len)
        size_recv_buf = (sum(comm_splits.recv_splits), feat_len)
        self.send_buf = torch.zeros(size_send_buf, dtype=torch.float32, device=device)
        self.recv_buf = torch.zeros(size_recv_buf, dtype=torch.float32, device=device)
        self.send_buf_fp16 = None
        self.recv_buf_fp16 = None
        if bits == 16:
            self.send_buf_fp16 = torch.zeros(size_send_buf, dtype=torch.bfloat16, device=device)
            self.recv_buf_fp16 = torch.zeros(size_recv_buf, dtype=torch.bfloat16, device=device)

    def resize_buffer(self, comm_splits: CommSplits, feat_len: int, bits: int) -> None:
        size_send_buf = (sum(comm_splits.send_splits), feat_len)
        size_recv_buf = (sum(comm_splits.recv_splits), feat_len)
        self.send_buf.resize_(size_send_buf)
        self.recv_buf.resize_(size_recv_buf)
        if bits == 16 and self.send_buf_fp16 is not None and self.recv_buf_fp16 is not None:
            self.send_buf_fp16.resize_(size_send_buf)
            self.recv_buf_fp16.resize_(size_recv_buf)


class CommBufferForQuantization(object):
    def __init__(self, comm_splits: CommSplits, feat_len: int, bits: int, device=None) -> None:
        device = device or default_device()
        ns, nr = sum(comm_splits.send_splits), sum(comm_splits.recv_splits)
        self.quantized_send_data_buf = torch.zeros((sum(comm_splits.send_splits_int2), feat_len), dtype=torch.uint8,
                                                   device=device)
        self.quantized_recv_data_buf = torch.zeros((sum(comm_splits.recv_splits_int2), feat_len), dtype=torch.uint8,
                                                   device=device)
        self.quantized_send_params_buf_fp32 = torch.zeros((ns, 2), dtype=torch.float32, device=device)
        self.quantized_recv_params_buf_fp32 = torch.zeros((nr, 2), dtype=torch.float32, device=device)
        self.quantized_send_params_buf_bf16 = torch.zeros((ns, 2), dtype=torch.bfloat16, device=device)
        self.quantized_recv_params_buf_bf16 = torch.zeros((nr, 2), dtype=torch.bfloat16, device=device)

        wr = torch.zeros(len(comm_splits.send_splits) + 1, dtype=torch.int32)
        wr[1:] = torch.tensor(comm_splits.send_splits, dtype=torch.int32).cumsum(0)
        self.quantized_work_range_per_proc = wr.to(device)
        wr = torch.zeros(len(comm_splits.recv_splits) + 1, dtype=torch.int32)
        wr[1:] = torch.tensor(comm_splits.recv_splits, dtype=torch.int32).cumsum(0)
        self.dequantized_work_range_per_proc = wr.to(device)

    def resize_buffer(self, comm_splits: CommSplits, feat_len: int, bits: int) -> None:
        px = getattr(self, "peer_exchange", None)
        if px is not None:
            px.check_capacity(feat_len)  # the buffers are views of one arena: growing one would overlap the next
        self.quantized_send_data_buf.resize_((sum(comm_splits.send_splits_int2), feat_len))
        self.quantized_recv_data_buf.resize_((sum(comm_splits.recv_splits_int2), feat_len))
