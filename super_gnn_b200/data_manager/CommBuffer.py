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
    """fp32 (and, at 16 bits, bf16) rows to send and received.  Same attribute names as the reference; the device
    memory behind each buffer is claimed on first use, at the widest layer's size, and then only re-shaped per
    layer: the fused quantised path never touches the fp32 send buffer, and with the remote gradient rows
    produced peer by peer it never touches the fp32 receive buffer either — on the largest graphs each would
    be tens of gigabytes."""

    def __init__(self, comm_splits: CommSplits, feat_len: int, bits: int, device=None) -> None:
        self._device = device or default_device()
        self._max_feat = int(feat_len)
        self._rows = dict(send=sum(comm_splits.send_splits), recv=sum(comm_splits.recv_splits))
        self._shape = dict(send=(self._rows["send"], feat_len), recv=(self._rows["recv"], feat_len))
        self._store = {}
        self._has_fp16 = bits == 16

    def _get(self, which: str, dtype) -> torch.Tensor:
        key = (which, dtype)
        t = self._store.get(key)
        if t is None:
            t = torch.zeros((self._rows[which], self._max_feat), dtype=dtype, device=self._device)
            self._store[key] = t
        if tuple(t.shape) != tuple(self._shape[which]):
            t.resize_(self._shape[which])
        return t

    send_buf = property(lambda self: self._get("send", torch.float32))
    recv_buf = property(lambda self: self._get("recv", torch.float32))
    send_buf_fp16 = property(lambda self: self._get("send", torch.bfloat16) if self._has_fp16 else None)
    recv_buf_fp16 = property(lambda self: self._get("recv", torch.bfloat16) if self._has_fp16 else None)

    def resize_buffer(self, comm_splits: CommSplits, feat_len: int, bits: int) -> None:
        if feat_len > self._max_feat:  # a wider layer than announced: grow the backing store
            self._max_feat = int(feat_len)
            self._store.clear()
        self._rows = dict(send=sum(comm_splits.send_splits), recv=sum(comm_splits.recv_splits))
        self._shape = dict(send=(self._rows["send"], feat_len), recv=(self._rows["recv"], feat_len))


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
