"""Boundary-feature exchange with the reference's ``Communicator`` interface
(super_gnn/communicator.py:18-306), on NCCL over NVLink / NVSwitch.

One process per GPU.  The personalised all-to-all of the reference
(``all_to_all_single`` over MPI / oneCCL) becomes ``all_to_all_single`` on
ProcessGroupNCCL, i.e. grouped ncclSend/ncclRecv to every peer.  With
``is_async=True`` the exchange runs on NCCL's own stream: it starts once the
work already enqueued on the current stream (gather / quantise) has finished,
and the caller's local aggregation then overlaps it; ``handle.wait()`` makes the
current stream wait, not the host.

Differences from the reference, on purpose:
* ``dist.barrier()`` before each exchange (communicator.py:95, 279) is dropped —
  stream ordering already gives what it was there for (``barrier=True`` restores it);
* in the 2/4/8-bit mode the (zero_point, scale) pairs are written as bf16 by the
  quantise kernel itself and read as bf16 by the dequantise kernels, so the two
  conversion passes (:283-284, :293-294) disappear; the bytes on the wire are the same;
  both messages are asynchronous;
* the bf16 mode converts after the wait (the reference converts before it, :124-127,
  which races with an asynchronous exchange).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import supergnn_ops
from .time_recorder import TimeRecorder


class _Handles:
    """Several asynchronous works behind one ``wait()``, plus a deferred epilogue."""

    def __init__(self, works, after=None):
        self.works = [w for w in works if w is not None]
        self.after = after

    def wait(self):
        for w in self.works:
            w.wait()
        if self.after is not None:
            self.after()
            self.after = None


class Communicator(object):
    ctx = None

    def __init__(self, num_bits=32, is_async=True, barrier=False) -> None:
        self.num_bits = num_bits
        self.is_async = is_async
        self.barrier = barrier
        self.world_size = -1
        self.rank = -1
        Communicator.ctx = self

    def init_dist_group(self):
        """env:// rendezvous (torchrun); NCCL when a GPU is present, gloo otherwise
        (host-logic tests).  Returns ``(rank, world_size)`` like communicator.py:26-51."""
        if not dist.is_initialized():
            if torch.cuda.is_available():
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
                dist.init_process_group(backend="nccl", init_method="env://",
                                        device_id=torch.device("cuda", torch.cuda.current_device()))
            else:
                dist.init_process_group(backend="gloo", init_method="env://")
        self.world_size = dist.get_world_size()
        self.rank = dist.get_rank()
        return (self.rank, self.world_size)

    # ------------------------------------------------------------------
    def comm(self, comm_splits, comm_buf, comm_buf_for_quantization, layer, is_training, direction,
             src=None, row_index=None):
        """Start the exchange of one layer/direction; returns a handle with ``wait()``.

        ``src`` / ``row_index`` (optional): the rows to send are ``src[row_index]``
        and have NOT been copied into the send buffer; the gather is then fused
        with the quantisation (or done here for the 32/16-bit modes)."""
        if self.num_bits == 32 or is_training is False:
            return self.comm_with_fp32(comm_splits, comm_buf, direction, src, row_index)
        if self.num_bits == 16:
            return self.comm_with_fp16(comm_splits, comm_buf, direction, src, row_index)
        if self.num_bits in (2, 4, 8):
            return self.comm_with_int2_quantization_for_all_procs(comm_splits, comm_buf, comm_buf_for_quantization,
                                                                  direction, src, row_index)
        raise RuntimeError(f"unsupported num_bits {self.num_bits}")

    @staticmethod
    def _roles(comm_splits, comm_buf, direction):
        if direction == "forward":
            return comm_buf.recv_buf, comm_buf.send_buf, comm_splits.recv_splits, comm_splits.send_splits
        return comm_buf.send_buf, comm_buf.recv_buf, comm_splits.send_splits, comm_splits.recv_splits

    def _maybe_barrier(self):
        if self.barrier:
            with TimeRecorder.ctx.time_block("barrier(inner)"):
                dist.barrier()

    def comm_with_fp32(self, comm_splits, comm_buf, direction, src=None, row_index=None):
        recv_buf, send_buf, recv_splits, send_splits = self._roles(comm_splits, comm_buf, direction)
        if row_index is not None:
            supergnn_ops.gather_rows(src, row_index, send_buf)
        self._maybe_barrier()
        with TimeRecorder.ctx.time_block("alltoallv(inner)"):
            work = dist.all_to_all_single(recv_buf, send_buf, recv_splits, send_splits, async_op=self.is_async)
        return _Handles([work])

    def comm_with_fp16(self, comm_splits, comm_buf, direction, src=None, row_index=None):
        recv_buf, send_buf, recv_splits, send_splits = self._roles(comm_splits, comm_buf, direction)
        if direction == "forward":
            recv16, send16 = comm_buf.recv_buf_fp16, comm_buf.send_buf_fp16
        else:
            recv16, send16 = comm_buf.send_buf_fp16, comm_buf.recv_buf_fp16
        if row_index is not None:
            supergnn_ops.gather_rows(src, row_index, send_buf)
        send16.copy_(send_buf)
        self._maybe_barrier()
        work = dist.all_to_all_single(recv16, send16, recv_splits, send_splits, async_op=self.is_async)
        return _Handles([work], after=lambda: recv_buf.copy_(recv16))

    def comm_with_int2_quantization_for_all_procs(self, comm_splits, comm_buf, qbuf, direction, src=None,
                                                  row_index=None):
        if direction == "forward":
            recv_splits, send_splits = comm_splits.recv_splits, comm_splits.send_splits
            recv_splits_q, send_splits_q = comm_splits.recv_splits_int2, comm_splits.send_splits_int2
            send_buf = comm_buf.send_buf
            q_recv, q_send = qbuf.quantized_recv_data_buf, qbuf.quantized_send_data_buf
            p_recv16, p_send16 = qbuf.quantized_recv_params_buf_bf16, qbuf.quantized_send_params_buf_bf16
            p_send32 = qbuf.quantized_send_params_buf_fp32
            work_range = qbuf.quantized_work_range_per_proc
        else:
            recv_splits, send_splits = comm_splits.send_splits, comm_splits.recv_splits
            recv_splits_q, send_splits_q = comm_splits.send_splits_int2, comm_splits.recv_splits_int2
            send_buf = comm_buf.recv_buf
            q_recv, q_send = qbuf.quantized_send_data_buf, qbuf.quantized_recv_data_buf
            p_recv16, p_send16 = qbuf.quantized_send_params_buf_bf16, qbuf.quantized_recv_params_buf_bf16
            p_send32 = qbuf.quantized_recv_params_buf_fp32
            work_range = qbuf.dequantized_work_range_per_proc
        world = len(recv_splits)
        px = getattr(qbuf, "peer_exchange", None)
        feat_len = (src if row_index is not None else send_buf).size(-1)
        if px is not None:
            px.check_capacity(feat_len)
        if px is not None and px.supports(feat_len):
            # one-sided exchange: quantise, pack and store into the peers' receive buffers in one kernel
            with TimeRecorder.ctx.time_block("quantization"):
                rows = src if row_index is not None else send_buf
                done = px.exchange(rows, row_index, work_range, direction, params_fp32=None)
            from .peer_exchange import EventHandle

            return EventHandle(done)
        with TimeRecorder.ctx.time_block("quantization"):
            if sum(send_splits) > 0:
                if row_index is not None:
                    supergnn_ops.quant_pack_rows(src, row_index, work_range, world, self.num_bits, q_send,
                                                 params=p_send32, params_bf16=p_send16)
                else:
                    supergnn_ops.quant_pack_rows(send_buf, None, work_range, world, self.num_bits, q_send,
                                                 params=p_send32, params_bf16=p_send16)
        self._maybe_barrier()
        with TimeRecorder.ctx.time_block("alltoallv_for_quantized_params"):
            w1 = dist.all_to_all_single(p_recv16, p_send16, recv_splits, send_splits, async_op=self.is_async)
        with TimeRecorder.ctx.time_block("alltoallv_for_quantized_data"):
            w2 = dist.all_to_all_single(q_recv, q_send, recv_splits_q, send_splits_q, async_op=self.is_async)
        return _Handles([w1, w2])

    def enable_peer_exchange(self, graph, max_feat_len: int, timeout_ms: int = 20000):
        """Switch the 2/4/8-bit exchange of ``graph`` to the one-sided NVLink path (collective call:
        every rank must make it).  Needs NCCL ranks on one NVLink domain."""
        from .peer_exchange import PeerExchange

        return PeerExchange(graph, max_feat_len, self.num_bits, timeout_ms)

    def get_splits_for_comm_quantized_data(self, recv_splits_tensor, send_splits_tensor,
                                           dequantized_nodes_feat_range, quantized_nodes_feat_range):
        """Bytes per peer for the per-row-bit-width layout (communicator.py:308-342)."""
        rb = torch.zeros(self.world_size + 1, dtype=torch.int64)
        rb[1:] = recv_splits_tensor.to(torch.int64).cumsum(0).cpu()
        sb = torch.zeros(self.world_size + 1, dtype=torch.int64)
        sb[1:] = send_splits_tensor.to(torch.int64).cumsum(0).cpu()
        dr = dequantized_nodes_feat_range.cpu()
        qr = quantized_nodes_feat_range.cpu()
        recv = [int(dr[rb[r + 1]] - dr[rb[r]]) for r in range(self.world_size)]
        send = [int(qr[sb[r + 1]] - qr[sb[r]]) for r in range(self.world_size)]
        return recv, send
