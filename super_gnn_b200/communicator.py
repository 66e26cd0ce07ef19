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

import math
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


class _Done:
    """Handle of an exchange that has already completed."""

    def wait(self):
        return None


def all_to_all_rows(recv, send, recv_splits, send_splits, async_op: bool):
    """``dist.all_to_all_single`` over the leading dimension.  NCCL takes the device tensors as they are.  A
    gloo group given device tensors (ranks that share one GPU, or hosts without NVLink: a test and debugging
    configuration) has no device all-to-all, so the rows are staged through host memory and the call
    completes before it returns."""
    if dist.get_backend() == "nccl" or not send.is_cuda:
        return dist.all_to_all_single(recv, send, recv_splits, send_splits, async_op=async_op)

    def as_bytes(t):  # [rows, bytes per row]: gloo moves bytes, whatever the element type
        return t.view(torch.uint8).reshape(t.size(0), t.element_size() * math.prod(t.shape[1:]))

    send_h = as_bytes(send.contiguous()).cpu()
    recv_d = as_bytes(recv)
    recv_h = torch.empty(recv_d.shape, dtype=torch.uint8)
    dist.all_to_all_single(recv_h, send_h, recv_splits, send_splits)
    recv_d.copy_(recv_h)
    return _Done()


class _BackwardByPeer:
    def __init__(self, comm, comm_splits, qbuf, feat_len: int):
        self.comm, self.cs, self.qbuf, self.F = comm, comm_splits, qbuf, int(feat_len)
        self.bits = comm.num_bits
        self.row_codes = comm.uses_row_codes(feat_len)
        self.world = len(comm_splits.recv_splits)
        n = comm_splits.recv_splits  # the rows received in the forward pass are the rows sent back now
        self.begin = [sum(n[:p]) for p in range(self.world + 1)]
        self.px = getattr(qbuf, "peer_exchange", None)
        if self.px is not None:
            self.px.check_capacity(feat_len)
            if not self.px.supports(feat_len):
                self.px = None
        if self.px is not None:
            self.px.begin(torch.cuda.current_stream())
        else:
            total = self.begin[-1]
            self.q_send = qbuf.quantized_recv_data_buf
            if self.row_codes:
                self.q_send = supergnn_ops.rowcodes_view(self.q_send, total, feat_len, self.bits)

    def send(self, p: int, rows: torch.Tensor):
        a, b = self.begin[p], self.begin[p + 1]
        if b == a:
            return
        qb = self.qbuf
        if self.px is not None:
            self.px.store(rows, None, self.px.single_peer_range(p, b - a), "backward", self.row_codes)
            return
        with TimeRecorder.ctx.time_block("quantization"):
            p32, p16 = qb.quantized_recv_params_buf_fp32[a:b], qb.quantized_recv_params_buf_bf16[a:b]
            if self.row_codes:
                supergnn_ops.quant_pack_rowcodes(rows, None, self.bits, self.q_send[a:b], params=p32, params_bf16=p16)
            else:
                epb = 8 // self.bits
                g0 = sum(self.cs.recv_splits_int2[:p])
                one = torch.tensor([0, b - a], dtype=torch.int32)
                supergnn_ops.quant_pack_rows(rows, None, one, 1, self.bits, self.q_send[g0:g0 + -(-(b - a) // epb)],
                                             params=p32, params_bf16=p16)

    def finish(self):
        if self.px is not None:
            from .peer_exchange import EventHandle

            return EventHandle(self.px.end(torch.cuda.current_stream()))
        cs, qb = self.cs, self.qbuf
        recv_splits, send_splits = cs.send_splits, cs.recv_splits
        q_recv = qb.quantized_send_data_buf
        if self.row_codes:
            q_recv = supergnn_ops.rowcodes_view(q_recv, sum(recv_splits), self.F, self.bits)
            recv_q, send_q = recv_splits, send_splits
        else:
            recv_q, send_q = cs.send_splits_int2, cs.recv_splits_int2
        self.comm._maybe_barrier()
        w1 = all_to_all_rows(qb.quantized_send_params_buf_bf16, qb.quantized_recv_params_buf_bf16, recv_splits,
                             send_splits, self.comm.is_async)
        w2 = all_to_all_rows(q_recv, self.q_send, recv_q, send_q, self.comm.is_async)
        return _Handles([w1, w2])


class Communicator(object):
    ctx = None

    # 2/4/8-bit modes: keep the quantised rows in the row-codes layout (every row in its own F*bits/8 bytes)
    # wherever the row width allows it, instead of the reference's row-group bytes.  Same codes, same
    # parameters, same number of bytes on the wire; the consumers' gathers then move a quarter (2 bits) or half
    # (4 bits) of the bytes.  False restores the reference's wire bytes.
    row_codes = True

    def uses_row_codes(self, feat_len: int) -> bool:
        return bool(self.row_codes) and self.num_bits in (2, 4, 8) and supergnn_ops.rowcodes_supported(feat_len)

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
            backend = os.environ.get("SGNN_DIST_BACKEND", "")
            if torch.cuda.is_available():
                # ranks normally own one GPU each; with fewer GPUs than ranks they share (gloo only, see below)
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)) % torch.cuda.device_count())
            if torch.cuda.is_available() and backend != "gloo":
                dist.init_process_group(backend="nccl", init_method="env://",
                                        device_id=torch.device("cuda", torch.cuda.current_device()))
            else:
                # SGNN_DIST_BACKEND=gloo with CUDA present: the kernels run on the GPU and the exchange is staged
                # through host memory (``all_to_all_rows``), so several ranks can share one GPU: no kernel of one
                # rank ever waits for a kernel of another
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
            work = all_to_all_rows(recv_buf, send_buf, recv_splits, send_splits, self.is_async)
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
        work = all_to_all_rows(recv16, send16, recv_splits, send_splits, self.is_async)
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
        row_codes = self.uses_row_codes(feat_len)
        rows = src if row_index is not None else send_buf
        if px is not None and px.supports(feat_len):
            # one-sided exchange: quantise, pack and store into the peers' receive buffers in one kernel
            with TimeRecorder.ctx.time_block("quantization"):
                done = px.exchange(rows, row_index, work_range, direction, params_fp32=None, row_codes=row_codes)
            from .peer_exchange import EventHandle

            return EventHandle(done)
        if row_codes:  # one row of F*bits/8 bytes per fp32 row: the data splits are the row splits
            n_send, n_recv = sum(send_splits), sum(recv_splits)
            q_send = supergnn_ops.rowcodes_view(q_send, n_send, feat_len, self.num_bits)
            q_recv = supergnn_ops.rowcodes_view(q_recv, n_recv, feat_len, self.num_bits)
            recv_splits_q, send_splits_q = recv_splits, send_splits
        with TimeRecorder.ctx.time_block("quantization"):
            if sum(send_splits) > 0:
                if row_codes:
                    supergnn_ops.quant_pack_rowcodes(rows, row_index, self.num_bits, q_send, params=p_send32,
                                                     params_bf16=p_send16)
                else:
                    supergnn_ops.quant_pack_rows(rows, row_index, work_range, world, self.num_bits, q_send,
                                                 params=p_send32, params_bf16=p_send16)
        self._maybe_barrier()
        with TimeRecorder.ctx.time_block("alltoallv_for_quantized_params"):
            w1 = all_to_all_rows(p_recv16, p_send16, recv_splits, send_splits, self.is_async)
        with TimeRecorder.ctx.time_block("alltoallv_for_quantized_data"):
            w2 = all_to_all_rows(q_recv, q_send, recv_splits_q, send_splits_q, self.is_async)
        return _Handles([w1, w2])

    def begin_backward_by_peer(self, comm_splits, comm_buf, qbuf, feat_len: int):
        """Quantised backward exchange fed one destination peer at a time (2/4/8 bits): the caller produces the
        fp32 gradient rows that go back to peer p — rows [wr[p], wr[p+1]) of the full remote-gradient buffer —
        and hands them to ``send(p, rows)``; ``finish()`` returns the usual handle.  The bytes delivered are
        those of ``comm(..., "backward")`` on the full buffer; only one peer's fp32 rows exist at a time."""
        assert self.num_bits in (2, 4, 8)
        return _BackwardByPeer(self, comm_splits, qbuf, feat_len)

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
