"""One-sided boundary exchange over NVLink peer memory (2/4/8-bit modes).

The reference quantises into a send buffer and then runs two all_to_all collectives
(parameters, packed codes; super_gnn/communicator.py:268-301).  Here every rank's *receive*
buffers live in one symmetric allocation that all peers map, and the quantise-pack kernel
stores each packed row and each bf16 (zero_point, scale) pair straight into the destination
peer's buffer: the compute step and its collective are one kernel, there is no send buffer,
and no library collective sits on the data path.

Ordering is two device-side barriers on the exchange stream (``ops.peer_barrier``: flags in the
same symmetric allocation, release stores and acquire loads at system scope): one before the
stores — every peer has consumed what it received last time — and one after them — every
sender's stores have landed.  The wait is bounded: a rank that does not arrive within
``timeout_ms`` makes the kernel give up and record which peer was missing in a status word in
pinned host memory; nothing traps, the context stays usable, and the next call of
``begin``/``exchange`` (or ``check``) raises ``PeerTimeout`` on the host.  The exchange stream
runs beside the compute stream, so the local aggregation overlaps the transfer exactly as with
the asynchronous collectives.

Only plain loads and stores touch peer memory (no multicast, no TMA).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class PeerTimeout(RuntimeError):
    """A peer did not reach a barrier of the one-sided exchange within the limit; what was received since
    then is not to be trusted.  The ranks' barrier counters no longer agree after that: the exchange object has
    to be built again (a collective call) once every rank is back."""


class PeerExchange:
    def __init__(self, graph, max_feat_len: int, bits: int, timeout_ms: int = 20000):
        import torch.distributed._symmetric_memory as symm_mem

        assert bits in (2, 4, 8), "the one-sided exchange exists for the quantised modes"
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.bits, self.timeout_ms = bits, int(timeout_ms)
        self.max_feat_len = int(max_feat_len)
        self._single_ranges = {}
        cs = graph.comm_splits
        qbuf = graph.comm_buf_for_quantization
        device = qbuf.quantized_recv_data_buf.device
        mine = dict(recv=cs.recv_splits, send=cs.send_splits, recv_q=cs.recv_splits_int2, send_q=cs.send_splits_int2,
                    gpu=str(torch.cuda.get_device_properties(device).uuid))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine)
        if len({a["gpu"] for a in everyone}) != self.world:
            # the ranks' barrier kernels wait on one another: two of them on one GPU need not run at the same time
            raise RuntimeError("the one-sided exchange needs one GPU per rank; ranks that share a GPU use the collectives")
        # capacity of every region = the largest any rank needs (a symmetric allocation has one size)
        fwd_q = max(sum(a["recv_q"]) for a in everyone) * max_feat_len
        fwd_p = max(sum(a["recv"]) for a in everyone) * 4
        bwd_q = max(sum(a["send_q"]) for a in everyone) * max_feat_len
        bwd_p = max(sum(a["send"]) for a in everyone) * 4
        off, offs = 0, {}
        for name, size in (("flags", 4 * self.world), ("fwd_q", fwd_q), ("fwd_p", fwd_p), ("bwd_q", bwd_q),
                           ("bwd_p", bwd_p)):
            offs[name] = off
            off = _align(off + max(size, 256))
        group = dist.group.WORLD
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # newer releases enable every group implicitly
            pass
        self.arena = symm_mem.empty(off, dtype=torch.uint8, device=device)
        self.arena.zero_()
        self.handle = symm_mem.rendezvous(self.arena, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]

        def table(values):
            return torch.tensor(values, dtype=torch.int64, device=device)

        r = self.rank
        # barrier state: every rank's flag array, the number of the last barrier, who failed to arrive
        self.flag_ptrs = table([ptrs[p] + offs["flags"] for p in range(self.world)])
        self.epoch = 0
        self.status = torch.zeros(self.world, dtype=torch.int32).pin_memory()
        # forward: my rows for peer p land in p's fwd regions after the segments of the ranks before me
        self.fwd_tables = (table([ptrs[p] + offs["fwd_q"] for p in range(self.world)]),
                           table([sum(everyone[p]["recv_q"][:r]) for p in range(self.world)]),
                           table([ptrs[p] + offs["fwd_p"] for p in range(self.world)]),
                           table([sum(everyone[p]["recv"][:r]) for p in range(self.world)]))
        # backward: my gradient rows for owner p land in p's bwd regions
        self.bwd_tables = (table([ptrs[p] + offs["bwd_q"] for p in range(self.world)]),
                           table([sum(everyone[p]["send_q"][:r]) for p in range(self.world)]),
                           table([ptrs[p] + offs["bwd_p"] for p in range(self.world)]),
                           table([sum(everyone[p]["send"][:r]) for p in range(self.world)]))
        # the graph's receive-side buffers become views of the arena, so the consumers are unchanged
        a = self.arena
        qbuf.quantized_recv_data_buf = a[offs["fwd_q"]: offs["fwd_q"] + fwd_q].view(-1, max_feat_len)
        qbuf.quantized_recv_params_buf_bf16 = a[offs["fwd_p"]: offs["fwd_p"] + max(fwd_p, 4)].view(torch.bfloat16).view(-1, 2)[: fwd_p // 4]
        qbuf.quantized_send_data_buf = a[offs["bwd_q"]: offs["bwd_q"] + bwd_q].view(-1, max_feat_len)
        qbuf.quantized_send_params_buf_bf16 = a[offs["bwd_p"]: offs["bwd_p"] + max(bwd_p, 4)].view(torch.bfloat16).view(-1, 2)[: bwd_p // 4]
        self.stream = torch.cuda.Stream(device=device, priority=-1)
        qbuf.peer_exchange = self
        torch.cuda.synchronize(device)  # the zeroed flags are in memory ...
        dist.barrier()                  # ... on every rank before the first device-side barrier reads them

    def _barrier(self):
        """One device-side barrier on the current stream (every rank calls it the same number of times)."""
        from . import supergnn_ops as ops

        self.epoch += 1
        if self.epoch & 0xFFFFFFFF == 0:  # 0 is the flags' initial value: skipped when the 32-bit counter wraps
            self.epoch += 1
        ops.peer_barrier(self.flag_ptrs, self.rank, self.world, self.epoch, self.timeout_ms * 1000, self.status)

    def check(self) -> None:
        """Raise if a barrier that has finished by now gave up on a peer (reads pinned host memory: no
        synchronisation; call after one to cover everything launched so far)."""
        if bool(self.status.any()):
            missing = {p: int(e) for p, e in enumerate(self.status.tolist()) if e}
            raise PeerTimeout(f"rank {self.rank}: no signal within {self.timeout_ms} ms from peer(s) "
                              + ", ".join(f"{p} at barrier {e & 0xFFFFFFFF}" for p, e in missing.items()))

    @staticmethod
    def supports(feat_len: int) -> bool:
        """Row widths the one-sided kernel takes (vector path of the quantiser); other widths go through the
        collectives, which deliver the same bytes into the same receive buffers."""
        return feat_len % 4 == 0 and 0 < feat_len <= 512

    def check_capacity(self, feat_len: int) -> None:
        """The receive regions were sized for ``max_feat_len``: a wider layer would spill into the next region."""
        if feat_len > self.max_feat_len:
            raise RuntimeError(f"boundary rows of {feat_len} values do not fit the exchange buffers, which were "
                               f"sized for at most {self.max_feat_len}")

    # --- the same exchange in pieces: begin(), any number of store() calls on the caller's stream, end() ---
    def begin(self, stream):
        """Peers are done with the previous contents of their receive buffers: ``stream`` waits for that."""
        self.check()
        self.stream.wait_stream(stream)
        with torch.cuda.stream(self.stream):
            self._barrier()
        stream.wait_stream(self.stream)

    def store(self, src, row_index, work_range, direction: str, row_codes: bool, params_fp32=None):
        """One quantise-pack-store kernel on the current stream (between ``begin`` and ``end``)."""
        from . import supergnn_ops as ops

        tables = self.fwd_tables if direction == "forward" else self.bwd_tables
        if row_codes:
            ops.quant_pack_rowcodes_p2p(src, row_index, work_range, self.world, self.bits,
                                        (tables[0], tables[2], tables[3]), params=params_fp32)
        else:
            ops.quant_pack_rows_p2p(src, row_index, work_range, self.world, self.bits, tables, params=params_fp32)

    def end(self, stream):
        """Every sender's stores have landed: returns the event consumers wait for."""
        self.stream.wait_stream(stream)
        with torch.cuda.stream(self.stream):
            self._barrier()
            done = torch.cuda.Event()
            done.record(self.stream)
        return done

    def single_peer_range(self, p: int, rows: int) -> torch.Tensor:
        """Work range under which all ``rows`` rows belong to peer ``p`` (cached device tensors)."""
        key = (p, rows)
        t = self._single_ranges.get(key)
        if t is None:
            t = torch.tensor([0] * (p + 1) + [rows] * (self.world - p), dtype=torch.int32, device=self.arena.device)
            self._single_ranges[key] = t
        return t

    def exchange(self, src, row_index, work_range, direction: str, params_fp32=None, row_codes: bool = False):
        """Quantise ``src[row_index]`` (or ``src``) per destination peer and store it into the peers' receive
        buffers, in the reference's row-group bytes or (``row_codes``) one run of F*bits/8 bytes per row.
        Returns an event on the exchange stream; consumers wait for it."""
        from . import supergnn_ops as ops

        self.check()
        cur = torch.cuda.current_stream()
        self.stream.wait_stream(cur)  # the rows to send are complete
        with torch.cuda.stream(self.stream):
            self._barrier()  # peers are done with the previous contents
            tables = self.fwd_tables if direction == "forward" else self.bwd_tables
            S = row_index.numel() if row_index is not None else src.size(0)
            if S > 0 and row_codes:
                ops.quant_pack_rowcodes_p2p(src, row_index, work_range, self.world, self.bits,
                                            (tables[0], tables[2], tables[3]), params=params_fp32)
            elif S > 0:
                ops.quant_pack_rows_p2p(src, row_index, work_range, self.world, self.bits, tables, params=params_fp32)
            self._barrier()  # every sender's stores have landed
            done = torch.cuda.Event()
            done.record(self.stream)
        return done


class EventHandle:
    """``wait()`` like a collective's Work: the current stream waits for the exchange stream."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)
