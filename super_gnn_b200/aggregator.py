"""``Aggregator``: the per-layer neighbour aggregation across graph partitions,
with the reference's autograd interface (super_gnn/aggregator.py:15-177).

Forward:  out = A_local x  +  A_remote x_boundary      (boundary rows exchanged)
Backward: grad_x = A_local^T g + scatter(exchanged A_remote^T g)

Phase order and buffer roles follow the reference.  On the GPU the exchange is
asynchronous on NCCL's stream and overlaps the local SpMM, and where a copy or a
materialised fp32 buffer sat between two steps of the reference, the steps are
fused (``Aggregator.fused = True``, the default):

* forward, post mode: index_select into the send buffer (:48) + quantise
  -> one gather-quantise-pack kernel (the fp32 send buffer is not written);
* forward: dequantise into the receive buffer (:74-79) + remote SpMM (:88-92)
  -> one SpMM that reads the packed rows;
* backward, post mode: dequantise into the send buffer (:157-164) + index_add_
  (:173-175) -> one unpack-dequantise-scatter-add kernel;
* the first SpMM of a pass overwrites its output, so no zero-fill + re-read.

``Aggregator.fused = False`` runs the reference's unfused sequence step by step
on the same kernels (used to check the fused path).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import supergnn_ops
from .communicator import Communicator
from .ops.spmm_kernel import SPMM_backward, SPMM_forward, _algo_from_slot, choose_algo
from .quantizer import Quantizer_for_all_procs
from .time_recorder import TimeRecorder


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def _mean_scale(graph):
    """1 / in_degree per local node when the graph asks for the mean normalisation to be folded
    into the aggregation (``graph.fold_mean``); the caller then must not divide again."""
    return graph.inv_in_degrees if getattr(graph, "fold_mean", False) else None


def _transposed_values_with_scale(src, scale):
    """Edge values of A^T diag(scale): value_T[e] * scale[destination of e], built once per matrix and kept on
    it.  A streamed per-edge value is cheaper in the gather than a dependent lookup of scale[col[e]]."""
    cached = getattr(src, "_scaled_value_T", None)
    if cached is not None and cached[0] is scale:
        return cached[1]
    vals = scale[src.storage.row_T().to(torch.int64)]
    if src.storage.value_T() is not None:
        vals = vals * src.storage.value_T()
    src._scaled_value_T = (scale, vals.contiguous())
    return src._scaled_value_T[1]


def _spmm_overwrite(src, x, out, transpose: bool, row_scale=None, col_scale=None, accumulate: bool = False,
                    row_range=None):
    """First SpMM of a pass: ``out = A x`` (or ``A^T x``), no prior zero-fill needed; with ``accumulate`` the
    product is added to what ``out`` already holds.  ``row_range = (first row, last row + 1, first nonzero,
    nonzeros)`` restricts the product to those rows of the (transposed) matrix; ``out`` then has that many rows."""
    if transpose:
        rowptr, col, value = src.storage.colptr(), src.storage.row_T(), src.storage.value_T()
        if col_scale is not None:
            value, col_scale = _transposed_values_with_scale(src, col_scale), None
        slot_get, slot_set = src.get_work_range_for_transpose, src.set_work_range_for_transpose
    else:
        rowptr, col, value = src.csr()
        slot_get, slot_set = src.get_work_range, src.set_work_range
    algo = _algo_from_slot(slot_get())
    if algo < 0:
        algo = choose_algo(rowptr, col.numel())
        slot_set(torch.tensor([algo], dtype=torch.int32), torch.empty(0, dtype=torch.int32))
    if row_range is not None:
        a, b, e0, cnt = row_range
        supergnn_ops.spmm(rowptr[a:b + 1], col, value, x, out, b - a, None, None, algo=algo, accumulate=accumulate,
                          row_scale=None if row_scale is None else row_scale[a:b], col_scale=col_scale,
                          nnz_range=(e0, cnt))
        return
    supergnn_ops.spmm(rowptr, col, value, x, out, rowptr.numel() - 1, None, None, algo=algo, accumulate=accumulate,
                      row_scale=row_scale, col_scale=col_scale)


def _peer_cuts(remote_adj, recv_splits):
    """Per source peer: (first row, last row + 1, first nonzero, nonzeros) of its block of rows in A_remote^T
    (the received rows are grouped per peer, so are the rows of the transposed matrix).  Read back once."""
    cached = getattr(remote_adj, "_peer_cuts", None)
    if cached is not None and cached[0] == tuple(recv_splits):
        return cached[1]
    begin = [0]
    for n in recv_splits:
        begin.append(begin[-1] + int(n))
    colptr = remote_adj.storage.colptr()
    at = colptr[torch.tensor(begin, dtype=torch.int64, device=colptr.device)].tolist()
    cuts = [(begin[p], begin[p + 1], int(at[p]), int(at[p + 1] - at[p])) for p in range(len(recv_splits))]
    remote_adj._peer_cuts = (tuple(recv_splits), cuts)
    return cuts


def _by_peer(graph, num_bits: int, feat_len: int, quantized: bool, fused: bool) -> bool:
    """Produce the remote gradient rows one peer at a time?  ``Aggregator.remote_gradient_by_peer``: True, False,
    or "auto" = when the fp32 buffer for all of them would exceed 1 GiB."""
    mode = Aggregator.remote_gradient_by_peer
    if not (quantized and fused):
        return False
    if mode == "auto":
        return sum(graph.comm_splits.recv_splits) * feat_len * 4 > (1 << 30)
    return bool(mode)


class Aggregator(torch.autograd.Function):
    """The reference's autograd interface (super_gnn/aggregator.py:15-177):
    ``Aggregator.apply(graph, local_nodes_feat, layer, num_bits, is_pre_delay, is_training)``; the backward
    returns six gradients, one per argument.  The work itself is in ``aggregate_forward`` /
    ``aggregate_backward`` below, which the fused layers call directly with their extra keyword arguments."""
    fused = True
    # backward pass, quantised exchange: produce the gradient rows that go back to the peers (A_remote^T g) one
    # peer at a time, each block quantised and sent before the next is computed, so that the fp32 buffer
    # between the transposed aggregation and the quantiser holds one peer's rows instead of all of them
    remote_gradient_by_peer = "auto"

    @staticmethod
    def forward(ctx, graph, local_nodes_feat, layer, num_bits: int, is_pre_delay: bool, is_training: bool):
        return aggregate_forward(ctx, graph, local_nodes_feat, layer, num_bits, is_pre_delay, is_training)

    @staticmethod
    def backward(ctx, local_out_grad):
        return None, aggregate_backward(ctx, local_out_grad), None, None, None, None


def aggregate_forward(ctx, graph, local_nodes_feat, layer, num_bits: int, is_pre_delay: bool, is_training: bool, *,
                      out=None, accumulate: bool = False, local_work=None):
    """Forward aggregation; ``ctx`` is any object (an autograd context or a plain holder) that carries the
    state to ``aggregate_backward``.  Keyword-only extras, not part of the reference's interface: ``out``: an
    [n_local, F] buffer with contiguous rows that receives
    the result, added to what it holds when ``accumulate`` is set.  ``local_work``: a callable run in place of
    the local SpMM, while the exchange is in flight; it returns the packed [n_local, F] buffer the remote
    contributions are then added to (the caller has dealt with the local edges itself)."""
    ctx.graph = graph
    ctx.num_bits = num_bits
    ctx.is_pre_delay = is_pre_delay
    ctx.layer = layer
    _, world_size = _world()
    fused = Aggregator.fused
    x = local_nodes_feat
    if x.stride(-1) != 1 or (world_size > 1 and num_bits == 16 and not x.is_contiguous()):
        x = x.contiguous()  # every kernel takes a row stride; only the bf16 staging copy wants packed rows
    feat_len = x.size(-1)
    quantized = world_size > 1 and num_bits in (2, 4, 8) and is_training
    result = out
    if out is not None and out.stride(-1) != 1:
        out, result = None, out  # assemble in a packed buffer, then add / copy into the caller's rows
    rec = TimeRecorder.ctx
    scale = _mean_scale(graph)  # out = diag(scale) (A_local x + A_remote x_remote)

    comm_handle = None
    with rec.time_block("total_aggregator(inner)"):
        if world_size > 1:
            with rec.time_block("resize_comm_buffer"):
                graph.comm_buf.resize_buffer(graph.comm_splits, feat_len, num_bits)
                if num_bits not in (32, 16) and graph.comm_buf_for_quantization is not None:
                    graph.comm_buf_for_quantization.resize_buffer(graph.comm_splits, feat_len, num_bits)
            send_buf = graph.comm_buf.send_buf
            src = row_index = None
            with rec.time_block("pre_aggregation"):
                if is_pre_delay:
                    _spmm_overwrite(graph.adj_t_pre_post_aggr_to, x, send_buf, transpose=False)
                elif fused:
                    src, row_index = x, graph.idx_nodes_send_to_others  # gathered inside comm()
                else:
                    supergnn_ops.gather_rows(x, graph.idx_nodes_send_to_others, send_buf)
            with rec.time_block("total_communication(outer)"):
                comm_handle = Communicator.ctx.comm(graph.comm_splits, graph.comm_buf,
                                                    graph.comm_buf_for_quantization, f"forward{layer}",
                                                    is_training, "forward", src=src, row_index=row_index)

        with rec.time_block("local_aggregation"):
            n_out = graph.local_adj_t.sparse_size(0)
            if local_work is not None:
                assert out is None and not accumulate
                out = local_work()
                assert tuple(out.shape) == (n_out, feat_len) and out.stride(1) == 1
            elif out is None:
                out = torch.empty([n_out, feat_len], dtype=torch.float32, device=x.device)
                _spmm_overwrite(graph.local_adj_t, x, out, transpose=False, row_scale=scale)
            else:
                assert tuple(out.shape) == (n_out, feat_len)
                _spmm_overwrite(graph.local_adj_t, x, out, transpose=False, row_scale=scale, accumulate=accumulate)

        with rec.time_block("wait_for_async_comm"):
            if comm_handle is not None:
                comm_handle.wait()

        if world_size > 1 and sum(graph.comm_splits.recv_splits) != 0:
            remote_adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t
            qbuf = graph.comm_buf_for_quantization
            row_codes = quantized and Communicator.ctx.uses_row_codes(feat_len)
            n_recv = sum(graph.comm_splits.recv_splits)
            if quantized and fused:
                with rec.time_block("post_aggregation"):
                    rowptr, col, value = remote_adj.csr()
                    algo = _algo_from_slot(remote_adj.get_work_range())
                    if algo < 0:
                        algo = choose_algo(rowptr, col.numel())
                        remote_adj.set_work_range(torch.tensor([algo], dtype=torch.int32),
                                                  torch.empty(0, dtype=torch.int32))
                    if row_codes:
                        codes = supergnn_ops.rowcodes_view(qbuf.quantized_recv_data_buf, n_recv, feat_len, num_bits)
                        supergnn_ops.spmm_dequant_rowcodes(rowptr, col, value, codes,
                                                           qbuf.quantized_recv_params_buf_bf16[:n_recv], num_bits, out,
                                                           rowptr.numel() - 1, algo=algo, row_scale=scale)
                    else:
                        supergnn_ops.spmm_dequant(rowptr, col, value, qbuf.quantized_recv_data_buf,
                                                  qbuf.quantized_recv_params_buf_bf16,
                                                  qbuf.dequantized_work_range_per_proc, world_size, num_bits, out,
                                                  rowptr.numel() - 1, algo=algo, row_scale=scale)
            else:
                if quantized:
                    with rec.time_block("dequantization"):
                        if row_codes:
                            codes = supergnn_ops.rowcodes_view(qbuf.quantized_recv_data_buf, n_recv, feat_len,
                                                               num_bits)
                            supergnn_ops.unpack_dequant_rowcodes(codes, graph.comm_buf.recv_buf,
                                                                 qbuf.quantized_recv_params_buf_bf16, num_bits)
                        else:
                            supergnn_ops.dequantize_tensor_for_all_procs(
                                qbuf.quantized_recv_data_buf, graph.comm_buf.recv_buf,
                                qbuf.quantized_recv_params_buf_bf16, qbuf.dequantized_work_range_per_proc,
                                world_size, num_bits)
                with rec.time_block("post_aggregation"):
                    SPMM_forward(remote_adj, graph.comm_buf.recv_buf, out, row_scale=scale)
    if result is not None and result is not out:
        if accumulate:
            result.add_(out)
        else:
            result.copy_(out)
        return result
    return out

def aggregate_backward(ctx, local_out_grad, *, out=None, accumulate: bool = False, local_work=None):
    """Backward aggregation: returns the gradient with respect to the local node features.  Keyword-only
    extras (used by the fused layers).  ``out``: an [n_local, F] buffer with contiguous rows (any row stride) that receives the
    gradient; with ``accumulate`` the gradient is added to what it holds, so that a term computed elsewhere
    (the self path of a SAGE layer) needs no separate addition.  ``local_work``: a callable run in place of
    the local transposed SpMM, while the exchange is in flight; it returns the packed [n_local, F] buffer the
    gradients received from the peers are then added to."""
    graph = ctx.graph
    num_bits = ctx.num_bits
    is_pre_delay = ctx.is_pre_delay
    layer = f"backward{ctx.layer}"
    _, world_size = _world()
    fused = Aggregator.fused
    g = local_out_grad
    if g.stride(-1) != 1:
        g = g.contiguous()
    feat_len = g.size(-1)
    quantized = world_size > 1 and num_bits in (2, 4, 8)
    result = out
    if out is not None and out.stride(-1) != 1:
        out, result = None, out
    rec = TimeRecorder.ctx
    scale = _mean_scale(graph)  # gradient of the folded normalisation: the rows of g are scaled on the way in

    with rec.time_block("total_aggregator(inner)"):
        comm_handle = None
        if world_size > 1:
            with rec.time_block("resize_comm_buffer"):
                graph.comm_buf.resize_buffer(graph.comm_splits, feat_len, num_bits)
                if num_bits not in (32, 16) and graph.comm_buf_for_quantization is not None:
                    graph.comm_buf_for_quantization.resize_buffer(graph.comm_splits, feat_len, num_bits)
            remote_adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t
            n_remote = sum(graph.comm_splits.recv_splits)
            if n_remote != 0 and _by_peer(graph, num_bits, feat_len, quantized, fused):
                with rec.time_block("pre_aggregation"):
                    cuts = _peer_cuts(remote_adj, graph.comm_splits.recv_splits)
                    most = max(b - a for a, b, _, _ in cuts)
                    block = getattr(graph, "_peer_rows_buf", None)
                    if block is None or block.numel() < most * feat_len:
                        block = graph._peer_rows_buf = torch.empty(most * feat_len, dtype=torch.float32, device=g.device)
                    sender = Communicator.ctx.begin_backward_by_peer(graph.comm_splits, graph.comm_buf,
                                                                     graph.comm_buf_for_quantization, feat_len)
                    for p, (a, b, e0, cnt) in enumerate(cuts):
                        if b == a:
                            continue
                        rows = block[: (b - a) * feat_len].view(b - a, feat_len)
                        _spmm_overwrite(remote_adj, g, rows, transpose=True, col_scale=scale, row_range=(a, b, e0, cnt))
                        sender.send(p, rows)
                with rec.time_block("total_communication(outer)"):
                    comm_handle = sender.finish()
            else:
                remote_nodes_grad_buf = graph.comm_buf.recv_buf  # roles are swapped in the backward pass
                with rec.time_block("pre_aggregation"):
                    if remote_nodes_grad_buf.size(0) != 0:
                        _spmm_overwrite(remote_adj, g, remote_nodes_grad_buf, transpose=True, col_scale=scale)
                with rec.time_block("total_communication(outer)"):
                    comm_handle = Communicator.ctx.comm(graph.comm_splits, graph.comm_buf,
                                                        graph.comm_buf_for_quantization, layer, True, "backward")

        with rec.time_block("local_aggregation"):
            if local_work is not None:
                assert out is None and not accumulate
                local_nodes_grad = local_work()
                assert tuple(local_nodes_grad.shape) == (graph.local_adj_t.sparse_size(-1), feat_len)
                assert local_nodes_grad.stride(1) == 1
            elif out is not None:
                local_nodes_grad = out
                assert tuple(local_nodes_grad.shape) == (graph.local_adj_t.sparse_size(-1), feat_len)
            else:
                local_nodes_grad = torch.empty([graph.local_adj_t.sparse_size(-1), feat_len], dtype=torch.float32,
                                               device=g.device)
            if local_work is None:
                _spmm_overwrite(graph.local_adj_t, g, local_nodes_grad, transpose=True, col_scale=scale,
                                accumulate=accumulate and out is not None)

        with rec.time_block("wait_for_async_comm"):
            if comm_handle is not None:
                comm_handle.wait()

        if world_size > 1 and sum(graph.comm_splits.send_splits) != 0:
            qbuf = graph.comm_buf_for_quantization
            send_buf = graph.comm_buf.send_buf
            row_codes = quantized and Communicator.ctx.uses_row_codes(feat_len)
            codes = None
            if row_codes:  # the gradient rows this rank's nodes received, one run of F*bits/8 bytes per row
                codes = supergnn_ops.rowcodes_view(qbuf.quantized_send_data_buf,
                                                   sum(graph.comm_splits.send_splits), feat_len, num_bits)
            if quantized and fused and not is_pre_delay:
                with rec.time_block("post_aggregation"):
                    if row_codes:
                        supergnn_ops.unpack_dequant_rowcodes(codes, local_nodes_grad,
                                                             qbuf.quantized_send_params_buf_bf16, num_bits,
                                                             row_index=graph.idx_nodes_send_to_others)
                    else:
                        supergnn_ops.dequantize_tensor_for_all_procs(
                            qbuf.quantized_send_data_buf, local_nodes_grad, qbuf.quantized_send_params_buf_bf16,
                            qbuf.quantized_work_range_per_proc, world_size, num_bits,
                            row_index=graph.idx_nodes_send_to_others)
            elif quantized and fused and is_pre_delay:
                with rec.time_block("post_aggregation"):
                    # local_grad += adj_to^T @ dequantise(received rows), straight from the wire format
                    adj_to = graph.adj_t_pre_post_aggr_to
                    colptr, row_T, value_T = adj_to.storage.colptr(), adj_to.storage.row_T(), adj_to.storage.value_T()
                    algo = _algo_from_slot(adj_to.get_work_range_for_transpose())
                    if algo < 0:
                        algo = choose_algo(colptr, row_T.numel())
                        adj_to.set_work_range_for_transpose(torch.tensor([algo], dtype=torch.int32),
                                                            torch.empty(0, dtype=torch.int32))
                    if row_codes:
                        supergnn_ops.spmm_dequant_rowcodes(colptr, row_T, value_T, codes,
                                                           qbuf.quantized_send_params_buf_bf16[:codes.size(0)],
                                                           num_bits, local_nodes_grad, colptr.numel() - 1, algo=algo)
                    else:
                        supergnn_ops.spmm_dequant(colptr, row_T, value_T, qbuf.quantized_send_data_buf,
                                                  qbuf.quantized_send_params_buf_bf16,
                                                  qbuf.quantized_work_range_per_proc, world_size, num_bits,
                                                  local_nodes_grad, colptr.numel() - 1, algo=algo)
            else:
                if quantized:
                    with rec.time_block("dequantization"):
                        if row_codes:
                            supergnn_ops.unpack_dequant_rowcodes(codes, send_buf,
                                                                 qbuf.quantized_send_params_buf_bf16, num_bits)
                        else:
                            supergnn_ops.dequantize_tensor_for_all_procs(
                                qbuf.quantized_send_data_buf, send_buf, qbuf.quantized_send_params_buf_bf16,
                                qbuf.quantized_work_range_per_proc, world_size, num_bits)
                with rec.time_block("post_aggregation"):
                    if is_pre_delay:
                        SPMM_backward(graph.adj_t_pre_post_aggr_to, send_buf, local_nodes_grad)
                    else:
                        supergnn_ops.scatter_add_rows(send_buf, graph.idx_nodes_send_to_others, local_nodes_grad)

    if result is not None and result is not local_nodes_grad:
        if accumulate:
            result.add_(local_nodes_grad)
        else:
            result.copy_(local_nodes_grad)
        local_nodes_grad = result
    return local_nodes_grad
