/*
 * supergnn_b200 — C ABI of the B200 (sm_100a) implementation of SuperGNN's
 * full-batch GraphSAGE hot path: CSR SpMM aggregation, per-row min-max
 * quantize/pack and unpack/dequantize of boundary-node features, and the row
 * gather / scatter-add either side of the boundary exchange.
 *
 * Conventions (all entry points)
 *   - plain C: pointers and sizes only, no framework types;
 *   - every pointer named d_* is a DEVICE pointer on the current CUDA device; it
 *     is borrowed for the duration of the enqueued work, never freed or retained;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); work is enqueued and the call returns without synchronising,
 *     unless stated otherwise;
 *   - the return value is a status: 0 = ok, non-zero = SGNN_ERR_*; nothing
 *     throws or exits; sgnn_last_error_string() describes the last failure on the
 *     calling thread;
 *   - arguments are validated on the host BEFORE anything is launched, so a
 *     rejected call leaves the GPU untouched;
 *   - dense matrices are row-major fp32 with a leading dimension in elements.
 *
 * "Reference" below is zhuangbility111/super_gnn; citations are file:line
 * inside that project and name the interface each entry point replaces.
 */
#ifndef SUPERGNN_B200_H
#define SUPERGNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SGNN_OK 0
#define SGNN_ERR_INVALID_ARGUMENT 1 /* null pointer, negative size, bad bit width, misaligned ... */
#define SGNN_ERR_CUDA 2             /* a CUDA runtime call failed; see the error string */
#define SGNN_ERR_UNSUPPORTED 3      /* valid request outside what the kernels cover */
#define SGNN_ERR_TOO_LARGE 4        /* size beyond a stated limit */
#define SGNN_ERR_WORKSPACE 5        /* workspace missing or too small */

/* SpMM algorithm selector */
#define SGNN_SPMM_AUTO 0      /* = SGNN_SPMM_NNZ_SPLIT: safe for any degree distribution */
#define SGNN_SPMM_ROW_SPLIT 1 /* one warp (or sub-warp) per row; deterministic; for near-uniform degrees */
#define SGNN_SPMM_NNZ_SPLIT 2 /* merge-path style: equal nonzero chunks per warp; rows cut by a chunk end
                                 are finished with fp32 atomic adds (order not fixed) */
#define SGNN_SPMM_NNZ_SPLIT_STAGED 3 /* the same split with the gathered rows staged through shared memory by
                                 cp.async (more bytes in flight per SM); fp32 operand rows of 65..512 columns,
                                 16-byte aligned; other cases run SGNN_SPMM_NNZ_SPLIT.  Slower than
                                 SGNN_SPMM_NNZ_SPLIT on the graphs measured so far; never chosen by default. */

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int sgnn_version(void);

/* Text of the last error raised on the calling thread ("" if none).
 * Replaces the reference's AT_ASSERTM / TORCH_CHECK exceptions
 * (super_gnn/ops/csrc/utils.h:12-13, quantization_arm.cpp:501). */
const char *sgnn_last_error_string(void);

/* ---------------------------------------------------------------------------
 * CSR SpMM   Y[m, 0:N] (+)= sum_{e in row m} val[e] * X[col[e], 0:N]
 *
 * Replaces supergnn_ops.spmm (super_gnn/ops/csrc/spmm.h:3-6, spmm.cpp:594-608;
 * hot loop spmm.cpp:348-539 with kernel_1xN :87-162), called from
 * super_gnn/ops/spmm_kernel.py:65 (forward, CSR of A) and :91 (backward, CSR of
 * A^T).  The reference's per-thread row_split / col_split arguments have no
 * meaning on a GPU and are replaced by `algo`.
 *
 *   d_rowptr  int64[M+1]; d_col int32[nnz] (values in [0,K)); d_val fp32[nnz] or
 *             NULL for an all-ones matrix (sum aggregation);
 *   d_X       fp32[K, ldx], d_Y fp32[M, ldy];
 *   accumulate != 0: Y += A X (the reference contract: the caller zeroes Y);
 *   accumulate == 0: Y  = A X (rows without nonzeros become 0).
 *   nnz must equal rowptr[M]; it is passed in so that no device read is needed.
 *   d_row_scale fp32[M] or NULL, d_col_scale fp32[K] or NULL: the product becomes
 *   diag(row_scale) A diag(col_scale) X.  With row_scale = 1/in_degree this folds the mean
 *   normalisation that follows the aggregation (super_gnn/layers/sageconv.py:76-78) into the
 *   forward SpMM, and with col_scale = 1/in_degree its gradient into the transposed one.
 * ------------------------------------------------------------------------- */
int sgnn_spmm_csr_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                      const float *d_X, int64_t ldx, float *d_Y, int64_t ldy, int64_t M, int64_t K,
                      int64_t N, int accumulate, int algo, const float *d_row_scale, const float *d_col_scale,
                      void *stream);

/* The same product over a RANGE OF ROWS of a larger CSR matrix: d_rowptr points at the first row of the
 * range (M + 1 entries, still holding positions in the whole matrix), d_col / d_val at the WHOLE arrays,
 * nnz_begin = the value of d_rowptr[0] and nnz the number of nonzeros in the range (both known to the
 * caller, so that no device read is needed); d_Y / d_row_scale are those of the range.  Used to produce the
 * gradient rows that go back to one peer at a time (the rows of A_remote^T are grouped per peer,
 * super_gnn/aggregator.py:125-131), so that the fp32 buffer between the transposed aggregation and the
 * quantiser holds one peer's rows instead of all of them. */
int sgnn_spmm_csr_rows_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz_begin,
                           int64_t nnz, const float *d_X, int64_t ldx, float *d_Y, int64_t ldy, int64_t M,
                           int64_t K, int64_t N, int accumulate, int algo, const float *d_row_scale,
                           const float *d_col_scale, void *stream);

/* Structural check of a CSR matrix on the device (debugging aid; the reference has no bounds checks on `col`
 * or the splits, super_gnn/ops/csrc/spmm.cpp:348-539, and neither have the kernels here).  d_flags int64[4], zero
 * on entry, receives counts: [0] rows that end before they start, [1] column indices outside [0, K),
 * [2] rowptr[0] != 0, [3] rowptr[M] != nnz.  Nothing traps; the host reads the counts. */
int sgnn_csr_check(const int64_t *d_rowptr, const int32_t *d_col, int64_t M, int64_t K, int64_t nnz, int64_t *d_flags,
                   void *stream);

/* Degree statistics of a CSR matrix, used once per matrix to choose `algo`
 * (it takes the place of the reference's cached per-thread row split,
 * super_gnn/ops/spmm_kernel.py:8-29, 49-58).  Writes d_stats int64[2] =
 * {max row length, number of empty rows}.  d_stats must be zero on entry. */
int sgnn_csr_row_stats(const int64_t *d_rowptr, int64_t M, int64_t *d_stats, void *stream);

/* ---------------------------------------------------------------------------
 * CSR transpose (CSR of A^T, rows sorted), built once per matrix for the
 * backward aggregation.  Replaces the torch_sparse storage calls
 * colptr() / row_T() / value_T() used by super_gnn/ops/spmm_kernel.py:77-79.
 *
 *   in : d_rowptr int64[M+1], d_col int32[nnz], d_val fp32[nnz] or NULL
 *   out: d_colptr int64[K+1], d_row_T int32[nnz], d_val_T fp32[nnz] (ignored if d_val NULL)
 *   d_workspace: at least sgnn_csr_transpose_workspace_bytes(M, K, nnz) bytes,
 *   256-byte aligned.  Within a column the rows come out in ascending order
 *   (stable), so the result does not depend on scheduling.
 * ------------------------------------------------------------------------- */
size_t sgnn_csr_transpose_workspace_bytes(int64_t M, int64_t K, int64_t nnz);
int sgnn_csr_transpose(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t M,
                       int64_t K, int64_t nnz, int64_t *d_colptr, int32_t *d_row_T, float *d_val_T,
                       void *d_workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------
 * CSR transpose that allocates nothing.  No counterpart in the reference.
 *
 * Same result as sgnn_csr_transpose, for callers that cannot allocate device
 * memory: a process whose GPU memory is handed out entirely by a framework's
 * caching pool (a raw cudaMalloc would fail or fragment it), or a latency-bound
 * loop where the implicit synchronisation of an allocation is not acceptable.
 * The scratch is a static 48 MiB device array inside the library (every GPU that
 * loads the library holds it until the process exits).  Inputs and outputs are
 * still the caller's.
 *
 *   Limits: nnz <= SGNN_TRANSPOSE_NOALLOC_MAX_NNZ and K <= SGNN_TRANSPOSE_NOALLOC_MAX_COLS;
 *   larger sizes are rejected with SGNN_ERR_TOO_LARGE before anything is launched.
 *   The first call on a device looks up the device address of the scratch (with that
 *   device current); make that first call outside any stream capture.  It is also the
 *   moment at which the CUDA driver may make the library's module data resident on that
 *   device, so the 48 MiB of the array can leave the free-memory count then (not later).
 *   All calls on a device share the one scratch array: two calls whose work overlaps on
 *   the GPU (different streams) race; calls on one stream are ordered and safe.  The
 *   array keeps the previous call's contents; what must start at zero is cleared by
 *   each call.  No cudaMalloc, cudaFree or allocating library routine is called.
 * ------------------------------------------------------------------------- */
#define SGNN_TRANSPOSE_NOALLOC_MAX_NNZ (1 << 20)  /* 1 048 576 nonzeros */
#define SGNN_TRANSPOSE_NOALLOC_MAX_COLS (1 << 20) /* 1 048 576 columns  */
int sgnn_csr_transpose_noalloc(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t M,
                               int64_t K, int64_t nnz, int64_t *d_colptr, int32_t *d_row_T, float *d_val_T,
                               void *stream);

/* ---------------------------------------------------------------------------
 * Fused per-row min-max quantize + pack, per destination peer.
 *
 * Replaces supergnn_ops.quantize_tensor_for_all_procs
 * (super_gnn/ops/csrc/quantization_arm.cpp:496-578; kernels :79-301; packed
 * offsets :21-77), called from super_gnn/quantizer.py:81-84.  Semantics: IEEE
 * fp32 subtract and divide, round half to even (the reference's x86 ops and its
 * SVE remainder path), NOT the SVE reciprocal estimate.
 *
 *   d_X            fp32[*, ldx]: the source rows;
 *   d_row_index    int64[S] or NULL.  NULL: row r of the send buffer is X[r].
 *                  Otherwise it is X[row_index[r]]: this fuses the reference's
 *                  index_select into the send buffer (super_gnn/aggregator.py:48)
 *                  with the quantisation, so the fp32 send buffer is never written;
 *   d_work_range   int32[P+1], cumulative rows per peer, work_range[P] == S
 *                  (super_gnn/data_manager/CommBuffer.py:37-43);
 *   bits           2, 4 or 8;  EPB = 8/bits rows share one packed row;
 *   d_packed       uint8[sum_p ceil(n_p/EPB), F] (row stride exactly F bytes): inside
 *                  peer p, byte[off_p + i/EPB, k] |= code(i,k) << ((EPB-1-i%EPB)*bits);
 *                  missing rows of a peer's last group contribute zero bits;
 *   d_params       fp32[S,2] = (zero_point, scale) per row, or NULL;
 *   d_params_bf16  bf16[S,2] (round to nearest even), or NULL: the form the
 *                  parameters take on the wire (super_gnn/communicator.py:283-291).
 *   P <= SGNN_MAX_PEERS.
 * ------------------------------------------------------------------------- */
#define SGNN_MAX_PEERS 4096
int sgnn_quant_pack_rows(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                         const int32_t *d_work_range, int P, int bits, uint8_t *d_packed, float *d_params,
                         uint16_t *d_params_bf16, void *stream);

/* ---------------------------------------------------------------------------
 * One-sided boundary exchange: the same quantise + pack, but every packed row and every bf16
 * (zero_point, scale) pair is stored directly into the receive buffers of the destination
 * peer (peer device memory reached through NVLink / NVSwitch), so the quantisation and the
 * all-to-all of super_gnn/communicator.py:268-301 (quantise, params all_to_all, data
 * all_to_all) are one kernel.  Plain stores to peer memory only.
 *
 *   d_peer_packed[p]       address (uint8*) of peer p's packed receive buffer, row stride F;
 *   d_peer_packed_row0[p]  packed row at which this rank's segment starts in that buffer;
 *   d_peer_params[p]       address of peer p's bf16[.,2] parameter receive buffer;
 *   d_peer_params_row0[p]  row at which this rank's segment starts there;
 *   d_params_fp32          optional local copy of the fp32 parameters, [S,2].
 * The four tables are DEVICE arrays of length P.  The caller orders the exchange (peers
 * must have finished reading the previous contents before this runs, and must not read
 * before every sender's kernel has completed: a barrier either side).
 * Requires F % 4 == 0, F <= 512 and 16-byte aligned source rows.
 * ------------------------------------------------------------------------- */
int sgnn_quant_pack_rows_p2p(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                             const int32_t *d_work_range, int P, int bits, const uint64_t *d_peer_packed,
                             const int64_t *d_peer_packed_row0, const uint64_t *d_peer_params,
                             const int64_t *d_peer_params_row0, float *d_params_fp32, void *stream);

/* ---------------------------------------------------------------------------
 * Unpack + dequantize, per source peer:  out = zero_point + code * scale (one fused
 * multiply-add).
 *
 * Replaces supergnn_ops.dequantize_tensor_for_all_procs
 * (super_gnn/ops/csrc/quantization_arm.cpp:580-633; kernels :303-431), called
 * from super_gnn/quantizer.py:86-89.
 *
 *   d_params fp32[S,2] or NULL; d_params_bf16 bf16[S,2] or NULL — exactly one is
 *   given; the bf16 form is widened exactly (what communicator.py:293-294 does);
 *   d_row_index int64[S] or NULL.  NULL: row r is stored to out[r] (overwrite).
 *   Otherwise row r is ADDED to out[row_index[r]] with fp32 atomic adds: this
 *   fuses the backward index_add_ (super_gnn/aggregator.py:173-175) with the
 *   dequantisation, so the fp32 gradient buffer is never written.
 * ------------------------------------------------------------------------- */
int sgnn_unpack_dequant_rows(const uint8_t *d_packed, const float *d_params, const uint16_t *d_params_bf16,
                             int64_t S, int64_t F, const int32_t *d_work_range, int P, int bits,
                             float *d_out, int64_t ldo, const int64_t *d_row_index, void *stream);

/* ---------------------------------------------------------------------------
 * SpMM whose dense operand is still in wire format: the received packed rows
 * are dequantised inside the gather, so the fp32 receive buffer is never
 * materialised.   Y[m,:] += sum_e val[e] * (zp[c] + code[c,:] * scale[c]),
 * c = col[e] indexing the received rows (grouped per source peer).
 *
 * Fuses supergnn_ops.dequantize_tensor_for_all_procs with the remote-neighbour
 * supergnn_ops.spmm that follows it (super_gnn/aggregator.py:74-79 + :88-92).
 * Always accumulates (the local aggregation has already written Y).  d_row_scale fp32[M] or
 * NULL scales the added rows (mean normalisation, as in sgnn_spmm_csr_f32).
 * ------------------------------------------------------------------------- */
int sgnn_spmm_csr_dequant_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val,
                              int64_t nnz, const uint8_t *d_packed, const float *d_params,
                              const uint16_t *d_params_bf16, int64_t R, int64_t F,
                              const int32_t *d_work_range, int P, int bits, float *d_Y, int64_t ldy,
                              int64_t M, int algo, const float *d_row_scale, void *stream);

/* ---------------------------------------------------------------------------
 * "Row codes": the same quantised boundary rows (same min, scale, rounding and therefore the same
 * codes as sgnn_quant_pack_rows) in a layout that gives every row its own F*bits/8 contiguous
 * bytes.  The reference's wire format (quantization_arm.cpp:177-185) interleaves EPB = 8/bits rows
 * in every byte, which suits its streaming dequantiser but makes a consumer that needs ONE row —
 * the gather of the fused dequantise-SpMM — move F bytes per row at every bit width.  When both
 * ends of the exchange are this library (super_gnn/communicator.py:221-306 replaced on both
 * sides) the rows travel and are consumed in this layout instead; the bytes are a fixed
 * permutation of the reference's (the tests invert it and compare with the oracle's bytes).
 *
 *   Row r starts at byte r * F*bits/8.  Quad q = features 4q..4q+3 is one little-endian field of
 *   4*bits bits, feature j of the quad at bit j*bits.  Position of quad q in the row: q for
 *   F <= 128, else (q % 32) * NV + q / 32 with NV = F / 128 (the quads one lane of a warp owns are
 *   adjacent).  No per-peer padding: rows are indexed exactly as the fp32 rows are.
 *   Supported widths: F % 4 == 0 and (F <= 128 or F == 256 or F == 512); sgnn_rowcodes_width_supported.
 *   fp32 rows must be 16-byte aligned; a code buffer to NV*bits/2 bytes where it is written and to bits/2
 *   bytes where it is read (any row boundary of a 16-byte aligned buffer qualifies).
 *
 * sgnn_quant_pack_rowcodes      = sgnn_quant_pack_rows in this layout (no work range: there is no grouping);
 * sgnn_quant_pack_rowcodes_p2p  = sgnn_quant_pack_rows_p2p: row r of peer p's segment is stored to row
 *                                 d_peer_row0[p] + r - work_range[p] of that peer's code and bf16-parameter buffers;
 * sgnn_unpack_dequant_rowcodes  = sgnn_unpack_dequant_rows (store, or scatter-add with d_row_index);
 * sgnn_spmm_csr_dequant_rowcodes_f32 = sgnn_spmm_csr_dequant_f32: Y += A dequantise(codes), a gathered row
 *                                 costs F*bits/8 + 4 (bf16 parameters) bytes.
 * ------------------------------------------------------------------------- */
int sgnn_rowcodes_width_supported(int64_t F);
int sgnn_quant_pack_rowcodes(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                             int bits, uint8_t *d_codes, float *d_params, uint16_t *d_params_bf16, void *stream);
int sgnn_quant_pack_rowcodes_p2p(const float *d_X, int64_t ldx, const int64_t *d_row_index, int64_t S, int64_t F,
                                 const int32_t *d_work_range, int P, int bits, const uint64_t *d_peer_codes,
                                 const uint64_t *d_peer_params, const int64_t *d_peer_row0, float *d_params_fp32,
                                 void *stream);
int sgnn_unpack_dequant_rowcodes(const uint8_t *d_codes, const float *d_params, const uint16_t *d_params_bf16,
                                 int64_t S, int64_t F, int bits, float *d_out, int64_t ldo,
                                 const int64_t *d_row_index, void *stream);
int sgnn_spmm_csr_dequant_rowcodes_f32(const int64_t *d_rowptr, const int32_t *d_col, const float *d_val, int64_t nnz,
                                       const uint8_t *d_codes, const float *d_params, const uint16_t *d_params_bf16,
                                       int64_t R, int64_t F, int bits, float *d_Y, int64_t ldy, int64_t M, int algo,
                                       const float *d_row_scale, void *stream);

/* ---------------------------------------------------------------------------
 * Barrier among the ranks of the one-sided exchange (one GPU per rank), with a bounded wait.
 * Stands where the reference orders its exchange with dist.barrier() before the collectives
 * (super_gnn/communicator.py:95, 279): before the peer stores "every peer has consumed what it
 * received last time", after them "every sender's stores have landed".
 *
 *   d_flag_ptrs int64[world]: device address of every rank's flag array (uint32[world], zero at
 *   the start, in memory all ranks map).  Rank r stores `epoch` into flag r of every peer and
 *   waits until each of its own flags holds `epoch` or more; epochs start at 1, grow by one per
 *   barrier and are the same on all ranks (wrap-around is handled).
 *   A wait longer than timeout_us gives up WITHOUT trapping: the kernel stores `epoch` into
 *   status[p] for every peer p that did not arrive and returns, the context stays usable.
 *   status: uint32[world], zero at the start, in pinned host memory (the device writes it, the
 *   host reads it without a synchronisation of its own) or in device memory.
 *   One block of SGNN_PEER_BARRIER_MAX_RANKS threads; world == 1 launches nothing.
 *   The ranks' kernels wait on one another: one rank per GPU, never several ranks on one GPU.
 * ------------------------------------------------------------------------- */
#define SGNN_PEER_BARRIER_MAX_RANKS 64
int sgnn_peer_barrier(const int64_t *d_flag_ptrs, int rank, int world, uint32_t epoch, int64_t timeout_us,
                      uint32_t *status, void *stream);

/* ---------------------------------------------------------------------------
 * Single-segment row-group packing with caller-supplied min / scale.
 * Replaces the x86 supergnn_ops.quantize_tensor(input, output, min, scale, bits)
 * and dequantize_tensor (super_gnn/ops/csrc/quantization_x86.cpp:17-102, 104-168).
 * d_packed is uint8[ceil(S/EPB), F].
 * ------------------------------------------------------------------------- */
int sgnn_quantize_tensor(const float *d_X, int64_t S, int64_t F, const float *d_min, const float *d_scale,
                         int bits, uint8_t *d_packed, void *stream);
int sgnn_dequantize_tensor(const uint8_t *d_packed, int64_t S, int64_t F, const float *d_min,
                           const float *d_scale, int bits, float *d_out, void *stream);

/* ---------------------------------------------------------------------------
 * Per-row bit width, packed along the feature axis ("v1").
 * Replaces supergnn_ops.quantize_tensor_v1 / dequantize_tensor_v1
 * (super_gnn/ops/csrc/quantization_x86.cpp:170-253, 255-312), called from
 * super_gnn/quantizer.py:55,61.
 *   d_params fp32[S,3] = (bits, zero_point, scale); bits is read, the other two
 *   are written by the quantiser and read by the dequantiser;
 *   d_range int64[S+1]: first output byte of each row (quantizer.py:66-73).
 * A row whose bits is not 2, 4 or 8 is skipped (the reference prints and skips).
 * ------------------------------------------------------------------------- */
int sgnn_quantize_rows_v1(const float *d_X, int64_t S, int64_t F, const int64_t *d_range, float *d_params,
                          uint8_t *d_out, void *stream);
int sgnn_dequantize_rows_v1(const uint8_t *d_in, int64_t S, int64_t F, const int64_t *d_range,
                            const float *d_params, float *d_out, void *stream);

/* ---------------------------------------------------------------------------
 * torch.quantize_per_channel-compatible layout ("v2"): code = rne(x * (1/scale) + zero_point) (one fused
 * multiply-add; 1/scale taken as 1 when scale is 0), one bit width for all rows, packed along the feature axis
 * with the first element in the LOW bits; decode (code - zero_point) * scale.
 * Replaces supergnn_ops.quantize_tensor_v2_torch / dequantize_tensor_v2_torch
 * (super_gnn/ops/csrc/quantization_x86.cpp:314-388, 390-459; exported at ops.cpp:22-23; no caller on the
 * GraphSAGE path, kept so that the export list is a superset of the reference's x86 one).
 *   d_range int64[S+1]: first output byte of each row (super_gnn/quantizer.py:66-73); d_zero_points,
 *   d_scales fp32[S].
 * ------------------------------------------------------------------------- */
int sgnn_quantize_rows_v2(const float *d_X, int64_t S, int64_t F, const int64_t *d_range, const float *d_zero_points,
                          const float *d_scales, int bits, uint8_t *d_out, void *stream);
int sgnn_dequantize_rows_v2(const uint8_t *d_in, int64_t S, int64_t F, const int64_t *d_range,
                            const float *d_zero_points, const float *d_scales, int bits, float *d_out, void *stream);

/* ---------------------------------------------------------------------------
 * Row gather  out[r,:] = X[index[r],:]   and scatter-add  out[index[r],:] += src[r,:].
 * Replace torch.index_select(..., out=send_buf) and index_add_ on the boundary
 * rows (super_gnn/aggregator.py:48 and :173-175).  index is int64[S]; repeated
 * indices are allowed (a node sent to several peers); the scatter uses fp32
 * atomic adds.
 * ------------------------------------------------------------------------- */
int sgnn_gather_rows(const float *d_X, int64_t ldx, const int64_t *d_index, int64_t S, int64_t F,
                     float *d_out, int64_t ldo, void *stream);
int sgnn_scatter_add_rows(const float *d_src, int64_t lds, const int64_t *d_index, int64_t S, int64_t F,
                          float *d_out, int64_t ldo, void *stream);

/* ---------------------------------------------------------------------------
 * Fused epilogue of a hidden GraphSAGE layer and its backward:
 *     y = relu(LayerNorm(dropout(h + bias)))
 * Replaces the chain of framework ops the reference runs between two aggregations
 * (bias add super_gnn/layers/sageconv.py:86-87; F.dropout, LayerNorm, F.relu
 * examples/graphsage/sage.py:189-196) with one pass over the activations each way.
 *
 * forward:  d_h fp32[n, ldh] is read (not modified); d_y[n, ldy] receives the output; d_stats fp32[n, 2] receives
 *           (mean, reciprocal standard deviation) of every row.  d_bias may be NULL.  LayerNorm over the H columns
 *           of a row, biased variance, eps inside the square root, affine gamma/beta.
 * dropout_mode: 0 none (inference); 1 counter-based mask from `seed` (not stored: the backward
 *           regenerates it; element kept with probability 1-p and scaled by 1/(1-p));
 *           2 caller-supplied mask d_mask[n, ldm] that already carries the scale (reproducible
 *           runs against a CPU reference).
 * backward: reads d_gy and the SAME d_h, d_stats, bias, gamma, beta (and mask / seed) the forward saw, recomputes
 *           the normalised values and the sign of the output from them with the forward's own roundings, writes
 *           d_gh[n, ldgh] (gradient w.r.t. h) and d_grads3 fp32[3, H] = column sums (grad_bias, grad_gamma,
 *           grad_beta), reduced in a fixed order through d_partials fp32[sgnn_epilogue_blocks(), 3, H] (scratch).
 *           Nothing of size [n, H] is stored between the two calls besides h itself.
 * H % 4 == 0, H <= 512, 16-byte aligned rows.
 * ------------------------------------------------------------------------- */
int sgnn_epilogue_blocks(void);
int sgnn_sage_epilogue_forward(const float *d_h, int64_t ldh, const float *d_bias, const float *d_gamma,
                               const float *d_beta, const float *d_mask, int64_t ldm, int dropout_mode,
                               uint64_t seed, float p, float eps, float *d_y, int64_t ldy, float *d_stats, int64_t n,
                               int64_t H, void *stream);
int sgnn_sage_epilogue_backward(const float *d_gy, int64_t ldgy, const float *d_h, int64_t ldh, const float *d_stats,
                                const float *d_bias, const float *d_gamma, const float *d_beta, const float *d_mask,
                                int64_t ldm, int dropout_mode, uint64_t seed, float p, float *d_gh, int64_t ldgh,
                                float *d_partials, float *d_grads3, int64_t n, int64_t H, void *stream);
/* The scaled keep mask that dropout_mode 1 applies for (seed, p), materialised as fp32[n, H]. */
int sgnn_dropout_mask(uint64_t seed, float p, int64_t n, int64_t H, float *d_out, void *stream);

/* ---------------------------------------------------------------------------
 * Training loss of the node classifier and its gradient in one pass:
 *     logp = log_softmax(logits + bias, dim=1)
 *     loss = - sum over rows r with mask[r] != 0 of logp[r, labels[r]] * inv_count
 *     grad[r, c] = mask[r] * inv_count * (exp(logp[r, c]) - [c == labels[r]])
 * Replaces F.log_softmax at the end of the model (examples/graphsage/sage.py:211) followed by
 * F.nll_loss(out[mask], labels[mask], reduction="sum") / num_train in the training loop
 * (examples/graphsage/train.py:41-44) and the autograd walk back through both.
 *
 *   d_logits fp32[n, ld] (C columns used), d_bias fp32[C] or NULL, d_labels int64[n] (read only where the mask
 *   is set; a label outside [0, C), such as the -1 of an unlabelled node, takes the row out of the loss),
 *   d_mask uint8[n] or NULL (= every row), inv_count = 1 / number of training nodes of ALL partitions.
 *   d_grad fp32[n, ldg]: Cg >= C columns are written, columns [C, Cg) with zeros (padding of the class dimension).
 *   d_partials fp32[sgnn_softmax_nll_blocks()] scratch; d_loss fp32[1].  Sums in a fixed order (reproducible).
 *   C, Cg <= 256.
 * ------------------------------------------------------------------------- */
int sgnn_softmax_nll_blocks(void);
int sgnn_softmax_nll_loss(const float *d_logits, int64_t ld, const float *d_bias, const int64_t *d_labels,
                          const uint8_t *d_mask, float inv_count, int64_t n, int64_t C, float *d_grad, int64_t ldg,
                          int64_t Cg, float *d_partials, float *d_loss, void *stream);

/* ---------------------------------------------------------------------------
 * Dense fp32 GEMM with fp32 accuracy on the tensor cores, for the two linear maps of a
 * GraphSAGE layer and their gradients: the work the reference hands to torch.nn.Linear
 * (self.lin_neigh / self.lin_self in super_gnn/layers/sageconv.py:62-89, forward
 * `lin_neigh(out) + lin_self(x)`, and the autograd backward of both).
 *
 *   SGNN_GEMM_NT: C[M,N] = A[M,K] B[N,K]^T + beta C     y = x W^T; with B = W^T: grad_x = g W
 *   SGNN_GEMM_TN: C[M,N] = A[K,M]^T B[K,N] + beta C     grad_W = g^T x (K = number of nodes)
 *
 * All matrices are row-major fp32 with leading dimensions lda/ldb/ldc (multiples of 4
 * elements, 16-byte aligned bases).  Every fp32 operand is split into three bf16 terms in
 * the kernel and the nine cross products are accumulated in fp32 (tcgen05 MMAs): the
 * result is at least as close to the exact product as a plain fp32 GEMM's, so the
 * 1e-5 layer-output contract holds (TF32 would not meet it).  With SGNN_GEMM_SIX_PRODUCTS
 * or-ed into op the three smallest products (a1 b2, a2 b1, a2 b2: at most 2^-23 of a0 b0 per
 * element pair, the order of one fp32 rounding) are left out: two thirds of the tensor-core
 * work, an error against the exact product of the size a plain fp32 GEMM makes.
 * SGNN_GEMM_TN splits K over
 * the SMs and combines the partial tiles through d_workspace in a fixed order.
 * d_workspace: at least the bytes sgnn_gemm_f32_workspace_bytes reports (may be 0 -> NULL
 * allowed); it must not be shared by calls that can run concurrently.
 * M, N, K < 2^31.  M == 0 or N == 0 is a no-op.
 * ------------------------------------------------------------------------- */
#define SGNN_GEMM_NT 0
#define SGNN_GEMM_TN 1
#define SGNN_GEMM_SIX_PRODUCTS 16 /* or-ed into op: see above */
int sgnn_gemm_f32_workspace_bytes(int op, int64_t M, int64_t N, int64_t K, size_t *bytes);
int sgnn_gemm_f32(int op, const float *d_A, int64_t lda, const float *d_B, int64_t ldb, float *d_C, int64_t ldc,
                  int64_t M, int64_t N, int64_t K, float beta, void *d_workspace, size_t workspace_bytes,
                  void *stream);

/* ---------------------------------------------------------------------------
 * Minimum vertex cover of a bipartite graph (HOST arrays, set-up code): Hopcroft-Karp
 * matching + Koenig's construction from the unmatched left vertices.
 *
 * Replaces the networkx-derived Python of the reference's pre/post-aggregation
 * planner: VertexCoverFinder.find_minimum_vertex_cover
 * (super_gnn/data_manager/VertexCoverFinder.py:685-753; matching :58-181, cover
 * :561-680), called from DataProcessor.decide_pre_or_post_aggr_v2
 * (super_gnn/data_manager/DataProcessor.py:259-281).  Left = source nodes of the
 * cross edges between one pair of ranks, right = their destination nodes; a source
 * in the cover is shipped raw ("post"), every other edge is summed at the sender.
 *
 *   h_rowptr int64[num_left+1], h_col int32[nnz]: adjacency of the left vertices
 *   (right ids in [0, num_right)); duplicates allowed.
 *   h_cover_left uint8[num_left], h_cover_right uint8[num_right]: 1 = in the cover.
 *   h_matching_size (nullable): size of the maximum matching = size of the cover.
 * ------------------------------------------------------------------------- */
int sgnn_bipartite_min_vertex_cover(int64_t num_left, int64_t num_right, const int64_t *h_rowptr,
                                    const int32_t *h_col, uint8_t *h_cover_left, uint8_t *h_cover_right,
                                    int64_t *h_matching_size);

#ifdef __cplusplus
}
#endif
#endif /* SUPERGNN_B200_H */
