/*
 * exact_b200.h -- C ABI of libexact_b200.so: the activation-compression hot path of EXACT
 * (zirui-ray-liu/Exact) as hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * The reference exposes this path as pybind11 torch-extension functions taking at::Tensor.  Each
 * entry point below names the reference function it stands in for (paths relative to the reference
 * checkout) and takes the same operands as plain device pointers and sizes.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the current CUDA device unless stated otherwise.
 *   - Nothing is allocated or freed here: the caller owns inputs, outputs and scratch.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).  Kernels are only
 *     enqueued; the call does not synchronise.
 *   - Return value 0 = success.  Non-zero: 1 bad argument, 2 CUDA runtime error, 3 unsupported
 *     shape, 4 device-side status.  exact_last_error() gives the message (thread-local).
 *   - Tensors are dense row-major ("contiguous"), as the reference requires
 *     (exact/exact/cpp_extension/ext_common.h:2-32).
 */
#ifndef EXACT_B200_H_
#define EXACT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EXACT_API __attribute__((visibility("default")))
#else
#define EXACT_API
#endif

enum { EXACT_DTYPE_F32 = 0, EXACT_DTYPE_BF16 = 1 };
enum { EXACT_REDUCE_SUM = 0, EXACT_REDUCE_MEAN = 1 };
/* May be OR-ed into `reduce`; accepted and ignored.  (It used to let operands of at most 64 columns take a
 * kernel that interleaved partial sums of a row; that kernel now gives several rows to a warp instead and sums
 * every row up to the long-row threshold in edge order, bit-identical to the reference kernel, flag or not.) */
enum { EXACT_SPMM_REGROUP = 0x100 };

/* Library version (major * 100 + minor) and the last error message of the calling thread. */
EXACT_API int exact_version(void);
EXACT_API const char* exact_last_error(void);

/* Device-side status.  The kernels that wait on on-chip barriers (exact_rp_quantize_pack,
 * exact_unpack_dequant_rp, exact_linear_forward, exact_grad_weight_from_packed) bound every wait; a kernel
 * whose wait runs out abandons its tile, returns, and ORs a bit into one status word per device (1, 2, 4, 8
 * in that order) besides the word in its own workspace.  exact_status copies the word of the current device
 * to *status (it synchronises `stream`); non-zero means some output since the last exact_clear_status is
 * incomplete.  exact_set_status writes the word, so that a host can exercise its error path without making
 * a wait expire.  No counterpart in the reference (its kernels never wait). */
EXACT_API int exact_status(int* status, void* stream);
/* The same copy without the synchronisation: *pinned_host_status (page-locked host memory) is valid once the
 * work enqueued on `stream` so far has completed. */
EXACT_API int exact_status_async(int* pinned_host_status, void* stream);
EXACT_API int exact_clear_status(void* stream);
EXACT_API int exact_set_status(int code, void* stream);

/* Bytes of the packed stream for an [N, D] activation at `bits` per element: ceil(N / (8/bits)) * D.
 * The reference allocates one more byte and never writes it (quantization_cuda_kernel.cu:110-113);
 * callers that mirror its tensor shape allocate exact_packed_bytes() + 1. */
EXACT_API int64_t exact_packed_bytes(int64_t N, int64_t D, int bits);

/* Fused quantize_activation.  Replaces the chain exact/exact/ops.py:69-83 -> ops.py:61-66 (row
 * min/max) -> ops.py:36-40 (scale = reciprocal(max - min) * (2^bits - 1)) ->
 * quantization.pack_single_precision (quantization.cc:37-48, quantization_cuda_kernel.cu:63-155) ->
 * ops.py:80-81 (statistics stored as bf16), in one pass over x.
 *   x          [N, D], fp32 or bf16 (dtype = EXACT_DTYPE_*); bf16 is widened to fp32 first
 *   noise      [N, D] fp32 uniform noise added before rounding, or NULL to draw Philox4x32-10 noise
 *              keyed by (seed, offset, global row, column)
 *   row_offset global index of row 0 (multiple of 8) so that row shards draw the noise of the whole
 *   packed     [exact_packed_bytes(N, D, bits)] out
 *   scale_bf16, min_bf16  [N] bf16 bit patterns out (either may be NULL)
 *   scale_f32, min_f32    [N] the fp32 statistics the codes were computed with (either may be NULL) */
EXACT_API int exact_quantize_pack(const void* x, int dtype, int64_t N, int64_t D, int bits,
                                  const float* noise, uint64_t seed, uint64_t offset,
                                  int64_t row_offset, uint8_t* packed, uint16_t* scale_bf16,
                                  uint16_t* min_bf16, float* scale_f32, float* min_f32, void* stream);

/* quantization.pack_single_precision(data, min, max, scale, bits, stochastic)
 * (quantization.cc:37-48; kernel quantization_cuda_kernel.cu:63-94) with caller-computed fp32 row
 * statistics.  `max` is unused by the reference kernel and is not taken.  Noise as above. */
EXACT_API int exact_pack_single_precision(const void* data, int dtype, const float* min,
                                          const float* scale, int64_t N, int64_t D, int bits,
                                          const float* noise, uint64_t seed, uint64_t offset,
                                          int64_t row_offset, uint8_t* packed, void* stream);

/* quantization.unpack_single_precision(data, bits, scale, min, N, group_size)
 * (quantization.cc:50-62; kernel quantization_cuda_kernel.cu:158-185): out[n, d] = code / scale[n] +
 * min[n].  scale/min are fp32 (the reference signature) or bf16 bit patterns (stats_dtype), which
 * folds the widening of exact/exact/ops.py:94-96 into the kernel.  out is [N, D] fp32. */
EXACT_API int exact_unpack_single_precision(const uint8_t* packed, int bits, const void* scale,
                                            const void* min, int stats_dtype, int64_t N, int64_t D,
                                            float* out, void* stream);

/* fp16 activations: the half instantiations of the reference's pack / unpack kernels
 * (quantization_cuda_kernel.cu:132, 209; AMP runs cast the inputs of the quantised ops to fp16,
 * exact/exact/ops.py:130) and the fp16 row statistics that go with them (ops.py:82-83: the statistics of an
 * fp16 activation stay fp16).  Every Half (op) Half is computed in fp32 and rounded back to half, as c10::Half
 * does: pack  code = rint(max(float(half(half(x - min) * scale)) + noise - 0.5, 0));
 *       unpack out = half(half(float(code) / scale) + min);
 *       statistics min = min_d x, scale = half(float(half(1 / float(half(max - min)))) * (2^bits - 1)).
 * data / x / out [N, D] and min / scale [N] are fp16 bit patterns; packed layout and noise as in the fp32 entry
 * points. */
EXACT_API int exact_quantize_pack_f16(const void* x, int64_t N, int64_t D, int bits, const float* noise, uint64_t seed,
                                      uint64_t offset, int64_t row_offset, uint8_t* packed, uint16_t* scale_f16,
                                      uint16_t* min_f16, void* stream);
EXACT_API int exact_pack_single_precision_f16(const void* data, const void* min, const void* scale, int64_t N, int64_t D,
                                              int bits, const float* noise, uint64_t seed, uint64_t offset,
                                              int64_t row_offset, uint8_t* packed, void* stream);
EXACT_API int exact_unpack_single_precision_f16(const uint8_t* packed, int bits, const void* scale, const void* min,
                                                int64_t N, int64_t D, void* out, void* stream);

/* The 1-bit-mask activations on fp16 tensors (the reference's half instantiations,
 * quantization_cuda_kernel.cu:284, 324, 387, 428, 535, 586): the arithmetic of the fp32 entry points on widened
 * values, rounded to half once on the store (Half (op) float is a float in the reference).  op: EXACT_ACT_*;
 * param: the dropout probability or the negative slope (ignored by ReLU); uniforms / seed / offset / index_offset
 * as in exact_act_quantized_dropout_forward.  The backward of EXACT_ACT_RELU_DROPOUT is that of
 * EXACT_ACT_DROPOUT with the saved mask.  x / out / grad_out / grad_in: n fp16 bit patterns. */
enum { EXACT_ACT_RELU = 0, EXACT_ACT_DROPOUT = 1, EXACT_ACT_RELU_DROPOUT = 2, EXACT_ACT_LEAKY_RELU = 3 };
EXACT_API int exact_act_quantized_forward_f16(int op, const void* x, int64_t n, float param, const float* uniforms,
                                              uint64_t seed, uint64_t offset, int64_t index_offset, void* out,
                                              uint32_t* mask, void* stream);
EXACT_API int exact_act_quantized_backward_f16(int op, const void* grad_out, const uint32_t* mask, int64_t n, float param,
                                               void* grad_in, void* stream);

/* Number of 32-bit mask words the 1-bit-mask activations need for n elements: 8 * ceil(n / 256); the mask must be
 * 16-byte aligned. */
EXACT_API int64_t exact_mask_words(int64_t n);

/* quantization.act_quantized_relu forward / backward (quantization.cc:66-84;
 * quantization_cuda_kernel.cu:237-331): out = x > 0 ? x : 0 and a 1-bit mask; grad_in = bit ?
 * grad_out : 0.  The mask layout is private to this library (the reference's never leaves its
 * extension either). */
EXACT_API int exact_act_quantized_relu_forward(const float* x, int64_t n, float* out, uint32_t* mask,
                                               void* stream);
EXACT_API int exact_act_quantized_relu_backward(const float* grad_out, const uint32_t* mask, int64_t n,
                                                float* grad_in, void* stream);

/* quantization.act_quantized_leaky_relu forward / backward (quantization.cc:87-107;
 * quantization_cuda_kernel.cu:339-435): out = x > 0 ? x : x * slope with the same 1-bit mask;
 * grad_in = bit ? grad_out : grad_out * slope. */
EXACT_API int exact_act_quantized_leaky_relu_forward(const float* x, int64_t n, float slope, float* out,
                                                     uint32_t* mask, void* stream);
EXACT_API int exact_act_quantized_leaky_relu_backward(const float* grad_out, const uint32_t* mask, int64_t n,
                                                      float slope, float* grad_in, void* stream);

/* quantization.act_quantized_dropout forward / backward (quantization.cc:111-134;
 * quantization_cuda_kernel.cu:442-594): keep = u > p, out = (x * keep) * float(1 / (1 - p));
 * grad_in = keep ? grad_out / float(1 - p) : 0.  `uniforms` [n] supplies u, or NULL draws them: one
 * Philox4x32-10 block keyed by (seed, offset, (index_offset + element index) / 8) gives eight 16-bit values h,
 * u = (h + 0.5) / 65536 (the probability is resolved to 2^-16);
 * index_offset (multiple of 8) is the global index of element 0 when rows are sharded. */
EXACT_API int exact_act_quantized_dropout_forward(const float* x, int64_t n, float p,
                                                  const float* uniforms, uint64_t seed, uint64_t offset,
                                                  int64_t index_offset, float* out, uint32_t* mask,
                                                  void* stream);
EXACT_API int exact_act_quantized_dropout_backward(const float* grad_out, const uint32_t* mask,
                                                   int64_t n, float p, float* grad_in, void* stream);

/* ReLU followed by dropout in one pass over the activation (act_quantized_relu then
 * act_quantized_dropout, quantization.cc:66-84 and 111-134, as models apply them back to back):
 * out = dropout(max(x, 0)), bit-identical to the two calls with the same uniforms, and ONE 1-bit mask,
 * set where the ReLU passed and the dropout kept.  Its backward is exact_act_quantized_dropout_backward
 * with that mask (g / (1 - p) where set, else 0), which equals the two separate backward passes. */
EXACT_API int exact_act_quantized_relu_dropout_forward(const float* x, int64_t n, float prob, const float* uniforms,
                                                       uint64_t seed, uint64_t offset, int64_t index_offset,
                                                       float* out, uint32_t* mask, void* stream);

/* spmm.spmm_sum_fw / spmm_mean_fw (spmm.cc:31-55, 84-113 -> spmm_cuda.cu:27-170, reducer.cuh):
 * out[r, :] = reduce_{e in row r} value[e] * mat[col[e], :].  rowptr [M+1] and col [nnz] are int32
 * (idx_bytes = 4) or int64 (8); value [nnz] fp32 or NULL (all ones); mat [*, K]; out [M, K].
 * Mean divides by max(row length, 1).  The gradient with respect to mat (spmm.cc:57-79, 115-139) is
 * this same call on the transposed structure with reduce = sum. */
EXACT_API int exact_spmm(const void* rowptr, const void* col, int idx_bytes, const float* value,
                         const float* mat, int64_t M, int64_t K, int reduce, float* out, void* stream);

/* spmm.spmm_max_fw / spmm_min_fw (spmm.cc:145-157, 195-208 -> spmm_cuda.cu:27-170 with REDUCE = MAX / MIN,
 * reducer.cuh:43-85): out[r, c] = max (min) over the edges e of row r of value[e] * mat[col[e], c], and
 * arg_out[r, c] = the first edge attaining it (same index type as rowptr / col); rows without edges give 0
 * and arg = nnz.  The backward of these reductions (spmm.cc:159-193, 210-241) is index arithmetic on arg_out
 * and stays library ops. */
EXACT_API int exact_spmm_minmax(const void* rowptr, const void* col, int idx_bytes, const float* value,
                                const float* mat, int64_t M, int64_t K, int64_t nnz, int is_max, float* out,
                                void* arg_out, void* stream);

/* Gradient with respect to the edge values, spmm_value_bw of spmm.cc:66-68, 125-126 (kernel
 * spmm_cuda.cu:172-209): out[e] = dot(mat[col[e], :], grad[row[e], :]), divided by max(length of row[e], 1)
 * for mean.  row [E] is the COO row of every edge, rowptr [M+1] is read for mean only.  Same lane-strided
 * FMAs and the same shuffle tree as the reference kernel: bit-identical. */
EXACT_API int exact_spmm_value_bw(const void* row, const void* rowptr, const void* col, int idx_bytes,
                                  const float* mat, const float* grad, int64_t E, int64_t K, int reduce,
                                  float* out, void* stream);

/* exact_spmm with long rows cut into pieces (no counterpart in the reference, whose kernel gives
 * every row to one warp: spmm_cuda.cu:35-57).  Rows with more than long_threshold edges are left out
 * of the row kernel; the caller lists them and their pieces:
 *   long_row      [n_long]      int32  indices of the long rows, ascending
 *   long_item_ptr [n_long + 1]  int32  pieces of long row i are items long_item_ptr[i] .. [i+1]
 *   item_row      [n_items]     int32  row of each piece
 *   item_begin / item_end [n_items] int64  edge range of each piece (at most long_threshold edges; the
 *                                      pieces of a row tile its edge range)
 *   item_slot     [n_items]     int32  or NULL: the slot of scratch each listed piece writes.  Slots
 *                                      long_item_ptr[i] .. [i+1] hold the pieces of long row i in edge
 *                                      order; the pieces themselves may be listed (= processed) in any
 *                                      order.  Listing them by the column of their first edge lets pieces
 *                                      of different hub rows that gather the same source rows run
 *                                      together, so those rows are read from HBM once (10.1 -> 8.7 ms at
 *                                      125.8 M edges x 256 columns).  NULL: piece j writes slot j.
 *   scratch       [n_items, K]  fp32   caller-owned; holds the partial sums of the pieces
 * Rows up to the threshold are summed exactly as exact_spmm sums them; a long row is the in-order sum
 * of its pieces' sums.  Every row longer than long_threshold must be listed: with n_items = 0 such rows
 * are left unwritten.  Column indices are staged as 32-bit values, so M (and the operand) stay below 2^32
 * rows (refused otherwise). */
EXACT_API int exact_spmm_split(const void* rowptr, const void* col, int idx_bytes, const float* value,
                               const float* mat, int64_t M, int64_t K, int reduce, int64_t long_threshold,
                               const int32_t* item_row, const int64_t* item_begin, const int64_t* item_end,
                               const int32_t* item_slot, int64_t n_items, const int32_t* long_row,
                               const int32_t* long_item_ptr, int64_t n_long, float* scratch, float* out,
                               void* stream);

/* Compact rows: a dense operand whose entries are mostly exact zeros, in the form row shards write it into
 * each other's memory before an aggregation.  No counterpart in the reference (it is single-GPU and gathers dense
 * rows, spmm_cuda.cu:86-93).  Row r of x [n, K] fp32 (0 < K <= 256, row pitch ldx) goes to a slot of
 * exact_crows_slot_bytes(K) = 16 + pad16(K) + 4 K bytes at slot index row0 + r of each destination buffer:
 *   +0  uint32 cnt;   +16  uint8 col[cnt] (ascending);   +16 + pad16(K)  fp32 val[cnt].
 * An entry is kept when any of its 32 bits is set: only +0.0 is dropped, so unpack(pack(x)) == x bit for bit
 * (-0.0, NaN, inf and denormals included).
 *   rowscale   [n] fp32 or NULL: row r is multiplied by rowscale[r] first (the 1/deg scaling of the
 *              transposed mean, spmm.cc:128-133, folded into this pass)
 *   dst        host array of n_dst (1..8) device pointers, 16-byte aligned, each with room for every slot
 *              written.  A pointer may be a peer GPU's buffer (mapped into this process): the rows are then
 *              written there with plain stores over NVLink; the caller orders those writes before the
 *              peer's reads (stream order on this GPU, then a collective or event both sides wait on).
 *   kept_total device uint64 or NULL: the number of kept entries is added to it (one atomic per CTA).
 * exact_crows_unpack writes dense rows out [n, K] (row pitch ldo) from slots row0 .. row0 + n - 1. */
EXACT_API int64_t exact_crows_slot_bytes(int64_t K);
EXACT_API int exact_crows_pack(const float* x, int64_t n, int64_t K, int64_t ldx, const float* rowscale, int64_t row0,
                               void* const* dst, int n_dst, uint64_t* kept_total, void* stream);
EXACT_API int exact_crows_unpack(const void* buf, int64_t n, int64_t K, int64_t row0, float* out, int64_t ldo,
                                 void* stream);

/* The two exchanges of the feature-parallel aggregation of a row-sharded run (no counterpart in the reference).
 * Between aggregations rank p holds rows [p * shard, (p + 1) * shard) with all K columns.  For out = A x the
 * ranks switch to a column split and back:
 *   exact_cols_scatter  x [n, K] fp32 (pitch ldx; K, ldx multiples of 4; 16-byte aligned), optionally times
 *       rowscale[r]: dst[q][(row0 + r) * Kp + c] = x[r, q * Kp + c] for every rank q (columns past K: zero).
 *       Rank q then owns columns [q Kp, (q + 1) Kp) of all rows and multiplies the whole adjacency with them.
 *   exact_rows_scatter  y [n_total, Kp], this rank's column slice of the result:
 *       dst[p][(row - p * shard) * ldd + col0 + c] = y[row, c] for the rows of block p (col0 = rank * Kp).
 * dst: host array of n_dst (1..8) device pointers, one per rank, which may be peers' buffers (exact_peer_import):
 * plain 16-byte stores over NVLink; the caller orders them before the readers (stream order, then a collective).
 * Two all-to-all exchanges of N K / P elements per rank replace the all-gather of N K (P - 1) / P. */
EXACT_API int exact_cols_scatter(const float* x, int64_t n, int64_t K, int64_t ldx, const float* rowscale, int64_t row0,
                                 int64_t Kp, void* const* dst, int n_dst, void* stream);
EXACT_API int exact_rows_scatter(const float* y, int64_t n_total, int64_t Kp, int64_t shard, int64_t col0, int64_t ldd,
                                 void* const* dst, int n_dst, void* stream);

/* One pass over the gradient g [n, K] (pitch ldg) of a layer's output for the two things its backward needs besides the
 * GEMMs (no single counterpart in the reference, which leaves both to the framework):
 *   colsum[c] = sum_r g[r, c]          the bias gradient, grad_output.sum(0) of backward_func.cc:88-90 (or NULL);
 *   out[r, c] = g[r, c] * rowscale[r]  for c < K, zero for K <= c < Kout (pitch ldo): the operand D^-1 g of the
 *                                      transposed mean aggregation (spmm.cc:128-137), or NULL.  rowscale NULL: ones.
 * Column sums are added in a fixed order (run-to-run identical).  16-byte accesses when K, Kout and the pitches are
 * multiples of 4 and the pointers 16-byte aligned, scalar ones otherwise.  workspace (needed for colsum):
 * exact_rows_scale_colsum_workspace_bytes(Kout), 256-byte aligned. */
EXACT_API int64_t exact_rows_scale_colsum_workspace_bytes(int64_t Kout);
EXACT_API int exact_rows_scale_colsum(const float* g, int64_t n, int64_t K, int64_t ldg, const float* rowscale, float* out,
                                      int64_t Kout, int64_t ldo, float* colsum, void* workspace,
                                      int64_t workspace_bytes, void* stream);

/* Batch-norm backward straight from the packed input: native_batch_norm_backward as called by the reference's
 * qbatch_norm.backward (exact/exact/ops.py:248-251) with the dequantize_activation of ops.py:238 folded into
 * both of its passes, so the [N, D] reconstruction is never written.
 *   grad_out [N, D] fp32 (16-byte aligned, D % 4 == 0, else code 3); packed / scale_bf16 / min_bf16: the saved
 *   input as exact_quantize_pack wrote it; weight [D] or NULL (ones);
 *   training != 0: mean = save_mean, invstd = save_invstd of the forward;
 *       grad_input = (g - sum(g)/N - (x - mean) * invstd^2 * sum(g (x - mean))/N) * invstd * weight
 *   training == 0: mean = running_mean, invstd = 1/sqrt(running_var + eps); grad_input = g * invstd * weight
 *   grad_weight = invstd * sum_n g (x - mean), grad_bias = sum_n g; any of the three outputs may be NULL.
 * Column sums are added in a fixed order (per-CTA partial rows, then CTA order): results are run-to-run
 * identical and differ from ATen's by fp32 reassociation.  workspace: exact_bn_backward_workspace_bytes(D),
 * 256-byte aligned. */
EXACT_API int64_t exact_bn_backward_workspace_bytes(int64_t D);
EXACT_API int exact_bn_backward_from_packed(const float* grad_out, int64_t N, int64_t D, const uint8_t* packed, int bits,
                                            const uint16_t* scale_bf16, const uint16_t* min_bf16, const float* weight,
                                            const float* mean, const float* invstd, int training, void* workspace,
                                            int64_t workspace_bytes, float* grad_input, float* grad_weight,
                                            float* grad_bias, void* stream);

/* CSR SpMM on fp16 operands with the arithmetic of the reference's half instantiation (spmm_cuda.cu:142; AMP runs
 * cast the operands to fp16, exact/exact/ops.py:260, 313): term = half(value[e] * mat[col[e], c]) (the bare operand
 * without values), result = half(result + term) in CSR order, mean = half(result / half(max(count, 1))); every
 * Half (op) Half an fp32 operation on the widened values.  value (or NULL), mat [N, K], out [M, K]: fp16 bit
 * patterns.  Rounding after every edge makes the order part of the result: one warp sums a row in CSR order
 * whatever its length. */
EXACT_API int exact_spmm_f16(const void* rowptr, const void* col, int idx_bytes, const void* value, const void* mat,
                             int64_t M, int64_t K, int reduce, void* out, void* stream);

/* exact_spmm_split with the second exchange folded into it (no counterpart in the reference): instead of a local
 * [M, K] result followed by exact_rows_scatter, every output row r is stored, by the warp that summed it,
 * straight into its owner's buffer, dst[r / shard][(r % shard) * ldd + col0 + c], c < K (plain stores, peers'
 * memory included), so the result slice is neither written to nor read back from local memory and the
 * transfer overlaps the gathers.  n_dst * shard >= M; ldd >= col0 + K; for 16-byte stores dst, ldd and col0
 * are 16-byte / 4-element aligned (else narrower stores).  A plan is optional (n_items = 0: every row is
 * summed by one warp).  row_order (optional, [M] int32, a permutation of the rows): the order in which a narrow
 * operand (EXACT_SPMM_REGROUP, K <= 64) takes the rows, several rows per warp; sorted by row length it gives
 * every warp rows of equal length.  With n_dst = 1, shard = M, col0 = 0 and ldd = K this is exact_spmm_split
 * with a row order.  Ordering against the readers is the caller's, as for exact_rows_scatter. */
EXACT_API int exact_spmm_split_routed(const void* rowptr, const void* col, int idx_bytes, const float* value,
                                      const float* mat, int64_t M, int64_t K, int reduce, int64_t long_threshold,
                                      const int32_t* item_row, const int64_t* item_begin, const int64_t* item_end,
                                      const int32_t* item_slot, int64_t n_items, const int32_t* long_row,
                                      const int32_t* long_item_ptr, int64_t n_long, float* scratch,
                                      const int32_t* row_order, int64_t shard, int64_t col0, int64_t ldd,
                                      void* const* dst, int n_dst, void* stream);

/* Buffers that the ranks of a row-sharded run write into each other (one process per GPU, one node).  No
 * counterpart in the reference.  These are the only entry points that allocate or free device memory:
 *   exact_peer_alloc   cudaMalloc of `bytes` on the current device;
 *   exact_peer_export  the buffer's CUDA IPC handle (EXACT_PEER_HANDLE_BYTES bytes, host memory) for the other
 *                      processes of the node;
 *   exact_peer_import  in another process: opens a handle and returns a device pointer to the owner's buffer,
 *                      valid on the current device (peer access is enabled);  exact_peer_close  unmaps it;
 *   exact_peer_free    in the owner, after the peers have closed their mappings. */
#define EXACT_PEER_HANDLE_BYTES 64
EXACT_API int exact_peer_alloc(int64_t bytes, void** ptr);
EXACT_API int exact_peer_free(void* ptr);
EXACT_API int exact_peer_export(const void* ptr, void* handle64);
EXACT_API int exact_peer_import(const void* handle64, void** ptr);
EXACT_API int exact_peer_close(void* ptr);

/* exact_spmm_split without the scratch argument (no counterpart in the reference).  Meant for hosts
 * that must not allocate device memory around the call -- a serving loop with a frozen memory plan, a
 * plugin running inside another framework's allocator, a region being recorded for replay.  The
 * partial sums go to an array of EXACT_SPMM_STATIC_SCRATCH_FLOATS floats (16 MiB) that is part of the
 * library image: every GPU that loads the library holds it until the process exits.
 *   - n_items * K must not exceed EXACT_SPMM_STATIC_SCRATCH_FLOATS; larger plans are refused (code 1).
 *   - The plan arrays live on the device and are trusted: item_slot must be a permutation of
 *     [0, n_items) and long_item_ptr[n_long] == n_items, or a piece writes outside the array.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress with
 *     that device current) and keeps it; make that first call before recording or capturing anything.
 *   - All calls on a device share the array: calls that may overlap on the GPU (different streams) race.
 *     Nothing in it needs clearing -- every piece overwrites its own slice before it is read.
 *   - No cudaMalloc / cudaFree or other allocating call is made. */
#define EXACT_SPMM_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
EXACT_API int exact_spmm_split_static(const void* rowptr, const void* col, int idx_bytes, const float* value,
                                      const float* mat, int64_t M, int64_t K, int reduce,
                                      int64_t long_threshold, const int32_t* item_row,
                                      const int64_t* item_begin, const int64_t* item_end,
                                      const int32_t* item_slot, int64_t n_items, const int32_t* long_row,
                                      const int32_t* long_item_ptr, int64_t n_long, float* out, void* stream);

/* Fused random projection + quantise + pack: the chain input2rp -> quantize_activation of
 * exact/exact/ops.py:142-149 (torch.matmul(input, rand_matrix), ops.py:117, then ops.py:61-83) as one
 * TMA-fed tcgen05 (tf32) GEMM whose epilogue computes the row statistics and packs, so the [N, k]
 * product never reaches HBM.
 *   x [N, D] fp32, rows of any length (rows a tensor map cannot describe, D % 4 != 0 or a base that is not
 *   16-byte aligned, are brought in by cp.async instead of TMA); packed 4-byte aligned when k % 4 == 0;  R [D, k]
 *   fp32 with entries +-1/sqrt(k) (only the signs are read; 1/sqrt(k) is applied in fp32);  k up to 512 after
 *   padding to 16.  Other shapes return code 3 and the caller uses the unfused chain.
 *   workspace: exact_rp_workspace_bytes(D, k) bytes, 256-byte aligned, caller-owned.  Its first int32
 *   is a status word the kernels clear and set non-zero only if a bounded on-chip wait expired.
 *   Noise: Philox4x32-10 keyed by (seed, offset); one call per (global row, block of 8 columns).
 *   y_out (optional, [N, k] fp32): the projection as the epilogue saw it (1/sqrt(k) applied).
 * packed / scale_bf16 / min_bf16 as in exact_quantize_pack with D := k. */
EXACT_API int64_t exact_rp_workspace_bytes(int64_t D, int64_t k);
EXACT_API int exact_rp_quantize_pack(const float* x, int64_t N, int64_t D, const float* R, int64_t k, int bits,
                                     uint64_t seed, uint64_t offset, int64_t row_offset, void* workspace,
                                     uint8_t* packed, uint16_t* scale_bf16, uint16_t* min_bf16, float* y_out,
                                     void* stream);

/* Fused unpack + dequantise + transpose projection: the backward chain dequantize_activation ->
 * rp2input of exact/exact/ops.py:164-166 (unpack_single_precision, quantization.cc:50-62, then
 * torch.matmul(., rand_matrix.t()), ops.py:124) as one tcgen05 (tf32) GEMM whose A operand is
 * dequantised straight into shared memory, so the [N, k] dequantised projection never reaches HBM.
 *   packed / scale_bf16 / min_bf16: a packed [N, k] activation as exact_quantize_pack or
 *   exact_rp_quantize_pack produce it;  R [D, k] fp32 (+-1/sqrt(k));  out [N, D] fp32.
 *   sign(R) stays resident in shared memory when it fits beside the A tiles (D <= 256, small k); otherwise it is
 *   streamed in panels and the output is produced in blocks of up to 256 columns.  workspace: exact_unpack_rp_workspace_bytes(D, k)
 *   bytes, 256-byte aligned; its first int32 is the status word (see exact_rp_quantize_pack). */
EXACT_API int64_t exact_unpack_rp_workspace_bytes(int64_t D, int64_t k);
EXACT_API int exact_unpack_dequant_rp(const uint8_t* packed, int bits, const uint16_t* scale_bf16,
                                      const uint16_t* min_bf16, int64_t N, int64_t k, const float* R, int64_t D,
                                      void* workspace, float* out, void* stream);

/* Dense layer GEMM with fp32-equivalent accuracy on the tensor cores (each operand split into a tf32
 * head and tail, three tcgen05 MMAs per tile, fp32 accumulation):
 *     C[M, N] (+)= A[M, K] B[N, K]^T  (+ A2[M, K2] B2[N, K2]^T)  (+ bias[N])
 * Replaces the fp32 cuBLAS GEMMs of the quantised linear layer: F.linear(input, weight, bias) in
 * qlinear.forward (exact/exact/ops.py:150) with A = input, B = weight [out, in]; and
 * grad_input = grad_output.mm(weight) of linear_backward (exact/exact/cpp_extension/backward_func.cc:86)
 * with A = grad_output, B = weight^T.  The optional second pair sums two layers that share their output,
 * W_l mean_j(x_j) + W_r x of the GraphSAGE layer (exact/exact/layers.py:163-170), in one pass.
 *   lda / ldb / lda2 / ldb2 / ldc: row pitches in elements.  A (and A2) must be 16-byte aligned with
 *   lda % 4 == 0; N <= 256 per call (wider outputs: one call per 256-column block of B / C); other
 *   shapes return code 3 and the caller uses a library GEMM.  accumulate != 0 adds to C.
 *   workspace: exact_linear_workspace_bytes(N, K, K2) bytes, 256-byte aligned; its first int32 is the
 *   status word (see exact_rp_quantize_pack). */
EXACT_API int64_t exact_linear_workspace_bytes(int64_t N, int64_t K, int64_t K2);
EXACT_API int exact_linear_forward(const float* A, int64_t M, int64_t K, int64_t lda, const float* B, int64_t ldb,
                                   const float* A2, int64_t K2, int64_t lda2, const float* B2, int64_t ldb2,
                                   int64_t N, const float* bias, int accumulate, void* workspace, float* C,
                                   int64_t ldc, void* stream);

/* Weight gradient of a quantised linear layer from the packed activation(s), on the tensor cores:
 *     out[O, kpad] = g^T [O x N] . dequantise(packed) [N x k]
 * grad_weight = grad_output.t().mm(input) of linear_backward (exact/exact/cpp_extension/backward_func.cc:87) with
 * `input` as qlinear.forward saved it (exact/exact/ops.py:149-154: packed codes + bf16 row statistics), fusing
 * dequantize_activation (ops.py:164) into the product.  With a random projection the caller multiplies the
 * result by R^T ((g^T Xq) R^T = g^T (Xq R^T), ops.py:165-169).  Two packed activations that share g (the two
 * inputs of a GraphSAGE layer, layers.py:163-170) go in one pass: columns [0, k0) of `out` belong to the first,
 * columns [pad16(k0), pad16(k0) + k1) to the second (k1 = 0: one activation); ldo >= pad16(k0) + pad16(k1).
 *   g [N, O] fp32, 16-byte aligned, O % 4 == 0, O <= 256; other shapes return code 3 (the caller unpacks and
 *   uses a library GEMM).  tf32 inputs, fp32 accumulation: about 5e-4 relative.
 *   workspace: exact_grad_weight_workspace_bytes(O, pad16(k0) + pad16(k1), SM count) bytes, 256-byte aligned:
 *   its first int32 is the status word (see exact_rp_quantize_pack), the rest holds one partial result per CTA,
 *   added in CTA order by a second kernel (the result does not depend on timing). */
EXACT_API int64_t exact_grad_weight_workspace_bytes(int64_t O, int64_t k_total_padded, int max_ctas);
EXACT_API int exact_grad_weight_from_packed(const float* g, int64_t N, int64_t O, const uint8_t* packed0,
                                            const uint16_t* scale0, const uint16_t* min0, int64_t k0,
                                            const uint8_t* packed1, const uint16_t* scale1, const uint16_t* min1,
                                            int64_t k1, int bits, void* workspace, int64_t workspace_bytes,
                                            float* out, int64_t ldo, void* stream);

/* Zero-compacted rows, the exchange format of the row-sharded aggregation.  No counterpart in the
 * reference (it is single-GPU).  A shard x [n, K] fp32 (row pitch ldx, K % 32 == 0) whose entries are
 * mostly exact zeros (outputs of ReLU + dropout, gradients that passed their masks) is sent as
 *   mask   uint32 [n, K/32]  bit c % 32 of word c / 32: element (row, c) is kept (any of its 32 bits set,
 *                            so only +0.0 is dropped and the round trip is bit-exact);
 *   rowoff int64  [n + 1]    exclusive prefix sum of the rows' kept counts (the caller scans rowcnt);
 *   vals   fp32   [rowoff[n]] the kept elements, row-major.
 * exact_rows_mask_count writes mask and rowcnt [n]; exact_rows_compact_write writes vals;
 * exact_rows_expand writes dense rows out [n, K] (row pitch ldo) from the concatenation of several shards:
 * rows [b * block_rows, (b + 1) * block_rows) use rowoff + b * rowoff_stride and vals + b * vals_stride. */
EXACT_API int exact_rows_mask_count(const float* x, int64_t n, int64_t K, int64_t ldx, uint32_t* mask,
                                    int32_t* rowcnt, void* stream);
EXACT_API int exact_rows_compact_write(const float* x, int64_t n, int64_t K, int64_t ldx, const int64_t* rowoff,
                                       float* vals, void* stream);
EXACT_API int exact_rows_expand(const uint32_t* mask, const int64_t* rowoff, const float* vals, int64_t n, int64_t K,
                                int64_t block_rows, int64_t rowoff_stride, int64_t vals_stride, float* out,
                                int64_t ldo, void* stream);

/* The random matrix of input2rp (exact/exact/ops.py:107-118, gen_rad_mat at ops.py:112-114):
 * out [D, k] row-major fp32, entries +-1/sqrt(k).  Sign i (row-major index) is bit i % 128 of the
 * Philox4x32-10 block with counter (i / 128, offset) and key `seed`, instead of a draw from torch's
 * global generator, so that every rank and the CPU oracle regenerate the same matrix. */
EXACT_API int exact_rademacher(uint64_t seed, uint64_t offset, int64_t D, int64_t k, float* out,
                               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EXACT_B200_H_ */
