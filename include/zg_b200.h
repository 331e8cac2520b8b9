/* Entry points that the reference's CUDA library does not have.
 *
 * The reference host backend implements these ops (or, for the loss and the
 * Adam update, runs them as raw loops over host memory); its CUDA backend
 * has no counterpart, so the Zig CudaDevice cannot run a training step on the
 * device today.  Each declaration cites the HOST code whose semantics it
 * follows.
 *
 * All calls are asynchronous on the given stream and never exit the
 * process: errors are recorded in a sticky per-process status.
 */
#ifndef ZG_B200_EXT_H
#define ZG_B200_EXT_H

#include "decls.h"

/* ------------------------------------------------------------------ status
 * Replaces the reference's print-and-exit error macros
 * (src/cuda/cuda_helpers.cu:21-91). 0 = no error since the last clear. */
EXTERN_C int zg_last_error(void);
EXTERN_C const char* zg_last_error_message(void);
EXTERN_C void zg_clear_error(void);
/* 1 if a CUDA device is usable by this process, else 0 (never errors). */
EXTERN_C int zg_device_available(void);
/* Binds the calling thread to a device ordinal (multi-device processes). */
EXTERN_C void zg_set_device(unsigned device_number);

/* Orders `waiter` after everything enqueued on `signaller` so far (an event
 * recorded on one stream and waited on by the other).  Lets independent
 * kernels of one step run side by side -- the weight-gradient GEMMs next to the
 * dX chain -- and, while `signaller` is being captured, pulls `waiter` into the
 * same capture so that the branch becomes a parallel branch of the graph (join
 * it back with the arguments swapped before the capture is saved).  No
 * counterpart in the reference, whose device owns a single stream
 * (src/device/cuda_device.zig:24-33). */
EXTERN_C void zg_stream_wait(StreamWrapper waiter, StreamWrapper signaller);

/* Events for ordering that outlives the call: zg_event_record marks the work
 * enqueued on `stream` so far, zg_stream_wait_event makes everything enqueued
 * on `stream` afterwards wait for that mark (a never-recorded event does not
 * block).  The input pipeline keeps one "copied" and one "consumed" event per
 * staging slot, so a step waits for ITS batch only and a copy for the step that
 * last read ITS slot.  No counterpart in the reference (one stream, synchronous
 * copies: src/device/cuda_device.zig:24-33, 520-531). */
EXTERN_C void* zg_event_create(void);
EXTERN_C void zg_event_destroy(void* event);
EXTERN_C void zg_event_record(void* event, StreamWrapper stream);
EXTERN_C void zg_stream_wait_event(StreamWrapper stream, void* event);

/* Page-locked host memory for the input pipeline: host-to-device copies from
 * it run asynchronously on a copy stream while the previous batch trains (the
 * reference's loader copies pageable memory synchronously, tensor by tensor:
 * examples/mnist/src/dataset.zig:11-67).  NULL on failure. */
EXTERN_C void* zg_host_alloc_pinned(len_t nbytes);
EXTERN_C void zg_host_free_pinned(void* hptr);

/* Number of kernel nodes in a saved capture (cuda_utils.h: open_capture /
 * save_capture): what one run_capture launches. */
EXTERN_C len_t zg_capture_kernel_count(GraphWrapper graph);

/* --------------------------------------------------------------- math mode
 * How SINGLE-precision GEMMs use the tensor cores:
 *   ZG_MATH_FP32X3  three TF32 passes on an error-compensated hi/lo split
 *                   (fp32-level accuracy; default)
 *   ZG_MATH_TF32    one TF32 pass (10-bit mantissa products)
 *   ZG_MATH_FFMA    CUDA-core FFMA kernel, no tensor cores */
enum { ZG_MATH_FP32X3 = 0, ZG_MATH_TF32 = 1, ZG_MATH_FFMA = 2 };
EXTERN_C void zg_set_math_mode(int mode);
EXTERN_C int zg_get_math_mode(void);

/* -------------------------------------------------------------------- GEMM
 * opspec.bmm_acc (src/device/opspec.zig:144-162) as HostDevice.bmm_acc runs
 * it (src/device/host_device.zig:277-313): for b in [0,nC):
 *   C[b] = epilogue(alpha * op(A[b % nA]) * op(B[b % nB]) + beta * C[b])
 * A[.] is m x k (k x m when trans_a), B[.] is k x n (n x k when trans_b),
 * row-major with leading dimensions lda/ldb/ldc; batches are contiguous
 * (rows*ld elements apart).  id selects the A/B element type (SINGLE, DOUBLE
 * or BF16); c_id the C element type (SINGLE/DOUBLE, or BF16 with BF16 inputs).
 *
 * Fused epilogues (the reference issues these as separate device calls):
 *   ZG_EPI_NONE
 *   ZG_EPI_BIAS       + bias[j]               (bias.add_(y), examples/mnist/src/model.zig:108)
 *   ZG_EPI_BIAS_RELU  max(0, . + bias[j])     (+ nn.relu_, src/nn/nn.zig:39-62)
 *   ZG_EPI_RELU_MASK  0 where mask_src[i,j] <= 0 (relu_inplace_bwd on the result,
 *                     src/device/host_device.zig:543-547); mask_src has C's shape and ld
 * bias is fp32 [n]; mask_src has C's element type.
 * colsum (optional, fp32 [n]): the column sums of the values stored to C are
 * ADDED to it with fp32 atomics (order not fixed) -- the bias gradient that
 * InplaceAddBwd's unbroadcast (src/ndtensor.zig:783-788) would compute from C
 * in a separate pass.  Not available together with split-K (plain epilogue,
 * deep k, few tiles). */
enum { ZG_EPI_NONE = 0, ZG_EPI_BIAS = 1, ZG_EPI_BIAS_RELU = 2, ZG_EPI_RELU_MASK = 3 };
/* SM budget for the NEXT zg_bmm call of the calling thread (consumed by it; 0 = all SMs).
 * GEMMs issued on parallel streams (the weight gradients of different layers) each take a
 * share: the split-K grid is then sized for that many SMs, so that the concurrent launches
 * fit in one wave together instead of pushing one another's CTAs into a second wave. */
EXTERN_C void zg_bmm_sm_budget(int sms);
EXTERN_C int zg_sm_count(void);
EXTERN_C void zg_bmm(dtype id, dtype c_id, StreamWrapper stream,
                     const void* A, const void* B, void* C,
                     len_t nA, len_t nB, len_t nC, len_t m, len_t n, len_t k,
                     bool trans_a, bool trans_b, len_t lda, len_t ldb, len_t ldc,
                     double alpha, double beta,
                     int epilogue, const void* bias, const void* mask_src, void* colsum);

/* ------------------------------------------------------------- elementwise */
/* opspec.relu_inplace_bwd (host_device.zig:543-547): if (x <= 0) x_g = 0 */
EXTERN_C void zg_relu_inplace_bwd(dtype id, StreamWrapper stream, const void* x, void* x_g, len_t n);
/* opspec.clamp_bwd (host_device.zig:594-598): if (lo < x && x < hi) x_g += y_g */
EXTERN_C void zg_clamp_bwd(dtype id, StreamWrapper stream, const void* x, const void* y_g, void* x_g,
                           len_t n, double lo, double hi);
/* Unary maps y = f(x) (host_device.zig:383-387 sqrt, :480-482 rsqrt with
 * p = eps, :497-510 exp, :549-551 tanh, :561-563 sigmoid) */
/* ZG_UN_POW: y = x^p (host_device.zig:353-361, pow_fwd / pow_fwd_).  x == y is
 * allowed for every op: the in-place forms pow_fwd_ and sqrt_fwd_
 * (host_device.zig:358-361, 390-392) are the same call with one pointer. */
enum { ZG_UN_EXP = 0, ZG_UN_SQRT = 1, ZG_UN_RSQRT = 2, ZG_UN_TANH = 3, ZG_UN_SIGM = 4, ZG_UN_POW = 5 };
EXTERN_C void zg_unary_fwd(dtype id, StreamWrapper stream, int op, const void* x, void* y, len_t n, double p);
/* Their accumulating backward passes: x_g += f'(.) * y_g.  `v` is y for
 * exp/tanh/sigm (host_device.zig:512-515,553-555,565-567) and x for
 * sqrt/rsqrt, where entries with x < p (eps) receive no gradient
 * (host_device.zig:396-408, 485-503). */
EXTERN_C void zg_unary_bwd(dtype id, StreamWrapper stream, int op, const void* v, const void* y_g, void* x_g,
                           len_t n, double p);
/* opspec.pow_bwd (host_device.zig:365-379): x_g += exponent * x^(exponent-1) * y_g,
 * entries with x < eps receive no gradient (eps is an f32 in the op struct). */
EXTERN_C void zg_pow_bwd(dtype id, StreamWrapper stream, const void* x, const void* y_g, void* x_g, len_t n,
                         double exponent, double eps);
/* opspec.tanh_inplace_bwd / sigm_inplace_bwd (host_device.zig:557-559, 569-571):
 * x holds the activation's OUTPUT; x_g *= (1 - x*x) for ZG_UN_TANH,
 * x_g *= x*(1 - x) for ZG_UN_SIGM.  Other ops are refused. */
EXTERN_C void zg_unary_inplace_bwd(dtype id, StreamWrapper stream, int op, const void* x, void* x_g, len_t n);
/* Byte-mask activations (host_device.zig:600-701): one bit per element, bit
 * (i % 8) of mask[i / 8]; mask holds ceil(n/8) bytes (mem_alloc_byte_mask,
 * device_reference.zig:41-43).
 *   relu_mask_fwd   x <= 0: x = 0 and the bit is set        (in place)
 *   relu_mask_bwd   bit set: x_g = 0
 *   clamp_mask_fwd  y = x UNCHANGED (what the reference stores, :611) and the
 *                   bit is set where min(hi, max(lo, x)) != x
 *   clamp_mask_bwd  bit set: x_g += y_g                     (:636-640)
 * The reference's code for the last n % 8 elements of the two clamp forms names
 * fields its op structs do not have (p.x_g in :621, p.x in :633), so it cannot
 * be instantiated; here the tail follows the same per-element rule as the full
 * bytes. */
EXTERN_C void zg_relu_mask_fwd(dtype id, StreamWrapper stream, void* x, unsigned char* mask, len_t n);
EXTERN_C void zg_relu_mask_bwd(dtype id, StreamWrapper stream, void* x_g, const unsigned char* mask, len_t n);
EXTERN_C void zg_clamp_mask_fwd(dtype id, StreamWrapper stream, const void* x, void* y, unsigned char* mask, len_t n,
                                double lo, double hi);
EXTERN_C void zg_clamp_mask_bwd(dtype id, StreamWrapper stream, void* x_g, const void* y_g, const unsigned char* mask, len_t n);
/* opspec.transpose (host_device.zig:261-267): B[j,i] = A[i,j] + alpha*B[j,i] */
EXTERN_C void zg_transpose(dtype id, StreamWrapper stream, const void* A, void* B, len_t m, len_t n, double alpha);

/* -------------------------------------------------------------- reductions
 * reduce.zig:49-164 and host_device.zig:709-874.  y = alpha*reduce + beta*y. */
EXTERN_C void zg_fold_rows(dtype id, StreamWrapper stream, const void* x, void* y, len_t row, len_t col,
                           double alpha, double beta);               /* [row,col] -> [col] */
/* Same result as zg_fold_rows for callers that cannot allocate device memory.
 * (No counterpart in the reference: its reductions go through cuTENSOR with a
 * caller-supplied workspace.)  Who needs it: code that runs while a stream is
 * being captured into a CUDA graph, latency-critical loops such as an agent
 * acting inside a simulator tick, and hosts whose device-memory budget is
 * fixed and audited up front.  zg_fold_rows keeps its cross-CTA partial sums
 * in a library workspace that grows with cudaMalloc on first use; this entry
 * point keeps them in a fixed ~256 KiB array that is part of the library
 * image (resident on every GPU that loads the library until the process
 * exits) and calls no cudaMalloc, cudaFree or any other allocating routine.
 * Limit: the fixed array holds 65536 fp32 (32768 fp64) partial sums, so
 * col must be <= 65536 (fp32; rounded up to a multiple of 128, or of 32 when
 * x is not 16-byte aligned or col is not a multiple of 4) -- wider inputs are
 * rejected with a kBadArgument status and a message that names the limit.
 * The FIRST call on each device resolves the array's device address
 * (cudaGetSymbolAddress); make that call before starting any stream capture.
 * Every call shares the one array per device and leaves its partial sums
 * there, so calls that overlap on the GPU (other streams) race; issue them on
 * one stream or order them with events.  The resolved address is cached per
 * device for the life of the process: after a cudaDeviceReset of that device it
 * is stale, so do not reset a device between calls. */
EXTERN_C void zg_fold_rows_noalloc(dtype id, StreamWrapper stream, const void* x, void* y, len_t row, len_t col,
                                   double alpha, double beta);
EXTERN_C void zg_fold_cols(dtype id, StreamWrapper stream, const void* x, void* y, len_t row, len_t col,
                           double alpha, double beta);               /* [row,col] -> [row] */
EXTERN_C void zg_sum_along(dtype id, StreamWrapper stream, const void* x, const len_t* x_shape, len_t ndim,
                           len_t dim, void* y, double alpha, double beta);
/* max_along ignores alpha/beta, as the host does (host_device.zig:853-874) */
EXTERN_C void zg_max_along(dtype id, StreamWrapper stream, const void* x, const len_t* x_shape, len_t ndim,
                           len_t dim, void* y);
/* opspec.unbroadcast (host_device.zig:709-780).  `scratch` is accepted for
 * signature compatibility with the op struct and may be NULL: intermediates of
 * multi-stage reductions are kept in the library's own workspace, because the
 * size NDArray.unbroadcast_ computes (src/ndarray.zig:697-715) does not cover
 * a leading fold followed by an interior reduction. */
EXTERN_C void zg_unbroadcast(dtype id, StreamWrapper stream, const void* x, const len_t* x_shape, len_t x_ndim,
                             void* y, const len_t* y_shape, len_t y_ndim, void* scratch,
                             double alpha, double beta);
/* opspec.broadcast (host_device.zig:782-795): y[i] = alpha*x[i % |x|] + beta*y[i] */
EXTERN_C void zg_broadcast(dtype id, StreamWrapper stream, const void* x, len_t x_len, void* y, len_t y_len,
                           double alpha, double beta);

/* ------------------------------------------------------------------ losses
 * Fused row-softmax + cross-entropy, forward and backward in one pass
 * (src/nn/loss.zig:130-215):
 *   p = exp(x - (max + log sum exp(x - max)))
 *   loss_out[0] = (sum_rows -sum_j t_j log(clamp(p_j, 1e-7, 1-1e-7))) / loss_div
 *   dlogits (+)= (p - t) / loss_div           (when dlogits != NULL)
 * labels: ZG_LABEL_ONEHOT = fp32 [rows,C] probability rows (what the
 * reference feeds); ZG_LABEL_INDEX = u64 class index per row.
 * loss_out is ONE device scalar (overwritten); probs_out (optional) receives
 * p.  loss_div = the batch size; a data-parallel shard passes the GLOBAL
 * batch and sums loss_out over the shards.  accumulate != 0 adds into dlogits
 * (the reference's `+=` into a zero-filled gradient), 0 overwrites.
 * ld = row stride (elements) of logits, dlogits and probs_out (0 means C);
 * one-hot labels are contiguous [rows, C].  dbias (optional, fp32 [C],
 * C <= 1024) receives the column sums of (p - t)/loss_div, i.e. the bias
 * gradient of the layer that produced the logits (what InplaceAddBwd's
 * unbroadcast computes, src/ndtensor.zig:783-788), saving a pass over dlogits. */
enum { ZG_LABEL_ONEHOT = 0, ZG_LABEL_INDEX = 1 };
EXTERN_C void zg_softmax_ce_fwd_bwd(dtype id, StreamWrapper stream, const void* logits, const void* labels,
                                    int label_kind, len_t rows, len_t C, len_t ld, double loss_div,
                                    void* loss_out, void* dlogits, int accumulate, void* probs_out, void* dbias);
/* Smooth-L1 / Huber, mean reduction (src/nn/loss.zig:259-305):
 * loss_out[0] = mean(huber(pred - target)) (overwritten);
 * grad += d/(beta*n) or sign(d)/n  (when grad != NULL) */
EXTERN_C void zg_smooth_l1_fwd_bwd(dtype id, StreamWrapper stream, const void* pred, const void* target,
                                   len_t n, double beta, void* loss_out, void* grad);

/* The middle of an MLP training step as ONE launch, for the layer widths of the
 * MNIST model (h1 = 128 -> h2 = 64 -> C <= 16 classes; examples/mnist/src/model.zig:34-55).
 * Given act0 [rows, h1] (the post-ReLU output of the preceding layer) it does
 * what the reference issues as six device calls and two host loops:
 *   act1 = relu(act0 W1^T + b1)                       bmm_acc, add, relu_fwd (model.zig:100-112, src/nn/nn.zig:39-62)
 *   logits = act1 W2^T + b2                           bmm_acc, add
 *   loss_out[0], dlogits = softmax cross-entropy      src/nn/loss.zig:130-215 (as zg_softmax_ce_fwd_bwd, accumulate = 0)
 *   db2 += colsum(dlogits)                            InplaceAddBwd (src/ndtensor.zig:783-788)
 *   dact1 = (dlogits W2) where act1 > 0; db1 += ..    BmmAccBwd dX (src/ndtensor.zig:1107-1109) + relu_inplace_bwd
 *   dact0 = (dact1 W1) where act0 > 0;  db0 += ..     (src/device/host_device.zig:543-547)
 * W1 [h2, h1], b1 [h2], W2 [C, h2], b2 [C]; logits / dlogits have row stride
 * ld_out >= C (only C columns are written); act1 / dact1 [rows, h2], dact0
 * [rows, h1], all fp32 and contiguous.  db2 / db1 / db0 are ADDED to with fp32
 * atomics (zero them first: in a step they are slices of the zero-filled
 * gradient buffer).  The weight gradients are NOT formed here: dW2 = dlogits^T
 * act1, dW1 = dact1^T act0 and the preceding layer's dW = dact0^T x are three
 * independent zg_bmm calls afterwards.  3xTF32 tensor-core products, fp32
 * everywhere else.
 * weights_ready != 0: the caller vouches that W1, b1, W2 and b2 are not written
 * by the kernel launched immediately before this call on the stream, so they
 * are fetched while that kernel still runs (true inside a training step, where
 * that kernel is the preceding layer's forward GEMM).
 * zg_mlp_tail_supported: 1 when the widths (and the math mode) have a kernel;
 * otherwise the caller issues the separate ops. */
EXTERN_C int zg_mlp_tail_supported(dtype id, len_t h1, len_t h2, len_t C);
EXTERN_C void zg_mlp_tail_fwd_bwd(dtype id, StreamWrapper stream, len_t rows, len_t h1, len_t h2, len_t C,
                                  const void* act0, const void* W1, const void* b1, const void* W2, const void* b2,
                                  const void* labels, int label_kind, len_t ld_out, double loss_div,
                                  void* act1, void* logits, void* loss_out, void* dlogits, void* dact1, void* dact0,
                                  void* db2, void* db1, void* db0, int weights_ready);

/* -------------------------------------------------------------- optimizers
 * One launch over a whole parameter set.  The tensors of a model live back to
 * back (attach order) in one parameter buffer and one gradient buffer; seg
 * describes them.  offset/len are in elements. */
typedef struct {
  len_t offset;
  len_t len;
} zg_segment;

/* SGD.update over every segment (src/nn/optim.zig:100-122): per tensor
 * [if clip: nrm = ||g||; if nrm > max_norm: g *= max_norm/(nrm+delta)] then
 * p += (-lr)*g.  norms is a device scratch of n_seg floats (used when clip). */
/* clip: 0 = off; 1 = the call computes the per-tensor norms itself; 2 = norms[j]
 * already holds ||g_j|| of tensor j (a sharded optimizer sums the squares of its
 * shard with zg_segment_sumsq, adds them up over the ranks and takes the root).
 * A segment may be empty (len 0): it still counts as a tensor for Adam's step
 * counter, which lets a rank list every tensor and own only parts of some. */
/* zero_grads != 0: the kernel also clears every gradient it has applied, which
 * is the next step's zero_grad (src/nn/model.zig:57-62) without a launch of its
 * own; the gradients are then NOT readable after the call. */
EXTERN_C void zg_sgd_step(dtype id, StreamWrapper stream, void* params, void* grads,
                          const zg_segment* seg, len_t n_seg, double lr,
                          int clip, double max_norm, double delta, void* norms, int zero_grads);
/* Adam.update over every segment (src/nn/optim.zig:177-234), all in fp32:
 * the step counter advances once per TENSOR (optim.zig:189): segment j uses
 * t = t_first + j.  m, v are laid out like params.  When bf16_copy != NULL
 * the updated parameters are also written there as bfloat16.
 * step_counter (optional): a device u64 holding the number of tensor updates
 * done so far.  When given, t comes from it (segment j uses counter + j + 1,
 * t_first is ignored) and it is advanced by n_seg after the update, so a step
 * captured into a CUDA graph keeps counting when it is replayed. */
EXTERN_C void zg_adam_step(dtype id, StreamWrapper stream, void* params, void* grads, void* m, void* v,
                           const zg_segment* seg, len_t n_seg, len_t t_first,
                           double lr, double beta1, double beta2, double eps,
                           int clip, double max_norm, double delta, void* norms, void* bf16_copy, void* step_counter);
/* The same over PART of a model: seg lists every tensor of the model in attach order with
 * length 0 for those this call leaves alone (an empty segment costs nothing and keeps the
 * positions, hence the per-tensor step counts, of the others).  advance_counter = 0 reads
 * step_counter without advancing it, so that the tensors of one optimizer step can be
 * updated by several calls (a layer at a time, as its gradient becomes final during the
 * backward pass); the last call of the step passes 1. */
EXTERN_C void zg_adam_step_part(dtype id, StreamWrapper stream, void* params, void* grads, void* m, void* v,
                                const zg_segment* seg, len_t n_seg, len_t t_first,
                                double lr, double beta1, double beta2, double eps,
                                int clip, double max_norm, double delta, void* norms, void* bf16_copy, void* step_counter,
                                int advance_counter);
/* out[j] = sum of squares of segment j (fp64 accumulation, deterministic two-stage): the
 * shard-local part of the per-tensor gradient norm of host_device.zig:339-346 */
EXTERN_C void zg_segment_sumsq(dtype id, StreamWrapper stream, const void* x, const zg_segment* seg, len_t n_seg, void* out);
/* target[i] = tau*src[i] + (1-tau)*target[i] (examples/dqn/src/dqn_agent.zig:111-123) */
EXTERN_C void zg_soft_update(dtype id, StreamWrapper stream, const void* src, void* target, len_t n, double tau);
/* fp32 -> bf16 (round to nearest even) and back */
EXTERN_C void zg_cast(dtype src_id, dtype dst_id, StreamWrapper stream, const void* src, void* dst, len_t n);

/* ------------------------------------------------------------------- index
 * opspec.scatter_add (host_device.zig:1039-1086): dst[offsets[i]] += src[i] */
EXTERN_C void zg_scatter_add(dtype id, StreamWrapper stream, const void* src, const len_t* offsets, len_t n, void* dst);
/* opspec.scatter_add_2d (host_device.zig:1137-1160): dst[indices[i], :] += src[i, :]
 * for n_blocks blocks of `stride` contiguous elements (fp atomics: the values
 * added are the reference's, the order in which duplicates land is not). */
EXTERN_C void zg_scatter_add_2d(dtype id, StreamWrapper stream, const void* src, const len_t* indices, len_t n_blocks,
                                len_t stride, void* dst);
/* opspec.scatter_add_csr (host_device.zig:1325-1335): dst[j] += src[i] for
 * j in [row_ptr[i], row_ptr[i+1]); row_ptr has n_segments + 1 entries. Exact. */
EXTERN_C void zg_scatter_add_csr(dtype id, StreamWrapper stream, const void* src, const len_t* row_ptr, len_t n_segments, void* dst);
/* opspec.segment_sum_csr (host_device.zig:1337-1351): dst[i] = sum of
 * src[row_offsets[i] .. row_offsets[i+1]) (overwritten).  Segments of up to 32
 * elements are added left to right like the host loop; longer ones by 32
 * strided partial sums and a fixed shuffle tree. */
EXTERN_C void zg_segment_sum_csr(dtype id, StreamWrapper stream, const void* src, const len_t* row_offsets, len_t n_segments, void* dst);
/* NDArray.gather along dim 1 of a [rows, cols] array with one index per row
 * (src/ndarray.zig:593-633; offsets are computed on the host there):
 * dst[r] = src[r*cols + idx[r]]; offsets_out (optional) receives r*cols+idx[r] */
EXTERN_C void zg_gather_rows(dtype id, StreamWrapper stream, const void* src, const len_t* idx, len_t rows,
                             len_t cols, void* dst, len_t* offsets_out);
/* opspec.scatter_gcn_deg_scaled (+_bwd) (host_device.zig:1356-1403) */
EXTERN_C void zg_scatter_gcn_deg_scaled(dtype id, StreamWrapper stream, void* dst, const void* h, const void* deg,
                                        const len_t* src_idx, const len_t* tgt_idx, len_t stride, len_t n_edge);
EXTERN_C void zg_scatter_gcn_deg_scaled_bwd(dtype id, StreamWrapper stream, const void* grad_out, const void* h,
                                            const void* deg, const len_t* src_idx, const len_t* tgt_idx,
                                            void* grad_h, void* grad_deg, len_t stride, len_t n_edge);
/* The same propagation over a CSR form of the edge list, without atomics
 * (deterministic; the graph is static, so the CSR is built once on the host by a
 * STABLE sort of the edges, which keeps every sum in edge order and the result
 * bit-identical to the host loops above):
 *   transpose_form == 0, edges grouped by target (row = t, col_idx = s):
 *       out[t,j] = sum_e (deg[s]*deg[t]) * x[s,j]   [+ bias[j]] [ReLU]   -- scatter_gcn_deg_scaled on a zero dst
 *   transpose_form == 1, edges grouped by source (row = s, col_idx = t):
 *       out[s,j] = sum_e (x[t,j]*deg[s]) * deg[t]                        -- grad_h of scatter_gcn_deg_scaled_bwd
 * out is overwritten; ld_x / ld_out are row strides in elements; epilogue is
 * ZG_EPI_NONE, ZG_EPI_BIAS or ZG_EPI_BIAS_RELU (GraphConvLayer's `+ bias` and the
 * ReLU after it, examples/gcn/src/model.zig:36,100-112). */
EXTERN_C void zg_csr_gcn_propagate(dtype id, StreamWrapper stream, void* out, const void* x, const void* deg,
                                   const len_t* row_ptr, const len_t* col_idx, len_t n_rows, len_t n_feat,
                                   len_t ld_x, len_t ld_out, int transpose_form, int epilogue, const void* bias);

/* ------------------------------------------------- peer-memory all-reduce
 * Sum all-reduce of a small fp32 buffer (the data-parallel step's flat gradient
 * buffer) across the GPUs of one box in ONE kernel per rank, over NVLink loads
 * and stores to peer memory instead of a library collective.  The reference has
 * no distributed code (docs/roadmap.norg:74-76 lists it as future work).
 *
 * Set-up, once per process group: every rank allocates a comm region
 * (zg_comm_alloc: plain device memory, cleared, holding a control block and, per
 * epoch parity and source rank, a receive slot of cap_elems {value, epoch}
 * words; cap_elems even), exports its IPC handle (zg_ipc_export, 64 bytes),
 * exchanges handles with the other ranks by any host channel, maps theirs
 * (zg_ipc_open) and synchronises on the host before the first call.
 *
 * zg_allreduce_oneshot(stream, buf, n, rank, world, comm, cap_elems): comm[r] is
 * rank r's region as mapped in THIS process (comm[rank] the local one).  After
 * the kernel buf holds the sum over ranks, added in rank order on every rank
 * (bit-identical replicas).  Every rank must launch it the same number of times
 * (an epoch counter in device memory pairs the launches, so captured graphs can
 * replay it); world <= 8; n <= cap_elems.  Waits on peers are bounded: when one
 * runs out the kernel stops reducing, leaves buf partly reduced and reports it. */
EXTERN_C void* zg_comm_alloc(len_t cap_elems, unsigned world);
EXTERN_C void zg_comm_free(void* region);
EXTERN_C void zg_ipc_export(void* dptr, unsigned char* handle_out64);
EXTERN_C void* zg_ipc_open(const unsigned char* handle64);
EXTERN_C void zg_ipc_close(void* dptr);
/* zg_comm_error synchronises the stream, returns the region's error word (1 = a
 * launch since the last call gave up waiting) and clears it; the same event also
 * raises the library-wide time-out status (zg_last_error() == 4 after the next
 * stream_synchronize).  zg_comm_set_spin_limit sets how many polls a wait may
 * take (0 restores the default, about seconds; ZG_SPIN_LIMIT in the environment
 * sets the initial value) -- a short limit is how a host notices a missing peer
 * quickly, and how the give-up path is tested without hanging a GPU. */
EXTERN_C int zg_comm_error(void* region, StreamWrapper stream);
EXTERN_C void zg_comm_set_spin_limit(unsigned polls);
EXTERN_C void zg_allreduce_oneshot(StreamWrapper stream, void* buf, len_t n, unsigned rank, unsigned world,
                                   void* const* comm, len_t cap_elems);
/* The same reduction with the SGD update of src/nn/optim.zig:100-122 (no
 * clipping) applied to the reduced gradient in the same kernel:
 * params[i] += (-lr) * sum_r grads_r[i]; grads receives the sum as well, or
 * zeros when zero_grads != 0 (the next step's zero_grad, as in zg_sgd_step). */
EXTERN_C void zg_allreduce_sgd_oneshot(StreamWrapper stream, void* grads, void* params, len_t n, double lr,
                                       unsigned rank, unsigned world, void* const* comm, len_t cap_elems, int zero_grads);

/* ------------------------------------------------------ library collectives
 * The gradient exchange of a data-parallel step for buffers that are
 * bandwidth-bound (the wide model's 218 MB of gradients): sum all-reduce,
 * reduce-scatter and all-gather through NCCL over NVLink / NVSwitch, one
 * communicator per process (= per GPU).  The reference has no distributed code
 * (docs/roadmap.norg:74-76); the contract is "the same update as on a single
 * device": gradients are summed over the ranks BEFORE clipping and the
 * optimizer (src/nn/optim.zig:100-122, 177-234).
 *
 * NCCL is bound at run time: zg_nccl_load(path) loads the given library (NULL:
 * $ZG_NCCL_LIB, then a copy already loaded in the process, then libnccl.so.2
 * from the loader path) and returns its version code, 0 if none was found.  The
 * other calls bind it on first use and set status 5 when there is none.
 *
 * Rendezvous: rank 0 calls zg_nccl_unique_id (128 bytes), hands the bytes to the
 * other ranks over any host channel, then EVERY rank calls zg_comm_init_rank
 * with its device current (collective, blocking).  All calls below are
 * asynchronous on `stream`, in place where one buffer is given, and may be
 * captured into a CUDA graph like any kernel launch.
 *   zg_allreduce       buf[i] = sum over ranks of buf[i], n elements
 *   zg_reduce_scatter  recv[i] = sum over ranks of send[rank*recv_n + i]
 *                      (recv may point into send at rank*recv_n: in place)
 *   zg_all_gather      recv[r*send_n + i] = rank r's send[i]
 *                      (send may be recv + rank*send_n: in place)
 * id is SINGLE, DOUBLE or BF16.
 * zg_comm_peer_regions does the host-side set-up of the peer-memory all-reduce
 * above over an existing communicator: exports my_region (from zg_comm_alloc),
 * all-gathers the IPC handles and maps the peers' regions; regions_out[world]
 * is then the `comm` argument of zg_allreduce_oneshot.  Returns 0 on success. */
typedef struct { void* ptr; } CommWrapper;
EXTERN_C int zg_nccl_load(const char* path);
EXTERN_C void zg_nccl_unique_id(unsigned char* id_out128);
EXTERN_C CommWrapper zg_comm_init_rank(const unsigned char* id128, unsigned rank, unsigned world);
EXTERN_C void zg_comm_destroy(CommWrapper comm);
EXTERN_C unsigned zg_comm_rank(CommWrapper comm);
EXTERN_C unsigned zg_comm_world(CommWrapper comm);
EXTERN_C void zg_allreduce(CommWrapper comm, void* buf, len_t n, dtype id, StreamWrapper stream);
EXTERN_C void zg_reduce_scatter(CommWrapper comm, const void* send, void* recv, len_t recv_n, dtype id, StreamWrapper stream);
EXTERN_C void zg_all_gather(CommWrapper comm, const void* send, void* recv, len_t send_n, dtype id, StreamWrapper stream);
EXTERN_C int zg_comm_peer_regions(CommWrapper comm, void* my_region, void** regions_out, StreamWrapper stream);

/* --------------------------------------------- stream-ordered caching allocator
 * Device-side replacement for the Zig CachingAllocator + BlockPool
 * (src/allocators/caching_allocator.zig:15-162, block_pool.zig:103-412) behind
 * mem_cache_alloc / mem_cache_free / mem_scratch
 * (src/device/device_reference.zig:29-60).  A freed block is reusable at once
 * by later work on the SAME stream; reuse from another stream waits on an event
 * recorded at free time.  `ctx` is the opaque block handle that DeviceData.ctx
 * carries (src/allocators/device_data.zig:32-40). */
typedef struct { void* ptr; } CacheWrapper;
typedef struct { void* ptr; len_t ctx; } zg_block;
EXTERN_C CacheWrapper zg_cache_create(unsigned device_id, len_t max_bytes /* 0 = no limit */);
EXTERN_C void zg_cache_destroy(CacheWrapper cache);
EXTERN_C zg_block zg_cache_alloc(CacheWrapper cache, len_t nbytes, StreamWrapper stream); /* ptr NULL on OOM */
EXTERN_C void zg_cache_free(CacheWrapper cache, zg_block block, StreamWrapper stream);
EXTERN_C void* zg_cache_scratch(CacheWrapper cache, len_t nbytes, StreamWrapper stream);  /* valid until next call */
EXTERN_C void zg_cache_clear(CacheWrapper cache);   /* returns cached (unused) blocks to the driver */
/* stats: [0] bytes reserved from the driver, [1] bytes in live blocks,
 * [2] allocations served from cache, [3] allocations that grew the arena */
EXTERN_C void zg_cache_stats(CacheWrapper cache, len_t* out4);

#endif
