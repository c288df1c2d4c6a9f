/*
 * supa_b200_kernels.h -- C ABI of the B200 (sm_100a) kernel library behind the
 * torch-supa operator hot path.
 *
 * Every entry point is a plain `extern "C"` launcher: POD descriptors, raw device
 * pointers, sizes and a CUDA stream.  Launchers are asynchronous on the given stream,
 * never allocate, never synchronise, never change the current device and are
 * thread-safe.  They return 0 on success or a negative sb_status.  Errors found in the
 * *data* on the device (an out-of-range class index) are never a trap: the kernel sets
 * bits in a caller-supplied status word and treats the row as ignored; the host reads
 * the word at its next natural synchronisation point.
 *
 * Each declaration names the reference interface it replaces; paths are relative to the
 * torch-supa source tree.
 */
#ifndef SUPA_B200_KERNELS_H_
#define SUPA_B200_KERNELS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_API __attribute__((visibility("default")))

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer; NULL is the legacy
 * default stream. */
typedef void* sb_stream_t;

typedef enum sb_status {
  SB_OK = 0,
  SB_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, bad enum value */
  SB_ERR_UNSUPPORTED = -2,      /* dtype / op combination that has no kernel */
  SB_ERR_CUDA = -3,             /* the launch itself failed (cudaGetLastError) */
  SB_ERR_TOO_LARGE = -4,        /* a size beyond what the entry point documents */
  SB_ERR_MISALIGNED = -5        /* pointer not aligned to its element size */
} sb_status;

/* Element types.  The numbering is private to this library (the ATen shim maps
 * c10::ScalarType onto it). */
typedef enum sb_dtype {
  SB_BOOL = 0,
  SB_U8 = 1,
  SB_I8 = 2,
  SB_I16 = 3,
  SB_I32 = 4,
  SB_I64 = 5,
  SB_F16 = 6,
  SB_BF16 = 7,
  SB_F32 = 8,
  SB_F64 = 9,
  SB_DTYPE_COUNT = 10
} sb_dtype;

/* Bits of the device status word. */
#define SB_STATUS_TARGET_OUT_OF_RANGE 0x1 /* a class index outside [0, classes) and != ignore_index */
#define SB_STATUS_KERNEL_TIMEOUT 0x2      /* a bounded wait inside a kernel ran out; its results are invalid */
#define SB_STATUS_GRADIENT_LOST 0x4      /* sb_ce_rescale_grad was asked to undo a factor of zero */

typedef enum sb_reduction { SB_REDUCTION_NONE = 0, SB_REDUCTION_MEAN = 1, SB_REDUCTION_SUM = 2 } sb_reduction;

/* Library identification: version string and the SM architecture the kernels were built for. */
SB_API const char* sb_version(void);
SB_API int sb_built_for_sm(void);
/* Human-readable text for an sb_status. */
SB_API const char* sb_status_string(int status);
/* sizeof one element of `dtype`, 0 if unknown. */
SB_API size_t sb_dtype_size(int dtype);

/* ------------------------------------------------------------------------------------------
 * Cross entropy (class-index targets), forward and backward in one sweep.
 *
 * Replaces cross_entropy_loss_2d_kernel_supa and its kernel family
 * (torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:71-195,580-749) and the
 * backward chain nll_loss_backward -> _log_softmax_backward_data of
 * CrossEntropyLossFastPathFunction (torch_supa/csrc/aten/ops/CrossEntropyLoss.cpp:94-135), plus the
 * ignore_index / label_smoothing arithmetic of the upstream composite the reference falls back to
 * (CrossEntropyLoss.cpp:50).
 *
 * Protocol for reduction = mean / sum on one or several GPUs (acc is two doubles on the device:
 * acc[0] = loss sum, acc[1] = number of rows whose target != ignore_index):
 *   1. sb_ce_count_valid      -> acc[1]            (then all-reduce acc[1] when rows are sharded)
 *   2. sb_ce_forward_backward -> row_loss, grad    (reads acc[1] for the 1/|V| scale of `mean`)
 *   3. sb_ce_loss_sum         -> acc[0]            (then all-reduce acc[0] when rows are sharded)
 *   4. sb_ce_loss_finish      -> loss scalar in the logits' dtype
 * For reduction = none only step 2 is needed and row_loss is the result.
 * ------------------------------------------------------------------------------------------ */
typedef struct sb_ce_args {
  const void* logits;      /* [rows, classes], row-major, row stride = classes elements */
  int32_t dtype;           /* SB_F32, SB_BF16 or SB_F16 (math is fp32 for all three) */
  int32_t reduction;       /* sb_reduction: selects the gradient scale (mean: 1/acc[1]; sum, none: 1) */
  const int64_t* target;   /* [rows] class indices; rows equal to ignore_index contribute nothing */
  void* grad_logits;       /* [rows, classes] same dtype as logits, or NULL for forward only.
                              May alias `logits` (in-place gradient). */
  float* row_loss;         /* [rows] per-row loss, 0 for ignored rows (the result for `none`) */
  float* row_lse;          /* [rows] per-row log-sum-exp, or NULL */
  const float* row_grad_out; /* [rows] upstream gradient per row (for `none`), or NULL for 1 */
  const double* acc;       /* device pointer to {loss_sum, valid_count}; acc[1] is read when
                              reduction == mean and grad_logits != NULL.  May be NULL otherwise. */
  int64_t rows;
  int64_t classes;
  int64_t ignore_index;
  float label_smoothing;   /* in [0, 1] */
  float grad_scale;        /* extra host-side factor on the gradient (the upstream scalar, usually 1) */
  int32_t* status;         /* device status word, OR-ed with SB_STATUS_* bits; may be NULL */
  const float* class_weight; /* [classes] fp32 per-class weights (the `weight` argument of cross_entropy), or NULL.
                                Row i's loss and gradient are multiplied by class_weight[target_i]; with mean the
                                denominator acc[1] must then be the sum of those weights (sb_ce_count_weighted).
                                With label_smoothing > 0 the smoothing term weights every class c of the row by
                                class_weight[c], as the upstream composite does (CrossEntropyLoss.cpp:50); that
                                combination runs on the two-sweep kernel. */
  uint32_t flags;            /* SB_CE_FLAG_* */
} sb_ce_args;

/* The launch directly before this one on the same stream is sb_ce_count_valid / sb_ce_count_weighted /
 * sb_ce_count_exchange of the same call (it produces acc[1]).  The sweep may then start its loads while that
 * kernel still runs (programmatic dependent launch); it waits for acc[1] before the first gradient is formed.
 * Do not set it when anything else precedes the sweep on the stream. */
#define SB_CE_FLAG_AFTER_COUNT 0x1u

/* Counts rows with target != ignore_index into acc[1] (as a double) and zeroes acc[0]; flags
 * out-of-range targets in *status.  Replaces the `counts[row]` side buffer of
 * cross_entropy_index_mean_kernel (CrossEntropyLossKernel.cu:121-162). */
SB_API int sb_ce_count_valid(const int64_t* target, int64_t rows, int64_t classes, int64_t ignore_index,
                             double* acc, int32_t* status, sb_stream_t stream);

/* The same with class weights: acc[1] = sum of class_weight[target_i] over the rows that count, added in a fixed
 * order (bit-reproducible); acc[0] = 0. */
SB_API int sb_ce_count_weighted(const int64_t* target, const float* class_weight, int64_t rows, int64_t classes,
                                int64_t ignore_index, double* acc, int32_t* status, sb_stream_t stream);

/* The fused sweep (see protocol above). */
SB_API int sb_ce_forward_backward(const sb_ce_args* args, sb_stream_t stream);

/* acc[0] = sum(row_loss[0..rows)) in a fixed order (bit-reproducible; no float atomics, unlike the
 * atomicAdd of cross_entropy_index_kernel, CrossEntropyLossKernel.cu:113). */
SB_API int sb_ce_loss_sum(const float* row_loss, int64_t rows, double* acc, sb_stream_t stream);

/* loss = acc[0] / acc[1] for mean (NaN when acc[1] == 0, as
 * cross_entropy_finalize_mean_buffer_kernel, CrossEntropyLossKernel.cu:164-195), acc[0] for sum;
 * written as one element of `dtype` at `out`. */
SB_API int sb_ce_loss_finish(const double* acc, int32_t reduction, void* out, int32_t dtype, sb_stream_t stream);

/* sb_ce_loss_sum followed by sb_ce_loss_finish in one launch (single-GPU case: no all-reduce between). */
SB_API int sb_ce_loss_sum_finish(const float* row_loss, int64_t rows, double* acc, int32_t reduction, void* out,
                                 int32_t dtype, sb_stream_t stream);

/* dst[i] = src[i] * factor where factor = *scale / *applied_in (device floats; a null applied_in stands for 1, the
 * state right after the fused sweep).  dst may be src (in place): the sweep is then skipped on the device when the
 * factor is exactly 1.  When applied_out is not null, *applied_out = *scale records the factor now folded into an
 * in-place buffer; it must be a different word from applied_in (callers alternate between two).  A stored factor
 * of zero cannot be undone: the kernel then sets SB_STATUS_GRADIENT_LOST in *status (may be NULL) and writes NaN,
 * unless *scale is zero too.  Used by the autograd node when the upstream gradient of a mean/sum loss is not 1. */
SB_API int sb_ce_rescale_grad(const void* src, void* dst, int32_t dtype, int64_t numel, const void* scale, int32_t scale_dtype,
                              const float* applied_in, float* applied_out, int32_t* status, sb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * The two scalar exchanges of row-sharded cross entropy, done by the bookkeeping kernels themselves.
 *
 * Replaces the all-reduce of ProcessGroupBCCL::allreduce (torch_supa/csrc/distributed/ProcessGroupBCCL.cpp:3723-3790)
 * for the two 8-byte messages of this path: every rank (one process per GPU) owns a small slot array in its device
 * memory that all other ranks have mapped (CUDA IPC); a kernel publishes its partial with plain stores into every
 * peer's array, then waits (bounded) for the partials of all ranks in its own array and adds them in rank order,
 * so that every rank gets the same bits.  No NCCL launch sits between the count, the sweep and the loss.
 *
 *   slots[r]  device address, valid on THIS GPU, of rank r's slot array (SB_XCHG_SLOT_BYTES bytes, zeroed once
 *             before first use); slots[rank] is this GPU's own array.
 *   seq       number of this exchange on the communicator: 1, 2, 3, ... in the same order on every rank.
 * A wait that runs out (default 10 s, see sb_set_tuning key 5) sets SB_STATUS_KERNEL_TIMEOUT in *status, and the
 * kernel finishes with the partials that did arrive; nothing hangs.
 * ------------------------------------------------------------------------------------------ */
#define SB_XCHG_MAX_RANKS 8
#define SB_XCHG_DEPTH 4
#define SB_XCHG_SLOT_BYTES (SB_XCHG_DEPTH * SB_XCHG_MAX_RANKS * 16)
typedef struct sb_xchg {
  void* slots[SB_XCHG_MAX_RANKS];
  int32_t rank;
  int32_t nranks;
  uint64_t seq;
} sb_xchg;

/* sb_ce_count_valid (class_weight == NULL) or sb_ce_count_weighted in one launch and with no memset, followed, when
 * x is not NULL, by the exchange: acc[1] = sum over ranks, acc[0] = 0. */
SB_API int sb_ce_count_exchange(const int64_t* target, const float* class_weight, int64_t rows, int64_t classes,
                                int64_t ignore_index, double* acc, int32_t* status, const sb_xchg* x, sb_stream_t stream);

/* sb_ce_loss_sum_finish with the exchange of the loss sum between the sum and the division when x is not NULL:
 * acc[0] = sum over ranks of the local fixed-order sums.  Launched as a programmatic dependent of the kernel
 * before it (it waits for that kernel's results before it reads anything). */
SB_API int sb_ce_loss_exchange(const float* row_loss, int64_t rows, double* acc, int32_t reduction, void* out, int32_t dtype,
                               int32_t* status, const sb_xchg* x, sb_stream_t stream);

/* Cross entropy (mean or sum) for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference.  The other cross-entropy launchers need two small
 * scratch buffers from the caller (the per-row losses and the {loss sum, valid rows} accumulator).  Some
 * callers have nowhere to get them: a host runtime that binds this C ABI from another language and owns no
 * device allocator, a serving process whose memory is fully committed at start-up, or a section in which
 * cudaMalloc's implicit device-wide synchronisation is not acceptable.  For them the scratch lives in a
 * file-scope array in device memory inside the library (SB_CE_STATIC_MAX_ROWS * 4 + 256 bytes, held by every
 * GPU that loads the library until the process exits).  The call runs the whole sequence -- valid-row
 * count, fused sweep, loss sum and finish -- and calls no cudaMalloc, cudaFree or other allocating routine.
 *
 *   args      as for sb_ce_forward_backward, with reduction = mean or sum; grad_logits may be NULL.  The
 *             fields row_loss, row_lse, row_grad_out and acc must be NULL: the library supplies them.
 *   loss_out  one element of args->dtype in device memory.
 *
 * Returns SB_ERR_TOO_LARGE when args->rows exceeds SB_CE_STATIC_MAX_ROWS.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before any stream capture begins.
 * All calls share the one array and it keeps the previous call's contents; everything a call reads from it
 * is rewritten by that call first.  Two calls that overlap on the GPU (different streams, no dependency)
 * race on it: serialise them. */
#define SB_CE_STATIC_MAX_ROWS 65536
SB_API int sb_ce_loss_static_scratch(const sb_ce_args* args, void* loss_out, sb_stream_t stream);

/* Which kernel family sb_ce_forward_backward will use for this shape: 0 = generic two-sweep rows,
 * 1 = row resident in shared memory of one CTA (TMA bulk ring), 2/4 = resident across a cluster
 * of 2/4 CTAs, 16 = aligned rows of 256 B to 32 KB on the shared-memory slot ring (part of a warp, a warp or four warps per row), 8 = other rows
 * shorter than 16 KB held in registers.  For diagnostics and benchmarks. */
SB_API int sb_ce_kernel_variant(int32_t dtype, int64_t rows, int64_t classes);

/* Tuning hook for benchmarks and profiling (process-wide, not thread-safe against running launches):
 * key 1 = cross-entropy kernel family (-1 automatic, 0 always the generic two-sweep kernel, 1/2/4 the
 * resident kernel with that cluster size where the shape qualifies for a resident kernel at all, 8 = short rows in
 * registers also where the slot ring would take them);
 * key 2 = chunks of the next row the resident kernel folds while a row's statistics are exchanged
 * (-1 automatic, 0..64);
 * key 3 = how the resident kernel forms bf16 gradients: 1 (default) rescales the exponentials kept from the statistics
 * sweep (one ex2 per logit, one more bf16 rounding), 0 recomputes them (two ex2 per logit);
 * key 5 = limit, in milliseconds, of the waits of sb_ce_count_exchange / sb_ce_loss_exchange (1..60000, default 10000);
 * key 6 = consumer warps per CTA of the slot-ring kernel (0 automatic, 1..16);
 * key 7 = longest row, in bytes, the slot-ring kernel takes (16384..65536, default 32768);
 * key 8 = longest row, in bytes, that one warp reduces in sb_reduce before a CTA takes each row (0 = the 16-byte
 * vector row kernels off, 4096..262144, default 8192). */
SB_API int sb_set_tuning(int32_t key, int32_t value);

/* ------------------------------------------------------------------------------------------
 * log_softmax / nll_loss as separate operators.
 *
 * Replace the kernels behind aten::_log_softmax(.out), aten::_log_softmax_backward_data(.out),
 * aten::nll_loss_forward(.output) and aten::nll_loss_backward(.grad_input) that the reference takes
 * from its external native-op library (call sites: torch_supa/csrc/aten/ops/CrossEntropyLoss.cpp:76,79,127,132).
 * The tensor is viewed as [outer, dim, inner] with the softmax taken over `dim`.
 * ------------------------------------------------------------------------------------------ */
SB_API int sb_log_softmax_forward(const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t outer,
                                  int64_t dim, int64_t inner, sb_stream_t stream);
/* grad_in = grad_out - exp(out) * sum_dim(grad_out) */
SB_API int sb_log_softmax_backward(const void* grad_out, const void* out, int32_t dtype, void* grad_in,
                                   int32_t grad_in_dtype, int64_t outer, int64_t dim, int64_t inner,
                                   sb_stream_t stream);

/* softmax (not log) with the same layout and dtype pairs: out = exp(x - logsumexp);
 * backward: grad_in = out * (grad_out - sum(grad_out * out)).  One of the neighbouring operators of the
 * external native-op library (reference tests: test/test_softmax.py, test/test_persistent_softmax.py). */
SB_API int sb_softmax_forward(const void* in, int32_t in_dtype, void* out, int32_t out_dtype, int64_t outer, int64_t dim,
                              int64_t inner, sb_stream_t stream);
SB_API int sb_softmax_backward(const void* grad_out, const void* out, int32_t dtype, void* grad_in, int32_t grad_in_dtype,
                               int64_t outer, int64_t dim, int64_t inner, sb_stream_t stream);

typedef struct sb_nll_args {
  const void* log_probs;  /* [rows, classes] contiguous */
  int32_t dtype;          /* SB_F32, SB_BF16, SB_F16, SB_F64 */
  int32_t target_dtype;   /* SB_I64 or SB_U8 */
  const void* target;     /* [rows] */
  const void* weight;     /* [classes] in `dtype`, or NULL */
  int64_t rows;
  int64_t classes;
  int64_t ignore_index;
  int32_t reduction;
  int32_t* status;
} sb_nll_args;
/* output: [rows] for none, one element otherwise; total_weight: one element (sum of the weights of
 * the rows that count).  Both in args->dtype. */
SB_API int sb_nll_loss_forward(const sb_nll_args* args, void* output, void* total_weight, sb_stream_t stream);
/* grad_input[rows, classes] = 0 except [i, target_i] = -w * g (/ total_weight for mean). */
SB_API int sb_nll_loss_backward(const sb_nll_args* args, const void* grad_output, const void* total_weight,
                                void* grad_input, sb_stream_t stream);

/* nll_loss over [outer, classes, inner] log-probabilities with [outer, inner] targets: the 4-D (N, C, H, W)
 * form of nll_loss2d_forward / nll_loss2d_backward (inner = H * W), which the reference takes from its
 * external native-op library (exercised by test/test_loss.py:24,150-233 with the shape (2, 19, 512, 1024));
 * inner = 1 is the plain [rows, classes] form.  Forward mean / sum reduce in two fixed-order stages through
 * `scratch` (sb_nll_loss_nd_scratch_bytes bytes, 16-byte aligned, caller-owned); backward writes every
 * element of grad_input exactly once (no separate zero-fill). */
typedef struct sb_nll_nd_args {
  const void* log_probs;  /* [outer, classes, inner] contiguous */
  int32_t dtype;          /* SB_F32, SB_BF16, SB_F16, SB_F64 */
  int32_t target_dtype;   /* SB_I64 or SB_U8 */
  const void* target;     /* [outer, inner] */
  const void* weight;     /* [classes] in `dtype`, or NULL */
  int64_t outer;
  int64_t classes;
  int64_t inner;
  int64_t ignore_index;
  int32_t reduction;
  int32_t* status;
  void* scratch;          /* forward with mean / sum only */
  size_t scratch_bytes;
} sb_nll_nd_args;
SB_API size_t sb_nll_loss_nd_scratch_bytes(const sb_nll_nd_args* args);
/* output: [outer, inner] for none, one element otherwise; total_weight: one element.  Both in args->dtype. */
SB_API int sb_nll_loss_nd_forward(const sb_nll_nd_args* args, void* output, void* total_weight, sb_stream_t stream);
/* grad_output: [outer, inner] for none, one element otherwise. */
SB_API int sb_nll_loss_nd_backward(const sb_nll_nd_args* args, const void* grad_output, const void* total_weight,
                                   void* grad_input, sb_stream_t stream);

/* binary_cross_entropy_with_logits with reduction mean or sum in one pass: the unreduced loss of SB_EW_BCE_LOGITS /
 * SB_EW_BCE_LOGITS_PW (times `weight` when given) is summed without being stored, where the reference writes it and
 * calls mean() / sum() (torch_supa/csrc/aten/ops/BinaryCrossEntropyWithLogits.cpp:39-72).  x, target and weight
 * are contiguous arrays of `numel` elements of `dtype` (SB_F32, SB_BF16, SB_F16, SB_F64); pos_weight has pw_len
 * elements and is indexed by (flat index % pw_len), i.e. it runs along the last dimension; weight and pos_weight may
 * be NULL.  `out` receives one element of `dtype`.  scratch: sb_bce_logits_scratch_bytes(numel) bytes, 8-byte aligned.
 * The summation order is fixed (bit-reproducible). */
SB_API size_t sb_bce_logits_scratch_bytes(int64_t numel);
SB_API int sb_bce_logits_reduce(const void* x, const void* target, const void* pos_weight, int64_t pw_len, const void* weight,
                                int32_t dtype, int64_t numel, int32_t reduction, void* out, void* scratch, size_t scratch_bytes,
                                sb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * TensorIterator-style elementwise engine.
 *
 * Replaces gpu_kernel / gpu_kernel_impl and its launch policies
 * (torch_supa/csrc/aten/ops/kernels/elementwise/Loops.cuh:110-134, CUDALoops.cuh:382-937) together with the
 * functors of add (UfuncCUDA_add.cu:77-341), mul (BinaryMulKernel.cu:25-43) and the gelu / silu / glu
 * stubs of the external native-op library.  Operand 0 is the output.  Shapes arrive already broadcast
 * (stride 0) and coalesced, fastest dimension first, strides in ELEMENTS of the operand's own dtype.
 * Arithmetic runs in the op-math type of `common_dtype` (fp32 for fp16/bf16) and is cast to the
 * output dtype on store, as Loops.cuh:176-209 does.
 * ------------------------------------------------------------------------------------------ */
#define SB_MAX_DIMS 25
#define SB_MAX_OPERANDS 4

typedef enum sb_ew_op {
  SB_EW_COPY = 0,          /* out = cast(in0) */
  SB_EW_FILL = 1,          /* out = scalar */
  SB_EW_ADD = 2,           /* out = in0 + alpha * in1      (bool: logical or) */
  SB_EW_MUL = 3,           /* out = in0 * in1              (bool: logical and) */
  SB_EW_SUB = 4,           /* out = in0 - alpha * in1 */
  SB_EW_DIV = 5,           /* out = in0 / in1 (true division, floating compute types) */
  SB_EW_GELU_ERF = 6,      /* unary */
  SB_EW_GELU_TANH = 7,     /* unary */
  SB_EW_SILU = 8,          /* unary */
  SB_EW_GLU = 9,           /* out = in0 * sigmoid(in1) */
  SB_EW_GELU_ERF_BWD = 10, /* out = in0(grad) * gelu'(in1(self)) */
  SB_EW_GELU_TANH_BWD = 11,
  SB_EW_SILU_BWD = 12,     /* out = in0(grad) * silu'(in1(self)) */
  SB_EW_GLU_BWD_A = 13,    /* out = sigmoid(in1(b)) * in0(grad)                      (gradient of the first half) */
  SB_EW_GLU_BWD_B = 14,    /* out = (1 - s) * s * in0(grad) * in2(a), s = sigmoid(in1(b)) (gradient of the second half) */
  SB_EW_ADD_SCALAR = 15,   /* out = in0 + alpha * scalar */
  SB_EW_MUL_SCALAR = 16,   /* out = in0 * scalar */
  SB_EW_NEG = 17,          /* unary */
  /* binary_cross_entropy_with_logits (torch_supa/csrc/aten/ops/kernels/elementwise/BinaryCrossEntropyWithLogitsKernel.cu:16-113):
   * loss = (1 - t) x + lw * softplus(-x), lw = 1 + (pw - 1) t; the result is multiplied by `alpha`. */
  SB_EW_BCE_LOGITS = 18,        /* in0 = x, in1 = t                      (lw = 1) */
  SB_EW_BCE_LOGITS_PW = 19,     /* in0 = x, in1 = t, in2 = pos_weight */
  SB_EW_BCE_LOGITS_BWD = 20,    /* alpha * in2(upstream gradient) * (sigmoid(x) - t) */
  SB_EW_BCE_LOGITS_PW_BWD = 21, /* alpha * (lw * sigmoid(x) - pw * t), in2 = pos_weight */
  SB_EW_SIGMOID = 22,           /* unary */
  /* Neighbouring TensorIterator operators of the external native-op library, served by the same engine. */
  SB_EW_TANH = 23,              /* unary */
  SB_EW_EXP = 24,               /* unary */
  SB_EW_LOG = 25,               /* unary */
  SB_EW_SIGMOID_BWD = 26,       /* in0(grad) * y * (1 - y), in1 = y = sigmoid output */
  SB_EW_TANH_BWD = 27,          /* in0(grad) * (1 - y * y), in1 = y = tanh output */
  SB_EW_MAXIMUM = 28,           /* NaN propagates */
  SB_EW_MINIMUM = 29,
  SB_EW_EQ = 30,                /* comparisons: 1 or 0 in the compute type, stored as the output dtype (bool) */
  SB_EW_NE = 31,
  SB_EW_LT = 32,
  SB_EW_LE = 33,
  SB_EW_GT = 34,
  SB_EW_GE = 35,
  SB_EW_WHERE = 36,             /* in0(condition) ? in1 : in2 */
  SB_EW_MASKED_FILL = 37,       /* in1(mask) ? scalar : in0 */
  /* div with a rounding mode (torch_supa/csrc/aten/ops/kernels/elementwise/BinaryDivTruncKernel.cu,
   * BinaryDivFloorKernel.cu).  Floating types: trunc(a / b), and the floor division of Python (quotient from the
   * exact remainder, corrected by one where the signs differ).  Integer types: C division, and the same rounded
   * towards minus infinity; an integer division by zero yields 0 instead of raising as the CPU does. */
  SB_EW_DIV_TRUNC = 38,
  SB_EW_DIV_FLOOR = 39,
  SB_EW_OP_COUNT = 40
} sb_ew_op;

typedef struct sb_ew_desc {
  int32_t op;            /* sb_ew_op */
  int32_t ndim;          /* 1..SB_MAX_DIMS (a 0-dim tensor is ndim 1, size 1) */
  int32_t noperands;     /* outputs + inputs, 1..SB_MAX_OPERANDS; operand 0 is the output */
  int32_t common_dtype;  /* dtype the arithmetic is defined on (result of type promotion) */
  int64_t sizes[SB_MAX_DIMS];
  int64_t strides[SB_MAX_OPERANDS][SB_MAX_DIMS]; /* elements; 0 = broadcast */
  void* data[SB_MAX_OPERANDS];
  int32_t dtype[SB_MAX_OPERANDS];
  double alpha;          /* add/sub scale when the compute type is floating */
  int64_t ialpha;        /* add/sub scale when the compute type is integral */
  double scalar;         /* FILL / *_SCALAR operand (floating compute types) */
  int64_t iscalar;       /* FILL / *_SCALAR operand (integral and bool compute types) */
} sb_ew_desc;

SB_API int sb_elementwise(const sb_ew_desc* desc, sb_stream_t stream);
/* Which launch path the engine picks for this descriptor: 0 contiguous-vectorised, 1 row-vectorised
 * (unit inner stride, broadcast/strided outer dims), 2 tiled 2-D transpose, 3 generic strided. */
SB_API int sb_elementwise_path(const sb_ew_desc* desc);

/* ------------------------------------------------------------------------------------------
 * Reductions.
 *
 * Replaces gpu_reduce_kernel / ReduceOp / setReduceConfig
 * (torch_supa/csrc/aten/ops/kernels/reduce/Reduce.cuh:220-224,400-476,1040-1333) for sum_kernel_cuda
 * (ReduceSumKernel.cu:80-113), mean_kernel_cuda (ReduceMomentKernel.cu:16-55) and the amax stub of the
 * external native-op library.  Dimensions in any order (the planner orders them by input stride itself: a TensorIterator lists
 * the reduced dimensions first); a reduced dimension has out_stride 0.
 * Accumulation is fp32 for fp16/bf16/fp32 inputs, fp64 for fp64, int64 for integers; amax is exact and
 * propagates NaN.
 * ------------------------------------------------------------------------------------------ */
typedef enum sb_reduce_op {
  SB_RED_SUM = 0,
  SB_RED_MEAN = 1,
  SB_RED_AMAX = 2,
  SB_RED_AMIN = 3,
  SB_RED_PROD = 4,   /* prod_kernel_cuda of the reference's reduce family (kernels/reduce/ReduceOps) */
  SB_RED_NANSUM = 5, /* sum with NaN counted as zero */
  SB_RED_OP_COUNT = 6
} sb_reduce_op;

typedef struct sb_reduce_desc {
  int32_t op;        /* sb_reduce_op */
  int32_t ndim;      /* 1..SB_MAX_DIMS */
  int32_t in_dtype;
  int32_t out_dtype;
  int64_t sizes[SB_MAX_DIMS];
  int64_t in_strides[SB_MAX_DIMS];  /* elements */
  int64_t out_strides[SB_MAX_DIMS]; /* elements; 0 on reduced dimensions */
  const void* in;
  void* out;
  void* scratch;        /* device scratch of at least sb_reduce_scratch_bytes(desc) bytes, or NULL if that is 0 */
  size_t scratch_bytes;
} sb_reduce_desc;

/* Scratch the launch needs (when one output is split over several CTAs: few long rows, or column sums whose rows are
 * cut into chunks); 0 for most shapes. */
SB_API size_t sb_reduce_scratch_bytes(const sb_reduce_desc* desc);
SB_API int sb_reduce(const sb_reduce_desc* desc, sb_stream_t stream);
/* 0 = inner-contiguous rows, 1 = rows split over several CTAs (two stage), 2 = outer (column) reduce,
 * 3 = generic. */
SB_API int sb_reduce_path(const sb_reduce_desc* desc);

/* ------------------------------------------------------------------------------------------
 * Reductions with an index or a second moment, over the middle dimension of a contiguous [outer, L, inner] view.
 *
 * sb_arg_reduce: extremum and / or its position along L (argmax, argmin, max.dim, min.dim; the reference routes them
 * through the same reduce family, kernels/reduce/Reduce.cuh:1040-1333, with the index rules of its CPU golden): of equal
 * extrema the lowest index wins; a NaN beats every number, for max and for min, and of several NaN the first.
 * `values` (in `dtype`) and `indices` (int64) have outer * inner elements; either may be NULL.  Bit-exact.
 *
 * sb_moments: variance or standard deviation with the given correction (M2 / max(0, L - correction)), and optionally
 * the mean, in `dtype` (torch_supa/csrc/aten/ops/StdVar.cpp:34-63).  The running sums are fp64; over rows of fp32 / bf16 /
 * fp16 values the sums of up to eight neighbouring terms are formed in fp32 first.
 *
 * scratch: sb_reduce_ext_scratch_bytes(...) bytes, 8-byte aligned, needed when few long rows are cut into segments
 * or the rows of a column reduction (inner > 1) into chunks (the call returns 0 otherwise).
 * ------------------------------------------------------------------------------------------ */
SB_API size_t sb_reduce_ext_scratch_bytes(int32_t dtype, int64_t outer, int64_t L, int64_t inner, int32_t moments);
SB_API int sb_arg_reduce(const void* in, int32_t dtype, int64_t outer, int64_t L, int64_t inner, int32_t is_max, void* values,
                         int64_t* indices, void* scratch, size_t scratch_bytes, sb_stream_t stream);
SB_API int sb_moments(const void* in, int32_t dtype, int64_t outer, int64_t L, int64_t inner, double correction, int32_t take_sqrt,
                      void* out, void* mean_out, void* scratch, size_t scratch_bytes, sb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Cross entropy with class-probability ("soft") targets, forward and backward.
 *
 * Replaces cross_entropy_prob_kernel (torch_supa/csrc/aten/ops/kernels/elementwise/CrossEntropyLossKernel.cu:532-576,
 * selected at :721) and, for the gradient, the composite the reference differentiates through.  With
 * q_c = target_c (1 - eps) + eps / C and w = class_weight (1 when NULL):
 *   loss_i  = sum_c w_c q_ic (lse_i - x_ic)
 *   grad_ic = (softmax_ic * sum_k w_k q_ik - w_c q_ic) * grad_scale * row_grad_out_i
 * row_loss[i] = loss_i * loss_scale.  `mean` divides by the number of rows, which the caller folds into loss_scale and
 * grad_scale (no count is needed); sum the row losses with sb_ce_loss_sum_finish(reduction = sum).
 * ------------------------------------------------------------------------------------------ */
typedef struct sb_ce_prob_args {
  const void* logits;        /* [rows, classes] row-major */
  const void* target;        /* [rows, classes] probabilities, same dtype */
  int32_t dtype;             /* SB_F32, SB_BF16 or SB_F16 */
  void* grad_logits;         /* [rows, classes] same dtype, or NULL for forward only; must not alias logits or target */
  float* row_loss;           /* [rows] */
  const float* row_grad_out; /* [rows] upstream gradient per row, or NULL for 1 */
  const float* class_weight; /* [classes] fp32, or NULL */
  int64_t rows;
  int64_t classes;
  float label_smoothing;
  float grad_scale;
  float loss_scale;
} sb_ce_prob_args;
SB_API int sb_ce_prob_forward_backward(const sb_ce_prob_args* args, sb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Random fills and dropout from a (seed, offset) pair.
 *
 * The pair is what the device generator hands out (philox_engine_inputs,
 * torch_supa/csrc/aten/SUPAGeneratorImpl.cpp:450-455; the reference feeds it to its vendor library's Philox4_32_10).  The
 * stream is a function of the element index alone: group g = elements [g*E, (g+1)*E) with E = 4 for element types of up
 * to 4 bytes and 2 for 8-byte types; words = philox4x32_10(counter {lo(offset/4), hi(offset/4), lo(g), hi(g)},
 * key {lo(seed), hi(seed)}); element k uses word k (E = 4) or words 2k, 2k+1 (E = 2).  A fill consumes one 128-bit block
 * per group: advance the offset by 4 per call.  offset must be a multiple of 4.
 *   SB_RNG_UNIFORM    a + u (b - a), u = (word >> 8) 2^-24 (53 bits for doubles); a value that rounds to b becomes a
 *   SB_RNG_NORMAL     a + b z; Box-Muller on (word 2j, word 2j+1): u1 = ((w >> 8) + 1) 2^-24, u2 = (w >> 8) 2^-24,
 *                     z = sqrt(-2 ln u1) (cos, sin)(2 pi u2)
 *   SB_RNG_INTEGER    low + r mod range (range = 0 means 2^64, 8-byte types only; r is one word when range <= 2^32)
 *   SB_RNG_BERNOULLI  1 where u < a
 * sb_dropout: keep_i = (u_i >= p), out = x * keep / (1 - p), mask = keep (one byte per element).
 * ------------------------------------------------------------------------------------------ */
typedef enum sb_rng_kind { SB_RNG_UNIFORM = 0, SB_RNG_NORMAL = 1, SB_RNG_INTEGER = 2, SB_RNG_BERNOULLI = 3 } sb_rng_kind;
typedef struct sb_rng_args {
  void* dst;       /* contiguous, numel elements of dtype */
  int32_t dtype;   /* uniform / normal: SB_F32, SB_F64, SB_BF16, SB_F16; integer / bernoulli: any */
  int32_t kind;    /* sb_rng_kind */
  int64_t numel;
  double a, b;
  int64_t low;
  uint64_t range;
  uint64_t seed;
  uint64_t offset;
} sb_rng_args;
SB_API int sb_rng_fill(const sb_rng_args* args, sb_stream_t stream);
SB_API int sb_dropout(const void* x, void* out, void* mask, int32_t dtype, int64_t numel, double p, uint64_t seed,
                      uint64_t offset, sb_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* SUPA_B200_KERNELS_H_ */
