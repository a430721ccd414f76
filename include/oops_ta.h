/*
 * oops_ta.h -- C ABI of the B200 (sm_100a) triangle-attention library.
 *
 * The library replaces the backend of OOps' `oops.attention.triangle_attention`
 * operator.  In the reference that backend is a set of Triton kernels reached
 * through Python; it has no C interface of its own, so every entry point below
 * names the Python function whose work it takes over (paths are relative to the
 * reference checkout).
 *
 * Conventions
 *   - Plain C: raw device pointers, 64-bit element strides, no framework types.
 *   - The library never allocates, frees or retains device memory.  The caller
 *     owns every buffer, including the scratch workspace, whose size it asks
 *     for with oops_ta_*_workspace_bytes().
 *   - All work is enqueued on the CUDA stream passed in (a cudaStream_t cast to
 *     void*); no call synchronises the device.  The current device must be the
 *     one that owns the buffers.
 *   - Every function returns an oops_ta_status; 0 is success.  Unsupported
 *     requests are reported, never served by a fallback.
 *
 * Tensor model
 *   A "pair tensor" (query, key, value, output and their gradients) is addressed
 *   as  ptr[b*sb + r*sr + c*sc + h*sh + d]  for b<batch, r<rows, c<cols,
 *   h<heads, d<head_dim: the head_dim axis is contiguous, every other axis has a
 *   free element stride.  The starting-node form has sr > sc; the ending-node
 *   form of the reference (pair axes swapped in memory,
 *   oops/attention/triangle/triangle_attention.py:249-258) is the same call
 *   with sr < sc.  Ragged (NestedTensor) batches are one call per sample with
 *   the sample's base pointer and strides (the eight columns of the reference's
 *   sample table, oops/attention/triangle/nested.py:275-288, become these
 *   fields).
 */
#ifndef OOPS_TA_H_
#define OOPS_TA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OOPS_TA_ABI_VERSION 1

typedef enum oops_ta_dtype {
  OOPS_TA_F32 = 0,
  OOPS_TA_F16 = 1,
  OOPS_TA_BF16 = 2
} oops_ta_dtype;

typedef enum oops_ta_status {
  OOPS_TA_OK = 0,
  OOPS_TA_INVALID_ARGUMENT = 1,   /* null pointer, bad size, wrong ABI version      */
  OOPS_TA_UNSUPPORTED_DTYPE = 2,  /* dtype outside {f32, f16, bf16}                  */
  OOPS_TA_UNSUPPORTED_HEAD_DIM = 3, /* head_dim outside [1, 256]                     */
  OOPS_TA_UNSUPPORTED_LAYOUT = 4, /* a stride or alignment the kernels cannot take   */
  OOPS_TA_LIMIT_EXCEEDED = 5,     /* grid or index range beyond 2^31-1               */
  OOPS_TA_WORKSPACE_TOO_SMALL = 6,
  OOPS_TA_CUDA_ERROR = 7,         /* a CUDA runtime/driver call failed               */
  OOPS_TA_DEVICE_TIMEOUT = 8,     /* a bounded device-side wait gave up              */
  OOPS_TA_WRONG_DEVICE = 9        /* the device is not compute capability 10.x       */
} oops_ta_status;

/* flags of oops_ta_problem.flags */
#define OOPS_TA_FLAG_FORCE_GENERIC 1u /* take the layout-agnostic FFMA kernels even
                                         where the tcgen05 kernels apply (testing) */
#define OOPS_TA_FLAG_SPLIT_REVERSE 4u /* reverse pass: take the separate dQ and dK/dV
                                         kernels even where the single-pass kernel that
                                         produces all three applies (testing)           */

#define OOPS_TA_FLAG_DBIAS_F32 8u     /* reverse pass: the gradient buffer of a row-shared bias (bias_groups == 1)
                                         holds f32 values whatever the bias type.  For callers that add the
                                         gradients of several calls -- the row shards of one problem on several
                                         GPUs -- and round once.  No counterpart in the reference, which has no
                                         multi-GPU path.                                                         */
#define OOPS_TA_FLAG_REUSE_DELTA 16u  /* reverse pass: the workspace already holds delta = rowsum(O * dO) from an
                                         earlier oops_ta_backward call on the same problem, output, upstream
                                         gradient and workspace; it is not recomputed.  Lets a caller split one
                                         reverse pass into two calls (bias gradient first, so that its exchange
                                         overlaps the other gradients) without paying for delta twice.  Honoured by
                                         the tcgen05 kernels; the layout-agnostic kernels recompute.            */

typedef struct oops_ta_pair {
  void* ptr;
  int64_t sb, sr, sc, sh; /* element strides of batch, row, column, head */
} oops_ta_pair;

/*
 * One uniform problem: `batch` independent pair tensors of rows x cols cells.
 * Replaces the argument bundle the reference hands to its Triton launchers
 * (oops/attention/triangle/triton/generic.py:173-317 forward, :320-534 reverse).
 */
typedef struct oops_ta_problem {
  uint32_t abi_version; /* OOPS_TA_ABI_VERSION */
  uint32_t flags;
  int32_t dtype;       /* oops_ta_dtype of q, k, v, out and their gradients         */
  int32_t bias_dtype;  /* oops_ta_dtype of bias and its gradient (dtype or F32)     */
  int32_t batch, rows, cols, heads, head_dim;
  int32_t bias_groups; /* 0: no bias; 1: one bias shared by all rows; rows: per row  */
  float scale;         /* multiplies q.k before the bias is added                   */
  int32_t reserved;

  oops_ta_pair q, k, v;

  /* keep-mask over keys: nonzero byte keeps key column c of row r.  NULL keeps all.
     Strides may be 0 (broadcast).  Replaces the int16 mask of
     oops/attention/triangle/triangle_attention.py:135. */
  const uint8_t* mask;
  int64_t mask_sb, mask_sr, mask_sc;

  /* bias[b*sb + g*sg + h*sh + q*sq + k*sk], g = 0 when bias_groups == 1 else r. */
  const void* bias;
  int64_t bias_sb, bias_sg, bias_sh, bias_sq, bias_sk;

  void* workspace;
  uint64_t workspace_bytes;
} oops_ta_problem;

/* Gradient request of the reverse pass; a NULL ptr skips that gradient
   (the reference's need_grad_{query,key,value,bias}, generic.py:320-343). */
typedef struct oops_ta_grads {
  oops_ta_pair dq, dk, dv;
  void* dbias; /* same dtype as bias; row-shared biases receive the sum over rows */
  int64_t dbias_sb, dbias_sg, dbias_sh, dbias_sq, dbias_sk;
} oops_ta_grads;

/* ABI version the library was built with. */
int oops_ta_abi_version(void);

/* Static text for a status code. */
const char* oops_ta_status_string(int status);

/* Detail of the last failure on the calling thread (empty string if none). */
const char* oops_ta_last_error(void);

/*
 * Admission test: OOPS_TA_OK if oops_ta_forward/backward can serve the problem,
 * otherwise the status they would return.  Pointers are not dereferenced.
 * Replaces supports_triangle_attention (generic.py:64-154).
 */
int oops_ta_supported(const oops_ta_problem* problem);

/* 1 if the problem takes the tcgen05/TMEM/TMA kernels, 0 if it takes the
   layout-agnostic kernels, negative status on error.  `backward` selects which
   pass is asked about. */
int oops_ta_uses_tensor_path(const oops_ta_problem* problem, int backward);

/* Scratch bytes oops_ta_forward needs for this problem (may be 0). */
uint64_t oops_ta_forward_workspace_bytes(const oops_ta_problem* problem);

/* Scratch bytes oops_ta_backward needs for this problem and gradient request. */
uint64_t oops_ta_backward_workspace_bytes(const oops_ta_problem* problem, const oops_ta_grads* grads);

/*
 * Forward pass.  Writes out (same dtype as q) and, when lse is not NULL, the
 * natural-log row normaliser lse[((b*rows + r)*heads + h)*cols + q] (0 for rows
 * with no kept key, whose output is 0 too).
 * Replaces _run_forward / _run_inference and the Triton kernels `_forward` /
 * `_inference` (generic.py:173-317; triton/kernel.py:150-371).
 */
int oops_ta_forward(const oops_ta_problem* problem, const oops_ta_pair* out, float* lse, void* stream);

/*
 * Reverse pass for the gradients requested in `grads`, from the forward output,
 * its lse and the upstream gradient `dout` (dtype of q).
 * Replaces _run_backward and the Triton kernels `_backward_preprocess`,
 * `_backward_query`, `_backward_key_value`, `_backward_shared_bias`
 * (generic.py:320-534; triton/kernel.py:374-873).
 */
int oops_ta_backward(const oops_ta_problem* problem, const oops_ta_pair* out, const oops_ta_pair* dout,
                     const float* lse, const oops_ta_grads* grads, void* stream);

/*
 * Forward pass with the sigmoid gate of the following output projection applied in the epilogue:
 * gated = sigmoid(gate) * attention, where `gate` holds the gate logits as a pair tensor of the problem's shape and
 * dtype.  `plain` (may be NULL or have a NULL ptr) additionally receives the ungated attention values, which the
 * reverse pass needs (oops_ta_gate_backward, then oops_ta_backward with `plain` as the forward output).  Workspace
 * and lse as for oops_ta_forward.  The tcgen05 kernels apply the gate to the output tile in registers; the
 * layout-agnostic kernels run the forward pass and then the element-wise gate.
 * Fuses the element-wise core of the reference's gate_attention_output (oops/attention/gate/composed.py:47-53,
 * `sigmoid(linear(single, gate_weight)) * attention`) into the operator that produces its input
 * (oops/attention/gate/gate_attention_output.py:36-100 consumes triangle attention's output in a pair block).
 */
int oops_ta_forward_gated(const oops_ta_problem* problem, const oops_ta_pair* gate, const oops_ta_pair* gated,
                          const oops_ta_pair* plain, float* lse, void* stream);

/*
 * The gate on its own: out = sigmoid(gate) * attention for pair tensors (batch, rows, cols, heads, head_dim) with free
 * strides, and its reverse pass: dattention = dout * sigmoid(gate), dgate = dout * attention * s * (1 - s); a NULL
 * gradient (or NULL ptr) is skipped.  With strides, the reference's head-major (*, H, Q, D) attention layout and its
 * token-major (*, Q, H*D) gate layout are the same call (rows = 1, cols = Q).
 * Replaces the element-wise part of the reference's `project_gate` Triton kernel and of its composed fallback
 * (oops/attention/gate/composed.py:36-53); the two linear maps around it stay library GEMMs.
 */
int oops_ta_gate_forward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair* attention,
                         const oops_ta_pair* gate, const oops_ta_pair* out, void* stream);
int oops_ta_gate_backward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair* attention,
                          const oops_ta_pair* gate, const oops_ta_pair* dout, const oops_ta_pair* dattention,
                          const oops_ta_pair* dgate, void* stream);

/*
 * Layer normalisation over the last axis of (rows, width) activations, 1 <= width <= 8192: the step before the
 * projections that produce q, k, v and the pair bias.  Replaces the backend of the reference's layer_norm
 * (oops/normalization/layer_norm/layer_norm.py:37-110, `triton_layer_norm`).
 *   forward:  y = (x - mean) * rstd * weight + bias; `mean` and `rstd` (f32 per row; either may be NULL) are what the
 *             reverse pass needs.  `weight` / `bias` may be NULL.
 *   backward: dx, dweight, dbias (each may be NULL) from dy, x, weight, mean, rstd.  The parameter gradients are sums
 *             over rows: per-CTA f32 partial rows in `workspace` (oops_ta_layer_norm_backward_workspace_bytes) added in
 *             a fixed order, so the result is bitwise reproducible.
 * `dtype` is the activation type (OOPS_TA_F32 / F16 / BF16); `affine_dtype` the type of weight, bias and their
 * gradients: the same, or OOPS_TA_F32 with 16-bit activations.  Rows are contiguous; row strides are in elements.
 */
uint64_t oops_ta_layer_norm_backward_workspace_bytes(int64_t rows, int32_t width);
int oops_ta_layer_norm_forward(int dtype, int affine_dtype, int64_t rows, int32_t width, const void* x, int64_t x_stride,
                               const void* weight, const void* bias, float eps, void* y, int64_t y_stride, float* mean,
                               float* rstd, void* stream);
int oops_ta_layer_norm_backward(int dtype, int affine_dtype, int64_t rows, int32_t width, const void* dy, int64_t dy_stride,
                                const void* x, int64_t x_stride, const void* weight, const float* mean, const float* rstd,
                                void* dx, int64_t dx_stride, void* dweight, void* dbias, void* workspace,
                                uint64_t workspace_bytes, void* stream);

/*
 * Pair validity of a packed ragged batch: for sample s with n_s tokens, out holds the samples' row-major n_s x n_s
 * squares one after the other, cell (i, j) = token i is valid and token j is valid (bytes 0 / 1).  `token_values` are
 * bytes (nonzero = valid), `token_offsets` the samples + 1 cumulative token counts (int64, device memory), `chunks`
 * the sum over samples of n_s * ceil(n_s / 16) (the launch extent, computed by the caller from the lengths it already
 * has on the host).  Replaces the packed arm of the reference's pair_mask_from_token_mask
 * (oops/mask/pair_mask_from_token_mask.py:100-103, `packed_pair_mask`); the dense arm is a broadcast AND (:68-70).
 */
int oops_ta_pair_mask_packed(const uint8_t* token_values, const int64_t* token_offsets, int32_t samples, int64_t chunks,
                             uint8_t* out, void* stream);

/*
 * Forward pass that needs no workspace from the caller and allocates nothing.
 *
 * It has no counterpart in the reference.  It is for hosts that cannot hand over scratch memory when
 * they call: a serving process whose device memory pool was sized and frozen at start-up, a latency-
 * critical loop that must not run into cudaMalloc's device-wide synchronisation, or code that is in the
 * middle of recording work and may not touch the allocator.  Same arguments, outputs and numerics as
 * oops_ta_forward with OOPS_TA_FLAG_FORCE_GENERIC (the layout-agnostic kernels, any dtype, head size
 * and strides); `problem->workspace` is ignored.  The logits of a block of pair rows are kept in a
 * fixed array inside the library (oops_ta_forward_static_capacity() bytes, 32 MiB, resident on every
 * GPU that loads the library until the process exits).
 *
 * Limits and rules:
 *   - one pair row must fit: batch * heads * cols * cols * 4 bytes <= the capacity, otherwise
 *     OOPS_TA_LIMIT_EXCEEDED is returned and nothing is launched;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call before any stream capture begins;
 *   - all calls on a device share the one array: calls whose kernels may overlap on the GPU (different
 *     streams without ordering) race on it -- order them.  Nothing needs clearing between calls;
 *   - no cudaMalloc/cudaFree or allocating library routine is called.
 */
int oops_ta_forward_static(const oops_ta_problem* problem, const oops_ta_pair* out, float* lse, void* stream);

/* Size in bytes of the built-in scratch array used by oops_ta_forward_static. */
uint64_t oops_ta_forward_static_capacity(void);

/*
 * Device-side status of the current device: OOPS_TA_OK, or OOPS_TA_DEVICE_TIMEOUT if a kernel
 * gave up a bounded wait since the last reset (its outputs are then undefined).  Unlike every
 * other call this one synchronises with the device.  `reset` != 0 clears the word.
 * No counterpart in the reference (Triton kernels have no device-side waits).
 */
int oops_ta_device_status(int reset);

/*
 * Self-test of the bounded device-side wait.  Enqueues a one-CTA kernel whose only wait is on a barrier
 * that nothing completes, with a limit of one millisecond: the wait gives up, the CTA tears down the way a
 * compute kernel does after a wait that ran out, and the kernel returns by itself.  Afterwards
 * oops_ta_device_status reports OOPS_TA_DEVICE_TIMEOUT until it is reset, and the tensor kernels of the
 * forward pass return at once.  Meant for tests and for checking a deployment's status polling.
 * No counterpart in the reference.
 */
int oops_ta_selftest_wait_limit(void* stream);

/* Number of kernels the library has launched in this process (all streams). */
uint64_t oops_ta_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* OOPS_TA_H_ */
