// C ABI of liboops_ta_sm100.so: argument checks, kernel selection, error text.
// Declarations and the reference functions each entry point replaces are in
// include/oops_ta.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "ta_internal.h"

namespace oops_ta {
namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};
}  // namespace

int fail(int status, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_error, sizeof(g_error), format, args);
  va_end(args);
  return status;
}

void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int check_launch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return fail(OOPS_TA_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(err));
  return OOPS_TA_OK;
}

size_t dtype_size(int dtype) { return dtype == OOPS_TA_F32 ? 4 : 2; }

namespace {

bool valid_dtype(int d) { return d == OOPS_TA_F32 || d == OOPS_TA_F16 || d == OOPS_TA_BF16; }

int validate(const oops_ta_problem* p, bool need_pointers) {
  if (!p) return fail(OOPS_TA_INVALID_ARGUMENT, "problem is NULL");
  if (p->abi_version != OOPS_TA_ABI_VERSION)
    return fail(OOPS_TA_INVALID_ARGUMENT, "ABI version %u, library has %d", p->abi_version, OOPS_TA_ABI_VERSION);
  if (!valid_dtype(p->dtype)) return fail(OOPS_TA_UNSUPPORTED_DTYPE, "q/k/v dtype %d is not f32/f16/bf16", p->dtype);
  if (p->batch <= 0 || p->rows <= 0 || p->cols <= 0 || p->heads <= 0)
    return fail(OOPS_TA_INVALID_ARGUMENT, "empty dimension (batch=%d rows=%d cols=%d heads=%d)", p->batch, p->rows,
                p->cols, p->heads);
  if (p->head_dim < 1 || p->head_dim > 256)
    return fail(OOPS_TA_UNSUPPORTED_HEAD_DIM, "head_dim %d outside [1, 256]", p->head_dim);
  if (p->bias_groups != 0) {
    if (p->bias_groups != 1 && p->bias_groups != p->rows)
      return fail(OOPS_TA_INVALID_ARGUMENT, "bias_groups %d must be 0, 1 or rows=%d", p->bias_groups, p->rows);
    if (!valid_dtype(p->bias_dtype) || (p->bias_dtype != p->dtype && p->bias_dtype != OOPS_TA_F32))
      return fail(OOPS_TA_UNSUPPORTED_DTYPE, "bias dtype %d must equal the q/k/v dtype or be f32", p->bias_dtype);
    if (need_pointers && !p->bias) return fail(OOPS_TA_INVALID_ARGUMENT, "bias_groups set but bias is NULL");
  }
  if (need_pointers && (!p->q.ptr || !p->k.ptr || !p->v.ptr))
    return fail(OOPS_TA_INVALID_ARGUMENT, "q, k or v is NULL");
  const int64_t problems = int64_t(p->batch) * p->rows * p->heads;
  if (problems > 0x7fffffffll || int64_t(p->cols) * p->cols > 0x7fffffffll)
    return fail(OOPS_TA_LIMIT_EXCEEDED, "batch*rows*heads=%lld or cols^2 exceeds 2^31-1", (long long)problems);
  return OOPS_TA_OK;
}

bool force_generic(const oops_ta_problem* p) { return (p->flags & OOPS_TA_FLAG_FORCE_GENERIC) != 0; }

int check_device() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return fail(OOPS_TA_CUDA_ERROR, "cudaGetDevice failed");
  static thread_local int cached_device = -1, cached_major = 0;
  if (cached_device != device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
      return fail(OOPS_TA_CUDA_ERROR, "cudaDeviceGetAttribute failed");
    cached_device = device;
    cached_major = major;
  }
  if (cached_major != 10)
    return fail(OOPS_TA_WRONG_DEVICE, "device %d has compute capability %d.x; this library is sm_100a only", device,
                cached_major);
  return OOPS_TA_OK;
}

}  // namespace
}  // namespace oops_ta

using namespace oops_ta;

extern "C" {

int oops_ta_abi_version(void) { return OOPS_TA_ABI_VERSION; }

const char* oops_ta_status_string(int status) {
  switch (status) {
    case OOPS_TA_OK: return "ok";
    case OOPS_TA_INVALID_ARGUMENT: return "invalid argument";
    case OOPS_TA_UNSUPPORTED_DTYPE: return "unsupported dtype";
    case OOPS_TA_UNSUPPORTED_HEAD_DIM: return "unsupported head size";
    case OOPS_TA_UNSUPPORTED_LAYOUT: return "unsupported layout";
    case OOPS_TA_LIMIT_EXCEEDED: return "launch limit exceeded";
    case OOPS_TA_WORKSPACE_TOO_SMALL: return "workspace too small";
    case OOPS_TA_CUDA_ERROR: return "CUDA error";
    case OOPS_TA_DEVICE_TIMEOUT: return "device-side wait timed out";
    case OOPS_TA_WRONG_DEVICE: return "not an sm_100 device";
    default: return "unknown status";
  }
}

const char* oops_ta_last_error(void) { return g_error; }

int oops_ta_supported(const oops_ta_problem* problem) { return validate(problem, false); }

int oops_ta_uses_tensor_path(const oops_ta_problem* problem, int backward) {
  const int status = validate(problem, false);
  if (status) return -status;
  if (force_generic(problem)) return 0;
  return backward ? (tensor_backward_applies(*problem, nullptr) ? 1 : 0) : (tensor_forward_applies(*problem) ? 1 : 0);
}

uint64_t oops_ta_forward_workspace_bytes(const oops_ta_problem* problem) {
  if (validate(problem, false)) return 0;
  if (!force_generic(problem) && tensor_forward_applies(*problem)) return tensor_forward_workspace(*problem);
  return generic_forward_workspace(*problem);
}

uint64_t oops_ta_backward_workspace_bytes(const oops_ta_problem* problem, const oops_ta_grads* grads) {
  if (validate(problem, false) || !grads) return 0;
  if (!force_generic(problem) && tensor_backward_applies(*problem, grads))
    return tensor_backward_workspace(*problem, *grads);
  return generic_backward_workspace(*problem, *grads);
}

int oops_ta_forward(const oops_ta_problem* problem, const oops_ta_pair* out, float* lse, void* stream) {
  int status = validate(problem, true);
  if (status) return status;
  if (!out || !out->ptr) return fail(OOPS_TA_INVALID_ARGUMENT, "out is NULL");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!force_generic(problem) && tensor_forward_applies(*problem)) return tensor_forward(*problem, *out, lse, s);
  return generic_forward(*problem, *out, lse, s);
}

int oops_ta_forward_gated(const oops_ta_problem* problem, const oops_ta_pair* gate, const oops_ta_pair* gated,
                          const oops_ta_pair* plain, float* lse, void* stream) {
  int status = validate(problem, true);
  if (status) return status;
  if (!gate || !gate->ptr || !gated || !gated->ptr) return fail(OOPS_TA_INVALID_ARGUMENT, "gate or gated is NULL");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const oops_ta_pair none{nullptr, 0, 0, 0, 0};
  const oops_ta_pair& kept = plain && plain->ptr ? *plain : none;
  if (!force_generic(problem) && tensor_forward_applies(*problem))
    return tensor_forward_gated(*problem, *gate, *gated, kept, lse, s);
  // layout-agnostic kernels: the attention values first (into `plain`, or into `gated` itself when the caller
  // keeps no ungated copy), then the element-wise gate
  const oops_ta_pair& values = kept.ptr ? kept : *gated;
  status = generic_forward(*problem, values, lse, s);
  if (status) return status;
  return gate_forward(problem->dtype, problem->batch, problem->rows, problem->cols, problem->heads, problem->head_dim, values,
                      *gate, *gated, s);
}

int oops_ta_gate_forward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair* attention,
                         const oops_ta_pair* gate, const oops_ta_pair* out, void* stream) {
  if (!attention || !attention->ptr || !gate || !gate->ptr || !out || !out->ptr)
    return fail(OOPS_TA_INVALID_ARGUMENT, "attention, gate or out is NULL");
  const int status = check_device();
  if (status) return status;
  g_error[0] = 0;
  return gate_forward(dtype, batch, rows, cols, heads, head_dim, *attention, *gate, *out, reinterpret_cast<cudaStream_t>(stream));
}

int oops_ta_gate_backward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair* attention,
                          const oops_ta_pair* gate, const oops_ta_pair* dout, const oops_ta_pair* dattention,
                          const oops_ta_pair* dgate, void* stream) {
  if (!attention || !attention->ptr || !gate || !gate->ptr || !dout || !dout->ptr)
    return fail(OOPS_TA_INVALID_ARGUMENT, "attention, gate or dout is NULL");
  const int status = check_device();
  if (status) return status;
  g_error[0] = 0;
  const oops_ta_pair none{nullptr, 0, 0, 0, 0};
  return gate_backward(dtype, batch, rows, cols, heads, head_dim, *attention, *gate, *dout, dattention ? *dattention : none,
                       dgate ? *dgate : none, reinterpret_cast<cudaStream_t>(stream));
}

uint64_t oops_ta_layer_norm_backward_workspace_bytes(int64_t rows, int32_t width) {
  return layer_norm_backward_workspace_bytes(rows, width);
}

static int check_layer_norm(int64_t rows, int32_t width, int64_t a_stride, int64_t b_stride) {
  if (rows < 0) return fail(OOPS_TA_INVALID_ARGUMENT, "negative row count");
  if (width < 1 || width > layer_norm_max_width())
    return fail(OOPS_TA_UNSUPPORTED_LAYOUT, "layer_norm width %d outside [1, %d]", width, layer_norm_max_width());
  if (rows > 1 && (a_stride < width || b_stride < width))
    return fail(OOPS_TA_UNSUPPORTED_LAYOUT, "layer_norm rows overlap (row stride below the width)");
  return OOPS_TA_OK;
}

int oops_ta_layer_norm_forward(int dtype, int affine_dtype, int64_t rows, int32_t width, const void* x, int64_t x_stride,
                               const void* weight, const void* bias, float eps, void* y, int64_t y_stride, float* mean,
                               float* rstd, void* stream) {
  int status = check_layer_norm(rows, width, x_stride, y_stride);
  if (status) return status;
  if (rows > 0 && (!x || !y)) return fail(OOPS_TA_INVALID_ARGUMENT, "x or y is NULL");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  status = layer_norm_forward(dtype, affine_dtype, rows, width, x, x_stride, weight, bias, eps, y, y_stride, mean, rstd,
                              reinterpret_cast<cudaStream_t>(stream));
  return status == OOPS_TA_UNSUPPORTED_DTYPE ? fail(status, "layer_norm dtype %d / parameter dtype %d", dtype, affine_dtype) : status;
}

int oops_ta_layer_norm_backward(int dtype, int affine_dtype, int64_t rows, int32_t width, const void* dy, int64_t dy_stride,
                                const void* x, int64_t x_stride, const void* weight, const float* mean, const float* rstd,
                                void* dx, int64_t dx_stride, void* dweight, void* dbias, void* workspace,
                                uint64_t workspace_bytes, void* stream) {
  int status = check_layer_norm(rows, width, x_stride, dy_stride);
  if (status) return status;
  if (rows > 0 && (!x || !dy || !mean || !rstd)) return fail(OOPS_TA_INVALID_ARGUMENT, "dy, x, mean or rstd is NULL");
  if (rows > 0 && (dweight || dbias) &&
      (!workspace || workspace_bytes < layer_norm_backward_workspace_bytes(rows, width)))
    return fail(OOPS_TA_INVALID_ARGUMENT, "layer_norm workspace too small for the parameter gradients");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  status = layer_norm_backward(dtype, affine_dtype, rows, width, dy, dy_stride, x, x_stride, weight, mean, rstd, dx, dx_stride,
                               dweight, dbias, workspace, reinterpret_cast<cudaStream_t>(stream));
  return status == OOPS_TA_UNSUPPORTED_DTYPE ? fail(status, "layer_norm dtype %d / parameter dtype %d", dtype, affine_dtype) : status;
}

int oops_ta_pair_mask_packed(const uint8_t* token_values, const int64_t* token_offsets, int32_t samples, int64_t chunks,
                             uint8_t* out, void* stream) {
  if (samples < 0 || chunks < 0) return fail(OOPS_TA_INVALID_ARGUMENT, "negative sample or chunk count");
  if (chunks > 0 && (!token_values || !token_offsets || !out))
    return fail(OOPS_TA_INVALID_ARGUMENT, "token_values, token_offsets or out is NULL");
  if (samples > packed_pair_mask_max_samples())
    return fail(OOPS_TA_UNSUPPORTED_LAYOUT, "%d samples in one call (at most %d)", samples, packed_pair_mask_max_samples());
  const int status = check_device();
  if (status) return status;
  g_error[0] = 0;
  return packed_pair_mask(token_values, token_offsets, samples, chunks, out, reinterpret_cast<cudaStream_t>(stream));
}

int oops_ta_backward(const oops_ta_problem* problem, const oops_ta_pair* out, const oops_ta_pair* dout,
                     const float* lse, const oops_ta_grads* grads, void* stream) {
  int status = validate(problem, true);
  if (status) return status;
  if (!out || !out->ptr || !dout || !dout->ptr || !lse || !grads)
    return fail(OOPS_TA_INVALID_ARGUMENT, "out, dout, lse or grads is NULL");
  if (grads->dbias && problem->bias_groups == 0)
    return fail(OOPS_TA_INVALID_ARGUMENT, "dbias requested but the problem has no bias");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (!force_generic(problem) && tensor_backward_applies(*problem, grads))
    return tensor_backward(*problem, *out, *dout, lse, *grads, s);
  return generic_backward(*problem, *out, *dout, lse, *grads, s);
}

int oops_ta_forward_static(const oops_ta_problem* problem, const oops_ta_pair* out, float* lse, void* stream) {
  int status = validate(problem, true);
  if (status) return status;
  if (!out || !out->ptr) return fail(OOPS_TA_INVALID_ARGUMENT, "out is NULL");
  status = check_device();
  if (status) return status;
  g_error[0] = 0;
  return static_forward(*problem, *out, lse, reinterpret_cast<cudaStream_t>(stream));
}

uint64_t oops_ta_forward_static_capacity(void) { return static_forward_capacity(); }

int oops_ta_device_status(int reset) {
  const int forward = forward_device_status(reset);
  const int backward = backward_device_status(reset);
  return forward ? forward : backward;
}

int oops_ta_selftest_wait_limit(void* stream) {
  const int status = check_device();
  if (status) return status;
  g_error[0] = 0;
  return wait_limit_selftest(reinterpret_cast<cudaStream_t>(stream));
}

uint64_t oops_ta_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
