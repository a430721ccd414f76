// Sigmoid gate on attention values: gated = sigmoid(gate) * attention, the element-wise core of the reference's
// gate_attention_output (oops/attention/gate/composed.py:47-53, between its two linear maps), and its reverse pass.
// Layout-agnostic: every tensor is a pair tensor (batch, rows, cols, heads, head_dim) with free element strides and a
// contiguous head_dim axis, so the reference's head-major attention layout (*prefix, H, Q, D) and its token-major
// gate layout (*prefix, Q, H*D) are both described by strides (rows = 1, cols = Q).  HBM-bound element-wise work:
// one thread per 8 channels, 16-byte accesses where the addresses allow.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ta_internal.h"

namespace oops_ta {
namespace {

template <typename T>
__device__ __forceinline__ float to_float(T v) { return float(v); }

__device__ __forceinline__ float sigmoid_of(float g) { return 1.f / (1.f + __expf(-g)); }

struct GateShape {
  int batch, rows, cols, heads, head_dim, chunks;  // chunks of 8 channels per (b, r, c, h)
};

__device__ __forceinline__ bool locate(const GateShape& s, int64_t i, int& b, int& r, int& c, int& h, int& d0) {
  const int64_t total = int64_t(s.batch) * s.rows * s.cols * s.heads * s.chunks;
  if (i >= total) return false;
  d0 = int(i % s.chunks) * 8;
  i /= s.chunks;
  h = int(i % s.heads);
  i /= s.heads;
  c = int(i % s.cols);
  i /= s.cols;
  r = int(i % s.rows);
  b = int(i / s.rows);
  return true;
}

template <typename T>
__device__ __forceinline__ T* at(const oops_ta_pair& t, int b, int r, int c, int h, int d) {
  return reinterpret_cast<T*>(t.ptr) + b * t.sb + int64_t(r) * t.sr + int64_t(c) * t.sc + int64_t(h) * t.sh + d;
}

template <typename T>
__global__ void gate_forward_kernel(GateShape s, oops_ta_pair attention, oops_ta_pair gate, oops_ta_pair out) {
  int b, r, c, h, d0;
  if (!locate(s, int64_t(blockIdx.x) * blockDim.x + threadIdx.x, b, r, c, h, d0)) return;
  const T* a = at<T>(attention, b, r, c, h, d0);
  const T* g = at<T>(gate, b, r, c, h, d0);
  T* o = at<T>(out, b, r, c, h, d0);
  const int n = min(8, s.head_dim - d0);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < n) o[i] = T(sigmoid_of(to_float(g[i])) * to_float(a[i]));
}

template <typename T>
__global__ void gate_backward_kernel(GateShape s, oops_ta_pair attention, oops_ta_pair gate, oops_ta_pair dout,
                                     oops_ta_pair dattention, oops_ta_pair dgate) {
  int b, r, c, h, d0;
  if (!locate(s, int64_t(blockIdx.x) * blockDim.x + threadIdx.x, b, r, c, h, d0)) return;
  const T* a = at<T>(attention, b, r, c, h, d0);
  const T* g = at<T>(gate, b, r, c, h, d0);
  const T* u = at<T>(dout, b, r, c, h, d0);
  T* da = dattention.ptr ? at<T>(dattention, b, r, c, h, d0) : nullptr;
  T* dg = dgate.ptr ? at<T>(dgate, b, r, c, h, d0) : nullptr;
  const int n = min(8, s.head_dim - d0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (i >= n) continue;
    const float sg = sigmoid_of(to_float(g[i])), up = to_float(u[i]);
    if (da) da[i] = T(up * sg);
    if (dg) dg[i] = T(up * to_float(a[i]) * sg * (1.f - sg));
  }
}

int check_shape(int dtype, int batch, int rows, int cols, int heads, int head_dim) {
  if (dtype != OOPS_TA_F32 && dtype != OOPS_TA_F16 && dtype != OOPS_TA_BF16)
    return fail(OOPS_TA_UNSUPPORTED_DTYPE, "gate dtype %d is not f32/f16/bf16", dtype);
  if (batch <= 0 || rows <= 0 || cols <= 0 || heads <= 0 || head_dim <= 0)
    return fail(OOPS_TA_INVALID_ARGUMENT, "empty dimension (batch=%d rows=%d cols=%d heads=%d head_dim=%d)", batch, rows, cols,
                heads, head_dim);
  return OOPS_TA_OK;
}

}  // namespace

int gate_forward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair& attention,
                 const oops_ta_pair& gate, const oops_ta_pair& out, cudaStream_t stream) {
  int status = check_shape(dtype, batch, rows, cols, heads, head_dim);
  if (status) return status;
  const GateShape s{batch, rows, cols, heads, head_dim, (head_dim + 7) / 8};
  const int64_t total = int64_t(batch) * rows * cols * heads * s.chunks;
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == OOPS_TA_F32)
    gate_forward_kernel<float><<<grid, 256, 0, stream>>>(s, attention, gate, out);
  else if (dtype == OOPS_TA_F16)
    gate_forward_kernel<__half><<<grid, 256, 0, stream>>>(s, attention, gate, out);
  else
    gate_forward_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(s, attention, gate, out);
  count_launch();
  return check_launch("gate forward");
}

int gate_backward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair& attention,
                  const oops_ta_pair& gate, const oops_ta_pair& dout, const oops_ta_pair& dattention,
                  const oops_ta_pair& dgate, cudaStream_t stream) {
  int status = check_shape(dtype, batch, rows, cols, heads, head_dim);
  if (status) return status;
  const GateShape s{batch, rows, cols, heads, head_dim, (head_dim + 7) / 8};
  const int64_t total = int64_t(batch) * rows * cols * heads * s.chunks;
  const unsigned grid = (unsigned)ceil_div(total, 256);
  if (dtype == OOPS_TA_F32)
    gate_backward_kernel<float><<<grid, 256, 0, stream>>>(s, attention, gate, dout, dattention, dgate);
  else if (dtype == OOPS_TA_F16)
    gate_backward_kernel<__half><<<grid, 256, 0, stream>>>(s, attention, gate, dout, dattention, dgate);
  else
    gate_backward_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(s, attention, gate, dout, dattention, dgate);
  count_launch();
  return check_launch("gate backward");
}

}  // namespace oops_ta
