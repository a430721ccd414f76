// Internal declarations shared by the translation units of liboops_ta_sm100.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "oops_ta.h"

namespace oops_ta {

// Records a message for oops_ta_last_error() and returns `status`.
int fail(int status, const char* format, ...);

// Bumps the process-wide launch counter reported by oops_ta_launch_count().
void count_launch(int n = 1);

// Checks the last launch and converts a CUDA error into a status.
int check_launch(const char* what);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

size_t dtype_size(int dtype);

// Layout-agnostic FFMA kernels (any head_dim <= 256, any strides, f32/f16/bf16).
uint64_t generic_forward_workspace(const oops_ta_problem& p);
uint64_t generic_backward_workspace(const oops_ta_problem& p, const oops_ta_grads& g);
int generic_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream);
int generic_backward(const oops_ta_problem& p, const oops_ta_pair& out, const oops_ta_pair& dout, const float* lse,
                     const oops_ta_grads& g, cudaStream_t stream);

// The layout-agnostic forward pass on the library's built-in scratch array (no caller workspace).
uint64_t static_forward_capacity();
int static_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream);

// tcgen05/TMEM/TMA kernels (f16/bf16, head_dim 32, 16-byte aligned rows).
bool tensor_forward_applies(const oops_ta_problem& p);
bool tensor_backward_applies(const oops_ta_problem& p, const oops_ta_grads* g);
uint64_t tensor_forward_workspace(const oops_ta_problem& p);
uint64_t tensor_backward_workspace(const oops_ta_problem& p, const oops_ta_grads& g);
int tensor_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream);
int tensor_backward(const oops_ta_problem& p, const oops_ta_pair& out, const oops_ta_pair& dout, const float* lse,
                    const oops_ta_grads& g, cudaStream_t stream);

// Sigmoid gate on attention values and its reverse pass (any strides, f32/f16/bf16); a NULL gradient pointer skips it.
int gate_forward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair& attention,
                 const oops_ta_pair& gate, const oops_ta_pair& out, cudaStream_t stream);
int gate_backward(int dtype, int batch, int rows, int cols, int heads, int head_dim, const oops_ta_pair& attention,
                  const oops_ta_pair& gate, const oops_ta_pair& dout, const oops_ta_pair& dattention,
                  const oops_ta_pair& dgate, cudaStream_t stream);
// Pair validity of a packed ragged batch (token bytes, samples + 1 cumulative token counts on the device, number of
// 16-cell chunks over all rows); at most packed_pair_mask_max_samples() samples per call.
int packed_pair_mask(const uint8_t* tokens, const int64_t* token_offsets, int samples, int64_t chunks, uint8_t* out,
                     cudaStream_t stream);
int packed_pair_mask_max_samples();
// Layer normalisation over the last axis of (rows, width) activations (row strides in elements, contiguous rows);
// weight / bias / gradients of them may be NULL; affine_dtype is the activation dtype or f32.
uint64_t layer_norm_backward_workspace_bytes(int64_t rows, int width);
int layer_norm_max_width();
int layer_norm_forward(int dtype, int affine_dtype, int64_t rows, int width, const void* x, int64_t x_stride, const void* weight,
                       const void* bias, float eps, void* y, int64_t y_stride, float* mean, float* rstd, cudaStream_t stream);
int layer_norm_backward(int dtype, int affine_dtype, int64_t rows, int width, const void* dy, int64_t dy_stride, const void* x,
                        int64_t x_stride, const void* weight, const float* mean, const float* rstd, void* dx, int64_t dx_stride,
                        void* dweight, void* dbias, void* workspace, cudaStream_t stream);
// Forward pass of the tcgen05 kernels with the gate applied in the epilogue: writes sigmoid(gate) * out to `gated`
// and, when plain.ptr is not NULL, the ungated values to `plain`.
int tensor_forward_gated(const oops_ta_problem& p, const oops_ta_pair& gate, const oops_ta_pair& gated,
                         const oops_ta_pair& plain, float* lse, cudaStream_t stream);

// Read (and optionally clear) the device-side status words of the two tcgen05 translation units;
// both synchronise with the device.
int forward_device_status(int reset);
// Launches the bounded-wait self-test kernel of the forward translation unit (its wait runs out after 1 ms).
int wait_limit_selftest(cudaStream_t stream);
int backward_device_status(int reset);

}  // namespace oops_ta
