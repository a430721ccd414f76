// Host/device helpers shared by the tcgen05 forward and reverse translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "sm100_ptx.cuh"
#include "ta_internal.h"

namespace oops_ta {
namespace {

constexpr int kHeadDim = 32;
constexpr int kTile = 128;  // queries per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// First device-side failure recorded by a kernel of this translation unit (an oops_ta_status value).
__device__ int g_tu_device_status = 0;

int read_tu_device_status(int reset) {
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_tu_device_status, sizeof(int)) != cudaSuccess)
    return fail(OOPS_TA_CUDA_ERROR, "cannot read the device status word");
  if (reset && value != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_tu_device_status, &zero, sizeof(int));
  }
  return value;
}

// After a kernel has given up a wait, the kernels of this translation unit return at once until the host
// clears the word (oops_ta_device_status(1)): one stuck wait must not be repeated by every later CTA.
__device__ __forceinline__ bool device_failed() { return *reinterpret_cast<volatile int*>(&g_tu_device_status) != 0; }

// Shared tail of every tcgen05 kernel: after the CTA-wide barrier, a CTA that abandoned a wait lets
// its in-flight copies land and records the failure; then the allocating warp frees tensor memory.
__device__ __forceinline__ void teardown(volatile int* abort_flag, uint32_t tmem_base, int alloc_warp,
                                         uint32_t tmem_cols = 512) {
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t start = ptx::globaltimer_ns();
    while (ptx::globaltimer_ns() - start < 200000ull) __nanosleep(1000);
    if (threadIdx.x == 0) atomicCAS(&g_tu_device_status, 0, (int)OOPS_TA_DEVICE_TIMEOUT);
    __syncthreads();
  }
  if ((int)(threadIdx.x >> 5) == alloc_warp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, tmem_cols);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &query) == cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 5-D map over (inner, d1, d2, d3, d4); strides in elements for d1..d4 (inner stride is 1).
int encode_map(CUtensorMap* map, int dtype, const void* ptr, const uint64_t dims[5], const int64_t strides[4],
               const uint32_t box[5], CUtensorMapSwizzle swizzle, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(OOPS_TA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t gbox[5], estride[5] = {1, 1, 1, 1, 1};
  uint64_t fallback = dims[0] * 2;
  for (int i = 0; i < 5; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
  }
  for (int i = 0; i < 4; ++i) {
    uint64_t bytes = uint64_t(strides[i]) * 2;
    if (dims[i + 1] == 1 && (strides[i] <= 0 || bytes % 16 != 0)) bytes = (fallback + 15) & ~uint64_t(15);
    gstride[i] = bytes;
    fallback = bytes * dims[i + 1];
  }
  const CUtensorMapDataType type = dtype == OOPS_TA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult rc = fn(map, type, 5, const_cast<void*>(ptr), gdim, gstride, gbox, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return fail(OOPS_TA_UNSUPPORTED_LAYOUT, "tensor map for %s rejected (CUresult %d)", what, (int)rc);
  return OOPS_TA_OK;
}

bool stride_ok(int64_t stride, int size) { return size == 1 || (stride > 0 && stride % 8 == 0); }

bool pair_ok(const oops_ta_pair& t, const oops_ta_problem& p) {
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && stride_ok(t.sb, p.batch) && stride_ok(t.sr, p.rows) &&
         stride_ok(t.sc, p.cols) && stride_ok(t.sh, p.heads);
}

// Map over a pair tensor viewed as (channel, head, column, row, batch); the box is `box_cols` columns of one head.
int encode_pair(CUtensorMap* map, const oops_ta_problem& p, const oops_ta_pair& t, uint32_t box_cols, const char* what) {
  const uint64_t dims[5] = {uint64_t(p.head_dim), uint64_t(p.heads), uint64_t(p.cols), uint64_t(p.rows), uint64_t(p.batch)};
  const int64_t strides[4] = {t.sh, t.sc, t.sr, t.sb};
  const uint32_t box[5] = {kHeadDim, 1, box_cols, 1, 1};
  return encode_map(map, p.dtype, t.ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B, what);
}

// Map over a bias viewed as (inner, outer, head, group, batch) with `inner` contiguous; box = 64 x `box_outer`.
int encode_bias(CUtensorMap* map, const oops_ta_problem& p, const void* ptr, int64_t s_outer, int64_t sh, int64_t sg,
                int64_t sb, uint32_t box_outer, const char* what) {
  const uint64_t dims[5] = {uint64_t(p.cols), uint64_t(p.cols), uint64_t(p.heads), uint64_t(p.bias_groups), uint64_t(p.batch)};
  const int64_t strides[4] = {s_outer, sh, sg, sb};
  const uint32_t box[5] = {64, box_outer, 1, 1, 1};
  return encode_map(map, p.dtype, ptr, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, what);
}

template <typename Kernel>
int reserve_smem(Kernel kernel, int bytes) {
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return fail(OOPS_TA_CUDA_ERROR, "cannot reserve %d bytes of shared memory", bytes);
  return OOPS_TA_OK;
}

}  // namespace
}  // namespace oops_ta
