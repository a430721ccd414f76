// Layer normalisation over the last axis of (rows, width) activations, forward and reverse: the step before the q/k/v
// and bias projections of a pair block (reference: oops/normalization/layer_norm/layer_norm.py:37-110 and its Triton
// kernels).  Byte work bound by HBM: one warp owns a row, 16-byte accesses, every statistic in f32.
//   forward:  y = (x - mean) * rstd * weight + bias,  mean and rstd (f32 per row) kept for the reverse pass
//   reverse:  g = dy * weight, xhat = (x - mean) * rstd,
//             dx = rstd * (g - mean_c(g) - xhat * mean_c(g * xhat)),  dweight = sum_rows dy * xhat,  dbias = sum_rows dy
// Rows of up to 1024 elements live in registers between the passes over them (one read of x per kernel); wider rows
// (up to 8192) are read again from L2.  dweight and dbias are summed per warp in registers over the rows the warp
// walks, then per CTA in shared memory, written as f32 partial rows and added in a fixed order by a second small
// kernel: bitwise reproducible, no atomics.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <initializer_list>
#include <type_traits>

#include "ta_internal.h"

namespace oops_ta {
namespace {

constexpr int kLnWarps = 8;             // warps (= rows in flight) per CTA
constexpr int kLnCached = 1024;         // widest row kept in registers
constexpr int kLnPerLane = kLnCached / 32;
#ifndef TA_LN_CTAS
#define TA_LN_CTAS 4
#endif
#ifndef TA_LN_UNROLL
#define TA_LN_UNROLL 4
#endif
constexpr int kLnCtasPerSm = TA_LN_CTAS;        // resident CTAs the row-sharing kernels are compiled for (register cap 64)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// V consecutive elements of a row: one element (any alignment), or 16 bytes (V = 4 for f32, 8 for 16-bit types).
template <typename T, int V>
struct LnVec {
  static __device__ __forceinline__ void load(const T* p, float (&out)[V]) {
    if constexpr (V == 1) {
      out[0] = float(*p);
    } else if constexpr (sizeof(T) == 4) {
      const float4 v = *reinterpret_cast<const float4*>(p);
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(p);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = float(e[i]);
    }
  }
  static __device__ __forceinline__ void store(T* p, const float (&in)[V]) {
    if constexpr (V == 1) {
      *p = T(in[0]);
    } else if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
    } else {
      uint4 v;
      T* e = reinterpret_cast<T*>(&v);
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = T(in[i]);
      *reinterpret_cast<uint4*>(p) = v;
    }
  }
};

// First element of group g of lane `lane`: a warp's accesses are 32 * V contiguous elements.
template <int V>
__device__ __forceinline__ int ln_first(int lane, int g) { return (g * 32 + lane) * V; }

struct LnShape {
  int64_t rows;
  int width;
  int64_t x_stride, y_stride, dy_stride, dx_stride;  // row strides in elements
};

// affine parameters may be of the activation type or f32 ("master" parameters of 16-bit activations)
template <typename A>
__device__ __forceinline__ float affine_at(const void* p, int i, float missing) {
  return p ? float(reinterpret_cast<const A*>(p)[i]) : missing;
}

template <typename T, typename A, int V, bool CACHED>
__global__ void __launch_bounds__(kLnWarps * 32) layer_norm_forward_kernel(LnShape s, const T* __restrict__ x,
                                                                           const void* __restrict__ weight,
                                                                           const void* __restrict__ bias, float eps,
                                                                           T* __restrict__ y, float* __restrict__ mean_out,
                                                                           float* __restrict__ rstd_out) {
  constexpr int kGroups = kLnPerLane / V;  // groups of V elements a lane holds of a cached row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_width = 1.f / float(s.width);
  for (int64_t row = int64_t(blockIdx.x) * kLnWarps + warp; row < s.rows; row += int64_t(gridDim.x) * kLnWarps) {
    const T* xr = x + row * s.x_stride;
    T* yr = y + row * s.y_stride;
    float vals[CACHED ? kGroups : 1][V];
    float sum = 0.f;
    if (CACHED) {
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const int i = ln_first<V>(lane, g);
#pragma unroll
        for (int e = 0; e < V; ++e) vals[g][e] = 0.f;
        if (i < s.width) LnVec<T, V>::load(xr + i, vals[g]);
#pragma unroll
        for (int e = 0; e < V; ++e) sum += vals[g][e];
      }
    } else {
      for (int i = lane; i < s.width; i += 32) sum += float(xr[i]);
    }
    const float mean = warp_sum(sum) * inv_width;
    float sq = 0.f;
    if (CACHED) {
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        if (ln_first<V>(lane, g) < s.width) {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            const float d = vals[g][e] - mean;
            sq += d * d;
          }
        }
      }
    } else {
      for (int i = lane; i < s.width; i += 32) {
        const float d = float(xr[i]) - mean;
        sq += d * d;
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * inv_width + eps);
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    if (CACHED) {
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const int i = ln_first<V>(lane, g);
        if (i < s.width) {
          float out[V];
#pragma unroll
          for (int e = 0; e < V; ++e)
            out[e] = (vals[g][e] - mean) * rstd * affine_at<A>(weight, i + e, 1.f) + affine_at<A>(bias, i + e, 0.f);
          LnVec<T, V>::store(yr + i, out);
        }
      }
    } else {
      for (int i = lane; i < s.width; i += 32)
        yr[i] = T((float(xr[i]) - mean) * rstd * affine_at<A>(weight, i, 1.f) + affine_at<A>(bias, i, 0.f));
    }
  }
}

// Reverse pass.  dweight/dbias: every lane sums its columns over the rows its warp walks (cached rows only), the
// eight warps of a CTA are added through shared memory, and the CTA writes one f32 partial row per tensor.
template <typename T, typename A, int V, bool CACHED>
__global__ void __launch_bounds__(kLnWarps * 32) layer_norm_backward_kernel(LnShape s, const T* __restrict__ dy,
                                                                            const T* __restrict__ x,
                                                                            const void* __restrict__ weight,
                                                                            const float* __restrict__ mean_in,
                                                                            const float* __restrict__ rstd_in,
                                                                            T* __restrict__ dx, float* __restrict__ dw_parts,
                                                                            float* __restrict__ db_parts) {
  constexpr int kGroups = kLnPerLane / V;
  extern __shared__ float ln_smem[];  // [kLnWarps][width] when partials are wanted
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_width = 1.f / float(s.width);
  const bool want_parts = CACHED && (dw_parts != nullptr || db_parts != nullptr);
  float dw[CACHED ? kGroups : 1][V], db[CACHED ? kGroups : 1][V];
#pragma unroll
  for (int g = 0; g < (CACHED ? kGroups : 1); ++g)
#pragma unroll
    for (int e = 0; e < V; ++e) dw[g][e] = db[g][e] = 0.f;

  for (int64_t row = int64_t(blockIdx.x) * kLnWarps + warp; row < s.rows; row += int64_t(gridDim.x) * kLnWarps) {
    const T* xr = x + row * s.x_stride;
    const T* gr = dy + row * s.dy_stride;
    const float mean = mean_in[row], rstd = rstd_in[row];
    if (CACHED) {
      float xh[kGroups][V], gw[kGroups][V];
      float c1 = 0.f, c2 = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const int i = ln_first<V>(lane, g);
#pragma unroll
        for (int e = 0; e < V; ++e) xh[g][e] = gw[g][e] = 0.f;
        if (i < s.width) {
          float xv[V], gv[V];
          LnVec<T, V>::load(xr + i, xv);
          LnVec<T, V>::load(gr + i, gv);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            xh[g][e] = (xv[e] - mean) * rstd;
            dw[g][e] += gv[e] * xh[g][e];
            db[g][e] += gv[e];
            gw[g][e] = gv[e] * affine_at<A>(weight, i + e, 1.f);
            c1 += gw[g][e] * xh[g][e];
            c2 += gw[g][e];
          }
        }
      }
      c1 = warp_sum(c1) * inv_width;
      c2 = warp_sum(c2) * inv_width;
      if (dx) {
        T* dr = dx + row * s.dx_stride;
#pragma unroll
        for (int g = 0; g < kGroups; ++g) {
          const int i = ln_first<V>(lane, g);
          if (i < s.width) {
            float out[V];
#pragma unroll
            for (int e = 0; e < V; ++e) out[e] = rstd * (gw[g][e] - c2 - xh[g][e] * c1);
            LnVec<T, V>::store(dr + i, out);
          }
        }
      }
    } else {
      float c1 = 0.f, c2 = 0.f;
      for (int i = lane; i < s.width; i += 32) {
        const float xhat = (float(xr[i]) - mean) * rstd, g = float(gr[i]) * affine_at<A>(weight, i, 1.f);
        c1 += g * xhat;
        c2 += g;
      }
      c1 = warp_sum(c1) * inv_width;
      c2 = warp_sum(c2) * inv_width;
      if (dx) {
        T* dr = dx + row * s.dx_stride;
        for (int i = lane; i < s.width; i += 32) {
          const float xhat = (float(xr[i]) - mean) * rstd, g = float(gr[i]) * affine_at<A>(weight, i, 1.f);
          dr[i] = T(rstd * (g - c2 - xhat * c1));
        }
      }
    }
  }
  if (want_parts) {
    for (int pass = 0; pass < 2; ++pass) {
      float* parts = pass == 0 ? dw_parts : db_parts;
      if (!parts) continue;
      __syncthreads();
#pragma unroll
      for (int g = 0; g < kGroups; ++g) {
        const int i = ln_first<V>(lane, g);
        if (i < s.width) {
#pragma unroll
          for (int e = 0; e < V; ++e) ln_smem[warp * s.width + i + e] = pass == 0 ? dw[g][e] : db[g][e];
        }
      }
      __syncthreads();
      for (int i = threadIdx.x; i < s.width; i += kLnWarps * 32) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kLnWarps; ++w) total += ln_smem[w * s.width + i];
        parts[int64_t(blockIdx.x) * s.width + i] = total;
      }
    }
  }
}

// ---- rows of up to 1024 elements with 16-byte accesses: LPR lanes share a row, each holding GROUPS groups of V
// elements; a warp works on 32 / LPR rows at once and on kLnUnroll such row blocks per loop turn, so that enough
// loads are in flight to cover the memory latency (a 128-channel bf16 row is only 256 bytes).
constexpr int kLnUnroll = TA_LN_UNROLL;

template <int LPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Packed arithmetic: a group of V elements is V / 2 pairs of f32, and every add / multiply-add below works on a pair
// (fma.rn.f32x2 and friends), which halves the instructions per byte; 16-bit rows were bound by instruction issue.
typedef float2 ln2;
__device__ __forceinline__ ln2 ln_fma2(ln2 a, ln2 b, ln2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ ln2 ln_add2(ln2 a, ln2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ ln2 ln_mul2(ln2 a, ln2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ ln2 ln_both(float v) { return make_float2(v, v); }

template <typename T, int V>
__device__ __forceinline__ void ln_unpack2(const uint4& raw, ln2 (&out)[V / 2]) {
  static_assert(V * sizeof(T) == 16, "a raw group is 16 bytes");
  if constexpr (sizeof(T) == 4) {
    out[0] = make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
    out[1] = make_float2(__uint_as_float(raw.z), __uint_as_float(raw.w));
  } else {
    const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        out[i] = make_float2(__uint_as_float(words[i] << 16), __uint_as_float(words[i] & 0xffff0000u));
      } else {
        out[i] = __half22float2(*reinterpret_cast<const __half2*>(&words[i]));
      }
    }
  }
}

template <typename T, int V>
__device__ __forceinline__ uint4 ln_pack2(const ln2 (&in)[V / 2]) {
  if constexpr (sizeof(T) == 4) {
    return make_uint4(__float_as_uint(in[0].x), __float_as_uint(in[0].y), __float_as_uint(in[1].x), __float_as_uint(in[1].y));
  } else {
    uint32_t words[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        const __nv_bfloat162 h = __float22bfloat162_rn(in[i]);
        words[i] = *reinterpret_cast<const uint32_t*>(&h);
      } else {
        const __half2 h = __float22half2_rn(in[i]);
        words[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    }
    return make_uint4(words[0], words[1], words[2], words[3]);
  }
}

template <typename T, typename A, int V, int GROUPS, int LPR>
__global__ void __launch_bounds__(kLnWarps * 32, GROUPS == 1 ? kLnCtasPerSm : 1) layer_norm_forward_rows_kernel(LnShape s, const T* __restrict__ x,
                                                                                const void* __restrict__ weight,
                                                                                const void* __restrict__ bias, float eps,
                                                                                T* __restrict__ y, float* __restrict__ mean_out,
                                                                                float* __restrict__ rstd_out) {
  constexpr int kRowsPerWarp = 32 / LPR, P = V / 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const float inv_width = 1.f / float(s.width);
  // this lane's affine parameters, fetched once (zero outside the row)
  ln2 w[GROUPS][P], b[GROUPS][P];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int e = 0; e < P; ++e) {
      const int i = (g * LPR + l) * V + 2 * e;
      const bool in = i < s.width;
      w[g][e] = make_float2(in ? affine_at<A>(weight, i, 1.f) : 0.f, in ? affine_at<A>(weight, i + 1, 1.f) : 0.f);
      b[g][e] = make_float2(in ? affine_at<A>(bias, i, 0.f) : 0.f, in ? affine_at<A>(bias, i + 1, 0.f) : 0.f);
    }
  const int64_t blocks = (s.rows + kRowsPerWarp - 1) / kRowsPerWarp;  // row blocks of one warp
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t blk0 = int64_t(blockIdx.x) * kLnWarps + warp; blk0 < blocks; blk0 += stride * kLnUnroll) {
    uint4 raw[kLnUnroll][GROUPS];
#pragma unroll
    for (int u = 0; u < kLnUnroll; ++u) {
      const int64_t row = (blk0 + u * stride) * kRowsPerWarp + sub;
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        const int i = (g * LPR + l) * V;
        raw[u][g] = make_uint4(0, 0, 0, 0);  // zero bits are 0.0 in every served type
        if (blk0 + u * stride < blocks && row < s.rows && i < s.width)
          raw[u][g] = *reinterpret_cast<const uint4*>(x + row * s.x_stride + i);
      }
    }
#pragma unroll
    for (int u = 0; u < kLnUnroll; ++u) {
      const int64_t row = (blk0 + u * stride) * kRowsPerWarp + sub;
      const bool live = blk0 + u * stride < blocks && row < s.rows;
      ln2 v[GROUPS][P];
      ln2 sum2 = ln_both(0.f);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        ln_unpack2<T, V>(raw[u][g], v[g]);
#pragma unroll
        for (int e = 0; e < P; ++e) sum2 = ln_add2(sum2, v[g][e]);
      }
      const float mean = row_sum<LPR>(sum2.x + sum2.y) * inv_width;
      const ln2 neg_mean = ln_both(-mean);
      ln2 sq2 = ln_both(0.f);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g)
        if ((g * LPR + l) * V < s.width) {
#pragma unroll
          for (int e = 0; e < P; ++e) {
            v[g][e] = ln_add2(v[g][e], neg_mean);  // centred from here on
            sq2 = ln_fma2(v[g][e], v[g][e], sq2);
          }
        }
      const float rstd = rsqrtf(row_sum<LPR>(sq2.x + sq2.y) * inv_width + eps);
      if (!live) continue;
      if (l == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
      }
      const ln2 rstd2 = ln_both(rstd);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        const int i = (g * LPR + l) * V;
        if (i < s.width) {
          ln2 out[P];
#pragma unroll
          for (int e = 0; e < P; ++e) out[e] = ln_fma2(ln_mul2(v[g][e], rstd2), w[g][e], b[g][e]);
          *reinterpret_cast<uint4*>(y + row * s.y_stride + i) = ln_pack2<T, V>(out);
        }
      }
    }
  }
}

template <typename T, typename A, int V, int GROUPS, int LPR>
__global__ void __launch_bounds__(kLnWarps * 32, GROUPS == 1 ? kLnCtasPerSm : 1) layer_norm_backward_rows_kernel(LnShape s, const T* __restrict__ dy,
                                                                                 const T* __restrict__ x,
                                                                                 const void* __restrict__ weight,
                                                                                 const float* __restrict__ mean_in,
                                                                                 const float* __restrict__ rstd_in,
                                                                                 T* __restrict__ dx, float* __restrict__ dw_parts,
                                                                                 float* __restrict__ db_parts) {
  constexpr int kRowsPerWarp = 32 / LPR, P = V / 2;
  constexpr int kU = kLnUnroll / 2;  // two tensors are read per row
  extern __shared__ float ln_smem[];  // [kLnWarps * kRowsPerWarp][width] when partials are wanted
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
  const float inv_width = 1.f / float(s.width);
  ln2 w[GROUPS][P], dw[GROUPS][P], db[GROUPS][P];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int e = 0; e < P; ++e) {
      const int i = (g * LPR + l) * V + 2 * e;
      const bool in = i < s.width;
      w[g][e] = make_float2(in ? affine_at<A>(weight, i, 1.f) : 0.f, in ? affine_at<A>(weight, i + 1, 1.f) : 0.f);
      dw[g][e] = db[g][e] = ln_both(0.f);
    }
  const int64_t blocks = (s.rows + kRowsPerWarp - 1) / kRowsPerWarp;
  const int64_t stride = int64_t(gridDim.x) * kLnWarps;
  for (int64_t blk0 = int64_t(blockIdx.x) * kLnWarps + warp; blk0 < blocks; blk0 += stride * kU) {
    uint4 xraw[kU][GROUPS], graw[kU][GROUPS];
    float mean[kU], rstd[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t row = (blk0 + u * stride) * kRowsPerWarp + sub;
      const bool live = blk0 + u * stride < blocks && row < s.rows;
      mean[u] = live ? mean_in[row] : 0.f;
      rstd[u] = live ? rstd_in[row] : 0.f;
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        const int i = (g * LPR + l) * V;
        xraw[u][g] = graw[u][g] = make_uint4(0, 0, 0, 0);
        if (live && i < s.width) {
          xraw[u][g] = *reinterpret_cast<const uint4*>(x + row * s.x_stride + i);
          graw[u][g] = *reinterpret_cast<const uint4*>(dy + row * s.dy_stride + i);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t row = (blk0 + u * stride) * kRowsPerWarp + sub;
      const bool live = blk0 + u * stride < blocks && row < s.rows;
      const ln2 rstd2 = ln_both(rstd[u]), neg_mean2 = ln_both(-mean[u]);
      ln2 xh[GROUPS][P], gw[GROUPS][P];
      ln2 c1 = ln_both(0.f), c2 = ln_both(0.f);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        ln2 gv[P];
        ln_unpack2<T, V>(xraw[u][g], xh[g]);
        ln_unpack2<T, V>(graw[u][g], gv);
        const bool inside = live && (g * LPR + l) * V < s.width;
#pragma unroll
        for (int e = 0; e < P; ++e) {
          xh[g][e] = inside ? ln_mul2(ln_add2(xh[g][e], neg_mean2), rstd2) : ln_both(0.f);
          dw[g][e] = ln_fma2(gv[e], xh[g][e], dw[g][e]);
          db[g][e] = ln_add2(db[g][e], gv[e]);
          gw[g][e] = ln_mul2(gv[e], w[g][e]);
          c1 = ln_fma2(gw[g][e], xh[g][e], c1);
          c2 = ln_add2(c2, gw[g][e]);
        }
      }
      const float m1 = row_sum<LPR>(c1.x + c1.y) * inv_width, m2 = row_sum<LPR>(c2.x + c2.y) * inv_width;
      if (!live || !dx) continue;
      const ln2 neg_m1 = ln_both(-m1), neg_m2 = ln_both(-m2);
#pragma unroll
      for (int g = 0; g < GROUPS; ++g) {
        const int i = (g * LPR + l) * V;
        if (i < s.width) {
          ln2 out[P];
#pragma unroll
          for (int e = 0; e < P; ++e) out[e] = ln_mul2(ln_fma2(xh[g][e], neg_m1, ln_add2(gw[g][e], neg_m2)), rstd2);
          *reinterpret_cast<uint4*>(dx + row * s.dx_stride + i) = ln_pack2<T, V>(out);
        }
      }
    }
  }
  if (dw_parts != nullptr || db_parts != nullptr) {
    constexpr int kSubs = kLnWarps * kRowsPerWarp;
    for (int pass = 0; pass < 2; ++pass) {
      float* parts = pass == 0 ? dw_parts : db_parts;
      if (!parts) continue;
      __syncthreads();
#pragma unroll
      for (int g = 0; g < GROUPS; ++g)
#pragma unroll
        for (int e = 0; e < P; ++e) {
          const int i = (g * LPR + l) * V + 2 * e;
          if (i < s.width) {
            const ln2 v = pass == 0 ? dw[g][e] : db[g][e];
            ln_smem[(warp * kRowsPerWarp + sub) * s.width + i] = v.x;
            ln_smem[(warp * kRowsPerWarp + sub) * s.width + i + 1] = v.y;
          }
        }
      __syncthreads();
      for (int i = threadIdx.x; i < s.width; i += kLnWarps * 32) {
        float total = 0.f;
        for (int k = 0; k < kSubs; ++k) total += ln_smem[k * s.width + i];
        parts[int64_t(blockIdx.x) * s.width + i] = total;
      }
    }
  }
}

// Column sums for rows too wide to keep per-lane sums in registers: CTA (column block, row part), one column per thread.
template <typename T>
__global__ void layer_norm_wide_parts_kernel(LnShape s, const T* __restrict__ dy, const T* __restrict__ x,
                                             const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                                             int64_t rows_per_part, float* __restrict__ dw_parts, float* __restrict__ db_parts) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= s.width) return;
  const int64_t first = int64_t(blockIdx.y) * rows_per_part, last = min(first + rows_per_part, s.rows);
  float dw = 0.f, db = 0.f;
  for (int64_t row = first; row < last; ++row) {
    const float g = float(dy[row * s.dy_stride + col]);
    dw += g * (float(x[row * s.x_stride + col]) - mean_in[row]) * rstd_in[row];
    db += g;
  }
  if (dw_parts) dw_parts[int64_t(blockIdx.y) * s.width + col] = dw;
  if (db_parts) db_parts[int64_t(blockIdx.y) * s.width + col] = db;
}

// out[col] = sum over parts of parts[part][col], stored in the parameter's type, for dweight (blockIdx.y = 0) and
// dbias (1) in one launch.  A block owns 32 columns; its eight warps each add every eighth partial row (coalesced
// 128-byte reads), and the eight sums are added in warp order: the order is fixed, so the result is reproducible.
template <typename A>
__global__ void __launch_bounds__(256) layer_norm_reduce_parts_kernel(const float* __restrict__ dw_parts,
                                                                      const float* __restrict__ db_parts, int num_parts, int width,
                                                                      A* __restrict__ dweight, A* __restrict__ dbias) {
  __shared__ float sums[8][32];
  const float* parts = blockIdx.y == 0 ? dw_parts : db_parts;
  A* out = blockIdx.y == 0 ? dweight : dbias;
  if (!parts || !out) return;  // the whole block takes the same branch
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, col = blockIdx.x * 32 + lane;
  float total = 0.f;
  if (col < width)
    for (int p = warp; p < num_parts; p += 8) total += parts[int64_t(p) * width + col];
  sums[warp][lane] = total;
  __syncthreads();
  if (warp == 0 && col < width) {
    float all = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) all += sums[w][lane];
    out[col] = A(all);
  }
}

constexpr int kLnMaxWidth = 8192;
constexpr int kLnWideParts = 64;

int ln_grid(int64_t rows) {
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int64_t wanted = (rows + kLnWarps - 1) / kLnWarps;
  return int(wanted < int64_t(sms) * kLnCtasPerSm ? wanted : int64_t(sms) * kLnCtasPerSm);
}

bool ln_vector_ok(int vec, int width, std::initializer_list<const void*> pointers, std::initializer_list<int64_t> strides) {
  if (width % vec) return false;
  for (const void* p : pointers)
    if (p && (reinterpret_cast<uintptr_t>(p) & 15)) return false;
  for (int64_t st : strides)
    if (st % vec) return false;
  return true;
}

template <typename T, typename A>
int forward_typed(const LnShape& s, const void* x, const void* weight, const void* bias, float eps, void* y, float* mean,
                  float* rstd, cudaStream_t stream) {
  constexpr int kVec = 16 / int(sizeof(T));
  const bool vec = ln_vector_ok(kVec, s.width, {x, y}, {s.x_stride, s.y_stride});
  const bool cached = s.width <= kLnCached;
  const int grid = ln_grid(s.rows), threads = kLnWarps * 32;
  const T* xp = reinterpret_cast<const T*>(x);
  T* yp = reinterpret_cast<T*>(y);
  const int units = (s.width + kVec - 1) / kVec;  // 16-byte groups of a row
  if (vec && units <= 128) {
#define OOPS_LN_FWD(GROUPS, LPR)                                                                                         \
  layer_norm_forward_rows_kernel<T, A, kVec, GROUPS, LPR>                                                                \
      <<<ln_grid((s.rows + 32 / LPR - 1) / (32 / LPR)), threads, 0, stream>>>(s, xp, weight, bias, eps, yp, mean, rstd)
    if (units <= 8) OOPS_LN_FWD(1, 8);
    else if (units <= 16) OOPS_LN_FWD(1, 16);
    else if (units <= 32) OOPS_LN_FWD(1, 32);
    else if (units <= 64) OOPS_LN_FWD(2, 32);
    else OOPS_LN_FWD(4, 32);
#undef OOPS_LN_FWD
  } else if (cached && vec)
    layer_norm_forward_kernel<T, A, kVec, true><<<grid, threads, 0, stream>>>(s, xp, weight, bias, eps, yp, mean, rstd);
  else if (cached)
    layer_norm_forward_kernel<T, A, 1, true><<<grid, threads, 0, stream>>>(s, xp, weight, bias, eps, yp, mean, rstd);
  else
    layer_norm_forward_kernel<T, A, 1, false><<<grid, threads, 0, stream>>>(s, xp, weight, bias, eps, yp, mean, rstd);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OOPS_TA_OK : OOPS_TA_CUDA_ERROR;
}

template <typename T, typename A>
int backward_typed(const LnShape& s, const void* dy, const void* x, const void* weight, const float* mean, const float* rstd,
                   void* dx, void* dweight, void* dbias, float* workspace, cudaStream_t stream) {
  constexpr int kVec = 16 / int(sizeof(T));
  const bool vec = ln_vector_ok(kVec, s.width, {x, dy, dx}, {s.x_stride, s.dy_stride, s.dx_stride});
  const bool cached = s.width <= kLnCached;
  int grid = ln_grid(s.rows);
  const int threads = kLnWarps * 32;
  const bool parts_wanted = dweight != nullptr || dbias != nullptr;
  const int units = (s.width + kVec - 1) / kVec;
  const bool shared_rows = vec && units <= 128;  // several lanes (not always a whole warp) share a row
  const int lpr = units <= 8 ? 8 : units <= 16 ? 16 : 32;
  if (shared_rows) grid = ln_grid((s.rows + 32 / lpr - 1) / (32 / lpr));
  const int num_parts = cached ? grid : int(s.rows < kLnWideParts ? s.rows : kLnWideParts);
  float* dw_parts = dweight ? workspace : nullptr;
  float* db_parts = dbias ? workspace + int64_t(num_parts) * s.width : nullptr;
  const T* gp = reinterpret_cast<const T*>(dy);
  const T* xp = reinterpret_cast<const T*>(x);
  T* dp = reinterpret_cast<T*>(dx);
  const size_t smem = cached && parts_wanted ? size_t(kLnWarps) * s.width * sizeof(float) : 0;
  if (shared_rows) {
    const size_t rows_smem = parts_wanted ? size_t(kLnWarps) * (32 / lpr) * s.width * sizeof(float) : 0;
#define OOPS_LN_BWD(GROUPS, LPR)                                                                                         \
  layer_norm_backward_rows_kernel<T, A, kVec, GROUPS, LPR>                                                               \
      <<<grid, threads, rows_smem, stream>>>(s, gp, xp, weight, mean, rstd, dp, dw_parts, db_parts)
    if (units <= 8) OOPS_LN_BWD(1, 8);
    else if (units <= 16) OOPS_LN_BWD(1, 16);
    else if (units <= 32) OOPS_LN_BWD(1, 32);
    else if (units <= 64) OOPS_LN_BWD(2, 32);
    else OOPS_LN_BWD(4, 32);
#undef OOPS_LN_BWD
  } else if (cached && vec)
    layer_norm_backward_kernel<T, A, kVec, true><<<grid, threads, smem, stream>>>(s, gp, xp, weight, mean, rstd, dp, dw_parts, db_parts);
  else if (cached)
    layer_norm_backward_kernel<T, A, 1, true><<<grid, threads, smem, stream>>>(s, gp, xp, weight, mean, rstd, dp, dw_parts, db_parts);
  else if (dx)
    layer_norm_backward_kernel<T, A, 1, false><<<grid, threads, 0, stream>>>(s, gp, xp, weight, mean, rstd, dp, nullptr, nullptr);
  if (cached || dx) count_launch();
  if (parts_wanted) {
    if (!cached) {
      const int64_t rows_per_part = (s.rows + num_parts - 1) / num_parts;
      layer_norm_wide_parts_kernel<T><<<dim3((s.width + 127) / 128, num_parts), 128, 0, stream>>>(s, gp, xp, mean, rstd, rows_per_part,
                                                                                                  dw_parts, db_parts);
      count_launch();
    }
    layer_norm_reduce_parts_kernel<A><<<dim3((s.width + 31) / 32, 2), 256, 0, stream>>>(
        dw_parts, db_parts, num_parts, s.width, reinterpret_cast<A*>(dweight), reinterpret_cast<A*>(dbias));
    count_launch();
  }
  return cudaGetLastError() == cudaSuccess ? OOPS_TA_OK : OOPS_TA_CUDA_ERROR;
}

// dtype of the activations and of the affine parameters: the same, or f32 parameters with 16-bit activations
template <typename F>
int ln_dispatch(int dtype, int affine_dtype, F&& run) {
  if (affine_dtype != dtype && affine_dtype != OOPS_TA_F32) return OOPS_TA_UNSUPPORTED_DTYPE;
  const bool master = affine_dtype == OOPS_TA_F32;
  switch (dtype) {
    case OOPS_TA_F32: return run(float{}, float{});
    case OOPS_TA_F16: return master ? run(__half{}, float{}) : run(__half{}, __half{});
    case OOPS_TA_BF16: return master ? run(__nv_bfloat16{}, float{}) : run(__nv_bfloat16{}, __nv_bfloat16{});
    default: return OOPS_TA_UNSUPPORTED_DTYPE;
  }
}

}  // namespace

uint64_t layer_norm_backward_workspace_bytes(int64_t rows, int width) {
  if (rows <= 0 || width <= 0) return 0;
  // cached rows: one partial row per CTA, and no launch has more CTAs than ln_grid of the row count
  const int64_t parts = width <= kLnCached ? ln_grid(rows) : (rows < kLnWideParts ? rows : kLnWideParts);
  return uint64_t(2) * uint64_t(parts) * uint64_t(width) * sizeof(float);
}

int layer_norm_max_width() { return kLnMaxWidth; }

int layer_norm_forward(int dtype, int affine_dtype, int64_t rows, int width, const void* x, int64_t x_stride, const void* weight,
                       const void* bias, float eps, void* y, int64_t y_stride, float* mean, float* rstd, cudaStream_t stream) {
  if (rows == 0) return OOPS_TA_OK;
  const LnShape s{rows, width, x_stride, y_stride, 0, 0};
  return ln_dispatch(dtype, affine_dtype, [&](auto t, auto a) {
    return forward_typed<decltype(t), decltype(a)>(s, x, weight, bias, eps, y, mean, rstd, stream);
  });
}

int layer_norm_backward(int dtype, int affine_dtype, int64_t rows, int width, const void* dy, int64_t dy_stride, const void* x,
                        int64_t x_stride, const void* weight, const float* mean, const float* rstd, void* dx, int64_t dx_stride,
                        void* dweight, void* dbias, void* workspace, cudaStream_t stream) {
  if (rows == 0) return OOPS_TA_OK;
  const LnShape s{rows, width, x_stride, 0, dy_stride, dx_stride};
  return ln_dispatch(dtype, affine_dtype, [&](auto t, auto a) {
    return backward_typed<decltype(t), decltype(a)>(s, dy, x, weight, mean, rstd, dx, dweight, dbias,
                                                    reinterpret_cast<float*>(workspace), stream);
  });
}

}  // namespace oops_ta
