// tcgen05 / TMEM / TMA reverse pass of triangle attention for sm_100a (f16 and bf16, head_dim 32).
//
// Replaces the reference's Triton kernels `_backward_preprocess`, `_backward_query`,
// `_backward_key_value` and `_backward_shared_bias` (oops/attention/triangle/triton/kernel.py:374-873).
// With P = exp(S - lse), dP = dO V^T, dS = P o (dP - delta) (kernel.py:499-564):
//
//   delta kernel     delta[q] = sum_d O[q,d] dO[q,d]                           (memory bound)
//   dQ kernel        CTA = (batch,row,head, one 128-query tile), streams 64-key steps:
//                    S = Q K^T, dP = dO V^T -> dS (16-bit, back into tensor memory) -> dQ += dS K.
//                    A per-row bias gradient is dS itself and is stored from here.
//   dK/dV kernel     CTA = (batch,row,head, one 128-key tile), streams 64-query steps, transposed:
//                    S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T (tensor memory) -> dV += P^T dO, dK += dS^T Q.
//                    It reads a transposed copy of the bias so that a thread (= one key) reads a bias row.
//   shared-bias      CTA = (row part, batch, head, query tile, key tile) loops over its rows:
//   gradient         S, dP -> dS accumulated in f32 registers over the rows (four warpgroups split the
//                    128 keys), one f32 partial plane per part; a last kernel adds the parts in a fixed
//                    order (no atomics, bitwise reproducible).
//
// All kernels share the forward kernel's structure: one TMA producer thread, one MMA-issuing thread,
// warpgroups of 128 threads that own one tensor-memory lane (= one query or key) each.  The dQ and dK/dV
// kernels keep 256 tensor-memory columns and under 113 KB of shared memory, so two CTAs share an SM: their
// MMA threads run independently and one CTA's prologue and epilogue overlap the other's steps.
#include <type_traits>

#include "ta_tensor_common.cuh"

namespace oops_ta {
namespace {

using namespace ptx;

constexpr int kTilesPerCta = 1;                          // dQ and dK/dV kernels: 128-row tiles owned by one CTA (1 or 2)
constexpr int kElemWarps = 8 * kTilesPerCta;             // two warpgroups per tile
constexpr int kThreads = (kElemWarps + (kTilesPerCta == 2 ? 3 : 2)) * 32;
constexpr int kCtasPerSm = kTilesPerCta == 2 ? 1 : 2;
constexpr int kDbElemWarps = 16;                         // shared-bias kernel: one warpgroup per 32 of the tile's 128 keys
constexpr int kDbThreads = (kDbElemWarps + 2) * 32;
constexpr int kStep = 64;                               // streamed keys (dQ) or queries (dK/dV) per step
constexpr int kBigTile = kTile * kHeadDim * 2;          // 8 KiB: 128 x 32 tile
constexpr int kSmallTile = kStep * kHeadDim * 2;        // 4 KiB: 64 x 32 tile
constexpr int kBiasStep = kTile * kStep * 2;            // 16 KiB: 128 x 64 bias tile (one swizzle-128 box)
constexpr int kRing = 4;                                // ring depth of the streamed operand pairs

// ---------------------------------------------------------------------------------------------
// small helper kernels
// ---------------------------------------------------------------------------------------------

template <typename T>
__global__ void delta_kernel(oops_ta_pair out, oops_ta_pair dout, float* delta, int64_t total, int cols, int heads,
                             int rows, int vec_ok) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int q = i % cols;
  const int h = (i / cols) % heads;
  const int r = (i / (int64_t(cols) * heads)) % rows;
  const int64_t b = i / (int64_t(cols) * heads * rows);
  const T* o = reinterpret_cast<const T*>(out.ptr) + b * out.sb + int64_t(r) * out.sr + int64_t(q) * out.sc + h * out.sh;
  const T* d = reinterpret_cast<const T*>(dout.ptr) + b * dout.sb + int64_t(r) * dout.sr + int64_t(q) * dout.sc + h * dout.sh;
  float total_dot = 0.f;
  if (vec_ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 a = reinterpret_cast<const uint4*>(o)[c];
      const uint4 g = reinterpret_cast<const uint4*>(d)[c];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        total_dot += Half2<T>::lo(aw[e]) * Half2<T>::lo(gw[e]) + Half2<T>::hi(aw[e]) * Half2<T>::hi(gw[e]);
    }
  } else {
    for (int c = 0; c < kHeadDim; ++c) total_dot += float(o[c]) * float(d[c]);
  }
  delta[i] = total_dot;
}

// dst[z][k][q] = src[z][q][k] for 16-bit elements; dst rows are `dst_stride` elements apart.
__global__ void transpose_bias_kernel(const uint16_t* src, uint16_t* dst, int cols, int64_t s_q, int64_t s_h, int64_t s_g,
                                      int64_t s_b, int heads, int groups, int64_t dst_stride) {
  __shared__ uint16_t tile[32][34];
  const int z = blockIdx.z;
  const int h = z % heads;
  const int g = (z / heads) % groups;
  const int64_t b = z / (heads * groups);
  const uint16_t* plane = src + b * s_b + g * s_g + h * s_h;
  uint16_t* out = dst + int64_t(z) * cols * dst_stride;
  const int k0 = blockIdx.x * 32, q0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int q = q0 + i, k = k0 + threadIdx.x;
    tile[i][threadIdx.x] = (q < cols && k < cols) ? plane[int64_t(q) * s_q + k] : uint16_t(0);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int k = k0 + i, q = q0 + threadIdx.x;
    if (k < cols && q < dst_stride) out[int64_t(k) * dst_stride + q] = q < cols ? tile[threadIdx.x][i] : uint16_t(0);
  }
}

template <typename T>
__global__ void reduce_parts_kernel(const float* parts, int num_parts, void* dbias, int64_t sb, int64_t sh, int64_t sq,
                                    int64_t sk, int batch, int heads, int cols) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t plane = int64_t(batch) * heads * cols * cols;
  if (i >= plane) return;
  float total = 0.f;
  for (int p = 0; p < num_parts; ++p) total += parts[int64_t(p) * plane + i];
  const int k = i % cols;
  const int q = (i / cols) % cols;
  const int h = (i / (int64_t(cols) * cols)) % heads;
  const int64_t b = i / (int64_t(cols) * cols * heads);
  reinterpret_cast<T*>(dbias)[b * sb + h * sh + int64_t(q) * sq + int64_t(k) * sk] = T(total);
}

// 16-bit row store of 32 channels from f32 accumulator words, scaled.
template <typename T>
__device__ __forceinline__ void store_row32(T* dst, const uint32_t (&acc)[32], float scale, bool vec_ok) {
  uint32_t o2[16];
#pragma unroll
  for (int i = 0; i < 16; ++i)
    o2[i] = Half2<T>::pack(__uint_as_float(acc[2 * i]) * scale, __uint_as_float(acc[2 * i + 1]) * scale);
  if (vec_ok) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) d4[i] = make_uint4(o2[4 * i], o2[4 * i + 1], o2[4 * i + 2], o2[4 * i + 3]);
  } else {
    unsigned short* d0 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      d0[2 * i] = (unsigned short)(o2[i] & 0xffffu);
      d0[2 * i + 1] = (unsigned short)(o2[i] >> 16);
    }
  }
}

__device__ __forceinline__ bool pair_vec_ok(const oops_ta_pair& t) {
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && t.sb % 8 == 0 && t.sr % 8 == 0 && t.sc % 8 == 0 && t.sh % 8 == 0;
}

// ---------------------------------------------------------------------------------------------
// shared pieces of the three tensor kernels
// ---------------------------------------------------------------------------------------------
// 608 threads: warps 0-15 are four warpgroups of 128 threads that do the element-wise work, warp 16 is
// the TMA producer, warp 17 issues the score products (S, dP) and owns the tensor-memory allocation, warp 18
// issues the accumulating products (dQ, or dK and dV); the shared-bias kernel leaves warp 18 idle.  Two issuing
// threads keep the tensor core fed: neither kind of product waits behind the other's barrier.  The element-wise
// work of the reverse pass has no reduction along a score row, so the 64 columns of a step are split
// between two warpgroups that address the same tensor-memory lanes (warp % 4 selects the lanes).

constexpr int kProducerWarp = kElemWarps, kMmaWarp = kElemWarps + 1, kAccWarp = kElemWarps + 2;
constexpr int kDbProducerWarp = kDbElemWarps, kDbMmaWarp = kDbElemWarps + 1;

constexpr int kMaxKeepWords = 512;  // keep-bit table: one bit per key column, cols <= 16384

// Eight columns of the reverse-pass element math on packed f32 pairs:
//   p  = 2^(s * (scale*log2e) + bias * log2e + nl)        nl = -lse * log2e
//   ds = p * (dp + nd)                                     nd = -delta
// sraw/draw are the tensor-memory words of S and dP (adjacent columns form a pair), bias_chunk points at
// eight 16-bit bias values, nl2/nd2 hold the four (nl, nl') and (nd, nd') pairs of these columns.
template <typename T, bool HAS_BIAS>
__device__ __forceinline__ void score_grad8(const uint32_t* sraw, const uint32_t* draw, const uint8_t* bias_chunk, f32x2 c2,
                                            f32x2 log2e2, const f32x2* nl2, const f32x2* nd2, f32x2* p2, f32x2* ds2) {
  uint32_t bw[4] = {0, 0, 0, 0};
  if (HAS_BIAS) {
    const uint4 v = *reinterpret_cast<const uint4*>(bias_chunk);
    bw[0] = v.x; bw[1] = v.y; bw[2] = v.z; bw[3] = v.w;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const f32x2 s2 = pack2(__uint_as_float(sraw[2 * i]), __uint_as_float(sraw[2 * i + 1]));
    const f32x2 d2 = pack2(__uint_as_float(draw[2 * i]), __uint_as_float(draw[2 * i + 1]));
    const f32x2 offset = HAS_BIAS ? fma2(Half2<T>::widen(bw[i]), log2e2, nl2[i]) : nl2[i];
    float lo, hi;
    unpack2(fma2(s2, c2, offset), lo, hi);
    const f32x2 p = pack2(ex2(lo), ex2(hi));
    p2[i] = p;
    ds2[i] = mul2(p, add2(d2, nd2[i]));
  }
}

// Same with the eight bias values already in registers (four packed words).
template <typename T, bool HAS_BIAS>
__device__ __forceinline__ void score_grad8_words(const uint32_t* sraw, const uint32_t* draw, const uint4 bias_words, f32x2 c2,
                                                  f32x2 log2e2, f32x2 nl, f32x2 nd, f32x2* p2, f32x2* ds2) {
  const uint32_t bw[4] = {bias_words.x, bias_words.y, bias_words.z, bias_words.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const f32x2 s2 = pack2(__uint_as_float(sraw[2 * i]), __uint_as_float(sraw[2 * i + 1]));
    const f32x2 d2 = pack2(__uint_as_float(draw[2 * i]), __uint_as_float(draw[2 * i + 1]));
    const f32x2 offset = HAS_BIAS ? fma2(Half2<T>::widen(bw[i]), log2e2, nl) : nl;
    float lo, hi;
    unpack2(fma2(s2, c2, offset), lo, hi);
    const f32x2 p = pack2(ex2(lo), ex2(hi));
    p2[i] = p;
    ds2[i] = mul2(p, add2(d2, nd));
  }
}

__device__ __forceinline__ f32x2 select2(f32x2 v, uint32_t bits, int at) {
  float lo, hi;
  unpack2(v, lo, hi);
  if (((bits >> at) & 1u) == 0) lo = 0.f;
  if (((bits >> (at + 1)) & 1u) == 0) hi = 0.f;
  return pack2(lo, hi);
}

template <typename T>
__device__ __forceinline__ uint32_t pack16(f32x2 v) {
  float lo, hi;
  unpack2(v, lo, hi);
  return Half2<T>::pack(lo, hi);
}

// ---------------------------------------------------------------------------------------------
// dQ kernel
// ---------------------------------------------------------------------------------------------

struct DqSmem {
  static constexpr int q = 0;                                         // [tiles] 128 x 32
  static constexpr int dout = q + kTilesPerCta * kBigTile;            // [tiles] 128 x 32
  static constexpr int kv = dout + kTilesPerCta * kBigTile;           // [kRing] K step (4 KiB) + V step (4 KiB)
  static constexpr int bias = kv + kRing * 2 * kSmallTile;            // [tiles][2 buffers] 128 x 64
  static constexpr int bars = bias + 2 * kTilesPerCta * kBiasStep;
  static constexpr int qd_full = 0;                      // [2]
  static constexpr int kv_full = qd_full + 2;            // [kRing]
  static constexpr int kv_empty = kv_full + kRing;       // [kRing]
  static constexpr int k_ready = kv_empty + kRing;       // [kRing]
  static constexpr int bias_full = k_ready + kRing;      // [4]
  static constexpr int bias_empty = bias_full + 4;       // [4]
  static constexpr int sd_full = bias_empty + 4;         // [2] S and dP of a step are in tensor memory
  static constexpr int sd_free = sd_full + 2;            // [2] both have been read into registers
  static constexpr int ds_full = sd_free + 2;            // [2] dS (16-bit) is in tensor memory
  static constexpr int ds_done = ds_full + 2;            // [2] the dQ product has consumed it
  static constexpr int dq_done = ds_done + 2;            // [2] last dQ product finished
  static constexpr int num_bars = dq_done + 2;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int drop_flags = abort_flag + 4;  // [<= 16] per-warp: the mask drops a key of this row
  static constexpr int keep = drop_flags + 64;
  static constexpr int total = keep + kMaxKeepWords * 4;
};
constexpr int kDqSmemBytes = DqSmem::total + 1024;

struct DqParams {
  CUtensorMap map_q, map_dout, map_k, map_v, map_bias;
  oops_ta_pair dq;
  const float* lse;
  const float* delta;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  void* dbias_rows;  // per-row bias gradient (may be null)
  int64_t db_sb, db_sg, db_sh, db_sq, db_sk;
  int batch, rows, cols, heads, bias_groups;
  int q_pairs, k_steps;
  int write_dq;
  float scale;
};

template <typename T, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) ta_bwd_dq_kernel(const __grid_constant__ DqParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + DqSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + DqSmem::tmem_slot);
  uint32_t* keep_words = reinterpret_cast<uint32_t*>(smem_gen + DqSmem::keep);
  auto bar = [&](int index) -> uint32_t { return smem_base + DqSmem::bars + index * 8; };

  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  if (device_failed()) return;
  int idx = blockIdx.x;
  const int qp = idx % P.q_pairs;
  idx /= P.q_pairs;
  const int h = idx % P.heads;
  idx /= P.heads;
  const int r = idx % P.rows;
  const int b = idx / P.rows;
  const int q0 = qp * kTilesPerCta * kTile;
  const int n_tiles = (kTilesPerCta == 2 && q0 + kTile < P.cols) ? 2 : 1;
  const int KS = P.k_steps;
  const int g = P.bias_groups == 1 ? 0 : r;
  const bool has_mask = P.mask != nullptr;
  const bool has_bits = has_mask || (P.cols % kStep) != 0;
  // tensor-memory columns of query tile w: S [0,64) | dP [64,128) | dS [128,160) | dQ [160,192)
  constexpr int kTileCols = 192, kDpCol = 64, kDsCol = 128, kDqCol = 160;
  constexpr int kTmemCols = kTilesPerCta == 2 ? 512 : 256;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kTilesPerCta; ++i) {
      mbar_init(bar(DqSmem::qd_full + i), 1);
      mbar_init(bar(DqSmem::sd_full + i), 1);
      mbar_init(bar(DqSmem::sd_free + i), 8);
      mbar_init(bar(DqSmem::ds_full + i), 8);
      mbar_init(bar(DqSmem::ds_done + i), 1);
      mbar_init(bar(DqSmem::dq_done + i), 1);
    }
    for (int i = 0; i < kRing; ++i) {
      mbar_init(bar(DqSmem::kv_full + i), 1);
      mbar_init(bar(DqSmem::kv_empty + i), 1);
      mbar_init(bar(DqSmem::k_ready + i), 4);
    }
    for (int i = 0; i < 2 * kTilesPerCta; ++i) {
      mbar_init(bar(DqSmem::bias_full + i), 1);
      mbar_init(bar(DqSmem::bias_empty + i), 8);
    }
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_base + DqSmem::tmem_slot, kTmemCols);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // The keep-bit table is built after the CTA-wide barrier, by the element-wise warps, while the producer's first
  // copies are already in flight; only its users (those warps and the issuing warps) meet at a named barrier.
  uint32_t* drop_flags = reinterpret_cast<uint32_t*>(smem_gen + DqSmem::drop_flags);
  bool signoff = false;
  if (has_bits && warp != kProducerWarp) {
    if (warp < kElemWarps) {
      const uint8_t* mask_row = has_mask ? P.mask + b * P.m_sb + int64_t(r) * P.m_sr : nullptr;
      bool dropped_any = false;
      for (int word = warp; word < KS * 2; word += kElemWarps) {
        const int key = word * 32 + lane;
        bool keep = key < P.cols;
        if (keep && has_mask) {
          keep = mask_row[int64_t(key) * P.m_sc] != 0;
          dropped_any |= !keep;
        }
        const uint32_t bits = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) keep_words[word] = bits;
      }
      dropped_any = __any_sync(0xffffffffu, dropped_any);
      if (lane == 0) drop_flags[warp] = dropped_any ? 1u : 0u;
    }
    named_barrier_sync(1, kThreads - 32);
    // Key rows only need the sign-off handshake when the mask really drops a key of this row.
    if (has_mask) {
#pragma unroll
      for (int i = 0; i < kElemWarps; ++i) signoff |= drop_flags[i] != 0;
    }
  }

  if (warp == kProducerWarp) {
    if (lane == 0) {
      bool ok = true;
      for (int w = 0; w < n_tiles; ++w) {
        mbar_expect_tx(bar(DqSmem::qd_full + w), 2 * kBigTile);
        tma_load_5d(smem_base + DqSmem::q + w * kBigTile, &P.map_q, bar(DqSmem::qd_full + w), 0, h, q0 + w * kTile, r, b);
        tma_load_5d(smem_base + DqSmem::dout + w * kBigTile, &P.map_dout, bar(DqSmem::qd_full + w), 0, h, q0 + w * kTile, r, b);
      }
      for (int j = 0; j < KS && ok; ++j) {
        const int st = j % kRing, round = j / kRing;
        if (j >= kRing) ok = mbar_wait(bar(DqSmem::kv_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(DqSmem::kv_full + st), 2 * kSmallTile);
        const uint32_t dst = smem_base + DqSmem::kv + st * 2 * kSmallTile;
        tma_load_5d(dst, &P.map_k, bar(DqSmem::kv_full + st), 0, h, j * kStep, r, b);
        tma_load_5d(dst + kSmallTile, &P.map_v, bar(DqSmem::kv_full + st), 0, h, j * kStep, r, b);
        if (HAS_BIAS) {
          for (int w = 0; w < n_tiles && ok; ++w) {
            const int slot = w * 2 + (j & 1);
            if (j >= 2) ok = mbar_wait(bar(DqSmem::bias_empty + slot), ((j >> 1) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar(DqSmem::bias_full + slot), kBiasStep);
            tma_load_5d(smem_base + DqSmem::bias + slot * kBiasStep, &P.map_bias, bar(DqSmem::bias_full + slot), j * kStep,
                        q0 + w * kTile, h, g, b);
          }
        }
      }
    }
  } else if (warp == kMmaWarp || (kTilesPerCta == 2 && warp == kAccWarp)) {
    // One tile per CTA: one thread issues everything in the order the events arrive (scores of step j+1 when the
    // warpgroups have read step j, dQ of step j when they have stored dS).  Two tiles per CTA: a second thread issues
    // the dQ products, so that neither kind of product waits behind the other tile's barrier.
    if (lane == 0) {
      constexpr uint32_t fmt = Half2<T>::kFormat;
      constexpr uint32_t idesc_s = instr_desc(fmt, 0, 0, kTile, kStep);
      constexpr uint32_t idesc_dq = instr_desc(fmt, 0, 1, kTile, kHeadDim);
      const bool do_scores = warp == kMmaWarp, do_acc = kTilesPerCta == 1 || warp == kAccWarp;
      bool ok = true;
      // a K/V step is usable once the copy has landed and, with a mask, once warpgroup 0 has signed it off
      auto wait_step = [&](int j) -> bool {
        bool ready = mbar_wait(bar(DqSmem::kv_full + j % kRing), (j / kRing) & 1, abort_flag);
        if (ready && signoff) ready = mbar_wait(bar(DqSmem::k_ready + j % kRing), (j / kRing) & 1, abort_flag);
        return ready;
      };
      // S = Q K^T and dP = dO V^T of step j for query tile w (all operands K-major, 64-byte swizzle)
      auto issue_scores = [&](int j, int w) {
        // the bias tile of the step has landed before the scores are announced: the warpgroups do not wait for it
        if (HAS_BIAS && !mbar_wait(bar(DqSmem::bias_full + w * 2 + (j & 1)), (j >> 1) & 1, abort_flag)) return;
        const uint32_t kv = smem_base + DqSmem::kv + (j % kRing) * 2 * kSmallTile;
        const uint32_t s_t = tmem_base + w * kTileCols;
        const uint64_t qdesc = smem_desc(smem_base + DqSmem::q + w * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t ddesc = smem_desc(smem_base + DqSmem::dout + w * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t kdesc = smem_desc(kv, 16, 512, kSwizzle64B);
        const uint64_t vdesc = smem_desc(kv + kSmallTile, 16, 512, kSwizzle64B);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(s_t, qdesc + uint64_t(kk * 2), kdesc + uint64_t(kk * 2), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(s_t + kDpCol, ddesc + uint64_t(kk * 2), vdesc + uint64_t(kk * 2), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(bar(DqSmem::sd_full + w));
      };
      // dQ[128 x 32] += dS[128 x 64] K[64 x 32]; K is MN-major (channel contiguous).
      auto issue_dq = [&](int j, int w) {
        const int st = j % kRing;
        const uint32_t tile_t = tmem_base + w * kTileCols;
        const uint64_t kdesc = smem_desc(smem_base + DqSmem::kv + st * 2 * kSmallTile, 16, 512, kSwizzle64B);
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)
          mma_ts(tile_t + kDqCol, tile_t + kDsCol + kk * 8, kdesc + uint64_t(kk * (1024 >> 4)), idesc_dq,
                 (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(DqSmem::ds_done + w));
        if (j == KS - 1) mma_commit(bar(DqSmem::dq_done + w));
        if (w == n_tiles - 1) mma_commit(bar(DqSmem::kv_empty + st));
      };
      if (do_scores) {
        for (int w = 0; w < n_tiles && ok; ++w) ok = mbar_wait(bar(DqSmem::qd_full + w), 0, abort_flag);
        if (ok) ok = wait_step(0);
        if (ok) {
          tc_fence_after_sync();
          for (int w = 0; w < n_tiles; ++w) issue_scores(0, w);
        }
      }
      for (int j = 0; j < KS && ok; ++j) {
        if (do_scores && j + 1 < KS) {
          ok = wait_step(j + 1);
          for (int w = 0; w < n_tiles && ok; ++w) {
            ok = mbar_wait(bar(DqSmem::sd_free + w), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(j + 1, w);
          }
        }
        if (do_acc && ok) {
          if (!do_scores) ok = wait_step(j);
          for (int w = 0; w < n_tiles && ok; ++w) {
            ok = mbar_wait(bar(DqSmem::ds_full + w), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_dq(j, w);
          }
        }
      }
    }
  } else if (warp < kElemWarps && (warp >> 3) < n_tiles) {
    const int w = warp >> 3;          // query tile
    const int half = (warp >> 2) & 1; // which 32 of the step's 64 keys
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tile_t = tmem_base + lane_field + w * kTileCols;
    const int q_index = q0 + w * kTile + t;
    const bool q_valid = q_index < P.cols;
    const int64_t stat_at = ((int64_t(b) * P.rows + r) * P.heads + h) * P.cols + q_index;
    const float neg_lse2 = q_valid ? -P.lse[stat_at] * kLog2e : -INFINITY;
    const float delta = q_valid ? P.delta[stat_at] : 0.f;
    const float scale = P.scale;
    const f32x2 c2 = pack2(scale * kLog2e, scale * kLog2e), log2e2 = pack2(kLog2e, kLog2e);
    const f32x2 nl2[4] = {pack2(neg_lse2, neg_lse2), pack2(neg_lse2, neg_lse2), pack2(neg_lse2, neg_lse2), pack2(neg_lse2, neg_lse2)};
    const f32x2 nd2[4] = {pack2(-delta, -delta), pack2(-delta, -delta), pack2(-delta, -delta), pack2(-delta, -delta)};
    T* db_row = nullptr;
    bool db_vec = false;
    if (P.dbias_rows && q_valid) {
      db_row = reinterpret_cast<T*>(P.dbias_rows) + b * P.db_sb + int64_t(r) * P.db_sg + h * P.db_sh + int64_t(q_index) * P.db_sq;
      db_vec = P.db_sk == 1 && (reinterpret_cast<uintptr_t>(db_row) & 15) == 0;
    }
    bool ok = true;

    for (int j = 0; j < KS && ok; ++j) {
      uint32_t my_bits = 0xffffffffu;
      bool step_all_kept = true;
      if (has_bits) {
        const uint2 wds = *reinterpret_cast<const uint2*>(keep_words + j * 2);
        my_bits = half ? wds.y : wds.x;
        step_all_kept = (wds.x & wds.y) == 0xffffffffu;
        if (signoff && warp < 4) {
          // Key rows of dropped keys must not reach the dQ product (0 * inf): clear them in shared memory.
          const int st = j % kRing;
          if (!step_all_kept) {
            ok = mbar_wait(bar(DqSmem::kv_full + st), (j / kRing) & 1, abort_flag);
            if (!ok) break;
            const uint32_t word = (t < 32) ? wds.x : wds.y;
            if (t < kStep && ((word >> (t & 31)) & 1u) == 0) {
              uint4* row = reinterpret_cast<uint4*>(smem_gen + DqSmem::kv + st * 2 * kSmallTile + t * 64);
              row[0] = row[1] = row[2] = row[3] = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
          mbar_arrive_warp(bar(DqSmem::k_ready + st));
        }
      }
      ok = mbar_wait(bar(DqSmem::sd_full + w), j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sraw[32], draw[32];
      tmem_ld32(tile_t + half * 32, sraw);
      tmem_ld32(tile_t + kDpCol + half * 32, draw);
      tmem_wait_ld();
      tmem_loaded(sraw);
      tmem_loaded(draw);
      tc_fence_before_sync();
      mbar_arrive_warp(bar(DqSmem::sd_free + w));
      const int slot = w * 2 + (j & 1);
      const uint8_t* bias_row = smem_gen + DqSmem::bias + slot * kBiasStep + t * 128 + (((t & 7) ^ (half * 4)) << 4);
      uint32_t packed[16];
      const int key0 = j * kStep + half * 32;
#pragma unroll
      for (int i8 = 0; i8 < 4; ++i8) {
        f32x2 p2[4], ds2[4];
        score_grad8<T, HAS_BIAS>(sraw + i8 * 8, draw + i8 * 8, swizzled_chunk(bias_row, i8), c2, log2e2, nl2,
                                 nd2, p2, ds2);
        if (my_bits != 0xffffffffu) {
#pragma unroll
          for (int i = 0; i < 4; ++i) ds2[i] = select2(ds2[i], my_bits, i8 * 8 + 2 * i);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) packed[i8 * 4 + i] = pack16<T>(ds2[i]);
        if (db_row) {
          if (db_vec && key0 + 32 <= P.cols) {
            *reinterpret_cast<uint4*>(db_row + key0 + i8 * 8) =
                make_uint4(packed[i8 * 4], packed[i8 * 4 + 1], packed[i8 * 4 + 2], packed[i8 * 4 + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float lo, hi;
              unpack2(ds2[i], lo, hi);
              if (key0 + i8 * 8 + 2 * i < P.cols) db_row[int64_t(key0 + i8 * 8 + 2 * i) * P.db_sk] = T(lo);
              if (key0 + i8 * 8 + 2 * i + 1 < P.cols) db_row[int64_t(key0 + i8 * 8 + 2 * i + 1) * P.db_sk] = T(hi);
            }
          }
        }
      }
      if (HAS_BIAS) mbar_arrive_warp(bar(DqSmem::bias_empty + slot));
      if (j > 0) {
        // the dQ product of the previous step must have finished reading the dS columns
        ok = mbar_wait(bar(DqSmem::ds_done + w), (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
      }
      tmem_st16(tile_t + kDsCol + half * 16, packed);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(bar(DqSmem::ds_full + w));
    }

    if (ok) ok = mbar_wait(bar(DqSmem::dq_done + w), 0, abort_flag);
    if (ok && half == 0) {
      tc_fence_after_sync();
      uint32_t acc[32];
      tmem_ld32(tile_t + kDqCol, acc);
      tmem_wait_ld();
      tmem_loaded(acc);
      if (q_valid && P.write_dq) {
        T* dst = reinterpret_cast<T*>(P.dq.ptr) + b * P.dq.sb + int64_t(r) * P.dq.sr + int64_t(q_index) * P.dq.sc + h * P.dq.sh;
        store_row32<T>(dst, acc, scale, pair_vec_ok(P.dq));
      }
    }
  }
  teardown(abort_flag, tmem_base, kMmaWarp, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// dK / dV kernel (transposed: a thread owns a key)
// ---------------------------------------------------------------------------------------------

struct DkvSmem {
  static constexpr int k = 0;                                          // [tiles] 128 x 32
  static constexpr int v = k + kTilesPerCta * kBigTile;                // [tiles] 128 x 32
  static constexpr int qd = v + kTilesPerCta * kBigTile;               // [kRing] Q step (4 KiB) + dO step (4 KiB)
  static constexpr int bias = qd + kRing * 2 * kSmallTile;             // [tiles][2 buffers] 128 keys x 64 queries
  static constexpr int stats = bias + 2 * kTilesPerCta * kBiasStep;    // [warps][2 buffers][64 floats]: -lse*log2e | -delta
  static constexpr int bars = stats + 2 * kElemWarps * 256;
  static constexpr int kv_full = 0;                      // [2]
  static constexpr int qd_full = kv_full + 2;            // [kRing]
  static constexpr int qd_empty = qd_full + kRing;       // [kRing]
  static constexpr int bias_full = qd_empty + kRing;     // [4]
  static constexpr int bias_empty = bias_full + 4;       // [4]
  static constexpr int sd_full = bias_empty + 4;         // [2] S^T and dP^T of a step are in tensor memory
  static constexpr int sd_free = sd_full + 2;            // [2] both have been read into registers
  static constexpr int pds_full = sd_free + 2;           // [2] P^T and dS^T (16-bit) are in tensor memory
  static constexpr int pds_done = pds_full + 2;          // [2] the dV / dK products have consumed them
  static constexpr int done = pds_done + 2;              // [2]
  static constexpr int num_bars = done + 2;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int total = abort_flag + 4;
};
constexpr int kDkvSmemBytes = DkvSmem::total + 1024;

struct DkvParams {
  CUtensorMap map_k, map_v, map_q, map_dout, map_bias_t;
  oops_ta_pair dk, dv;
  const float* lse;
  const float* delta;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  int batch, rows, cols, heads, bias_groups;
  int k_pairs, q_steps;
  int write_dk, write_dv;
  float scale;
};

template <typename T, bool HAS_BIAS>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) ta_bwd_dkv_kernel(const __grid_constant__ DkvParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + DkvSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + DkvSmem::tmem_slot);
  auto bar = [&](int index) -> uint32_t { return smem_base + DkvSmem::bars + index * 8; };

  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  if (device_failed()) return;
  int idx = blockIdx.x;
  const int kp = idx % P.k_pairs;
  idx /= P.k_pairs;
  const int h = idx % P.heads;
  idx /= P.heads;
  const int r = idx % P.rows;
  const int b = idx / P.rows;
  const int k0 = kp * kTilesPerCta * kTile;
  const int n_tiles = (kTilesPerCta == 2 && k0 + kTile < P.cols) ? 2 : 1;
  const int QS = P.q_steps;
  const int g = P.bias_groups == 1 ? 0 : r;
  // tensor-memory columns of key tile w: S^T [0,64) | dP^T [64,128) | P^T [128,160) | dS^T [160,192) | dK [192,224) | dV [224,256)
  constexpr int kTileCols = 256, kDpCol = 64, kPCol = 128, kDsCol = 160, kDkCol = 192, kDvCol = 224;
  constexpr int kTmemCols = kTilesPerCta * kTileCols;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kTilesPerCta; ++i) {
      mbar_init(bar(DkvSmem::kv_full + i), 1);
      mbar_init(bar(DkvSmem::sd_full + i), 1);
      mbar_init(bar(DkvSmem::sd_free + i), 8);
      mbar_init(bar(DkvSmem::pds_full + i), 8);
      mbar_init(bar(DkvSmem::pds_done + i), 1);
      mbar_init(bar(DkvSmem::done + i), 1);
    }
    for (int i = 0; i < kRing; ++i) {
      mbar_init(bar(DkvSmem::qd_full + i), 1);
      mbar_init(bar(DkvSmem::qd_empty + i), 1);
    }
    for (int i = 0; i < 2 * kTilesPerCta; ++i) {
      mbar_init(bar(DkvSmem::bias_full + i), 1);
      mbar_init(bar(DkvSmem::bias_empty + i), 8);
    }
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_base + DkvSmem::tmem_slot, kTmemCols);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kProducerWarp) {
    if (lane == 0) {
      bool ok = true;
      for (int w = 0; w < n_tiles; ++w) {
        mbar_expect_tx(bar(DkvSmem::kv_full + w), 2 * kBigTile);
        tma_load_5d(smem_base + DkvSmem::k + w * kBigTile, &P.map_k, bar(DkvSmem::kv_full + w), 0, h, k0 + w * kTile, r, b);
        tma_load_5d(smem_base + DkvSmem::v + w * kBigTile, &P.map_v, bar(DkvSmem::kv_full + w), 0, h, k0 + w * kTile, r, b);
      }
      for (int j = 0; j < QS && ok; ++j) {
        const int st = j % kRing, round = j / kRing;
        if (j >= kRing) ok = mbar_wait(bar(DkvSmem::qd_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(DkvSmem::qd_full + st), 2 * kSmallTile);
        const uint32_t dst = smem_base + DkvSmem::qd + st * 2 * kSmallTile;
        tma_load_5d(dst, &P.map_q, bar(DkvSmem::qd_full + st), 0, h, j * kStep, r, b);
        tma_load_5d(dst + kSmallTile, &P.map_dout, bar(DkvSmem::qd_full + st), 0, h, j * kStep, r, b);
        if (HAS_BIAS) {
          for (int w = 0; w < n_tiles && ok; ++w) {
            const int slot = w * 2 + (j & 1);
            if (j >= 2) ok = mbar_wait(bar(DkvSmem::bias_empty + slot), ((j >> 1) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar(DkvSmem::bias_full + slot), kBiasStep);
            // transposed bias: inner axis = query, outer axis = key
            tma_load_5d(smem_base + DkvSmem::bias + slot * kBiasStep, &P.map_bias_t, bar(DkvSmem::bias_full + slot),
                        j * kStep, k0 + w * kTile, h, g, b);
          }
        }
      }
    }
  } else if (warp == kMmaWarp || (kTilesPerCta == 2 && warp == kAccWarp)) {
    // One tile per CTA: one thread issues everything in the order the events arrive (scores of step j+1 when the
    // warpgroups have read step j, dV and dK of step j when they have stored P and dS).  Two tiles per CTA: a second
    // thread issues the dV/dK products, so that neither kind of product waits behind the other tile's barrier.
    if (lane == 0) {
      constexpr uint32_t fmt = Half2<T>::kFormat;
      constexpr uint32_t idesc_s = instr_desc(fmt, 0, 0, kTile, kStep);
      constexpr uint32_t idesc_acc = instr_desc(fmt, 0, 1, kTile, kHeadDim);
      const bool do_scores = warp == kMmaWarp, do_acc = kTilesPerCta == 1 || warp == kAccWarp;
      bool ok = true;
      // S^T[128 k x 64 q] = K Q^T and dP^T = V dO^T of step j for key tile w
      auto issue_scores = [&](int j, int w) {
        // the bias tile of the step has landed before the scores are announced: the warpgroups do not wait for it
        if (HAS_BIAS && !mbar_wait(bar(DkvSmem::bias_full + w * 2 + (j & 1)), (j >> 1) & 1, abort_flag)) return;
        const uint32_t qd = smem_base + DkvSmem::qd + (j % kRing) * 2 * kSmallTile;
        const uint32_t st_t = tmem_base + w * kTileCols;
        const uint64_t kdesc = smem_desc(smem_base + DkvSmem::k + w * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t vdesc = smem_desc(smem_base + DkvSmem::v + w * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t qdesc = smem_desc(qd, 16, 512, kSwizzle64B);
        const uint64_t ddesc = smem_desc(qd + kSmallTile, 16, 512, kSwizzle64B);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(st_t, kdesc + uint64_t(kk * 2), qdesc + uint64_t(kk * 2), idesc_s, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(st_t + kDpCol, vdesc + uint64_t(kk * 2), ddesc + uint64_t(kk * 2), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(bar(DkvSmem::sd_full + w));
      };
      auto issue_acc = [&](int j, int w) {
        const int st = j % kRing;
        const uint32_t tile_t = tmem_base + w * kTileCols;
        const uint32_t qd = smem_base + DkvSmem::qd + st * 2 * kSmallTile;
        const uint64_t qdesc = smem_desc(qd, 16, 512, kSwizzle64B);                 // Q step, MN-major
        const uint64_t ddesc = smem_desc(qd + kSmallTile, 16, 512, kSwizzle64B);    // dO step, MN-major
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)  // dV[128 k x 32] += P^T[128 k x 64 q] dO[64 q x 32]
          mma_ts(tile_t + kDvCol, tile_t + kPCol + kk * 8, ddesc + uint64_t(kk * (1024 >> 4)), idesc_acc,
                 (j > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kStep / 16; ++kk)  // dK[128 k x 32] += dS^T[128 k x 64 q] Q[64 q x 32]
          mma_ts(tile_t + kDkCol, tile_t + kDsCol + kk * 8, qdesc + uint64_t(kk * (1024 >> 4)), idesc_acc,
                 (j > 0 || kk > 0) ? 1u : 0u);
        mma_commit(bar(DkvSmem::pds_done + w));
        if (j == QS - 1) mma_commit(bar(DkvSmem::done + w));
        if (w == n_tiles - 1) mma_commit(bar(DkvSmem::qd_empty + st));
      };
      if (do_scores) {
        for (int w = 0; w < n_tiles && ok; ++w) ok = mbar_wait(bar(DkvSmem::kv_full + w), 0, abort_flag);
        if (ok) ok = mbar_wait(bar(DkvSmem::qd_full), 0, abort_flag);
        if (ok) {
          tc_fence_after_sync();
          for (int w = 0; w < n_tiles; ++w) issue_scores(0, w);
        }
      }
      for (int j = 0; j < QS && ok; ++j) {
        if (do_scores && j + 1 < QS) {
          ok = mbar_wait(bar(DkvSmem::qd_full + (j + 1) % kRing), ((j + 1) / kRing) & 1, abort_flag);
          for (int w = 0; w < n_tiles && ok; ++w) {
            ok = mbar_wait(bar(DkvSmem::sd_free + w), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_scores(j + 1, w);
          }
        }
        if (do_acc && ok) {
          if (!do_scores) ok = mbar_wait(bar(DkvSmem::qd_full + j % kRing), (j / kRing) & 1, abort_flag);
          for (int w = 0; w < n_tiles && ok; ++w) {
            ok = mbar_wait(bar(DkvSmem::pds_full + w), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_acc(j, w);
          }
        }
      }
    }
  } else if (warp < kElemWarps && (warp >> 3) < n_tiles) {
    const int w = warp >> 3;           // key tile
    const int half = (warp >> 2) & 1;  // which 32 of the step's 64 queries
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const uint32_t tile_t = tmem_base + lane_field + w * kTileCols;
    const int key = k0 + w * kTile + t;
    bool keep = key < P.cols;
    if (keep && P.mask) keep = P.mask[b * P.m_sb + int64_t(r) * P.m_sr + int64_t(key) * P.m_sc] != 0;
    const float scale = P.scale;
    const f32x2 c2 = pack2(scale * kLog2e, scale * kLog2e), log2e2 = pack2(kLog2e, kLog2e);
    const int64_t stat_base = ((int64_t(b) * P.rows + r) * P.heads + h) * P.cols;
    bool ok = true;

    // Row statistics of the step's 32 queries of this warpgroup's half: every warp keeps its own copy in shared
    // memory (no cross-warp barrier): lane i fetches -lse*log2e and -delta of query i one step ahead.
    // The loaded words are not touched until the next step (any arithmetic on them here would wait for the load).
    auto fetch_stats = [&](int j, float& lse_raw, float& delta_raw) {
      lse_raw = INFINITY;
      delta_raw = 0.f;
      const int q = j * kStep + half * 32 + lane;
      if (j < QS && q < P.cols) {
        lse_raw = ldg_f32_here(P.lse + stat_base + q);
        delta_raw = ldg_f32_here(P.delta + stat_base + q);
      }
    };
    float nl_next, nd_next;
    fetch_stats(0, nl_next, nd_next);
    for (int j = 0; j < QS && ok; ++j) {
      float* stats = reinterpret_cast<float*>(smem_gen + DkvSmem::stats + (warp * 2 + (j & 1)) * 256);
      stats[lane] = -nl_next * kLog2e;
      stats[32 + lane] = -nd_next;
      fetch_stats(j + 1, nl_next, nd_next);
      __syncwarp();
      ok = mbar_wait(bar(DkvSmem::sd_full + w), j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      const int slot = w * 2 + (j & 1);
      const uint8_t* bias_row = smem_gen + DkvSmem::bias + slot * kBiasStep + t * 128 + (((t & 7) ^ (half * 4)) << 4);
      uint32_t p_packed[16], ds_packed[16];
      // two rounds of 16 queries keep the live registers low; the score columns are released after the second load
#pragma unroll
      for (int round = 0; round < 2; ++round) {
        uint32_t sraw[16], draw[16];
        tmem_ld16(tile_t + half * 32 + round * 16, sraw);
        tmem_ld16(tile_t + kDpCol + half * 32 + round * 16, draw);
        tmem_wait_ld();
        tmem_loaded(sraw);
        tmem_loaded(draw);
        if (round == 1) {
          tc_fence_before_sync();
          mbar_arrive_warp(bar(DkvSmem::sd_free + w));
        }
        if (keep) {
#pragma unroll
          for (int i8 = 0; i8 < 2; ++i8) {
            const int c8 = round * 2 + i8;  // which group of 8 queries of this half
            const float4 n01 = *reinterpret_cast<const float4*>(stats + c8 * 8);
            const float4 n23 = *reinterpret_cast<const float4*>(stats + c8 * 8 + 4);
            const float4 d01 = *reinterpret_cast<const float4*>(stats + 32 + c8 * 8);
            const float4 d23 = *reinterpret_cast<const float4*>(stats + 32 + c8 * 8 + 4);
            const f32x2 nl2[4] = {pack2(n01.x, n01.y), pack2(n01.z, n01.w), pack2(n23.x, n23.y), pack2(n23.z, n23.w)};
            const f32x2 nd2[4] = {pack2(d01.x, d01.y), pack2(d01.z, d01.w), pack2(d23.x, d23.y), pack2(d23.z, d23.w)};
            f32x2 p2[4], ds2[4];
            score_grad8<T, HAS_BIAS>(sraw + i8 * 8, draw + i8 * 8, swizzled_chunk(bias_row, c8), c2, log2e2,
                                     nl2, nd2, p2, ds2);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              p_packed[c8 * 4 + i] = pack16<T>(p2[i]);
              ds_packed[c8 * 4 + i] = pack16<T>(ds2[i]);
            }
          }
        } else {
          // a dropped (or out-of-range) key contributes nothing, whatever its row holds
#pragma unroll
          for (int i = 0; i < 8; ++i) p_packed[round * 8 + i] = ds_packed[round * 8 + i] = 0u;
        }
      }
      if (HAS_BIAS) mbar_arrive_warp(bar(DkvSmem::bias_empty + slot));
      if (j > 0) {
        ok = mbar_wait(bar(DkvSmem::pds_done + w), (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
      }
      tmem_st16(tile_t + kPCol + half * 16, p_packed);
      tmem_st16(tile_t + kDsCol + half * 16, ds_packed);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(bar(DkvSmem::pds_full + w));
    }

    if (ok) ok = mbar_wait(bar(DkvSmem::done + w), 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      uint32_t acc[32];
      if (half == 0 && P.write_dk) {
        tmem_ld32(tile_t + kDkCol, acc);
        tmem_wait_ld();
        tmem_loaded(acc);
        if (key < P.cols) {
          T* dst = reinterpret_cast<T*>(P.dk.ptr) + b * P.dk.sb + int64_t(r) * P.dk.sr + int64_t(key) * P.dk.sc + h * P.dk.sh;
          store_row32<T>(dst, acc, scale, pair_vec_ok(P.dk));
        }
      }
      if (half == 1 && P.write_dv) {
        tmem_ld32(tile_t + kDvCol, acc);
        tmem_wait_ld();
        tmem_loaded(acc);
        if (key < P.cols) {
          T* dst = reinterpret_cast<T*>(P.dv.ptr) + b * P.dv.sb + int64_t(r) * P.dv.sr + int64_t(key) * P.dv.sc + h * P.dv.sh;
          store_row32<T>(dst, acc, 1.f, pair_vec_ok(P.dv));
        }
      }
    }
  }
  teardown(abort_flag, tmem_base, kMmaWarp, kTmemCols);
}

// ---------------------------------------------------------------------------------------------
// fused dQ / dK / dV kernel: one pass over the score tiles of a pair row
// ---------------------------------------------------------------------------------------------
// CTA = (batch, row, head).  The row's query tiles are taken in groups of up to 6; for every group, every key tile and
// every query tile of the group: S = Q K^T and dP = dO V^T (128 x 128, tensor memory) -> the four warpgroups (a thread
// owns a query, a warpgroup 32 of the 128 keys) compute P and dS once and write them, 16-bit, into two shared-memory
// images whose rows are queries and whose 128-byte-swizzled columns are keys.  The tensor core reads those images three
// ways: dV += P^T dO and dK += dS^T Q take them as MN-major A operands (M = keys), dQ += dS K as a K-major A operand
// (M = queries).  dQ of the group's query tiles, dK and dV of the current key tile stay in tensor memory:
// S 128 | dP 128 | dK 32 | dV 32 | dQ 6 x 32 = 512 columns.  One `ex2` per logit and five products, where the
// separate dQ and dK/dV kernels spend two and seven.  The images cost shared-memory bandwidth (64 KB written and
// 96 KB read per 128 x 128 step), which is what bounds this kernel.
// Rows of more than 768 columns have several groups.  The CTA walks them in order and carries the f32 sums of dK and
// dV of every key tile from group to group in a scratch slot that belongs to its SM (one CTA is resident per SM, so
// the slot is private while the CTA runs, and at 128 bytes per key and tensor it stays in L2): the thread that owns a
// key adds what the slot holds, and stores 16-bit dK/dV after the last group.  The order of the sums is fixed, so the
// gradients are bitwise reproducible, and no partial planes or reduction kernels exist.

constexpr int kFMaxQTiles = 6;
constexpr int kFThreads = 608;  // 16 element-wise warps, TMA producer, score issuer, accumulation issuer
constexpr int kFProducerWarp = 16, kFScoreWarp = 17, kFAccWarp = 18;
constexpr int kFImage = 2 * 16384;       // P or dS of a step: two 64-key halves of 128 rows x 128 bytes
constexpr int kFBias = 2 * kBiasStep;    // 128 x 128 bias tile as two 64-key boxes (staging: copied to registers at once)
constexpr int kFKeepWords = 128;         // keep-bit table of a row
constexpr int kFSlots = 256;             // scratch slots of the group-to-group sums: one per SM id

struct FSmem {
  static constexpr int q = 0;                          // [3] 128 x 32 (a slot is held until the step's dK product ends)
  static constexpr int dout = q + 3 * kBigTile;        // [3]
  static constexpr int k = dout + 3 * kBigTile;        // [2]
  static constexpr int v = k + 2 * kBigTile;           // [2]
  static constexpr int ps = v + 2 * kBigTile;          // P image (read by the dV products only, freed early)
  static constexpr int dss = ps + kFImage;             // [2] dS image
  static constexpr int bias = dss + 2 * kFImage;       // one staging tile
  static constexpr int bars = bias + kFBias;
  static constexpr int qd_full = 0;                    // [3]
  static constexpr int qd_empty = qd_full + 3;         // [3]
  static constexpr int kv_full = qd_empty + 3;         // [2]
  static constexpr int kv_empty = kv_full + 2;         // [2]
  static constexpr int k_ready = kv_empty + 2;         // [2] dropped keys' rows cleared (only with a dropping mask)
  static constexpr int bias_full = k_ready + 2;
  static constexpr int bias_empty = bias_full + 1;     // every warp has copied its words of the tile to registers
  static constexpr int sd_full = bias_empty + 1;       // S and dP of a step are in tensor memory
  static constexpr int sd_free = sd_full + 1;          // all warps have read them
  static constexpr int pds_full = sd_free + 1;         // [2] the P and dS images of a buffer are written
  static constexpr int pds_done = pds_full + 2;        // [2] the dK and dQ products have consumed the dS image
  static constexpr int p_done = pds_done + 2;          // the dV products have consumed the P image
  static constexpr int dkv_free = p_done + 1;          // dK and dV of a finished key tile have been read out
  static constexpr int dq_free = dkv_free + 1;         // dQ of a finished group of query tiles has been read out
  static constexpr int num_bars = dq_free + 1;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int drop_flags = abort_flag + 4;    // [16]
  static constexpr int keep = drop_flags + 64;
  static constexpr int total = keep + kFKeepWords * 4;
};
constexpr int kFSmemBytes = FSmem::total + 1024;
static_assert(kFSmemBytes <= 232448, "fused reverse kernel: shared memory over the per-CTA limit");

struct FParams {
  CUtensorMap map_q, map_dout, map_k, map_v, map_bias;
  oops_ta_pair dq, dk, dv;
  float* slots;     // [kFSlots][2][8][slot_keys][4] f32: sums of dK and dV carried from group to group (groups > 1)
  int64_t slot_keys;
  const float* lse;
  const float* delta;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  int batch, rows, cols, heads, bias_groups;
  int q_tiles, k_tiles, groups, tiles_per_group;
  int write_dq, write_dk, write_dv;
  float scale;
};

// The walk over a pair row's steps, identical in every role of the kernel: groups of query tiles outermost, then key
// tiles, then the query tiles of the group.  Ring slots and barrier phases count steps and key tiles across groups.
struct FWalk {
  int tiles_per_group, q_tiles, k_tiles, groups;
  int g, kt, qi, nq;  // group, key tile, query tile within the group, query tiles of the group
  int s, ktc;         // steps and key tiles walked so far
  __device__ FWalk(const FParams& P)
      : tiles_per_group(P.tiles_per_group), q_tiles(P.q_tiles), k_tiles(P.k_tiles), groups(P.groups), g(0), kt(0), qi(0),
        nq(min(P.tiles_per_group, P.q_tiles)), s(0), ktc(0) {}
  __device__ bool done() const { return g >= groups; }
  __device__ int qt() const { return g * tiles_per_group + qi; }
  __device__ void next() {
    ++s;
    if (++qi < nq) return;
    qi = 0;
    ++ktc;
    if (++kt < k_tiles) return;
    kt = 0;
    ++g;
    nq = min(tiles_per_group, q_tiles - g * tiles_per_group);
  }
};

template <typename T, bool HAS_BIAS>
__global__ void __launch_bounds__(kFThreads, 1) ta_bwd_fused_kernel(const __grid_constant__ FParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + FSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + FSmem::tmem_slot);
  uint32_t* keep_words = reinterpret_cast<uint32_t*>(smem_gen + FSmem::keep);
  auto bar = [&](int index) -> uint32_t { return smem_base + FSmem::bars + index * 8; };

  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  if (device_failed()) return;
  int idx = blockIdx.x;
  const int h = idx % P.heads;
  idx /= P.heads;
  const int r = idx % P.rows;
  const int b = idx / P.rows;
  const int KT = P.k_tiles;
  const int bias_group = P.bias_groups == 1 ? 0 : r;
  const bool has_mask = P.mask != nullptr;
  const bool has_bits = has_mask || (P.cols % kTile) != 0;
  // tensor-memory columns
  constexpr int kSCol = 0, kDpCol = 128, kDkCol = 256, kDvCol = 288, kDqCol = 320;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 3; ++i) {
      mbar_init(bar(FSmem::qd_full + i), 1);
      mbar_init(bar(FSmem::qd_empty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(FSmem::pds_full + i), 16);
      mbar_init(bar(FSmem::pds_done + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(FSmem::kv_full + i), 1);
      mbar_init(bar(FSmem::kv_empty + i), 1);
      mbar_init(bar(FSmem::k_ready + i), 4);
    }
    mbar_init(bar(FSmem::p_done), 1);
    mbar_init(bar(FSmem::bias_full), 1);
    mbar_init(bar(FSmem::bias_empty), 16);
    mbar_init(bar(FSmem::sd_full), 1);
    mbar_init(bar(FSmem::sd_free), 16);
    mbar_init(bar(FSmem::dkv_free), 8);
    mbar_init(bar(FSmem::dq_free), 16);
    fence_barrier_init();
  }
  if (warp == kFScoreWarp) {
    tmem_alloc(smem_base + FSmem::tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // keep-bit table (one bit per key of this pair row), built by the element-wise warps while the first copies fly
  uint32_t* drop_flags = reinterpret_cast<uint32_t*>(smem_gen + FSmem::drop_flags);
  bool signoff = false;
  if (has_bits && warp != kFProducerWarp) {
    if (warp < 16) {
      const uint8_t* mask_row = has_mask ? P.mask + b * P.m_sb + int64_t(r) * P.m_sr : nullptr;
      bool dropped_any = false;
      for (int word = warp; word < KT * 4; word += 16) {
        const int key = word * 32 + lane;
        bool keep = key < P.cols;
        if (keep && has_mask) {
          keep = mask_row[int64_t(key) * P.m_sc] != 0;
          dropped_any |= !keep;
        }
        const uint32_t bits = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) keep_words[word] = bits;
      }
      dropped_any = __any_sync(0xffffffffu, dropped_any);
      if (lane == 0) drop_flags[warp] = dropped_any ? 1u : 0u;
    }
    named_barrier_sync(1, kFThreads - 32);
    if (has_mask) {
#pragma unroll
      for (int i = 0; i < 16; ++i) signoff |= drop_flags[i] != 0;
    }
  }

  if (warp == kFProducerWarp) {
    if (lane == 0) {
      bool ok = true;
      for (FWalk w(P); !w.done() && ok; w.next()) {
        const int s = w.s, kt = w.kt, qt = w.qt(), qs = s % 3;
        if (w.qi == 0) {
          const int ks = w.ktc & 1;
          if (w.ktc >= 2) ok = mbar_wait(bar(FSmem::kv_empty + ks), ((w.ktc >> 1) - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar(FSmem::kv_full + ks), 2 * kBigTile);
          tma_load_5d(smem_base + FSmem::k + ks * kBigTile, &P.map_k, bar(FSmem::kv_full + ks), 0, h, kt * kTile, r, b);
          tma_load_5d(smem_base + FSmem::v + ks * kBigTile, &P.map_v, bar(FSmem::kv_full + ks), 0, h, kt * kTile, r, b);
        }
        if (s >= 3) ok = mbar_wait(bar(FSmem::qd_empty + qs), ((s / 3) - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(FSmem::qd_full + qs), 2 * kBigTile);
        tma_load_5d(smem_base + FSmem::q + qs * kBigTile, &P.map_q, bar(FSmem::qd_full + qs), 0, h, qt * kTile, r, b);
        tma_load_5d(smem_base + FSmem::dout + qs * kBigTile, &P.map_dout, bar(FSmem::qd_full + qs), 0, h, qt * kTile, r, b);
        if (HAS_BIAS) {
          if (s >= 1) ok = mbar_wait(bar(FSmem::bias_empty), (s - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bar(FSmem::bias_full), kFBias);
          for (int box = 0; box < 2; ++box)
            tma_load_5d(smem_base + FSmem::bias + box * kBiasStep, &P.map_bias, bar(FSmem::bias_full), kt * kTile + box * 64,
                        qt * kTile, h, bias_group, b);
        }
      }
    }
  } else if (warp == kFScoreWarp) {
    {
      constexpr uint32_t idesc = instr_desc(Half2<T>::kFormat, 0, 0, kTile, kTile);
      bool ok = true;
      for (FWalk w(P); !w.done() && ok; w.next()) {
        const int s = w.s, qs = s % 3, ks = w.ktc & 1;
        ok = mbar_wait_warp(bar(FSmem::qd_full + qs), (s / 3) & 1, abort_flag);
        if (ok && w.qi == 0) {
          ok = mbar_wait_warp(bar(FSmem::kv_full + ks), (w.ktc >> 1) & 1, abort_flag);
          if (ok && signoff) ok = mbar_wait_warp(bar(FSmem::k_ready + ks), (w.ktc >> 1) & 1, abort_flag);
        }
        if (ok && s > 0) ok = mbar_wait_warp(bar(FSmem::sd_free), (s - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t qdesc = smem_desc(smem_base + FSmem::q + qs * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t ddesc = smem_desc(smem_base + FSmem::dout + qs * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t kdesc = smem_desc(smem_base + FSmem::k + ks * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t vdesc = smem_desc(smem_base + FSmem::v + ks * kBigTile, 16, 512, kSwizzle64B);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss_warp(tmem_base + kSCol, qdesc + uint64_t(kk * 2), kdesc + uint64_t(kk * 2), idesc, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss_warp(tmem_base + kDpCol, ddesc + uint64_t(kk * 2), vdesc + uint64_t(kk * 2), idesc, kk > 0 ? 1u : 0u);
        mma_commit_warp(bar(FSmem::sd_full));
      }
    }
  } else if (warp == kFAccWarp) {
    {
      constexpr uint32_t fmt = Half2<T>::kFormat;
      constexpr uint32_t idesc_t = instr_desc(fmt, 1, 1, kTile, kHeadDim);  // A = image^T (M = keys), B MN-major
      constexpr uint32_t idesc_q = instr_desc(fmt, 0, 1, kTile, kHeadDim);  // A = image (M = queries), B MN-major
      bool ok = true;
      for (FWalk w(P); !w.done() && ok; w.next()) {
        const int s = w.s, kt = w.kt, qi = w.qi, qs = s % 3, ks = w.ktc & 1;
        ok = mbar_wait_warp(bar(FSmem::qd_full + qs), (s / 3) & 1, abort_flag);
        if (ok) ok = mbar_wait_warp(bar(FSmem::kv_full + ks), (w.ktc >> 1) & 1, abort_flag);
        if (ok) ok = mbar_wait_warp(bar(FSmem::pds_full + (s & 1)), (s >> 1) & 1, abort_flag);
        // dK and dV of the previous key tile must have been read out before they are overwritten,
        // and so must dQ of the previous group of query tiles
        if (ok && qi == 0 && w.ktc > 0) ok = mbar_wait_warp(bar(FSmem::dkv_free), (w.ktc - 1) & 1, abort_flag);
        if (ok && qi == 0 && kt == 0 && w.g > 0) ok = mbar_wait_warp(bar(FSmem::dq_free), (w.g - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t ps = smem_base + FSmem::ps, dss = smem_base + FSmem::dss + (s & 1) * kFImage;
        const uint64_t qdesc = smem_desc(smem_base + FSmem::q + qs * kBigTile, 16, 512, kSwizzle64B);     // MN-major B
        const uint64_t ddesc = smem_desc(smem_base + FSmem::dout + qs * kBigTile, 16, 512, kSwizzle64B);  // MN-major B
        const uint64_t kdesc = smem_desc(smem_base + FSmem::k + ks * kBigTile, 16, 512, kSwizzle64B);       // MN-major B
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)  // dV[128 k x 32] += P^T[128 k x 128 q] dO[128 q x 32]
          mma_ss_warp(tmem_base + kDvCol, smem_desc(ps + kk * 2048, 16384, 1024, kSwizzle128B), ddesc + uint64_t(kk * (1024 >> 4)),
                 idesc_t, (qi > 0 || kk > 0) ? 1u : 0u);
        mma_commit_warp(bar(FSmem::p_done));
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)  // dK[128 k x 32] += dS^T[128 k x 128 q] Q[128 q x 32]
          mma_ss_warp(tmem_base + kDkCol, smem_desc(dss + kk * 2048, 16384, 1024, kSwizzle128B), qdesc + uint64_t(kk * (1024 >> 4)),
                 idesc_t, (qi > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kTile / 16; ++kk)  // dQ[128 q x 32] += dS[128 q x 128 k] K[128 k x 32]
          mma_ss_warp(tmem_base + kDqCol + qi * kHeadDim, smem_desc(dss + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024, kSwizzle128B),
                 kdesc + uint64_t(kk * (1024 >> 4)), idesc_q, (kt > 0 || kk > 0) ? 1u : 0u);
        mma_commit_warp(bar(FSmem::pds_done + (s & 1)));
        mma_commit_warp(bar(FSmem::qd_empty + qs));
        if (qi == w.nq - 1) mma_commit_warp(bar(FSmem::kv_empty + ks));
      }
    }
  } else if (warp < 16) {
    const int wg = warp >> 2;  // 32 of the step's 128 keys
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const uint32_t lanes_t = tmem_base + lane_field;
    const float scale = P.scale;
    const f32x2 c2 = pack2(scale * kLog2e, scale * kLog2e), log2e2 = pack2(kLog2e, kLog2e);
    const int64_t stat_base = ((int64_t(b) * P.rows + r) * P.heads + h) * P.cols;
    // statistics of this thread's query in a step's query tile, fetched one step ahead and left untouched till then
    auto fetch_stats = [&](const FWalk& at, float& lse_raw, float& delta_raw) {
      lse_raw = INFINITY;
      delta_raw = 0.f;
      const int q = at.qt() * kTile + t;
      if (!at.done() && q < P.cols) {
        lse_raw = ldg_f32_here(P.lse + stat_base + q);
        delta_raw = ldg_f32_here(P.delta + stat_base + q);
      }
    };
    uint32_t sm_id;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_id));
    // dK (warpgroup 0) and dV (warpgroup 1) of key tile kt, complete for the query tiles of group g: lanes are keys.
    // With several groups the f32 sums travel from group to group through this SM's scratch slot (the same thread
    // owns a key in every group), and the last group stores the 16-bit result.
    auto store_key_tile = [&](int g, int kt) {
      if (wg > 1) return;
      uint32_t acc[32];
      tmem_ld32(lanes_t + (wg == 0 ? kDkCol : kDvCol), acc);
      tmem_wait_ld();
      tmem_loaded(acc);
      tc_fence_before_sync();
      mbar_arrive_warp(bar(FSmem::dkv_free));
      const int key = kt * kTile + t;
      if (key >= P.cols) return;
      const bool wanted = wg == 0 ? P.write_dk != 0 : P.write_dv != 0;
      if (!wanted) return;
      if (P.groups > 1) {
        // plane i of the slot holds channels 4i .. 4i+3 of every key, so that a warp's 32 keys are 512 contiguous bytes
        float4* slot = reinterpret_cast<float4*>(P.slots) + (int64_t(sm_id) * 2 + wg) * 8 * P.slot_keys + key;
        if (g == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            slot[i * P.slot_keys] = make_float4(__uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                                                __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            red_add_f4(slot + i * P.slot_keys, __uint_as_float(acc[4 * i]), __uint_as_float(acc[4 * i + 1]),
                       __uint_as_float(acc[4 * i + 2]), __uint_as_float(acc[4 * i + 3]));
        }
        return;
      }
      const oops_ta_pair& o = wg == 0 ? P.dk : P.dv;
      T* dst = reinterpret_cast<T*>(o.ptr) + b * o.sb + int64_t(r) * o.sr + int64_t(key) * o.sc + h * o.sh;
      store_row32<T>(dst, acc, wg == 0 ? scale : 1.f, pair_vec_ok(o));
    };
    // dQ of the query tiles of group g (tile qi is read out by warpgroup qi % 4; lanes are queries); every warp then
    // reports that the accumulators may be overwritten by the next group
    auto store_query_tiles = [&](int g) {
      const int tiles = min(P.tiles_per_group, P.q_tiles - g * P.tiles_per_group);
      for (int qi = wg; qi < tiles; qi += 4) {
        uint32_t acc[32];
        tmem_ld32(lanes_t + kDqCol + qi * kHeadDim, acc);
        tmem_wait_ld();
        tmem_loaded(acc);
        const int q_index = (g * P.tiles_per_group + qi) * kTile + t;
        if (q_index < P.cols && P.write_dq) {
          T* dst = reinterpret_cast<T*>(P.dq.ptr) + b * P.dq.sb + int64_t(r) * P.dq.sr + int64_t(q_index) * P.dq.sc + h * P.dq.sh;
          store_row32<T>(dst, acc, scale, pair_vec_ok(P.dq));
        }
      }
      tc_fence_before_sync();
      mbar_arrive_warp(bar(FSmem::dq_free));
    };
    FWalk w(P);
    float lse_next, delta_next;
    fetch_stats(w, lse_next, delta_next);
    bool ok = true;
    if (P.groups > 1 && sm_id >= uint32_t(kFSlots)) {  // no scratch slot for this SM id: give up like a wait that ran out
      *abort_flag = 1;
      ok = false;
    }

    // bias row of this thread's query in the staging tile: box (wg >> 1), 16-byte chunks (wg & 1) * 4 .. + 3
    const uint8_t* bias_row = smem_gen + FSmem::bias + (wg >> 1) * kBiasStep + t * 128 + (((t & 7) ^ ((wg & 1) * 4)) << 4);

    int last_g = 0, last_kt = 0;  // group and key tile of the previous step
    for (; !w.done() && ok; last_g = w.g, last_kt = w.kt, w.next()) {
      const int s = w.s, kt = w.kt, qi = w.qi, buf = s & 1;
      if (s > 0) {
        // The images of step s - 1 are handed to the products only now: their stores have drained under the read-out
        // and the loop's turn-around, and the fence stands before anything this step requests, so it does not wait;
        // the accumulating issuer has slack to spare.
        fence_proxy_async_smem();
        mbar_arrive_warp(bar(FSmem::pds_full + (buf ^ 1)));
      }
      // The three phases the step needs first are probed together (one round trip to the barrier words); in the steady
      // state, where these warps are the slow side of the pipeline, all three are complete.
      const bool bias_there = HAS_BIAS && mbar_test(bar(FSmem::bias_full), s & 1);
      const bool image_free = s < 2 || mbar_test(bar(FSmem::pds_done + buf), ((s >> 1) - 1) & 1);
      const bool scores_there = mbar_test(bar(FSmem::sd_full), s & 1);
      const float neg_lse2 = -lse_next * kLog2e, neg_delta = -delta_next;
      {
        FWalk ahead = w;
        ahead.next();
        fetch_stats(ahead, lse_next, delta_next);
      }
      const f32x2 nl1 = pack2(neg_lse2, neg_lse2), nd1 = pack2(neg_delta, neg_delta);
      const uint32_t bits = has_bits ? keep_words[kt * 4 + wg] : 0xffffffffu;
      // The step's bias words are requested at once; the staging tile is handed back as soon as they have arrived
      // (below, after the first scores have been fetched), so that the next tile's copy runs under this step's arithmetic.
      uint4 bias_words[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
      if (HAS_BIAS) {
        ok = mbar_wait_probed(bias_there, bar(FSmem::bias_full), s & 1, abort_flag);
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < 4; ++c) bias_words[c] = lds_v4_here(swizzled_chunk(bias_row, c));
      }
      if (signoff && qi == 0 && warp < 4) {
        // key rows of dropped keys must not reach the dQ product (0 * inf): clear them in shared memory
        const int ks = w.ktc & 1;
        ok = mbar_wait(bar(FSmem::kv_full + ks), (w.ktc >> 1) & 1, abort_flag);
        if (!ok) break;
        if (((keep_words[kt * 4 + (t >> 5)] >> (t & 31)) & 1u) == 0) {
          uint4* row = reinterpret_cast<uint4*>(smem_gen + FSmem::k + ks * kBigTile + t * 64);
          row[0] = row[1] = row[2] = row[3] = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        mbar_arrive_warp(bar(FSmem::k_ready + ks));
      }
      // this step's dS image was last read by the products of step s - 2, the P image by the dV products of s - 1
      ok = mbar_wait_probed(image_free, bar(FSmem::pds_done + buf), ((s >> 1) - 1) & 1, abort_flag);
      if (ok) ok = mbar_wait_probed(scores_there, bar(FSmem::sd_full), s & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      // image rows are queries; this warpgroup's 32 keys are chunks (wg & 1) * 4 .. + 3 of half (wg >> 1)
      const int row_at = (wg >> 1) * 16384 + t * 128 + (((t & 7) ^ ((wg & 1) * 4)) << 4);
      uint8_t* p_row = smem_gen + FSmem::ps + row_at;
      uint8_t* ds_row = smem_gen + FSmem::dss + buf * kFImage + row_at;
      uint32_t p_packed[16];
      // Eight columns of S and dP at a time; the next eight are requested as soon as the current ones have arrived
      // and travel under the current eight's arithmetic.
      uint32_t sraw[2][8], draw[2][8];
      bool p_free = s < 1;
      tmem_ld8(lanes_t + kSCol + wg * 32, sraw[0]);
      tmem_ld8(lanes_t + kDpCol + wg * 32, draw[0]);
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        tmem_wait_ld();
        tmem_loaded(sraw[c8 & 1]);
        tmem_loaded(draw[c8 & 1]);
        if (c8 == 0 && HAS_BIAS) {
          // the bias words must have returned before the tile is handed back (the copy of the next tile may land at once)
#pragma unroll
          for (int c = 0; c < 4; ++c)
            asm volatile("" ::"r"(bias_words[c].x), "r"(bias_words[c].y), "r"(bias_words[c].z), "r"(bias_words[c].w) : "memory");
          mbar_arrive_warp(bar(FSmem::bias_empty));
        }
        if (c8 < 3) {
          tmem_ld8(lanes_t + kSCol + wg * 32 + (c8 + 1) * 8, sraw[(c8 + 1) & 1]);
          tmem_ld8(lanes_t + kDpCol + wg * 32 + (c8 + 1) * 8, draw[(c8 + 1) & 1]);
        } else {
          tc_fence_before_sync();
          mbar_arrive_warp(bar(FSmem::sd_free));
          // the P image's phase is probed here; the answer travels under the last eight columns' arithmetic
          if (s >= 1) p_free = mbar_test(bar(FSmem::p_done), (s - 1) & 1);
        }
        f32x2 p2[4], ds2[4];
        score_grad8_words<T, HAS_BIAS>(sraw[c8 & 1], draw[c8 & 1], bias_words[c8], c2, log2e2, nl1, nd1, p2, ds2);
        if (bits != 0xffffffffu) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            p2[i] = select2(p2[i], bits, c8 * 8 + 2 * i);
            ds2[i] = select2(ds2[i], bits, c8 * 8 + 2 * i);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) p_packed[c8 * 4 + i] = pack16<T>(p2[i]);
        *reinterpret_cast<uint4*>(const_cast<uint8_t*>(swizzled_chunk(ds_row, c8))) =
            make_uint4(pack16<T>(ds2[0]), pack16<T>(ds2[1]), pack16<T>(ds2[2]), pack16<T>(ds2[3]));
      }
      // the single P image is free once the dV products of the previous step have read it; by now they have
      ok = mbar_wait_probed(p_free, bar(FSmem::p_done), (s - 1) & 1, abort_flag);
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(const_cast<uint8_t*>(swizzled_chunk(p_row, c))) =
            make_uint4(p_packed[4 * c], p_packed[4 * c + 1], p_packed[4 * c + 2], p_packed[4 * c + 3]);
      if (qi == 0 && s > 0) {
        // A new key tile: dK and dV of the previous one are complete once the products of step s - 1 are (a commit
        // covers every product issued before it); a new group also finds its predecessor's dQ complete.  The products
        // of step s, which overwrite these accumulators, are issued after this step's images have been handed over,
        // which happens at the top of the next step: they wait for the read-out through dkv_free / dq_free only.
        ok = mbar_wait(bar(FSmem::pds_done + ((s - 1) & 1)), ((s - 1) >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        store_key_tile(last_g, last_kt);
        if (kt == 0) store_query_tiles(last_g);
      }
    }
    const int steps = w.s;
    if (ok && steps > 0) {  // the images of the last step
      fence_proxy_async_smem();
      mbar_arrive_warp(bar(FSmem::pds_full + ((steps - 1) & 1)));
    }

    // every product has finished when the products of the last step have
    if (ok && steps > 0) ok = mbar_wait(bar(FSmem::pds_done + ((steps - 1) & 1)), ((steps - 1) >> 1) & 1, abort_flag);
    if (ok && steps > 0) {
      tc_fence_after_sync();
      store_key_tile(P.groups - 1, KT - 1);
      store_query_tiles(P.groups - 1);
    }
    if (P.groups > 1) {
      // The row's dK and dV now stand complete in this SM's slot (f32, summed group by group in a fixed order by the
      // thread that owns the key).  Every warp passes the barrier, whatever became of its waits; the 16-bit rows are
      // then written by all of them: four lanes share a key, so a warp stores eight 64-byte rows per instruction.
      __threadfence();
      named_barrier_sync(2, 16 * 32);
      if (*abort_flag == 0) {
        const int items = 2 * P.cols * 4;  // (tensor, key, eight channels)
        for (int item = tid; item < items; item += 16 * 32) {
          const int j = item & 3, key = (item >> 2) % P.cols, which = (item >> 2) / P.cols;
          const bool wanted = which == 0 ? P.write_dk != 0 : P.write_dv != 0;
          if (!wanted) continue;
          const float4* slot = reinterpret_cast<const float4*>(P.slots) + (int64_t(sm_id) * 2 + which) * 8 * P.slot_keys + key;
          const float4 lo = ldcg_f4(slot + (2 * j) * P.slot_keys), hi = ldcg_f4(slot + (2 * j + 1) * P.slot_keys);
          const float f = which == 0 ? scale : 1.f;
          const oops_ta_pair& o = which == 0 ? P.dk : P.dv;
          T* dst = reinterpret_cast<T*>(o.ptr) + b * o.sb + int64_t(r) * o.sr + int64_t(key) * o.sc + h * o.sh + j * 8;
          const uint32_t w0 = Half2<T>::pack(lo.x * f, lo.y * f), w1 = Half2<T>::pack(lo.z * f, lo.w * f);
          const uint32_t w2 = Half2<T>::pack(hi.x * f, hi.y * f), w3 = Half2<T>::pack(hi.z * f, hi.w * f);
          if (pair_vec_ok(o)) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w0, w1, w2, w3);
          } else {
            unsigned short* d0 = reinterpret_cast<unsigned short*>(dst);
            const uint32_t ws[4] = {w0, w1, w2, w3};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              d0[2 * i] = (unsigned short)(ws[i] & 0xffffu);
              d0[2 * i + 1] = (unsigned short)(ws[i] >> 16);
            }
          }
        }
      }
    }
  }
  teardown(abort_flag, tmem_base, kFScoreWarp);
}

// ---------------------------------------------------------------------------------------------
// shared-bias gradient kernel
// ---------------------------------------------------------------------------------------------
// dBias[b, h, q, k] = sum over rows r of dS[b, r, h, q, k].  The sum runs over the rows, so this kernel's loop nest has
// the rows innermost: a CTA owns one 128-query x 128-key tile of one (batch, head) and walks the rows of its part.
// Per row the tensor core produces S = Q K^T and dP = dO V^T (two 128 x 128 x 32 products, full-rate N = 128
// instructions, double-buffered in all 512 tensor-memory columns) and the sixteen element-wise warps (a thread owns
// one query and 32 of the tile's keys) add dS into f32 registers.  Everything that does not depend on the row stays
// in registers for the whole kernel: the thread's 32 bias values, already multiplied by log2(e), and the running
// sums.  Per logit the loop then costs one packed add (bias - lse), one packed multiply-add (exponent), `ex2`, one
// packed add (dP - delta) and one packed multiply-add (sum += P (dP - delta)).  A compile-time share of the `ex2`
// runs as a polynomial on the FMA pipe.  With enough tiles to fill the SMs there is a single part and the CTA stores
// the final 16-bit gradient itself; small problems split the rows into parts whose f32 planes a last kernel adds in a
// fixed order (no atomics, bitwise reproducible either way).

constexpr int kDbRing = 4;
constexpr int kDbStage = 4 * kBigTile;  // Q | dO | K | V of one row: 128 x 32 each
#ifndef TA_DB_POLY_EVERY
#define TA_DB_POLY_EVERY 0
#endif
constexpr int kDbPolyEvery = TA_DB_POLY_EVERY;  // every n-th pair of a thread's logits takes the polynomial exp2 (0: none)
struct DbSmem {
  static constexpr int bias = 0;                         // 128 queries x 128 keys as two 64-key boxes (prologue only)
  static constexpr int ring = bias + 2 * kBiasStep;      // [kDbRing] stages
  static constexpr int bars = ring + kDbRing * kDbStage;
  static constexpr int bias_full = 0;
  static constexpr int row_full = 1;                     // [kDbRing]
  static constexpr int row_empty = row_full + kDbRing;   // [kDbRing]
  static constexpr int sd_full = row_empty + kDbRing;    // [2]
  static constexpr int sd_free = sd_full + 2;            // [2]
  static constexpr int num_bars = sd_free + 2;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int total = abort_flag + 4;
};
constexpr int kDbSmemBytes = DbSmem::total + 1024;
static_assert(kDbSmemBytes <= 232448, "shared-bias kernel: shared memory over the per-CTA limit");

struct DbParams {
  CUtensorMap map_q, map_dout, map_k, map_v, map_bias;
  float* parts;  // [parts][batch][heads][cols][cols] f32 (num_parts > 1)
  void* dbias;   // final gradient (num_parts == 1): the bias type, or f32 when dbias_f32 is set
  int64_t db_sb, db_sh, db_sq, db_sk;
  int dbias_f32;
  const float* lse;
  const float* delta;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  int batch, rows, cols, heads;
  int tiles, num_parts, rows_per_part;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kDbThreads, 1) ta_bwd_dbias_kernel(const __grid_constant__ DbParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + DbSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + DbSmem::tmem_slot);
  auto bar = [&](int index) -> uint32_t { return smem_base + DbSmem::bars + index * 8; };

  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  if (device_failed()) return;
  int idx = blockIdx.x;
  const int kt = idx % P.tiles;
  idx /= P.tiles;
  const int qt = idx % P.tiles;
  idx /= P.tiles;
  const int h = idx % P.heads;
  idx /= P.heads;
  const int b = idx % P.batch;
  const int part = idx / P.batch;
  const int row_lo = part * P.rows_per_part;
  const int row_hi = min(P.rows, row_lo + P.rows_per_part);
  const int n_rows = max(0, row_hi - row_lo);
  const bool has_mask = P.mask != nullptr;

  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar(DbSmem::bias_full), 1);
    for (int i = 0; i < kDbRing; ++i) {
      mbar_init(bar(DbSmem::row_full + i), 1);
      mbar_init(bar(DbSmem::row_empty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(DbSmem::sd_full + i), 1);
      mbar_init(bar(DbSmem::sd_free + i), kDbElemWarps);
    }
    fence_barrier_init();
  }
  if (warp == kDbMmaWarp) {
    tmem_alloc(smem_base + DbSmem::tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kDbProducerWarp) {
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(bar(DbSmem::bias_full), 2 * kBiasStep);
      for (int box = 0; box < 2; ++box)
        tma_load_5d(smem_base + DbSmem::bias + box * kBiasStep, &P.map_bias, bar(DbSmem::bias_full), kt * kTile + box * 64,
                    qt * kTile, h, 0, b);
      for (int i = 0; i < n_rows && ok; ++i) {
        const int st = i % kDbRing, round = i / kDbRing, r = row_lo + i;
        if (i >= kDbRing) ok = mbar_wait(bar(DbSmem::row_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(DbSmem::row_full + st), kDbStage);
        const uint32_t dst = smem_base + DbSmem::ring + st * kDbStage;
        tma_load_5d(dst, &P.map_q, bar(DbSmem::row_full + st), 0, h, qt * kTile, r, b);
        tma_load_5d(dst + kBigTile, &P.map_dout, bar(DbSmem::row_full + st), 0, h, qt * kTile, r, b);
        tma_load_5d(dst + 2 * kBigTile, &P.map_k, bar(DbSmem::row_full + st), 0, h, kt * kTile, r, b);
        tma_load_5d(dst + 3 * kBigTile, &P.map_v, bar(DbSmem::row_full + st), 0, h, kt * kTile, r, b);
      }
    }
  } else if (warp == kDbMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(Half2<T>::kFormat, 0, 0, kTile, kTile);
      bool ok = true;
      for (int i = 0; i < n_rows && ok; ++i) {
        const int st = i % kDbRing, buf = i & 1;
        ok = mbar_wait(bar(DbSmem::row_full + st), (i / kDbRing) & 1, abort_flag);
        if (ok && i >= 2) ok = mbar_wait(bar(DbSmem::sd_free + buf), ((i >> 1) - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t base = smem_base + DbSmem::ring + st * kDbStage;
        const uint64_t qdesc = smem_desc(base, 16, 512, kSwizzle64B);
        const uint64_t ddesc = smem_desc(base + kBigTile, 16, 512, kSwizzle64B);
        const uint64_t kdesc = smem_desc(base + 2 * kBigTile, 16, 512, kSwizzle64B);
        const uint64_t vdesc = smem_desc(base + 3 * kBigTile, 16, 512, kSwizzle64B);
        const uint32_t s_t = tmem_base + buf * 2 * kTile;
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(s_t, qdesc + uint64_t(kk * 2), kdesc + uint64_t(kk * 2), idesc, kk > 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(s_t + kTile, ddesc + uint64_t(kk * 2), vdesc + uint64_t(kk * 2), idesc, kk > 0 ? 1u : 0u);
        mma_commit(bar(DbSmem::sd_full + buf));
        mma_commit(bar(DbSmem::row_empty + st));
      }
    }
  } else if (warp < kDbElemWarps) {
    const int wg = warp >> 2;  // 32 of the tile's 128 keys
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const int q_index = qt * kTile + t;
    const bool q_valid = q_index < P.cols;
    const int key_base = kt * kTile + wg * 32;
    const float scale = P.scale;
    constexpr float kUnit = 1.f / 128.f, kUnitShift = float(-kExp2PolyLow) / 128.f;
    const f32x2 c2 = pack2(scale * kLog2e, scale * kLog2e);
    const float c_unit = scale * kLog2e * kUnit;

    // The thread's bias values, times log2(e), for the whole kernel.
    bool ok = mbar_wait(bar(DbSmem::bias_full), 0, abort_flag);
    f32x2 bias2[16];
    {
      const uint8_t* bias_row = smem_gen + DbSmem::bias + (wg >> 1) * kBiasStep + t * 128 + (((t & 7) ^ ((wg & 1) * 4)) << 4);
      const f32x2 log2e2 = pack2(kLog2e, kLog2e);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ok) v = *reinterpret_cast<const uint4*>(swizzled_chunk(bias_row, c));
        bias2[4 * c + 0] = mul2(Half2<T>::widen(v.x), log2e2);
        bias2[4 * c + 1] = mul2(Half2<T>::widen(v.y), log2e2);
        bias2[4 * c + 2] = mul2(Half2<T>::widen(v.z), log2e2);
        bias2[4 * c + 3] = mul2(Half2<T>::widen(v.w), log2e2);
      }
    }
    f32x2 acc2[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc2[i] = pack2(0.f, 0.f);

    const bool need_bits = has_mask || key_base + 32 > P.cols;
    const int64_t stat_stride = int64_t(P.heads) * P.cols;
    const int64_t stat_first = ((int64_t(b) * P.rows + row_lo) * P.heads + h) * P.cols + q_index;
    // Prefetch of the next row's statistics and mask byte: the loaded words stay untouched until that row's turn
    // (any arithmetic on them here would wait for the load).
    auto load_stats = [&](int i, float& lse_raw, float& delta_raw, uint32_t& keep_raw) {
      const int r = row_lo + i;
      lse_raw = INFINITY;
      delta_raw = 0.f;
      keep_raw = 0;
      if (i < n_rows) {
        if (q_valid) {
          lse_raw = ldg_f32_here(P.lse + stat_first + int64_t(i) * stat_stride);
          delta_raw = ldg_f32_here(P.delta + stat_first + int64_t(i) * stat_stride);
        }
        const int key = key_base + lane;
        if (key < P.cols) {
          keep_raw = 1;
          if (has_mask) keep_raw = ldg_u8_here(P.mask + b * P.m_sb + int64_t(r) * P.m_sr + int64_t(key) * P.m_sc);
        }
      }
    };
    float next_lse, next_dl;
    uint32_t next_keep;
    load_stats(0, next_lse, next_dl, next_keep);

    bool scores_there = false;  // answer of the probe the previous row sent for this row's scores
    for (int i = 0; i < n_rows && ok; ++i) {
      const int buf = i & 1;
      const float neg_lse2 = -next_lse * kLog2e, neg_delta = -next_dl;
      const bool keep_lane = next_keep != 0;
      load_stats(i + 1, next_lse, next_dl, next_keep);
      const uint32_t bits = need_bits ? __ballot_sync(0xffffffffu, keep_lane) : 0xffffffffu;
      const f32x2 nl1 = pack2(neg_lse2, neg_lse2), nd1 = pack2(neg_delta, neg_delta);
      const float nl_unit = fmaf(neg_lse2, kUnit, kUnitShift);
      ok = mbar_wait_probed(scores_there, bar(DbSmem::sd_full + buf), (i >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      scores_there = false;
      const uint32_t s_t = tmem_base + lane_field + buf * 2 * kTile + wg * 32;
      // The row's 32 logits of this thread, four tensor-memory columns of S and of dP at a time.  Rows with a dropped
      // key take a second copy of the body that zeroes the dropped columns: a test per element inside one body
      // would be compiled into selects that every row pays for.
      auto row_body = [&](auto drops_keys) {
        // two pairs (four tensor-memory columns of S and of dP) at a time; the loads of the next four columns are in
        // flight while the current four are worked on
        auto work4 = [&](int quad, const uint32_t (&sraw)[4], const uint32_t (&draw)[4]) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int pair = quad * 2 + j;
            const f32x2 s2 = pack2(__uint_as_float(sraw[2 * j]), __uint_as_float(sraw[2 * j + 1]));
            const f32x2 d2 = pack2(__uint_as_float(draw[2 * j]), __uint_as_float(draw[2 * j + 1]));
            f32x2 p;
            if (kDbPolyEvery > 0 && (pair % (kDbPolyEvery > 0 ? kDbPolyEvery : 1)) == kDbPolyEvery - 1) {
              // exponent x = s c + bias log2e - lse log2e, as u = sat((x - low) / 128)
              float b_lo, b_hi, s_lo, s_hi;
              unpack2(bias2[pair], b_lo, b_hi);
              unpack2(s2, s_lo, s_hi);
              const float u_lo = fma_sat(s_lo, c_unit, fmaf(b_lo, kUnit, nl_unit));
              const float u_hi = fma_sat(s_hi, c_unit, fmaf(b_hi, kUnit, nl_unit));
              p = ex2_poly_unit(pack2(u_lo, u_hi));
            } else {
              float lo, hi;
              unpack2(fma2(s2, c2, add2(bias2[pair], nl1)), lo, hi);
              p = pack2(ex2(lo), ex2(hi));
            }
            f32x2 dd = add2(d2, nd1);
            if (decltype(drops_keys)::value) {
              p = select2(p, bits, 2 * pair);
              dd = select2(dd, bits, 2 * pair);
            }
            acc2[pair] = fma2(p, dd, acc2[pair]);
          }
        };
        uint32_t s_a[4], d_a[4], s_b[4], d_b[4];
        tmem_ld4(s_t, s_a);
        tmem_ld4(s_t + kTile, d_a);
#pragma unroll
        for (int quad = 0; quad < 8; quad += 2) {
          // the next row's scores are probed half-way through this row: the answer travels under the arithmetic
          if (quad == 4 && i + 1 < n_rows) scores_there = mbar_test(bar(DbSmem::sd_full + (buf ^ 1)), ((i + 1) >> 1) & 1);
          tmem_wait_ld();
          tmem_loaded(s_a);
          tmem_loaded(d_a);
          tmem_ld4(s_t + (quad + 1) * 4, s_b);
          tmem_ld4(s_t + kTile + (quad + 1) * 4, d_b);
          work4(quad, s_a, d_a);
          tmem_wait_ld();
          tmem_loaded(s_b);
          tmem_loaded(d_b);
          if (quad + 2 < 8) {
            tmem_ld4(s_t + (quad + 2) * 4, s_a);
            tmem_ld4(s_t + kTile + (quad + 2) * 4, d_a);
          } else {
            tc_fence_before_sync();
            mbar_arrive_warp(bar(DbSmem::sd_free + buf));
          }
          work4(quad + 1, s_b, d_b);
        }
      };
      if (bits == 0xffffffffu)
        row_body(std::false_type{});
      else
        row_body(std::true_type{});
    }
    if (ok && q_valid) {
      if (P.num_parts == 1 && P.dbias_f32) {
        float* dst = reinterpret_cast<float*>(P.dbias) + b * P.db_sb + h * P.db_sh + int64_t(q_index) * P.db_sq +
                     int64_t(key_base) * P.db_sk;
        if (P.db_sk == 1 && key_base + 32 <= P.cols && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a, b2, c, d;
            unpack2(acc2[2 * i], a, b2);
            unpack2(acc2[2 * i + 1], c, d);
            reinterpret_cast<float4*>(dst)[i] = make_float4(a, b2, c, d);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float lo, hi;
            unpack2(acc2[i], lo, hi);
            if (key_base + 2 * i < P.cols) dst[int64_t(2 * i) * P.db_sk] = lo;
            if (key_base + 2 * i + 1 < P.cols) dst[int64_t(2 * i + 1) * P.db_sk] = hi;
          }
        }
      } else if (P.num_parts == 1) {
        T* dst = reinterpret_cast<T*>(P.dbias) + b * P.db_sb + h * P.db_sh + int64_t(q_index) * P.db_sq + int64_t(key_base) * P.db_sk;
        if (P.db_sk == 1 && key_base + 32 <= P.cols && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            reinterpret_cast<uint4*>(dst)[c] = make_uint4(pack16<T>(acc2[4 * c]), pack16<T>(acc2[4 * c + 1]),
                                                          pack16<T>(acc2[4 * c + 2]), pack16<T>(acc2[4 * c + 3]));
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float lo, hi;
            unpack2(acc2[i], lo, hi);
            if (key_base + 2 * i < P.cols) dst[int64_t(2 * i) * P.db_sk] = T(lo);
            if (key_base + 2 * i + 1 < P.cols) dst[int64_t(2 * i + 1) * P.db_sk] = T(hi);
          }
        }
      } else {
        float* dst = P.parts + (((int64_t(part) * P.batch + b) * P.heads + h) * P.cols + q_index) * P.cols + key_base;
        if (key_base + 32 <= P.cols && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a, b2, c, d;
            unpack2(acc2[2 * i], a, b2);
            unpack2(acc2[2 * i + 1], c, d);
            reinterpret_cast<float4*>(dst)[i] = make_float4(a, b2, c, d);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float lo, hi;
            unpack2(acc2[i], lo, hi);
            if (key_base + 2 * i < P.cols) dst[2 * i] = lo;
            if (key_base + 2 * i + 1 < P.cols) dst[2 * i + 1] = hi;
          }
        }
      }
    }
  }
  teardown(abort_flag, tmem_base, kDbMmaWarp, 512);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------

uint64_t align256(uint64_t v) { return (v + 255) & ~uint64_t(255); }

int64_t padded_cols(const oops_ta_problem& p) { return (int64_t(p.cols) + 7) & ~int64_t(7); }

// Row parts of the shared-bias kernel: one CTA per (part, batch, head, 128 x 128 tile) at one CTA per SM.  The
// smallest part count whose CTAs fill whole waves of the 148 SMs to 90 % is taken (the best one if none does);
// with a single part the kernel stores the final gradient and no partial planes exist.
int bias_parts(const oops_ta_problem& p) {
  const int64_t tiles = ceil_div(p.cols, kTile);
  const int64_t ctas = int64_t(p.batch) * p.heads * tiles * tiles;
  const int limit = (int)std::min<int64_t>(16, p.rows);
  int best = 1;
  double best_fill = 0.0;
  for (int parts = 1; parts <= limit; ++parts) {
    const int64_t total = ctas * parts;
    const double fill = double(total) / double(ceil_div(total, 148) * 148);
    if (fill > best_fill + 1e-9) {
      best = parts;
      best_fill = fill;
    }
    if (fill >= 0.9) return parts;
  }
  return best;
}

// rows of more than 6 query tiles are walked in groups of query tiles by one CTA
int fused_groups(const oops_ta_problem& p) { return (int)ceil_div(ceil_div(p.cols, kTile), kFMaxQTiles); }

// scratch slots that carry the f32 sums of dK and dV from group to group: one per SM id, two tensors, 32 floats per key
int64_t fused_slot_keys(const oops_ta_problem& p) { return ceil_div(p.cols, kTile) * kTile; }
uint64_t fused_slot_bytes(const oops_ta_problem& p) {
  return align256(uint64_t(kFSlots) * 2 * fused_slot_keys(p) * kHeadDim * sizeof(float));
}

// The single-pass kernel serves calls that want dQ together with dK or dV and no per-row bias gradient, on rows
// whose keep-bit table fits its shared memory (4096 columns).
bool fused_applies(const oops_ta_problem& p, const oops_ta_grads& g) {
  if ((p.flags & OOPS_TA_FLAG_SPLIT_REVERSE) != 0) return false;
  if (g.dbias && p.bias_groups > 1) return false;
  if (ceil_div(p.cols, 32) > kFKeepWords) return false;
  return g.dq.ptr != nullptr && (g.dk.ptr != nullptr || g.dv.ptr != nullptr);
}

struct Layout {
  uint64_t delta, bias_t, pair_parts, parts, total;
};

Layout workspace_layout(const oops_ta_problem& p, const oops_ta_grads& g) {
  Layout l{};
  uint64_t at = 0;
  l.delta = at;
  at += align256(uint64_t(p.batch) * p.rows * p.heads * p.cols * sizeof(float));
  l.bias_t = at;
  const bool fused = fused_applies(p, g);
  if (p.bias_groups != 0 && (g.dk.ptr || g.dv.ptr) && !fused)
    at += align256(uint64_t(p.batch) * p.bias_groups * p.heads * p.cols * padded_cols(p) * 2);
  l.pair_parts = at;  // per-SM slots of the single-pass kernel (rows of more than one group of query tiles)
  if (fused && fused_groups(p) > 1) at += fused_slot_bytes(p);
  l.parts = at;
  if (g.dbias && p.bias_groups == 1 && bias_parts(p) > 1)
    at += align256(uint64_t(bias_parts(p)) * p.batch * p.heads * p.cols * p.cols * sizeof(float));
  l.total = at;
  return l;
}

template <typename T, typename Params, typename K1, typename K0>
int launch_pair(bool has_bias, K1 with_bias, K0 without_bias, const Params& P, unsigned grid, int smem, cudaStream_t stream,
                const char* what) {
  auto go = [&](auto kernel) -> int {
    const int rc = reserve_smem(kernel, smem);
    if (rc) return rc;
    kernel<<<grid, kThreads, smem, stream>>>(P);
    count_launch();
    return check_launch(what);
  };
  return has_bias ? go(with_bias) : go(without_bias);
}

template <typename T>
int run_backward(const oops_ta_problem& p, const oops_ta_pair& out, const oops_ta_pair& dout, const float* lse,
                 const oops_ta_grads& g, cudaStream_t stream) {
  const Layout layout = workspace_layout(p, g);
  if (!p.workspace || p.workspace_bytes < layout.total)
    return fail(OOPS_TA_WORKSPACE_TOO_SMALL, "backward needs %llu scratch bytes, got %llu", (unsigned long long)layout.total,
                (unsigned long long)p.workspace_bytes);
  char* base = reinterpret_cast<char*>(p.workspace);
  float* delta = reinterpret_cast<float*>(base + layout.delta);
  const bool has_bias = p.bias_groups != 0;
  const bool row_bias_grad = g.dbias && p.bias_groups > 1;
  const bool shared_bias_grad = g.dbias && p.bias_groups == 1;
  int status;

  if ((p.flags & OOPS_TA_FLAG_REUSE_DELTA) == 0) {  // delta = rowsum(O * dO)
    const int64_t total = int64_t(p.batch) * p.rows * p.heads * p.cols;
    const int vec_ok = (reinterpret_cast<uintptr_t>(out.ptr) & 15) == 0 && (reinterpret_cast<uintptr_t>(dout.ptr) & 15) == 0 &&
                       out.sb % 8 == 0 && out.sr % 8 == 0 && out.sc % 8 == 0 && out.sh % 8 == 0 && dout.sb % 8 == 0 &&
                       dout.sr % 8 == 0 && dout.sc % 8 == 0 && dout.sh % 8 == 0;
    delta_kernel<T><<<(unsigned)ceil_div(total, 256), 256, 0, stream>>>(out, dout, delta, total, p.cols, p.heads, p.rows, vec_ok);
    count_launch();
    status = check_launch("tcgen05 delta");
    if (status) return status;
  }

  const bool fused = fused_applies(p, g);
  if (fused) {
    FParams P{};
    status = encode_pair(&P.map_q, p, p.q, kTile, "query");
    if (!status) status = encode_pair(&P.map_dout, p, dout, kTile, "upstream gradient");
    if (!status) status = encode_pair(&P.map_k, p, p.k, kTile, "key");
    if (!status) status = encode_pair(&P.map_v, p, p.v, kTile, "value");
    if (!status && has_bias)
      status = encode_bias(&P.map_bias, p, p.bias, p.bias_sq, p.bias_sh, p.bias_sg, p.bias_sb, kTile, "bias");
    if (status) return status;
    P.dq = g.dq;
    P.dk = g.dk;
    P.dv = g.dv;
    P.write_dq = g.dq.ptr != nullptr;
    P.write_dk = g.dk.ptr != nullptr;
    P.write_dv = g.dv.ptr != nullptr;
    P.lse = lse;
    P.delta = delta;
    P.mask = p.mask;
    P.m_sb = p.mask_sb;
    P.m_sr = p.mask_sr;
    P.m_sc = p.mask_sc;
    P.batch = p.batch;
    P.rows = p.rows;
    P.cols = p.cols;
    P.heads = p.heads;
    P.bias_groups = p.bias_groups;
    P.q_tiles = (int)ceil_div(p.cols, kTile);
    P.k_tiles = P.q_tiles;
    P.groups = fused_groups(p);
    P.tiles_per_group = (int)ceil_div(P.q_tiles, P.groups);
    P.scale = p.scale;
    if (P.groups > 1) {
      P.slots = reinterpret_cast<float*>(base + layout.pair_parts);
      P.slot_keys = fused_slot_keys(p);
    }
    const unsigned grid = (unsigned)(int64_t(p.batch) * p.rows * p.heads);
    auto go = [&](auto kernel) -> int {
      const int rc = reserve_smem(kernel, kFSmemBytes);
      if (rc) return rc;
      kernel<<<grid, kFThreads, kFSmemBytes, stream>>>(P);
      count_launch();
      return check_launch("tcgen05 dQ/dK/dV");
    };
    status = has_bias ? go(ta_bwd_fused_kernel<T, true>) : go(ta_bwd_fused_kernel<T, false>);
    if (status) return status;
  }

  if (!fused && (g.dq.ptr || row_bias_grad)) {
    DqParams P{};
    status = encode_pair(&P.map_q, p, p.q, kTile, "query");
    if (!status) status = encode_pair(&P.map_dout, p, dout, kTile, "upstream gradient");
    if (!status) status = encode_pair(&P.map_k, p, p.k, kStep, "key");
    if (!status) status = encode_pair(&P.map_v, p, p.v, kStep, "value");
    if (!status && has_bias)
      status = encode_bias(&P.map_bias, p, p.bias, p.bias_sq, p.bias_sh, p.bias_sg, p.bias_sb, kTile, "bias");
    if (status) return status;
    P.dq = g.dq;
    P.write_dq = g.dq.ptr != nullptr;
    P.lse = lse;
    P.delta = delta;
    P.mask = p.mask;
    P.m_sb = p.mask_sb;
    P.m_sr = p.mask_sr;
    P.m_sc = p.mask_sc;
    if (row_bias_grad) {
      P.dbias_rows = g.dbias;
      P.db_sb = g.dbias_sb;
      P.db_sg = g.dbias_sg;
      P.db_sh = g.dbias_sh;
      P.db_sq = g.dbias_sq;
      P.db_sk = g.dbias_sk;
    }
    P.batch = p.batch;
    P.rows = p.rows;
    P.cols = p.cols;
    P.heads = p.heads;
    P.bias_groups = p.bias_groups;
    P.q_pairs = (int)ceil_div(p.cols, kTilesPerCta * kTile);
    P.k_steps = (int)ceil_div(p.cols, kStep);
    P.scale = p.scale;
    const unsigned grid = (unsigned)(int64_t(p.batch) * p.rows * p.heads * P.q_pairs);
    status = launch_pair<T>(has_bias, ta_bwd_dq_kernel<T, true>, ta_bwd_dq_kernel<T, false>, P, grid, kDqSmemBytes, stream,
                            "tcgen05 dQ");
    if (status) return status;
  }

  if (!fused && (g.dk.ptr || g.dv.ptr)) {
    DkvParams P{};
    status = encode_pair(&P.map_k, p, p.k, kTile, "key");
    if (!status) status = encode_pair(&P.map_v, p, p.v, kTile, "value");
    if (!status) status = encode_pair(&P.map_q, p, p.q, kStep, "query");
    if (!status) status = encode_pair(&P.map_dout, p, dout, kStep, "upstream gradient");
    if (status) return status;
    if (has_bias) {
      uint16_t* bias_t = reinterpret_cast<uint16_t*>(base + layout.bias_t);
      const int64_t stride = padded_cols(p);
      dim3 grid((unsigned)ceil_div(stride, 32), (unsigned)ceil_div(p.cols, 32), (unsigned)(p.batch * p.bias_groups * p.heads));
      transpose_bias_kernel<<<grid, dim3(32, 8), 0, stream>>>(reinterpret_cast<const uint16_t*>(p.bias), bias_t, p.cols,
                                                              p.bias_sq, p.bias_sh, p.bias_sg, p.bias_sb, p.heads,
                                                              p.bias_groups, stride);
      count_launch();
      status = check_launch("tcgen05 bias transpose");
      if (status) return status;
      const int64_t plane = int64_t(p.cols) * stride;
      status = encode_bias(&P.map_bias_t, p, bias_t, stride, plane, plane * p.heads, plane * p.heads * p.bias_groups, kTile,
                           "transposed bias");
      if (status) return status;
    }
    P.dk = g.dk;
    P.dv = g.dv;
    P.write_dk = g.dk.ptr != nullptr;
    P.write_dv = g.dv.ptr != nullptr;
    P.lse = lse;
    P.delta = delta;
    P.mask = p.mask;
    P.m_sb = p.mask_sb;
    P.m_sr = p.mask_sr;
    P.m_sc = p.mask_sc;
    P.batch = p.batch;
    P.rows = p.rows;
    P.cols = p.cols;
    P.heads = p.heads;
    P.bias_groups = p.bias_groups;
    P.k_pairs = (int)ceil_div(p.cols, kTilesPerCta * kTile);
    P.q_steps = (int)ceil_div(p.cols, kStep);
    P.scale = p.scale;
    const unsigned grid = (unsigned)(int64_t(p.batch) * p.rows * p.heads * P.k_pairs);
    status = launch_pair<T>(has_bias, ta_bwd_dkv_kernel<T, true>, ta_bwd_dkv_kernel<T, false>, P, grid, kDkvSmemBytes, stream,
                            "tcgen05 dK/dV");
    if (status) return status;
  }

  if (shared_bias_grad) {
    DbParams P{};
    status = encode_pair(&P.map_q, p, p.q, kTile, "query");
    if (!status) status = encode_pair(&P.map_dout, p, dout, kTile, "upstream gradient");
    if (!status) status = encode_pair(&P.map_k, p, p.k, kTile, "key");
    if (!status) status = encode_pair(&P.map_v, p, p.v, kTile, "value");
    if (!status) status = encode_bias(&P.map_bias, p, p.bias, p.bias_sq, p.bias_sh, p.bias_sg, p.bias_sb, kTile, "bias");
    if (status) return status;
    P.num_parts = bias_parts(p);
    P.parts = P.num_parts > 1 ? reinterpret_cast<float*>(base + layout.parts) : nullptr;
    P.dbias = g.dbias;
    P.db_sb = g.dbias_sb;
    P.db_sh = g.dbias_sh;
    P.db_sq = g.dbias_sq;
    P.db_sk = g.dbias_sk;
    P.dbias_f32 = (p.flags & OOPS_TA_FLAG_DBIAS_F32) != 0;
    P.lse = lse;
    P.delta = delta;
    P.mask = p.mask;
    P.m_sb = p.mask_sb;
    P.m_sr = p.mask_sr;
    P.m_sc = p.mask_sc;
    P.batch = p.batch;
    P.rows = p.rows;
    P.cols = p.cols;
    P.heads = p.heads;
    P.tiles = (int)ceil_div(p.cols, kTile);
    P.rows_per_part = (int)ceil_div(p.rows, P.num_parts);
    P.scale = p.scale;
    const unsigned grid = (unsigned)(int64_t(P.num_parts) * p.batch * p.heads * P.tiles * P.tiles);
    auto kernel = ta_bwd_dbias_kernel<T>;
    status = reserve_smem(kernel, kDbSmemBytes);
    if (status) return status;
    kernel<<<grid, kDbThreads, kDbSmemBytes, stream>>>(P);
    count_launch();
    status = check_launch("tcgen05 shared-bias gradient");
    if (status) return status;
    if (P.num_parts > 1) {
      const int64_t plane = int64_t(p.batch) * p.heads * p.cols * p.cols;
      if (P.dbias_f32)
        reduce_parts_kernel<float><<<(unsigned)ceil_div(plane, 256), 256, 0, stream>>>(
            P.parts, P.num_parts, g.dbias, g.dbias_sb, g.dbias_sh, g.dbias_sq, g.dbias_sk, p.batch, p.heads, p.cols);
      else
        reduce_parts_kernel<T><<<(unsigned)ceil_div(plane, 256), 256, 0, stream>>>(
            P.parts, P.num_parts, g.dbias, g.dbias_sb, g.dbias_sh, g.dbias_sq, g.dbias_sk, p.batch, p.heads, p.cols);
      count_launch();
      status = check_launch("tcgen05 shared-bias reduce");
      if (status) return status;
    }
  }
  return OOPS_TA_OK;
}

}  // namespace

bool tensor_backward_applies(const oops_ta_problem& p, const oops_ta_grads* g) {
  if (!tensor_forward_applies(p)) return false;
  const int64_t rows = int64_t(p.batch) * p.rows * p.heads * p.cols;
  if (rows > 0x7fffffffll * 64) return false;
  (void)g;
  return true;
}

uint64_t tensor_backward_workspace(const oops_ta_problem& p, const oops_ta_grads& g) { return workspace_layout(p, g).total; }

int tensor_backward(const oops_ta_problem& p, const oops_ta_pair& out, const oops_ta_pair& dout, const float* lse,
                    const oops_ta_grads& g, cudaStream_t stream) {
  if ((reinterpret_cast<uintptr_t>(dout.ptr) & 15) != 0 || !stride_ok(dout.sb, p.batch) || !stride_ok(dout.sr, p.rows) ||
      !stride_ok(dout.sc, p.cols) || !stride_ok(dout.sh, p.heads))
    return fail(OOPS_TA_UNSUPPORTED_LAYOUT, "upstream gradient must be 16-byte aligned with strides that are multiples of 8");
  if (p.dtype == OOPS_TA_BF16) return run_backward<__nv_bfloat16>(p, out, dout, lse, g, stream);
  return run_backward<__half>(p, out, dout, lse, g, stream);
}

int backward_device_status(int reset) { return read_tu_device_status(reset); }

}  // namespace oops_ta
