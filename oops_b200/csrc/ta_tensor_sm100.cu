// tcgen05 / TMEM / TMA triangle-attention kernels for sm_100a (f16 and bf16, head_dim 32).
//
// Forward (replaces the reference's Triton `_attend`, oops/attention/triangle/triton/kernel.py:150-262):
// one CTA owns one (batch, row, head) and a pair of 128-query tiles.  A producer warp streams
// 128-key K/V tiles and 128x128 bias tiles into shared memory with TMA; one thread issues
// tcgen05.mma for S = Q K^T (accumulator in tensor memory) and O += P V (P read back from tensor
// memory, V from shared memory); two softmax warpgroups, one per query tile, read S from tensor
// memory, add the bias, apply the key mask, run the online softmax in base 2 and write P (packed
// 16-bit) over S.  While one warpgroup is in its softmax the tensor core works on the other tile.
#include "ta_tensor_common.cuh"

namespace oops_ta {
namespace {

using namespace ptx;


constexpr int kStages = 3;                       // K/V ring depth
constexpr int kKeys = 64;                        // keys per step
constexpr int kQBytes = kTile * kHeadDim * 2;    // 8 KiB: one 128-query Q tile
constexpr int kKvBytes = kKeys * kHeadDim * 2;   // 4 KiB: one K or V step
constexpr int kBiasBytes = kTile * kKeys * 2;    // 16 KiB: one 128 x 64 bias tile (one swizzle-128 box)
constexpr int kFwdThreads = 320;                 // 2 softmax warpgroups + producer warp + MMA warp
constexpr int kFwdTmemCols = 256;                // S 2x64 | P 2x32 | O 2x32; two CTAs share an SM
constexpr int kMaxKeepWords = 512;               // keep-bit table: one bit per key column, cols <= 16384
#ifndef TA_FWD_POLY_EVERY
#define TA_FWD_POLY_EVERY 0
#endif
constexpr int kFwdPolyEvery = TA_FWD_POLY_EVERY;  // every n-th pair of a thread's logits takes the polynomial exp2 (0: none)

struct FwdSmem {
  static constexpr int q = 0;                          // [2]
  static constexpr int k = q + 2 * kQBytes;            // [kStages]
  static constexpr int v = k + kStages * kKvBytes;     // [kStages]
  static constexpr int bias = v + kStages * kKvBytes;  // [2 tiles][2 buffers]
  static constexpr int bars = bias + 4 * kBiasBytes;
  // barrier indices (8 bytes each)
  static constexpr int q_full = 0;                     // [2]
  static constexpr int k_full = q_full + 2;            // [kStages]
  static constexpr int k_empty = k_full + kStages;     // [kStages]
  static constexpr int v_full = k_empty + kStages;     // [kStages]
  static constexpr int v_empty = v_full + kStages;     // [kStages]
  static constexpr int v_ready = v_empty + kStages;    // [kStages]
  static constexpr int bias_full = v_ready + kStages;  // [2 tiles][2 buffers]
  static constexpr int bias_empty = bias_full + 4;     // [2][2]
  static constexpr int s_full = bias_empty + 4;        // [2]
  static constexpr int p_full = s_full + 2;            // [2]
  static constexpr int o_final = p_full + 2;           // [2]
  static constexpr int s_free = o_final + 2;           // [2] S has been read into registers
  static constexpr int pv_done = s_free + 2;           // [2] the latest P V product has completed
  static constexpr int num_bars = pv_done + 2;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int drop_flags = abort_flag + 4;    // [8] per-warp: the mask drops a key of this row
  static constexpr int keep = drop_flags + 32;         // [kMaxKeepWords] u32
  static constexpr int total = keep + kMaxKeepWords * 4;
};
constexpr int kFwdSmemBytes = FwdSmem::total + 1024;  // slack to align the base to 1 KiB
static_assert(kFwdSmemBytes <= 113 * 1024, "two forward CTAs must fit in one SM's shared memory");

struct FwdParams {
  CUtensorMap map_q, map_k, map_v, map_bias;
  void* out;
  int64_t o_sb, o_sr, o_sc, o_sh;
  float* lse;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  int batch, rows, cols, heads, bias_groups;
  int q_pairs, k_steps;
  int out_vec16;
  float scale;
  // gated epilogue (GATED instantiations): gated = sigmoid(gate) * out goes to `out`, the ungated values to `plain`
  const void* gate;
  int64_t g_sb, g_sr, g_sc, g_sh;
  void* plain;  // may be null
  int64_t p_sb, p_sr, p_sc, p_sh;
  int gate_vec16, plain_vec16;
};

// The running maximum is only raised when a step exceeds it by more than this (natural-log units):
// probabilities then stay below e^kRescaleSlack, far inside the f32 / 16-bit ranges, and the
// accumulator rescale (a tensor-memory round trip) is skipped for almost every step.
constexpr float kRescaleSlack = 5.545177444f;  // 8 * ln 2

template <typename T, bool HAS_BIAS, bool GATED>
__global__ void __launch_bounds__(kFwdThreads, 2) ta_fwd_kernel(const __grid_constant__ FwdParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + FwdSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + FwdSmem::tmem_slot);
  uint32_t* keep_words = reinterpret_cast<uint32_t*>(smem_gen + FwdSmem::keep);
  auto bar = [&](int index) -> uint32_t { return smem_base + FwdSmem::bars + index * 8; };

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  if (device_failed()) return;

  // work decomposition: query pair fastest, then head, row, batch
  int idx = blockIdx.x;
  const int qp = idx % P.q_pairs;
  idx /= P.q_pairs;
  const int h = idx % P.heads;
  idx /= P.heads;
  const int r = idx % P.rows;
  const int b = idx / P.rows;
  const int q0 = qp * 2 * kTile;
  const int n_tiles = (q0 + kTile < P.cols) ? 2 : 1;
  const int KS = P.k_steps;
  const int g = P.bias_groups == 1 ? 0 : r;
  const bool has_mask = P.mask != nullptr;
  // Steps need keep-bits when there is a mask or when the last key step is ragged.
  const bool has_bits = has_mask || (P.cols % kKeys) != 0;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) mbar_init(bar(FwdSmem::q_full + i), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(FwdSmem::k_full + i), 1);
      mbar_init(bar(FwdSmem::k_empty + i), 1);
      mbar_init(bar(FwdSmem::v_full + i), 1);
      mbar_init(bar(FwdSmem::v_empty + i), 1);
      mbar_init(bar(FwdSmem::v_ready + i), kTile / 32);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(FwdSmem::bias_full + i), 1);
      mbar_init(bar(FwdSmem::bias_empty + i), kTile / 32);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(FwdSmem::s_full + i), 1);
      mbar_init(bar(FwdSmem::p_full + i), kTile / 32);
      mbar_init(bar(FwdSmem::o_final + i), 1);
      mbar_init(bar(FwdSmem::s_free + i), kTile / 32);
      mbar_init(bar(FwdSmem::pv_done + i), 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_base + FwdSmem::tmem_slot, kFwdTmemCols);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  uint32_t* drop_flags = reinterpret_cast<uint32_t*>(smem_gen + FwdSmem::drop_flags);
  if (has_bits && warp < 8) {
    // one bit per key of this pair row: kept by the mask and inside the row
    const uint8_t* mask_row = has_mask ? P.mask + b * P.m_sb + int64_t(r) * P.m_sr : nullptr;
    bool dropped_any = false;
    for (int word = warp; word < KS * 2; word += 8) {
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
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Value rows only need the sign-off handshake when the mask really drops a key of this row.
  bool signoff = false;
  if (has_mask) {
#pragma unroll
    for (int i = 0; i < 8; ++i) signoff |= drop_flags[i] != 0;
  }
  // tensor-memory columns
  constexpr int kSCol = 0, kPCol = 2 * kKeys, kOCol = 2 * kKeys + 2 * (kKeys / 2);

  if (warp == 8) {
    // ------------------------------------------------------------------ producer (one thread)
    if (lane == 0) {
      bool ok = true;
      for (int w = 0; w < n_tiles; ++w) {
        mbar_expect_tx(bar(FwdSmem::q_full + w), kQBytes);
        tma_load_5d(smem_base + FwdSmem::q + w * kQBytes, &P.map_q, bar(FwdSmem::q_full + w), 0, h, q0 + w * kTile, r, b);
      }
      for (int j = 0; j < KS && ok; ++j) {
        const int st = j % kStages, round = j / kStages;
        if (j >= kStages) ok = mbar_wait(bar(FwdSmem::k_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(FwdSmem::k_full + st), kKvBytes);
        tma_load_5d(smem_base + FwdSmem::k + st * kKvBytes, &P.map_k, bar(FwdSmem::k_full + st), 0, h, j * kKeys, r, b);
        if (HAS_BIAS) {
          const int buf = j & 1;
          for (int w = 0; w < n_tiles && ok; ++w) {
            const int slot = w * 2 + buf;
            if (j >= 2) ok = mbar_wait(bar(FwdSmem::bias_empty + slot), ((j >> 1) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar(FwdSmem::bias_full + slot), kBiasBytes);
            tma_load_5d(smem_base + FwdSmem::bias + slot * kBiasBytes, &P.map_bias, bar(FwdSmem::bias_full + slot),
                        j * kKeys, q0 + w * kTile, h, g, b);
          }
        }
        if (j >= kStages) ok = mbar_wait(bar(FwdSmem::v_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(FwdSmem::v_full + st), kKvBytes);
        tma_load_5d(smem_base + FwdSmem::v + st * kKvBytes, &P.map_v, bar(FwdSmem::v_full + st), 0, h, j * kKeys, r, b);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t fmt = Half2<T>::kFormat;
      constexpr uint32_t idesc_qk = instr_desc(fmt, 0, 0, kTile, kKeys);
      constexpr uint32_t idesc_pv = instr_desc(fmt, 0, 1, kTile, kHeadDim);
      bool ok = true;
      for (int w = 0; w < n_tiles && ok; ++w) ok = mbar_wait(bar(FwdSmem::q_full + w), 0, abort_flag);
      // S[128 x 64] = Q[128 x 32] K[64 x 32]^T; both K-major, 64-byte swizzle: 8-row groups 512 bytes apart,
      // each 16-channel step advances 32 bytes inside the swizzle span.
      auto issue_qk = [&](int j, int w) {
        const int st = j % kStages;
        const uint64_t qdesc = smem_desc(smem_base + FwdSmem::q + w * kQBytes, 16, 512, kSwizzle64B);
        const uint64_t kdesc = smem_desc(smem_base + FwdSmem::k + st * kKvBytes, 16, 512, kSwizzle64B);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk)
          mma_ss(tmem_base + kSCol + w * kKeys, qdesc + uint64_t(kk * 2), kdesc + uint64_t(kk * 2), idesc_qk, kk > 0 ? 1u : 0u);
        mma_commit(bar(FwdSmem::s_full + w));
        if (w == n_tiles - 1) mma_commit(bar(FwdSmem::k_empty + st));
      };
      if (ok) ok = mbar_wait(bar(FwdSmem::k_full), 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        for (int w = 0; w < n_tiles; ++w) issue_qk(0, w);
      }
      for (int j = 0; j < KS && ok; ++j) {
        if (j + 1 < KS) {
          // next score tiles: issued as soon as a warpgroup has pulled S(j) into registers, so that S(j+1) is
          // ready when its softmax of step j ends (P has its own tensor-memory columns)
          ok = mbar_wait(bar(FwdSmem::k_full + (j + 1) % kStages), ((j + 1) / kStages) & 1, abort_flag);
          for (int w = 0; w < n_tiles && ok; ++w) {
            ok = mbar_wait(bar(FwdSmem::s_free + w), j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_qk(j + 1, w);
          }
        }
        const int st = j % kStages;
        for (int w = 0; w < n_tiles && ok; ++w) {
          ok = mbar_wait(bar(FwdSmem::p_full + w), j & 1, abort_flag);
          if (ok && w == 0) {
            ok = mbar_wait(bar(FwdSmem::v_full + st), (j / kStages) & 1, abort_flag);
            // with a mask, warpgroup 0 signs off every value step after clearing the rows of dropped keys
            if (ok && signoff) ok = mbar_wait(bar(FwdSmem::v_ready + st), (j / kStages) & 1, abort_flag);
          }
          if (!ok) break;
          tc_fence_after_sync();
          // O[128 x 32] += P[128 x 64] V[64 x 32]; V is MN-major (channel contiguous), 64-byte swizzle:
          // 8-key groups are 512 bytes apart, each 16-key step advances 1024 bytes.
          const uint32_t p_tmem = tmem_base + kPCol + w * (kKeys / 2);
          const uint32_t o_tmem = tmem_base + kOCol + w * kHeadDim;
          const uint64_t vdesc = smem_desc(smem_base + FwdSmem::v + st * kKvBytes, 16, 512, kSwizzle64B);
#pragma unroll
          for (int kk = 0; kk < kKeys / 16; ++kk)
            mma_ts(o_tmem, p_tmem + kk * 8, vdesc + uint64_t(kk * (1024 >> 4)), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          mma_commit(bar(FwdSmem::pv_done + w));
          if (j == KS - 1) mma_commit(bar(FwdSmem::o_final + w));
          if (w == n_tiles - 1) mma_commit(bar(FwdSmem::v_empty + st));
        }
      }
    }
  } else if ((warp >> 2) < n_tiles) {
    // ------------------------------------------------------------------ softmax warpgroups
    const int w = warp >> 2;
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_field + kSCol + w * kKeys;
    const uint32_t p_tmem = tmem_base + lane_field + kPCol + w * (kKeys / 2);
    const uint32_t o_tmem = tmem_base + lane_field + kOCol + w * kHeadDim;
    const int q_index = q0 + w * kTile + t;
    const f32x2 scale2 = pack2(P.scale, P.scale);
    const f32x2 log2e2 = pack2(kLog2e, kLog2e);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < KS && ok; ++j) {
      uint32_t bits[2] = {0xffffffffu, 0xffffffffu};
      bool all_kept = true;
      if (has_bits) {
        const uint2 wds = *reinterpret_cast<const uint2*>(keep_words + j * 2);
        bits[0] = wds.x; bits[1] = wds.y;
        all_kept = (wds.x & wds.y) == 0xffffffffu;
      }
      if (signoff && w == 0) {
        // Values of dropped keys must not reach the tensor core (0 * inf): clear their rows in shared memory.
        // Every step is signed off (one barrier phase per step); only steps with dropped keys are touched.
        const int st = j % kStages;
        if (!all_kept) {
          ok = mbar_wait(bar(FwdSmem::v_full + st), (j / kStages) & 1, abort_flag);
          if (!ok) break;
          if (t < kKeys && ((bits[t >> 5] >> (t & 31)) & 1u) == 0) {
            uint4* row = reinterpret_cast<uint4*>(smem_gen + FwdSmem::v + st * kKvBytes + t * 64);
            row[0] = row[1] = row[2] = row[3] = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
        }
        mbar_arrive_warp(bar(FwdSmem::v_ready + st));
      }

      // the two phases the step needs are probed together: one round trip to the barrier words when both are complete
      const bool s_there = mbar_test(bar(FwdSmem::s_full + w), j & 1);
      const bool bias_there = HAS_BIAS && mbar_test(bar(FwdSmem::bias_full + w * 2 + (j & 1)), (j >> 1) & 1);
      ok = mbar_wait_probed(s_there, bar(FwdSmem::s_full + w), j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      f32x2 x[kKeys / 2];
      static_assert(kKeys == 64, "two 32-column loads per step");
      {
        // nothing stands between the loads and their wait, and the registers are read only after it
        uint32_t raw0[32], raw1[32];
        tmem_ld32(s_tmem, raw0);
        tmem_ld32(s_tmem + 32, raw1);
        tmem_wait_ld();
        tmem_loaded(raw0);
        tmem_loaded(raw1);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          x[i] = pack2(__uint_as_float(raw0[2 * i]), __uint_as_float(raw0[2 * i + 1]));
          x[16 + i] = pack2(__uint_as_float(raw1[2 * i]), __uint_as_float(raw1[2 * i + 1]));
        }
      }
      tc_fence_before_sync();
      mbar_arrive_warp(bar(FwdSmem::s_free + w));

      if (HAS_BIAS) {
        const int slot = w * 2 + (j & 1);
        ok = mbar_wait_probed(bias_there, bar(FwdSmem::bias_full + slot), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        const uint8_t* row = smem_gen + FwdSmem::bias + slot * kBiasBytes + t * 128;
        uint4 bv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) bv[c] = *reinterpret_cast<const uint4*>(row + ((c ^ (t & 7)) << 4));
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          x[c * 4 + 0] = fma2(x[c * 4 + 0], scale2, Half2<T>::widen(bv[c].x));
          x[c * 4 + 1] = fma2(x[c * 4 + 1], scale2, Half2<T>::widen(bv[c].y));
          x[c * 4 + 2] = fma2(x[c * 4 + 2], scale2, Half2<T>::widen(bv[c].z));
          x[c * 4 + 3] = fma2(x[c * 4 + 3], scale2, Half2<T>::widen(bv[c].w));
        }
        mbar_arrive_warp(bar(FwdSmem::bias_empty + slot));
      } else {
#pragma unroll
        for (int i = 0; i < kKeys / 2; ++i) x[i] = mul2(x[i], scale2);
      }
      if (!all_kept) {
#pragma unroll
        for (int i = 0; i < kKeys / 2; ++i) {
          float lo, hi;
          unpack2(x[i], lo, hi);
          if (((bits[(2 * i) >> 5] >> ((2 * i) & 31)) & 1u) == 0) lo = -INFINITY;
          if (((bits[(2 * i + 1) >> 5] >> ((2 * i + 1) & 31)) & 1u) == 0) hi = -INFINITY;
          x[i] = pack2(lo, hi);
        }
      }
      float peaks[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float lo, hi;
        unpack2(x[i], lo, hi);
        peaks[i] = fmaxf(lo, hi);
      }
#pragma unroll
      for (int i = 8; i < kKeys / 2; ++i) {
        float lo, hi;
        unpack2(x[i], lo, hi);
        peaks[i & 7] = max3(peaks[i & 7], lo, hi);
      }
      const float peak = fmaxf(max3(peaks[0], peaks[1], peaks[2]), max3(max3(peaks[3], peaks[4], peaks[5]), peaks[6], peaks[7]));
      // raise the running maximum only when it is exceeded by more than the slack (always on the first finite step)
      const bool raise = peak > m_run + kRescaleSlack || (m_run == -INFINITY && peak > -INFINITY);
      const float m_old = m_run;
      if (raise) m_run = peak;
      const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
      const float alpha = raise ? ex2((m_old - m_use) * kLog2e) : 1.f;
      const float shift = -m_use * kLog2e;
      const f32x2 shift2 = pack2(shift, shift);
      f32x2 totals[4] = {pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f), pack2(0.f, 0.f)};
      uint32_t packed[kKeys / 2];
      if (kFwdPolyEvery > 0 && all_kept) {
        // every kFwdPolyEvery-th pair takes its 2^x from the FMA pipe; steps with dropped keys (-inf logits, whose
        // probability must be exactly zero) keep the special-function unit for every element
        const float shift_unit = fmaf(shift, 1.f / 128.f, float(-kExp2PolyLow) / 128.f);
#pragma unroll
        for (int i = 0; i < kKeys / 2; ++i) {
          f32x2 p;
          if ((i % (kFwdPolyEvery > 0 ? kFwdPolyEvery : 1)) == kFwdPolyEvery - 1) {
            float x_lo, x_hi;
            unpack2(x[i], x_lo, x_hi);
            p = ex2_poly_unit(pack2(fma_sat(x_lo, kLog2e / 128.f, shift_unit), fma_sat(x_hi, kLog2e / 128.f, shift_unit)));
          } else {
            float lo, hi;
            unpack2(fma2(x[i], log2e2, shift2), lo, hi);
            p = pack2(ex2(lo), ex2(hi));
          }
          totals[i & 3] = add2(totals[i & 3], p);
          float p0, p1;
          unpack2(p, p0, p1);
          packed[i] = Half2<T>::pack(p0, p1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kKeys / 2; ++i) {
          float lo, hi;
          unpack2(fma2(x[i], log2e2, shift2), lo, hi);
          const float p0 = ex2(lo), p1 = ex2(hi);
          totals[i & 3] = add2(totals[i & 3], pack2(p0, p1));
          packed[i] = Half2<T>::pack(p0, p1);
        }
      }
      float t_lo, t_hi;
      unpack2(add2(add2(totals[0], totals[1]), add2(totals[2], totals[3])), t_lo, t_hi);
      l_run = l_run * alpha + (t_lo + t_hi);
      if (j > 0) {
        // the previous P V product must have finished with O and with the P columns before either is touched
        ok = mbar_wait(bar(FwdSmem::pv_done + w), (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        uint32_t acc[32];
        tmem_ld32(o_tmem, acc);
        tmem_wait_ld();
        tmem_loaded(acc);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
        tmem_st32(o_tmem, acc);
      }
      tmem_st32(p_tmem, packed);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive_warp(bar(FwdSmem::p_full + w));
    }

    // Gated epilogue: the thread's 32 gate logits are requested before the wait for the last product, so that their
    // trip from global memory runs under it (the words are not touched until the output row is ready).
    uint4 gate_words[4] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (GATED && P.gate_vec16 && ok && q_index < P.cols) {
      const T* g = reinterpret_cast<const T*>(P.gate) + b * P.g_sb + int64_t(r) * P.g_sr + int64_t(q_index) * P.g_sc + h * P.g_sh;
#pragma unroll
      for (int i = 0; i < 4; ++i) gate_words[i] = ldg_v4_here_if(reinterpret_cast<const uint4*>(g) + i, true);
    }
    if (ok) ok = mbar_wait(bar(FwdSmem::o_final + w), 0, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      uint32_t acc[32];
      tmem_ld32(o_tmem, acc);
      tmem_wait_ld();
      tmem_loaded(acc);
      if (q_index < P.cols) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint32_t o2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          o2[i] = Half2<T>::pack(__uint_as_float(acc[2 * i]) * inv, __uint_as_float(acc[2 * i + 1]) * inv);
        auto store_row = [&](void* base, int64_t sb, int64_t sr, int64_t sc, int64_t sh, int vec16, const uint32_t (&w)[16]) {
          T* dst = reinterpret_cast<T*>(base) + b * sb + int64_t(r) * sr + int64_t(q_index) * sc + h * sh;
          if (vec16) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int i = 0; i < 4; ++i) d4[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          } else {
            unsigned short* d0 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              d0[2 * i] = (unsigned short)(w[i] & 0xffffu);
              d0[2 * i + 1] = (unsigned short)(w[i] >> 16);
            }
          }
        };
        if (GATED) {
          // The sigmoid gate of the output projection that follows this operator in a pair block, applied to the
          // 16-bit attention values while they are still in registers: gated = sigmoid(gate) * out.  The ungated
          // values are stored too when the reverse pass will need them.
          if (P.plain) store_row(P.plain, P.p_sb, P.p_sr, P.p_sc, P.p_sh, P.plain_vec16, o2);
          const T* g = reinterpret_cast<const T*>(P.gate) + b * P.g_sb + int64_t(r) * P.g_sr + int64_t(q_index) * P.g_sc + h * P.g_sh;
          uint32_t gw[16];
          if (P.gate_vec16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 v = gate_words[i];
              gw[4 * i] = v.x; gw[4 * i + 1] = v.y; gw[4 * i + 2] = v.z; gw[4 * i + 3] = v.w;
            }
          } else {
            const unsigned short* g0 = reinterpret_cast<const unsigned short*>(g);
#pragma unroll
            for (int i = 0; i < 16; ++i) gw[i] = uint32_t(g0[2 * i]) | (uint32_t(g0[2 * i + 1]) << 16);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // the gate multiplies the attention values as they are returned, i.e. after their 16-bit rounding
            const float s_lo = rcp(1.f + ex2(-Half2<T>::lo(gw[i]) * kLog2e));
            const float s_hi = rcp(1.f + ex2(-Half2<T>::hi(gw[i]) * kLog2e));
            o2[i] = Half2<T>::pack(Half2<T>::lo(o2[i]) * s_lo, Half2<T>::hi(o2[i]) * s_hi);
          }
        }
        store_row(P.out, P.o_sb, P.o_sr, P.o_sc, P.o_sh, P.out_vec16, o2);
        if (P.lse) {
          const float m_use = (m_run == -INFINITY) ? 0.f : m_run;
          P.lse[((int64_t(b) * P.rows + r) * P.heads + h) * P.cols + q_index] =
              l_run > 0.f ? (m_use + lg2(l_run) * kLn2) : 0.f;
        }
      }
    }
  }
  teardown(abort_flag, tmem_base, 9, kFwdTmemCols);
}

// Self-test of the bounded wait: one CTA allocates tensor memory and waits, with a one-millisecond limit, on a barrier
// that nothing ever completes.  The wait gives up, the CTA tears down exactly like a compute kernel whose wait ran
// out (abort flag, grace period, status word, tensor memory freed) and returns by itself.
__global__ void __launch_bounds__(128, 1) wait_limit_selftest_kernel() {
  __shared__ __align__(8) uint64_t barrier_word;
  __shared__ uint32_t tmem_slot_word;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5;
  if (device_failed()) return;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(smem_u32(&barrier_word), 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot_word), 32);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot_word);
  if (threadIdx.x == 32) mbar_wait(smem_u32(&barrier_word), 0, abort_flag, 1000000ull);
  teardown(abort_flag, tmem_base, 0, 32);
}

}  // namespace

int wait_limit_selftest(cudaStream_t stream) {
  wait_limit_selftest_kernel<<<1, 128, 0, stream>>>();
  count_launch();
  return check_launch("bounded-wait self-test");
}

bool tensor_forward_applies(const oops_ta_problem& p) {
  if (p.dtype != OOPS_TA_BF16 && p.dtype != OOPS_TA_F16) return false;
  if (p.head_dim != kHeadDim) return false;
  if (!pair_ok(p.q, p) || !pair_ok(p.k, p) || !pair_ok(p.v, p)) return false;
  if (p.bias_groups != 0) {
    if (p.bias_dtype != p.dtype || p.bias_sk != 1) return false;
    if ((reinterpret_cast<uintptr_t>(p.bias) & 15) != 0) return false;
    if (!stride_ok(p.bias_sq, p.cols) || !stride_ok(p.bias_sh, p.heads) || !stride_ok(p.bias_sg, p.bias_groups) ||
        !stride_ok(p.bias_sb, p.batch))
      return false;
    if (p.cols == 1) return false;
  }
  if (p.cols > kMaxKeepWords * 32) return false;
  const int64_t ctas = int64_t(p.batch) * p.rows * p.heads * ceil_div(p.cols, 2 * kTile);
  return ctas <= 0x7fffffffll;
}

uint64_t tensor_forward_workspace(const oops_ta_problem&) { return 0; }

namespace {

bool vec16_ok(const oops_ta_pair& t) {
  return (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 && t.sb % 8 == 0 && t.sr % 8 == 0 && t.sc % 8 == 0 && t.sh % 8 == 0;
}

int launch_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, const oops_ta_pair* gate,
                   const oops_ta_pair* plain, cudaStream_t stream) {
  FwdParams P{};
  int status = encode_pair(&P.map_q, p, p.q, kTile, "query");
  if (!status) status = encode_pair(&P.map_k, p, p.k, kKeys, "key");
  if (!status) status = encode_pair(&P.map_v, p, p.v, kKeys, "value");
  if (status) return status;
  const bool has_bias = p.bias_groups != 0;
  if (has_bias) {
    status = encode_bias(&P.map_bias, p, p.bias, p.bias_sq, p.bias_sh, p.bias_sg, p.bias_sb, kTile, "bias");
    if (status) return status;
  }
  P.out = out.ptr;
  P.o_sb = out.sb;
  P.o_sr = out.sr;
  P.o_sc = out.sc;
  P.o_sh = out.sh;
  P.out_vec16 = vec16_ok(out);
  if (gate) {
    P.gate = gate->ptr;
    P.g_sb = gate->sb;
    P.g_sr = gate->sr;
    P.g_sc = gate->sc;
    P.g_sh = gate->sh;
    P.gate_vec16 = vec16_ok(*gate);
    if (plain && plain->ptr) {
      P.plain = plain->ptr;
      P.p_sb = plain->sb;
      P.p_sr = plain->sr;
      P.p_sc = plain->sc;
      P.p_sh = plain->sh;
      P.plain_vec16 = vec16_ok(*plain);
    }
  }
  P.lse = lse;
  P.mask = p.mask;
  P.m_sb = p.mask_sb;
  P.m_sr = p.mask_sr;
  P.m_sc = p.mask_sc;
  P.batch = p.batch;
  P.rows = p.rows;
  P.cols = p.cols;
  P.heads = p.heads;
  P.bias_groups = p.bias_groups;
  P.q_pairs = (int)ceil_div(p.cols, 2 * kTile);
  P.k_steps = (int)ceil_div(p.cols, kKeys);
  P.scale = p.scale;
  const unsigned grid = (unsigned)(int64_t(p.batch) * p.rows * p.heads * P.q_pairs);

  auto launch = [&](auto kernel) -> int {
    // the attribute belongs to the (kernel, device) pair: it is set on every launch so that a host thread that
    // moves between devices never launches without it (the call costs well under a microsecond)
    const int rc = reserve_smem(kernel, kFwdSmemBytes);
    if (rc) return rc;
    kernel<<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(P);
    count_launch();
    return check_launch("tcgen05 forward");
  };
  auto pick = [&](auto type_tag) -> int {
    using T = decltype(type_tag);
    if (gate) return has_bias ? launch(ta_fwd_kernel<T, true, true>) : launch(ta_fwd_kernel<T, false, true>);
    return has_bias ? launch(ta_fwd_kernel<T, true, false>) : launch(ta_fwd_kernel<T, false, false>);
  };
  return p.dtype == OOPS_TA_BF16 ? pick(__nv_bfloat16{}) : pick(__half{});
}

}  // namespace

int tensor_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream) {
  return launch_forward(p, out, lse, nullptr, nullptr, stream);
}

int tensor_forward_gated(const oops_ta_problem& p, const oops_ta_pair& gate, const oops_ta_pair& gated,
                         const oops_ta_pair& plain, float* lse, cudaStream_t stream) {
  return launch_forward(p, gated, lse, &gate, &plain, stream);
}

int forward_device_status(int reset) { return read_tu_device_status(reset); }


}  // namespace oops_ta
