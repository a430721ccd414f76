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

constexpr int kStages = 3;         // K/V ring depth
constexpr int kTileBytes = kTile * kHeadDim * 2;       // 8 KiB: one Q, K or V tile
constexpr int kBiasBytes = kTile * kTile * 2;          // 32 KiB: one bias tile (two 64-key boxes)
constexpr int kFwdThreads = 320;   // 2 softmax warpgroups + producer warp + MMA warp

struct FwdSmem {
  static constexpr int q = 0;
  static constexpr int k = q + 2 * kTileBytes;
  static constexpr int v = k + kStages * kTileBytes;
  static constexpr int bias = v + kStages * kTileBytes;
  static constexpr int bars = bias + 4 * kBiasBytes;
  // barrier indices (8 bytes each)
  static constexpr int q_full = 0;                   // [2]
  static constexpr int k_full = q_full + 2;          // [kStages]
  static constexpr int k_empty = k_full + kStages;   // [kStages]
  static constexpr int v_full = k_empty + kStages;   // [kStages]
  static constexpr int v_empty = v_full + kStages;   // [kStages]
  static constexpr int v_ready = v_empty + kStages;  // [kStages]
  static constexpr int bias_full = v_ready + kStages;  // [2 tiles][2 buffers]
  static constexpr int bias_empty = bias_full + 4;     // [2][2]
  static constexpr int s_full = bias_empty + 4;        // [2]
  static constexpr int p_full = s_full + 2;            // [2]
  static constexpr int o_done = p_full + 2;            // [2]
  static constexpr int num_bars = o_done + 2;
  static constexpr int tmem_slot = bars + num_bars * 8;
  static constexpr int abort_flag = tmem_slot + 4;
  static constexpr int total = abort_flag + 4;
};
constexpr int kFwdSmemBytes = FwdSmem::total + 1024;  // slack to align the base to 1 KiB

struct FwdParams {
  CUtensorMap map_q, map_k, map_v, map_bias;
  void* out;
  int64_t o_sb, o_sr, o_sc, o_sh;
  float* lse;
  const uint8_t* mask;
  int64_t m_sb, m_sr, m_sc;
  int batch, rows, cols, heads, bias_groups;
  int q_pairs, k_tiles;
  int out_vec16;
  float scale;
};

template <typename T, bool HAS_BIAS>
__global__ void __launch_bounds__(kFwdThreads, 1) ta_fwd_kernel(const __grid_constant__ FwdParams P) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + FwdSmem::abort_flag);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + FwdSmem::tmem_slot);
  auto bar = [&](int index) -> uint32_t { return smem_base + FwdSmem::bars + index * 8; };

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

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
  const int KT = P.k_tiles;
  const int g = P.bias_groups == 1 ? 0 : r;
  const bool has_mask = P.mask != nullptr;

  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2; ++i) mbar_init(bar(FwdSmem::q_full + i), 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(FwdSmem::k_full + i), 1);
      mbar_init(bar(FwdSmem::k_empty + i), 1);
      mbar_init(bar(FwdSmem::v_full + i), 1);
      mbar_init(bar(FwdSmem::v_empty + i), 1);
      mbar_init(bar(FwdSmem::v_ready + i), kTile);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar(FwdSmem::bias_full + i), 1);
      mbar_init(bar(FwdSmem::bias_empty + i), kTile);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(FwdSmem::s_full + i), 1);
      mbar_init(bar(FwdSmem::p_full + i), kTile);
      mbar_init(bar(FwdSmem::o_done + i), 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_base + FwdSmem::tmem_slot, 512);
    tmem_relinquish();
    tc_fence_before_sync();
  }
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------ producer (one thread)
    if (lane == 0) {
      bool ok = true;
      for (int w = 0; w < n_tiles; ++w) {
        mbar_expect_tx(bar(FwdSmem::q_full + w), kTileBytes);
        tma_load_5d(smem_base + FwdSmem::q + w * kTileBytes, &P.map_q, bar(FwdSmem::q_full + w), 0, h, q0 + w * kTile, r, b);
      }
      for (int j = 0; j < KT && ok; ++j) {
        const int st = j % kStages, round = j / kStages;
        if (j >= kStages) ok = mbar_wait(bar(FwdSmem::k_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(FwdSmem::k_full + st), kTileBytes);
        tma_load_5d(smem_base + FwdSmem::k + st * kTileBytes, &P.map_k, bar(FwdSmem::k_full + st), 0, h, j * kTile, r, b);
        if (j >= kStages) ok = mbar_wait(bar(FwdSmem::v_empty + st), (round - 1) & 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bar(FwdSmem::v_full + st), kTileBytes);
        tma_load_5d(smem_base + FwdSmem::v + st * kTileBytes, &P.map_v, bar(FwdSmem::v_full + st), 0, h, j * kTile, r, b);
        if (HAS_BIAS) {
          const int buf = j & 1;
          for (int w = 0; w < n_tiles && ok; ++w) {
            const int slot = w * 2 + buf;
            if (j >= 2) ok = mbar_wait(bar(FwdSmem::bias_empty + slot), ((j >> 1) - 1) & 1, abort_flag);
            if (!ok) break;
            mbar_expect_tx(bar(FwdSmem::bias_full + slot), kBiasBytes);
            const uint32_t dst = smem_base + FwdSmem::bias + slot * kBiasBytes;
            tma_load_5d(dst, &P.map_bias, bar(FwdSmem::bias_full + slot), j * kTile, q0 + w * kTile, h, g, b);
            tma_load_5d(dst + kBiasBytes / 2, &P.map_bias, bar(FwdSmem::bias_full + slot), j * kTile + 64,
                        q0 + w * kTile, h, g, b);
          }
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      constexpr uint32_t fmt = Half2<T>::kFormat;
      constexpr uint32_t idesc_qk = instr_desc(fmt, 0, 0, kTile, kTile);
      constexpr uint32_t idesc_pv = instr_desc(fmt, 0, 1, kTile, kHeadDim);
      const uint32_t v_ready_base = has_mask ? FwdSmem::v_ready : FwdSmem::v_full;
      bool ok = true;
      for (int w = 0; w < n_tiles && ok; ++w) ok = mbar_wait(bar(FwdSmem::q_full + w), 0, abort_flag);
      for (int j = 0; j <= KT && ok; ++j) {
        if (j < KT) ok = mbar_wait(bar(FwdSmem::k_full + j % kStages), (j / kStages) & 1, abort_flag);
        for (int w = 0; w < n_tiles && ok; ++w) {
          const uint32_t s_tmem = tmem_base + w * kTile;
          const uint32_t o_tmem = tmem_base + 2 * kTile + w * kHeadDim;
          if (j > 0) {
            const int jj = j - 1, st = jj % kStages;
            ok = mbar_wait(bar(FwdSmem::p_full + w), jj & 1, abort_flag);
            if (ok && w == 0) ok = mbar_wait(bar(v_ready_base + st), (jj / kStages) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            // O[128 x 32] += P[128 x 128] V[128 x 32]; V is MN-major (channel contiguous), 64-byte swizzle:
            // 8-key groups are 512 bytes apart, each 16-key step advances 1024 bytes.
            const uint64_t vdesc = smem_desc(smem_base + FwdSmem::v + st * kTileBytes, 16, 512, kSwizzle64B);
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk)
              mma_ts(o_tmem, s_tmem + kk * 8, vdesc + uint64_t(kk * (1024 >> 4)), idesc_pv, (jj > 0 || kk > 0) ? 1u : 0u);
            mma_commit(bar(FwdSmem::o_done + w));
            if (w == n_tiles - 1) mma_commit(bar(FwdSmem::v_empty + st));
          }
          if (j < KT) {
            const int st = j % kStages;
            tc_fence_after_sync();
            // S[128 x 128] = Q[128 x 32] K[128 x 32]^T; both K-major, 64-byte swizzle: 8-row groups 512 bytes apart,
            // each 16-channel step advances 32 bytes inside the swizzle span.
            const uint64_t qdesc = smem_desc(smem_base + FwdSmem::q + w * kTileBytes, 16, 512, kSwizzle64B);
            const uint64_t kdesc = smem_desc(smem_base + FwdSmem::k + st * kTileBytes, 16, 512, kSwizzle64B);
#pragma unroll
            for (int kk = 0; kk < kHeadDim / 16; ++kk)
              mma_ss(s_tmem, qdesc + uint64_t(kk * 2), kdesc + uint64_t(kk * 2), idesc_qk, kk > 0 ? 1u : 0u);
            mma_commit(bar(FwdSmem::s_full + w));
            if (w == n_tiles - 1) mma_commit(bar(FwdSmem::k_empty + st));
          }
        }
      }
    }
  } else if ((warp >> 2) < n_tiles) {
    // ------------------------------------------------------------------ softmax warpgroups
    const int w = warp >> 2;
    const int t = tid & (kTile - 1);
    const uint32_t lane_field = uint32_t((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_field + w * kTile;
    const uint32_t o_tmem = tmem_base + lane_field + 2 * kTile + w * kHeadDim;
    const int q_index = q0 + w * kTile + t;
    const uint8_t* mask_row = has_mask ? P.mask + b * P.m_sb + int64_t(r) * P.m_sr : nullptr;
    const float scale = P.scale;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < KT && ok; ++j) {
      // keep-bits of this key tile (all threads of a warp hold all four words)
      uint32_t bits[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
      const bool need_bits = has_mask || (j == KT - 1 && (P.cols % kTile) != 0);
      if (need_bits) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = j * kTile + i * 32 + lane;
          bool keep = key < P.cols;
          if (keep && has_mask) keep = mask_row[int64_t(key) * P.m_sc] != 0;
          bits[i] = __ballot_sync(0xffffffffu, keep);
        }
      }
      const bool all_kept = (bits[0] & bits[1] & bits[2] & bits[3]) == 0xffffffffu;
      if (has_mask && w == 0) {
        // Values of dropped keys must not reach the tensor core (0 * inf): clear their rows in shared memory.
        const int st = j % kStages;
        ok = mbar_wait(bar(FwdSmem::v_full + st), (j / kStages) & 1, abort_flag);
        if (!ok) break;
        if (!all_kept && ((bits[t >> 5] >> (t & 31)) & 1u) == 0) {
          uint4* row = reinterpret_cast<uint4*>(smem_gen + FwdSmem::v + st * kTileBytes + t * 64);
          row[0] = row[1] = row[2] = row[3] = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar(FwdSmem::v_ready + st));
      }

      ok = mbar_wait(bar(FwdSmem::s_full + w), j & 1, abort_flag);
      if (!ok) break;
      tc_fence_after_sync();
      float x[kTile];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t raw[32];
        tmem_ld32(s_tmem + c * 32, raw);
#pragma unroll
        for (int i = 0; i < 32; ++i) x[c * 32 + i] = __uint_as_float(raw[i]);
      }
      tmem_wait_ld();

      if (HAS_BIAS) {
        const int slot = w * 2 + (j & 1);
        ok = mbar_wait(bar(FwdSmem::bias_full + slot), (j >> 1) & 1, abort_flag);
        if (!ok) break;
        const uint8_t* tile = smem_gen + FwdSmem::bias + slot * kBiasBytes;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const uint8_t* row = tile + half * (kBiasBytes / 2) + t * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + ((c ^ (t & 7)) << 4));
            const int at = half * 64 + c * 8;
            x[at + 0] = fmaf(x[at + 0], scale, Half2<T>::lo(v.x));
            x[at + 1] = fmaf(x[at + 1], scale, Half2<T>::hi(v.x));
            x[at + 2] = fmaf(x[at + 2], scale, Half2<T>::lo(v.y));
            x[at + 3] = fmaf(x[at + 3], scale, Half2<T>::hi(v.y));
            x[at + 4] = fmaf(x[at + 4], scale, Half2<T>::lo(v.z));
            x[at + 5] = fmaf(x[at + 5], scale, Half2<T>::hi(v.z));
            x[at + 6] = fmaf(x[at + 6], scale, Half2<T>::lo(v.w));
            x[at + 7] = fmaf(x[at + 7], scale, Half2<T>::hi(v.w));
          }
        }
        mbar_arrive(bar(FwdSmem::bias_empty + slot));
      } else {
#pragma unroll
        for (int i = 0; i < kTile; ++i) x[i] *= scale;
      }
      if (!all_kept) {
#pragma unroll
        for (int i = 0; i < kTile; ++i)
          if (((bits[i >> 5] >> (i & 31)) & 1u) == 0) x[i] = -INFINITY;
      }
      float peak = x[0];
#pragma unroll
      for (int i = 1; i < kTile; ++i) peak = fmaxf(peak, x[i]);
      const float m_new = fmaxf(m_run, peak);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = ex2((m_run - m_use) * kLog2e);
      const float shift = -m_use * kLog2e;
      float total = 0.f;
      uint32_t packed[kTile / 2];
#pragma unroll
      for (int i = 0; i < kTile; i += 2) {
        const float p0 = ex2(fmaf(x[i], kLog2e, shift));
        const float p1 = ex2(fmaf(x[i + 1], kLog2e, shift));
        total += p0 + p1;
        packed[i >> 1] = Half2<T>::pack(p0, p1);
      }
      l_run = l_run * alpha + total;
      m_run = m_new;

      if (j > 0) {
        // rescale the running output once the previous P V product has landed
        ok = mbar_wait(bar(FwdSmem::o_done + w), (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t acc[32];
        tmem_ld32(o_tmem, acc);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
        tmem_st32(o_tmem, acc);
      }
      {
        uint32_t part[32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int i = 0; i < 32; ++i) part[i] = packed[c * 32 + i];
          tmem_st32(s_tmem + c * 32, part);
        }
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(FwdSmem::p_full + w));
    }

    if (ok) ok = mbar_wait(bar(FwdSmem::o_done + w), (KT - 1) & 1, abort_flag);
    if (ok) {
      tc_fence_after_sync();
      uint32_t acc[32];
      tmem_ld32(o_tmem, acc);
      tmem_wait_ld();
      if (q_index < P.cols) {
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        uint32_t o2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          o2[i] = Half2<T>::pack(__uint_as_float(acc[2 * i]) * inv, __uint_as_float(acc[2 * i + 1]) * inv);
        T* dst = reinterpret_cast<T*>(P.out) + b * P.o_sb + int64_t(r) * P.o_sr + int64_t(q_index) * P.o_sc + h * P.o_sh;
        if (P.out_vec16) {
          uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
          for (int i = 0; i < 4; ++i) d4[i] = make_uint4(o2[4 * i], o2[4 * i + 1], o2[4 * i + 2], o2[4 * i + 3]);
        } else {
          uint32_t* d1 = reinterpret_cast<uint32_t*>(dst);
          if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) d1[i] = o2[i];
          } else {
            unsigned short* d0 = reinterpret_cast<unsigned short*>(dst);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              d0[2 * i] = (unsigned short)(o2[i] & 0xffffu);
              d0[2 * i + 1] = (unsigned short)(o2[i] >> 16);
            }
          }
        }
        if (P.lse)
          P.lse[((int64_t(b) * P.rows + r) * P.heads + h) * P.cols + q_index] =
              l_run > 0.f ? (m_run + lg2(l_run) * kLn2) : 0.f;
      }
    }
  }

  teardown(abort_flag, tmem_base, 9);
}

}  // namespace

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
  const int64_t ctas = int64_t(p.batch) * p.rows * p.heads * ceil_div(p.cols, 2 * kTile);
  return ctas <= 0x7fffffffll;
}

uint64_t tensor_forward_workspace(const oops_ta_problem&) { return 0; }

int tensor_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream) {
  FwdParams P{};
  int status = encode_pair(&P.map_q, p, p.q, kTile, "query");
  if (!status) status = encode_pair(&P.map_k, p, p.k, kTile, "key");
  if (!status) status = encode_pair(&P.map_v, p, p.v, kTile, "value");
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
  P.out_vec16 = (reinterpret_cast<uintptr_t>(out.ptr) & 15) == 0 && out.sb % 8 == 0 && out.sr % 8 == 0 &&
                out.sc % 8 == 0 && out.sh % 8 == 0;
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
  P.k_tiles = (int)ceil_div(p.cols, kTile);
  P.scale = p.scale;
  const unsigned grid = (unsigned)(int64_t(p.batch) * p.rows * p.heads * P.q_pairs);

  auto launch = [&](auto kernel) -> int {
    static thread_local const void* configured = nullptr;
    if (configured != reinterpret_cast<const void*>(kernel)) {
      const int rc = reserve_smem(kernel, kFwdSmemBytes);
      if (rc) return rc;
      configured = reinterpret_cast<const void*>(kernel);
    }
    kernel<<<grid, kFwdThreads, kFwdSmemBytes, stream>>>(P);
    count_launch();
    return check_launch("tcgen05 forward");
  };
  if (p.dtype == OOPS_TA_BF16)
    return has_bias ? launch(ta_fwd_kernel<__nv_bfloat16, true>) : launch(ta_fwd_kernel<__nv_bfloat16, false>);
  return has_bias ? launch(ta_fwd_kernel<__half, true>) : launch(ta_fwd_kernel<__half, false>);
}

int forward_device_status(int reset) { return read_tu_device_status(reset); }

}  // namespace oops_ta
