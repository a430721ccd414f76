// Layout-agnostic triangle-attention kernels for sm_100a.
//
// These kernels serve every request the tcgen05 kernels do not take: f32 inputs
// (full-precision FFMA products, which is what the reference's "ieee" mode
// promises, oops/runtime/dispatch.py:260-328), head sizes that are not a
// multiple of 16 (the reference accepts 1..256, oops/attention/triangle/triton/
// schedule.py:34), and operands whose strides a TMA descriptor cannot express.
// They follow the operator's definition literally (oops/attention/triangle/
// triton/kernel.py:128-147 scores, :250-261 normalisation, :499-564 dQ,
// :682-714 dK/dV, :856 shared-bias gradient) on blocks of pair rows, with the
// logits of a block held in caller-provided scratch memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <mutex>

#include "ta_internal.h"

namespace oops_ta {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;
constexpr uint64_t kBlockBudget = 256ull << 20;  // bytes of logits per block of rows

enum Epilogue { EPI_SCORES = 0, EPI_PROBS = 1, EPI_STORE = 2, EPI_DSCORES = 3 };

struct Operand {
  const void* ptr;
  int64_t sb, sr, sh;  // batch, pair-row and head strides (elements)
  int64_t s_mn, s_k;   // stride of this side's free index and of the contraction index
  int row_base;        // added to the block-relative row (0 for scratch, first row for user tensors)
};

struct GemmArgs {
  Operand a, b;
  int M, N, K;
  int heads, block_rows, row0;
  const uint8_t* mask;
  int64_t mask_sb, mask_sr, mask_sc;
  int mask_on_k;  // the contraction index is the key: masked keys contribute nothing
  float alpha;
  float* ws_out;
  const float* ws_in;
  const float* lse;
  const float* delta;
  int rows_total;
  const void* bias;
  int64_t bias_sb, bias_sg, bias_sh, bias_sq, bias_sk;
  int bias_groups, bias_dtype;
  oops_ta_pair dst;
  int dst_dtype;
  int zero_masked_rows;
  void* dbias_rows;
  int64_t db_sb, db_sg, db_sh, db_sq, db_sk;
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
  if (dtype == OOPS_TA_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == OOPS_TA_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int64_t i, int dtype, float v) {
  if (dtype == OOPS_TA_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == OOPS_TA_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// C[z][m][n] = sum_k A[z][m][k] * B[z][n][k] over independent problems z = (batch, row, head).
template <typename TA, typename TB, int EPI>
__global__ void __launch_bounds__(THREADS) gemm_kernel(const GemmArgs g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int z = blockIdx.x;
  const int h = z % g.heads;
  const int rest = z / g.heads;
  const int rr = rest % g.block_rows;
  const int b = rest / g.block_rows;
  const int r = g.row0 + rr;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.z * BN;

  const TA* A = reinterpret_cast<const TA*>(g.a.ptr) + b * g.a.sb + int64_t(rr + g.a.row_base) * g.a.sr + h * g.a.sh;
  const TB* B = reinterpret_cast<const TB*>(g.b.ptr) + b * g.b.sb + int64_t(rr + g.b.row_base) * g.b.sr + h * g.b.sh;
  const uint8_t* keep = g.mask ? g.mask + b * g.mask_sb + int64_t(r) * g.mask_sr : nullptr;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int ty = tid / 16, tx = tid % 16;
  const bool a_k_fast = g.a.s_k == 1, b_k_fast = g.b.s_k == 1;
  for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / THREADS; ++i) {
      const int idx = tid + i * THREADS;
      const int kk = a_k_fast ? idx % BK : idx / BM;
      const int mm = a_k_fast ? idx / BK : idx % BM;
      float v = 0.f;
      if (m0 + mm < g.M && k0 + kk < g.K) v = to_float<TA>(A[int64_t(m0 + mm) * g.a.s_mn + int64_t(k0 + kk) * g.a.s_k]);
      As[kk][mm] = v;
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / THREADS; ++i) {
      const int idx = tid + i * THREADS;
      const int kk = b_k_fast ? idx % BK : idx / BN;
      const int nn = b_k_fast ? idx / BK : idx % BN;
      float v = 0.f;
      if (n0 + nn < g.N && k0 + kk < g.K) {
        const bool dropped = g.mask_on_k && keep && keep[int64_t(k0 + kk) * g.mask_sc] == 0;
        if (!dropped) v = to_float<TB>(B[int64_t(n0 + nn) * g.b.s_mn + int64_t(k0 + kk) * g.b.s_k]);
      }
      Bs[kk][nn] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      const float value = acc[i][j];
      if (EPI == EPI_SCORES || EPI == EPI_PROBS) {
        // m = query, n = key
        const bool kept = !keep || keep[int64_t(n) * g.mask_sc] != 0;
        float s = value * g.alpha;
        if (g.bias) {
          const int64_t group = g.bias_groups == 1 ? 0 : r;
          s += load_as_float(g.bias,
                             b * g.bias_sb + group * g.bias_sg + h * g.bias_sh + int64_t(m) * g.bias_sq +
                                 int64_t(n) * g.bias_sk,
                             g.bias_dtype);
        }
        float result;
        if (EPI == EPI_SCORES) {
          result = kept ? s : -CUDART_INF_F;
        } else {
          const float norm = g.lse[((int64_t(b) * g.rows_total + r) * g.heads + h) * g.M + m];
          result = kept ? expf(s - norm) : 0.f;
        }
        g.ws_out[(int64_t(z) * g.M + m) * g.N + n] = result;
      } else if (EPI == EPI_DSCORES) {
        const bool kept = !keep || keep[int64_t(n) * g.mask_sc] != 0;
        const int64_t at = (int64_t(z) * g.M + m) * g.N + n;
        const float ds = kept ? g.ws_in[at] * (value - g.delta[int64_t(z) * g.M + m]) : 0.f;
        g.ws_out[at] = ds;
        if (g.dbias_rows) {
          store_from_float(g.dbias_rows,
                           b * g.db_sb + int64_t(r) * g.db_sg + h * g.db_sh + int64_t(m) * g.db_sq + int64_t(n) * g.db_sk,
                           g.bias_dtype, ds);
        }
      } else {
        // m = cell column (query or key), n = channel
        float result = value * g.alpha;
        if (g.zero_masked_rows && keep && keep[int64_t(m) * g.mask_sc] == 0) result = 0.f;
        store_from_float(g.dst.ptr, b * g.dst.sb + int64_t(r) * g.dst.sr + int64_t(m) * g.dst.sc + h * g.dst.sh + n,
                         g.dst_dtype, result);
      }
    }
  }
}

// One warp per logit row: max, sum, normalise in place; lse = max + log(sum), or 0 with no kept key.
__global__ void softmax_rows_kernel(float* scores, int64_t num_rows, int cols, float* lse, int heads, int block_rows,
                                    int row0, int rows_total) {
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (row >= num_rows) return;
  float* s = scores + row * cols;
  float peak = -CUDART_INF_F;
  for (int i = lane; i < cols; i += 32) peak = fmaxf(peak, s[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  const bool empty = !(peak > -CUDART_INF_F) && !(peak != peak);
  float total = 0.f;
  if (!empty) {
    for (int i = lane; i < cols; i += 32) {
      const float e = expf(s[i] - peak);
      s[i] = e;
      total += e;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  const float inv = empty ? 0.f : 1.f / total;
  for (int i = lane; i < cols; i += 32) s[i] = empty ? 0.f : s[i] * inv;
  if (lse && lane == 0) {
    const int64_t q = row % cols;  // rows of a problem are its queries (square logits)
    const int64_t z = row / cols;
    const int h = z % heads;
    const int64_t rest = z / heads;
    const int rr = rest % block_rows;
    const int64_t b = rest / block_rows;
    lse[((b * rows_total + row0 + rr) * heads + h) * cols + q] = empty ? 0.f : peak + logf(total);
  }
}

// delta[z][q] = sum_d out * dout, one warp per (problem, query).
__global__ void delta_kernel(oops_ta_pair out, oops_ta_pair dout, int dtype, float* delta, int64_t num, int cols,
                             int heads, int block_rows, int row0, int head_dim) {
  const int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (item >= num) return;
  const int64_t q = item % cols;
  const int64_t z = item / cols;
  const int h = z % heads;
  const int64_t rest = z / heads;
  const int r = row0 + rest % block_rows;
  const int64_t b = rest / block_rows;
  const int64_t o_at = b * out.sb + int64_t(r) * out.sr + q * out.sc + h * out.sh;
  const int64_t d_at = b * dout.sb + int64_t(r) * dout.sr + q * dout.sc + h * dout.sh;
  float total = 0.f;
  for (int d = lane; d < head_dim; d += 32)
    total += load_as_float(out.ptr, o_at + d, dtype) * load_as_float(dout.ptr, d_at + d, dtype);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) delta[item] = total;
}

// acc[b][h][q][k] += sum over the block's rows of ds[(b, rr, h)][q][k]; fixed order, no atomics.
__global__ void shared_bias_accumulate_kernel(const float* ds, float* acc, int64_t plane, int heads, int block_rows,
                                              int batch) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = int64_t(batch) * heads * plane;
  if (i >= total) return;
  const int64_t e = i % plane;
  const int64_t bh = i / plane;
  const int h = bh % heads;
  const int64_t b = bh / heads;
  float sum = acc[i];
  for (int rr = 0; rr < block_rows; ++rr) sum += ds[((b * block_rows + rr) * heads + h) * plane + e];
  acc[i] = sum;
}

__global__ void shared_bias_store_kernel(const float* acc, void* dbias, int dtype, int64_t sb, int64_t sh, int64_t sq,
                                         int64_t sk, int batch, int heads, int cols) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = int64_t(batch) * heads * cols * cols;
  if (i >= total) return;
  const int k = i % cols;
  const int q = (i / cols) % cols;
  const int h = (i / (int64_t(cols) * cols)) % heads;
  const int64_t b = i / (int64_t(cols) * cols * heads);
  store_from_float(dbias, b * sb + h * sh + int64_t(q) * sq + int64_t(k) * sk, dtype, acc[i]);
}

template <int EPI, typename TA, typename TB>
int launch_gemm(const GemmArgs& g, int batch, cudaStream_t stream, const char* what) {
  const int64_t problems = int64_t(batch) * g.block_rows * g.heads;
  dim3 grid((unsigned)problems, (unsigned)ceil_div(g.M, BM), (unsigned)ceil_div(g.N, BN));
  gemm_kernel<TA, TB, EPI><<<grid, THREADS, 0, stream>>>(g);
  count_launch();
  return check_launch(what);
}

template <int EPI, bool A_IS_SCRATCH>
int launch_gemm_dtype(const GemmArgs& g, int dtype, int batch, cudaStream_t stream, const char* what) {
  if (A_IS_SCRATCH) {
    if (dtype == OOPS_TA_F32) return launch_gemm<EPI, float, float>(g, batch, stream, what);
    if (dtype == OOPS_TA_F16) return launch_gemm<EPI, float, __half>(g, batch, stream, what);
    return launch_gemm<EPI, float, __nv_bfloat16>(g, batch, stream, what);
  }
  if (dtype == OOPS_TA_F32) return launch_gemm<EPI, float, float>(g, batch, stream, what);
  if (dtype == OOPS_TA_F16) return launch_gemm<EPI, __half, __half>(g, batch, stream, what);
  return launch_gemm<EPI, __nv_bfloat16, __nv_bfloat16>(g, batch, stream, what);
}

int block_rows_for(const oops_ta_problem& p, uint64_t budget = kBlockBudget) {
  const uint64_t per_row = uint64_t(p.batch) * p.heads * p.cols * p.cols * sizeof(float);
  uint64_t rows = std::max<uint64_t>(1, budget / std::max<uint64_t>(per_row, 1));
  return (int)std::min<uint64_t>(rows, (uint64_t)p.rows);
}

uint64_t align256(uint64_t v) { return (v + 255) & ~uint64_t(255); }

Operand user_operand(const oops_ta_pair& t, int64_t s_mn, int64_t s_k, int row0) {
  return Operand{t.ptr, t.sb, t.sr, t.sh, s_mn, s_k, row0};
}

Operand scratch_operand(const float* ptr, int block_rows, int heads, int cols, bool transposed) {
  const int64_t plane = int64_t(cols) * cols;
  return Operand{ptr, int64_t(block_rows) * heads * plane, int64_t(heads) * plane, plane,
                 transposed ? 1 : int64_t(cols), transposed ? int64_t(cols) : 1, 0};
}

void fill_common(GemmArgs& g, const oops_ta_problem& p, int block_rows, int row0) {
  g.heads = p.heads;
  g.block_rows = block_rows;
  g.row0 = row0;
  g.rows_total = p.rows;
  g.mask = p.mask;
  g.mask_sb = p.mask_sb;
  g.mask_sr = p.mask_sr;
  g.mask_sc = p.mask_sc;
  g.alpha = 1.f;
}

void fill_bias(GemmArgs& g, const oops_ta_problem& p) {
  g.bias = p.bias_groups ? p.bias : nullptr;
  g.bias_sb = p.bias_sb;
  g.bias_sg = p.bias_sg;
  g.bias_sh = p.bias_sh;
  g.bias_sq = p.bias_sq;
  g.bias_sk = p.bias_sk;
  g.bias_groups = p.bias_groups;
  g.bias_dtype = p.bias_dtype;
}

}  // namespace

uint64_t generic_forward_workspace(const oops_ta_problem& p) {
  const int rows = block_rows_for(p);
  return align256(uint64_t(p.batch) * rows * p.heads * p.cols * p.cols * sizeof(float));
}

uint64_t generic_backward_workspace(const oops_ta_problem& p, const oops_ta_grads& g) {
  const int rows = block_rows_for(p);
  const uint64_t logits = align256(uint64_t(p.batch) * rows * p.heads * p.cols * p.cols * sizeof(float));
  const uint64_t delta = align256(uint64_t(p.batch) * rows * p.heads * p.cols * sizeof(float));
  uint64_t total = 2 * logits + delta;
  if (g.dbias && p.bias_groups == 1) total += align256(uint64_t(p.batch) * p.heads * p.cols * p.cols * sizeof(float));
  return total;
}

namespace {
int forward_blocks(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, float* logits, int block,
                   cudaStream_t stream);
}

int generic_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream) {
  if (p.workspace_bytes < generic_forward_workspace(p) || !p.workspace)
    return fail(OOPS_TA_WORKSPACE_TOO_SMALL, "forward needs %llu scratch bytes, got %llu",
                (unsigned long long)generic_forward_workspace(p), (unsigned long long)p.workspace_bytes);
  return forward_blocks(p, out, lse, reinterpret_cast<float*>(p.workspace), block_rows_for(p), stream);
}

namespace {
// Forward pass over blocks of `block` pair rows whose logits live in `logits`.
int forward_blocks(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, float* logits, int block,
                   cudaStream_t stream) {
  for (int row0 = 0; row0 < p.rows; row0 += block) {
    const int rows = std::min(block, p.rows - row0);
    GemmArgs s{};
    fill_common(s, p, rows, row0);
    fill_bias(s, p);
    s.a = user_operand(p.q, p.q.sc, 1, row0);
    s.b = user_operand(p.k, p.k.sc, 1, row0);
    s.M = p.cols;
    s.N = p.cols;
    s.K = p.head_dim;
    s.alpha = p.scale;
    s.ws_out = logits;
    int status = launch_gemm_dtype<EPI_SCORES, false>(s, p.dtype, p.batch, stream, "generic scores");
    if (status) return status;

    const int64_t logit_rows = int64_t(p.batch) * rows * p.heads * p.cols;
    softmax_rows_kernel<<<(unsigned)ceil_div(logit_rows * 32, 256), 256, 0, stream>>>(logits, logit_rows, p.cols, lse,
                                                                                      p.heads, rows, row0, p.rows);
    count_launch();
    status = check_launch("generic softmax");
    if (status) return status;

    GemmArgs o{};
    fill_common(o, p, rows, row0);
    o.a = scratch_operand(logits, rows, p.heads, p.cols, false);
    o.b = user_operand(p.v, 1, p.v.sc, row0);
    o.M = p.cols;
    o.N = p.head_dim;
    o.K = p.cols;
    o.mask_on_k = 1;
    o.dst = out;
    o.dst_dtype = p.dtype;
    status = launch_gemm_dtype<EPI_STORE, true>(o, p.dtype, p.batch, stream, "generic values");
    if (status) return status;
  }
  return OOPS_TA_OK;
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// Forward pass with built-in scratch memory
// ---------------------------------------------------------------------------------------------
// Some hosts may not allocate device memory at the time they call in: a serving process whose memory
// pool was sized and frozen at start-up, a real-time loop where cudaMalloc's implicit device
// synchronisation is not acceptable, or code that runs between stream-capture begin and end.  For them
// the logits of a block of rows live in this fixed array instead of a caller-provided workspace.  Every
// GPU that loads the library holds the array until the process exits, so it is kept modest.
constexpr uint64_t kStaticScratchBytes = 32ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// The array's name is only a host-side handle; kernels need its device address, which differs per device.
int static_scratch_address(float** address) {
  constexpr int kMaxDevices = 64;
  static std::mutex lock;
  static void* cached[kMaxDevices] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(OOPS_TA_CUDA_ERROR, "cudaGetDevice failed");
  std::lock_guard<std::mutex> guard(lock);
  if (!cached[device]) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || !ptr)
      return fail(OOPS_TA_CUDA_ERROR, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(err));
    cached[device] = ptr;
  }
  *address = reinterpret_cast<float*>(cached[device]);
  return OOPS_TA_OK;
}
}  // namespace

uint64_t static_forward_capacity() { return kStaticScratchBytes; }

int static_forward(const oops_ta_problem& p, const oops_ta_pair& out, float* lse, cudaStream_t stream) {
  const uint64_t per_row = uint64_t(p.batch) * p.heads * p.cols * p.cols * sizeof(float);
  if (per_row > kStaticScratchBytes)
    return fail(OOPS_TA_LIMIT_EXCEEDED,
                "one pair row needs batch*heads*cols*cols*4 = %llu scratch bytes, the built-in scratch holds %llu",
                (unsigned long long)per_row, (unsigned long long)kStaticScratchBytes);
  float* logits = nullptr;
  const int status = static_scratch_address(&logits);
  if (status) return status;
  // every logit of a block is written before it is read, so nothing has to be cleared between calls
  return forward_blocks(p, out, lse, logits, block_rows_for(p, kStaticScratchBytes), stream);
}

int generic_backward(const oops_ta_problem& p, const oops_ta_pair& out, const oops_ta_pair& dout, const float* lse,
                     const oops_ta_grads& g, cudaStream_t stream) {
  const uint64_t need = generic_backward_workspace(p, g);
  if (p.workspace_bytes < need || !p.workspace)
    return fail(OOPS_TA_WORKSPACE_TOO_SMALL, "backward needs %llu scratch bytes, got %llu", (unsigned long long)need,
                (unsigned long long)p.workspace_bytes);
  const int block = block_rows_for(p);
  const uint64_t logits_bytes = align256(uint64_t(p.batch) * block * p.heads * p.cols * p.cols * sizeof(float));
  const uint64_t delta_bytes = align256(uint64_t(p.batch) * block * p.heads * p.cols * sizeof(float));
  char* base = reinterpret_cast<char*>(p.workspace);
  float* probs = reinterpret_cast<float*>(base);
  float* dscores = reinterpret_cast<float*>(base + logits_bytes);
  float* delta = reinterpret_cast<float*>(base + 2 * logits_bytes);
  float* shared_acc = reinterpret_cast<float*>(base + 2 * logits_bytes + delta_bytes);
  const bool shared_bias_grad = g.dbias && p.bias_groups == 1;
  const bool row_bias_grad = g.dbias && p.bias_groups > 1;
  const int64_t plane = int64_t(p.cols) * p.cols;
  if (shared_bias_grad) {
    if (cudaMemsetAsync(shared_acc, 0, size_t(p.batch) * p.heads * plane * sizeof(float), stream) != cudaSuccess)
      return fail(OOPS_TA_CUDA_ERROR, "cudaMemsetAsync failed");
  }
  const bool need_ds = g.dq.ptr || g.dk.ptr || g.dbias;

  for (int row0 = 0; row0 < p.rows; row0 += block) {
    const int rows = std::min(block, p.rows - row0);
    int status;
    {  // P = exp(scale * q.k + bias - lse), 0 at dropped keys
      GemmArgs s{};
      fill_common(s, p, rows, row0);
      fill_bias(s, p);
      s.a = user_operand(p.q, p.q.sc, 1, row0);
      s.b = user_operand(p.k, p.k.sc, 1, row0);
      s.M = p.cols;
      s.N = p.cols;
      s.K = p.head_dim;
      s.alpha = p.scale;
      s.ws_out = probs;
      s.lse = lse;
      status = launch_gemm_dtype<EPI_PROBS, false>(s, p.dtype, p.batch, stream, "generic probabilities");
      if (status) return status;
    }
    if (g.dv.ptr) {  // dV[k][d] = sum_q P[q][k] dO[q][d]
      GemmArgs a{};
      fill_common(a, p, rows, row0);
      a.a = scratch_operand(probs, rows, p.heads, p.cols, true);
      a.b = user_operand(dout, 1, dout.sc, row0);
      a.M = p.cols;
      a.N = p.head_dim;
      a.K = p.cols;
      a.dst = g.dv;
      a.dst_dtype = p.dtype;
      a.zero_masked_rows = 1;
      status = launch_gemm_dtype<EPI_STORE, true>(a, p.dtype, p.batch, stream, "generic dV");
      if (status) return status;
    }
    if (!need_ds) continue;
    {
      const int64_t items = int64_t(p.batch) * rows * p.heads * p.cols;
      delta_kernel<<<(unsigned)ceil_div(items * 32, 256), 256, 0, stream>>>(out, dout, p.dtype, delta, items, p.cols,
                                                                            p.heads, rows, row0, p.head_dim);
      count_launch();
      status = check_launch("generic delta");
      if (status) return status;
    }
    {  // dS = P * (dO.V^T - delta), 0 at dropped keys; per-row bias gradient is dS itself
      GemmArgs a{};
      fill_common(a, p, rows, row0);
      a.a = user_operand(dout, dout.sc, 1, row0);
      a.b = user_operand(p.v, p.v.sc, 1, row0);
      a.M = p.cols;
      a.N = p.cols;
      a.K = p.head_dim;
      a.ws_in = probs;
      a.ws_out = dscores;
      a.delta = delta;
      a.bias_dtype = p.bias_dtype;
      if (row_bias_grad) {
        a.dbias_rows = g.dbias;
        a.db_sb = g.dbias_sb;
        a.db_sg = g.dbias_sg;
        a.db_sh = g.dbias_sh;
        a.db_sq = g.dbias_sq;
        a.db_sk = g.dbias_sk;
      }
      status = launch_gemm_dtype<EPI_DSCORES, false>(a, p.dtype, p.batch, stream, "generic dS");
      if (status) return status;
    }
    if (g.dq.ptr) {  // dQ[q][d] = scale * sum_k dS[q][k] K[k][d]
      GemmArgs a{};
      fill_common(a, p, rows, row0);
      a.a = scratch_operand(dscores, rows, p.heads, p.cols, false);
      a.b = user_operand(p.k, 1, p.k.sc, row0);
      a.M = p.cols;
      a.N = p.head_dim;
      a.K = p.cols;
      a.mask_on_k = 1;
      a.alpha = p.scale;
      a.dst = g.dq;
      a.dst_dtype = p.dtype;
      status = launch_gemm_dtype<EPI_STORE, true>(a, p.dtype, p.batch, stream, "generic dQ");
      if (status) return status;
    }
    if (g.dk.ptr) {  // dK[k][d] = scale * sum_q dS[q][k] Q[q][d]
      GemmArgs a{};
      fill_common(a, p, rows, row0);
      a.a = scratch_operand(dscores, rows, p.heads, p.cols, true);
      a.b = user_operand(p.q, 1, p.q.sc, row0);
      a.M = p.cols;
      a.N = p.head_dim;
      a.K = p.cols;
      a.alpha = p.scale;
      a.dst = g.dk;
      a.dst_dtype = p.dtype;
      a.zero_masked_rows = 1;
      status = launch_gemm_dtype<EPI_STORE, true>(a, p.dtype, p.batch, stream, "generic dK");
      if (status) return status;
    }
    if (shared_bias_grad) {
      const int64_t total = int64_t(p.batch) * p.heads * plane;
      shared_bias_accumulate_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, stream>>>(dscores, shared_acc, plane,
                                                                                       p.heads, rows, p.batch);
      count_launch();
      status = check_launch("generic shared-bias accumulate");
      if (status) return status;
    }
  }
  if (shared_bias_grad) {
    const int64_t total = int64_t(p.batch) * p.heads * plane;
    shared_bias_store_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, stream>>>(
        shared_acc, g.dbias, (p.flags & OOPS_TA_FLAG_DBIAS_F32) != 0 ? int(OOPS_TA_F32) : p.bias_dtype, g.dbias_sb,
        g.dbias_sh, g.dbias_sq, g.dbias_sk, p.batch, p.heads, p.cols);
    count_launch();
    const int status = check_launch("generic shared-bias store");
    if (status) return status;
  }
  return OOPS_TA_OK;
}

}  // namespace oops_ta
