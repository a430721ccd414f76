// Pair validity of a packed ragged batch: for sample s with n_s tokens, pair[s][i][j] = token[s][i] && token[s][j],
// written as the concatenation of the samples' row-major n_s x n_s squares.  This is the packed arm of the reference's
// pair_mask_from_token_mask (oops/mask/pair_mask_from_token_mask.py:33-103, kernel oops/mask/triton/); its dense arm is
// one broadcast AND and stays in the host language.  Byte work bound by the store bandwidth: one thread writes 16
// consecutive cells of one row (one 16-byte store), the row's own token byte and the 16 column bytes are the loads.
#include "ta_internal.h"

namespace oops_ta {
namespace {

constexpr int kMaxSamples = 1024;
constexpr int kCellsPerThread = 16;

// token_offsets: samples + 1 cumulative token counts.  Every block rebuilds the cumulative *chunk* counts of the
// samples in shared memory (a sample's rows are padded to whole 16-cell chunks only in this index space, never in
// the output), then a thread finds its sample by bisection.
__global__ void packed_pair_mask_kernel(const uint8_t* __restrict__ tokens, const int64_t* __restrict__ token_offsets,
                                        int samples, uint8_t* __restrict__ out) {
  __shared__ int64_t chunk_start[kMaxSamples + 1];  // first chunk of sample s in the launch's chunk index space
  __shared__ int64_t cell_start[kMaxSamples + 1];   // first output cell of sample s
  if (threadIdx.x == 0) {
    int64_t chunks = 0, cells = 0;
    for (int s = 0; s < samples; ++s) {
      chunk_start[s] = chunks;
      cell_start[s] = cells;
      const int64_t n = token_offsets[s + 1] - token_offsets[s];
      chunks += n * ((n + kCellsPerThread - 1) / kCellsPerThread);
      cells += n * n;
    }
    chunk_start[samples] = chunks;
    cell_start[samples] = cells;
  }
  __syncthreads();
  const int64_t chunk = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (chunk >= chunk_start[samples]) return;
  int lo = 0, hi = samples;  // chunk_start[lo] <= chunk < chunk_start[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_start[mid] <= chunk) lo = mid; else hi = mid;
  }
  const int64_t first = token_offsets[lo], n = token_offsets[lo + 1] - first;
  const int64_t per_row = (n + kCellsPerThread - 1) / kCellsPerThread;
  const int64_t local = chunk - chunk_start[lo];
  const int64_t row = local / per_row, col0 = (local % per_row) * kCellsPerThread;
  const bool row_valid = tokens[first + row] != 0;
  uint8_t cells[kCellsPerThread];
#pragma unroll
  for (int i = 0; i < kCellsPerThread; ++i)
    cells[i] = (col0 + i < n && row_valid && tokens[first + col0 + i] != 0) ? 1 : 0;
  uint8_t* dst = out + cell_start[lo] + row * n + col0;
  if (col0 + kCellsPerThread <= n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(cells);
  } else {
    for (int i = 0; i < kCellsPerThread && col0 + i < n; ++i) dst[i] = cells[i];
  }
}

}  // namespace

int packed_pair_mask(const uint8_t* tokens, const int64_t* token_offsets, int samples, int64_t chunks, uint8_t* out,
                     cudaStream_t stream) {
  if (samples > kMaxSamples) return OOPS_TA_UNSUPPORTED_LAYOUT;
  if (chunks == 0) return OOPS_TA_OK;
  const int threads = 256;
  const int64_t blocks = (chunks + threads - 1) / threads;
  if (blocks > 0x7fffffff) return OOPS_TA_UNSUPPORTED_LAYOUT;
  packed_pair_mask_kernel<<<unsigned(blocks), threads, 0, stream>>>(tokens, token_offsets, samples, out);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? OOPS_TA_OK : OOPS_TA_CUDA_ERROR;
}

int packed_pair_mask_max_samples() { return kMaxSamples; }

}  // namespace oops_ta
