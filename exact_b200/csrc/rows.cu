// Zero-compacted rows: the exchange format of the row-sharded aggregation.
//
// The dense operands that cross NVLink before an SpMM are, past the first layer, outputs of
// ReLU + dropout (forward) or gradients that went through their masks (backward): about three quarters
// of the entries are exact zeros.  A shard [n, K] fp32 is sent as
//     mask    uint32 [n, K/32]   bit c % 32 of word c / 32 set when element (row, c) is kept
//     rowoff  int64  [n + 1]     exclusive prefix sum of the rows' popcounts
//     vals    fp32   [rowoff[n]] the kept elements, row-major
// and expanded back to dense rows in the receiver's HBM.  An element is kept when any of its 32 bits is
// set: +0.0 is the only value dropped, so expand(compact(x)) == x bit for bit (NaN, inf, denormals and
// -0.0 included).
//
// The reference is single-GPU and has no counterpart of these kernels.
#include "exact_b200.h"
#include "common.cuh"

namespace exb {

constexpr int kRowsWarps = 8;

// One warp per row: mask words and the row's popcount.
__global__ void __launch_bounds__(kRowsWarps * 32)
rows_mask_count_kernel(const float* __restrict__ x, long long n, int K, long long ldx, uint32_t* __restrict__ mask,
                       int* __restrict__ rowcnt) {
  const int lane = threadIdx.x & 31;
  const int W = K >> 5;
  for (long long row = (long long)blockIdx.x * kRowsWarps + (threadIdx.x >> 5); row < n;
       row += (long long)gridDim.x * kRowsWarps) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(x + row * ldx);
    int cnt = 0;
    for (int w = 0; w < W; w++) {
      const uint32_t bits = __ldg(src + w * 32 + lane);
      const uint32_t m = __ballot_sync(0xffffffffu, bits != 0u);
      if (lane == 0) mask[row * W + w] = m;
      cnt += __popc(m);
    }
    if (lane == 0) rowcnt[row] = cnt;
  }
}

// One warp per row: kept elements to vals[rowoff[row] ...] in column order.
__global__ void __launch_bounds__(kRowsWarps * 32)
rows_compact_write_kernel(const float* __restrict__ x, long long n, int K, long long ldx,
                          const long long* __restrict__ rowoff, float* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const int W = K >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  for (long long row = (long long)blockIdx.x * kRowsWarps + (threadIdx.x >> 5); row < n;
       row += (long long)gridDim.x * kRowsWarps) {
    const uint32_t* src = reinterpret_cast<const uint32_t*>(x + row * ldx);
    uint32_t* dst = reinterpret_cast<uint32_t*>(vals) + rowoff[row];
    int pos = 0;
    for (int w = 0; w < W; w++) {
      const uint32_t bits = __ldg(src + w * 32 + lane);
      const uint32_t m = __ballot_sync(0xffffffffu, bits != 0u);
      if (bits != 0u) dst[pos + __popc(m & lt)] = bits;
      pos += __popc(m);
    }
  }
}

// One warp per output row.  Rows come in blocks of `block_rows` (one block per sending shard); block b
// has its own rowoff array (stride rowoff_stride) and vals array (stride vals_stride).
__global__ void __launch_bounds__(kRowsWarps * 32)
rows_expand_kernel(const uint32_t* __restrict__ mask, const long long* __restrict__ rowoff,
                   const float* __restrict__ vals, long long n, int K, long long block_rows,
                   long long rowoff_stride, long long vals_stride, float* __restrict__ out, long long ldo) {
  const int lane = threadIdx.x & 31;
  const int W = K >> 5;
  const uint32_t lt = (1u << lane) - 1u;
  for (long long row = (long long)blockIdx.x * kRowsWarps + (threadIdx.x >> 5); row < n;
       row += (long long)gridDim.x * kRowsWarps) {
    const long long b = row / block_rows, r = row - b * block_rows;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(vals + b * vals_stride) + rowoff[b * rowoff_stride + r];
    const uint32_t* mrow = mask + row * W;
    uint32_t* dst = reinterpret_cast<uint32_t*>(out + row * ldo);
    int pos = 0;
    for (int w = 0; w < W; w++) {
      const uint32_t m = __ldg(mrow + w);
      uint32_t bits = 0u;
      if ((m >> lane) & 1u) bits = __ldg(src + pos + __popc(m & lt));
      __stcs(dst + w * 32 + lane, bits);
      pos += __popc(m);
    }
  }
}

static int rows_grid(long long n) {
  long long g = (n + kRowsWarps - 1) / kRowsWarps;
  const long long cap = (long long)sm_count() * 16;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_rows_mask_count(const float* x, int64_t n, int64_t K, int64_t ldx, uint32_t* mask, int32_t* rowcnt,
                          void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K % 32 == 0 && ldx >= K, "rows_mask_count: K must be a positive multiple of 32 and ldx >= K");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(x && mask && rowcnt, "rows_mask_count: null pointer");
  rows_mask_count_kernel<<<rows_grid(n), kRowsWarps * 32, 0, (cudaStream_t)stream>>>(x, n, (int)K, ldx, mask, rowcnt);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_rows_compact_write(const float* x, int64_t n, int64_t K, int64_t ldx, const int64_t* rowoff, float* vals,
                             void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K % 32 == 0 && ldx >= K, "rows_compact_write: K must be a positive multiple of 32 and ldx >= K");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(x && rowoff && vals, "rows_compact_write: null pointer");
  rows_compact_write_kernel<<<rows_grid(n), kRowsWarps * 32, 0, (cudaStream_t)stream>>>(
      x, n, (int)K, ldx, reinterpret_cast<const long long*>(rowoff), vals);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_rows_expand(const uint32_t* mask, const int64_t* rowoff, const float* vals, int64_t n, int64_t K,
                      int64_t block_rows, int64_t rowoff_stride, int64_t vals_stride, float* out, int64_t ldo,
                      void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K % 32 == 0 && ldo >= K && block_rows > 0, "rows_expand: K must be a positive multiple of 32, ldo >= K, block_rows > 0");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(mask && rowoff && vals && out, "rows_expand: null pointer");
  rows_expand_kernel<<<rows_grid(n), kRowsWarps * 32, 0, (cudaStream_t)stream>>>(
      mask, reinterpret_cast<const long long*>(rowoff), vals, n, (int)K, block_rows, rowoff_stride, vals_stride, out, ldo);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
