// Exchange kernels of the feature-parallel aggregation of a row-sharded run.
//
// Between aggregations every rank holds the rows of its shard with all K columns (the dense layers, the
// compression and the masks are row-local).  For an aggregation out = A x the ranks switch to a column
// split: rank q receives columns [q Kp, (q + 1) Kp) of EVERY row, multiplies the whole adjacency with that
// [N, Kp] slice, and sends each row block of the result back to its owner.  Two all-to-all exchanges of
// N K / P elements per rank replace the all-gather of N K (P - 1) / P elements a row-split SpMM needs, every
// rank does the same share of every row (no imbalance from hub rows), and a rank's gathers range over
// N Kp instead of N K elements, which the L2 holds a P times larger part of.
//
// Both exchanges are plain stores into the peers' buffers (mapped with CUDA IPC, see peer.cu): a rank writes
// its piece to all ranks in one kernel; the caller orders the stores before the readers with a one-word
// all-reduce.  Pieces are moved as 16-byte vectors; consecutive threads write consecutive addresses of one
// destination, so the stores cross NVLink as full lines.
//
// The reference is single-GPU and has no counterpart.
#include "common.cuh"
#include "exact_b200.h"

namespace exb {

constexpr int kColMaxDst = 8;

struct ColDst {
  float* p[kColMaxDst];
  int n;
};

// x [n, K] (pitch ldx) -> dst[q][(row0 + r) * Kp + c] = x[r, q * Kp + c] * rowscale[r], zero past column K.
__global__ void __launch_bounds__(256)
cols_scatter_kernel(const float* __restrict__ x, long long n, int K, long long ldx, const float* __restrict__ rowscale,
                    long long row0, int Kp, const __grid_constant__ ColDst dst) {
  const int kp4 = Kp >> 2;
  const long long per_dst = n * kp4;              // 16-byte pieces one destination receives: a contiguous block
  const long long total = per_dst * dst.n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    // destination-major: consecutive threads write consecutive addresses of ONE destination across rows (its
    // [n, Kp] block is dense), so every warp store is 512 contiguous bytes whatever Kp; the reads are strided
    // pieces of Kp * 4 bytes, which local memory serves well
    const int q = (int)(i / per_dst);
    const long long rem = i - (long long)q * per_dst;
    const long long r = rem / kp4;
    const int cc = (int)(rem - r * kp4);
    const int c4 = q * kp4 + cc;                  // 16-byte piece of the padded row: source column 4 * c4
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (4 * c4 < K) {
      v = __ldcs(reinterpret_cast<const float4*>(x + r * ldx + 4 * c4));
      if (rowscale != nullptr) {
        const float s = __ldg(rowscale + r);
        v.x = __fmul_rn(v.x, s); v.y = __fmul_rn(v.y, s); v.z = __fmul_rn(v.z, s); v.w = __fmul_rn(v.w, s);
      }
    }
    *reinterpret_cast<float4*>(dst.p[q] + (row0 + r) * Kp + 4 * cc) = v;
  }
}

// y [n_total, Kp] -> dst[p][(row - p * shard) * ldd + col0 + c] = y[row, c] for the rows of block p.
__global__ void __launch_bounds__(256)
rows_scatter_kernel(const float* __restrict__ y, long long n_total, int Kp, long long shard, long long col0, long long ldd,
                    const __grid_constant__ ColDst dst) {
  const int kp4 = Kp >> 2;
  const long long total = n_total * kp4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / kp4;
    const int cc = (int)(i - row * kp4);
    const long long p = row / shard, rl = row - p * shard;
    const float4 v = __ldcs(reinterpret_cast<const float4*>(y + row * Kp + 4 * cc));
    *reinterpret_cast<float4*>(dst.p[p] + rl * ldd + col0 + 4 * cc) = v;
  }
}

static int col_grid(long long total) {
  long long g = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  return (int)(g > 0 ? g : 1);
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_cols_scatter(const float* x, int64_t n, int64_t K, int64_t ldx, const float* rowscale, int64_t row0,
                       int64_t Kp, void* const* dst, int n_dst, void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K % 4 == 0 && ldx >= K && ldx % 4 == 0, "cols_scatter: K and ldx must be positive multiples of 4");
  EXB_REQUIRE(Kp > 0 && Kp % 4 == 0 && n_dst >= 1 && n_dst <= kColMaxDst && dst != nullptr && Kp * n_dst >= K,
              "cols_scatter: 1 to %d destinations of Kp columns (a multiple of 4) that cover K", kColMaxDst);
  EXB_REQUIRE(row0 >= 0, "cols_scatter: negative row offset");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(x != nullptr && (reinterpret_cast<uintptr_t>(x) & 15) == 0, "cols_scatter: x is null or not 16-byte aligned");
  ColDst d{};
  d.n = n_dst;
  for (int i = 0; i < n_dst; i++) {
    EXB_REQUIRE(dst[i] != nullptr && (reinterpret_cast<uintptr_t>(dst[i]) & 15) == 0,
                "cols_scatter: destination %d is null or not 16-byte aligned", i);
    d.p[i] = static_cast<float*>(dst[i]);
  }
  cols_scatter_kernel<<<col_grid(n * n_dst * (Kp / 4)), 256, 0, (cudaStream_t)stream>>>(x, n, (int)K, ldx, rowscale, row0,
                                                                                       (int)Kp, d);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_rows_scatter(const float* y, int64_t n_total, int64_t Kp, int64_t shard, int64_t col0, int64_t ldd,
                       void* const* dst, int n_dst, void* stream) {
  EXB_REQUIRE(n_total >= 0 && Kp > 0 && Kp % 4 == 0 && shard > 0, "rows_scatter: Kp must be a positive multiple of 4, shard > 0");
  EXB_REQUIRE(col0 >= 0 && col0 % 4 == 0 && ldd % 4 == 0 && ldd >= col0 + Kp, "rows_scatter: col0 and ldd must be multiples of 4, ldd >= col0 + Kp");
  EXB_REQUIRE(n_dst >= 1 && n_dst <= kColMaxDst && dst != nullptr && (int64_t)n_dst * shard >= n_total,
              "rows_scatter: 1 to %d destinations of `shard` rows that cover n_total", kColMaxDst);
  if (n_total == 0) return EXB_OK;
  EXB_REQUIRE(y != nullptr && (reinterpret_cast<uintptr_t>(y) & 15) == 0, "rows_scatter: y is null or not 16-byte aligned");
  ColDst d{};
  d.n = n_dst;
  for (int i = 0; i < n_dst; i++) {
    EXB_REQUIRE(dst[i] != nullptr && (reinterpret_cast<uintptr_t>(dst[i]) & 15) == 0,
                "rows_scatter: destination %d is null or not 16-byte aligned", i);
    d.p[i] = static_cast<float*>(dst[i]);
  }
  rows_scatter_kernel<<<col_grid(n_total * (Kp / 4)), 256, 0, (cudaStream_t)stream>>>(y, n_total, (int)Kp, shard, col0, ldd, d);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
