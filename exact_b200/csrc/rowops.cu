// One pass over the gradient of a layer's output for the two things its backward needs besides the GEMMs:
//   colsum[c] = sum_r g[r, c]               the bias gradient (grad_output.sum(0), backward_func.cc:88-90)
//   out[r, c] = g[r, c] * rowscale[r]       D^-1 g, the operand of the transposed mean aggregation
//                                           (A_mean^T g = A^T (D^-1 g), spmm.cc:128-137), zero-padded to Kout columns
// The framework's own route is a broadcast multiply (a non-vectorised element-wise kernel, split in two above
// 2 GB: 1.64 ms at 2,449,029 x 256) and a two-stage column reduction (0.58 ms); this kernel reads g once with
// 16-byte accesses.  Column sums are added in a fixed order (per-CTA partial rows, then CTA order): results are
// run-to-run identical.  A thread owns VEC adjacent columns and walks down the rows.
#include "exact_b200.h"
#include "common.cuh"

namespace exb {

constexpr int kRowOpsThreads = 256;

struct RowOpsParams {
  const float* g;
  const float* rowscale;   // or null (ones)
  float* out;              // or null
  float* partial;          // [grid, Kout] or null
  long long n, ldg, ldo;
  int K, Kout, cg_total, cg, ry;
};

template <int VEC>
__global__ void __launch_bounds__(kRowOpsThreads) rows_scale_colsum_kernel(const __grid_constant__ RowOpsParams p) {
  __shared__ float s_red[kRowOpsThreads * VEC];
  const int tx = threadIdx.x % p.cg, ty = threadIdx.x / p.cg;
  const bool active = ty < p.ry;
  for (int cg0 = 0; cg0 < p.cg_total; cg0 += p.cg) {
    const int cgi = cg0 + tx;
    const int c = cgi * VEC;
    const bool col_ok = active && cgi < p.cg_total;
    const bool in_g = c < p.K;            // VEC == 4: K is a multiple of 4, so a group is inside or outside as a whole
    float acc[VEC];
#pragma unroll
    for (int x = 0; x < VEC; x++) acc[x] = 0.f;
    if (col_ok) {
      // four rows per step: four loads in flight per thread (one per step left the kernel waiting on memory:
      // 59 % DRAM throughput at 0.18 issue slots per cycle)
      constexpr int kRowsPerStep = 4;
      const long long rstride = (long long)gridDim.x * p.ry;
      for (long long r0 = (long long)blockIdx.x * p.ry + ty; r0 < p.n; r0 += rstride * kRowsPerStep) {
        float v[kRowsPerStep][VEC], s[kRowsPerStep];
#pragma unroll
        for (int u = 0; u < kRowsPerStep; u++) {
          const long long r = r0 + u * rstride;
#pragma unroll
          for (int x = 0; x < VEC; x++) v[u][x] = 0.f;
          s[u] = 1.f;
          if (r < p.n) {
            if (in_g) Ld<float, VEC>::load(p.g + r * p.ldg + c, v[u]);
            if (p.out != nullptr && p.rowscale != nullptr) s[u] = __ldg(p.rowscale + r);
          }
        }
#pragma unroll
        for (int u = 0; u < kRowsPerStep; u++) {
          const long long r = r0 + u * rstride;
          if (r >= p.n) break;
#pragma unroll
          for (int x = 0; x < VEC; x++) acc[x] = __fadd_rn(acc[x], v[u][x]);
          if (p.out != nullptr) {
#pragma unroll
            for (int x = 0; x < VEC; x++) v[u][x] = __fmul_rn(v[u][x], s[u]);
            StF32<VEC>::store(p.out + r * p.ldo + c, v[u]);
          }
        }
      }
    }
    if (p.partial != nullptr) {
      float* mine = s_red + threadIdx.x * VEC;
#pragma unroll
      for (int x = 0; x < VEC; x++) mine[x] = acc[x];
      __syncthreads();
      if (ty == 0 && cgi < p.cg_total) {
        float t[VEC];
#pragma unroll
        for (int x = 0; x < VEC; x++) t[x] = 0.f;
        for (int y = 0; y < p.ry; y++) {
#pragma unroll
          for (int x = 0; x < VEC; x++) t[x] = __fadd_rn(t[x], s_red[(y * p.cg + tx) * VEC + x]);
        }
#pragma unroll
        for (int x = 0; x < VEC; x++) p.partial[(long long)blockIdx.x * p.Kout + c + x] = t[x];
      }
      __syncthreads();
    }
  }
}

__global__ void rows_colsum_finish_kernel(const float* __restrict__ partial, int n_partial, int K, int Kout,
                                          float* __restrict__ colsum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= K) return;
  float a = 0.f;
  for (int i = 0; i < n_partial; i++) a = __fadd_rn(a, partial[(long long)i * Kout + c]);
  colsum[c] = a;
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_rows_scale_colsum_workspace_bytes(int64_t Kout) {
  if (Kout <= 0) return 256;
  return 256 + (int64_t)sm_count() * 8 * Kout * 4;
}

int exact_rows_scale_colsum(const float* g, int64_t n, int64_t K, int64_t ldg, const float* rowscale, float* out,
                            int64_t Kout, int64_t ldo, float* colsum, void* workspace, int64_t workspace_bytes,
                            void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && ldg >= K, "rows_scale_colsum: bad shape");
  EXB_REQUIRE(K <= (1 << 20), "rows_scale_colsum: too many columns");
  if (out == nullptr) Kout = K;
  EXB_REQUIRE(Kout >= K && (out == nullptr || ldo >= Kout), "rows_scale_colsum: out must hold at least K columns per row");
  EXB_REQUIRE(g != nullptr && (out != nullptr || colsum != nullptr), "rows_scale_colsum: null pointer");
  if (colsum != nullptr) {
    EXB_REQUIRE(workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0 &&
                    workspace_bytes >= exact_rows_scale_colsum_workspace_bytes(Kout),
                "rows_scale_colsum: workspace missing, misaligned or too small");
  }
  cudaStream_t st = (cudaStream_t)stream;
  uintptr_t a = reinterpret_cast<uintptr_t>(g) | (uintptr_t)(ldg * 4);
  if (out != nullptr) a |= reinterpret_cast<uintptr_t>(out) | (uintptr_t)(ldo * 4);
  const bool vec = K % 4 == 0 && Kout % 4 == 0 && a % 16 == 0;
  const int V = vec ? 4 : 1;
  RowOpsParams p{};
  p.g = g; p.rowscale = rowscale; p.out = out; p.n = n; p.ldg = ldg; p.ldo = ldo; p.K = (int)K; p.Kout = (int)Kout;
  p.partial = colsum != nullptr ? reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256) : nullptr;
  p.cg_total = (int)((Kout + V - 1) / V);
  p.cg = p.cg_total < (vec ? 64 : 256) ? p.cg_total : (vec ? 64 : 256);
  p.ry = kRowOpsThreads / p.cg;
  long long want = (n + p.ry - 1) / p.ry;
  const long long cap = (long long)sm_count() * 8;
  if (want > cap) want = cap;
  const int grid = (int)(want < 1 ? 1 : want);
  if (vec) rows_scale_colsum_kernel<4><<<grid, kRowOpsThreads, 0, st>>>(p);
  else rows_scale_colsum_kernel<1><<<grid, kRowOpsThreads, 0, st>>>(p);
  EXB_CUDA_OK(cudaGetLastError());
  if (colsum != nullptr) {
    rows_colsum_finish_kernel<<<(unsigned)((K + 127) / 128), 128, 0, st>>>(p.partial, grid, (int)K, (int)Kout, colsum);
    EXB_CUDA_OK(cudaGetLastError());
  }
  return EXB_OK;
}

}  // extern "C"
