// CSR x dense SpMM (sum / mean), the aggregation of the quantised GCN / GraphSAGE layers.
//
// Replaces spmm.spmm_sum_fw / spmm_mean_fw and, on the transposed structure, the dense-operand
// gradient of spmm_sum_bw / spmm_mean_bw (exact/exact/cpp_extension/spmm.cc:31-139; kernel
// spmm_cuda.cu:27-104; reducer.cuh:43-85).
//
// One warp owns one output row and a tile of 32*KVT*VEC columns.  Column indices (pre-multiplied to
// element offsets) and edge values are fetched 32 at a time with one coalesced load and staged in
// shared memory; every lane then walks the staged list and gathers VEC-wide (128-bit when K % 4 == 0)
// slices of the neighbour rows, four edges in flight at a time.  Edges are accumulated in CSR order
// with one FMA per edge, which is the reference's summation order (spmm_cuda.cu:86-93).
#include "common.cuh"
#include "exact_b200.h"

namespace exb {

struct SpmmParams {
  const void* rowptr;
  const void* col;
  const float* val;
  const float* mat;
  float* out;
  long long M, K;
  int mean;
};

constexpr int kSpmmWarps = 4;

template <int VEC>
__device__ __forceinline__ void ldg_vec(const float* p, float (&o)[VEC]);
template <>
__device__ __forceinline__ void ldg_vec<4>(const float* p, float (&o)[4]) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(p));
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <>
__device__ __forceinline__ void ldg_vec<2>(const float* p, float (&o)[2]) {
  const float2 v = __ldg(reinterpret_cast<const float2*>(p));
  o[0] = v.x; o[1] = v.y;
}
template <>
__device__ __forceinline__ void ldg_vec<1>(const float* p, float (&o)[1]) { o[0] = __ldg(p); }

template <typename IdxT, int VEC, int KVT, bool HAS_VAL>
__global__ void __launch_bounds__(kSpmmWarps * 32) spmm_csr_kernel(const __grid_constant__ SpmmParams p) {
  __shared__ long long s_off[kSpmmWarps][32];
  __shared__ float s_val[kSpmmWarps][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kSpmmWarps + warp;
  if (row >= p.M) return;
  const IdxT* __restrict__ rowptr = reinterpret_cast<const IdxT*>(p.rowptr);
  const IdxT* __restrict__ col = reinterpret_cast<const IdxT*>(p.col);
  const long long K = p.K;

  long long coff[KVT];
  bool cvalid[KVT];
#pragma unroll
  for (int j = 0; j < KVT; j++) {
    coff[j] = ((long long)blockIdx.y * (32 * KVT) + lane + 32 * j) * VEC;
    cvalid[j] = coff[j] < K;
  }

  const long long start = (long long)rowptr[row], end = (long long)rowptr[row + 1];
  float acc[KVT][VEC];
#pragma unroll
  for (int j = 0; j < KVT; j++)
#pragma unroll
    for (int e = 0; e < VEC; e++) acc[j][e] = 0.f;

  for (long long base = start; base < end; base += 32) {
    const long long e = base + lane;
    long long off = 0;
    float v = 0.f;
    if (e < end) {
      off = (long long)col[e] * K;
      if (HAS_VAL) v = __ldg(p.val + e);
    }
    __syncwarp();
    s_off[warp][lane] = off;
    if (HAS_VAL) s_val[warp][lane] = v;
    __syncwarp();
    const int cnt = (end - base) < 32 ? (int)(end - base) : 32;
    for (int i = 0; i < cnt; i += 4) {
      float m[4][KVT][VEC];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (i + u < cnt) {
          const float* src = p.mat + s_off[warp][i + u];
          if (HAS_VAL) w[u] = s_val[warp][i + u];
#pragma unroll
          for (int j = 0; j < KVT; j++)
            if (cvalid[j]) ldg_vec<VEC>(src + coff[j], m[u][j]);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        if (i + u < cnt) {
#pragma unroll
          for (int j = 0; j < KVT; j++) {
            if (cvalid[j]) {
#pragma unroll
              for (int x = 0; x < VEC; x++) {
                if (HAS_VAL) acc[j][x] = __fmaf_rn(w[u], m[u][j][x], acc[j][x]);
                else acc[j][x] = __fadd_rn(acc[j][x], m[u][j][x]);
              }
            }
          }
        }
      }
    }
  }

  if (p.mean) {
    const long long cnt = end - start;
    const float dv = (float)(cnt > 0 ? cnt : 1);  // reducer.cuh:75-76
#pragma unroll
    for (int j = 0; j < KVT; j++)
#pragma unroll
      for (int x = 0; x < VEC; x++) acc[j][x] = __fdiv_rn(acc[j][x], dv);
  }
  float* orow = p.out + row * K;
#pragma unroll
  for (int j = 0; j < KVT; j++) {
    if (cvalid[j]) {
      if (VEC == 4) *reinterpret_cast<float4*>(orow + coff[j]) = make_float4(acc[j][0], acc[j][1 % VEC], acc[j][2 % VEC], acc[j][3 % VEC]);
      else if (VEC == 2) *reinterpret_cast<float2*>(orow + coff[j]) = make_float2(acc[j][0], acc[j][1 % VEC]);
      else orow[coff[j]] = acc[j][0];
    }
  }
}

template <typename IdxT, int VEC, bool HAS_VAL>
static int launch_spmm_kvt(const SpmmParams& p, cudaStream_t st) {
  const long long C = p.K / VEC;
  const long long per32 = (C + 31) / 32;
  const int kvt = per32 >= 4 ? 4 : (per32 >= 2 ? 2 : 1);
  dim3 grid((unsigned)((p.M + kSpmmWarps - 1) / kSpmmWarps), (unsigned)((C + 32 * kvt - 1) / (32 * kvt)));
  if (kvt == 4) spmm_csr_kernel<IdxT, VEC, 4, HAS_VAL><<<grid, kSpmmWarps * 32, 0, st>>>(p);
  else if (kvt == 2) spmm_csr_kernel<IdxT, VEC, 2, HAS_VAL><<<grid, kSpmmWarps * 32, 0, st>>>(p);
  else spmm_csr_kernel<IdxT, VEC, 1, HAS_VAL><<<grid, kSpmmWarps * 32, 0, st>>>(p);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

template <typename IdxT, bool HAS_VAL>
static int launch_spmm_vec(const SpmmParams& p, cudaStream_t st) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p.mat) | reinterpret_cast<uintptr_t>(p.out);
  if (p.K % 4 == 0 && a % 16 == 0) return launch_spmm_kvt<IdxT, 4, HAS_VAL>(p, st);
  if (p.K % 2 == 0 && a % 8 == 0) return launch_spmm_kvt<IdxT, 2, HAS_VAL>(p, st);
  return launch_spmm_kvt<IdxT, 1, HAS_VAL>(p, st);
}

}  // namespace exb

using namespace exb;

extern "C" int exact_spmm(const void* rowptr, const void* col, int idx_bytes, const float* value,
                          const float* mat, int64_t M, int64_t K, int reduce, float* out, void* stream) {
  EXB_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "spmm: idx_bytes must be 4 or 8 (got %d)", idx_bytes);
  EXB_REQUIRE(reduce == EXACT_REDUCE_SUM || reduce == EXACT_REDUCE_MEAN, "spmm: reduce must be sum or mean");
  EXB_REQUIRE(M >= 0 && K >= 0, "spmm: negative shape");
  if (M == 0 || K == 0) return EXB_OK;
  EXB_REQUIRE(rowptr && mat && out, "spmm: null pointer");
  EXB_REQUIRE((M + kSpmmWarps - 1) / kSpmmWarps <= 2147483647LL, "spmm: too many rows");
  SpmmParams p;
  p.rowptr = rowptr; p.col = col; p.val = value; p.mat = mat; p.out = out; p.M = M; p.K = K;
  p.mean = reduce == EXACT_REDUCE_MEAN;
  cudaStream_t st = (cudaStream_t)stream;
  if (idx_bytes == 4) {
    return value ? launch_spmm_vec<int32_t, true>(p, st) : launch_spmm_vec<int32_t, false>(p, st);
  }
  return value ? launch_spmm_vec<int64_t, true>(p, st) : launch_spmm_vec<int64_t, false>(p, st);
}
