// CSR SpMM on fp16 operands with the arithmetic of the reference's half instantiation.
//
// The reference dispatches spmm_kernel on half as well (exact/exact/cpp_extension/spmm_cuda.cu:142, AMP runs:
// exact/exact/ops.py:260, 313 cast the operands to fp16).  With scalar_t = c10::Half every step of the row sum is
// rounded to half (spmm_cuda.cu:83-92, reducer.cuh:53-60, 72-77):
//     term   = half(value[e] * mat[col[e], c])            (with edge values; the bare operand otherwise)
//     result = half(result + term)                        in edge order, starting from 0
//     mean:    out = half(result / half(max(count, 1)))   (the count itself is rounded to half first)
// each Half (op) Half being an fp32 operation on the widened values.  Rounding after every edge makes the order of
// the edges part of the result, so a row is always summed by one warp in CSR order (no long-row pieces here).
// One warp per row and tile of 128 (or 32) columns; a lane owns four adjacent columns (one 8-byte load per edge)
// when K % 4 == 0 and the rows are 8-byte aligned, one column otherwise; eight gathers in flight per lane.
#include <cuda_fp16.h>

#include "exact_b200.h"
#include "common.cuh"

namespace exb {

__device__ __forceinline__ float rh(float f) { return __half2float(__float2half_rn(f)); }

template <int VEC>
__device__ __forceinline__ void ld_h(const __half* p, float (&o)[VEC]);
template <>
__device__ __forceinline__ void ld_h<4>(const __half* p, float (&o)[4]) {
  const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y;
}
template <>
__device__ __forceinline__ void ld_h<1>(const __half* p, float (&o)[1]) { o[0] = __half2float(__ldg(p)); }

template <typename IdxT, bool HAS_VAL, int VEC>
__global__ void __launch_bounds__(128) spmm_f16_kernel(const IdxT* __restrict__ rowptr, const IdxT* __restrict__ col,
                                                       const __half* __restrict__ val, const __half* __restrict__ mat,
                                                       __half* __restrict__ out, long long M, long long K, int mean) {
  constexpr int kDepth = 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 4 + warp;
  if (row >= M) return;
  const long long c = ((long long)blockIdx.y * 32 + lane) * VEC;
  const bool cvalid = c < K;
  const long long begin = (long long)rowptr[row], end = (long long)rowptr[row + 1];
  float acc[VEC];
#pragma unroll
  for (int x = 0; x < VEC; x++) acc[x] = 0.f;
  const __half* __restrict__ mat0 = mat + (cvalid ? c : 0);
  for (long long base = begin; base < end; base += 32) {
    const long long e = base + lane;
    uint32_t idx = 0;
    float v = 0.f;
    if (e < end) {
      idx = (uint32_t)col[e];
      if (HAS_VAL) v = __half2float(__ldg(val + e));
    }
    const int cnt = (end - base) < 32 ? (int)(end - base) : 32;
    for (int t0 = 0; t0 < cnt; t0 += kDepth) {
      float m[kDepth][VEC], w[kDepth];
#pragma unroll
      for (int u = 0; u < kDepth; u++) {
        const uint32_t j = __shfl_sync(0xffffffffu, idx, (t0 + u) & 31);
        w[u] = HAS_VAL ? __shfl_sync(0xffffffffu, v, (t0 + u) & 31) : 0.f;
#pragma unroll
        for (int x = 0; x < VEC; x++) m[u][x] = 0.f;
        if (t0 + u < cnt && cvalid) ld_h<VEC>(mat0 + (unsigned long long)j * (unsigned long long)K, m[u]);
      }
#pragma unroll
      for (int u = 0; u < kDepth; u++) {
        if (t0 + u < cnt) {
#pragma unroll
          for (int x = 0; x < VEC; x++) {
            const float term = HAS_VAL ? rh(__fmul_rn(w[u], m[u][x])) : m[u][x];
            acc[x] = rh(__fadd_rn(acc[x], term));
          }
        }
      }
    }
  }
  if (mean) {
    const long long count = end - begin;
    const float dv = rh((float)(count > 0 ? count : 1));   // (scalar_t)count, reducer.cuh:75-76
#pragma unroll
    for (int x = 0; x < VEC; x++) acc[x] = rh(__fdiv_rn(acc[x], dv));
  }
  if (cvalid) {
    __half* dst = out + row * K + c;
    if (VEC == 4) {
      const __half2 a = __floats2half2_rn(acc[0], acc[VEC > 1 ? 1 : 0]), b = __floats2half2_rn(acc[VEC > 2 ? 2 : 0], acc[VEC > 3 ? 3 : 0]);
      uint2 t;
      t.x = *reinterpret_cast<const uint32_t*>(&a);
      t.y = *reinterpret_cast<const uint32_t*>(&b);
      *reinterpret_cast<uint2*>(dst) = t;
    } else {
      dst[0] = __float2half_rn(acc[0]);
    }
  }
}

template <typename IdxT, bool HAS_VAL>
static int launch_spmm_f16(const void* rowptr, const void* col, const void* val, const void* mat, void* out, long long M,
                           long long K, int mean, cudaStream_t st) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(mat) | reinterpret_cast<uintptr_t>(out);
  const bool vec = K % 4 == 0 && a % 8 == 0;
  const long long per_tile = vec ? 128 : 32;
  dim3 grid((unsigned)((M + 3) / 4), (unsigned)((K + per_tile - 1) / per_tile));
  if (vec)
    spmm_f16_kernel<IdxT, HAS_VAL, 4><<<grid, 128, 0, st>>>(static_cast<const IdxT*>(rowptr), static_cast<const IdxT*>(col),
                                                            static_cast<const __half*>(val), static_cast<const __half*>(mat),
                                                            static_cast<__half*>(out), M, K, mean);
  else
    spmm_f16_kernel<IdxT, HAS_VAL, 1><<<grid, 128, 0, st>>>(static_cast<const IdxT*>(rowptr), static_cast<const IdxT*>(col),
                                                            static_cast<const __half*>(val), static_cast<const __half*>(mat),
                                                            static_cast<__half*>(out), M, K, mean);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_spmm_f16(const void* rowptr, const void* col, int idx_bytes, const void* value, const void* mat, int64_t M,
                   int64_t K, int reduce, void* out, void* stream) {
  EXB_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "spmm_f16: idx_bytes must be 4 or 8 (got %d)", idx_bytes);
  reduce &= ~EXACT_SPMM_REGROUP;
  EXB_REQUIRE(reduce == EXACT_REDUCE_SUM || reduce == EXACT_REDUCE_MEAN, "spmm_f16: reduce must be sum or mean");
  EXB_REQUIRE(M >= 0 && K >= 0, "spmm_f16: negative shape");
  if (M == 0 || K == 0) return EXB_OK;
  EXB_REQUIRE(rowptr && mat && out, "spmm_f16: null pointer");
  EXB_REQUIRE((M + 3) / 4 <= 2147483647LL && M < (1LL << 32), "spmm_f16: too many rows");
  EXB_REQUIRE((K + 31) / 32 <= 65535, "spmm_f16: K too large");
  cudaStream_t st = (cudaStream_t)stream;
  const int mean = reduce == EXACT_REDUCE_MEAN;
  if (idx_bytes == 4)
    return value ? launch_spmm_f16<int32_t, true>(rowptr, col, value, mat, out, M, K, mean, st)
                 : launch_spmm_f16<int32_t, false>(rowptr, col, value, mat, out, M, K, mean, st);
  return value ? launch_spmm_f16<int64_t, true>(rowptr, col, value, mat, out, M, K, mean, st)
               : launch_spmm_f16<int64_t, false>(rowptr, col, value, mat, out, M, K, mean, st);
}

}  // extern "C"
