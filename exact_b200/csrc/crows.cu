// Compact rows: the sparse form of a dense operand whose entries are mostly exact zeros, as the SpMM of
// the quantised GCN / GraphSAGE layers gathers it and as row shards exchange it between GPUs.
//
// Past the first layer the dense operand of an aggregation is an output of ReLU + dropout (forward) or
// a gradient that passed their masks (backward): about three quarters of its entries are +0.0.  Adding
// +0.0 to an fp32 sum that started at +0.0 never changes it, so a gather that skips those entries
// produces bit-identical sums while moving a third of the bytes.
//
// Row r of an [n, K] fp32 matrix (K <= 256) lives in a slot of fixed size at slot index row0 + r:
//     +0                 uint32  cnt            number of kept entries
//     +16                uint8   col[cnt]       their columns, ascending
//     +16 + pad16(K)     fp32    val[cnt]       their values (any entry whose 32 bits are not all zero,
//                                               so -0.0, NaN, inf and denormals are kept)
// The slot size does not depend on the data, so a producer needs no prefix sum, a consumer finds row r
// without an offset table, and a rank can write its rows straight into the same slots of every peer's
// buffer (plain stores through NVLink): only the used prefix of a slot is ever written or read.
//
// The reference is single-GPU and gathers dense rows (spmm_cuda.cu:86-93); it has no counterpart.
#include "common.cuh"
#include "crows.cuh"
#include "exact_b200.h"

namespace exb {

constexpr int kCrowsWarps = 8;
constexpr int kCrowsMaxDst = 8;

struct CrowsDst {
  unsigned char* p[kCrowsMaxDst];
  int n;
};

// One warp per row.  The row is compacted into a staging slot in shared memory (ballot + popcount give
// every kept entry its place) and the used prefix of the slot is then copied to each destination with
// 16-byte stores: whole sectors, which is what crosses NVLink well.
__global__ void __launch_bounds__(kCrowsWarps * 32)
crows_pack_kernel(const float* __restrict__ x, long long n, int K, long long ldx, const float* __restrict__ rowscale,
                  long long row0, const __grid_constant__ CrowsDst dst, unsigned long long* __restrict__ kept_total) {
  extern __shared__ __align__(16) unsigned char s_stage[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = (K + 31) >> 5;
  const int cols_bytes = crows_cols_bytes(K);
  const long long stride = crows_stride_bytes(K);
  unsigned char* stage = s_stage + (size_t)warp * stride;
  unsigned char* s_col = stage + 16;
  uint32_t* s_val = reinterpret_cast<uint32_t*>(stage + 16 + cols_bytes);
  const uint32_t lt = (1u << lane) - 1u;
  unsigned long long kept = 0;
  for (long long row = (long long)blockIdx.x * kCrowsWarps + warp; row < n; row += (long long)gridDim.x * kCrowsWarps) {
    const float* src = x + row * ldx;
    const float sc = rowscale ? __ldg(rowscale + row) : 1.f;
    // all loads of the row first (K <= 256: at most 8 per lane), then the compaction
    uint32_t bits[8];
#pragma unroll
    for (int w = 0; w < 8; w++) {
      const int c = w * 32 + lane;
      bits[w] = 0u;
      if (c < K) {
        float v = __ldcs(src + c);
        if (rowscale) v = __fmul_rn(v, sc);
        bits[w] = __float_as_uint(v);
      }
    }
    int pos = 0;
#pragma unroll
    for (int w = 0; w < 8; w++) {
      if (w < W) {
        const uint32_t m = __ballot_sync(0xffffffffu, bits[w] != 0u);
        if (bits[w] != 0u) {
          const int q = pos + __popc(m & lt);
          s_col[q] = (unsigned char)(w * 32 + lane);
          s_val[q] = bits[w];
        }
        pos += __popc(m);
      }
    }
    if (lane == 0) *reinterpret_cast<uint32_t*>(stage) = (uint32_t)pos;
    __syncwarp();
    kept += (unsigned long long)pos;
    const int head16 = (16 + pos + 15) >> 4;     // header + columns, in 16-byte units
    const int val16 = (pos + 3) >> 2;            // values, in 16-byte units
    const uint4* sh = reinterpret_cast<const uint4*>(stage);
    const uint4* sv = reinterpret_cast<const uint4*>(stage + 16 + cols_bytes);
    for (int d = 0; d < dst.n; d++) {
      unsigned char* slot = dst.p[d] + (row0 + row) * stride;
      uint4* gh = reinterpret_cast<uint4*>(slot);
      uint4* gv = reinterpret_cast<uint4*>(slot + 16 + cols_bytes);
      for (int i = lane; i < head16; i += 32) gh[i] = sh[i];
      for (int i = lane; i < val16; i += 32) gv[i] = sv[i];
    }
    __syncwarp();
  }
  if (kept_total != nullptr) {
    // one atomic per CTA
    __shared__ unsigned long long s_kept[kCrowsWarps];
    if (lane == 0) s_kept[warp] = kept;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long t = 0;
      for (int i = 0; i < kCrowsWarps; i++) t += s_kept[i];
      if (t) atomicAdd(kept_total, t);
    }
  }
}

// Dense rows back from compact slots.  One warp per row: the row is assembled in shared memory (zeros, then
// the kept entries at their columns) and written out in full 128-bit pieces.
__global__ void __launch_bounds__(kCrowsWarps * 32)
crows_unpack_kernel(const unsigned char* __restrict__ buf, long long n, int K, long long row0, float* __restrict__ out,
                    long long ldo) {
  __shared__ __align__(16) uint32_t s_row[kCrowsWarps][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cols_bytes = crows_cols_bytes(K);
  const long long stride = crows_stride_bytes(K);
  uint32_t* row_s = s_row[warp];
  const bool vec4 = (K & 3) == 0 && (ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  for (long long row = (long long)blockIdx.x * kCrowsWarps + warp; row < n; row += (long long)gridDim.x * kCrowsWarps) {
    const unsigned char* slot = buf + (row0 + row) * stride;
    int cnt = (int)__ldcs(reinterpret_cast<const uint32_t*>(slot));
    if (cnt > K) cnt = K;
    const uint32_t* v = reinterpret_cast<const uint32_t*>(slot + 16 + cols_bytes);
    // issue the loads of the first 64 entries before touching shared memory
    uint32_t c0 = 0, c1 = 0, v0 = 0, v1 = 0;
    if (lane < cnt) { c0 = slot[16 + lane]; v0 = __ldcs(v + lane); }
    if (lane + 32 < cnt) { c1 = slot[48 + lane]; v1 = __ldcs(v + 32 + lane); }
    for (int c = lane; c < K; c += 32) row_s[c] = 0u;
    __syncwarp();
    if (lane < cnt) row_s[c0] = v0;
    if (lane + 32 < cnt) row_s[c1] = v1;
    for (int i = lane + 64; i < cnt; i += 32) row_s[slot[16 + i]] = __ldcs(v + i);
    __syncwarp();
    float* dst = out + row * ldo;
    if (vec4) {
      for (int c = lane * 4; c < K; c += 128)
        __stcs(reinterpret_cast<uint4*>(dst + c), *reinterpret_cast<const uint4*>(row_s + c));
    } else {
      for (int c = lane; c < K; c += 32) reinterpret_cast<uint32_t*>(dst)[c] = row_s[c];
    }
    __syncwarp();
  }
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_crows_slot_bytes(int64_t K) {
  if (K <= 0 || K > 256) return -1;
  return crows_stride_bytes((int)K);
}

int exact_crows_pack(const float* x, int64_t n, int64_t K, int64_t ldx, const float* rowscale, int64_t row0,
                     void* const* dst, int n_dst, uint64_t* kept_total, void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K <= 256 && ldx >= K, "crows_pack: need 0 < K <= 256 and ldx >= K (K = %lld)", (long long)K);
  EXB_REQUIRE(n_dst >= 1 && n_dst <= kCrowsMaxDst && dst != nullptr, "crows_pack: 1 to %d destination buffers", kCrowsMaxDst);
  EXB_REQUIRE(row0 >= 0, "crows_pack: negative slot index");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(x != nullptr, "crows_pack: null input");
  CrowsDst d{};
  d.n = n_dst;
  for (int i = 0; i < n_dst; i++) {
    EXB_REQUIRE(dst[i] != nullptr && reinterpret_cast<uintptr_t>(dst[i]) % 16 == 0,
                "crows_pack: destination %d is null or not 16-byte aligned", i);
    d.p[i] = static_cast<unsigned char*>(dst[i]);
  }
  const size_t smem = (size_t)kCrowsWarps * (size_t)crows_stride_bytes((int)K);
  long long g = (n + kCrowsWarps - 1) / kCrowsWarps;
  const long long cap = (long long)sm_count() * 8;
  if (g > cap) g = cap;
  crows_pack_kernel<<<(unsigned)g, kCrowsWarps * 32, smem, (cudaStream_t)stream>>>(
      x, n, (int)K, ldx, rowscale, row0, d, reinterpret_cast<unsigned long long*>(kept_total));
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_crows_unpack(const void* buf, int64_t n, int64_t K, int64_t row0, float* out, int64_t ldo, void* stream) {
  EXB_REQUIRE(n >= 0 && K > 0 && K <= 256 && ldo >= K && row0 >= 0, "crows_unpack: need 0 < K <= 256, ldo >= K");
  if (n == 0) return EXB_OK;
  EXB_REQUIRE(buf != nullptr && out != nullptr, "crows_unpack: null pointer");
  long long g = (n + kCrowsWarps - 1) / kCrowsWarps;
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  crows_unpack_kernel<<<(unsigned)g, kCrowsWarps * 32, 0, (cudaStream_t)stream>>>(
      static_cast<const unsigned char*>(buf), n, (int)K, row0, out, ldo);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
