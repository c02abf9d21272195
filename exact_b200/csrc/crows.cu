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

// One warp per row, two rows per step so that twice the loads are in flight.  A row is compacted into a
// staging slot in shared memory (ballot + popcount give every kept entry its place) and the used prefix of
// the slot is then copied to each destination with 16-byte stores: whole sectors, which is what crosses
// NVLink well.
constexpr int kCrowsRows = 2;   // rows per warp and step

__global__ void __launch_bounds__(kCrowsWarps * 32)
crows_pack_kernel(const float* __restrict__ x, long long n, int K, long long ldx, const float* __restrict__ rowscale,
                  long long row0, const __grid_constant__ CrowsDst dst, unsigned long long* __restrict__ kept_total) {
  extern __shared__ __align__(16) unsigned char s_stage[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int W = (K + 31) >> 5;
  const int cols_bytes = crows_cols_bytes(K);
  const long long stride = crows_stride_bytes(K);
  const uint32_t lt = (1u << lane) - 1u;
  unsigned long long kept = 0;
  const long long step = (long long)gridDim.x * kCrowsWarps * kCrowsRows;
  for (long long base = ((long long)blockIdx.x * kCrowsWarps + warp) * kCrowsRows; base < n; base += step) {
    // all loads of the rows first (K <= 256: at most 8 per lane and row), then the compaction
    uint32_t bits[kCrowsRows][8];
#pragma unroll
    for (int r = 0; r < kCrowsRows; r++) {
      const long long row = base + r;
      const float* src = x + row * ldx;
#pragma unroll
      for (int w = 0; w < 8; w++) {
        const int c = w * 32 + lane;
        bits[r][w] = 0u;
        if (row < n && c < K) bits[r][w] = __float_as_uint(__ldcs(src + c));
      }
    }
#pragma unroll
    for (int r = 0; r < kCrowsRows; r++) {
      const long long row = base + r;
      if (row >= n) break;
      unsigned char* stage = s_stage + (size_t)(warp * kCrowsRows + r) * stride;
      unsigned char* s_col = stage + 16;
      uint32_t* s_val = reinterpret_cast<uint32_t*>(stage + 16 + cols_bytes);
      if (rowscale) {
        const float sc = __ldg(rowscale + row);
#pragma unroll
        for (int w = 0; w < 8; w++) bits[r][w] = __float_as_uint(__fmul_rn(__uint_as_float(bits[r][w]), sc));
      }
      int pos = 0;
#pragma unroll
      for (int w = 0; w < 8; w++) {
        if (w < W) {
          const uint32_t m = __ballot_sync(0xffffffffu, bits[r][w] != 0u);
          if (bits[r][w] != 0u) {
            const int q = pos + __popc(m & lt);
            s_col[q] = (unsigned char)(w * 32 + lane);
            s_val[q] = bits[r][w];
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

// Dense rows back from compact slots.  One warp per row, two rows per step: the count and the first 64
// entries of each row are requested together (a row of 256 columns at 25 % density has about 64), the row is
// assembled in shared memory (zeros, then the kept entries at their columns) and written out in full 128-bit
// pieces.
__global__ void __launch_bounds__(kCrowsWarps * 32)
crows_unpack_kernel(const unsigned char* __restrict__ buf, long long n, int K, long long row0, float* __restrict__ out,
                    long long ldo) {
  __shared__ __align__(16) uint32_t s_row[kCrowsWarps][kCrowsRows][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cols_bytes = crows_cols_bytes(K);
  const long long stride = crows_stride_bytes(K);
  const bool vec4 = (K & 3) == 0 && (ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  const bool in0 = lane < K, in1 = lane + 32 < K;
  const long long step = (long long)gridDim.x * kCrowsWarps * kCrowsRows;
  for (long long base = ((long long)blockIdx.x * kCrowsWarps + warp) * kCrowsRows; base < n; base += step) {
    int cnt[kCrowsRows];
    uint32_t c0[kCrowsRows], c1[kCrowsRows], v0[kCrowsRows], v1[kCrowsRows];
#pragma unroll
    for (int r = 0; r < kCrowsRows; r++) {
      cnt[r] = 0; c0[r] = c1[r] = v0[r] = v1[r] = 0u;
      if (base + r < n) {
        // the entries are requested before the count is known: they lie inside the slot whatever the count is
        const unsigned char* slot = buf + (row0 + base + r) * stride;
        const uint32_t* v = reinterpret_cast<const uint32_t*>(slot + 16 + cols_bytes);
        cnt[r] = (int)__ldcs(reinterpret_cast<const uint32_t*>(slot));
        if (in0) { c0[r] = slot[16 + lane]; v0[r] = __ldcs(v + lane); }
        if (in1) { c1[r] = slot[48 + lane]; v1[r] = __ldcs(v + 32 + lane); }
      }
    }
#pragma unroll
    for (int r = 0; r < kCrowsRows; r++) {
      if (base + r >= n) break;
      uint32_t* row_s = s_row[warp][r];
      const int m = cnt[r] < K ? cnt[r] : K;
      for (int c = lane; c < K; c += 32) row_s[c] = 0u;
      __syncwarp();
      if (lane < m) row_s[c0[r]] = v0[r];
      if (lane + 32 < m) row_s[c1[r]] = v1[r];
      if (m > 64) {
        const unsigned char* slot = buf + (row0 + base + r) * stride;
        const uint32_t* v = reinterpret_cast<const uint32_t*>(slot + 16 + cols_bytes);
        for (int i = lane + 64; i < m; i += 32) row_s[slot[16 + i]] = __ldcs(v + i);
      }
      __syncwarp();
      float* dst = out + (base + r) * ldo;
      if (vec4) {
        for (int c = lane * 4; c < K; c += 128)
          __stcs(reinterpret_cast<uint4*>(dst + c), *reinterpret_cast<const uint4*>(row_s + c));
      } else {
        for (int c = lane; c < K; c += 32) reinterpret_cast<uint32_t*>(dst)[c] = row_s[c];
      }
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
  const size_t smem = (size_t)kCrowsWarps * kCrowsRows * (size_t)crows_stride_bytes((int)K);
  long long g = (n + kCrowsWarps * kCrowsRows - 1) / (kCrowsWarps * kCrowsRows);
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
  long long g = (n + kCrowsWarps * kCrowsRows - 1) / (kCrowsWarps * kCrowsRows);
  const long long cap = (long long)sm_count() * 16;
  if (g > cap) g = cap;
  crows_unpack_kernel<<<(unsigned)g, kCrowsWarps * 32, 0, (cudaStream_t)stream>>>(
      static_cast<const unsigned char*>(buf), n, (int)K, row0, out, ldo);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
