// CSR x dense SpMM (sum / mean), the aggregation of the quantised GCN / GraphSAGE layers.
//
// Replaces spmm.spmm_sum_fw / spmm_mean_fw and, on the transposed structure, the dense-operand
// gradient of spmm_sum_bw / spmm_mean_bw (exact/exact/cpp_extension/spmm.cc:31-139; kernel
// spmm_cuda.cu:27-104; reducer.cuh:43-85).
//
// One warp owns one output row and a tile of 32*KVT*VEC columns.  Column indices and edge values are
// fetched 32 at a time with one coalesced load and staged in shared memory; every lane then walks
// the staged list and gathers VEC-wide (128-bit when K % 4 == 0) slices of the neighbour rows, sixteen
// edges in flight at a time.  Edges are accumulated in CSR order with one FMA (or add) per edge and
// element, which is the reference's summation order (spmm_cuda.cu:86-93), so rows handled this way
// are bit-identical to it.
//
// Power-law graphs have rows with 10^4..10^5 edges; a single warp walking such a row is the whole
// kernel's critical path.  Rows longer than a threshold are therefore left out of the row kernel and
// cut into items of at most `threshold` edges; one warp per item writes a partial sum to caller-owned
// scratch, and a last small kernel adds each long row's partials in order.  Only those rows differ
// from the reference's summation order (by regrouping, within fp32 rounding).
#include <mutex>

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
  int regroup;   // the caller accepts a regrouped per-row sum (EXACT_SPMM_REGROUP)
  long long long_threshold;  // rows with more edges are skipped by the row kernel (0: none)
  // long-row items
  const int* item_row;
  const long long* item_begin;
  const long long* item_end;
  const int* item_slot;      // scratch slot of each listed piece, or null (slot = position)
  long long n_items;
  const int* long_row;
  const int* long_item_ptr;
  long long n_long;
  float* scratch;  // [n_items, K]
  // Routed output (feature-parallel aggregation): row r is written to columns route_col0 .. + K - 1 of row
  // r % route_shard of the [route_shard, route_ld] matrix at route_dst[r / route_shard], which may be another
  // GPU's memory (plain stores).  route_n == 0: the rows go to `out`.
  float* route_dst[8];
  int route_n;
  const int* row_order;  // narrow operands: the order in which the rows are taken (a permutation), or null
  long long route_shard, route_ld, route_col0;
};

__device__ __forceinline__ float* output_row(const SpmmParams& p, long long row) {
  if (p.route_n == 0) return p.out + row * p.K;
  const long long owner = row / p.route_shard;
  return p.route_dst[owner] + (row - owner * p.route_shard) * p.route_ld + p.route_col0;
}

constexpr int kSpmmWarps = 4;
constexpr int kEdgeUnroll = 16;   // gathers in flight per lane (16 against 8: 3 % faster at 128 M edges x 256 columns)

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

template <int VEC>
__device__ __forceinline__ void st_vec(float* p, const float (&a)[VEC]) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1 % VEC], a[2 % VEC], a[3 % VEC]);
  else if (VEC == 2) *reinterpret_cast<float2*>(p) = make_float2(a[0], a[1 % VEC]);
  else p[0] = a[0];
}

// acc += sum over edges [begin, end) of val[e] * mat[col[e], column tile], in edge order.
// FULL: every lane's KVT chunks lie inside K (no column predicate in the inner loop).
template <typename IdxT, int VEC, int KVT, bool HAS_VAL, bool FULL>
__device__ __forceinline__ void accumulate_edges(const SpmmParams& p, long long begin, long long end,
                                                 const long long (&coff)[KVT], const bool (&cvalid)[KVT],
                                                 uint32_t* s_idx, float* s_val, int lane,
                                                 float (&acc)[KVT][VEC]) {
  const IdxT* __restrict__ col = reinterpret_cast<const IdxT*>(p.col);
  const unsigned long long row_bytes = (unsigned long long)p.K * 4ull;
  const char* __restrict__ mat0 = reinterpret_cast<const char*>(p.mat + coff[0]);
  for (long long base = begin; base < end; base += 32) {
    const long long e = base + lane;
    uint32_t idx = 0;
    float v = 0.f;
    if (e < end) {
      idx = (uint32_t)col[e];
      if (HAS_VAL) v = __ldg(p.val + e);
    }
    __syncwarp();
    s_idx[lane] = idx;
    if (HAS_VAL) s_val[lane] = v;
    __syncwarp();
    const int cnt = (end - base) < 32 ? (int)(end - base) : 32;
    int i = 0;
    // full groups of kEdgeUnroll edges: all gathers issued before the first add
    for (; i + kEdgeUnroll <= cnt; i += kEdgeUnroll) {
      float m[kEdgeUnroll][KVT][VEC];
      float w[kEdgeUnroll];
#pragma unroll
      for (int u = 0; u < kEdgeUnroll; u++) {
        const float* src = reinterpret_cast<const float*>(mat0 + (unsigned long long)s_idx[i + u] * row_bytes);
        if (HAS_VAL) w[u] = s_val[i + u];
#pragma unroll
        for (int j = 0; j < KVT; j++)
          if (FULL || cvalid[j]) ldg_vec<VEC>(src + j * (32 * VEC), m[u][j]);
      }
#pragma unroll
      for (int u = 0; u < kEdgeUnroll; u++) {
#pragma unroll
        for (int j = 0; j < KVT; j++) {
          if (FULL || cvalid[j]) {
#pragma unroll
            for (int x = 0; x < VEC; x++) {
              if (HAS_VAL) acc[j][x] = __fmaf_rn(w[u], m[u][j][x], acc[j][x]);
              else acc[j][x] = __fadd_rn(acc[j][x], m[u][j][x]);
            }
          }
        }
      }
    }
    // remainder, one edge at a time
    for (; i < cnt; i++) {
      const float* src = reinterpret_cast<const float*>(mat0 + (unsigned long long)s_idx[i] * row_bytes);
      const float w = HAS_VAL ? s_val[i] : 1.f;
      float m[KVT][VEC];
#pragma unroll
      for (int j = 0; j < KVT; j++)
        if (FULL || cvalid[j]) ldg_vec<VEC>(src + j * (32 * VEC), m[j]);
#pragma unroll
      for (int j = 0; j < KVT; j++) {
        if (FULL || cvalid[j]) {
#pragma unroll
          for (int x = 0; x < VEC; x++) {
            if (HAS_VAL) acc[j][x] = __fmaf_rn(w, m[j][x], acc[j][x]);
            else acc[j][x] = __fadd_rn(acc[j][x], m[j][x]);
          }
        }
      }
    }
  }
}

enum SpmmMode { MODE_ROWS = 0, MODE_ITEMS = 1 };

// MODE_ROWS: warp per row (rows longer than long_threshold are skipped when it is non-zero).
// MODE_ITEMS: warp per long-row item, partial sums to scratch.
template <typename IdxT, int VEC, int KVT, bool HAS_VAL, bool FULL, int MODE>
__global__ void __launch_bounds__(kSpmmWarps * 32) spmm_csr_kernel(const __grid_constant__ SpmmParams p) {
  __shared__ uint32_t s_idx[kSpmmWarps][32];
  __shared__ float s_val[kSpmmWarps][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * kSpmmWarps + warp;
  const IdxT* __restrict__ rowptr = reinterpret_cast<const IdxT*>(p.rowptr);
  const long long K = p.K;

  long long coff[KVT];
  bool cvalid[KVT];
#pragma unroll
  for (int j = 0; j < KVT; j++) {
    coff[j] = ((long long)blockIdx.y * (32 * KVT) + lane + 32 * j) * VEC;
    cvalid[j] = coff[j] < K;
  }
  float acc[KVT][VEC];
#pragma unroll
  for (int j = 0; j < KVT; j++)
#pragma unroll
    for (int e = 0; e < VEC; e++) acc[j][e] = 0.f;

  long long begin, end;
  float* dst;
  long long count = 0;
  if (MODE == MODE_ROWS) {
    if (unit >= p.M) return;
    begin = (long long)rowptr[unit];
    end = (long long)rowptr[unit + 1];
    count = end - begin;
    if (p.long_threshold > 0 && count > p.long_threshold) return;
    dst = output_row(p, unit);
  } else {
    if (unit >= p.n_items) return;
    begin = p.item_begin[unit];
    end = p.item_end[unit];
    dst = p.scratch + (long long)(p.item_slot ? p.item_slot[unit] : (int)unit) * K;
  }
  // Lanes past the last column gather the row's first columns instead (an address the lanes before them read
  // anyway) and their sums are dropped: the inner loop then carries no column predicate.  With one, the
  // compiler kept all gathers of a group live at once (96 registers against 40) and an operand of 80 - 100
  // columns took 7.0 ms at 128 M edges where 128 columns take 4.5 ms.
  long long cload[KVT];
#pragma unroll
  for (int j = 0; j < KVT; j++) cload[j] = cvalid[j] ? coff[j] : (long long)j * (32 * VEC);
  accumulate_edges<IdxT, VEC, KVT, HAS_VAL, true>(p, begin, end, cload, cvalid, s_idx[warp], s_val[warp], lane, acc);

  if (MODE == MODE_ROWS && p.mean) {
    const float dv = (float)(count > 0 ? count : 1);  // reducer.cuh:75-76
#pragma unroll
    for (int j = 0; j < KVT; j++)
#pragma unroll
      for (int x = 0; x < VEC; x++) acc[j][x] = __fdiv_rn(acc[j][x], dv);
  }
#pragma unroll
  for (int j = 0; j < KVT; j++)
    if (FULL || cvalid[j]) st_vec<VEC>(dst + coff[j], acc[j]);
}

// Adds the partial sums of each long row in item order and writes the row of the output.
template <typename IdxT>
__global__ void __launch_bounds__(128) spmm_long_reduce_kernel(const __grid_constant__ SpmmParams p) {
  const long long i = blockIdx.x;
  if (i >= p.n_long) return;
  const IdxT* __restrict__ rowptr = reinterpret_cast<const IdxT*>(p.rowptr);
  const long long row = p.long_row[i];
  const int s0 = p.long_item_ptr[i], s1 = p.long_item_ptr[i + 1];
  const long long cnt = (long long)rowptr[row + 1] - (long long)rowptr[row];
  const float dv = (float)(cnt > 0 ? cnt : 1);
  float* __restrict__ dst = output_row(p, row);
  for (long long c = threadIdx.x; c < p.K; c += blockDim.x) {
    float a = 0.f;
    for (int s = s0; s < s1; s++) a = __fadd_rn(a, p.scratch[(long long)s * p.K + c]);
    dst[c] = p.mean ? __fdiv_rn(a, dv) : a;
  }
}

// Narrow operands (K <= 64): a group of LPE = 4, 8 or 16 lanes (LPE x float4 = the whole row of the operand) owns
// one row of the adjacency, so a warp works on 32 / LPE rows at once and keeps that many independent chains of
// index load -> gathers in flight.  With one row per warp a narrow operand is bound by those chains, not by
// bytes: at 128 M edges a pass over 16, 32 or 64 columns took 1.8, 2.0 and 2.8 ms against 4.4 ms for 128
// columns.  A group walks its row eight edges at a time: its lanes load the eight column indices (the next
// eight are requested before the gathers of the current ones are consumed), every lane gets each index by a
// shuffle, gathers its float4 of that source row and adds the eight in edge order, so a row's sum is the
// strict CSR-order sum (the pieces of long rows are still added separately).  The groups of a warp run until
// the longest of their rows is done; callers that pass `row_order` (rows sorted by length) give every warp rows
// of equal length.
template <typename IdxT, bool HAS_VAL, int MODE, int LPE>
__global__ void __launch_bounds__(kSpmmWarps * 32) spmm_csr_multi_kernel(const __grid_constant__ SpmmParams p) {
  constexpr int kRows = 32 / LPE;              // rows (or long-row pieces) per warp
  constexpr int kBatch = 8;                    // edges per step and group
  constexpr int NI = LPE >= kBatch ? 1 : kBatch / LPE;   // index registers per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPE, hl = lane % LPE;
  const long long unit = ((long long)blockIdx.x * kSpmmWarps + warp) * kRows + grp;
  const IdxT* __restrict__ rowptr = reinterpret_cast<const IdxT*>(p.rowptr);
  const IdxT* __restrict__ col = reinterpret_cast<const IdxT*>(p.col);
  const long long K = p.K;
  const long long coff = ((long long)blockIdx.y * LPE + hl) * 4;
  const bool cvalid = coff < K;

  long long begin = 0, len = 0;
  float* dst = nullptr;
  bool live = false;
  if (MODE == MODE_ROWS) {
    if (unit < p.M) {
      const long long row = p.row_order ? (long long)p.row_order[unit] : unit;
      begin = (long long)rowptr[row];
      len = (long long)rowptr[row + 1] - begin;
      live = !(p.long_threshold > 0 && len > p.long_threshold);
      dst = output_row(p, row);
    }
  } else {
    if (unit < p.n_items) {
      begin = p.item_begin[unit];
      len = p.item_end[unit] - begin;
      live = true;
      dst = p.scratch + (long long)(p.item_slot ? p.item_slot[unit] : (int)unit) * K;
    }
  }
  const long long count = len;
  if (!live) len = 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const unsigned long long row_bytes = (unsigned long long)K * 4ull;
  const char* __restrict__ mat0 = reinterpret_cast<const char*>(p.mat + (cvalid ? coff : 0));
  const IdxT* __restrict__ mycol = col + begin;
  const float* __restrict__ myval = HAS_VAL ? p.val + begin : nullptr;

  uint32_t idx[NI];
  float val[NI];
#pragma unroll
  for (int q = 0; q < NI; q++) {
    const int pos = q * LPE + hl;
    idx[q] = 0;
    val[q] = 0.f;
    if (pos < kBatch && pos < len) {
      idx[q] = (uint32_t)mycol[pos];
      if (HAS_VAL) val[q] = __ldg(myval + pos);
    }
  }
  for (long long b = 0; __any_sync(0xffffffffu, b < len); b += kBatch) {
    uint32_t nidx[NI];
    float nval[NI];
#pragma unroll
    for (int q = 0; q < NI; q++) {
      const int in_batch = q * LPE + hl;
      const long long pos = b + kBatch + in_batch;
      nidx[q] = 0;
      nval[q] = 0.f;
      if (in_batch < kBatch && pos < len) {
        nidx[q] = (uint32_t)mycol[pos];
        if (HAS_VAL) nval[q] = __ldg(myval + pos);
      }
    }
    float4 m[kBatch];
    float w[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      const uint32_t ij = __shfl_sync(0xffffffffu, idx[j / LPE], j % LPE, LPE);
      w[j] = HAS_VAL ? __shfl_sync(0xffffffffu, val[j / LPE], j % LPE, LPE) : 0.f;
      m[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (b + j < len && cvalid) m[j] = __ldg(reinterpret_cast<const float4*>(mat0 + (unsigned long long)ij * row_bytes));
    }
#pragma unroll
    for (int j = 0; j < kBatch; j++) {
      if (HAS_VAL) {
        acc[0] = __fmaf_rn(w[j], m[j].x, acc[0]); acc[1] = __fmaf_rn(w[j], m[j].y, acc[1]);
        acc[2] = __fmaf_rn(w[j], m[j].z, acc[2]); acc[3] = __fmaf_rn(w[j], m[j].w, acc[3]);
      } else {
        acc[0] = __fadd_rn(acc[0], m[j].x); acc[1] = __fadd_rn(acc[1], m[j].y);
        acc[2] = __fadd_rn(acc[2], m[j].z); acc[3] = __fadd_rn(acc[3], m[j].w);
      }
    }
#pragma unroll
    for (int q = 0; q < NI; q++) {
      idx[q] = nidx[q];
      val[q] = nval[q];
    }
  }
  if (MODE == MODE_ROWS && p.mean) {
    const float dv = (float)(count > 0 ? count : 1);  // reducer.cuh:75-76
#pragma unroll
    for (int x = 0; x < 4; x++) acc[x] = __fdiv_rn(acc[x], dv);
  }
  if (live && cvalid) *reinterpret_cast<float4*>(dst + coff) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

template <typename IdxT, bool HAS_VAL, int LPE>
static int launch_spmm_multi(const SpmmParams& p, cudaStream_t st) {
  const unsigned gy = (unsigned)((p.K + 4 * LPE - 1) / (4 * LPE));
  constexpr long long per_cta = (long long)kSpmmWarps * (32 / LPE);
  {
    dim3 grid((unsigned)((p.M + per_cta - 1) / per_cta), gy);
    spmm_csr_multi_kernel<IdxT, HAS_VAL, MODE_ROWS, LPE><<<grid, kSpmmWarps * 32, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
  }
  if (p.n_items > 0) {
    dim3 grid((unsigned)((p.n_items + per_cta - 1) / per_cta), gy);
    spmm_csr_multi_kernel<IdxT, HAS_VAL, MODE_ITEMS, LPE><<<grid, kSpmmWarps * 32, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
    spmm_long_reduce_kernel<IdxT><<<(unsigned)p.n_long, 128, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
  }
  return EXB_OK;
}

template <typename IdxT, bool HAS_VAL>
static int launch_spmm_pair(const SpmmParams& p, cudaStream_t st) {
  if (p.K <= 16) return launch_spmm_multi<IdxT, HAS_VAL, 4>(p, st);
  if (p.K <= 32) return launch_spmm_multi<IdxT, HAS_VAL, 8>(p, st);
  return launch_spmm_multi<IdxT, HAS_VAL, 16>(p, st);
}

template <typename IdxT, int VEC, int KVT, bool HAS_VAL, bool FULL>
static int launch_spmm_mode(const SpmmParams& p, cudaStream_t st) {
  const long long C = p.K / VEC;
  const unsigned gy = (unsigned)((C + 32 * KVT - 1) / (32 * KVT));
  {
    dim3 grid((unsigned)((p.M + kSpmmWarps - 1) / kSpmmWarps), gy);
    spmm_csr_kernel<IdxT, VEC, KVT, HAS_VAL, FULL, MODE_ROWS><<<grid, kSpmmWarps * 32, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
  }
  if (p.n_items > 0) {
    dim3 grid((unsigned)((p.n_items + kSpmmWarps - 1) / kSpmmWarps), gy);
    spmm_csr_kernel<IdxT, VEC, KVT, HAS_VAL, FULL, MODE_ITEMS><<<grid, kSpmmWarps * 32, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
    spmm_long_reduce_kernel<IdxT><<<(unsigned)p.n_long, 128, 0, st>>>(p);
    EXB_CUDA_OK(cudaGetLastError());
  }
  return EXB_OK;
}

template <typename IdxT, int VEC, bool HAS_VAL>
static int launch_spmm_kvt(const SpmmParams& p, cudaStream_t st) {
  const long long C = p.K / VEC;
  const long long per32 = (C + 31) / 32;
  // 128-column tiles (one float4 per lane): narrower tiles keep more source rows of a large operand in L2
  // per pass over the graph and were 5 - 13 % faster than 256- or 512-column tiles at every size measured.
  (void)per32;
  const int kvt = 1;
  const bool full = C % (32 * kvt) == 0;
#define EXB_SPMM_CASE(KVT_)                                                                          \
  if (kvt == KVT_) {                                                                                 \
    return full ? launch_spmm_mode<IdxT, VEC, KVT_, HAS_VAL, true>(p, st)                            \
                : launch_spmm_mode<IdxT, VEC, KVT_, HAS_VAL, false>(p, st);                          \
  }
  EXB_SPMM_CASE(1)
#undef EXB_SPMM_CASE
  return EXB_ERR_UNSUPPORTED;
}

template <typename IdxT, bool HAS_VAL>
static int launch_spmm_vec(const SpmmParams& p, cudaStream_t st) {
  uintptr_t a = reinterpret_cast<uintptr_t>(p.mat) | reinterpret_cast<uintptr_t>(p.out);
  if (p.scratch) a |= reinterpret_cast<uintptr_t>(p.scratch);
  for (int i = 0; i < p.route_n; i++) a |= reinterpret_cast<uintptr_t>(p.route_dst[i]);
  if (p.route_n) a |= (uintptr_t)(p.route_ld * 4) | (uintptr_t)(p.route_col0 * 4);
  if (p.K <= 64 && p.K % 4 == 0 && a % 16 == 0) return launch_spmm_pair<IdxT, HAS_VAL>(p, st);
  if (p.K % 4 == 0 && a % 16 == 0) return launch_spmm_kvt<IdxT, 4, HAS_VAL>(p, st);
  if (p.K % 2 == 0 && a % 8 == 0) return launch_spmm_kvt<IdxT, 2, HAS_VAL>(p, st);
  return launch_spmm_kvt<IdxT, 1, HAS_VAL>(p, st);
}

static int spmm_common(SpmmParams& p, int idx_bytes, int reduce, cudaStream_t st) {
  EXB_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "spmm: idx_bytes must be 4 or 8 (got %d)", idx_bytes);
  p.regroup = (reduce & EXACT_SPMM_REGROUP) != 0;
  reduce &= ~EXACT_SPMM_REGROUP;
  EXB_REQUIRE(reduce == EXACT_REDUCE_SUM || reduce == EXACT_REDUCE_MEAN, "spmm: reduce must be sum or mean");
  EXB_REQUIRE(p.M >= 0 && p.K >= 0, "spmm: negative shape");
  if (p.M == 0 || p.K == 0) return EXB_OK;
  EXB_REQUIRE(p.rowptr && p.mat && (p.out || p.route_n > 0), "spmm: null pointer");
  EXB_REQUIRE((p.M + kSpmmWarps - 1) / kSpmmWarps <= 2147483647LL, "spmm: too many rows");
  EXB_REQUIRE(p.K * 4 < (1LL << 32), "spmm: K too large");
  // Column indices are staged as 32-bit values (also on the int64 path): operands of 2^32 rows or more are
  // out of range.  The number of operand rows is not an argument, so the bound is stated on M (square
  // adjacencies and their row shards satisfy it whenever the operand does).
  EXB_REQUIRE(p.M < (1LL << 32), "spmm: more than 2^32 - 1 rows");
  p.mean = reduce == EXACT_REDUCE_MEAN;
  if (idx_bytes == 4) {
    return p.val ? launch_spmm_vec<int32_t, true>(p, st) : launch_spmm_vec<int32_t, false>(p, st);
  }
  return p.val ? launch_spmm_vec<int64_t, true>(p, st) : launch_spmm_vec<int64_t, false>(p, st);
}

// Gradient with respect to the edge values (spmm_cuda.cu:172-209): one warp per edge,
// out[e] = dot(mat[col[e], :], grad[row[e], :]) (/ max(row length, 1) for mean).  Lane l accumulates columns
// l, l + 32, ... with one FMA each, then the lanes are added by the reference's shuffle-down tree, so the
// value equals the reference's bit for bit.
template <typename IdxT>
__global__ void __launch_bounds__(256) spmm_value_bw_kernel(const IdxT* __restrict__ row, const IdxT* __restrict__ rowptr,
                                                            const IdxT* __restrict__ col, const float* __restrict__ mat,
                                                            const float* __restrict__ grad, long long E, long long K,
                                                            int mean, float* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (e >= E) return;
  const long long r = (long long)row[e], c = (long long)col[e];
  const float* m = mat + c * K;
  const float* g = grad + r * K;
  float val = 0.f;
  for (long long k = lane; k < K; k += 32) val = __fmaf_rn(__ldg(m + k), __ldg(g + k), val);
#pragma unroll
  for (int i = 16; i > 0; i >>= 1) val = __fadd_rn(val, __shfl_down_sync(0xffffffffu, val, i));
  if (lane == 0) {
    if (mean) {
      const long long deg = (long long)rowptr[r + 1] - (long long)rowptr[r];
      val = __fdiv_rn(val, (float)(deg > 1 ? deg : 1));
    }
    out[e] = val;
  }
}

// max / min aggregation with the position of the winning edge (spmm_cuda.cu:27-104 with REDUCE = MAX / MIN;
// reducer.cuh:43-85): out[r, c] = max_e value[e] * mat[col[e], c], arg[r, c] = the first edge that attains it
// (a later edge replaces the current one only when strictly greater / smaller), rows without edges give 0 and
// arg = nnz.  One warp per row and 32 columns; lane = column, edges in CSR order.
template <typename IdxT, bool HAS_VAL, bool IS_MAX>
__global__ void __launch_bounds__(256) spmm_minmax_kernel(const IdxT* __restrict__ rowptr, const IdxT* __restrict__ col,
                                                          const float* __restrict__ val, const float* __restrict__ mat,
                                                          long long M, long long K, long long nnz, float* __restrict__ out,
                                                          IdxT* __restrict__ arg_out) {
  const int lane = threadIdx.x & 31;
  const long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long c = (long long)blockIdx.y * 32 + lane;
  if (r >= M) return;
  const long long begin = (long long)rowptr[r], end = (long long)rowptr[r + 1];
  float best = IS_MAX ? -3.402823466e+38f : 3.402823466e+38f;   // numeric_limits lowest() / max()
  long long arg = nnz;
  for (long long e = begin; e < end; e++) {
    const long long src = (long long)col[e];
    if (c < K) {
      float v = __ldg(mat + src * K + c);
      if (HAS_VAL) v = __fmul_rn(__ldg(val + e), v);
      if (IS_MAX ? (v > best) : (v < best)) {
        best = v;
        arg = e;
      }
    }
  }
  if (c < K) {
    out[r * K + c] = end > begin ? best : 0.f;           // reducer.cuh:78-84
    arg_out[r * K + c] = end > begin ? (IdxT)arg : (IdxT)nnz;
  }
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_spmm_minmax(const void* rowptr, const void* col, int idx_bytes, const float* value, const float* mat,
                      int64_t M, int64_t K, int64_t nnz, int is_max, float* out, void* arg_out, void* stream) {
  EXB_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "spmm_minmax: idx_bytes must be 4 or 8 (got %d)", idx_bytes);
  EXB_REQUIRE(M >= 0 && K >= 0 && nnz >= 0, "spmm_minmax: negative shape");
  if (M == 0 || K == 0) return EXB_OK;
  EXB_REQUIRE(rowptr && mat && out && arg_out && (nnz == 0 || col), "spmm_minmax: null pointer");
  EXB_REQUIRE((M + 7) / 8 <= 2147483647LL && (K + 31) / 32 <= 65535, "spmm_minmax: shape too large");
  dim3 grid((unsigned)((M + 7) / 8), (unsigned)((K + 31) / 32));
  cudaStream_t st = (cudaStream_t)stream;
#define EXB_MM(IDX_, HV_, MX_)                                                                                   \
  spmm_minmax_kernel<IDX_, HV_, MX_><<<grid, 256, 0, st>>>(static_cast<const IDX_*>(rowptr), static_cast<const IDX_*>(col), \
                                                           value, mat, M, K, nnz, out, static_cast<IDX_*>(arg_out))
  if (idx_bytes == 4) {
    if (value) { if (is_max) EXB_MM(int32_t, true, true); else EXB_MM(int32_t, true, false); }
    else { if (is_max) EXB_MM(int32_t, false, true); else EXB_MM(int32_t, false, false); }
  } else {
    if (value) { if (is_max) EXB_MM(int64_t, true, true); else EXB_MM(int64_t, true, false); }
    else { if (is_max) EXB_MM(int64_t, false, true); else EXB_MM(int64_t, false, false); }
  }
#undef EXB_MM
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_spmm_value_bw(const void* row, const void* rowptr, const void* col, int idx_bytes, const float* mat,
                        const float* grad, int64_t E, int64_t K, int reduce, float* out, void* stream) {
  EXB_REQUIRE(idx_bytes == 4 || idx_bytes == 8, "spmm_value_bw: idx_bytes must be 4 or 8 (got %d)", idx_bytes);
  EXB_REQUIRE(reduce == EXACT_REDUCE_SUM || reduce == EXACT_REDUCE_MEAN, "spmm_value_bw: reduce must be sum or mean");
  EXB_REQUIRE(E >= 0 && K >= 0, "spmm_value_bw: negative shape");
  if (E == 0) return EXB_OK;
  EXB_REQUIRE(row && col && mat && grad && out && (reduce == EXACT_REDUCE_SUM || rowptr), "spmm_value_bw: null pointer");
  EXB_REQUIRE((E + 7) / 8 <= 2147483647LL, "spmm_value_bw: too many edges");
  const unsigned blocks = (unsigned)((E + 7) / 8);
  const int mean = reduce == EXACT_REDUCE_MEAN;
  if (idx_bytes == 4)
    spmm_value_bw_kernel<int32_t><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        static_cast<const int32_t*>(row), static_cast<const int32_t*>(rowptr), static_cast<const int32_t*>(col), mat, grad, E,
        K, mean, out);
  else
    spmm_value_bw_kernel<int64_t><<<blocks, 256, 0, (cudaStream_t)stream>>>(
        static_cast<const int64_t*>(row), static_cast<const int64_t*>(rowptr), static_cast<const int64_t*>(col), mat, grad, E,
        K, mean, out);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

int exact_spmm(const void* rowptr, const void* col, int idx_bytes, const float* value, const float* mat,
               int64_t M, int64_t K, int reduce, float* out, void* stream) {
  SpmmParams p{};
  p.rowptr = rowptr; p.col = col; p.val = value; p.mat = mat; p.out = out; p.M = M; p.K = K;
  return spmm_common(p, idx_bytes, reduce, (cudaStream_t)stream);
}

int exact_spmm_split(const void* rowptr, const void* col, int idx_bytes, const float* value, const float* mat,
                     int64_t M, int64_t K, int reduce, int64_t long_threshold, const int32_t* item_row,
                     const int64_t* item_begin, const int64_t* item_end, const int32_t* item_slot,
                     int64_t n_items, const int32_t* long_row, const int32_t* long_item_ptr, int64_t n_long,
                     float* scratch, float* out, void* stream) {
  EXB_REQUIRE(long_threshold > 0, "spmm_split: long_threshold must be positive");
  EXB_REQUIRE(n_items >= 0 && n_long >= 0, "spmm_split: negative plan size");
  EXB_REQUIRE(n_items <= 2147483647LL && n_long <= 2147483647LL, "spmm_split: plan too large");
  if (n_items > 0)
    EXB_REQUIRE(item_row && item_begin && item_end && long_row && long_item_ptr && scratch && n_long > 0,
                "spmm_split: null plan array or scratch");
  SpmmParams p{};
  p.rowptr = rowptr; p.col = col; p.val = value; p.mat = mat; p.out = out; p.M = M; p.K = K;
  p.long_threshold = long_threshold;
  p.item_row = item_row; p.item_begin = reinterpret_cast<const long long*>(item_begin);
  p.item_end = reinterpret_cast<const long long*>(item_end); p.item_slot = item_slot; p.n_items = n_items;
  p.long_row = long_row; p.long_item_ptr = long_item_ptr; p.n_long = n_long; p.scratch = scratch;
  return spmm_common(p, idx_bytes, reduce, (cudaStream_t)stream);
}

int exact_spmm_split_routed(const void* rowptr, const void* col, int idx_bytes, const float* value, const float* mat,
                            int64_t M, int64_t K, int reduce, int64_t long_threshold, const int32_t* item_row,
                            const int64_t* item_begin, const int64_t* item_end, const int32_t* item_slot,
                            int64_t n_items, const int32_t* long_row, const int32_t* long_item_ptr, int64_t n_long,
                            float* scratch, const int32_t* row_order, int64_t shard, int64_t col0, int64_t ldd,
                            void* const* dst, int n_dst, void* stream) {
  EXB_REQUIRE(long_threshold >= 0 && n_items >= 0 && n_long >= 0, "spmm_split_routed: negative plan size");
  EXB_REQUIRE(n_items <= 2147483647LL && n_long <= 2147483647LL, "spmm_split_routed: plan too large");
  if (n_items > 0)
    EXB_REQUIRE(long_threshold > 0 && item_row && item_begin && item_end && long_row && long_item_ptr && scratch &&
                    n_long > 0,
                "spmm_split_routed: null plan array or scratch");
  EXB_REQUIRE(n_dst >= 1 && n_dst <= 8 && dst != nullptr, "spmm_split_routed: 1 to 8 destinations");
  EXB_REQUIRE(shard > 0 && (int64_t)n_dst * shard >= M, "spmm_split_routed: %d destinations of %lld rows do not hold %lld rows",
              n_dst, (long long)shard, (long long)M);
  EXB_REQUIRE(col0 >= 0 && K >= 0 && ldd >= col0 + K, "spmm_split_routed: columns %lld .. %lld exceed the row pitch %lld",
              (long long)col0, (long long)(col0 + K), (long long)ldd);
  SpmmParams p{};
  p.rowptr = rowptr; p.col = col; p.val = value; p.mat = mat; p.out = nullptr; p.M = M; p.K = K;
  p.long_threshold = n_items > 0 ? long_threshold : 0;
  p.item_row = item_row; p.item_begin = reinterpret_cast<const long long*>(item_begin);
  p.item_end = reinterpret_cast<const long long*>(item_end); p.item_slot = item_slot; p.n_items = n_items;
  p.long_row = long_row; p.long_item_ptr = long_item_ptr; p.n_long = n_long; p.scratch = scratch;
  p.route_n = n_dst; p.route_shard = shard; p.route_ld = ldd; p.route_col0 = col0;
  p.row_order = row_order;
  for (int i = 0; i < n_dst; i++) {
    EXB_REQUIRE(dst[i] != nullptr, "spmm_split_routed: null destination %d", i);
    p.route_dst[i] = static_cast<float*>(dst[i]);
  }
  return spmm_common(p, idx_bytes, reduce, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------
// exact_spmm_split for callers that cannot allocate device memory: the partial sums of the long-row
// pieces live in a fixed array inside the library image instead of a caller-supplied buffer.
static __device__ __align__(256) float g_split_scratch[EXACT_SPMM_STATIC_SCRATCH_FLOATS];

// The array's name is only a host-side handle; the device address the kernels need is looked up once
// per device (with that device current) and remembered.
static int static_scratch_address(float** out) {
  static std::mutex mu;
  static float* addr[64] = {nullptr};
  int dev = 0;
  EXB_CUDA_OK(cudaGetDevice(&dev));
  EXB_REQUIRE(dev >= 0 && dev < 64, "spmm_split_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    EXB_CUDA_OK(cudaGetSymbolAddress(&p, g_split_scratch));
    addr[dev] = static_cast<float*>(p);
  }
  *out = addr[dev];
  return EXB_OK;
}

int exact_spmm_split_static(const void* rowptr, const void* col, int idx_bytes, const float* value,
                            const float* mat, int64_t M, int64_t K, int reduce, int64_t long_threshold,
                            const int32_t* item_row, const int64_t* item_begin, const int64_t* item_end,
                            const int32_t* item_slot, int64_t n_items, const int32_t* long_row,
                            const int32_t* long_item_ptr, int64_t n_long, float* out, void* stream) {
  EXB_REQUIRE(n_items >= 0 && K >= 0, "spmm_split_static: negative size");
  // compared by division: n_items * K may not fit in 64 bits
  EXB_REQUIRE(K == 0 || n_items <= (int64_t)EXACT_SPMM_STATIC_SCRATCH_FLOATS / K,
              "spmm_split_static: %lld pieces x %lld columns exceed the %lld floats of the built-in scratch array; "
              "use exact_spmm_split with a caller-owned buffer",
              (long long)n_items, (long long)K, (long long)EXACT_SPMM_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  return exact_spmm_split(rowptr, col, idx_bytes, value, mat, M, K, reduce, long_threshold, item_row, item_begin,
                          item_end, item_slot, n_items, long_row, long_item_ptr, n_long, scratch, out, stream);
}

}  // extern "C"
