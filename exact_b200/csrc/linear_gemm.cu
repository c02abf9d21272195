// Dense layer GEMM with fp32-equivalent accuracy on the tensor cores ("3xTF32"):
//
//     C[M, N] (+)= A[M, K] B[N, K]^T  (+ A2[M, K2] B2[N, K2]^T)  (+ bias[N])
//
// Replaces the fp32 cuBLAS GEMMs of the quantised linear layer: F.linear in qlinear.forward
// (exact/exact/ops.py:150) and grad_input = grad_output.mm(weight) of linear_backward
// (exact/exact/cpp_extension/backward_func.cc:86).  M is the number of node rows (millions), K and N are
// feature widths (<= 256 per call for N).
//
// Arithmetic.  Every fp32 operand is split into a tf32 head and a tf32 tail,
//     a = a_hi + a_lo,   a_hi = rna_tf32(a),   a_lo = rna_tf32(a - a_hi)      (|a_lo| <= 2^-11 |a|),
// and the product is accumulated in fp32 as  a_hi b_hi + a_lo b_hi + a_hi b_lo.  The dropped terms
// (a_lo b_lo and the rounding of the tails) are below 2^-21 |a b|, the size of the fp32 rounding of a
// plain fp32 dot product, so the result is as accurate as an fp32 SIMT GEMM at three tensor-core MMAs
// per tile instead of one fp32 FMA per product.  Non-finite inputs stay non-finite and confined to their
// rows, but an infinite element turns its output row into NaN where an fp32 GEMM gives +-inf (its tail is
// inf - inf).
//
// Structure (one CTA per SM, persistent over 128-row tiles of A, 14 warps):
//   warp 0     TMA producer.  Shared memory is a 192 KB ring of K-tile stages; a 32-column K tile uses three
//              parts: A (raw fp32 [128 x 32], 16 KB, the tail tile goes into the part's other half),
//              B_hi [Npad x 32] and B_lo [Npad x 32]: two stages at Npad = 256, up to four for narrow
//              outputs.  128-byte swizzle, no multicast.
//              The A tile of four K tiles ahead is requested into L2 (tensor prefetch): A is read from
//              HBM exactly once and the ring is only two K tiles deep.
//   warps 2-9  converter: rewrite the raw A tile in place as a_hi and write a_lo beside it (same swizzled
//              offsets), fence.proxy.async, signal.
//   warp 1     MMA issuer: tcgen05.mma.cta_group::1.kind::tf32, M = 128, N = Npad, K = 8; per K tile
//              8 MMAs (hi*hi, lo*hi) then release B_hi, 4 MMAs (hi*lo) then release A and B_lo.
//              Accumulators are double-buffered in TMEM.
//   warps 10-13 epilogue: tcgen05.ld -> per-warp staging tile in shared memory -> (+ bias, + old C)
//              -> coalesced global stores.
// B_hi / B_lo are produced once per call from the (small) weight matrix by a preparation kernel.
//
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, all roles leave their loops,
// bulk copies in flight are waited for (bounded), TMEM is freed and the status word is set.
#include <mutex>

#include "exact_b200.h"
#include "tc.cuh"

namespace exb {

constexpr int kLinTileM = 128;
constexpr int kLinTileK = 32;
constexpr int kLinConvWarps = 8;
constexpr int kLinThreads = (2 + kLinConvWarps + 4) * 32;   // TMA, MMA, converters, epilogue
constexpr int kLinSlots = 6;                    // ring capacity in 32 KB units
constexpr int kLinMaxStages = 4;
constexpr int kLinBars = kLinMaxStages * 3;
constexpr uint32_t kLinSlotBytes = 32 * 1024;
constexpr uint32_t kLinHalf = 16 * 1024;        // raw / tail halves of an A slot
constexpr int kLinSleepNs = 200;                // back-off between polls of the roles that wait long (producer, epilogue)
constexpr int kLinPrefetch = 4;                 // K tiles of A requested into L2 ahead of their TMA load

struct LinParams {
  float* C;
  const float* bias;
  int* status;
  int* lib_status;    // library-wide status word of this device (capi.cu), or null
  long long M, ldc;
  int N, Npad;
  int kblocks1, kblocks;   // K tiles of the first operand pair, and of both pairs together
  int num_tiles;
  int accumulate;          // C += ... instead of C = ...
  int stages;              // K tiles the ring holds (2 at Npad = 256, up to 4 for narrow outputs)
  unsigned b_slot;         // bytes of a B_hi / B_lo slot = Npad * 128
  unsigned stage_bytes;    // A slot (32 KB) + two B slots
  unsigned tmem_cols;
};

__device__ __forceinline__ uint32_t rna_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
// (head, tail) of the split.  A non-finite element has a NaN tail (inf - inf), so its output row is NaN.
__device__ __forceinline__ void split_tf32(float a, float& hi, float& lo) {
  hi = __uint_as_float(rna_tf32(a));
  lo = __uint_as_float(rna_tf32(__fsub_rn(a, hi)));
}
__device__ __forceinline__ void fence_proxy_async_smem_lin() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Part `it` of the stream of ring parts (three per K tile: A, B_hi, B_lo): barrier index, phase, address.
struct LinPart { int b; uint32_t ph; uint32_t addr; };
__device__ __forceinline__ LinPart lin_part(int it, const LinParams& p, uint32_t ring) {
  const int kt = it / 3, part = it - kt * 3;
  const int stage = kt % p.stages;
  LinPart r;
  r.b = stage * 3 + part;
  r.ph = (uint32_t)(kt / p.stages) & 1u;
  r.addr = ring + (uint32_t)stage * p.stage_bytes +
           (part == 0 ? 0u : (part == 1 ? kLinSlotBytes : kLinSlotBytes + p.b_slot));
  return r;
}

__global__ void __launch_bounds__(kLinThreads, 1)
linear_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_a2,
                     const __grid_constant__ CUtensorMap tm_bh, const __grid_constant__ CUtensorMap tm_bl,
                     const __grid_constant__ LinParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_full[kLinBars];
  __shared__ __align__(8) unsigned long long s_empty[kLinBars];
  __shared__ __align__(8) unsigned long long s_conv[kLinBars];
  __shared__ __align__(8) unsigned long long s_tfull[2];
  __shared__ __align__(8) unsigned long long s_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_base = ring + kLinSlots * kLinSlotBytes;   // 4 x 4 KB epilogue staging tiles
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < kLinBars; s++) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
      mbar_init(smem_u32(&s_conv[s]), kLinConvWarps);   // one arrival per converter warp
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&s_tfull[b]), 1);
      mbar_init(smem_u32(&s_tempty[b]), 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int first = blockIdx.x, step = gridDim.x;
  const uint32_t b_bytes = (uint32_t)p.Npad * kLinTileK * 4;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;   // slot uses so far (three per K tile)
      bool ok = true;
      for (int tile = first; tile < p.num_tiles && ok; tile += step) {
        for (int kb = 0; kb < p.kblocks && ok; kb++) {
          for (int u = 0; u < 3; u++, it++) {
            const LinPart pt_ = lin_part(it, p, ring);
            if (!mbar_wait<kLinSleepNs>(smem_u32(&s_empty[pt_.b]), pt_.ph ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t full = smem_u32(&s_full[pt_.b]);
            const uint32_t dst = pt_.addr;
            if (u == 0) {
              mbar_arrive_expect_tx(full, kLinHalf);
              if (kb < p.kblocks1) tma_load_2d(dst, &tm_a, kb * kLinTileK, tile * kLinTileM, full);
              else tma_load_2d(dst, &tm_a2, (kb - p.kblocks1) * kLinTileK, tile * kLinTileM, full);
              // A comes from HBM exactly once: pull the tile that will be loaded kLinPrefetch K tiles from
              // now into L2, so that its TMA load later pays L2 latency only (the ring holds two K tiles)
              int pk = kb + kLinPrefetch, pt = tile;
              if (pk >= p.kblocks) { pk -= p.kblocks; pt += step; }
              if (pt < p.num_tiles && pk < p.kblocks) {
                if (pk < p.kblocks1) tma_prefetch_2d(&tm_a, pk * kLinTileK, pt * kLinTileM);
                else tma_prefetch_2d(&tm_a2, (pk - p.kblocks1) * kLinTileK, pt * kLinTileM);
              }
            } else {
              mbar_arrive_expect_tx(full, b_bytes);
              tma_load_2d(dst, u == 1 ? &tm_bh : &tm_bl, kb * kLinTileK, 0, full);
            }
          }
        }
      }
      if (!ok) {
        // leave no bulk copy in flight: wait (bounded) for every slot that was armed last
        const long long t0 = clock64();
        for (int j = 0; j < p.stages * 3 && j < it; j++) {
          const LinPart q = lin_part(it - 1 - j, p, ring);
          const uint32_t bar = smem_u32(&s_full[q.b]);
          const uint32_t ph = q.ph;
          while (!mbar_try_wait(bar, ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(kLinTileM, p.Npad);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
        const int buf = t & 1;
        const uint32_t tph = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(smem_u32(&s_tempty[buf]), tph ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.Npad);
        for (int kb = 0; kb < p.kblocks; kb++, it += 3) {
          const LinPart qa = lin_part(it, p, ring), qh = lin_part(it + 1, p, ring), ql = lin_part(it + 2, p, ring);
          const int sa = qa.b, sh = qh.b, sl = ql.b;
          const uint32_t pl = ql.ph;
          if (!mbar_wait(smem_u32(&s_conv[sa]), qa.ph, abort_flag)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&s_full[sh]), qh.ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t ahi = umma_desc_sw128(qa.addr);
          const uint64_t alo = umma_desc_sw128(qa.addr + kLinHalf);
          const uint64_t bhi = umma_desc_sw128(qh.addr);
          const uint64_t blo = umma_desc_sw128(ql.addr);
#pragma unroll
          for (int k4 = 0; k4 < kLinTileK / 8; k4++) {
            const uint64_t o = (uint64_t)(k4 * 2);   // 8 tf32 = 32 bytes along K inside the swizzle atom
            umma_tf32(d_tmem, alo + o, bhi + o, idesc, (kb | k4) != 0);
            umma_tf32(d_tmem, ahi + o, bhi + o, idesc, 1);
          }
          umma_commit(smem_u32(&s_empty[sh]));
          if (!mbar_wait(smem_u32(&s_full[sl]), pl, abort_flag)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < kLinTileK / 8; k4++) {
            const uint64_t o = (uint64_t)(k4 * 2);
            umma_tf32(d_tmem, ahi + o, blo + o, idesc, 1);
          }
          umma_commit(smem_u32(&s_empty[sa]));
          umma_commit(smem_u32(&s_empty[sl]));
        }
        if (ok) umma_commit(smem_u32(&s_tfull[buf]));
      }
    }
  } else if (warp < 2 + kLinConvWarps) {
    // ---------------- converter: warps 2 .. 2 + kLinConvWarps - 1 ----------------
    const int ct = threadIdx.x - 64;   // 0 .. 32 * kLinConvWarps - 1
    constexpr int kPer = (int)(kLinHalf / 16) / (32 * kLinConvWarps);   // 16-byte chunks per thread
    int it = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step) {
      for (int kb = 0; kb < p.kblocks; kb++, it += 3) {
        const LinPart qa = lin_part(it, p, ring);
        const int s = qa.b;
        if (!mbar_wait(smem_u32(&s_full[s]), qa.ph, abort_flag)) { ok = false; break; }
        const uint32_t base = qa.addr + (uint32_t)ct * 16u;
#pragma unroll
        for (int i = 0; i < kPer; i++) {
          const uint32_t addr = base + (uint32_t)i * (32u * kLinConvWarps * 16u);
          float a[4], h[4], l[4];
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a[0]), "=f"(a[1]), "=f"(a[2]), "=f"(a[3]) : "r"(addr));
#pragma unroll
          for (int e = 0; e < 4; e++) h[e] = __uint_as_float(rna_tf32(a[e]));
#pragma unroll
          for (int e = 0; e < 4; e += 2) {   // tails: paired subtract, then round to tf32
            float d0, d1;
            f2_unpack(f2_sub(f2_pack(a[e], a[e + 1]), f2_pack(h[e], h[e + 1])), d0, d1);
            l[e] = __uint_as_float(rna_tf32(d0));
            l[e + 1] = __uint_as_float(rna_tf32(d1));
          }
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(h[0]), "f"(h[1]), "f"(h[2]), "f"(h[3]) : "memory");
          asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr + kLinHalf), "f"(l[0]), "f"(l[1]), "f"(l[2]), "f"(l[3]) : "memory");
        }
        fence_proxy_async_smem_lin();  // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&s_conv[s]));
      }
    }
  } else {
    // ---------------- epilogue: the last four warps ----------------
    const int quad = warp & 3;   // TMEM lanes 32*quad .. 32*quad+31
    const bool vec = (p.N & 3) == 0 && (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0;
    const uint32_t stage_addr = stage_base + (uint32_t)quad * 4096u;
    int t = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
      const int buf = t & 1;
      const uint32_t ph = (uint32_t)(t >> 1) & 1u;
      if (!mbar_wait<kLinSleepNs>(smem_u32(&s_tfull[buf]), ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * p.Npad);
      const long long row_base = (long long)tile * kLinTileM + quad * 32;
      for (int c0 = 0; c0 < p.Npad; c0 += 32) {
        const int cols = (p.Npad - c0) < 32 ? (p.Npad - c0) : 32;   // 16 or 32
        for (int h = 0; h * 16 < cols; h++) {
          float v[16];
          tmem_ld16(taddr + (uint32_t)(c0 + h * 16), v);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t ci = (uint32_t)(h * 4 + j);
            const uint32_t addr = stage_addr + (uint32_t)lane * 128u + ((ci ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[4 * j]), "f"(v[4 * j + 1]),
                         "f"(v[4 * j + 2]), "f"(v[4 * j + 3])
                         : "memory");
          }
        }
        __syncwarp();
        const uint32_t ci = (uint32_t)lane & 7u;
        const int c = c0 + (int)ci * 4;
        float bv[4] = {0.f, 0.f, 0.f, 0.f};
        if (p.bias != nullptr) {
#pragma unroll
          for (int bb = 0; bb < 4; bb++)
            if (c + bb < p.N) bv[bb] = __ldg(p.bias + c + bb);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int rr = 4 * i + (lane >> 3);
          const long long nn = row_base + rr;
          float4 o;
          const uint32_t addr = stage_addr + (uint32_t)rr * 128u + ((ci ^ ((uint32_t)rr & 7u)) << 4);
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(addr));
          if (nn < p.M && (int)ci * 4 < cols && c < p.N) {
            float* __restrict__ d = p.C + nn * p.ldc + c;
            o.x += bv[0]; o.y += bv[1]; o.z += bv[2]; o.w += bv[3];
            if (vec) {   // N % 4 == 0, so c + 4 <= N
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(d);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              __stcs(reinterpret_cast<float4*>(d), o);
            } else {
              const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
              for (int bb = 0; bb < 4; bb++)
                if (c + bb < p.N) d[bb] = p.accumulate ? d[bb] + ov[bb] : ov[bb];
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_tempty[buf]));
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0 && s_abort) {
    atomicExch(p.status, 1);
    if (p.lib_status) atomicOr(p.lib_status, EXB_STATUS_LINEAR);
  }
}

// Heads and tails of [B | B2] (rows = output features), zero padded to [Npad, Kpad1 + Kpad2]; also
// clears the status word.
__global__ void linear_prepare_kernel(const float* __restrict__ B, int K, long long ldb, const float* __restrict__ B2,
                                      int K2, long long ldb2, int N, int Npad, int Kpad1, int Kpad,
                                      float* __restrict__ bh, float* __restrict__ bl, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *status = 0;
  if (i >= Npad * Kpad) return;
  const int n = i / Kpad, kk = i - n * Kpad;
  float v = 0.f;
  if (n < N) {
    if (kk < Kpad1) {
      if (kk < K) v = B[(long long)n * ldb + kk];
    } else if (kk - Kpad1 < K2) {
      v = B2[(long long)n * ldb2 + (kk - Kpad1)];
    }
  }
  float hi, lo;
  split_tf32(v, hi, lo);
  bh[i] = hi;
  bl[i] = lo;
}

static inline int lin_kpad(long long K) { return (int)((K + kLinTileK - 1) / kLinTileK * kLinTileK); }

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_linear_workspace_bytes(int64_t N, int64_t K, int64_t K2) {
  if (N <= 0 || K <= 0 || K2 < 0) return 256;
  const int64_t Npad = (N + 15) / 16 * 16;
  return 256 + 2 * Npad * (int64_t)(lin_kpad(K) + lin_kpad(K2)) * 4;
}

int exact_linear_forward(const float* A, int64_t M, int64_t K, int64_t lda, const float* B, int64_t ldb,
                         const float* A2, int64_t K2, int64_t lda2, const float* B2, int64_t ldb2, int64_t N,
                         const float* bias, int accumulate, void* workspace, float* C, int64_t ldc, void* stream) {
  EXB_REQUIRE(M >= 0 && K > 0 && N > 0 && K2 >= 0, "linear_forward: bad shape");
  if (M == 0) return EXB_OK;
  EXB_REQUIRE(A && B && C && workspace, "linear_forward: null pointer");
  EXB_REQUIRE((A2 != nullptr) == (K2 > 0) && (B2 != nullptr) == (K2 > 0), "linear_forward: the second operand pair needs A2, B2 and K2 > 0");
  EXB_REQUIRE(lda >= K && ldb >= K && ldc >= N && (K2 == 0 || (lda2 >= K2 && ldb2 >= K2)), "linear_forward: leading dimension smaller than the row");
  if (N > 256) return fail(EXB_ERR_UNSUPPORTED, "linear_forward: N = %lld exceeds one MMA tile (256); call per 256-column block", (long long)N);
  if (lda % 4 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) != 0 ||
      (K2 > 0 && (lda2 % 4 != 0 || (reinterpret_cast<uintptr_t>(A2) & 15) != 0)))
    return fail(EXB_ERR_UNSUPPORTED, "linear_forward: the TMA path needs 16-byte aligned rows of A (lda %% 4 == 0)");
  EXB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "linear_forward: workspace must be 256-byte aligned");
  EXB_REQUIRE((M + kLinTileM - 1) / kLinTileM < 2147483647LL / kLinTileM, "linear_forward: too many rows");
  cudaStream_t st = (cudaStream_t)stream;
  const int Npad = (int)((N + 15) / 16 * 16);
  const int Kpad1 = lin_kpad(K), Kpad2 = lin_kpad(K2), Kpad = Kpad1 + Kpad2;
  int* status = reinterpret_cast<int*>(workspace);
  float* bh = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
  float* bl = bh + (size_t)Npad * Kpad;

  linear_prepare_kernel<<<(Npad * Kpad + 255) / 256, 256, 0, st>>>(B, (int)K, ldb, B2, (int)K2, ldb2, (int)N, Npad,
                                                                   Kpad1, Kpad, bh, bl, status);
  EXB_CUDA_OK(cudaGetLastError());

  CUtensorMap tm_a, tm_a2, tm_bh, tm_bl;
  int rc = make_tensor_map_2d_f32(&tm_a, A, (unsigned long long)K, (unsigned long long)M, (unsigned long long)lda * 4, kLinTileK, kLinTileM);
  if (rc) return rc;
  if (K2 > 0) {
    rc = make_tensor_map_2d_f32(&tm_a2, A2, (unsigned long long)K2, (unsigned long long)M, (unsigned long long)lda2 * 4, kLinTileK, kLinTileM);
    if (rc) return rc;
  } else {
    tm_a2 = tm_a;
  }
  rc = make_tensor_map_2d_f32(&tm_bh, bh, (unsigned long long)Kpad, (unsigned long long)Npad, (unsigned long long)Kpad * 4, kLinTileK, (unsigned)Npad);
  if (rc) return rc;
  rc = make_tensor_map_2d_f32(&tm_bl, bl, (unsigned long long)Kpad, (unsigned long long)Npad, (unsigned long long)Kpad * 4, kLinTileK, (unsigned)Npad);
  if (rc) return rc;

  LinParams p{};
  p.C = C; p.bias = bias; p.status = status; p.lib_status = status_word_ptr(); p.M = M; p.ldc = ldc; p.N = (int)N; p.Npad = Npad;
  p.kblocks1 = Kpad1 / kLinTileK; p.kblocks = Kpad / kLinTileK;
  p.num_tiles = (int)((M + kLinTileM - 1) / kLinTileM);
  p.accumulate = accumulate ? 1 : 0;
  p.b_slot = (unsigned)Npad * kLinTileK * 4;
  p.stage_bytes = kLinSlotBytes + 2 * p.b_slot;
  p.stages = (int)((kLinSlots * kLinSlotBytes) / p.stage_bytes);
  if (p.stages > kLinMaxStages) p.stages = kLinMaxStages;
  unsigned cols = 32;
  while (cols < (unsigned)(2 * Npad)) cols <<= 1;
  p.tmem_cols = cols;
  const size_t dyn = (size_t)kLinSlots * kLinSlotBytes + 4 * 4096 + 1024;
  int grid = sm_count();
  if (grid > p.num_tiles) grid = p.num_tiles;
  EXB_CUDA_OK(cudaFuncSetAttribute(linear_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
  linear_tf32x3_kernel<<<grid, kLinThreads, dyn, st>>>(tm_a, tm_a2, tm_bh, tm_bl, p);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
