// Fused random projection + quantise + pack:  packed(quantise(X @ R))  in one kernel.
//
// Replaces the chain input2rp -> quantize_activation of exact/exact/ops.py:142-149 (and :273-280,
// layers.py:153-159): torch.matmul(input, rand_matrix) (ops.py:117, a cuBLAS SGEMM that writes the
// [N, k] fp32 product to HBM), then two row reductions, the scale, pack_single_precision and the bf16
// casts (ops.py:61-83).  Here the product never leaves the chip.
//
// Shape of the work.  X is [N, D] fp32 (row-major, so K-major for the MMA), R is [D, k] with entries
// +-1/sqrt(k), k = ceil(kept_frac * D) is small (8..128).  The arithmetic intensity is 2k/4 flop per
// byte of X, far below the tensor-core ridge: the kernel is bound by streaming X from HBM once, and the
// tensor core is what makes the k multiply-adds per loaded element free.
//
// Structure (one CTA per SM, persistent over 128-row tiles, 6 warps):
//   warp 0   TMA producer: cp.async.bulk.tensor 2D loads of a [128 x 32] fp32 box of X and a
//            [kpad x 32] box of sign(R)^T into a ring of shared-memory stages (128-byte swizzle),
//            completion on mbarriers.  No multicast anywhere.
//   warp 1   MMA issuer: tcgen05.mma.cta_group::1.kind::tf32, M = 128, N = kpad, K = 8 per instruction,
//            accumulating in TMEM; tcgen05.commit releases smem stages and publishes finished tiles.
//            Two accumulator buffers in TMEM let the epilogue of tile i overlap the MMAs of tile i+1.
//   warps 2-5  epilogue: tcgen05.ld 32x32b (thread = row), * 1/sqrt(k), row min / max, scale,
//            Philox noise, quantise, bytes assembled across the 8/bits adjacent lanes with shuffles,
//            packed stream + bf16 statistics to HBM.
// The B operand holds +-1 (exact in tf32); 1/sqrt(k) is applied in fp32 in the epilogue.  X is
// truncated to tf32 by the tensor core (10-bit mantissa): the product differs from the fp32 one by
// about 1e-3 relative, inside the 1e-2 relative-Frobenius criterion of this operator.
//
// Rows that are not 16-byte aligned (D % 4 != 0, e.g. the 602 features of the reddit-shaped configuration:
// 2408-byte rows) cannot be described by a tensor map.  For them the A operand is brought in by four more
// warps with cp.async (8-byte pieces when rows are 8-byte aligned, else 4-byte), each piece written straight
// to its place in the 128-byte-swizzled tile, columns past D and rows past N zero-filled; a thread signals a
// stage after its own copies of that stage have landed (cp.async.wait_group) and a fence.proxy.async has made
// them visible to the tensor core.  Several stages stay in flight per thread.
//
// k up to 512: an accumulator wider than one MMA (N <= 256) is produced by two MMAs per K step, side by
// side in TMEM; when two such accumulators no longer fit the 512 TMEM columns a single buffer is used.
//
// Every wait on an mbarrier is bounded (about one second of SM clock).  When a wait expires the CTA
// raises an abort flag, all roles leave their loops, outstanding bulk copies are waited for (bounded),
// TMEM is freed and a non-zero status word is left for the host.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "exact_b200.h"
#include "tc.cuh"

namespace exb {

constexpr int kRpTileM = 128;       // rows per tile = MMA M
constexpr int kRpTileK = 32;        // fp32 elements per smem row = 128 bytes = one swizzle atom
constexpr int kRpThreads = 192;     // 6 warps
constexpr int kRpAsyncThreads = 320;  // + 4 warps that copy A with cp.async
constexpr int kRpMaxStages = 10;

struct RpParams {
  uint8_t* packed;
  uint16_t* scale_bf16;
  uint16_t* min_bf16;
  float* y_out;       // optional [N, k] fp32 copy of the projection (tests)
  const float* x;     // A operand, read directly by the cp.async producers
  int piece;          // bytes per cp.async piece (8 or 4)
  int lag;            // stages a cp.async producer thread keeps in flight before it signals one
  int nbuf;           // accumulator buffers in TMEM (2, or 1 when 2 * kpad columns do not fit)
  int* status;        // device word: 0 = ok
  int* lib_status;    // library-wide status word of this device (capi.cu), or null
  long long N;
  long long row_offset;
  int D, k, kpad, bits;
  int num_tiles, kblocks, stages;
  unsigned stage_bytes;
  unsigned tmem_cols;
  float inv_sqrt_k;
  uint32_t off_lo, off_hi;
  PhiloxKey key;
};

// ---- the kernel -----------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most n of this thread's most recent cp.async groups are still pending.
__device__ __forceinline__ void cp_async_wait_pending(int n) {
  switch (n) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int BITS, bool ASYNC_A>
__global__ void __launch_bounds__(ASYNC_A ? kRpAsyncThreads : kRpThreads, ASYNC_A ? 1 : 4)
rp_pack_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_rt,
               const __grid_constant__ RpParams p) {
  constexpr int WPT = 8 / BITS;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_full[kRpMaxStages];
  __shared__ __align__(8) unsigned long long s_empty[kRpMaxStages];
  __shared__ __align__(8) unsigned long long s_tfull[2];
  __shared__ __align__(8) unsigned long long s_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // 1024-byte aligned stage ring
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < p.stages; s++) {
      // a stage is full when the TMA thread's bytes have landed and, with cp.async producers, each of their
      // 128 threads has signalled its pieces
      mbar_init(smem_u32(&s_full[s]), ASYNC_A ? 129 : 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&s_tfull[b]), 1);
      mbar_init(smem_u32(&s_tempty[b]), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  const int first = blockIdx.x, step = gridDim.x;
  const uint32_t a_bytes = kRpTileM * kRpTileK * 4;
  const uint32_t b_bytes = (uint32_t)p.kpad * kRpTileK * 4;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = first; tile < p.num_tiles && ok; tile += step) {
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int s = it % p.stages;
          const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t full = smem_u32(&s_full[s]);
          const uint32_t dst = tiles_base + (uint32_t)s * p.stage_bytes;
          mbar_arrive_expect_tx(full, (ASYNC_A ? 0u : a_bytes) + b_bytes);
          if (!ASYNC_A) tma_load_2d(dst, &tm_x, kb * kRpTileK, tile * kRpTileM, full);
          if (p.kpad <= 256) {
            tma_load_2d(dst + a_bytes, &tm_rt, kb * kRpTileK, 0, full);
          } else {   // two boxes of kpad / 2 rows (a box holds at most 256)
            tma_load_2d(dst + a_bytes, &tm_rt, kb * kRpTileK, 0, full);
            tma_load_2d(dst + a_bytes + b_bytes / 2, &tm_rt, kb * kRpTileK, p.kpad / 2, full);
          }
        }
      }
      if (!ok) {
        // leave no bulk copy in flight: wait (bounded) for every stage that was armed last
        const long long t0 = clock64();
        for (int j = 0; j < p.stages && j < it; j++) {
          const int jt = it - 1 - j;
          const uint32_t bar = smem_u32(&s_full[jt % p.stages]);
          const uint32_t ph = (uint32_t)(jt / p.stages) & 1u;
          while (!mbar_try_wait(bar, ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const int n_lo = p.kpad <= 256 ? p.kpad : 256, n_hi = p.kpad - n_lo;
      const uint32_t idesc = umma_idesc_tf32(kRpTileM, n_lo);
      const uint32_t idesc_hi = umma_idesc_tf32(kRpTileM, n_hi > 0 ? n_hi : 16);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
        const int buf = p.nbuf == 2 ? (t & 1) : 0;
        const uint32_t tph = (uint32_t)(p.nbuf == 2 ? (t >> 1) : t) & 1u;
        if (!mbar_wait(smem_u32(&s_tempty[buf]), tph ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.kpad);
        for (int kb = 0; kb < p.kblocks; kb++, it++) {
          const int s = it % p.stages;
          const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&s_full[s]), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles_base + (uint32_t)s * p.stage_bytes;
          const uint64_t a_desc = umma_desc_sw128(a_addr);
          const uint64_t b_desc = umma_desc_sw128(a_addr + a_bytes);
#pragma unroll
          for (int k4 = 0; k4 < kRpTileK / 8; k4++) {
            // advance 8 tf32 = 32 bytes along K inside the swizzle atom: +2 in the (addr >> 4) field
            umma_tf32(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0);
            // columns 256 .. kpad-1: rows 256.. of the B tile (32 KB further: a whole number of swizzle atoms)
            if (n_hi > 0)
              umma_tf32(d_tmem + 256u, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)((256 * 128) >> 4) + (uint64_t)(k4 * 2),
                        idesc_hi, (kb | k4) != 0);
          }
          umma_commit(smem_u32(&s_empty[s]));  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(smem_u32(&s_tfull[buf]));  // the tile's accumulator is complete
      }
    }
  } else if (ASYNC_A && warp >= 6) {
    // ---------------- cp.async producers of A: warps 6..9 ----------------
    const int t = threadIdx.x - kRpThreads;                 // 0 .. 127
    const int ppr = 128 / p.piece;                          // pieces per 128-byte tile row: 16 or 32
    const int pi = t % ppr, rg = t / ppr, rpp = 128 / ppr;  // this thread's piece, row group, rows per pass
    const int cbytes = pi * p.piece;                        // byte offset of the piece inside a tile row
    const int chunk = cbytes >> 4, within = cbytes & 15;
    int it = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step) {
      for (int kb = 0; kb < p.kblocks; kb++, it++) {
        const int s = it % p.stages;
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
        const int col = kb * kRpTileK + (cbytes >> 2);
        // a piece is inside the row or outside as a whole: 8-byte pieces are only used for even D
        const bool col_ok = col < p.D;
        // A producer warp has an SM sub-partition to itself, so the per-piece address arithmetic is kept to a
        // few independent instructions: source and destination advance by constants from row to row.
        const long long n0 = (long long)tile * kRpTileM + rg;
        const float* src = p.x + n0 * p.D + col;
        const long long src_step = (long long)rpp * p.D;
        uint32_t dst_row = tiles_base + (uint32_t)s * p.stage_bytes + (uint32_t)(rg * 128 + within);
        const long long rows_left = p.N - n0;     // rows n0, n0 + rpp, ... below N are real
        const int passes = kRpTileM / rpp;        // 16 (8-byte pieces) or 32 (4-byte pieces)
        if (p.piece == 8) {
#pragma unroll 4
          for (int i = 0; i < passes; i++) {
            const bool in = col_ok && (long long)(i * rpp) < rows_left;
            // rows advance by 8: the swizzle term (row % 8) is that of the first row
            const uint32_t dst = dst_row + (uint32_t)(i * rpp * 128) + (uint32_t)((chunk ^ (rg & 7)) << 4);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(in ? src : p.x), "r"(in ? 8u : 0u) : "memory");
            src += src_step;
          }
        } else {
#pragma unroll 4
          for (int i = 0; i < passes; i++) {
            const int r = rg + i * rpp;
            const bool in = col_ok && (long long)(i * rpp) < rows_left;
            const uint32_t dst = dst_row + (uint32_t)(i * rpp * 128) + (uint32_t)((chunk ^ (r & 7)) << 4);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(in ? src : p.x), "r"(in ? 4u : 0u) : "memory");
            src += src_step;
          }
        }
        cp_async_commit();
        if (it >= p.lag) {
          cp_async_wait_pending(p.lag);          // the copies of iteration it - lag have landed
          fence_proxy_async_smem();
          mbar_arrive(smem_u32(&s_full[(it - p.lag) % p.stages]));
        }
      }
    }
    cp_async_wait_pending(0);
    if (ok) {
      fence_proxy_async_smem();
      for (int j = it > p.lag ? it - p.lag : 0; j < it; j++) mbar_arrive(smem_u32(&s_full[j % p.stages]));
    }
  } else {
    // ---------------- epilogue: warps 2..5, thread = row ----------------
    const int quad = warp & 3;                 // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    const int row_in_tile = quad * 32 + lane;
    const float B = (float)((1 << BITS) - 1);
    const int CB8 = (p.k + 7) >> 3;
    int t = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
      const int buf = p.nbuf == 2 ? (t & 1) : 0;
      const uint32_t tph = (uint32_t)(p.nbuf == 2 ? (t >> 1) : t) & 1u;
      if (!mbar_wait(smem_u32(&s_tfull[buf]), tph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * p.kpad);
      const long long n = (long long)tile * kRpTileM + row_in_tile;
      const bool row_ok = n < p.N;

      // pass 1: row min / max of y = acc / sqrt(k) over the k real columns
      float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
      for (int c0 = 0; c0 < p.kpad; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + (uint32_t)c0, v);
#pragma unroll
        for (int j = 0; j < 16; j++) {
          if (c0 + j < p.k) {
            lo = min_nan(lo, v[j]);
            hi = max_nan(hi, v[j]);
          }
        }
      }
      // y = acc * (1/sqrt(k)) is monotone in acc, so min / max commute with the scaling
      lo = __fmul_rn(lo, p.inv_sqrt_k);
      hi = __fmul_rn(hi, p.inv_sqrt_k);
      const float sc = __fmul_rn(__frcp_rn(__fsub_rn(hi, lo)), B);  // exact/exact/ops.py:39
      if (row_ok) {
        p.scale_bf16[n] = f32_to_bf16_bits(sc);
        p.min_bf16[n] = f32_to_bf16_bits(lo);
      }

      // pass 2: quantise, assemble bytes over the WPT adjacent rows (= lanes), store
      const bool fast_tile = ((long long)(tile + 1) * kRpTileM <= p.N) && p.y_out == nullptr &&
                             __all_sync(0xffffffffu, sc > 0.f && sc < __int_as_float(0x7f800000));
      const long long gn = n + p.row_offset;
      const int sh = (lane % WPT) * BITS;
      const uint32_t keep = 0x01010101u * ((0xffu << sh) & 0xffu);
      const long long g = n / WPT;
      for (int c0 = 0; c0 < p.kpad; c0 += 16) {
        float v[16];
        tmem_ld16(taddr + (uint32_t)c0, v);
        if (c0 >= p.k) continue;  // uniform: padded columns only
        uint32_t code[16];
        if (fast_tile && c0 + 16 <= p.k) {
          // all 128 rows exist, all 16 columns are real, every scale of the warp is finite and non-zero:
          // paired fp32 arithmetic, rounding by adding 1.5 * 2^23 (the code is the low byte of the sum)
          const f32x2 inv2 = f2_pack(p.inv_sqrt_k, p.inv_sqrt_k);
          const f32x2 lo2 = f2_pack(lo, lo), sc2 = f2_pack(sc, sc);
          const f32x2 neg_half = f2_pack(-0.5f, -0.5f), magic = f2_pack(12582912.f, 12582912.f);
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const unsigned long long q = (unsigned long long)(gn * CB8 + ((c0 >> 3) + h));
            uint32_t w[4];
            philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
#pragma unroll
            for (int jp = 0; jp < 4; jp++) {
              const int c = h * 8 + 2 * jp;
              const f32x2 u2 = noise16_to_unit(f2_pack(u16_lo_to_1p(w[jp]), u16_hi_to_1p(w[jp])));
              const f32x2 y2 = f2_mul(f2_pack(v[c], v[c + 1]), inv2);
              const f32x2 t2 = f2_add(f2_add(f2_fma(f2_sub(y2, lo2), sc2, u2), neg_half), magic);
              float t0, t1;
              f2_unpack(t2, t0, t1);
              code[c] = __float_as_uint(t0);
              code[c + 1] = __float_as_uint(t1);
            }
          }
        } else
#pragma unroll
        for (int h = 0; h < 2; h++) {  // two blocks of 8 columns, one Philox call each
          const unsigned long long q = (unsigned long long)(gn * CB8 + ((c0 >> 3) + h));
          uint32_t w[4];
          philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int c = h * 8 + j;
            const float u = (j & 1) ? u16_hi_to_unit(w[j >> 1]) : u16_lo_to_unit(w[j >> 1]);
            const float y = __fmul_rn(v[c], p.inv_sqrt_k);
            if (p.y_out != nullptr && row_ok && c0 + c < p.k) p.y_out[n * p.k + c0 + c] = y;
            // quantization_cuda_kernel.cu:89
            const float tq = __fsub_rn(__fmaf_rn(__fsub_rn(y, lo), sc, u), 0.5f);
            code[c] = (row_ok && c0 + c < p.k) ? (uint32_t)__float2int_rn(fmaxf(tq, 0.f)) : 0u;
          }
        }
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
          const uint32_t t01 = __byte_perm(code[wd * 4], code[wd * 4 + 1], 0x0040);
          const uint32_t t23 = __byte_perm(code[wd * 4 + 2], code[wd * 4 + 3], 0x0040);
          uint32_t word = (__byte_perm(t01, t23, 0x5410) << sh) & keep;  // uint8 narrowing per byte
#pragma unroll
          for (int m = 1; m < WPT; m <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, m);
          const int c = c0 + wd * 4;
          if ((lane % WPT) == 0 && row_ok && c < p.k) {
            uint8_t* dst = p.packed + g * p.k + c;
            if ((p.k & 3) == 0) {
              *reinterpret_cast<uint32_t*>(dst) = word;
            } else {
#pragma unroll
              for (int bb = 0; bb < 4; bb++)
                if (c + bb < p.k) dst[bb] = (uint8_t)(word >> (8 * bb));
            }
          }
        }
      }
      // this warp is done reading the accumulator buffer
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
    if (p.lib_status) atomicOr(p.lib_status, EXB_STATUS_RP_PACK);
  }
}

// sign(R)^T, zero padded to [kpad, Dpad]; also clears the status word.
__global__ void rp_prepare_kernel(const float* __restrict__ R, int D, int k, int kpad, int Dpad,
                                  float* __restrict__ rt, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *status = 0;
  if (i >= kpad * Dpad) return;
  const int j = i / Dpad, d = i - j * Dpad;
  float v = 0.f;
  if (j < k && d < D) v = R[(long long)d * k + j] > 0.f ? 1.f : -1.f;
  rt[i] = v;
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

int make_tensor_map_2d_f32(CUtensorMap* map, const void* base, unsigned long long inner, unsigned long long outer,
                           unsigned long long pitch_bytes, unsigned box_inner, unsigned box_outer, bool swizzle128) {
  auto enc = get_encode();
  if (enc == nullptr) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EXB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return EXB_OK;
}

static int rp_dims(long long D, long long k, int* kpad, int* Dpad) {
  *kpad = (int)((k + 15) / 16 * 16);
  *Dpad = (int)((D + kRpTileK - 1) / kRpTileK * kRpTileK);
  return 0;
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_rp_workspace_bytes(int64_t D, int64_t k) {
  if (D <= 0 || k <= 0) return 256;
  int kpad, Dpad;
  rp_dims(D, k, &kpad, &Dpad);
  return 256 + (int64_t)kpad * Dpad * 4;
}

int exact_rp_quantize_pack(const float* x, int64_t N, int64_t D, const float* R, int64_t k, int bits,
                           uint64_t seed, uint64_t offset, int64_t row_offset, void* workspace,
                           uint8_t* packed, uint16_t* scale_bf16, uint16_t* min_bf16, float* y_out,
                           void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D > 0 && k > 0, "rp_quantize_pack: bad shape");
  EXB_REQUIRE(row_offset >= 0 && row_offset % 8 == 0, "rp_quantize_pack: row_offset must be a non-negative multiple of 8");
  if (N == 0) return EXB_OK;
  EXB_REQUIRE(x && R && workspace && packed && scale_bf16 && min_bf16, "rp_quantize_pack: null pointer");
  int kpad, Dpad;
  rp_dims(D, k, &kpad, &Dpad);
  if (kpad > 512) return fail(EXB_ERR_UNSUPPORTED, "rp_quantize_pack: k = %lld exceeds the 512 accumulator columns of TMEM", (long long)k);
  EXB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 3) == 0, "rp_quantize_pack: x must be 4-byte aligned");
  // rows that a tensor map cannot describe (pitch or base not a multiple of 16 bytes) are copied by cp.async
  const bool async_a = D % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0;
  EXB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "rp_quantize_pack: workspace must be 256-byte aligned");
  // the epilogue stores 32-bit words of packed bytes when k % 4 == 0
  EXB_REQUIRE(k % 4 != 0 || (reinterpret_cast<uintptr_t>(packed) & 3) == 0, "rp_quantize_pack: packed must be 4-byte aligned when k %% 4 == 0");
  EXB_REQUIRE((N + kRpTileM - 1) / kRpTileM < 2147483647LL / kRpTileM, "rp_quantize_pack: too many rows");
  cudaStream_t st = (cudaStream_t)stream;
  int* status = reinterpret_cast<int*>(workspace);
  float* rt = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);

  rp_prepare_kernel<<<(kpad * Dpad + 255) / 256, 256, 0, st>>>(R, (int)D, (int)k, kpad, Dpad, rt, status);
  EXB_CUDA_OK(cudaGetLastError());

  CUtensorMap tm_x, tm_rt;
  int rc;
  if (!async_a) {
    rc = make_tensor_map_2d_f32(&tm_x, x, (unsigned long long)D, (unsigned long long)N, (unsigned long long)D * 4, kRpTileK, kRpTileM);
    if (rc) return rc;
  } else {
    memset(&tm_x, 0, sizeof(tm_x));   // not read: the cp.async producers take x itself
  }
  rc = make_tensor_map_2d_f32(&tm_rt, rt, (unsigned long long)Dpad, (unsigned long long)kpad, (unsigned long long)Dpad * 4, kRpTileK,
                              (unsigned)(kpad <= 256 ? kpad : kpad / 2));
  if (rc) return rc;

  RpParams p{};
  p.packed = packed; p.scale_bf16 = scale_bf16; p.min_bf16 = min_bf16; p.y_out = y_out; p.status = status; p.lib_status = status_word_ptr();
  p.x = x;
  p.piece = (D % 2 == 0 && (reinterpret_cast<uintptr_t>(x) & 7) == 0) ? 8 : 4;
  p.N = N; p.row_offset = row_offset; p.D = (int)D; p.k = (int)k; p.kpad = kpad; p.bits = bits;
  p.num_tiles = (int)((N + kRpTileM - 1) / kRpTileM);
  p.kblocks = Dpad / kRpTileK;
  p.stage_bytes = (unsigned)(kRpTileM * kRpTileK * 4 + kpad * kRpTileK * 4);
  p.nbuf = 2 * kpad <= 512 ? 2 : 1;
  unsigned cols = 32;
  while (cols < (unsigned)(p.nbuf * kpad)) cols <<= 1;
  p.tmem_cols = cols;
  // Up to four CTAs per SM when they fit (TMEM: 512 columns per SM; shared memory: about 200 KB for the rings):
  // their load / MMA / epilogue phases interleave and hide each other's hand-over gaps.  The cp.async variant
  // runs one CTA of ten warps per SM with a deep ring.
  int ctas_per_sm = 1;
  if (!async_a)
    for (int c = 2; c <= 4; c++)
      if ((unsigned)c * cols <= 512 && (long long)c * 2 * p.stage_bytes + 4096 <= 200 * 1024) ctas_per_sm = c;
  int stages = (int)((200 * 1024 / ctas_per_sm) / p.stage_bytes);
  if (stages > kRpMaxStages) stages = kRpMaxStages;
  if (async_a) {
    if (stages < 3) return fail(EXB_ERR_UNSUPPORTED, "rp_quantize_pack: k = %lld leaves room for fewer than three stages", (long long)k);
    p.lag = stages - 2 < 4 ? stages - 2 : 4;
  } else if (stages < 2) {
    stages = 2;
  }
  p.stages = stages;
  p.inv_sqrt_k = (float)(1.0 / sqrt((double)k));
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.key = make_philox_key(seed);
  const size_t dyn = (size_t)stages * p.stage_bytes + 1024;
  int grid = sm_count() * ctas_per_sm;
  if (grid > p.num_tiles) grid = p.num_tiles;

#define EXB_RP_LAUNCH(BITS_)                                                                                  \
  if (async_a) {                                                                                              \
    EXB_CUDA_OK(cudaFuncSetAttribute(rp_pack_kernel<BITS_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn)); \
    rp_pack_kernel<BITS_, true><<<grid, kRpAsyncThreads, dyn, st>>>(tm_x, tm_rt, p);                          \
  } else {                                                                                                    \
    EXB_CUDA_OK(cudaFuncSetAttribute(rp_pack_kernel<BITS_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn)); \
    rp_pack_kernel<BITS_, false><<<grid, kRpThreads, dyn, st>>>(tm_x, tm_rt, p);                              \
  }
  switch (bits) {
    case 1: EXB_RP_LAUNCH(1) break;
    case 2: EXB_RP_LAUNCH(2) break;
    case 4: EXB_RP_LAUNCH(4) break;
    default: EXB_RP_LAUNCH(8) break;
  }
#undef EXB_RP_LAUNCH
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
