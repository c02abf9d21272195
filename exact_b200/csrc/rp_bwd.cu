// Fused unpack + dequantise + transpose projection:  X_hat = dequantise(packed) @ R^T  in one kernel.
//
// Replaces the backward chain dequantize_activation -> rp2input of exact/exact/ops.py:164-166 (and
// :298-300, :356-358): unpack_single_precision (quantization_cuda_kernel.cu:158-185) writes the [N, k]
// fp32 dequantised projection to HBM, torch.matmul(., rand_matrix.t()) (ops.py:124) reads it back.
// Here the dequantised tile is produced straight into shared memory as the A operand of a tcgen05
// GEMM; only the packed stream is read and only the [N, D] reconstruction is written.
//
// One CTA per SM, persistent over 128-row tiles, 9 warps:
//   warp 0     loads sign(R) (the B operand, [D x k], K-major, 128-byte swizzle) once by TMA and keeps
//              it resident; then issues tcgen05.mma.kind::tf32 (M = 128, N = D padded to 16, K = 8)
//              per tile into one of two TMEM accumulator buffers.
//   warps 1-4  A producers, thread = row: read the row's packed bytes and bf16 statistics, dequantise
//              (code / scale + min, IEEE), store 16-byte chunks into the 128-byte-swizzled K-major
//              layout the MMA expects (chunk index XOR row % 8), fence.proxy.async, signal.
//   warps 5-8  epilogue: tcgen05.ld (thread = row), * 1/sqrt(k), transposed through a warp-private
//              swizzled staging tile so that the fp32 reconstruction leaves in full 128-byte lines.
// Two A buffers and two accumulator buffers overlap producer, MMA and epilogue of consecutive tiles.
// All mbarrier waits are bounded; on expiry the CTA aborts cleanly and leaves a non-zero status word.
//
// Shapes whose sign(R) does not fit beside the A tiles (256 -> 128, every D = 602 shape) take
// rp_unpack_stream_kernel: a work item is (128-row tile, block of up to 256 output columns), and the
// contraction is streamed in panels of 32 projected columns through a ring of stages, each holding the
// dequantised A panel (producer warps) and the matching panel of sign(R) (one TMA box, served by L2).  The
// packed bytes of a tile are dequantised once per column block; that costs a few instructions per value
// and the packed stream is a few per cent of the bytes written.
#include "exact_b200.h"
#include "tc.cuh"

namespace exb {

constexpr int kBwdTileM = 128;
constexpr int kBwdThreads = 288;  // 9 warps

struct RpBwdParams {
  const uint8_t* packed;
  const uint16_t* scale_bf16;
  const uint16_t* min_bf16;
  float* out;
  int* status;
  int* lib_status;    // library-wide status word of this device (capi.cu), or null
  long long N;
  int D, k, Dpad, kpanels, kmma, bits;
  int num_tiles;
  int nbuf;  // TMEM accumulator buffers per CTA: 2, or 1 when two CTAs share the SM's 512 columns at D > 128
  unsigned a_bytes, b_bytes, panel_b_bytes, tmem_cols;
  float inv_sqrt_k;
};

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <int BITS>
__global__ void __launch_bounds__(kBwdThreads, 2)
rp_unpack_kernel(const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ RpBwdParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_bfull;
  __shared__ __align__(8) unsigned long long s_afull[2];
  __shared__ __align__(8) unsigned long long s_aempty[2];
  __shared__ __align__(8) unsigned long long s_tfull[2];
  __shared__ __align__(8) unsigned long long s_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t b_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t a_base = b_base + p.b_bytes;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    mbar_init(smem_u32(&s_bfull), 1);
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&s_afull[b]), 4);   // one arrival per producer warp
      mbar_init(smem_u32(&s_aempty[b]), 1);  // tcgen05.commit
      mbar_init(smem_u32(&s_tfull[b]), 1);   // tcgen05.commit
      mbar_init(smem_u32(&s_tempty[b]), 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int first = blockIdx.x, step = gridDim.x;

  if (warp == 0) {
    // ---------------- B load (once) + MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      const uint32_t bfull = smem_u32(&s_bfull);
      mbar_arrive_expect_tx(bfull, p.b_bytes);
      for (int pn = 0; pn < p.kpanels; pn++) tma_load_2d(b_base + (uint32_t)pn * p.panel_b_bytes, &tm_r, pn * 32, 0, bfull);
      ok = mbar_wait(bfull, 0, abort_flag);
      const uint32_t idesc = umma_idesc_tf32(kBwdTileM, p.Dpad);
      int t = 0;
      for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
        const int buf = t & 1;                              // A buffer
        const uint32_t ph = (uint32_t)(t >> 1) & 1u;
        const int tb = t % p.nbuf;                          // accumulator buffer
        const uint32_t tph = (uint32_t)(t / p.nbuf) & 1u;
        if (!mbar_wait(smem_u32(&s_tempty[tb]), tph ^ 1u, abort_flag)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&s_afull[buf]), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(tb * p.Dpad);
        for (int j = 0; j < p.kmma; j++) {
          const int pn = j >> 2, k4 = j & 3;
          const uint64_t a_desc = umma_desc_sw128(a_base + (uint32_t)buf * p.a_bytes + (uint32_t)pn * (kBwdTileM * 128));
          const uint64_t b_desc = umma_desc_sw128(b_base + (uint32_t)pn * p.panel_b_bytes);
          umma_tf32(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc, j != 0);
        }
        umma_commit(smem_u32(&s_aempty[buf]));
        umma_commit(smem_u32(&s_tfull[tb]));
      }
    }
  } else if (warp <= 4) {
    // ---------------- A producers: unpack + dequantise into swizzled shared memory ----------------
    const int r = (warp - 1) * 32 + lane;  // row within the tile
    const int chunks = p.kpanels * 8;      // 16-byte chunks per row
    const bool vec = (p.k & 3) == 0;
    int t = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
      const int buf = t & 1;
      const uint32_t ph = (uint32_t)(t >> 1) & 1u;
      if (!mbar_wait(smem_u32(&s_aempty[buf]), ph ^ 1u, abort_flag)) { ok = false; break; }
      const long long n = (long long)tile * kBwdTileM + r;
      const bool row_ok = n < p.N;
      float s = 1.f, m = 0.f;
      if (row_ok) {
        s = bf16_bits_to_f32(__ldg(p.scale_bf16 + n));
        m = bf16_bits_to_f32(__ldg(p.min_bf16 + n));
      }
      // code / s as q0 = c*r, rem = fma(-q0, s, c), q = fma(rem, r, q0) with r the correctly rounded
      // reciprocal: equal to the IEEE quotient for codes 0..255 and 2^-100 <= |s| <= 2^100; other scales
      // (inf of a constant row, NaN, denormal) take the division sequence.
      const float rcp = __frcp_rn(s);
      const uint32_t sexp = (__float_as_uint(s) >> 23) & 0xffu;
      const bool tame = __all_sync(0xffffffffu, sexp >= 27u && sexp <= 227u);
      const f32x2 r2 = f2_pack(rcp, rcp), ns2 = f2_pack(-s, -s), m2 = f2_pack(m, m);
      const f32x2 neg_2p23 = f2_pack(-8388608.f, -8388608.f);
      const uint8_t* __restrict__ src = p.packed + (n / WPT) * p.k;
      const int sh = (int)(n % WPT) * BITS;
      const uint32_t row_addr = a_base + (uint32_t)buf * p.a_bytes + (uint32_t)r * 128u;
      for (int c4 = 0; c4 < chunks; c4++) {
        const int c = c4 * 4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (row_ok && c < p.k) {
          uint32_t w;
          if (vec) {
            w = __ldg(reinterpret_cast<const uint32_t*>(src + c));
          } else {
            w = 0;
#pragma unroll
            for (int b = 0; b < 4; b++)
              if (c + b < p.k) w |= (uint32_t)__ldg(src + c + b) << (8 * b);
          }
          if (tame && c + 4 <= p.k) {
            const uint32_t t4 = (w >> sh) & (0x01010101u * MASK);
            float cf[4];
#pragma unroll
            for (int b = 0; b < 4; b++) cf[b] = __uint_as_float(__byte_perm(t4, 0x4b000000u, 0x7540 | b));  // 2^23 + code
#pragma unroll
            for (int b = 0; b < 4; b += 2) {
              const f32x2 c2 = f2_add(f2_pack(cf[b], cf[b + 1]), neg_2p23);
              const f32x2 q0 = f2_mul(c2, r2);
              const f32x2 q = f2_fma(f2_fma(q0, ns2, c2), r2, q0);
              f2_unpack(f2_add(q, m2), v[b], v[b + 1]);
            }
          } else {
#pragma unroll
            for (int b = 0; b < 4; b++) {
              if (c + b < p.k) {
                const uint32_t code = ((w >> (8 * b)) >> sh) & MASK;
                v[b] = __fadd_rn(__fdiv_rn((float)code, s), m);  // quantization_cuda_kernel.cu:182
              }
            }
          }
        }
        const uint32_t pn = (uint32_t)c4 >> 3, ci = (uint32_t)c4 & 7u;
        const uint32_t addr = row_addr + pn * (kBwdTileM * 128) + ((ci ^ ((uint32_t)r & 7u)) << 4);
        asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
                     : "memory");
      }
      fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_afull[buf]));
    }
  } else {
    // ---------------- epilogue: warps 5..8, thread = row ----------------
    const int quad = warp & 3;
    const bool vec = (p.D & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    const uint32_t stage_addr = a_base + 2u * p.a_bytes + (uint32_t)quad * 4096u;  // 32 rows x 128 bytes per warp
    int t = 0;
    bool ok = true;
    for (int tile = first; tile < p.num_tiles && ok; tile += step, t++) {
      const int buf = t % p.nbuf;
      const uint32_t ph = (uint32_t)(t / p.nbuf) & 1u;
      if (!mbar_wait(smem_u32(&s_tfull[buf]), ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * p.Dpad);
      // 32 columns at a time: accumulators -> this warp's private staging tile in shared memory
      // (16-byte chunks XOR-swizzled by row) -> coalesced global stores, 4 rows x 128 bytes per instruction.
      const long long row_base = (long long)tile * kBwdTileM + quad * 32;
      for (int c0 = 0; c0 < p.Dpad; c0 += 32) {
        const int cols = (p.Dpad - c0) < 32 ? (p.Dpad - c0) : 32;   // 16 or 32 (Dpad is a multiple of 16)
        for (int h = 0; h * 16 < cols; h++) {
          float v[16];
          tmem_ld16(taddr + (uint32_t)(c0 + h * 16), v);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t ci = (uint32_t)(h * 4 + j);
            const uint32_t addr = stage_addr + (uint32_t)lane * 128u + ((ci ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(__fmul_rn(v[4 * j], p.inv_sqrt_k)),
                         "f"(__fmul_rn(v[4 * j + 1], p.inv_sqrt_k)), "f"(__fmul_rn(v[4 * j + 2], p.inv_sqrt_k)),
                         "f"(__fmul_rn(v[4 * j + 3], p.inv_sqrt_k))
                         : "memory");
          }
        }
        __syncwarp();
        const uint32_t ci = (uint32_t)lane & 7u;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int rr = 4 * i + (lane >> 3);
          const long long nn = row_base + rr;
          const int c = c0 + (int)ci * 4;
          float4 o;
          const uint32_t addr = stage_addr + (uint32_t)rr * 128u + ((ci ^ ((uint32_t)rr & 7u)) << 4);
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(addr));
          if (nn < p.N && (int)ci * 4 < cols) {
            float* __restrict__ d = p.out + nn * p.D + c;
            if (vec && c + 4 <= p.D) {
              __stcs(reinterpret_cast<float4*>(d), o);
            } else {
              const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
              for (int bb = 0; bb < 4; bb++)
                if (c + bb < p.D) d[bb] = ov[bb];
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
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0 && s_abort) {
    atomicExch(p.status, 1);
    if (p.lib_status) atomicOr(p.lib_status, EXB_STATUS_UNPACK_RP);
  }
}

// ---------------------------------------------------------------------------------------------------
// Streaming variant: neither operand resident.
constexpr int kStreamThreads = 448;  // 14 warps: MMA, 4 A producers, 4 epilogue, B loader, 4 more epilogue
constexpr unsigned kStreamAPanel = kBwdTileM * 128;  // bytes of a [128 x 32] fp32 panel

struct RpBwdStreamParams {
  const uint8_t* packed;
  const uint16_t* scale_bf16;
  const uint16_t* min_bf16;
  float* out;
  int* status;
  int* lib_status;
  long long N;
  int D, k, kpanels, kmma;
  int DB, ndb;          // output columns per block (multiple of 16, <= 256), blocks per tile
  long long num_tiles;
  int stages;
  unsigned stage_bytes;  // A panel + B panel
  unsigned warp_bytes;   // shared memory per producer warp for the packed bytes of its 32 rows
  float inv_sqrt_k;
};

template <int BITS>
__global__ void __launch_bounds__(kStreamThreads, 1)
rp_unpack_stream_kernel(const __grid_constant__ CUtensorMap tm_r, const __grid_constant__ RpBwdStreamParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  constexpr int kMaxStages = 8;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_full[kMaxStages];
  __shared__ __align__(8) unsigned long long s_empty[kMaxStages];
  __shared__ __align__(8) unsigned long long s_tfull[2];
  __shared__ __align__(8) unsigned long long s_tempty[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t stage_area = ring + (uint32_t)p.stages * p.stage_bytes;  // 8 x 4 KB epilogue staging tiles
  const uint32_t bytes_area = stage_area + 8u * 4096u;                    // 4 x warp_bytes of packed bytes
  volatile int* abort_flag = &s_abort;
  const uint32_t b_bytes = (uint32_t)p.DB * 128u;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int i = 0; i < p.stages; i++) {
      mbar_init(smem_u32(&s_full[i]), 5);   // four producer warps + the loader's expect_tx arrival
      mbar_init(smem_u32(&s_empty[i]), 1);  // tcgen05.commit
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&s_tfull[b]), 1);
      mbar_init(smem_u32(&s_tempty[b]), 8);   // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tmem_alloc(smem_u32(&s_tmem_base), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  if (warp == 9) {
    // ---------------- B loader: one [32 x DB] box of sign(R) per stage ----------------
    if (lane == 0) {
      long long g = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        for (int db = 0; db < p.ndb && ok; db++) {
          for (int kp = 0; kp < p.kpanels; kp++, g++) {
            const int st = (int)(g % p.stages);
            const uint32_t ph = (uint32_t)(g / p.stages) & 1u;
            if (!mbar_wait<64>(smem_u32(&s_empty[st]), ph ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t full = smem_u32(&s_full[st]);
            mbar_arrive_expect_tx(full, b_bytes);
            tma_load_2d(ring + (uint32_t)st * p.stage_bytes + kStreamAPanel, &tm_r, kp * 32, db * p.DB, full);
          }
        }
      }
    }
  } else if (warp == 0) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(kBwdTileM, p.DB);
      long long g = 0;
      int t = 0;
      bool ok = true;
      const long long my_tiles = p.num_tiles > blockIdx.x ? (p.num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      for (long long it = 0; it < my_tiles * p.ndb && ok; it++, t++) {
        const int tb = t & 1;
        const uint32_t tph = (uint32_t)(t >> 1) & 1u;
        if (!mbar_wait(smem_u32(&s_tempty[tb]), tph ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t d_tmem = tmem_base + (uint32_t)(tb * 256);
        for (int kp = 0; kp < p.kpanels; kp++, g++) {
          const int st = (int)(g % p.stages);
          const uint32_t ph = (uint32_t)(g / p.stages) & 1u;
          if (!mbar_wait(smem_u32(&s_full[st]), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = ring + (uint32_t)st * p.stage_bytes;
          const uint64_t a_desc = umma_desc_sw128(a_addr), b_desc = umma_desc_sw128(a_addr + kStreamAPanel);
          for (int k4 = 0; k4 < 4 && kp * 4 + k4 < p.kmma; k4++)
            umma_tf32(d_tmem, a_desc + (uint64_t)(k4 * 2), b_desc + (uint64_t)(k4 * 2), idesc, (kp | k4) != 0);
          umma_commit(smem_u32(&s_empty[st]));
        }
        if (ok) umma_commit(smem_u32(&s_tfull[tb]));
      }
    }
  } else if (warp <= 4) {
    // ---------------- A producers: thread = row, one panel of 32 projected columns per stage ----------------
    // The packed bytes of a warp's 32 rows (32 / WPT row groups, contiguous in the stream) are brought into
    // shared memory once per tile with coalesced 16-byte loads and read from there for every column block and
    // panel: no global-memory latency between the panels.
    const int r = (warp - 1) * 32 + lane;
    const uint32_t wbuf = bytes_area + (uint32_t)(warp - 1) * p.warp_bytes;
    long long g = 0;
    bool ok = true;
    for (long long tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
      const long long n = tile * kBwdTileM + r;
      const bool row_ok = n < p.N;
      float s = 1.f, m = 0.f;
      if (row_ok) {
        s = bf16_bits_to_f32(__ldg(p.scale_bf16 + n));
        m = bf16_bits_to_f32(__ldg(p.min_bf16 + n));
      }
      // this warp's bytes: row groups [grp0, grp1) of the stream
      const long long n_w = tile * kBwdTileM + (warp - 1) * 32;
      const long long rows_w = p.N - n_w < 32 ? p.N - n_w : 32;
      uint32_t head = 0;
      __syncwarp();   // the previous tile's reads of the buffer are done
      if (rows_w > 0) {
        const long long grp0 = n_w / WPT, grp1 = (n_w + rows_w + WPT - 1) / WPT;
        const uint8_t* first = p.packed + grp0 * p.k;
        const uint8_t* last = p.packed + grp1 * p.k;
        head = (uint32_t)(reinterpret_cast<uintptr_t>(first) & 15u);
        const uint8_t* base16 = first - head;
        const long long words = (last - base16 + 15) / 16;
        for (long long i = lane; i < words; i += 32) {
          const uint8_t* src = base16 + i * 16;
          uint4 v = make_uint4(0u, 0u, 0u, 0u);
          if (src >= first && src + 16 <= last) {
            v = __ldg(reinterpret_cast<const uint4*>(src));
          } else {
            uint32_t q[4] = {0u, 0u, 0u, 0u};
            for (int b = 0; b < 16; b++)
              if (src + b >= first && src + b < last) q[b >> 2] |= (uint32_t)__ldg(src + b) << (8 * (b & 3));
            v = make_uint4(q[0], q[1], q[2], q[3]);
          }
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(wbuf + (uint32_t)i * 16u), "r"(v.x), "r"(v.y),
                       "r"(v.z), "r"(v.w)
                       : "memory");
        }
      }
      __syncwarp();
      // code / s by the correctly rounded reciprocal sequence (see rp_unpack_kernel); other scales divide
      const float rcp = __frcp_rn(s);
      const uint32_t sexp = (__float_as_uint(s) >> 23) & 0xffu;
      const bool tame = __all_sync(0xffffffffu, sexp >= 27u && sexp <= 227u);
      const f32x2 r2 = f2_pack(rcp, rcp), ns2 = f2_pack(-s, -s), m2 = f2_pack(m, m);
      const f32x2 neg_2p23 = f2_pack(-8388608.f, -8388608.f);
      const uint32_t row_bytes = wbuf + head + (uint32_t)(lane / WPT) * (uint32_t)p.k;   // this row's group
      const int sh = (lane % WPT) * BITS;   // n % WPT: tiles and warps start at multiples of 32 rows
      for (int db = 0; db < p.ndb && ok; db++) {
        for (int kp = 0; kp < p.kpanels; kp++, g++) {
          const int st = (int)(g % p.stages);
          const uint32_t ph = (uint32_t)(g / p.stages) & 1u;
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_empty[st]), ph ^ 1u, abort_flag))) { ok = false; break; }
          const uint32_t row_addr = ring + (uint32_t)st * p.stage_bytes + (uint32_t)r * 128u;
#pragma unroll
          for (int ci = 0; ci < 8; ci++) {
            const int c = kp * 32 + ci * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (row_ok && c < p.k) {
              // four bytes at any alignment: two aligned words and a funnel shift (the buffer is padded)
              const uint32_t a = row_bytes + (uint32_t)c;
              uint32_t lo, hi;
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(lo) : "r"(a & ~3u));
              asm volatile("ld.shared.b32 %0, [%1];" : "=r"(hi) : "r"((a & ~3u) + 4u));
              const uint32_t w = __funnelshift_r(lo, hi, 8u * (a & 3u));
              if (tame && c + 4 <= p.k) {
                const uint32_t t4 = (w >> sh) & (0x01010101u * MASK);
                float cf[4];
#pragma unroll
                for (int b = 0; b < 4; b++) cf[b] = __uint_as_float(__byte_perm(t4, 0x4b000000u, 0x7540 | b));  // 2^23 + code
#pragma unroll
                for (int b = 0; b < 4; b += 2) {
                  const f32x2 c2 = f2_add(f2_pack(cf[b], cf[b + 1]), neg_2p23);
                  const f32x2 q0 = f2_mul(c2, r2);
                  const f32x2 q = f2_fma(f2_fma(q0, ns2, c2), r2, q0);
                  f2_unpack(f2_add(q, m2), v[b], v[b + 1]);
                }
              } else {
#pragma unroll
                for (int b = 0; b < 4; b++) {
                  if (c + b < p.k) {
                    const uint32_t code = ((w >> (8 * b)) >> sh) & MASK;
                    v[b] = __fadd_rn(__fdiv_rn((float)code, s), m);  // quantization_cuda_kernel.cu:182
                  }
                }
              }
            }
            const uint32_t addr = row_addr + (((uint32_t)ci ^ ((uint32_t)r & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&s_full[st]));
        }
      }
    }
  } else {
    // ---------------- epilogue: warps 5..8 and 10..13, thread = row; the two warps of a TMEM lane quadrant
    // take alternate chunks of 32 columns ----------------
    const int quad = warp & 3, half = warp >= 10 ? 1 : 0;
    const bool vec4 = (p.D & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
    const bool vec2 = (p.D & 1) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0;
    const uint32_t stage_addr = stage_area + (uint32_t)(quad + 4 * half) * 4096u;
    int t = 0;
    bool ok = true;
    const long long my_tiles = p.num_tiles > blockIdx.x ? (p.num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    for (long long it = 0; it < my_tiles * p.ndb && ok; it++, t++) {
      const long long tile = blockIdx.x + (it / p.ndb) * gridDim.x;
      const int col_base = (int)(it % p.ndb) * p.DB;
      const int buf = t & 1;
      const uint32_t ph = (uint32_t)(t >> 1) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_tfull[buf]), ph, abort_flag))) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * 256);
      const long long row_base = tile * kBwdTileM + quad * 32;
      for (int c0 = half * 32; c0 < p.DB && col_base + c0 < p.D; c0 += 64) {
        const int cols = (p.DB - c0) < 32 ? (p.DB - c0) : 32;   // 16 or 32
        for (int h = 0; h * 16 < cols; h++) {
          float v[16];
          tmem_ld16(taddr + (uint32_t)(c0 + h * 16), v);
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const uint32_t ci = (uint32_t)(h * 4 + j);
            const uint32_t addr = stage_addr + (uint32_t)lane * 128u + ((ci ^ ((uint32_t)lane & 7u)) << 4);
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(__fmul_rn(v[4 * j], p.inv_sqrt_k)),
                         "f"(__fmul_rn(v[4 * j + 1], p.inv_sqrt_k)), "f"(__fmul_rn(v[4 * j + 2], p.inv_sqrt_k)),
                         "f"(__fmul_rn(v[4 * j + 3], p.inv_sqrt_k))
                         : "memory");
          }
        }
        __syncwarp();
        const uint32_t ci = (uint32_t)lane & 7u;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int rr = 4 * i + (lane >> 3);
          const long long nn = row_base + rr;
          const int c = col_base + c0 + (int)ci * 4;
          float4 o;
          const uint32_t addr = stage_addr + (uint32_t)rr * 128u + ((ci ^ ((uint32_t)rr & 7u)) << 4);
          asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(o.x), "=f"(o.y), "=f"(o.z), "=f"(o.w) : "r"(addr));
          if (nn < p.N && (int)ci * 4 < cols && c < p.D) {
            float* __restrict__ d = p.out + nn * p.D + c;
            if (vec4 && c + 4 <= p.D) {
              __stcs(reinterpret_cast<float4*>(d), o);
            } else if (vec2 && c + 4 <= p.D) {
              __stcs(reinterpret_cast<float2*>(d), make_float2(o.x, o.y));
              __stcs(reinterpret_cast<float2*>(d) + 1, make_float2(o.z, o.w));
            } else {
              const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
              for (int bb = 0; bb < 4; bb++)
                if (c + bb < p.D) d[bb] = ov[bb];
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
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && s_abort) {
    atomicExch(p.status, 1);
    if (p.lib_status) atomicOr(p.lib_status, EXB_STATUS_UNPACK_RP);
  }
}

// sign(R), zero padded to [Dpad, kpad32]; also clears the status word.
__global__ void rp_bwd_prepare_kernel(const float* __restrict__ R, int D, int k, int Dpad, int kpad32,
                                      float* __restrict__ rs, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) *status = 0;
  if (i >= Dpad * kpad32) return;
  const int d = i / kpad32, j = i - d * kpad32;
  float v = 0.f;
  if (d < D && j < k) v = R[(long long)d * k + j] > 0.f ? 1.f : -1.f;
  rs[i] = v;
}

static void bwd_dims(long long D, long long k, int* Dpad, int* kpad32) {
  *Dpad = (int)((D + 15) / 16 * 16);
  *kpad32 = (int)((k + 31) / 32 * 32);
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_unpack_rp_workspace_bytes(int64_t D, int64_t k) {
  if (D <= 0 || k <= 0) return 256;
  int Dpad, kpad32;
  bwd_dims(D, k, &Dpad, &kpad32);
  return 256 + (int64_t)Dpad * kpad32 * 4;
}

int exact_unpack_dequant_rp(const uint8_t* packed, int bits, const uint16_t* scale_bf16, const uint16_t* min_bf16,
                            int64_t N, int64_t k, const float* R, int64_t D, void* workspace, float* out,
                            void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D > 0 && k > 0, "unpack_dequant_rp: bad shape");
  if (N == 0) return EXB_OK;
  EXB_REQUIRE(packed && scale_bf16 && min_bf16 && R && workspace && out, "unpack_dequant_rp: null pointer");
  EXB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "unpack_dequant_rp: workspace must be 256-byte aligned");
  int Dpad, kpad32;
  bwd_dims(D, k, &Dpad, &kpad32);
  const int kpanels = kpad32 / 32;
  const long long a_bytes = (long long)kBwdTileM * kpanels * 128;
  const long long b_bytes = (long long)Dpad * kpanels * 128;
  const bool resident = Dpad <= 256 && b_bytes + 2 * a_bytes + 4 * 4096 + 2048 <= 200 * 1024;
  EXB_REQUIRE((long long)Dpad * kpad32 < (1LL << 28), "unpack_dequant_rp: D x k out of range");
  EXB_REQUIRE((N + kBwdTileM - 1) / kBwdTileM < 2147483647LL / kBwdTileM, "unpack_dequant_rp: too many rows");
  if ((k & 3) == 0) EXB_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 3) == 0, "unpack_dequant_rp: packed must be 4-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  int* status = reinterpret_cast<int*>(workspace);
  float* rs = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
  rp_bwd_prepare_kernel<<<(unsigned)(((long long)Dpad * kpad32 + 255) / 256), 256, 0, st>>>(R, (int)D, (int)k, Dpad, kpad32, rs,
                                                                                         status);
  EXB_CUDA_OK(cudaGetLastError());

  if (!resident) {
    // column blocks of equal width (a multiple of 16, at most 256); rows of sign(R) past Dpad read as zeros
    RpBwdStreamParams q{};
    q.ndb = (Dpad + 255) / 256;
    q.DB = ((Dpad + q.ndb - 1) / q.ndb + 15) / 16 * 16;
    CUtensorMap tm_rs;
    int rcs = make_tensor_map_2d_f32(&tm_rs, rs, (unsigned long long)kpad32, (unsigned long long)Dpad,
                                     (unsigned long long)kpad32 * 4, 32, (unsigned)q.DB);
    if (rcs) return rcs;
    q.packed = packed; q.scale_bf16 = scale_bf16; q.min_bf16 = min_bf16; q.out = out; q.status = status;
    q.lib_status = status_word_ptr();
    q.N = N; q.D = (int)D; q.k = (int)k; q.kpanels = kpanels; q.kmma = (int)((k + 7) / 8);
    q.num_tiles = (N + kBwdTileM - 1) / kBwdTileM;
    q.stage_bytes = kStreamAPanel + (unsigned)q.DB * 128u;
    // packed bytes of 32 rows (32 / wpt row groups of k bytes), 16 bytes of alignment slack at either end
    q.warp_bytes = (unsigned)(((32 / (8 / bits)) * k + 15 + 16 + 15) / 16 * 16);
    const long long ring_budget = 226ll * 1024 - 8 * 4096 - 1024 - 4ll * q.warp_bytes;
    if (ring_budget < 2ll * q.stage_bytes)
      return fail(EXB_ERR_UNSUPPORTED, "unpack_dequant_rp: k = %lld too large for the shared-memory ring", (long long)k);
    q.stages = (int)(ring_budget / q.stage_bytes);
    if (q.stages > 8) q.stages = 8;
    q.inv_sqrt_k = (float)(1.0 / sqrt((double)k));
    const size_t dyn_s = (size_t)q.stages * q.stage_bytes + 8 * 4096 + 4 * (size_t)q.warp_bytes + 1024;
    long long grid_s = sm_count();
    if (grid_s > q.num_tiles) grid_s = q.num_tiles;
#define EXB_BWD_STREAM(BITS_)                                                                                          \
  {                                                                                                                    \
    EXB_CUDA_OK(cudaFuncSetAttribute(rp_unpack_stream_kernel<BITS_>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                     (int)dyn_s));                                                                     \
    rp_unpack_stream_kernel<BITS_><<<(unsigned)grid_s, kStreamThreads, dyn_s, st>>>(tm_rs, q);                         \
  }
    switch (bits) {
      case 1: EXB_BWD_STREAM(1) break;
      case 2: EXB_BWD_STREAM(2) break;
      case 4: EXB_BWD_STREAM(4) break;
      default: EXB_BWD_STREAM(8) break;
    }
#undef EXB_BWD_STREAM
    EXB_CUDA_OK(cudaGetLastError());
    return EXB_OK;
  }

  CUtensorMap tm_r;
  int rc = make_tensor_map_2d_f32(&tm_r, rs, (unsigned long long)kpad32, (unsigned long long)Dpad,
                                  (unsigned long long)kpad32 * 4, 32, (unsigned)Dpad);
  if (rc) return rc;

  RpBwdParams p{};
  p.packed = packed; p.scale_bf16 = scale_bf16; p.min_bf16 = min_bf16; p.out = out; p.status = status; p.lib_status = status_word_ptr();
  p.N = N; p.D = (int)D; p.k = (int)k; p.Dpad = Dpad; p.kpanels = kpanels; p.kmma = (int)((k + 7) / 8); p.bits = bits;
  p.num_tiles = (int)((N + kBwdTileM - 1) / kBwdTileM);
  p.a_bytes = (unsigned)a_bytes; p.b_bytes = (unsigned)b_bytes; p.panel_b_bytes = (unsigned)(Dpad * 128);
  const size_t dyn = (size_t)(b_bytes + 2 * a_bytes) + 4 * 4096 + 1024;  // + epilogue staging tiles
  // CTAs per SM: bounded by shared memory (about 200 KB) and by the 512 TMEM columns of the SM.
  int ctas = (int)((200 * 1024) / (dyn + 1024));
  if (ctas > 4) ctas = 4;
  if (ctas < 1) ctas = 1;
  p.nbuf = 2;
  unsigned cols = 32;
  while (cols < (unsigned)(2 * Dpad)) cols <<= 1;
  if (ctas >= 2 && cols * 2 > 512) {  // D > 128: one accumulator buffer per CTA, two CTAs overlap each other
    p.nbuf = 1;
    cols = 32;
    while (cols < (unsigned)Dpad) cols <<= 1;
  }
  while (ctas > 1 && (unsigned)ctas * cols > 512) ctas--;
  p.tmem_cols = cols;
  p.inv_sqrt_k = (float)(1.0 / sqrt((double)k));
  int grid = sm_count() * ctas;
  if (grid > p.num_tiles) grid = p.num_tiles;

#define EXB_BWD_LAUNCH(BITS_)                                                                                   \
  {                                                                                                             \
    EXB_CUDA_OK(cudaFuncSetAttribute(rp_unpack_kernel<BITS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn)); \
    rp_unpack_kernel<BITS_><<<grid, kBwdThreads, dyn, st>>>(tm_r, p);                                           \
  }
  switch (bits) {
    case 1: EXB_BWD_LAUNCH(1) break;
    case 2: EXB_BWD_LAUNCH(2) break;
    case 4: EXB_BWD_LAUNCH(4) break;
    default: EXB_BWD_LAUNCH(8) break;
  }
#undef EXB_BWD_LAUNCH
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
