// Per-row stochastic quantise + bit-pack of saved activations, and unpack + dequantise.
//
// Replaces, behind a C ABI:
//   pack_single_precision    exact/exact/cpp_extension/quantization.cc:37-48,
//                            quantization_cuda_kernel.cu:63-155
//   unpack_single_precision  quantization.cc:50-62, quantization_cuda_kernel.cu:158-229
//   the torch glue around them in exact/exact/ops.py:20-98 (row min/max, scale, bf16 statistics),
//   which the fused entry point folds into the same pass over the activation.
//
// Work decomposition.  The packed stream stores, for column d, the codes of `8/bits` consecutive rows
// in one byte at (n / (8/bits)) * D + d.  An 8-row tile therefore covers whole bytes for every bit
// width.  `tpt` threads own one tile; each thread keeps 8 rows x V chunks x VEC columns in registers,
// so bytes are assembled thread-locally and stored VEC at a time, and the activation is read from
// HBM exactly once.  Row min/max go through redux.sync (sub-warp groups when tpt < 32) and, when a
// tile spans several warps, a double-buffered shared-memory exchange with named barriers.  While a
// tile is processed, the next one (a contiguous run of 8*D elements) is pulled into L2 with one
// cp.async.bulk.prefetch.  The arithmetic uses the paired fp32 instructions of sm_100 (two elements per issue slot,
// each rounded exactly like the scalar instruction).
#include "common.cuh"
#include "exact_b200.h"

namespace exb {

struct PackParams {
  const void* x;          // [N, D] fp32 or bf16 bits
  const float* noise;     // [N, D] supplied U[0,1) noise, or null -> Philox
  const float* mn_in;     // [N] caller-computed row min (reference-signature entry only)
  const float* scale_in;  // [N] caller-computed row scale (reference-signature entry only)
  uint8_t* packed;        // [ceil(N/(8/bits)) * D]
  uint16_t* scale_bf16;   // [N] or null
  uint16_t* min_bf16;     // [N] or null
  float* scale_f32;       // [N] or null
  float* min_f32;         // [N] or null
  long long N, D;
  long long row_offset;   // global index of row 0 (multiple of 8): keys the noise for row-sharded runs
  int tpt;                // threads per 8-row tile
  uint32_t off_lo, off_hi;
  PhiloxKey key;
};

constexpr int kMaxWarpsPerTile = 8;
constexpr int kMaxGroupsPerCta = 2;  // tiles of more than one warp: at most two per CTA

// Barrier over the threads of one multi-warp tile group; ids are literals.
__device__ __forceinline__ void group_barrier(int grp, int nthreads) {
  if (grp == 0) named_barrier<1>(nthreads);
  else named_barrier<2>(nthreads);
}

// Per-thread view of the tiling, fixed for the whole kernel.
struct TileCtx {
  long long N, D, G;
  int tpt, grp, tl, lane, lane_base;
  unsigned gmask;
  bool multi;
};

// FULL: all 8 rows of the tile exist; one 64-bit base per chunk, rows addressed by 32-bit offsets.
template <typename InT, int VEC, int V, bool FULL>
__device__ __forceinline__ void load_tile(const InT* __restrict__ x, const TileCtx& c, long long tile,
                                          const long long (&col)[V], const bool (&cvalid)[V],
                                          float (&xv)[8][V][VEC]) {
  const long long row0 = tile << 3;
  const int rows_valid = FULL ? 8 : ((c.N - row0 >= 8) ? 8 : (int)(c.N - row0));
  const unsigned Du = (unsigned)c.D;
#pragma unroll
  for (int v = 0; v < V; v++) {
    const InT* __restrict__ base = x + row0 * c.D + col[v];
#pragma unroll
    for (int r = 0; r < 8; r++) {
      if ((FULL || r < rows_valid) && cvalid[v]) {
        Ld<InT, VEC>::load(base + r * Du, xv[r][v]);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; e++) xv[r][v][e] = 0.f;
      }
    }
  }
}

// Four (two, one) 8-bit codes -> one word with a code per byte.
template <int VEC>
__device__ __forceinline__ uint32_t bytes_of(const uint32_t (&code)[VEC]) {
  if (VEC == 4) {
    const uint32_t t01 = __byte_perm(code[0], code[1 % VEC], 0x0040);
    const uint32_t t23 = __byte_perm(code[2 % VEC], code[3 % VEC], 0x0040);
    return __byte_perm(t01, t23, 0x5410);
  } else if (VEC == 2) {
    return __byte_perm(code[0], code[1 % VEC], 0x0040);  // bytes 2, 3 are never stored
  }
  return code[0];
}
template <int VEC>
__device__ __forceinline__ void store_bytes(uint8_t* p, uint32_t w) {
  if (VEC == 4) __stcs(reinterpret_cast<uint32_t*>(p), w);
  else if (VEC == 2) __stcs(reinterpret_cast<uint16_t*>(p), (uint16_t)w);
  else __stcs(p, (uint8_t)w);
}
template <int VEC>
__device__ __forceinline__ uint32_t load_bytes(const uint8_t* p) {
  if (VEC == 4) return __ldcs(reinterpret_cast<const uint32_t*>(p));
  if (VEC == 2) return __ldcs(reinterpret_cast<const uint16_t*>(p));
  return __ldcs(p);
}

// Quantise the 8 x (V*VEC) register tile with stochastic rounding and assemble the packed bytes.
// MAGIC (only with FAST, and only when every scale of the tile is a finite non-zero number): the
// rounding is done by adding 1.5 * 2^23, the code being the low byte of the sum.
template <typename InT, int BITS, int VEC, int V, bool FAST, bool MAGIC>
__device__ __forceinline__ void quantize_rows(const PackParams& p, const TileCtx& c, long long tile, int rows_valid,
                                              const long long (&col)[V], const bool (&cvalid)[V],
                                              float (&xv)[8][V][VEC], const float (&mn)[8], const float (&sc)[8]) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  const long long row0 = tile << 3;
  // quantization_cuda_kernel.cu:89: t = fma(x - mn, s, u) - 0.5 (nvcc contracts the mul+add),
  // code = rint(max(t, 0)), no upper clamp.  With true row statistics and noise in [0, 1],
  // -0.5 <= t < 2^bits + 2, so the saturating float->unsigned conversion (NaN -> 0) equals
  // max-then-convert, and so does the low byte of t + 1.5 * 2^23 whenever the scale is finite.
  const long long noise_tile = (row0 + p.row_offset) >> 3;
  const f32x2 neg_half = f2_pack(-0.5f, -0.5f);
  const f32x2 magic = f2_pack(12582912.f, 12582912.f);
  const unsigned Du = (unsigned)c.D;
#pragma unroll
  for (int v = 0; v < V; v++) {
    if (!cvalid[v]) continue;
    uint32_t acc[GPT];
#pragma unroll
    for (int g = 0; g < GPT; g++) acc[g] = 0u;

    // One Philox block per 8-row tile and PAIR of columns: its 16 bytes are the noise of rows 0..7 of the
    // even and the odd column (byte 2 r + (column & 1)), 8 bits per element: u = (h + 0.5) / 256.
    constexpr int NP = (VEC + 1) / 2;
    uint32_t w[NP][4];
    const uint32_t odd = (VEC == 1) ? (uint32_t)(col[v] & 1) : 0u;
    if (FAST || p.noise == nullptr) {
      const unsigned long long q0 = (unsigned long long)(noise_tile * ((c.D + 1) >> 1) + (col[v] >> 1));
#pragma unroll
      for (int e = 0; e < NP; e++) {
        const unsigned long long q = q0 + e;
        philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w[e]);
      }
    }
    const float* __restrict__ nbase = FAST ? nullptr : (p.noise ? p.noise + row0 * c.D + col[v] : nullptr);

#pragma unroll
    for (int r = 0; r < 8; r++) {
      if (FAST || r < rows_valid) {
        float un[VEC];
        if (!FAST && nbase != nullptr) Ld<float, VEC>::load(nbase + r * Du, un);
        uint32_t code[VEC];
        if (VEC >= 2) {
          const f32x2 mn2 = f2_pack(mn[r], mn[r]);
          const f32x2 sc2 = f2_pack(sc[r], sc[r]);
#pragma unroll
          for (int e = 0; e < VEC; e += 2) {
            f32x2 u2;
            if (!FAST && nbase != nullptr) {
              u2 = f2_pack(un[e], un[(e + 1) % VEC]);
            } else {
              // columns e (even) and e + 1 of this thread share the block w[e / 2]
              const float f0 = u8_to_1p(w[e >> 1][r >> 1], (r & 1) * 2);
              const float f1 = u8_to_1p(w[e >> 1][r >> 1], (r & 1) * 2 + 1);
              u2 = noise8_to_unit(f2_pack(f0, f1));
            }
            const f32x2 a2 = f2_sub(f2_pack(xv[r][v][e], xv[r][v][(e + 1) % VEC]), mn2);
            f32x2 t2 = f2_add(f2_fma(a2, sc2, u2), neg_half);
            float t0, t1;
            if (MAGIC) {
              t2 = f2_add(t2, magic);
              f2_unpack(t2, t0, t1);
              code[e] = __float_as_uint(t0);            // low byte = rint(t); higher bytes are dropped below
              code[(e + 1) % VEC] = __float_as_uint(t1);
            } else {
              f2_unpack(t2, t0, t1);
              code[e] = __float2uint_rn(t0);
              code[(e + 1) % VEC] = __float2uint_rn(t1);
            }
          }
        } else {
          const float u = (!FAST && nbase != nullptr) ? un[0]
                          : noise8_to_unit(u8_to_1p(w[0][r >> 1], (r & 1) * 2 + odd));
          const float t = __fsub_rn(__fmaf_rn(__fsub_rn(xv[r][v][0], mn[r]), sc[r], u), 0.5f);
          code[0] = __float2uint_rn(t) & 0xffu;
        }
        const uint32_t word = bytes_of<VEC>(code);
        constexpr uint32_t kOnes = 0x01010101u;
        const int sh = (r % WPT) * BITS;
        if (sh == 0) acc[r / WPT] = word;
        else acc[r / WPT] |= (word << sh) & (kOnes * ((0xffu << sh) & 0xffu));  // uint8 narrowing per byte
      }
    }

    uint8_t* __restrict__ obase = p.packed + (tile * GPT) * c.D + col[v];
#pragma unroll
    for (int g = 0; g < GPT; g++) {
      if (FAST || tile * GPT + g < c.G) store_bytes<VEC>(obase + g * Du, acc[g]);
    }
  }
}

// FAST: the tile has all 8 rows and the noise is drawn from Philox.  Then there is no per-row
// validity test, and -- when all 8 scales are finite and non-zero, i.e. no row is constant or holds
// an infinity or a NaN -- round-to-nearest-even is done by adding 1.5 * 2^23 (the code is then the
// low byte of the float) instead of a float->int conversion.
template <typename InT, int BITS, int VEC, int V, bool FAST>
__device__ __forceinline__ bool process_tile(const PackParams& p, const TileCtx& c, long long tile, int it,
                                             const long long (&col)[V], const bool (&cvalid)[V],
                                             float (&xv)[8][V][VEC], float* s_part, float* s_fin) {
  const long long row0 = tile << 3;
  const int rows_valid = FAST ? 8 : ((c.N - row0 >= 8) ? 8 : (int)(c.N - row0));
  const float B = (float)((1 << BITS) - 1);

  // ---- row statistics ----------------------------------------------------------------------------
  float lo[8], hi[8], mn[8], sc[8];
#pragma unroll
  for (int r = 0; r < 8; r++) {
    lo[r] = __int_as_float(0x7f800000);
    hi[r] = __int_as_float(0xff800000);
#pragma unroll
    for (int v = 0; v < V; v++) {
      if (cvalid[v]) {
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          lo[r] = min_nan(lo[r], xv[r][v][e]);
          hi[r] = max_nan(hi[r], xv[r][v][e]);
        }
      }
    }
    lo[r] = redux_min_nan(lo[r], c.gmask);
    hi[r] = redux_max_nan(hi[r], c.gmask);
  }
  bool finite = true;  // all 8 scales are finite numbers (warp-uniform)
  if (!c.multi) {
    // lane (tl & 7) turns row (tl & 7)'s range into a scale, then the group shares the 8 scales.
    const int my = c.tl & 7;
    float lo_my = lo[0], hi_my = hi[0];
#pragma unroll
    for (int r = 1; r < 8; r++) {
      lo_my = (my == r) ? lo[r] : lo_my;
      hi_my = (my == r) ? hi[r] : hi_my;
    }
    // ops.py:39 evaluates (2^b - 1) / (mx - mn) as reciprocal(mx - mn) * (2^b - 1).
    const float s_my = __fmul_rn(__frcp_rn(__fsub_rn(hi_my, lo_my)), B);
    // 0 < s < inf  <=>  the row's range is a finite non-zero number, hence every x in it is finite
    if (FAST) finite = __all_sync(c.gmask, s_my > 0.f && s_my < __int_as_float(0x7f800000));
#pragma unroll
    for (int r = 0; r < 8; r++) {
      sc[r] = __shfl_sync(c.gmask, s_my, c.lane_base + r);
      mn[r] = lo[r];
    }
    if (c.tl < rows_valid) {  // tl < 8 here because rows_valid <= 8
      const long long row = row0 + c.tl;
      if (p.scale_bf16) p.scale_bf16[row] = f32_to_bf16_bits(s_my);
      if (p.min_bf16) p.min_bf16[row] = f32_to_bf16_bits(lo_my);
      if (p.scale_f32) p.scale_f32[row] = s_my;
      if (p.min_f32) p.min_f32[row] = lo_my;
    }
  } else {
    float* part = s_part + ((it & 1) * kMaxGroupsPerCta + c.grp) * (kMaxWarpsPerTile * 16);
    float* fin = s_fin + ((it & 1) * kMaxGroupsPerCta + c.grp) * 16;
    const int wt = c.tl >> 5;  // warp within the tile
    const int nwt = c.tpt >> 5;
    if (c.lane == 0) {
#pragma unroll
      for (int r = 0; r < 8; r++) {
        part[wt * 16 + r] = lo[r];
        part[wt * 16 + 8 + r] = hi[r];
      }
    }
    group_barrier(c.grp, c.tpt);
    if (c.tl < 8) {
      float lo_f = part[c.tl], hi_f = part[8 + c.tl];
      for (int w = 1; w < nwt; w++) {
        lo_f = min_nan(lo_f, part[w * 16 + c.tl]);
        hi_f = max_nan(hi_f, part[w * 16 + 8 + c.tl]);
      }
      const float s_f = __fmul_rn(__frcp_rn(__fsub_rn(hi_f, lo_f)), B);
      fin[c.tl] = lo_f;
      fin[8 + c.tl] = s_f;
      if (c.tl < rows_valid) {
        const long long row = row0 + c.tl;
        if (p.scale_bf16) p.scale_bf16[row] = f32_to_bf16_bits(s_f);
        if (p.min_bf16) p.min_bf16[row] = f32_to_bf16_bits(lo_f);
        if (p.scale_f32) p.scale_f32[row] = s_f;
        if (p.min_f32) p.min_f32[row] = lo_f;
      }
    }
    group_barrier(c.grp, c.tpt);
    const float4* f = reinterpret_cast<const float4*>(fin);
    const float4 a = f[0], b = f[1], cc = f[2], d = f[3];
    mn[0] = a.x; mn[1] = a.y; mn[2] = a.z; mn[3] = a.w;
    mn[4] = b.x; mn[5] = b.y; mn[6] = b.z; mn[7] = b.w;
    sc[0] = cc.x; sc[1] = cc.y; sc[2] = cc.z; sc[3] = cc.w;
    sc[4] = d.x; sc[5] = d.y; sc[6] = d.z; sc[7] = d.w;
    if (FAST) {
      float mx_s = sc[0], mn_s = sc[0];
#pragma unroll
      for (int r = 1; r < 8; r++) {
        mx_s = max_nan(mx_s, sc[r]);
        mn_s = min_nan(mn_s, sc[r]);
      }
      finite = mn_s > 0.f && mx_s < __int_as_float(0x7f800000);
    }
  }

  // ---- quantise with stochastic rounding and assemble bytes ---------------------------------------
  // `finite` is uniform over the threads of the tile; tiles with a constant / inf / NaN row take the
  // general path, which is also the one of ragged and supplied-noise tiles.
  // `finite` is uniform over the threads of the tile.  A full Philox tile with a constant / inf / NaN
  // row is handed back to the caller, which redoes it on the general path.
  if (FAST) {
    if (!finite) return false;
    quantize_rows<InT, BITS, VEC, V, true, true>(p, c, tile, 8, col, cvalid, xv, mn, sc);
  } else {
    quantize_rows<InT, BITS, VEC, V, false, false>(p, c, tile, rows_valid, col, cvalid, xv, mn, sc);
  }
  return true;
}

template <typename InT, int BITS, int VEC, int V>
__global__ void __launch_bounds__(256)
quantize_pack_kernel(const __grid_constant__ PackParams p) {
  constexpr int WPT = 8 / BITS;
  __shared__ float s_part[2 * kMaxGroupsPerCta * kMaxWarpsPerTile * 16];
  __shared__ __align__(16) float s_fin[2 * kMaxGroupsPerCta * 16];

  TileCtx c;
  c.N = p.N; c.D = p.D;
  c.G = (p.N + WPT - 1) / WPT;
  c.tpt = p.tpt;
  c.grp = threadIdx.x / c.tpt;
  c.tl = threadIdx.x - c.grp * c.tpt;
  c.lane = threadIdx.x & 31;
  c.lane_base = (c.tpt < 32) ? (c.lane / c.tpt) * c.tpt : 0;
  c.gmask = (c.tpt < 32) ? (((1u << c.tpt) - 1u) << c.lane_base) : 0xffffffffu;
  c.multi = c.tpt > 32;
  const int tiles_per_cta = blockDim.x / c.tpt;
  const long long num_tiles = (p.N + 7) >> 3;
  const long long full_tiles = p.N >> 3;
  const long long stride = (long long)gridDim.x * tiles_per_cta;
  const InT* __restrict__ x = reinterpret_cast<const InT*>(p.x);

  long long col[V];
  bool cvalid[V];
#pragma unroll
  for (int v = 0; v < V; v++) {
    col[v] = (long long)(c.tl + v * c.tpt) * VEC;
    cvalid[v] = col[v] < p.D;
  }

  // The next tile (one contiguous run of 8 * D elements) is pulled into L2 by a single bulk-prefetch
  // instruction while the current one is processed, so the register loads of the next iteration
  // find their lines on chip.
  const long long tile_bytes = 8 * p.D * (long long)sizeof(InT);
  const bool can_prefetch = (reinterpret_cast<uintptr_t>(p.x) & 15) == 0 && (tile_bytes & 15) == 0;
  const bool philox = p.noise == nullptr;
  float xv[8][V][VEC];
  int it = 0;
  for (long long tile = (long long)blockIdx.x * tiles_per_cta + c.grp; tile < num_tiles; tile += stride, ++it) {
    const long long next = tile + stride;
    if (c.tl == 0 && can_prefetch && next < full_tiles) {  // never the ragged last tile
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(x + (next << 3) * p.D), "r"((uint32_t)tile_bytes)
                   : "memory");
    }
    bool done = false;
    if (philox && tile < full_tiles) {
      load_tile<InT, VEC, V, true>(x, c, tile, col, cvalid, xv);
      done = process_tile<InT, BITS, VEC, V, true>(p, c, tile, it, col, cvalid, xv, s_part, s_fin);
      if (!done) ++it;  // the redo below exchanges its statistics through the other shared-memory buffer
    }
    if (!done) {
      load_tile<InT, VEC, V, false>(x, c, tile, col, cvalid, xv);
      process_tile<InT, BITS, VEC, V, false>(p, c, tile, it, col, cvalid, xv, s_part, s_fin);
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// pack_single_precision with caller-computed statistics (the reference signature).  One thread per
// (8-row tile, column): any D, any alignment, and the reference's exact conversion
// __float2int_rn(fmax(t, 0)) for arbitrary caller-supplied scales.
template <typename InT, int BITS>
__global__ void __launch_bounds__(256) pack_given_stats_kernel(const __grid_constant__ PackParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  const InT* __restrict__ x = reinterpret_cast<const InT*>(p.x);
  const long long num_tiles = (p.N + 7) >> 3;
  const long long total = num_tiles * p.D;
  const long long G = (p.N + WPT - 1) / WPT;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long tile = idx / p.D;
    const long long d = idx - tile * p.D;
    const long long row0 = tile << 3;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (p.noise == nullptr) {
      const unsigned long long q = (unsigned long long)(((row0 + p.row_offset) >> 3) * ((p.D + 1) >> 1) + (d >> 1));
      philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
    }
    uint32_t acc[GPT];
#pragma unroll
    for (int g = 0; g < GPT; g++) acc[g] = 0u;
#pragma unroll
    for (int r = 0; r < 8; r++) {
      const long long n = row0 + r;
      if (n < p.N) {
        float xv[1];
        Ld<InT, 1>::load(x + n * p.D + d, xv);
        const float u = (p.noise != nullptr) ? __ldcs(p.noise + n * p.D + d)
                        : noise8_to_unit(u8_to_1p(w[r >> 1], (r & 1) * 2 + (uint32_t)(d & 1)));
        const float t = __fsub_rn(__fmaf_rn(__fsub_rn(xv[0], __ldg(p.mn_in + n)), __ldg(p.scale_in + n), u), 0.5f);
        const uint32_t code = (uint32_t)__float2int_rn(fmaxf(t, 0.f));  // quantization_cuda_kernel.cu:89
        acc[r / WPT] |= code << ((r % WPT) * BITS);
      }
    }
#pragma unroll
    for (int g = 0; g < GPT; g++) {
      const long long gi = tile * GPT + g;
      if (gi < G) p.packed[gi * p.D + d] = (uint8_t)acc[g];
    }
  }
}

// ---------------------------------------------------------------------------------------------------
struct UnpackParams {
  const uint8_t* packed;
  const void* scale;  // [N] fp32 or bf16 bits
  const void* mn;     // [N]
  float* out;         // [N, D]
  long long N, D;
  int tpt;
  int vec_stats;  // 1: scale/min are 16-byte aligned, whole-tile vector loads are legal
};

// code / s by the Markstein sequence q0 = c*r, rem = fma(-q0, s, c), q = fma(rem, r, q0) with r the
// correctly rounded reciprocal of s: equal to the IEEE quotient for every code 0..255 and every normal
// s (checked exhaustively over all 2^23 significands), used when 2^-100 <= |s| <= 2^100; any other
// scale (inf from a constant row, NaN, denormal) takes the division instruction sequence.
__device__ __forceinline__ bool scale_is_tame(float s) {
  const uint32_t e = (__float_as_uint(s) >> 23) & 0xffu;
  return e >= 27u && e <= 227u;
}

template <int BITS, int VEC, int V, bool STATS_BF16>
__global__ void __launch_bounds__(256)
unpack_dequant_kernel(const __grid_constant__ UnpackParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  constexpr uint32_t MASKREP = 0x01010101u * ((1u << BITS) - 1u);
  const long long N = p.N, D = p.D;
  const int tpt = p.tpt;
  const int grp = threadIdx.x / tpt;
  const int tl = threadIdx.x - grp * tpt;
  const int lane = threadIdx.x & 31;
  const int lane_base = (tpt < 32) ? (lane / tpt) * tpt : 0;
  const unsigned gmask = (tpt < 32) ? (((1u << tpt) - 1u) << lane_base) : 0xffffffffu;
  const int tiles_per_cta = blockDim.x / tpt;
  const long long num_tiles = (N + 7) >> 3;
  const long long G = (N + WPT - 1) / WPT;
  const f32x2 neg_2p23 = f2_pack(-8388608.f, -8388608.f);

  long long col[V];
  bool cvalid[V];
#pragma unroll
  for (int v = 0; v < V; v++) {
    col[v] = (long long)(tl + v * tpt) * VEC;
    cvalid[v] = col[v] < D;
  }

  for (long long tile = (long long)blockIdx.x * tiles_per_cta + grp; tile < num_tiles;
       tile += (long long)gridDim.x * tiles_per_cta) {
    const long long row0 = tile << 3;
    const int rows_valid = (N - row0 >= 8) ? 8 : (int)(N - row0);

    uint32_t b[GPT][V];
#pragma unroll
    for (int g = 0; g < GPT; g++) {
      const long long gi = tile * GPT + g;
#pragma unroll
      for (int v = 0; v < V; v++) b[g][v] = (gi < G && cvalid[v]) ? load_bytes<VEC>(p.packed + gi * D + col[v]) : 0u;
    }

    float s[8], m[8];
    if (rows_valid == 8 && p.vec_stats) {
      if (STATS_BF16) {
        const uint4 sv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.scale) + row0));
        const uint4 mv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.mn) + row0));
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        const uint32_t mw[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          s[2 * i] = __uint_as_float(sw[i] << 16);
          s[2 * i + 1] = __uint_as_float(sw[i] & 0xffff0000u);
          m[2 * i] = __uint_as_float(mw[i] << 16);
          m[2 * i + 1] = __uint_as_float(mw[i] & 0xffff0000u);
        }
      } else {
        const float4* sp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.scale) + row0);
        const float4* mp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.mn) + row0);
        const float4 s0 = __ldg(sp), s1 = __ldg(sp + 1), m0 = __ldg(mp), m1 = __ldg(mp + 1);
        s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
        m[0] = m0.x; m[1] = m0.y; m[2] = m0.z; m[3] = m0.w; m[4] = m1.x; m[5] = m1.y; m[6] = m1.z; m[7] = m1.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < 8; r++) {
        if (r < rows_valid) {
          if (STATS_BF16) {
            s[r] = bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p.scale) + row0 + r));
            m[r] = bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p.mn) + row0 + r));
          } else {
            s[r] = __ldg(reinterpret_cast<const float*>(p.scale) + row0 + r);
            m[r] = __ldg(reinterpret_cast<const float*>(p.mn) + row0 + r);
          }
        } else {
          s[r] = 1.f;
          m[r] = 0.f;
        }
      }
    }

    // one correctly rounded reciprocal per row, computed by lane (lane & 7) and shared in the group
    const int my = lane & 7;
    float s_my = s[0];
#pragma unroll
    for (int r = 1; r < 8; r++) s_my = (my == r) ? s[r] : s_my;
    const float r_my = __frcp_rn(s_my);
    const bool tame = __all_sync(gmask, scale_is_tame(s_my));
    float rcp[8];
#pragma unroll
    for (int r = 0; r < 8; r++) rcp[r] = __shfl_sync(gmask, r_my, lane_base + r);

#pragma unroll
    for (int r = 0; r < 8; r++) {
      if (r < rows_valid) {
        const int sh = (r % WPT) * BITS;
        const f32x2 r2 = f2_pack(rcp[r], rcp[r]);
        const f32x2 ns2 = f2_pack(-s[r], -s[r]);
        const f32x2 m2 = f2_pack(m[r], m[r]);
#pragma unroll
        for (int v = 0; v < V; v++) {
          if (cvalid[v]) {
            const uint32_t t = (BITS == 8) ? b[r / WPT][v] : ((b[r / WPT][v] >> sh) & MASKREP);
            float cf[VEC], o[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++)  // 0x4B0000cc = 2^23 + code
              cf[e] = __uint_as_float(__byte_perm(t, 0x4b000000u, 0x7540 | e));
            if (VEC >= 2 && tame) {
#pragma unroll
              for (int e = 0; e < VEC; e += 2) {
                const f32x2 c2 = f2_add(f2_pack(cf[e], cf[(e + 1) % VEC]), neg_2p23);
                const f32x2 q0 = f2_mul(c2, r2);
                const f32x2 rem = f2_fma(q0, ns2, c2);
                const f32x2 q = f2_fma(rem, r2, q0);
                f2_unpack(f2_add(q, m2), o[e], o[(e + 1) % VEC]);
              }
            } else {
#pragma unroll
              for (int e = 0; e < VEC; e++)  // quantization_cuda_kernel.cu:182: IEEE division, then addition
                o[e] = __fadd_rn(__fdiv_rn(__fsub_rn(cf[e], 8388608.f), s[r]), m[r]);
            }
            StF32<VEC>::store(p.out + (row0 + r) * D + col[v], o);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Host side: shape -> (VEC, V, tpt, block) and launch.
struct TileShape {
  int vec, v, tpt, block;
};

static int pow2ceil(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

// Chooses the register tiling for D columns whose accesses may use `max_vec` elements per load.
static bool choose_shape(long long D, int max_vec, TileShape* s) {
  int vec = (max_vec >= 4 && D % 4 == 0) ? 4 : (max_vec >= 2 && D % 2 == 0) ? 2 : 1;
  long long C = D / vec;
  int v, tpt;
  if (C <= 32) {
    v = 1;
    tpt = pow2ceil((int)C);
    if (tpt < 8) tpt = 8;
  } else if (C <= 64) {
    v = 2;
    tpt = 32;
  } else if (C <= 512) {
    v = 2;
    tpt = (int)(((C + 1) / 2 + 31) / 32) * 32;
  } else if (C <= 1024 && vec == 4) {
    v = 4;
    tpt = (int)(((C + 3) / 4 + 31) / 32) * 32;
  } else {
    return false;
  }
  int block = tpt >= 128 ? tpt : tpt * (128 / tpt);
  s->vec = vec; s->v = v; s->tpt = tpt; s->block = block;
  return true;
}

template <typename K>
static int persistent_grid(K kernel, int block, long long work_ctas, int* grid) {
  int per_sm = 0;
  EXB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, 0));
  if (per_sm < 1) per_sm = 1;
  long long g = (long long)sm_count() * per_sm;
  if (g > work_ctas) g = work_ctas;
  if (g < 1) g = 1;
  *grid = (int)g;
  return EXB_OK;
}

template <typename InT, int BITS>
static int launch_pack(const PackParams& p, const TileShape& s, cudaStream_t st) {
  const long long tiles = (p.N + 7) / 8;
  const int tiles_per_cta = s.block / s.tpt;
  const long long ctas = (tiles + tiles_per_cta - 1) / tiles_per_cta;
  int grid = 1;
#define EXB_PACK_CASE(VEC_, V_)                                                        \
  if (s.vec == VEC_ && s.v == V_) {                                                    \
    auto k = quantize_pack_kernel<InT, BITS, VEC_, V_>;                                \
    int rc = persistent_grid(k, s.block, ctas, &grid);                                 \
    if (rc) return rc;                                                                 \
    k<<<grid, s.block, 0, st>>>(p);                                                    \
    EXB_CUDA_OK(cudaGetLastError());                                                   \
    return EXB_OK;                                                                     \
  }
  EXB_PACK_CASE(4, 1) EXB_PACK_CASE(4, 2) EXB_PACK_CASE(4, 4)
  EXB_PACK_CASE(2, 1) EXB_PACK_CASE(2, 2)
  EXB_PACK_CASE(1, 1) EXB_PACK_CASE(1, 2)
#undef EXB_PACK_CASE
  return fail(EXB_ERR_UNSUPPORTED, "no pack kernel for vec=%d v=%d", s.vec, s.v);
}

template <typename InT>
static int launch_pack_bits(const PackParams& p, int bits, const TileShape& s, cudaStream_t st) {
  switch (bits) {
    case 1: return launch_pack<InT, 1>(p, s, st);
    case 2: return launch_pack<InT, 2>(p, s, st);
    case 4: return launch_pack<InT, 4>(p, s, st);
    case 8: return launch_pack<InT, 8>(p, s, st);
  }
  return fail(EXB_ERR_ARG, "bits must be 1, 2, 4 or 8 (got %d)", bits);
}

template <typename InT>
static int launch_given_stats(const PackParams& p, int bits, cudaStream_t st) {
  const long long total = ((p.N + 7) / 8) * p.D;
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  switch (bits) {
    case 1: pack_given_stats_kernel<InT, 1><<<(int)blocks, 256, 0, st>>>(p); break;
    case 2: pack_given_stats_kernel<InT, 2><<<(int)blocks, 256, 0, st>>>(p); break;
    case 4: pack_given_stats_kernel<InT, 4><<<(int)blocks, 256, 0, st>>>(p); break;
    default: pack_given_stats_kernel<InT, 8><<<(int)blocks, 256, 0, st>>>(p); break;
  }
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

static int align_vec(const void* ptr, int elem_bytes) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
  if (a % (4 * elem_bytes) == 0) return 4;
  if (a % (2 * elem_bytes) == 0) return 2;
  return 1;
}

static int pack_common(const void* x, int dtype, long long N, long long D, int bits,
                       const float* noise, const float* mn_in, const float* scale_in,
                       unsigned long long seed, unsigned long long offset, long long row_offset,
                       uint8_t* packed, uint16_t* scale_bf16, uint16_t* min_bf16, float* scale_f32,
                       float* min_f32, cudaStream_t st) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(dtype == EXACT_DTYPE_F32 || dtype == EXACT_DTYPE_BF16,
              "pack: dtype must be EXACT_DTYPE_F32 or EXACT_DTYPE_BF16 (got %d)", dtype);
  EXB_REQUIRE(N >= 0 && D >= 0, "pack: negative shape %lld x %lld", N, D);
  EXB_REQUIRE(row_offset >= 0 && row_offset % 8 == 0, "pack: row_offset must be a non-negative multiple of 8");
  if (N == 0 || D == 0) return EXB_OK;
  EXB_REQUIRE(x != nullptr && packed != nullptr, "pack: null data or output pointer");
  PackParams p;
  p.x = x; p.noise = noise; p.mn_in = mn_in; p.scale_in = scale_in;
  p.packed = packed; p.scale_bf16 = scale_bf16; p.min_bf16 = min_bf16;
  p.scale_f32 = scale_f32; p.min_f32 = min_f32;
  p.N = N; p.D = D; p.row_offset = row_offset; p.tpt = 0;
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.key = make_philox_key(seed);
  if (mn_in != nullptr) {
    if (dtype == EXACT_DTYPE_F32) return launch_given_stats<float>(p, bits, st);
    return launch_given_stats<uint16_t>(p, bits, st);
  }
  const int eb = dtype == EXACT_DTYPE_F32 ? 4 : 2;
  int max_vec = align_vec(x, eb);
  if (noise) max_vec = max_vec < align_vec(noise, 4) ? max_vec : align_vec(noise, 4);
  const int pa = (int)(reinterpret_cast<uintptr_t>(packed) & 3);
  if (pa != 0) max_vec = (pa == 2 && max_vec >= 2) ? 2 : 1;
  TileShape s;
  if (!choose_shape(D, max_vec, &s))
    return fail(EXB_ERR_UNSUPPORTED, "pack: D=%lld is beyond the register-tiled kernels (max 4096 when D%%4==0, 1024 when D%%2==0, 512 otherwise)", D);
  p.tpt = s.tpt;
  if (dtype == EXACT_DTYPE_F32) return launch_pack_bits<float>(p, bits, s, st);
  return launch_pack_bits<uint16_t>(p, bits, s, st);
}

template <int BITS, bool BF>
static int launch_unpack(const UnpackParams& p, const TileShape& s, cudaStream_t st) {
  const long long tiles = (p.N + 7) / 8;
  const int tiles_per_cta = s.block / s.tpt;
  const long long ctas = (tiles + tiles_per_cta - 1) / tiles_per_cta;
  int grid = 1;
#define EXB_UNPACK_CASE(VEC_, V_)                                                      \
  if (s.vec == VEC_ && s.v == V_) {                                                    \
    auto k = unpack_dequant_kernel<BITS, VEC_, V_, BF>;                                \
    int rc = persistent_grid(k, s.block, ctas, &grid);                                 \
    if (rc) return rc;                                                                 \
    k<<<grid, s.block, 0, st>>>(p);                                                    \
    EXB_CUDA_OK(cudaGetLastError());                                                   \
    return EXB_OK;                                                                     \
  }
  EXB_UNPACK_CASE(4, 1) EXB_UNPACK_CASE(4, 2) EXB_UNPACK_CASE(4, 4)
  EXB_UNPACK_CASE(2, 1) EXB_UNPACK_CASE(2, 2)
  EXB_UNPACK_CASE(1, 1) EXB_UNPACK_CASE(1, 2)
#undef EXB_UNPACK_CASE
  return fail(EXB_ERR_UNSUPPORTED, "no unpack kernel for vec=%d v=%d", s.vec, s.v);
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_quantize_pack(const void* x, int dtype, int64_t N, int64_t D, int bits, const float* noise,
                        uint64_t seed, uint64_t offset, int64_t row_offset, uint8_t* packed,
                        uint16_t* scale_bf16, uint16_t* min_bf16, float* scale_f32, float* min_f32,
                        void* stream) {
  return pack_common(x, dtype, N, D, bits, noise, nullptr, nullptr, seed, offset, row_offset, packed,
                     scale_bf16, min_bf16, scale_f32, min_f32, (cudaStream_t)stream);
}

int exact_pack_single_precision(const void* data, int dtype, const float* min, const float* scale,
                                int64_t N, int64_t D, int bits, const float* noise, uint64_t seed,
                                uint64_t offset, int64_t row_offset, uint8_t* packed, void* stream) {
  if (N > 0 && D > 0) EXB_REQUIRE(min != nullptr && scale != nullptr, "pack_single_precision: null min/scale");
  return pack_common(data, dtype, N, D, bits, noise, min, scale, seed, offset, row_offset, packed,
                     nullptr, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

int exact_unpack_single_precision(const uint8_t* packed, int bits, const void* scale, const void* min,
                                  int stats_dtype, int64_t N, int64_t D, float* out, void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(stats_dtype == EXACT_DTYPE_F32 || stats_dtype == EXACT_DTYPE_BF16,
              "unpack: scale/min dtype must be EXACT_DTYPE_F32 or EXACT_DTYPE_BF16 (got %d)", stats_dtype);
  EXB_REQUIRE(N >= 0 && D >= 0, "unpack: negative shape");
  if (N == 0 || D == 0) return EXB_OK;
  EXB_REQUIRE(packed && scale && min && out, "unpack: null pointer");
  int max_vec = align_vec(out, 4);
  const int pa = (int)(reinterpret_cast<uintptr_t>(packed) & 3);
  if (pa != 0) max_vec = (pa == 2 && max_vec >= 2) ? 2 : 1;
  TileShape s;
  if (!choose_shape(D, max_vec, &s))
    return fail(EXB_ERR_UNSUPPORTED, "unpack: D=%lld is beyond the register-tiled kernels", (long long)D);
  UnpackParams p;
  p.packed = packed; p.scale = scale; p.mn = min; p.out = out; p.N = N; p.D = D; p.tpt = s.tpt;
  p.vec_stats = (reinterpret_cast<uintptr_t>(scale) % 16 == 0 && reinterpret_cast<uintptr_t>(min) % 16 == 0) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf = stats_dtype == EXACT_DTYPE_BF16;
  switch (bits) {
    case 1: return bf ? launch_unpack<1, true>(p, s, st) : launch_unpack<1, false>(p, s, st);
    case 2: return bf ? launch_unpack<2, true>(p, s, st) : launch_unpack<2, false>(p, s, st);
    case 4: return bf ? launch_unpack<4, true>(p, s, st) : launch_unpack<4, false>(p, s, st);
    default: return bf ? launch_unpack<8, true>(p, s, st) : launch_unpack<8, false>(p, s, st);
  }
}

}  // extern "C"
