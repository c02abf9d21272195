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
// tile spans several warps, a double-buffered shared-memory exchange with named barriers.
#include "common.cuh"
#include "exact_b200.h"

namespace exb {

struct PackParams {
  const void* x;          // [N, D] fp32 or bf16 bits
  const float* noise;     // [N, D] supplied U[0,1) noise, or null -> Philox
  const float* mn_in;     // [N] precomputed row min (reference-signature entry) or null
  const float* scale_in;  // [N] precomputed row scale or null
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

// Barrier over the threads of one tile group; ids are literals so the kernel reserves only those.
__device__ __forceinline__ void group_barrier(int grp, int nthreads) {
  if (grp == 0) named_barrier<1>(nthreads);
  else if (grp == 1) named_barrier<2>(nthreads);
  else named_barrier<3>(nthreads);
}

constexpr int kMaxWarpsPerTile = 8;
constexpr int kMaxGroupsPerCta = 4;

template <typename InT, int BITS, int VEC, int V>
__global__ void __launch_bounds__(256)
quantize_pack_kernel(const __grid_constant__ PackParams p) {
  constexpr int WPT = 8 / BITS;  // rows per packed byte
  constexpr int GPT = BITS;      // packed byte-rows per 8-row tile (8 / WPT)
  const long long N = p.N, D = p.D;
  const int tpt = p.tpt;
  const int grp = threadIdx.x / tpt;
  const int tl = threadIdx.x - grp * tpt;
  const int tiles_per_cta = blockDim.x / tpt;
  const long long num_tiles = (N + 7) >> 3;
  const long long G = (N + WPT - 1) / WPT;
  const InT* __restrict__ x = reinterpret_cast<const InT*>(p.x);
  const bool multi = tpt > 32;
  const int lane = threadIdx.x & 31;
  const int lane_base = (tpt < 32) ? (lane / tpt) * tpt : 0;
  const unsigned gmask = (tpt < 32) ? (((1u << tpt) - 1u) << lane_base) : 0xffffffffu;
  const float B = (float)((1 << BITS) - 1);

  __shared__ float s_part[2][kMaxGroupsPerCta][kMaxWarpsPerTile][16];
  __shared__ __align__(16) float s_fin[2][kMaxGroupsPerCta][16];

  long long col[V];
  bool cvalid[V];
#pragma unroll
  for (int v = 0; v < V; v++) {
    col[v] = (long long)(tl + v * tpt) * VEC;
    cvalid[v] = col[v] < D;
  }

  int it = 0;
  for (long long tile = (long long)blockIdx.x * tiles_per_cta + grp; tile < num_tiles;
       tile += (long long)gridDim.x * tiles_per_cta, ++it) {
    const long long row0 = tile << 3;
    const int rows_valid = (N - row0 >= 8) ? 8 : (int)(N - row0);

    // ---- one pass over HBM: the whole tile into registers ---------------------------------------
    float xv[8][V][VEC];
#pragma unroll
    for (int r = 0; r < 8; r++) {
#pragma unroll
      for (int v = 0; v < V; v++) {
        if (r < rows_valid && cvalid[v]) {
          Ld<InT, VEC>::load(x + (row0 + r) * D + col[v], xv[r][v]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; e++) xv[r][v][e] = 0.f;
        }
      }
    }

    // ---- row statistics --------------------------------------------------------------------------
    float mn[8], sc[8];
    if (p.mn_in == nullptr) {
      float lo[8], hi[8];
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
        lo[r] = redux_min_nan(lo[r], gmask);
        hi[r] = redux_max_nan(hi[r], gmask);
      }
      if (!multi) {
        // lane (tl & 7) turns row (tl & 7)'s range into a scale, then the group shares the 8 scales.
        const int my = tl & 7;
        float lo_my = lo[0], hi_my = hi[0];
#pragma unroll
        for (int r = 1; r < 8; r++) {
          lo_my = (my == r) ? lo[r] : lo_my;
          hi_my = (my == r) ? hi[r] : hi_my;
        }
        // ops.py:39 evaluates (2^b - 1) / (mx - mn) as reciprocal(mx - mn) * (2^b - 1).
        const float s_my = __fmul_rn(__frcp_rn(__fsub_rn(hi_my, lo_my)), B);
#pragma unroll
        for (int r = 0; r < 8; r++) {
          sc[r] = __shfl_sync(gmask, s_my, lane_base + r);
          mn[r] = lo[r];
        }
        if (tl < rows_valid) {  // tl < 8 here because rows_valid <= 8
          const long long row = row0 + tl;
          if (p.scale_bf16) p.scale_bf16[row] = f32_to_bf16_bits(s_my);
          if (p.min_bf16) p.min_bf16[row] = f32_to_bf16_bits(lo_my);
          if (p.scale_f32) p.scale_f32[row] = s_my;
          if (p.min_f32) p.min_f32[row] = lo_my;
        }
      } else {
        const int buf = it & 1;
        const int wt = tl >> 5;  // warp within the tile
        const int nwt = tpt >> 5;
        if (lane == 0) {
#pragma unroll
          for (int r = 0; r < 8; r++) {
            s_part[buf][grp][wt][r] = lo[r];
            s_part[buf][grp][wt][8 + r] = hi[r];
          }
        }
        group_barrier(grp, tpt);
        if (tl < 8) {
          float lo_f = s_part[buf][grp][0][tl], hi_f = s_part[buf][grp][0][8 + tl];
          for (int w = 1; w < nwt; w++) {
            lo_f = min_nan(lo_f, s_part[buf][grp][w][tl]);
            hi_f = max_nan(hi_f, s_part[buf][grp][w][8 + tl]);
          }
          const float s_f = __fmul_rn(__frcp_rn(__fsub_rn(hi_f, lo_f)), B);
          s_fin[buf][grp][tl] = lo_f;
          s_fin[buf][grp][8 + tl] = s_f;
          if (tl < rows_valid) {
            const long long row = row0 + tl;
            if (p.scale_bf16) p.scale_bf16[row] = f32_to_bf16_bits(s_f);
            if (p.min_bf16) p.min_bf16[row] = f32_to_bf16_bits(lo_f);
            if (p.scale_f32) p.scale_f32[row] = s_f;
            if (p.min_f32) p.min_f32[row] = lo_f;
          }
        }
        group_barrier(grp, tpt);
        const float4* f = reinterpret_cast<const float4*>(&s_fin[buf][grp][0]);
        const float4 a = f[0], b = f[1], c = f[2], d = f[3];
        mn[0] = a.x; mn[1] = a.y; mn[2] = a.z; mn[3] = a.w;
        mn[4] = b.x; mn[5] = b.y; mn[6] = b.z; mn[7] = b.w;
        sc[0] = c.x; sc[1] = c.y; sc[2] = c.z; sc[3] = c.w;
        sc[4] = d.x; sc[5] = d.y; sc[6] = d.z; sc[7] = d.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < 8; r++) {
        const bool ok = r < rows_valid;
        mn[r] = ok ? __ldg(p.mn_in + row0 + r) : 0.f;
        sc[r] = ok ? __ldg(p.scale_in + row0 + r) : 0.f;
      }
    }

    // ---- quantise with stochastic rounding and assemble bytes -------------------------------------
    const long long noise_tile = (row0 + p.row_offset) >> 3;
#pragma unroll
    for (int v = 0; v < V; v++) {
      if (!cvalid[v]) continue;
      uint32_t acc[GPT][VEC];
#pragma unroll
      for (int g = 0; g < GPT; g++)
#pragma unroll
        for (int e = 0; e < VEC; e++) acc[g][e] = 0u;

      float un[8][VEC];
      if (p.noise != nullptr) {
#pragma unroll
        for (int r = 0; r < 8; r++) {
          if (r < rows_valid) {
            Ld<float, VEC>::load(p.noise + (row0 + r) * D + col[v], un[r]);
          } else {
#pragma unroll
            for (int e = 0; e < VEC; e++) un[r][e] = 0.f;
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          const unsigned long long q = (unsigned long long)(noise_tile * D + col[v] + e);
          uint32_t w[4];
          philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
#pragma unroll
          for (int r = 0; r < 8; r++) un[r][e] = (r & 1) ? u16_hi_to_unit(w[r >> 1]) : u16_lo_to_unit(w[r >> 1]);
        }
      }

#pragma unroll
      for (int r = 0; r < 8; r++) {
        if (r < rows_valid) {
#pragma unroll
          for (int e = 0; e < VEC; e++) {
            // quantization_cuda_kernel.cu:89: (x - mn) * s + u contracted to one FMA, then - 0.5,
            // fmax(., 0), round to nearest even; no upper clamp.
            float t = __fmaf_rn(__fsub_rn(xv[r][v][e], mn[r]), sc[r], un[r][e]);
            t = fmaxf(__fsub_rn(t, 0.5f), 0.f);
            const uint32_t code = (uint32_t)__float2int_rn(t);
            acc[r / WPT][e] |= code << ((r % WPT) * BITS);
          }
        }
      }

#pragma unroll
      for (int g = 0; g < GPT; g++) {
        const long long gi = tile * GPT + g;
        if (gi < G) {
          uint32_t b[VEC];
#pragma unroll
          for (int e = 0; e < VEC; e++) b[e] = acc[g][e] & 0xffu;  // the reference's uint8 narrowing
          StBytes<VEC>::store(p.packed + gi * D + col[v], b);
        }
      }
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

template <int BITS, int VEC, int V, bool STATS_BF16>
__global__ void __launch_bounds__(256)
unpack_dequant_kernel(const __grid_constant__ UnpackParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  const long long N = p.N, D = p.D;
  const int tpt = p.tpt;
  const int grp = threadIdx.x / tpt;
  const int tl = threadIdx.x - grp * tpt;
  const int tiles_per_cta = blockDim.x / tpt;
  const long long num_tiles = (N + 7) >> 3;
  const long long G = (N + WPT - 1) / WPT;

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

    uint32_t b[GPT][V][VEC];
#pragma unroll
    for (int g = 0; g < GPT; g++) {
      const long long gi = tile * GPT + g;
#pragma unroll
      for (int v = 0; v < V; v++) {
        if (gi < G && cvalid[v]) {
          StBytes<VEC>::load(p.packed + gi * D + col[v], b[g][v]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; e++) b[g][v][e] = 0u;
        }
      }
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

#pragma unroll
    for (int r = 0; r < 8; r++) {
      if (r < rows_valid) {
#pragma unroll
        for (int v = 0; v < V; v++) {
          if (cvalid[v]) {
            float o[VEC];
#pragma unroll
            for (int e = 0; e < VEC; e++) {
              const uint32_t code = (b[r / WPT][v][e] >> ((r % WPT) * BITS)) & MASK;
              // quantization_cuda_kernel.cu:182: IEEE division, then addition.
              o[e] = __fadd_rn(__fdiv_rn((float)code, s[r]), m[r]);
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
  EXB_REQUIRE((mn_in == nullptr) == (scale_in == nullptr), "pack: min and scale must be given together");
  const int eb = dtype == EXACT_DTYPE_F32 ? 4 : 2;
  int max_vec = align_vec(x, eb);
  if (noise) max_vec = max_vec < align_vec(noise, 4) ? max_vec : align_vec(noise, 4);
  const int pa = (int)(reinterpret_cast<uintptr_t>(packed) & 3);
  if (pa != 0) max_vec = (pa == 2 && max_vec >= 2) ? 2 : 1;
  TileShape s;
  if (!choose_shape(D, max_vec, &s))
    return fail(EXB_ERR_UNSUPPORTED, "pack: D=%lld is beyond the register-tiled kernels (max 4096 when D%%4==0, 1024 when D%%2==0, 512 otherwise)", D);
  PackParams p;
  p.x = x; p.noise = noise; p.mn_in = mn_in; p.scale_in = scale_in;
  p.packed = packed; p.scale_bf16 = scale_bf16; p.min_bf16 = min_bf16;
  p.scale_f32 = scale_f32; p.min_f32 = min_f32;
  p.N = N; p.D = D; p.row_offset = row_offset; p.tpt = s.tpt;
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.key = make_philox_key(seed);
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
