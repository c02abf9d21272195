// fp16 activations: quantise + pack and unpack + dequantise with the arithmetic of the reference's half
// instantiations.
//
// The reference dispatches its pack / unpack kernels on float and half
// (exact/exact/cpp_extension/quantization_cuda_kernel.cu:132, 209).  With scalar_t = c10::Half every
// Half (op) Half is computed in fp32 and rounded back to half, so
//   pack    (quantization_cuda_kernel.cu:89)   t = half(half(x - min) * scale) ; code = rint(max(float(t) + noise - 0.5, 0))
//   unpack  (quantization_cuda_kernel.cu:182)  out = half(half(float(code) / scale) + min)
// and the row statistics of an fp16 activation stay fp16 (exact/exact/ops.py:82-83): min = min_d x,
// scale = half(float(half(1 / float(half(max - min)))) * (2^bits - 1)), the half ops of torch behind
// `(2 ** bits - 1) / (mx - mn)` (ops.py:39: reciprocal, then multiplication by the scalar).
// The packed layout is that of the fp32 path.  These are plain streaming kernels (one thread per 8-row tile and
// column, one warp per row for the statistics); the fp32 / bf16 path is the tuned one.
#include <cuda_fp16.h>

#include "exact_b200.h"
#include "common.cuh"

namespace exb {

__device__ __forceinline__ float h_bits_to_f32(uint16_t b) { return __half2float(__ushort_as_half(b)); }
__device__ __forceinline__ uint16_t f32_to_h_bits(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float round_h(float f) { return __half2float(__float2half_rn(f)); }

// min / max of a row of halves and the half scale; NaN anywhere in the row gives NaN statistics (torch.min / max).
__global__ void __launch_bounds__(256) f16_row_stats_kernel(const uint16_t* __restrict__ x, long long N, long long D, float B,
                                                            uint16_t* __restrict__ mn_out, uint16_t* __restrict__ scale_out) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long n = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < N; n += warps) {
    const uint16_t* __restrict__ r = x + n * D;
    float lo = __int_as_float(0x7f800000), hi = __int_as_float(0xff800000);
    for (long long d = lane; d < D; d += 32) {
      const float v = h_bits_to_f32(__ldg(r + d));
      lo = min_nan(lo, v);
      hi = max_nan(hi, v);
    }
    lo = redux_min_nan(lo, 0xffffffffu);
    hi = redux_max_nan(hi, 0xffffffffu);
    if (lane == 0) {
      const float diff = round_h(__fsub_rn(hi, lo));
      const float rcp = round_h(__fdiv_rn(1.0f, diff));
      mn_out[n] = f32_to_h_bits(lo);
      scale_out[n] = f32_to_h_bits(__fmul_rn(rcp, B));
    }
  }
}

struct PackF16Params {
  const uint16_t* x;
  const uint16_t* mn;
  const uint16_t* scale;
  const float* noise;
  uint8_t* packed;
  long long N, D, row_offset;
  uint32_t off_lo, off_hi;
  PhiloxKey key;
};

template <int BITS>
__global__ void __launch_bounds__(256) f16_pack_kernel(const __grid_constant__ PackF16Params p) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  const long long num_tiles = (p.N + 7) >> 3;
  const long long total = num_tiles * p.D;
  const long long G = (p.N + WPT - 1) / WPT;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long tile = idx / p.D;
    const long long d = idx - tile * p.D;
    const long long row0 = tile << 3;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (p.noise == nullptr) {   // the noise stream of the fp32 pack kernels: one Philox block per (8-row tile, column pair)
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
        const float xv = h_bits_to_f32(__ldg(p.x + n * p.D + d));
        const float u = (p.noise != nullptr) ? __ldcs(p.noise + n * p.D + d)
                        : noise8_to_unit(u8_to_1p(w[r >> 1], (r & 1) * 2 + (uint32_t)(d & 1)));
        const float t1 = round_h(__fsub_rn(xv, h_bits_to_f32(__ldg(p.mn + n))));
        const float t2 = round_h(__fmul_rn(t1, h_bits_to_f32(__ldg(p.scale + n))));
        // Half + float is a float; "- 0.5" is a double subtraction narrowed by __float2int_rn's argument,
        // one correctly rounded fp32 subtraction either way
        const float t = __fsub_rn(__fadd_rn(t2, u), 0.5f);
        const uint32_t code = (uint32_t)__float2int_rn(fmaxf(t, 0.f));
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

template <int BITS>
__global__ void __launch_bounds__(256) f16_unpack_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scale,
                                                         const uint16_t* __restrict__ mn, long long N, long long D,
                                                         uint16_t* __restrict__ out) {
  constexpr int WPT = 8 / BITS;
  constexpr int GPT = BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  const long long num_tiles = (N + 7) >> 3;
  const long long total = num_tiles * D;
  const long long G = (N + WPT - 1) / WPT;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long tile = idx / D;
    const long long d = idx - tile * D;
    const long long row0 = tile << 3;
#pragma unroll
    for (int g = 0; g < GPT; g++) {
      const long long gi = tile * GPT + g;
      if (gi >= G) break;
      const uint32_t byte = __ldg(packed + gi * D + d);
#pragma unroll
      for (int i = 0; i < WPT; i++) {
        const long long n = row0 + g * WPT + i;
        if (n < N) {
          const float c = (float)((byte >> (i * BITS)) & MASK);   // exact in half
          const float q = round_h(__fdiv_rn(c, h_bits_to_f32(__ldg(scale + n))));
          out[n * D + d] = f32_to_h_bits(__fadd_rn(q, h_bits_to_f32(__ldg(mn + n))));
        }
      }
    }
  }
}

static int f16_grid(long long total) {
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

static int f16_pack_launch(const uint16_t* x, const uint16_t* mn, const uint16_t* scale, long long N, long long D, int bits,
                           const float* noise, unsigned long long seed, unsigned long long offset, long long row_offset,
                           uint8_t* packed, cudaStream_t st) {
  PackF16Params p;
  p.x = x; p.mn = mn; p.scale = scale; p.noise = noise; p.packed = packed;
  p.N = N; p.D = D; p.row_offset = row_offset;
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.key = make_philox_key(seed);
  const int grid = f16_grid(((N + 7) / 8) * D);
  switch (bits) {
    case 1: f16_pack_kernel<1><<<grid, 256, 0, st>>>(p); break;
    case 2: f16_pack_kernel<2><<<grid, 256, 0, st>>>(p); break;
    case 4: f16_pack_kernel<4><<<grid, 256, 0, st>>>(p); break;
    default: f16_pack_kernel<8><<<grid, 256, 0, st>>>(p); break;
  }
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // namespace exb

using namespace exb;

extern "C" {

int exact_pack_single_precision_f16(const void* data, const void* min, const void* scale, int64_t N, int64_t D, int bits,
                                    const float* noise, uint64_t seed, uint64_t offset, int64_t row_offset,
                                    uint8_t* packed, void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D >= 0, "pack_f16: negative shape");
  EXB_REQUIRE(row_offset >= 0 && row_offset % 8 == 0, "pack_f16: row_offset must be a non-negative multiple of 8");
  if (N == 0 || D == 0) return EXB_OK;
  EXB_REQUIRE(data && min && scale && packed, "pack_f16: null pointer");
  return f16_pack_launch(static_cast<const uint16_t*>(data), static_cast<const uint16_t*>(min),
                         static_cast<const uint16_t*>(scale), N, D, bits, noise, seed, offset, row_offset, packed,
                         (cudaStream_t)stream);
}

int exact_quantize_pack_f16(const void* x, int64_t N, int64_t D, int bits, const float* noise, uint64_t seed,
                            uint64_t offset, int64_t row_offset, uint8_t* packed, uint16_t* scale_f16, uint16_t* min_f16,
                            void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D >= 0, "quantize_pack_f16: negative shape");
  EXB_REQUIRE(row_offset >= 0 && row_offset % 8 == 0, "quantize_pack_f16: row_offset must be a non-negative multiple of 8");
  if (N == 0 || D == 0) return EXB_OK;
  EXB_REQUIRE(x && packed && scale_f16 && min_f16, "quantize_pack_f16: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  long long blocks = (N + 7) / 8;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  f16_row_stats_kernel<<<(int)blocks, 256, 0, st>>>(static_cast<const uint16_t*>(x), N, D, (float)((1 << bits) - 1), min_f16,
                                                    scale_f16);
  EXB_CUDA_OK(cudaGetLastError());
  return f16_pack_launch(static_cast<const uint16_t*>(x), min_f16, scale_f16, N, D, bits, noise, seed, offset, row_offset,
                         packed, st);
}

int exact_unpack_single_precision_f16(const uint8_t* packed, int bits, const void* scale, const void* min, int64_t N,
                                      int64_t D, void* out, void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D >= 0, "unpack_f16: negative shape");
  if (N == 0 || D == 0) return EXB_OK;
  EXB_REQUIRE(packed && scale && min && out, "unpack_f16: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = f16_grid(((N + 7) / 8) * D);
  const uint16_t* s = static_cast<const uint16_t*>(scale);
  const uint16_t* m = static_cast<const uint16_t*>(min);
  uint16_t* o = static_cast<uint16_t*>(out);
  switch (bits) {
    case 1: f16_unpack_kernel<1><<<grid, 256, 0, st>>>(packed, s, m, N, D, o); break;
    case 2: f16_unpack_kernel<2><<<grid, 256, 0, st>>>(packed, s, m, N, D, o); break;
    case 4: f16_unpack_kernel<4><<<grid, 256, 0, st>>>(packed, s, m, N, D, o); break;
    default: f16_unpack_kernel<8><<<grid, 256, 0, st>>>(packed, s, m, N, D, o); break;
  }
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
