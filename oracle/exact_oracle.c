/*
 * exact_oracle.c -- CPU restatement of the activation-compression hot path of EXACT
 * (zirui-ray-liu/Exact).  TEST INFRASTRUCTURE ONLY: this file is the checker the CUDA kernels are
 * compared against and the timed CPU baseline.  Nothing in the product may call it.
 *
 * Parity pin: the reference holds no golden vectors for the packed stream, the row statistics, the
 * dequantised values or the projection (its tests are print-only for those).  The pin is therefore
 * (a) the reference's own asserting tests re-expressed on CPU (ReLU == F.relu, dropout mask/scale
 * consistency, SpMM forward == a scipy CSR product), and (b) fixtures under tests/golden/ produced by
 * the reference's unmodified CUDA kernels on a B200 (see tests/golden/make_ref_vectors.py), which this
 * file must reproduce bit for bit.  Without (b) the pack/unpack parity is "unpinned".
 *
 * Every function cites the reference lines it follows (paths relative to the reference checkout).
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC exact_oracle.c -o liboracle.so -lm
 * (-ffp-contract=off: every fused multiply-add below is written explicitly with fmaf()).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------------
 * bf16 <-> fp32, round-to-nearest-even, as torch's Tensor.to(torch.bfloat16) does.
 * exact/exact/ops.py:80-81 stores scale and min as bf16; ops.py:94-96 widens them again.
 * ---------------------------------------------------------------------------------------------- */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0; /* NaN -> canonical quiet NaN */
  uint32_t bias = 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)((u + bias) >> 16);
}
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
ORC_API void orc_f32_to_bf16(const float *x, int64_t n, uint16_t *out) {
  for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16(x[i]);
}
ORC_API void orc_bf16_to_f32(const uint16_t *x, int64_t n, float *out) {
  for (int64_t i = 0; i < n; i++) out[i] = bf16_to_f32(x[i]);
}

/* ------------------------------------------------------------------------------------------------
 * Row statistics.  exact/exact/ops.py:61-66 (== qsheme.py:41-48): mn = min_d x, mx = max_d x with
 * torch.min/max semantics (a NaN in the row makes the result NaN).  ops.py:39:
 *     scale = (2 ** bits - 1) / (mx - mn)
 * is "python int / tensor", which torch evaluates as Tensor.__rtruediv__ = reciprocal(t) * other
 * (torch/_tensor.py): TWO fp32 roundings, fl(fl(1/(mx-mn)) * B), not one IEEE division.
 * mx == mn gives 1/0 = inf, inf * B = inf.
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_row_stats(const float *x, int64_t N, int64_t D, int bits, float *mn, float *mx,
                           float *scale) {
  const float B = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const float *r = x + n * D;
    float lo = r[0], hi = r[0];
    int nan = isnan(r[0]);
    for (int64_t d = 1; d < D; d++) {
      float v = r[d];
      if (isnan(v)) nan = 1;
      if (v < lo) lo = v;
      if (v > hi) hi = v;
    }
    if (nan) lo = hi = NAN;
    mn[n] = lo;
    mx[n] = hi;
    float rcp = 1.0f / (hi - lo); /* IEEE-rounded reciprocal */
    scale[n] = rcp * B;
  }
}

/* ------------------------------------------------------------------------------------------------
 * pack_single_precision.  exact/exact/cpp_extension/quantization_cuda_kernel.cu:73-93.
 *   val  = __float2int_rn(fmax((data[id] - min[n]) * scale[n] + noise - 0.5, 0.0f));
 *   byte[(n / wpt) * D + d] |= val << ((n % wpt) * bits)            (uint8 accumulator, no clamp)
 * fp32 subtraction; mul+add contracted to one FMA by nvcc's default -fmad=true (use_fma=1; 0 gives
 * the uncontracted variant so that the question can be settled against the reference's binary);
 * "- 0.5" is a double-literal subtraction whose result is rounded back to fp32 by the implicit
 * conversion in __float2int_rn(float): identical to one fp32 subtraction because the double
 * difference is exact.  fmax(NaN, 0) = 0.  Rounding is to nearest even.  Rows >= N in the last
 * group contribute nothing (quantization_cuda_kernel.cu:85).  The int -> uint8 narrowing keeps the
 * low 8 bits of (val << shift), so a code of 2^bits spills into the next row's field or vanishes.
 * The reference allocates G*D + 1 bytes (quantization_cuda_kernel.cu:110-113) and never writes the
 * last one; this function writes G*D bytes.
 * ---------------------------------------------------------------------------------------------- */
static inline int32_t float2int_rn(float t) {
  /* CUDA __float2int_rn: NaN -> 0, saturating, ties to even. */
  if (isnan(t)) return 0;
  if (t >= 2147483648.0f) return INT32_MAX;
  if (t <= -2147483648.0f) return INT32_MIN;
  return (int32_t)nearbyintf(t); /* default rounding mode: to nearest even */
}

static inline int32_t quant_code(float x, float mn, float s, float u, int use_fma) {
  float a = x - mn;
  float t = use_fma ? fmaf(a, s, u) : (a * s) + u;
  t = t - 0.5f;
  t = fmaxf(t, 0.0f); /* fmaxf(NaN, 0) = 0 */
  return float2int_rn(t);
}

ORC_API void orc_pack(const float *x, const float *mn, const float *scale, const float *noise,
                      int64_t N, int64_t D, int bits, int use_fma, uint8_t *packed) {
  const int wpt = 8 / bits;
  const int64_t G = (N + wpt - 1) / wpt;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < G; g++) {
    for (int64_t d = 0; d < D; d++) {
      uint8_t acc = 0;
      for (int ni = 0; ni < wpt; ni++) {
        int64_t n = g * wpt + ni;
        if (n >= N) break;
        int64_t id = n * D + d;
        int32_t v = quant_code(x[id], mn[n], scale[n], noise[id], use_fma);
        acc |= (uint8_t)((uint32_t)v << (ni * bits));
      }
      packed[g * D + d] = acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------------
 * unpack_single_precision.  quantization_cuda_kernel.cu:167-184:
 *   unpacked[n*D+d] = (float)((byte >> (ni*bits)) & (2^bits-1)) / scale[n] + min[n]
 * IEEE fp32 division, then fp32 addition.
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_unpack(const uint8_t *packed, const float *scale, const float *mn, int64_t N,
                        int64_t D, int bits, float *out) {
  const int wpt = 8 / bits;
  const int mask = (1 << bits) - 1;
  const int64_t G = (N + wpt - 1) / wpt;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < G; g++) {
    for (int ni = 0; ni < wpt; ni++) {
      int64_t n = g * wpt + ni;
      if (n >= N) break;
      const float s = scale[n], m = mn[n];
      for (int64_t d = 0; d < D; d++) {
        int v = (packed[g * D + d] >> (ni * bits)) & mask;
        float q = (float)v / s;
        out[n * D + d] = q + m;
      }
    }
  }
}

/* ------------------------------------------------------------------------------------------------
 * quantize_activation for fp32 input.  exact/exact/ops.py:69-83 -> 20-43: row stats, pack with the
 * fp32 stats, return scale and min rounded to bf16.   dequantize_activation, ops.py:86-98: widen
 * the bf16 stats to fp32 and unpack with THOSE (not with the fp32 values pack used).
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_quantize_activation(const float *x, const float *noise, int64_t N, int64_t D,
                                     int bits, int use_fma, uint8_t *packed, uint16_t *scale_bf16,
                                     uint16_t *min_bf16, float *scale_f32, float *min_f32) {
  float *mn = (float *)malloc(sizeof(float) * (size_t)N);
  float *mx = (float *)malloc(sizeof(float) * (size_t)N);
  float *sc = (float *)malloc(sizeof(float) * (size_t)N);
  orc_row_stats(x, N, D, bits, mn, mx, sc);
  orc_pack(x, mn, sc, noise, N, D, bits, use_fma, packed);
  for (int64_t n = 0; n < N; n++) {
    scale_bf16[n] = f32_to_bf16(sc[n]);
    min_bf16[n] = f32_to_bf16(mn[n]);
    if (scale_f32) scale_f32[n] = sc[n];
    if (min_f32) min_f32[n] = mn[n];
  }
  free(mn);
  free(mx);
  free(sc);
}

/* ------------------------------------------------------------------------------------------------
 * fp16 activations: the half instantiations of the same kernels (dispatch at
 * quantization_cuda_kernel.cu:132, 209).  With scalar_t = c10::Half every Half (op) Half is computed in
 * fp32 and rounded back to half (c10/util/Half-inl.h), Half + float is a float, so
 *   pack    (quantization_cuda_kernel.cu:89)   t = half(half(x - min) * scale);
 *                                              code = rint(max(float(t) + noise - 0.5, 0))
 *   unpack  (quantization_cuda_kernel.cu:182)  out = half(half(float(code) / scale) + min)
 * and the statistics of an fp16 activation stay fp16 (exact/exact/ops.py:82-83) and come from half tensor
 * ops (ops.py:63, 39): mn = min_d x; scale = half(float(half(1 / float(half(mx - mn)))) * (2^bits - 1)).
 * Halves travel as their bit patterns (uint16).
 * ---------------------------------------------------------------------------------------------- */
static inline float h2f(uint16_t b) {
  _Float16 h;
  memcpy(&h, &b, 2);
  return (float)h;
}
static inline uint16_t f2h(float f) {
  _Float16 h = (_Float16)f; /* round to nearest even */
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

ORC_API void orc_row_stats_f16(const uint16_t *x, int64_t N, int64_t D, int bits, uint16_t *mn,
                               uint16_t *scale) {
  const float B = (float)((1 << bits) - 1);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const uint16_t *r = x + n * D;
    float lo = h2f(r[0]), hi = lo;
    int nan = isnan(lo);
    for (int64_t d = 1; d < D; d++) {
      float v = h2f(r[d]);
      if (isnan(v)) nan = 1;
      if (v < lo) lo = v;
      if (v > hi) hi = v;
    }
    if (nan) lo = hi = NAN;
    float diff = h2f(f2h(hi - lo));
    float rcp = h2f(f2h(1.0f / diff));
    mn[n] = f2h(lo);
    scale[n] = f2h(rcp * B);
  }
}

ORC_API void orc_pack_f16(const uint16_t *x, const uint16_t *mn, const uint16_t *scale, const float *noise,
                          int64_t N, int64_t D, int bits, uint8_t *packed) {
  const int wpt = 8 / bits;
  const int64_t G = (N + wpt - 1) / wpt;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < G; g++) {
    for (int64_t d = 0; d < D; d++) {
      uint8_t acc = 0;
      for (int ni = 0; ni < wpt; ni++) {
        int64_t n = g * wpt + ni;
        if (n >= N) break;
        int64_t id = n * D + d;
        float t1 = h2f(f2h(h2f(x[id]) - h2f(mn[n])));
        float t2 = h2f(f2h(t1 * h2f(scale[n])));
        double t = (double)(t2 + noise[id]) - 0.5;
        float tf = (float)fmax(t, 0.0); /* fmax(NaN, 0) = 0 */
        int32_t v = float2int_rn(tf);
        acc |= (uint8_t)((uint32_t)v << (ni * bits));
      }
      packed[g * D + d] = acc;
    }
  }
}

ORC_API void orc_unpack_f16(const uint8_t *packed, const uint16_t *scale, const uint16_t *mn, int64_t N,
                            int64_t D, int bits, uint16_t *out) {
  const int wpt = 8 / bits;
  const int mask = (1 << bits) - 1;
  const int64_t G = (N + wpt - 1) / wpt;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < G; g++) {
    for (int ni = 0; ni < wpt; ni++) {
      int64_t n = g * wpt + ni;
      if (n >= N) break;
      const float s = h2f(scale[n]), m = h2f(mn[n]);
      for (int64_t d = 0; d < D; d++) {
        int v = (packed[g * D + d] >> (ni * bits)) & mask;
        float q = h2f(f2h((float)v / s));
        out[n * D + d] = f2h(q + m);
      }
    }
  }
}

ORC_API void orc_dequantize_activation(const uint8_t *packed, const uint16_t *scale_bf16,
                                       const uint16_t *min_bf16, int64_t N, int64_t D, int bits,
                                       float *out) {
  float *mn = (float *)malloc(sizeof(float) * (size_t)N);
  float *sc = (float *)malloc(sizeof(float) * (size_t)N);
  for (int64_t n = 0; n < N; n++) {
    sc[n] = bf16_to_f32(scale_bf16[n]);
    mn[n] = bf16_to_f32(min_bf16[n]);
  }
  orc_unpack(packed, sc, mn, N, D, bits, out);
  free(mn);
  free(sc);
}

/* ------------------------------------------------------------------------------------------------
 * Philox4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11).
 * Used twice: (1) to regenerate the noise the reference's pack kernel draws from cuRAND, so that the
 * reference's own binary output can be compared bit for bit; (2) as the restatement of the
 * production noise of the CUDA library (see orc_noise_b200).
 * ---------------------------------------------------------------------------------------------- */
static inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                 uint32_t k1, uint32_t out[4]) {
  for (int r = 0; r < 10; r++) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

ORC_API void orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  philox4x32_10(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1], out);
}

/* The noise stream of the reference's pack kernel.  quantization_cuda_kernel.cu:78-88: thread
 * (group g, column d) calls curand_init(seed, subsequence = g*D + d, offset) and then draws
 * curand_uniform once per row of its group, in row order.  cuRAND's documented Philox layout: key =
 * seed, counter words 2..3 = subsequence, counter words 0..1 = offset / 4, and the (offset % 4)-th
 * 32-bit output is the first one returned; successive draws walk through the four outputs and then
 * bump the counter.  curand_uniform maps a 32-bit draw r to r * 2^-32 + 2^-33, in (0, 1]. */
ORC_API void orc_noise_reference_pack(uint64_t seed, uint64_t offset, int64_t N, int64_t D, int bits,
                                      float *noise) {
  const int wpt = 8 / bits;
  const int64_t G = (N + wpt - 1) / wpt;
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < G; g++) {
    for (int64_t d = 0; d < D; d++) {
      uint64_t sub = (uint64_t)(g * D + d);
      for (int ni = 0; ni < wpt; ni++) {
        int64_t n = g * wpt + ni;
        if (n >= N) break;
        uint64_t pos = offset + (uint64_t)ni;
        uint64_t blk = pos >> 2;
        uint32_t out[4];
        philox4x32_10((uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)sub, (uint32_t)(sub >> 32), k0,
                      k1, out);
        uint32_t r = out[pos & 3];
        noise[n * D + d] = fmaf((float)r, 2.3283064365386963e-10f, 1.1641532182693481e-10f);
      }
    }
  }
}

/* Production noise of the B200 library (no reference counterpart: the reference draws from torch's
 * global generator).  One Philox4x32-10 call serves a pair of columns of an 8-row tile with 8 bits per
 * element: call index q = (n/8) * ceil(D/2) + d/2, counter = (q_lo, q_hi, offset_lo, offset_hi), key = seed;
 * element (n, d) takes byte 2 * (n%8) + d%2 of the 16 output bytes (byte b = bits 8*(b%4).. of word b/4);
 * u = (h + 0.5) * 2^-8, in (0, 1).  n is the GLOBAL row index (row_offset + local row). */
ORC_API void orc_noise_b200(uint64_t seed, uint64_t offset, int64_t row_offset, int64_t N, int64_t D,
                            float *noise) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const int64_t Dh = (D + 1) / 2;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    int64_t gn = n + row_offset;
    for (int64_t d = 0; d < D; d++) {
      uint64_t q = (uint64_t)((gn >> 3) * Dh + (d >> 1));
      uint32_t out[4];
      philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)offset, (uint32_t)(offset >> 32), k0,
                    k1, out);
      int b = (int)(gn & 7) * 2 + (int)(d & 1);
      uint32_t h = (out[b >> 2] >> (8 * (b & 3))) & 0xffu;
      noise[n * D + d] = ((float)h + 0.5f) * 0.00390625f;
    }
  }
}

/* Noise of the B200 library's fused projection+pack kernel, whose epilogue threads own rows: one
 * Philox call per (global row, block of 8 columns), q = n * ceil(k/8) + c/8; element (n, c) takes
 * word (c%8)/2, low half for even c. */
ORC_API void orc_noise_b200_rows(uint64_t seed, uint64_t offset, int64_t row_offset, int64_t N, int64_t k,
                                 float *noise) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const int64_t CB8 = (k + 7) / 8;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    int64_t gn = n + row_offset;
    for (int64_t cb = 0; cb < CB8; cb++) {
      uint64_t q = (uint64_t)(gn * CB8 + cb);
      uint32_t out[4];
      philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), (uint32_t)offset, (uint32_t)(offset >> 32), k0, k1, out);
      for (int j = 0; j < 8 && cb * 8 + j < k; j++) {
        uint32_t w = out[j >> 1];
        uint32_t h = (j & 1) ? (w >> 16) : (w & 0xffffu);
        noise[n * k + cb * 8 + j] = ((float)h + 0.5f) * 1.52587890625e-05f;
      }
    }
  }
}

/* Production dropout uniforms of the B200 library: one Philox call per 8 consecutive elements,
 * counter = (i/8 lo, i/8 hi, offset lo, offset hi); element i takes the 16-bit field i % 8 of the 128-bit block
 * (word (i % 8) / 2, low half first), u = (h + 0.5) * 2^-16 in (0, 1). */
ORC_API void orc_uniform_b200(uint64_t seed, uint64_t offset, int64_t n, float *u) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma omp parallel for schedule(static)
  for (int64_t q = 0; q < (n + 7) / 8; q++) {
    uint32_t out[4];
    philox4x32_10((uint32_t)q, (uint32_t)((uint64_t)q >> 32), (uint32_t)offset,
                  (uint32_t)(offset >> 32), k0, k1, out);
    for (int j = 0; j < 8 && q * 8 + j < n; j++) {
      uint32_t h = (out[j >> 1] >> (16 * (j & 1))) & 0xffffu;
      u[q * 8 + j] = fmaf((float)h, 1.52587890625e-05f, 7.62939453125e-06f);
    }
  }
}

/* ------------------------------------------------------------------------------------------------
 * act_quantized_relu.  quantization_cuda_kernel.cu:243-267 (fw), 298-309 (bw): out = x > 0 ? x : 0,
 * one mask bit per element (x > 0); grad_in = bit ? grad_out : 0.  The mask never leaves the
 * extension (quantization.cc:71), so only its content per element is restated: keep[i] in {0,1}.
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_relu_fw(const float *x, int64_t n, float *out, uint8_t *keep) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    int bit = x[i] > 0.0f;
    out[i] = bit ? x[i] : 0.0f;
    keep[i] = (uint8_t)bit;
  }
}
ORC_API void orc_mask_bw(const float *g, const uint8_t *keep, int64_t n, float *gin) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) gin[i] = keep[i] ? g[i] : 0.0f;
}

/* ------------------------------------------------------------------------------------------------
 * act_quantized_dropout.  quantization_cuda_kernel.cu:450-506: keep = u > p with u in (0,1];
 * pinv = (float)(1.0 / (1.0 - (double)p)); out = (x * keep) * pinv  (two fp32 multiplies).
 * Backward, :557-570 with p1m = (float)(1.0 - (double)p) (quantization.cc:120,126):
 * grad_in = keep ? grad_out / p1m : 0   (IEEE division).
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_dropout_fw(const float *x, const float *u, float p, int64_t n, float *out,
                            uint8_t *keep) {
  const float pinv = (float)(1.0 / (1.0 - (double)p));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    float k = (u[i] > p) ? 1.0f : 0.0f;
    float t = x[i] * k;
    out[i] = t * pinv;
    keep[i] = (uint8_t)(k != 0.0f);
  }
}
ORC_API void orc_dropout_bw(const float *g, const uint8_t *keep, float p, int64_t n, float *gin) {
  const float p1m = (float)(1.0 - (double)p);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) gin[i] = keep[i] ? g[i] / p1m : 0.0f;
}

/* The seeded Rademacher matrix of the B200 library (stands in for gen_rad_mat, ops.py:112-114, which
 * draws from torch's global generator): sign i of the row-major [D,k] matrix is bit i%128 of the
 * Philox block with counter (i/128, offset); entries are +-(float)(1/sqrt(k)). */
ORC_API void orc_rademacher(uint64_t seed, uint64_t offset, int64_t D, int64_t k, float *out) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  const float mag = (float)(1.0 / sqrt((double)k));
  const int64_t n = D * k;
  for (int64_t q = 0; q < (n + 127) / 128; q++) {
    uint32_t w[4];
    philox4x32_10((uint32_t)q, (uint32_t)((uint64_t)q >> 32), (uint32_t)offset, (uint32_t)(offset >> 32),
                  k0, k1, w);
    for (int b = 0; b < 128 && q * 128 + b < n; b++)
      out[q * 128 + b] = ((w[b >> 5] >> (b & 31)) & 1u) ? mag : -mag;
  }
}

/* ------------------------------------------------------------------------------------------------
 * Random projection.  exact/exact/ops.py:107-118 input2rp: R[D,k] = (2*bern - 1) / sqrt(k), out =
 * x @ R.  ops.py:121-125 rp2input: x_hat = xq @ R^T.  The reference calls cuBLAS SGEMM whose
 * summation order is unspecified; the restatement accumulates in double and rounds once, i.e. it is
 * the correctly rounded product the 1e-2 relative-Frobenius criterion is measured against.
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_input2rp(const float *x, const float *R, int64_t N, int64_t D, int64_t k,
                          float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    double acc[512];
    for (int64_t j0 = 0; j0 < k; j0 += 512) {
      int64_t jb = (k - j0 < 512) ? (k - j0) : 512;
      for (int64_t j = 0; j < jb; j++) acc[j] = 0.0;
      for (int64_t d = 0; d < D; d++) {
        double xv = x[n * D + d];
        const float *r = R + d * k + j0;
        for (int64_t j = 0; j < jb; j++) acc[j] += xv * (double)r[j];
      }
      for (int64_t j = 0; j < jb; j++) out[n * k + j0 + j] = (float)acc[j];
    }
  }
}
ORC_API void orc_rp2input(const float *xq, const float *R, int64_t N, int64_t D, int64_t k,
                          float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    for (int64_t d = 0; d < D; d++) {
      double acc = 0.0;
      for (int64_t j = 0; j < k; j++) acc += (double)xq[n * k + j] * (double)R[d * k + j];
      out[n * D + d] = (float)acc;
    }
  }
}

/* ------------------------------------------------------------------------------------------------
 * CSR SpMM, reduce = sum (0) or mean (1).  exact/exact/cpp_extension/spmm_cuda.cu:54-103 with
 * reducer.cuh:55-84: edges of a row are accumulated in CSR order in fp32,
 *   result = result + val[e] * mat[col[e], c]      (one FMA under nvcc's default contraction),
 * mean divides the sum by max(row_end - row_start, 1) (edge values do not change the divisor).
 * val == NULL means all ones.  Index arrays are int64.
 * The backward pass (spmm.cc:57-79, 115-139) is this same function on the transposed structure
 * (colptr, row[csr2csc], weights) and is composed in Python.
 * ---------------------------------------------------------------------------------------------- */
ORC_API void orc_spmm(const int64_t *rowptr, const int64_t *col, const float *val, const float *mat,
                      int64_t M, int64_t K, int reduce, float *out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < M; r++) {
    float *o = out + r * K;
    for (int64_t c = 0; c < K; c++) o[c] = 0.0f;
    for (int64_t e = rowptr[r]; e < rowptr[r + 1]; e++) {
      const float *m = mat + col[e] * K;
      if (val) {
        const float v = val[e];
        for (int64_t c = 0; c < K; c++) o[c] = fmaf(v, m[c], o[c]);
      } else {
        for (int64_t c = 0; c < K; c++) o[c] = o[c] + m[c];
      }
    }
    if (reduce == 1) {
      int64_t cnt = rowptr[r + 1] - rowptr[r];
      float dv = (float)(cnt > 0 ? cnt : 1);
      for (int64_t c = 0; c < K; c++) o[c] = o[c] / dv;
    }
  }
}

/* CSR SpMM on halves: the reference's half instantiation (spmm_cuda.cu:142; operands cast to fp16 by
 * exact/exact/ops.py:260, 313 under AMP).  Every Half (op) Half is an fp32 operation rounded back to half
 * (spmm_cuda.cu:83-92, reducer.cuh:53-60, 72-77):
 *   term = half(val[e] * mat[col[e], c]) (the bare operand without edge values);
 *   result = half(result + term) in CSR order from 0;  mean: out = half(result / half(max(count, 1))). */
ORC_API void orc_spmm_f16(const int64_t *rowptr, const int64_t *col, const uint16_t *val, const uint16_t *mat,
                          int64_t M, int64_t K, int reduce, uint16_t *out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < M; r++) {
    int64_t cnt = rowptr[r + 1] - rowptr[r];
    float dv = h2f(f2h((float)(cnt > 0 ? cnt : 1)));
    for (int64_t c = 0; c < K; c++) {
      float acc = 0.0f;
      for (int64_t e = rowptr[r]; e < rowptr[r + 1]; e++) {
        float m = h2f(mat[col[e] * K + c]);
        if (val) m = h2f(f2h(h2f(val[e]) * m));
        acc = h2f(f2h(acc + m));
      }
      if (reduce == 1) acc = h2f(f2h(acc / dv));
      out[r * K + c] = f2h(acc);
    }
  }
}

/* spmm_value_bw.  spmm_cuda.cu:172-209: one warp per edge; lane l accumulates val += mat[col, k] * grad[row, k]
 * for k = l, l + 32, ... (one FMA each: nvcc contracts the mul+add), then the lanes are added by
 * val += shfl_down(val, i) for i = 16, 8, 4, 2, 1 (lane 0 holds the result; lanes beyond 31 - i add the value
 * of their own lane, which lane 0 never sees), and mean divides by max(row length, 1). */
ORC_API void orc_spmm_value_bw(const int64_t *row, const int64_t *rowptr, const int64_t *col, const float *mat,
                               const float *grad, int64_t E, int64_t K, int mean, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t e = 0; e < E; e++) {
    float lane[32];
    const float *m = mat + col[e] * K, *g = grad + row[e] * K;
    for (int l = 0; l < 32; l++) {
      float v = 0.0f;
      for (int64_t k = l; k < K; k += 32) v = fmaf(m[k], g[k], v);
      lane[l] = v;
    }
    for (int i = 16; i > 0; i >>= 1)
      for (int l = 0; l < i; l++) lane[l] = lane[l] + lane[l + i];
    float val = lane[0];
    if (mean) {
      int64_t deg = rowptr[row[e] + 1] - rowptr[row[e]];
      val = val / (float)(deg > 1 ? deg : 1);
    }
    out[e] = val;
  }
}

/* spmm_kernel with REDUCE = MAX / MIN.  spmm_cuda.cu:54-103 + reducer.cuh:43-85: val starts at lowest() / max(),
 * an edge replaces it only when strictly greater / smaller (so the first edge of a tie wins), its position is
 * kept in arg; rows without edges write 0 and arg = nnz (spmm_cuda.cu:152: arg_out is filled with col.numel()). */
ORC_API void orc_spmm_minmax(const int64_t *rowptr, const int64_t *col, const float *val, const float *mat,
                             int64_t M, int64_t K, int64_t nnz, int is_max, float *out, int64_t *arg_out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < M; r++) {
    for (int64_t c = 0; c < K; c++) {
      float best = is_max ? -3.402823466e+38f : 3.402823466e+38f;
      int64_t arg = nnz;
      for (int64_t e = rowptr[r]; e < rowptr[r + 1]; e++) {
        float v = mat[col[e] * K + c];
        if (val) v = val[e] * v;
        if (is_max ? (v > best) : (v < best)) { best = v; arg = e; }
      }
      int has = rowptr[r + 1] > rowptr[r];
      out[r * K + c] = has ? best : 0.0f;
      arg_out[r * K + c] = has ? arg : nnz;
    }
  }
}
