// 1-bit-mask activations: ReLU and dropout that keep one bit per element for backward.
//
// Replaces quantization.act_quantized_relu / act_quantized_leaky_relu / act_quantized_dropout
// (exact/exact/cpp_extension/quantization.cc:66-134; kernels quantization_cuda_kernel.cu:237-594).
//
// One bit per element, 32-bit words: word 8c + j, bit l holds element 256c + 8l + j (see the forward kernel).  The
// layout is private: the reference's mask never leaves its extension either (quantization.cc:71,92,119), only
// outputs and gradients are observable.
#include "common.cuh"
#include <cmath>
#include <cuda_fp16.h>

#include "exact_b200.h"

namespace exb {

enum MaskOp { OP_RELU = 0, OP_DROPOUT = 1, OP_RELU_DROPOUT = 2, OP_LEAKY_RELU = 3 };

struct MaskParams {
  const void* x;        // forward input or grad_out, fp32 or fp16 (the kernels' element type)
  const float* u;       // supplied uniforms (dropout forward) or null
  void* out;            // output or grad_in, same type as x
  uint32_t* mask;
  long long n;
  float p;              // dropout probability; the negative slope for LeakyReLU
  float pinv;           // float(1 / (1 - p))
  float p1m;            // float(1 - p)
  float p1m_inv_exact;  // 1 / p1m when p1m is a power of two (then g / p1m == g * that, bit for bit), else 0
  uint32_t off_lo, off_hi;
  unsigned long long q0;  // Philox block index of element 0 (global element index / 8)
  PhiloxKey key;
};

template <bool ALIGNED>
__device__ __forceinline__ void load4(const float* base, long long i, long long n, float (&v)[4]) {
  if (ALIGNED && i + 4 <= n) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(base + i));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = (i + j < n) ? __ldcs(base + i + j) : 0.f;
  }
}
template <bool ALIGNED>
__device__ __forceinline__ void store4(float* base, long long i, long long n, const float (&v)[4]) {
  if (ALIGNED && i + 4 <= n) {
    __stcs(reinterpret_cast<float4*>(base + i), make_float4(v[0], v[1], v[2], v[3]));
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++)
      if (i + j < n) __stcs(base + i + j, v[j]);
  }
}
// fp16 elements (the reference's half instantiations, quantization_cuda_kernel.cu:284, 324, 387, 428, 535, 586):
// Half (op) float is computed in fp32 there and the result rounded once when it is stored, so the kernels
// below do the same fp32 arithmetic on widened values and round on the store.
template <bool ALIGNED>
__device__ __forceinline__ void load4(const __half* base, long long i, long long n, float (&v)[4]) {
  if (ALIGNED && i + 4 <= n) {
    const uint2 t = __ldcs(reinterpret_cast<const uint2*>(base + i));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = (i + j < n) ? __half2float(base[i + j]) : 0.f;
  }
}
template <bool ALIGNED>
__device__ __forceinline__ void store4(__half* base, long long i, long long n, const float (&v)[4]) {
  if (ALIGNED && i + 4 <= n) {
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    __stcs(reinterpret_cast<uint2*>(base + i), t);
  } else {
#pragma unroll
    for (int j = 0; j < 4; j++)
      if (i + j < n) base[i + j] = __float2half_rn(v[j]);
  }
}

// Forward: a warp handles 256 consecutive elements per step, a lane eight of them (two 4-element vector loads);
// eight __ballot_sync calls turn the 256 predicates into eight mask words: word 8c + j, bit l = element 256c + 8l + j.
// Dropout draws one Philox4x32-10 block per lane and step: 128 bits = eight 16-bit uniforms (h + 0.5) / 65536, keyed
// by the global index of the lane's first element / 8.  (32-bit uniforms, one block per four elements, made the
// Philox rounds the largest share of the instructions: 66 % of the copy peak for ReLU + dropout.)
template <int OP, bool ALIGNED, typename T>
__global__ void __launch_bounds__(256) mask_forward_kernel(const __grid_constant__ MaskParams p) {
  const int lane = threadIdx.x & 31;
  const long long nchunks = (p.n + 255) >> 8;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long c = warp0; c < nchunks; c += nwarps) {
    const long long i = (c << 8) + 8 * lane;
    float v[8], o[8];
    bool keep[8];
    {
      float a[4], b[4];
      load4<ALIGNED>(static_cast<const T*>(p.x), i, p.n, a);
      load4<ALIGNED>(static_cast<const T*>(p.x), i + 4, p.n, b);
#pragma unroll
      for (int j = 0; j < 4; j++) { v[j] = a[j]; v[4 + j] = b[j]; }
    }
    if (OP == OP_RELU) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        keep[j] = v[j] > 0.f;           // quantization_cuda_kernel.cu:253
        o[j] = keep[j] ? v[j] : 0.f;
      }
    } else if (OP == OP_LEAKY_RELU) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        keep[j] = v[j] > 0.f;           // quantization_cuda_kernel.cu:356-361
        o[j] = keep[j] ? v[j] : __fmul_rn(v[j], p.p);
      }
    } else {
      if (OP == OP_RELU_DROPOUT) {
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = v[j] > 0.f ? v[j] : 0.f;   // the ReLU that precedes the dropout
      }
      float u[8];
      if (p.u != nullptr) {
        float a[4], b[4];
        load4<ALIGNED>(p.u, i, p.n, a);
        load4<ALIGNED>(p.u, i + 4, p.n, b);
#pragma unroll
        for (int j = 0; j < 4; j++) { u[j] = a[j]; u[4 + j] = b[j]; }
      } else {
        const unsigned long long q = p.q0 + (unsigned long long)((c << 5) + lane);  // global element index / 8
        uint32_t w[4];
        philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const uint32_t h = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
          u[j] = __fmaf_rn((float)h, 1.52587890625e-05f, 7.62939453125e-06f);   // (h + 0.5) / 65536, exact
        }
      }
#pragma unroll
      for (int j = 0; j < 8; j++) {
        keep[j] = (u[j] > p.p) && (i + j < p.n);  // quantization_cuda_kernel.cu:466-469
        // quantization_cuda_kernel.cu:490: src * keep * pinv, two fp32 multiplies
        o[j] = __fmul_rn(__fmul_rn(v[j], keep[j] ? 1.f : 0.f), p.pinv);
        // one mask serves both backward passes: the gradient survives where the ReLU passed and the
        // dropout kept
        if (OP == OP_RELU_DROPOUT) keep[j] = keep[j] && v[j] > 0.f;
      }
    }
    {
      const float a[4] = {o[0], o[1], o[2], o[3]}, b[4] = {o[4], o[5], o[6], o[7]};
      store4<ALIGNED>(static_cast<T*>(p.out), i, p.n, a);
      store4<ALIGNED>(static_cast<T*>(p.out), i + 4, p.n, b);
    }
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const uint32_t w = __ballot_sync(0xffffffffu, keep[j]);
      if (lane == j) p.mask[(c << 3) + j] = w;
    }
  }
}

template <int OP, bool ALIGNED, typename T>
__global__ void __launch_bounds__(256) mask_backward_kernel(const __grid_constant__ MaskParams p) {
  const int lane = threadIdx.x & 31;
  const long long nchunks = (p.n + 255) >> 8;
  const long long warp0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long c = warp0; c < nchunks; c += nwarps) {
    const long long i = (c << 8) + 8 * lane;
    float g[8], o[8];
    {
      float a[4], b[4];
      load4<ALIGNED>(static_cast<const T*>(p.x), i, p.n, a);
      load4<ALIGNED>(static_cast<const T*>(p.x), i + 4, p.n, b);
#pragma unroll
      for (int j = 0; j < 4; j++) { g[j] = a[j]; g[4 + j] = b[j]; }
    }
    const uint4 m0 = __ldg(reinterpret_cast<const uint4*>(p.mask) + 2 * c);
    const uint4 m1 = __ldg(reinterpret_cast<const uint4*>(p.mask) + 2 * c + 1);
    const uint32_t m[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const bool keep = (m[j] >> lane) & 1u;
      if (OP == OP_RELU) {
        o[j] = keep ? g[j] : 0.f;                      // quantization_cuda_kernel.cu:303-308
      } else if (OP == OP_LEAKY_RELU) {
        o[j] = keep ? g[j] : __fmul_rn(g[j], p.p);     // quantization_cuda_kernel.cu:408-412
      } else {
        // quantization_cuda_kernel.cu:565-569: g / float(1 - p); a power-of-two divisor (p = 0.5, 0.75, ...)
        // is an exact scaling, done as one multiply
        const float q = p.p1m_inv_exact != 0.f ? __fmul_rn(g[j], p.p1m_inv_exact) : __fdiv_rn(g[j], p.p1m);
        o[j] = keep ? q : 0.f;
      }
    }
    const float a[4] = {o[0], o[1], o[2], o[3]}, b[4] = {o[4], o[5], o[6], o[7]};
    store4<ALIGNED>(static_cast<T*>(p.out), i, p.n, a);
    store4<ALIGNED>(static_cast<T*>(p.out), i + 4, p.n, b);
  }
}

static bool aligned16(const void* a) { return (reinterpret_cast<uintptr_t>(a) & 15) == 0; }

static bool aligned_to(const void* a, unsigned bytes) { return (reinterpret_cast<uintptr_t>(a) & (bytes - 1)) == 0; }

template <int OP, typename T = float>
static int launch_mask(bool forward, const MaskParams& p, cudaStream_t st) {
  if (p.n == 0) return EXB_OK;
  EXB_REQUIRE(p.x && p.out && p.mask, "mask activation: null pointer");
  EXB_REQUIRE(aligned16(p.mask), "mask activation: mask must be 16-byte aligned");
  const unsigned vb = 4 * sizeof(T);   // one 4-element vector access
  const bool al = aligned_to(p.x, vb) && aligned_to(p.out, vb) && (p.u == nullptr || aligned16(p.u));
  const long long nchunks = (p.n + 255) >> 8;
  long long blocks = (nchunks + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (forward) {
    if (al) mask_forward_kernel<OP, true, T><<<(int)blocks, 256, 0, st>>>(p);
    else mask_forward_kernel<OP, false, T><<<(int)blocks, 256, 0, st>>>(p);
  } else {
    if (al) mask_backward_kernel<OP, true, T><<<(int)blocks, 256, 0, st>>>(p);
    else mask_backward_kernel<OP, false, T><<<(int)blocks, 256, 0, st>>>(p);
  }
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

static void dropout_constants(MaskParams& p, float prob) {
  p.p = prob;
  p.pinv = (float)(1.0 / (1.0 - (double)prob));  // quantization_cuda_kernel.cu:455
  p.p1m = (float)(1.0 - (double)prob);           // quantization.cc:120
  int ex = 0;
  const float mant = frexpf(p.p1m, &ex);   // p1m = mant * 2^ex, mant in [0.5, 1)
  p.p1m_inv_exact = (p.p1m > 0.f && mant == 0.5f && ex > -120 && ex < 120) ? ldexpf(1.f, 1 - ex) : 0.f;
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_mask_words(int64_t n) { return n <= 0 ? 0 : ((n + 255) / 256) * 8; }

int exact_act_quantized_relu_forward(const float* x, int64_t n, float* out, uint32_t* mask, void* stream) {
  EXB_REQUIRE(n >= 0, "relu: negative size");
  MaskParams p{};
  p.x = x; p.out = out; p.mask = mask; p.n = n;
  return launch_mask<OP_RELU>(true, p, (cudaStream_t)stream);
}

int exact_act_quantized_relu_backward(const float* grad_out, const uint32_t* mask, int64_t n,
                                      float* grad_in, void* stream) {
  EXB_REQUIRE(n >= 0, "relu: negative size");
  MaskParams p{};
  p.x = grad_out; p.out = grad_in; p.mask = const_cast<uint32_t*>(mask); p.n = n;
  return launch_mask<OP_RELU>(false, p, (cudaStream_t)stream);
}

int exact_act_quantized_leaky_relu_forward(const float* x, int64_t n, float slope, float* out, uint32_t* mask,
                                           void* stream) {
  EXB_REQUIRE(n >= 0, "leaky_relu: negative size");
  MaskParams p{};
  p.x = x; p.out = out; p.mask = mask; p.n = n; p.p = slope;
  return launch_mask<OP_LEAKY_RELU>(true, p, (cudaStream_t)stream);
}

int exact_act_quantized_leaky_relu_backward(const float* grad_out, const uint32_t* mask, int64_t n, float slope,
                                            float* grad_in, void* stream) {
  EXB_REQUIRE(n >= 0, "leaky_relu: negative size");
  MaskParams p{};
  p.x = grad_out; p.out = grad_in; p.mask = const_cast<uint32_t*>(mask); p.n = n; p.p = slope;
  return launch_mask<OP_LEAKY_RELU>(false, p, (cudaStream_t)stream);
}

int exact_act_quantized_dropout_forward(const float* x, int64_t n, float prob, const float* uniforms,
                                        uint64_t seed, uint64_t offset, int64_t index_offset, float* out,
                                        uint32_t* mask, void* stream) {
  EXB_REQUIRE(n >= 0, "dropout: negative size");
  EXB_REQUIRE(index_offset >= 0 && index_offset % 8 == 0, "dropout: index_offset must be a non-negative multiple of 8");
  EXB_REQUIRE(prob >= 0.f && prob <= 1.f, "dropout: p must be in [0, 1] (got %f)", (double)prob);
  MaskParams p{};
  p.x = x; p.u = uniforms; p.out = out; p.mask = mask; p.n = n;
  p.p = prob;
  p.pinv = (float)(1.0 / (1.0 - (double)prob));  // quantization_cuda_kernel.cu:455
  p.p1m = (float)(1.0 - (double)prob);
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.q0 = (unsigned long long)index_offset >> 3;
  p.key = make_philox_key(seed);
  return launch_mask<OP_DROPOUT>(true, p, (cudaStream_t)stream);
}

int exact_act_quantized_relu_dropout_forward(const float* x, int64_t n, float prob, const float* uniforms,
                                             uint64_t seed, uint64_t offset, int64_t index_offset, float* out,
                                             uint32_t* mask, void* stream) {
  EXB_REQUIRE(n >= 0, "relu_dropout: negative size");
  EXB_REQUIRE(index_offset >= 0 && index_offset % 8 == 0, "relu_dropout: index_offset must be a non-negative multiple of 8");
  EXB_REQUIRE(prob >= 0.f && prob <= 1.f, "relu_dropout: p must be in [0, 1] (got %f)", (double)prob);
  MaskParams p{};
  p.x = x; p.u = uniforms; p.out = out; p.mask = mask; p.n = n;
  p.p = prob;
  p.pinv = (float)(1.0 / (1.0 - (double)prob));  // quantization_cuda_kernel.cu:455
  p.p1m = (float)(1.0 - (double)prob);
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.q0 = (unsigned long long)index_offset >> 3;
  p.key = make_philox_key(seed);
  return launch_mask<OP_RELU_DROPOUT>(true, p, (cudaStream_t)stream);
}

int exact_act_quantized_dropout_backward(const float* grad_out, const uint32_t* mask, int64_t n,
                                         float prob, float* grad_in, void* stream) {
  EXB_REQUIRE(n >= 0, "dropout: negative size");
  MaskParams p{};
  p.x = grad_out; p.out = grad_in; p.mask = const_cast<uint32_t*>(mask); p.n = n;
  p.p = prob;
  p.p1m = (float)(1.0 - (double)prob);  // quantization.cc:120
  {
    int ex = 0;
    const float mant = frexpf(p.p1m, &ex);   // p1m = mant * 2^ex, mant in [0.5, 1)
    p.p1m_inv_exact = (p.p1m > 0.f && mant == 0.5f && ex > -120 && ex < 120) ? ldexpf(1.f, 1 - ex) : 0.f;
  }
  return launch_mask<OP_DROPOUT>(false, p, (cudaStream_t)stream);
}

int exact_act_quantized_forward_f16(int op, const void* x, int64_t n, float param, const float* uniforms, uint64_t seed,
                                    uint64_t offset, int64_t index_offset, void* out, uint32_t* mask, void* stream) {
  EXB_REQUIRE(n >= 0, "act_quantized_f16: negative size");
  EXB_REQUIRE(op >= EXACT_ACT_RELU && op <= EXACT_ACT_LEAKY_RELU, "act_quantized_f16: unknown op %d", op);
  MaskParams p{};
  p.x = x; p.out = out; p.mask = mask; p.n = n; p.p = param;
  cudaStream_t st = (cudaStream_t)stream;
  if (op == EXACT_ACT_RELU) return launch_mask<OP_RELU, __half>(true, p, st);
  if (op == EXACT_ACT_LEAKY_RELU) return launch_mask<OP_LEAKY_RELU, __half>(true, p, st);
  EXB_REQUIRE(index_offset >= 0 && index_offset % 8 == 0, "dropout: index_offset must be a non-negative multiple of 8");
  EXB_REQUIRE(param >= 0.f && param <= 1.f, "dropout: p must be in [0, 1] (got %f)", (double)param);
  p.u = uniforms;
  dropout_constants(p, param);
  p.off_lo = (uint32_t)offset; p.off_hi = (uint32_t)(offset >> 32);
  p.q0 = (unsigned long long)index_offset >> 3;
  p.key = make_philox_key(seed);
  if (op == EXACT_ACT_DROPOUT) return launch_mask<OP_DROPOUT, __half>(true, p, st);
  return launch_mask<OP_RELU_DROPOUT, __half>(true, p, st);
}

int exact_act_quantized_backward_f16(int op, const void* grad_out, const uint32_t* mask, int64_t n, float param,
                                     void* grad_in, void* stream) {
  EXB_REQUIRE(n >= 0, "act_quantized_f16: negative size");
  EXB_REQUIRE(op >= EXACT_ACT_RELU && op <= EXACT_ACT_LEAKY_RELU, "act_quantized_f16: unknown op %d", op);
  MaskParams p{};
  p.x = grad_out; p.out = grad_in; p.mask = const_cast<uint32_t*>(mask); p.n = n; p.p = param;
  cudaStream_t st = (cudaStream_t)stream;
  if (op == EXACT_ACT_RELU) return launch_mask<OP_RELU, __half>(false, p, st);
  if (op == EXACT_ACT_LEAKY_RELU) return launch_mask<OP_LEAKY_RELU, __half>(false, p, st);
  dropout_constants(p, param);
  return launch_mask<OP_DROPOUT, __half>(false, p, st);   // also the backward of ReLU + dropout (one mask)
}

}  // extern "C"
