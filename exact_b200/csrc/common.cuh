// Shared device helpers of the exact_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "exact_b200 kernels are written for sm_100a (B200) only"
#endif

namespace exb {

// ---- host-side error plumbing -------------------------------------------------------------------
enum Status : int {
  EXB_OK = 0,
  EXB_ERR_ARG = 1,       // bad argument (null pointer, unsupported bits / dtype / size, misalignment)
  EXB_ERR_CUDA = 2,      // a CUDA runtime call failed; see exact_last_error()
  EXB_ERR_UNSUPPORTED = 3,
  EXB_ERR_DEVICE = 4,    // a kernel reported a device-side status (bounded wait expired)
};

char* last_error_buf();  // thread-local, defined in capi.cu

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define EXB_CUDA_OK(expr)                                                                     \
  do {                                                                                        \
    cudaError_t _e = (expr);                                                                  \
    if (_e != cudaSuccess)                                                                    \
      return ::exb::fail(::exb::EXB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                 \
                         cudaGetErrorString(_e), __FILE__, __LINE__);                         \
  } while (0)

#define EXB_REQUIRE(cond, ...)                                                                \
  do {                                                                                        \
    if (!(cond)) return ::exb::fail(::exb::EXB_ERR_ARG, __VA_ARGS__);                         \
  } while (0)

int sm_count();  // cached multiProcessorCount of the current device (capi.cu)

// Device address of the library-wide status word on the current device (capi.cu), or null without a device.
// Kernels with bounded on-chip waits OR one of these codes into it when a wait expires; exact_status() reads it.
int* status_word_ptr();
enum DeviceStatusBits : int { EXB_STATUS_RP_PACK = 1, EXB_STATUS_UNPACK_RP = 2, EXB_STATUS_LINEAR = 4, EXB_STATUS_GRAD_WEIGHT = 8 };

// Round keys of Philox4x32-10 for a 64-bit seed; lives in kernel parameters (constant bank) so the
// per-round key XOR needs no register.
struct PhiloxKey {
  uint32_t rk[20];
};
inline PhiloxKey make_philox_key(uint64_t seed) {
  PhiloxKey k;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; r++) {
    k.rk[2 * r] = k0;
    k.rk[2 * r + 1] = k1;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return k;
}

#ifdef __CUDACC__
// ---- device helpers -----------------------------------------------------------------------------

// Philox4x32-10 (Salmon et al., SC'11).  Counter (c0..c3), round keys from the constant bank.
__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              const PhiloxKey& key, uint32_t (&out)[4]) {
#pragma unroll
  for (int r = 0; r < 10; r++) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ key.rk[2 * r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ key.rk[2 * r + 1];
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
  }
  out[0] = c0;
  out[1] = c1;
  out[2] = c2;
  out[3] = c3;
}

// 16-bit field h -> (h + 0.5) * 2^-16 in (0,1), without an int->float conversion:
// 0x3F800000 | (h << 7) is 1 + h*2^-16; subtracting (1 - 2^-17) is exact.
__device__ __forceinline__ float u16_lo_to_unit(uint32_t w) {
  return __uint_as_float(((w << 7) & 0x007fff80u) | 0x3f800000u) - 0.99999237060546875f;
}
__device__ __forceinline__ float u16_hi_to_unit(uint32_t w) {
  return __uint_as_float(((w >> 9) & 0x007fff80u) | 0x3f800000u) - 0.99999237060546875f;
}
// 32-bit draw r -> r * 2^-32 + 2^-33 in (0,1] (the usual "uniform excluding zero" map).
__device__ __forceinline__ float u32_to_unit(uint32_t r) {
  return __fmaf_rn((float)r, 2.3283064365386963e-10f, 1.1641532182693481e-10f);
}

// Two fp32 lanes in one 64-bit register and the paired arithmetic of sm_100 (each lane rounds exactly
// like the scalar instruction).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 f2_sub(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) {
  f32x2 r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 16-bit field of a Philox word -> the float 1 + h * 2^-23 (bits 0x3F80:h), by one byte permute.
// noise16_to_unit() turns a pair of those into (h + 0.5) * 2^-16 with one paired FMA:
// (1 + h 2^-23) * 128 - (128 - 2^-17), exact.
__device__ __forceinline__ float u16_lo_to_1p(uint32_t w) { return __uint_as_float(__byte_perm(w, 0x3f800000u, 0x7610)); }
__device__ __forceinline__ float u16_hi_to_1p(uint32_t w) { return __uint_as_float(__byte_perm(w, 0x3f800000u, 0x7632)); }
__device__ __forceinline__ f32x2 noise16_to_unit(f32x2 one_plus) {
  return f2_fma(one_plus, f2_pack(128.f, 128.f), f2_pack(-127.99999237060546875f, -127.99999237060546875f));
}

// Byte k (0..3, may be a run-time value) of a Philox word -> the float 1 + h * 2^-23 (bits 0x3F8000:h), by one
// byte permute; noise8_to_unit() turns those into (h + 0.5) * 2^-8 with one FMA:
// (1 + h 2^-23) * 2^15 - (2^15 - 2^-9), exact.
__device__ __forceinline__ float u8_to_1p(uint32_t w, uint32_t k) {
  return __uint_as_float(__byte_perm(w, 0x3f800000u, 0x7640u + k));
}
__device__ __forceinline__ f32x2 noise8_to_unit(f32x2 one_plus) {
  return f2_fma(one_plus, f2_pack(32768.f, 32768.f), f2_pack(-32767.998046875f, -32767.998046875f));
}
__device__ __forceinline__ float noise8_to_unit(float one_plus) {
  return __fmaf_rn(one_plus, 32768.f, -32767.998046875f);
}

// NaN-propagating min/max (torch.min / torch.max semantics) and their warp-wide forms.  redux.sync on
// f32 is an sm_100a instruction.
__device__ __forceinline__ float min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float redux_min_nan(float v, unsigned mask) {
  float r;
  asm volatile("redux.sync.min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "r"(mask));
  return r;
}
__device__ __forceinline__ float redux_max_nan(float v, unsigned mask) {
  float r;
  asm volatile("redux.sync.max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "r"(mask));
  return r;
}

// Named barrier over `nthreads` threads (a multiple of 32) of the CTA.
template <int ID>
__device__ __forceinline__ void named_barrier(int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(nthreads) : "memory");
}

// fp32 -> bf16 bits, round to nearest even, NaN -> 0x7FC0 (what Tensor.to(torch.bfloat16) produces).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) {
  return __uint_as_float(((uint32_t)h) << 16);
}

// Streaming (read-once / write-once) global accesses of 1, 2 or 4 elements.
template <typename T, int VEC>
struct Ld;
template <>
struct Ld<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[4]) {
    float4 v = __ldcs(reinterpret_cast<const float4*>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <>
struct Ld<float, 2> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[2]) {
    float2 v = __ldcs(reinterpret_cast<const float2*>(p));
    o[0] = v.x; o[1] = v.y;
  }
};
template <>
struct Ld<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float (&o)[1]) { o[0] = __ldcs(p); }
};
// bf16 stored as uint16_t bits; widening to fp32 is exact.
template <>
struct Ld<uint16_t, 4> {
  static __device__ __forceinline__ void load(const uint16_t* p, float (&o)[4]) {
    uint2 v = __ldcs(reinterpret_cast<const uint2*>(p));
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
  }
};
template <>
struct Ld<uint16_t, 2> {
  static __device__ __forceinline__ void load(const uint16_t* p, float (&o)[2]) {
    uint32_t v = __ldcs(reinterpret_cast<const uint32_t*>(p));
    o[0] = __uint_as_float(v << 16); o[1] = __uint_as_float(v & 0xffff0000u);
  }
};
template <>
struct Ld<uint16_t, 1> {
  static __device__ __forceinline__ void load(const uint16_t* p, float (&o)[1]) {
    o[0] = __uint_as_float(((uint32_t)__ldcs(p)) << 16);
  }
};

template <int VEC>
struct StBytes;
template <>
struct StBytes<4> {
  static __device__ __forceinline__ void store(uint8_t* p, const uint32_t (&b)[4]) {
    __stcs(reinterpret_cast<uint32_t*>(p), b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24));
  }
  static __device__ __forceinline__ void load(const uint8_t* p, uint32_t (&b)[4]) {
    uint32_t w = __ldcs(reinterpret_cast<const uint32_t*>(p));
    b[0] = w & 0xff; b[1] = (w >> 8) & 0xff; b[2] = (w >> 16) & 0xff; b[3] = w >> 24;
  }
};
template <>
struct StBytes<2> {
  static __device__ __forceinline__ void store(uint8_t* p, const uint32_t (&b)[2]) {
    __stcs(reinterpret_cast<uint16_t*>(p), (uint16_t)(b[0] | (b[1] << 8)));
  }
  static __device__ __forceinline__ void load(const uint8_t* p, uint32_t (&b)[2]) {
    uint32_t w = __ldcs(reinterpret_cast<const uint16_t*>(p));
    b[0] = w & 0xff; b[1] = (w >> 8) & 0xff;
  }
};
template <>
struct StBytes<1> {
  static __device__ __forceinline__ void store(uint8_t* p, const uint32_t (&b)[1]) {
    __stcs(p, (uint8_t)b[0]);
  }
  static __device__ __forceinline__ void load(const uint8_t* p, uint32_t (&b)[1]) { b[0] = __ldcs(p); }
};

template <int VEC>
struct StF32;
template <>
struct StF32<4> {
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3]));
  }
};
template <>
struct StF32<2> {
  static __device__ __forceinline__ void store(float* p, const float (&v)[2]) {
    __stcs(reinterpret_cast<float2*>(p), make_float2(v[0], v[1]));
  }
};
template <>
struct StF32<1> {
  static __device__ __forceinline__ void store(float* p, const float (&v)[1]) { __stcs(p, v[0]); }
};
#endif  // __CUDACC__

}  // namespace exb
