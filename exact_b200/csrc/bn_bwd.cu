// Batch-norm backward straight from the packed input.
//
// The reference's qbatch_norm.backward (exact/exact/ops.py:235-253) dequantises the saved input into a
// full [N, D] fp32 tensor (dequantize_activation, ops.py:86-98 -> quantization_cuda_kernel.cu:158-185) and
// hands it to native_batch_norm_backward, which reads it twice (the column sums, then the element-wise
// pass).  Here both passes read the packed bytes and the row statistics instead and dequantise in
// registers (code / scale + min, IEEE, the arithmetic of quantization_cuda_kernel.cu:182): the [N, D]
// reconstruction never exists, and the backward moves 12 N D bytes instead of 24 N D.
//
//   pass 1  bn_bwd_sums_kernel      per column d: sum_n g[n, d] and sum_n g[n, d] (x[n, d] - mean[d]); every CTA
//                                   writes its partial sums, bn_bwd_finish_kernel adds them in CTA order (no float
//                                   atomics: results are run-to-run identical) and forms
//                                   grad_bias = sum g, grad_weight = invstd * sum g (x - mean);
//   pass 2  bn_bwd_apply_kernel     training: grad_in = (g - sum_g / N - (x - mean) * invstd^2 * sum_gx / N) * invstd * w
//                                   eval:     grad_in = g * invstd * w
//
// A thread owns four adjacent columns (one 32-bit word of the packed stream = those columns of 8 / bits
// consecutive rows) and walks down the rows, so its per-column constants stay in registers and every access
// is a 16-byte piece of a row.
#include "exact_b200.h"
#include "common.cuh"

namespace exb {

constexpr int kBnThreads = 256;

struct BnBwdParams {
  const float* g;
  const uint8_t* packed;
  const uint16_t* scale_bf16;
  const uint16_t* min_bf16;
  const float* weight;   // or null (ones)
  const float* mean;
  const float* invstd;
  float* partial;        // [grid, 2, D]
  float* sums;           // [2, D]: sum g, sum g (x - mean)
  float* grad_in;
  float* grad_weight;    // or null
  float* grad_bias;      // or null
  long long N;
  int D, cg_total, cg, ry, training;
  long long groups;      // ceil(N / (8 / bits))
};

// code / s + m, IEEE: by the correctly rounded reciprocal when s is an ordinary number (equal to the quotient
// for every code 0..255 and 2^-100 <= |s| <= 2^100), by the division otherwise (inf of a constant row, NaN,
// denormals).
__device__ __forceinline__ float dequant_one(uint32_t code, float s, float rcp, float m, bool tame) {
  const float c = (float)code;
  if (tame) {
    const float q0 = __fmul_rn(c, rcp);
    const float q = __fmaf_rn(__fmaf_rn(-q0, s, c), rcp, q0);
    return __fadd_rn(q, m);
  }
  return __fadd_rn(__fdiv_rn(c, s), m);
}

template <int BITS, bool APPLY>
__global__ void __launch_bounds__(kBnThreads) bn_bwd_kernel(const __grid_constant__ BnBwdParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  __shared__ float s_red[APPLY ? 1 : kBnThreads * 8];
  const int tx = threadIdx.x % p.cg, ty = threadIdx.x / p.cg;
  const bool active = ty < p.ry;
  for (int cg0 = 0; cg0 < p.cg_total; cg0 += p.cg) {
    const int cgi = cg0 + tx;
    const bool col_ok = active && cgi < p.cg_total;
    const int d = cgi * 4;
    float mean[4] = {0.f, 0.f, 0.f, 0.f}, k2[4] = {0.f, 0.f, 0.f, 0.f}, k1[4] = {0.f, 0.f, 0.f, 0.f},
          gs[4] = {0.f, 0.f, 0.f, 0.f};
    if (col_ok) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        mean[c] = p.mean[d + c];
        if (APPLY) {
          const float is = p.invstd[d + c];
          gs[c] = __fmul_rn(is, p.weight ? p.weight[d + c] : 1.f);
          if (p.training) {
            const float inv_n = 1.f / (float)p.N;
            k1[c] = __fmul_rn(p.sums[d + c], inv_n);
            k2[c] = __fmul_rn(__fmul_rn(p.sums[p.D + d + c], inv_n), __fmul_rn(is, is));
          }
        }
      }
    }
    float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_gx[4] = {0.f, 0.f, 0.f, 0.f};
    if (col_ok) {
      for (long long grp = (long long)blockIdx.x * p.ry + ty; grp < p.groups; grp += (long long)gridDim.x * p.ry) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(p.packed + grp * p.D + d));
        const long long n0 = grp * WPT;
        float4 gv[WPT];
        float s[WPT], m[WPT];
#pragma unroll
        for (int i = 0; i < WPT; i++) {
          const long long n = n0 + i;
          if (n < p.N) {
            gv[i] = __ldcs(reinterpret_cast<const float4*>(p.g + n * p.D + d));
            s[i] = bf16_bits_to_f32(__ldg(p.scale_bf16 + n));
            m[i] = bf16_bits_to_f32(__ldg(p.min_bf16 + n));
          } else {
            gv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            s[i] = 1.f;
            m[i] = 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < WPT; i++) {
          const long long n = n0 + i;
          if (n >= p.N) break;
          const uint32_t sexp = (__float_as_uint(s[i]) >> 23) & 0xffu;
          const bool tame = sexp >= 27u && sexp <= 227u;
          const float rcp = __frcp_rn(s[i]);
          const float gg[4] = {gv[i].x, gv[i].y, gv[i].z, gv[i].w};
          float o[4];
#pragma unroll
          for (int c = 0; c < 4; c++) {
            const uint32_t code = ((w >> (8 * c)) >> (i * BITS)) & MASK;
            const float xc = __fsub_rn(dequant_one(code, s[i], rcp, m[i], tame), mean[c]);
            if (APPLY) {
              o[c] = p.training ? __fmul_rn(__fsub_rn(__fsub_rn(gg[c], k1[c]), __fmul_rn(xc, k2[c])), gs[c])
                                : __fmul_rn(gg[c], gs[c]);
            } else {
              acc_g[c] = __fadd_rn(acc_g[c], gg[c]);
              acc_gx[c] = __fmaf_rn(gg[c], xc, acc_gx[c]);
            }
          }
          if (APPLY) __stcs(reinterpret_cast<float4*>(p.grad_in + n * p.D + d), make_float4(o[0], o[1], o[2], o[3]));
        }
      }
    }
    if (!APPLY) {
      // add the row lanes of each column group in lane order, one partial row per CTA
      float* mine = s_red + threadIdx.x * 8;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        mine[c] = acc_g[c];
        mine[4 + c] = acc_gx[c];
      }
      __syncthreads();
      if (ty == 0 && cgi < p.cg_total) {
        float tg[4] = {0.f, 0.f, 0.f, 0.f}, tgx[4] = {0.f, 0.f, 0.f, 0.f};
        for (int y = 0; y < p.ry; y++) {
          const float* o = s_red + (y * p.cg + tx) * 8;
#pragma unroll
          for (int c = 0; c < 4; c++) {
            tg[c] = __fadd_rn(tg[c], o[c]);
            tgx[c] = __fadd_rn(tgx[c], o[4 + c]);
          }
        }
        float* dst = p.partial + (long long)blockIdx.x * 2 * p.D;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          dst[d + c] = tg[c];
          dst[p.D + d + c] = tgx[c];
        }
      }
      __syncthreads();
    }
  }
}

__global__ void bn_bwd_finish_kernel(const float* __restrict__ partial, int n_partial, int D, const float* __restrict__ invstd,
                                     float* __restrict__ sums, float* __restrict__ grad_weight, float* __restrict__ grad_bias) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float a = 0.f, b = 0.f;
  for (int i = 0; i < n_partial; i++) {
    a = __fadd_rn(a, partial[(long long)i * 2 * D + d]);
    b = __fadd_rn(b, partial[(long long)i * 2 * D + D + d]);
  }
  sums[d] = a;
  sums[D + d] = b;
  if (grad_bias) grad_bias[d] = a;
  if (grad_weight) grad_weight[d] = __fmul_rn(b, invstd[d]);
}

static int bn_grid(long long groups, int ry) {
  long long want = (groups + ry - 1) / ry;
  long long cap = (long long)sm_count() * 8;
  if (want > cap) want = cap;
  return (int)(want < 1 ? 1 : want);
}

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_bn_backward_workspace_bytes(int64_t D) {
  if (D <= 0) return 256;
  return 256 + ((int64_t)sm_count() * 8 + 1) * 2 * D * 4;
}

int exact_bn_backward_from_packed(const float* grad_out, int64_t N, int64_t D, const uint8_t* packed, int bits,
                                  const uint16_t* scale_bf16, const uint16_t* min_bf16, const float* weight,
                                  const float* mean, const float* invstd, int training, void* workspace,
                                  int64_t workspace_bytes, float* grad_input, float* grad_weight, float* grad_bias,
                                  void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && D > 0, "bn_backward_from_packed: bad shape");
  if (D % 4 != 0 || D > (1 << 20))
    return fail(EXB_ERR_UNSUPPORTED, "bn_backward_from_packed: D = %lld is not a multiple of 4", (long long)D);
  EXB_REQUIRE(grad_out && packed && scale_bf16 && min_bf16 && mean && invstd && workspace,
              "bn_backward_from_packed: null pointer");
  EXB_REQUIRE(workspace_bytes >= exact_bn_backward_workspace_bytes(D), "bn_backward_from_packed: workspace too small");
  EXB_REQUIRE(((reinterpret_cast<uintptr_t>(grad_out) | reinterpret_cast<uintptr_t>(grad_input)) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(packed) & 3) == 0 && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0,
              "bn_backward_from_packed: grad_out / grad_input must be 16-byte, packed 4-byte, workspace 256-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  BnBwdParams p{};
  p.g = grad_out; p.packed = packed; p.scale_bf16 = scale_bf16; p.min_bf16 = min_bf16; p.weight = weight;
  p.mean = mean; p.invstd = invstd; p.grad_in = grad_input; p.grad_weight = grad_weight; p.grad_bias = grad_bias;
  p.N = N; p.D = (int)D; p.training = training != 0;
  p.cg_total = (int)(D / 4);
  p.cg = p.cg_total < 64 ? p.cg_total : 64;
  p.ry = kBnThreads / p.cg;
  const int wpt = 8 / bits;
  p.groups = (N + wpt - 1) / wpt;
  p.sums = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
  p.partial = p.sums + 2 * D;
  const int grid = bn_grid(p.groups, p.ry);
#define EXB_BN_LAUNCH(BITS_, APPLY_) bn_bwd_kernel<BITS_, APPLY_><<<grid, kBnThreads, 0, st>>>(p)
#define EXB_BN_SWITCH(APPLY_)                  \
  switch (bits) {                              \
    case 1: EXB_BN_LAUNCH(1, APPLY_); break;   \
    case 2: EXB_BN_LAUNCH(2, APPLY_); break;   \
    case 4: EXB_BN_LAUNCH(4, APPLY_); break;   \
    default: EXB_BN_LAUNCH(8, APPLY_); break;  \
  }
  const bool need_sums = grad_weight || grad_bias || (grad_input && p.training);
  if (need_sums) {
    EXB_BN_SWITCH(false)
    EXB_CUDA_OK(cudaGetLastError());
    bn_bwd_finish_kernel<<<(unsigned)((D + 127) / 128), 128, 0, st>>>(p.partial, grid, (int)D, invstd, p.sums, grad_weight,
                                                                     grad_bias);
    EXB_CUDA_OK(cudaGetLastError());
  }
  if (grad_input && N > 0) {
    EXB_BN_SWITCH(true)
    EXB_CUDA_OK(cudaGetLastError());
  }
#undef EXB_BN_SWITCH
#undef EXB_BN_LAUNCH
  return EXB_OK;
}

}  // extern "C"
