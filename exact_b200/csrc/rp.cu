// Random projection helpers: the seeded Rademacher matrix of input2rp
// (exact/exact/ops.py:107-118, gen_rad_mat at ops.py:112-114).
//
// The reference draws the signs with torch.randint from the global CUDA generator.  Here sign i of the
// row-major [D, k] matrix is bit (i % 128) of the Philox4x32-10 block with counter
// (i / 128, offset) and key `seed`, so every rank of a row-sharded run, and the CPU oracle,
// regenerate the same matrix from (seed, offset) alone.
#include "common.cuh"
#include "exact_b200.h"

namespace exb {

struct RademacherParams {
  float* out;
  long long n;     // D * k
  float mag;       // 1 / sqrt(k)
  uint32_t off_lo, off_hi;
  PhiloxKey key;
};

__global__ void __launch_bounds__(128) rademacher_kernel(const __grid_constant__ RademacherParams p) {
  // one thread per 32-sign word; four consecutive threads share a Philox block
  const long long word = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long i0 = word << 5;
  if (i0 >= p.n) return;
  const unsigned long long q = (unsigned long long)(word >> 2);
  uint32_t w[4];
  philox4x32_10((uint32_t)q, (uint32_t)(q >> 32), p.off_lo, p.off_hi, p.key, w);
  const uint32_t bits = w[word & 3];
#pragma unroll 4
  for (int b = 0; b < 32; b++) {
    if (i0 + b < p.n) p.out[i0 + b] = ((bits >> b) & 1u) ? p.mag : -p.mag;
  }
}

}  // namespace exb

using namespace exb;

extern "C" int exact_rademacher(uint64_t seed, uint64_t offset, int64_t D, int64_t k, float* out, void* stream) {
  EXB_REQUIRE(D >= 0 && k >= 0, "rademacher: negative shape");
  if (D == 0 || k == 0) return EXB_OK;
  EXB_REQUIRE(out != nullptr, "rademacher: null output");
  RademacherParams p;
  p.out = out;
  p.n = D * k;
  p.mag = (float)(1.0 / sqrt((double)k));
  p.off_lo = (uint32_t)offset;
  p.off_hi = (uint32_t)(offset >> 32);
  p.key = make_philox_key(seed);
  const long long words = (p.n + 31) / 32;
  rademacher_kernel<<<(unsigned)((words + 127) / 128), 128, 0, (cudaStream_t)stream>>>(p);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}
