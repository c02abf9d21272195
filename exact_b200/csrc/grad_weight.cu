// Weight gradient of a quantised linear layer straight from the packed activation:
//     G[O, k] = g^T [O x N] . dequantise(packed) [N x k]
// the product grad_output.t().mm(input) of linear_backward (exact/exact/cpp_extension/backward_func.cc:87)
// with `input` still in the form qlinear.forward saved it (exact/exact/ops.py:149-154), so that the chain
// dequantize_activation -> mm of ops.py:164-169 needs neither the [N, k] fp32 activation in HBM nor a
// second pass over g.  Up to two packed activations (the two inputs of a GraphSAGE layer, which share g:
// layers.py:163-170) are multiplied in one pass; the result holds their column blocks side by side.  The
// caller applies the transposed projection to the small result: (g^T Xq) R^T.
//
// Shape of the work.  N is the number of nodes (millions), O <= 256, k <= 128: 2 N O k flop against
// 4 N O bytes of g, so the kernel is bound by reading g once; the tensor core makes the multiply-adds
// free.  The contraction runs over node rows, which are the slow dimension of both operands:
//   A = g^T   arrives by TMA as [32 rows x 32 columns] boxes of g (128-byte swizzle): 32 consecutive
//             outputs of one node row are contiguous, i.e. the tile is MN-major for the MMA (descriptor with
//             leading-dimension offset = one box, instruction descriptor with the transpose-A bit);
//   B = Xq    is produced K-major by four warps that read the packed bytes (one byte = 8/bits consecutive
//             node rows of one column, which is one 16-byte chunk of the tile at INT2) and the bf16 row
//             statistics, dequantise (code / scale + min) and store to the swizzled tile.
// Each CTA owns a contiguous range of 32-row blocks and accumulates its partial G in TMEM over the whole
// range (split over node rows across the SMs); partials go to the workspace and a second kernel adds them
// in CTA order, so the result does not depend on timing.  tf32 inputs, fp32 accumulation: about 5e-4
// relative on G, far below the quantisation noise of the activation it is computed from.
//
// Every mbarrier wait is bounded; on expiry the CTA abandons its range, frees TMEM and raises the status words.
#include <mutex>

#include "exact_b200.h"
#include "tc.cuh"

namespace exb {

constexpr int kGwRows = 32;          // node rows per pipeline stage (= the K extent of a stage)
constexpr int kGwThreads = 192;      // warp 0 TMA, warp 1 MMA, warps 2-5 producers of B and epilogue
constexpr int kGwMaxStages = 6;
constexpr int kGwMaxSeg = 2;

struct GwSegment {
  const uint8_t* packed;
  const uint16_t* scale_bf16;
  const uint16_t* min_bf16;
  int k;        // columns of this packed activation
  int col0;     // first column of its block in the result
};

struct GwParams {
  GwSegment seg[kGwMaxSeg];
  int nseg;
  float* partial;     // [grid, Opad, kpad]
  int* status;
  int* lib_status;
  long long N;
  int O, Opad, kpad, bits;
  int mtiles;         // Opad / 128
  int oblocks;        // ceil(O / 32): boxes of g per stage
  long long kblocks;  // ceil(N / 32)
  int stages;
  unsigned a_bytes, b_bytes, stage_bytes, tmem_cols;
};

// MN-major operand tile, 128-byte swizzle: blocks of 32 contiguous MN elements (128 bytes) x 8 K rows are
// 1024 bytes; K groups of 8 rows follow each other (stride 1024), blocks along MN are `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

__device__ __forceinline__ void gw_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int BITS>
__global__ void __launch_bounds__(kGwThreads, 1)
grad_weight_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ GwParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  constexpr int GROUPS = kGwRows / WPT;     // packed bytes per column and stage
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_full[kGwMaxStages];
  __shared__ __align__(8) unsigned long long s_empty[kGwMaxStages];
  __shared__ __align__(8) unsigned long long s_done;
  // row statistics of the stage a producer warp works on and of the next one: a private copy per warp, so the
  // producers need no barrier among themselves
  __shared__ float s_scale[2][4][kGwMaxSeg][kGwRows];
  __shared__ float s_min[2][4][kGwMaxSeg][kGwRows];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_base - smem_u32(smem_raw));
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&s_full[s]), 5);    // the TMA thread's bytes + one arrival per producer warp
      mbar_init(smem_u32(&s_empty[s]), 1);   // tcgen05.commit
    }
    mbar_init(smem_u32(&s_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
  // B rows that hold no column of any activation stay zero for the whole kernel
  for (int s = 0; s < p.stages; s++) {
    uint4* b = reinterpret_cast<uint4*>(tiles_ptr + (size_t)s * p.stage_bytes + p.a_bytes);
    for (unsigned i = threadIdx.x; i < p.b_bytes / 16; i += kGwThreads) b[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  gw_fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;

  // this CTA's range of 32-row blocks
  const long long per = (p.kblocks + gridDim.x - 1) / gridDim.x;
  const long long kb0 = (long long)blockIdx.x * per;
  const long long kb1 = kb0 + per < p.kblocks ? kb0 + per : p.kblocks;
  const long long nblk = kb1 > kb0 ? kb1 - kb0 : 0;

  if (warp == 0) {
    // ---------------- TMA producer of A = g^T ----------------
    if (lane == 0) {
      bool ok = true;
      long long it = 0;
      for (; it < nblk && ok; it++) {
        const int s = (int)(it % p.stages);
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t full = smem_u32(&s_full[s]);
        const uint32_t dst = tiles_base + (uint32_t)s * p.stage_bytes;
        mbar_arrive_expect_tx(full, (uint32_t)p.oblocks * (kGwRows * 128));
        const int row = (int)((kb0 + it) * kGwRows);
        for (int ob = 0; ob < p.oblocks; ob++) tma_load_2d(dst + (uint32_t)ob * (kGwRows * 128), &tm_g, ob * 32, row, full);
      }
      if (!ok) {
        const long long t0 = clock64();
        for (int j = 0; j < p.stages && j < it; j++) {
          const long long jt = it - 1 - j;
          const uint32_t bar = smem_u32(&s_full[jt % p.stages]);
          const uint32_t ph = (uint32_t)(jt / p.stages) & 1u;
          while (!mbar_try_wait(bar, ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      // transpose-A bit (15): A is MN-major
      const uint32_t idesc = umma_idesc_tf32(128, p.kpad) | (1u << 15);
      bool ok = true;
      for (long long it = 0; it < nblk && ok; it++) {
        const int s = (int)(it % p.stages);
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_full[s]), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = tiles_base + (uint32_t)s * p.stage_bytes;
        const uint64_t b_desc = umma_desc_sw128(a_addr + p.a_bytes);
        for (int mt = 0; mt < p.mtiles; mt++) {
          // four boxes (32 outputs each) make the 128 rows of one M tile
          const uint64_t a_desc = umma_desc_mn_sw128(a_addr + (uint32_t)mt * 4u * (kGwRows * 128), kGwRows * 128);
#pragma unroll
          for (int k8 = 0; k8 < kGwRows / 8; k8++) {
            // A: the next 8 node rows are 1024 bytes further; B: 8 tf32 = 32 bytes along its 128-byte rows
            umma_tf32(tmem_base + (uint32_t)(mt * p.kpad), a_desc + (uint64_t)(k8 * 64), b_desc + (uint64_t)(k8 * 2), idesc,
                      (it | k8) != 0);
          }
        }
        umma_commit(smem_u32(&s_empty[s]));
      }
      if (ok) umma_commit(smem_u32(&s_done));
    }
  } else {
    // ---------------- producers of B = dequantised activation (warps 2..5), then the epilogue ----------------
    const int t = threadIdx.x - 64;            // 0 .. 127
    bool ok = true;
    // items of a stage: (segment, column j, byte group q); thread t takes items t, t + 128, ...
    int total_items = 0;
    for (int sg = 0; sg < p.nseg; sg++) total_items += p.seg[sg].k * GROUPS;
    constexpr int kMaxItems = 8;               // per thread and stage: k_total * GROUPS <= 1024
    uint32_t bytes_next[kMaxItems];
    auto item_of = [&](int idx, int& sg, int& j, int& q) {
      sg = 0;
      int rest = idx;
      while (sg + 1 < p.nseg && rest >= p.seg[sg].k * GROUPS) { rest -= p.seg[sg].k * GROUPS; sg++; }
      q = rest / p.seg[sg].k;                  // consecutive threads take consecutive columns: coalesced bytes
      j = rest - q * p.seg[sg].k;
    };
    auto load_items = [&](long long kb) {
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) {
        const int idx = t + i * 128;
        bytes_next[i] = 0u;
        if (idx < total_items) {
          int sg, j, q;
          item_of(idx, sg, j, q);
          const long long grp = kb * GROUPS + q;           // row group of the packed stream
          if (grp * WPT < p.N) bytes_next[i] = __ldg(p.seg[sg].packed + grp * p.seg[sg].k + j);
        }
      }
    };
    const int pw = warp - 2;                   // producer warp 0 .. 3
    auto load_stats = [&](long long kb, int buf) {
      const long long n = kb * kGwRows + lane;
      for (int sg = 0; sg < p.nseg; sg++) {
        float sc = 1.f, mn = 0.f;
        if (n < p.N) {
          sc = bf16_bits_to_f32(__ldg(p.seg[sg].scale_bf16 + n));
          mn = bf16_bits_to_f32(__ldg(p.seg[sg].min_bf16 + n));
        }
        s_scale[buf][pw][sg][lane] = sc;
        s_min[buf][pw][sg][lane] = mn;
      }
    };
    if (nblk > 0) {
      load_items(kb0);
      load_stats(kb0, 0);
    }
    for (long long it = 0; it < nblk && ok; it++) {
      const int s = (int)(it % p.stages);
      const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
      const int sb = (int)(it & 1);
      uint32_t bytes_cur[kMaxItems];
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) bytes_cur[i] = bytes_next[i];
      __syncwarp();                           // this warp's copy of the stage's statistics is in shared memory
      if (it + 1 < nblk) {                    // next stage's bytes and statistics are requested now
        load_items(kb0 + it + 1);
        load_stats(kb0 + it + 1, sb ^ 1);
      }
      // the same verdict in every lane, so that a warp leaves the loop as a whole
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag))) { ok = false; break; }
      uint8_t* btile = tiles_ptr + (size_t)s * p.stage_bytes + p.a_bytes;
      const long long n0 = (kb0 + it) * kGwRows;
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) {
        const int idx = t + i * 128;
        if (idx < total_items) {
          int sg, j, q;
          item_of(idx, sg, j, q);
          const int jb = p.seg[sg].col0 + j;          // row of the B tile
          float v[WPT];
#pragma unroll
          for (int w = 0; w < WPT; w++) {
            const int r = q * WPT + w;
            const float code = (float)((bytes_cur[i] >> (w * BITS)) & MASK);
            // quantization_cuda_kernel.cu:179-183: code / scale + min; rows past N contribute nothing
            v[w] = (n0 + r < p.N) ? __fadd_rn(__fdiv_rn(code, s_scale[sb][pw][sg][r]), s_min[sb][pw][sg][r]) : 0.f;
          }
          // element (jb, r) of the K-major tile: row jb, 16-byte chunk (r / 4) ^ (jb % 8), word r % 4
#pragma unroll
          for (int w0 = 0; w0 < WPT; w0 += 4) {
            const int r = q * WPT + w0;
            uint8_t* dst = btile + jb * 128 + ((((r >> 2) ^ (jb & 7))) << 4) + (r & 3) * 4;
            if (WPT >= 4) *reinterpret_cast<float4*>(dst) = make_float4(v[w0], v[w0 + 1 < WPT ? w0 + 1 : 0], v[w0 + 2 < WPT ? w0 + 2 : 0], v[w0 + 3 < WPT ? w0 + 3 : 0]);
            else if (WPT == 2) *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1 < WPT ? 1 : 0]);
            else *reinterpret_cast<float*>(dst) = v[0];
          }
        }
      }
      gw_fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_full[s]));
    }
    // ---------------- epilogue: this CTA's partial G to the workspace ----------------
    if (ok && nblk > 0) ok = __all_sync(0xffffffffu, mbar_wait<64>(smem_u32(&s_done), 0, abort_flag));
    if (ok) {
      tc_fence_after();
      const int quad = warp & 3;
      float* dst0 = p.partial + (size_t)blockIdx.x * p.Opad * p.kpad;
      for (int mt = 0; mt < p.mtiles; mt++) {
        const int o = mt * 128 + quad * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * p.kpad);
        for (int c0 = 0; c0 < p.kpad; c0 += 16) {
          float v[16];
          if (nblk > 0) {
            tmem_ld16(taddr + (uint32_t)c0, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = 0.f;
          }
          float4* d4 = reinterpret_cast<float4*>(dst0 + (size_t)o * p.kpad + c0);
#pragma unroll
          for (int j = 0; j < 4; j++) d4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
      }
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
    if (p.lib_status) atomicOr(p.lib_status, EXB_STATUS_GRAD_WEIGHT);
  }
}

// out[o, j] = sum over CTAs, in CTA order, of partial[cta, o, j]; also used to clear the status word first.
__global__ void grad_weight_reduce_kernel(const float* __restrict__ partial, int ctas, int O, int Opad, int kpad, int ldo,
                                          float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= O * kpad) return;
  const int o = i / kpad, j = i - o * kpad;
  float a = 0.f;
  for (int c = 0; c < ctas; c++) a = __fadd_rn(a, partial[((size_t)c * Opad + o) * kpad + j]);
  out[(size_t)o * ldo + j] = a;
}

__global__ void grad_weight_clear_status_kernel(int* status) { *status = 0; }

}  // namespace exb

using namespace exb;

extern "C" {

int64_t exact_grad_weight_workspace_bytes(int64_t O, int64_t k_total_padded, int max_ctas) {
  if (O <= 0 || k_total_padded <= 0 || max_ctas <= 0) return 256;
  const int64_t Opad = (O + 127) / 128 * 128;
  return 256 + (int64_t)max_ctas * Opad * k_total_padded * 4;
}

int exact_grad_weight_from_packed(const float* g, int64_t N, int64_t O, const uint8_t* packed0, const uint16_t* scale0,
                                  const uint16_t* min0, int64_t k0, const uint8_t* packed1, const uint16_t* scale1,
                                  const uint16_t* min1, int64_t k1, int bits, void* workspace, int64_t workspace_bytes,
                                  float* out, int64_t ldo, void* stream) {
  EXB_REQUIRE(bits == 1 || bits == 2 || bits == 4 || bits == 8, "bits must be 1, 2, 4 or 8 (got %d)", bits);
  EXB_REQUIRE(N >= 0 && O > 0 && k0 > 0 && k1 >= 0, "grad_weight_from_packed: bad shape");
  const int64_t k0pad = (k0 + 15) / 16 * 16;
  const int64_t kpad = k0pad + (k1 > 0 ? (k1 + 15) / 16 * 16 : 0);
  EXB_REQUIRE(ldo >= kpad, "grad_weight_from_packed: ldo must be at least %lld (the column blocks are padded to 16)", (long long)kpad);
  if (O % 4 != 0 || O > 256 || (reinterpret_cast<uintptr_t>(g) & 15) != 0)
    return fail(EXB_ERR_UNSUPPORTED, "grad_weight_from_packed: needs O %% 4 == 0, O <= 256 and a 16-byte aligned g (O = %lld)", (long long)O);
  if (kpad > 256 || (k0 + k1) * (32 / (8 / bits)) > 8 * 128)
    return fail(EXB_ERR_UNSUPPORTED, "grad_weight_from_packed: too many activation columns (k = %lld + %lld)", (long long)k0, (long long)k1);
  EXB_REQUIRE(g && packed0 && scale0 && min0 && workspace && out, "grad_weight_from_packed: null pointer");
  EXB_REQUIRE(k1 == 0 || (packed1 && scale1 && min1), "grad_weight_from_packed: null pointer in the second activation");
  EXB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "grad_weight_from_packed: workspace must be 256-byte aligned");
  EXB_REQUIRE(N / kGwRows < 2147483647LL, "grad_weight_from_packed: too many rows");
  cudaStream_t st = (cudaStream_t)stream;
  const int Opad = (int)((O + 127) / 128 * 128);
  int* status = reinterpret_cast<int*>(workspace);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);

  GwParams p{};
  p.seg[0] = GwSegment{packed0, scale0, min0, (int)k0, 0};
  p.nseg = 1;
  if (k1 > 0) {
    p.seg[1] = GwSegment{packed1, scale1, min1, (int)k1, (int)k0pad};
    p.nseg = 2;
  }
  p.partial = partial; p.status = status; p.lib_status = status_word_ptr();
  p.N = N; p.O = (int)O; p.Opad = Opad; p.kpad = (int)kpad; p.bits = bits;
  p.mtiles = Opad / 128;
  p.oblocks = (int)((O + 31) / 32);
  p.kblocks = (N + kGwRows - 1) / kGwRows;
  p.a_bytes = (unsigned)(p.mtiles * 4 * kGwRows * 128);     // whole M tiles, box by box
  p.b_bytes = (unsigned)(kpad * 128);
  p.stage_bytes = (p.a_bytes + p.b_bytes + 1023u) & ~1023u;
  int stages = (int)((200 * 1024) / p.stage_bytes);
  if (stages > kGwMaxStages) stages = kGwMaxStages;
  EXB_REQUIRE(stages >= 2, "grad_weight_from_packed: a pipeline stage does not fit twice in shared memory");
  p.stages = stages;
  unsigned cols = 32;
  while (cols < (unsigned)(p.mtiles * kpad)) cols <<= 1;
  p.tmem_cols = cols;
  long long grid = sm_count();
  if (grid > p.kblocks) grid = p.kblocks > 0 ? p.kblocks : 1;
  EXB_REQUIRE(workspace_bytes >= 256 + grid * (int64_t)Opad * kpad * 4,
              "grad_weight_from_packed: workspace of %lld bytes is too small (%lld needed)", (long long)workspace_bytes,
              (long long)(256 + grid * (int64_t)Opad * kpad * 4));

  grad_weight_clear_status_kernel<<<1, 1, 0, st>>>(status);
  EXB_CUDA_OK(cudaGetLastError());
  if (N > 0) {
    CUtensorMap tm_g;
    int rc = make_tensor_map_2d_f32(&tm_g, g, (unsigned long long)O, (unsigned long long)N, (unsigned long long)O * 4, 32, kGwRows);
    if (rc) return rc;
    const size_t dyn = (size_t)stages * p.stage_bytes + 1024;
#define EXB_GW_LAUNCH(BITS_)                                                                                  \
  {                                                                                                           \
    EXB_CUDA_OK(cudaFuncSetAttribute(grad_weight_kernel<BITS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn)); \
    grad_weight_kernel<BITS_><<<(unsigned)grid, kGwThreads, dyn, st>>>(tm_g, p);                              \
  }
    switch (bits) {
      case 1: EXB_GW_LAUNCH(1) break;
      case 2: EXB_GW_LAUNCH(2) break;
      case 4: EXB_GW_LAUNCH(4) break;
      default: EXB_GW_LAUNCH(8) break;
    }
#undef EXB_GW_LAUNCH
    EXB_CUDA_OK(cudaGetLastError());
  }
  const int total = (int)(O * kpad);
  grad_weight_reduce_kernel<<<(total + 255) / 256, 256, 0, st>>>(partial, N > 0 ? (int)grid : 0, (int)O, Opad, (int)kpad,
                                                                 (int)ldo, out);
  EXB_CUDA_OK(cudaGetLastError());
  return EXB_OK;
}

}  // extern "C"
