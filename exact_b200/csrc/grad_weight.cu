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
// free.  The contraction runs over node rows, which are the slow dimension of both operands in memory,
// while the MMA wants the contraction dimension contiguous in shared memory (K-major tiles):
//   A = g^T   [32 rows x O] boxes of g arrive by TMA (no swizzle) in a ring of raw stages; four converter
//             warps transpose them: a thread reads one output column of the box (conflict-free: the 32
//             lanes read 32 consecutive words of a row) and writes the 32 node rows of that output as one
//             128-byte row of the 128-byte-swizzled K-major tile (eight 16-byte stores);
//   B = Xq    is produced K-major by four warps that read the packed bytes (one byte = 8/bits consecutive
//             node rows of one column, which is one 16-byte chunk of the tile at INT2) and the bf16 row
//             statistics, dequantise (code / scale + min) and store to the swizzled tile.
// A tile whose contraction dimension is the slow one (MN-major) could be fed to tcgen05.mma directly by
// setting the transpose bit of the instruction descriptor; with tf32 operands and the 128-byte swizzle that
// TMA writes the unit returned zeros on this hardware, hence the transposition in shared memory.
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
constexpr int kGwThreads = 320;      // warp 0 TMA, warp 1 MMA, warps 2-5 producers of B and epilogue, 6-9 converters
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
  long long kblocks;  // ceil(N / 32)
  int raw_stages, stages;
  unsigned raw_bytes;                    // one raw box of g: 32 rows x O fp32, padded to 1024 bytes
  unsigned a_bytes, b_bytes, stage_bytes, tmem_cols;
};

__device__ __forceinline__ void gw_fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int BITS>
__global__ void __launch_bounds__(kGwThreads, 1)
grad_weight_kernel(const __grid_constant__ CUtensorMap tm_g, const __grid_constant__ GwParams p) {
  constexpr int WPT = 8 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  constexpr int GROUPS = kGwRows / WPT;     // packed bytes per column and stage
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) unsigned long long s_rfull[kGwMaxStages];    // raw box of g landed
  __shared__ __align__(8) unsigned long long s_rempty[kGwMaxStages];   // raw box transposed
  __shared__ __align__(8) unsigned long long s_full[kGwMaxStages];     // A^T and B of an MMA stage written
  __shared__ __align__(8) unsigned long long s_empty[kGwMaxStages];    // MMA stage read by the tensor core
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
  // layout of the dynamic shared memory: raw ring, then the MMA stages (A^T tiles, B tile)
  const uint32_t mma_off = (uint32_t)p.raw_stages * p.raw_bytes;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < p.raw_stages; s++) {
      mbar_init(smem_u32(&s_rfull[s]), 1);    // the TMA thread's bytes
      mbar_init(smem_u32(&s_rempty[s]), 4);   // one arrival per converter warp
    }
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&s_full[s]), 8);     // one arrival per producer warp and per converter warp
      mbar_init(smem_u32(&s_empty[s]), 1);    // tcgen05.commit
    }
    mbar_init(smem_u32(&s_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), p.tmem_cols);
  // B rows that hold no column of any activation stay zero for the whole kernel
  for (int s = 0; s < p.stages; s++) {
    uint4* b = reinterpret_cast<uint4*>(tiles_ptr + mma_off + (size_t)s * p.stage_bytes + p.a_bytes);
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
    // ---------------- TMA producer: raw boxes of g ----------------
    if (lane == 0) {
      bool ok = true;
      long long it = 0;
      for (; it < nblk && ok; it++) {
        const int s = (int)(it % p.raw_stages);
        const uint32_t ph = (uint32_t)(it / p.raw_stages) & 1u;
        if (!mbar_wait(smem_u32(&s_rempty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
        const uint32_t full = smem_u32(&s_rfull[s]);
        mbar_arrive_expect_tx(full, (uint32_t)(kGwRows * p.O * 4));
        tma_load_2d(tiles_base + (uint32_t)s * p.raw_bytes, &tm_g, 0, (int)((kb0 + it) * kGwRows), full);
      }
      if (!ok) {   // leave no bulk copy in flight
        const long long t0 = clock64();
        for (int j = 0; j < p.raw_stages && j < it; j++) {
          const long long jt = it - 1 - j;
          const uint32_t bar = smem_u32(&s_rfull[jt % p.raw_stages]);
          const uint32_t ph = (uint32_t)(jt / p.raw_stages) & 1u;
          while (!mbar_try_wait(bar, ph) && clock64() - t0 < kWaitLimitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_tf32(128, p.kpad);
      bool ok = true;
      for (long long it = 0; it < nblk && ok; it++) {
        const int s = (int)(it % p.stages);
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(smem_u32(&s_full[s]), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a_addr = tiles_base + mma_off + (uint32_t)s * p.stage_bytes;
        const uint64_t b_desc = umma_desc_sw128(a_addr + p.a_bytes);
        for (int mt = 0; mt < p.mtiles; mt++) {
          const uint64_t a_desc = umma_desc_sw128(a_addr + (uint32_t)mt * (128 * 128));
#pragma unroll
          for (int k8 = 0; k8 < kGwRows / 8; k8++)   // 8 tf32 = 32 bytes along the 128-byte rows of both tiles
            umma_tf32(tmem_base + (uint32_t)(mt * p.kpad), a_desc + (uint64_t)(k8 * 2), b_desc + (uint64_t)(k8 * 2), idesc,
                      (it | k8) != 0);
        }
        umma_commit(smem_u32(&s_empty[s]));
      }
      if (ok) umma_commit(smem_u32(&s_done));
    }
  } else if (warp >= 6) {
    // ---------------- converters (warps 6..9): raw box [32 rows x O] -> A^T tiles [128 outputs x 32 rows] ----------------
    const int t = threadIdx.x - 192;           // 0 .. 127: output within an M tile
    bool ok = true;
    for (long long it = 0; it < nblk; it++) {
      const int rs = (int)(it % p.raw_stages), s = (int)(it % p.stages);
      const uint32_t rph = (uint32_t)(it / p.raw_stages) & 1u, ph = (uint32_t)(it / p.stages) & 1u;
      // the same outcome in every lane, so that a warp leaves the loop as a whole
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_rfull[rs]), rph, abort_flag))) { ok = false; break; }
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag))) { ok = false; break; }
      const float* raw = reinterpret_cast<const float*>(tiles_ptr + (size_t)rs * p.raw_bytes);
      uint8_t* at = tiles_ptr + mma_off + (size_t)s * p.stage_bytes;
      for (int mt = 0; mt < p.mtiles; mt++) {
        const int o = mt * 128 + t;
        float v[kGwRows];
#pragma unroll
        for (int n = 0; n < kGwRows; n++) v[n] = o < p.O ? raw[n * p.O + o] : 0.f;
        uint8_t* row = at + (size_t)mt * (128 * 128) + t * 128;
#pragma unroll
        for (int c = 0; c < kGwRows / 4; c++)
          *reinterpret_cast<float4*>(row + ((c ^ (t & 7)) << 4)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      }
      gw_fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&s_rempty[rs]));
        mbar_arrive(smem_u32(&s_full[s]));
      }
    }
    (void)ok;
  } else {
    // ---------------- producers of B = dequantised activation (warps 2..5), then the epilogue ----------------
    const int t = threadIdx.x - 64;            // 0 .. 127
    bool ok = true;
    // Items of a stage: (segment, column j, byte group q); thread t takes items t, t + 128, ...  Everything
    // about an item that does not change from stage to stage is worked out once, here: a producer warp has
    // an SM sub-partition to itself, so every dependent instruction inside the loop costs its full latency.
    int total_items = 0;
    for (int sg = 0; sg < p.nseg; sg++) total_items += p.seg[sg].k * GROUPS;
    constexpr int kMaxItems = 8;               // per thread and stage: k_total * GROUPS <= 1024
    const uint8_t* src[kMaxItems];             // the item's byte of the first stage
    int stride[kMaxItems];                     // bytes from one stage to the next
    int boff[kMaxItems];                       // byte offset of the item's first element in the B tile
    int soff[kMaxItems];                       // offset of its first row's statistics in a warp's copy
    long long row1[kMaxItems];                 // first row of the item in stage 0, relative to kb0 * 32
    bool valid[kMaxItems];
#pragma unroll
    for (int i = 0; i < kMaxItems; i++) {
      const int idx = t + i * 128;
      valid[i] = idx < total_items;
      src[i] = nullptr; stride[i] = 0; boff[i] = 0; soff[i] = 0; row1[i] = 0;
      if (valid[i]) {
        int sg = 0, rest = idx;
        while (sg + 1 < p.nseg && rest >= p.seg[sg].k * GROUPS) { rest -= p.seg[sg].k * GROUPS; sg++; }
        const int q = rest / p.seg[sg].k;      // consecutive threads take consecutive columns: coalesced bytes
        const int j = rest - q * p.seg[sg].k;
        const int jb = p.seg[sg].col0 + j;     // row of the B tile
        const int r = q * WPT;                 // first node row of the item within the stage
        src[i] = p.seg[sg].packed + (kb0 * GROUPS + q) * (long long)p.seg[sg].k + j;
        stride[i] = GROUPS * p.seg[sg].k;
        // element (jb, r) of the K-major tile: row jb, 16-byte chunk (r / 4) ^ (jb % 8), word r % 4
        boff[i] = jb * 128 + ((((r >> 2) ^ (jb & 7))) << 4) + (r & 3) * 4;
        soff[i] = sg * kGwRows + r;
        row1[i] = r;
      }
    }
    const int pw = warp - 2;                   // producer warp 0 .. 3
    uint32_t bytes_next[kMaxItems];
    auto load_items = [&](long long it) {      // the packed bytes of stage kb0 + it
      const long long n0 = (kb0 + it) * kGwRows;
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) {
        bytes_next[i] = 0u;
        if (valid[i] && n0 + row1[i] < p.N) bytes_next[i] = __ldg(src[i] + it * stride[i]);
      }
    };
    // Row statistics travel the same way: requested one stage ahead into registers (lane = row), turned into
    // 1 / scale (so that a code is dequantised with one FMA; a constant row has scale = inf and reciprocal 0,
    // its codes are 0 anyway) and min in this warp's shared-memory copy when their stage begins.  Rows past N
    // get 0, 0.
    // (the loaded values are not touched before their stage begins: a warp issues in order, and the first
    // instruction that needs a load result would make it wait for the load)
    uint16_t scale_next[kGwMaxSeg], min_next[kGwMaxSeg];
    auto load_stats = [&](long long it) {
      const long long n = (kb0 + it) * kGwRows + lane;
#pragma unroll
      for (int sg = 0; sg < kGwMaxSeg; sg++) {
        scale_next[sg] = 0x7f80;               // scale = inf, min = 0: reciprocal 0
        min_next[sg] = 0;
        if (sg < p.nseg && n < p.N) {
          scale_next[sg] = __ldg(p.seg[sg].scale_bf16 + n);
          min_next[sg] = __ldg(p.seg[sg].min_bf16 + n);
        }
      }
    };
    if (nblk > 0) {
      load_items(0);
      load_stats(0);
    }
    for (long long it = 0; it < nblk && ok; it++) {
      const int s = (int)(it % p.stages);
      const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
      const int sb = (int)(it & 1);
      uint32_t bytes_cur[kMaxItems];
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) bytes_cur[i] = bytes_next[i];
#pragma unroll
      for (int sg = 0; sg < kGwMaxSeg; sg++) {
        if (sg < p.nseg) {
          s_scale[sb][pw][sg][lane] = __frcp_rn(bf16_bits_to_f32(scale_next[sg]));
          s_min[sb][pw][sg][lane] = bf16_bits_to_f32(min_next[sg]);
        }
      }
      __syncwarp();                           // this warp's copy of the stage's statistics is in shared memory
      if (it + 1 < nblk) {                    // next stage's bytes and statistics are requested now
        load_items(it + 1);
        load_stats(it + 1);
      }
      // the same outcome in every lane, so that a warp leaves the loop as a whole
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_empty[s]), ph ^ 1u, abort_flag))) { ok = false; break; }
      uint8_t* btile = tiles_ptr + mma_off + (size_t)s * p.stage_bytes + p.a_bytes;
      const float* inv_s = &s_scale[sb][pw][0][0];
      const float* min_s = &s_min[sb][pw][0][0];
#pragma unroll
      for (int i = 0; i < kMaxItems; i++) {
        if (valid[i]) {
          float v[WPT];
#pragma unroll
          for (int w = 0; w < WPT; w++) {
            const float code = (float)((bytes_cur[i] >> (w * BITS)) & MASK);
            // quantization_cuda_kernel.cu:179-183 (code / scale + min) as code * (1 / scale) + min
            v[w] = __fmaf_rn(code, inv_s[soff[i] + w], min_s[soff[i] + w]);
          }
          uint8_t* dst = btile + boff[i];
          if (WPT == 8) {
            // rows r .. r+7: two chunks of the same tile row; the second is the next chunk before swizzling
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1 % WPT], v[2 % WPT], v[3 % WPT]);
            uint8_t* row = btile + (boff[i] & ~127);
            const int chunk = ((boff[i] >> 4) & 7) ^ ((boff[i] >> 7) & 7);      // the un-swizzled chunk index
            *reinterpret_cast<float4*>(row + ((((chunk + 1) ^ ((boff[i] >> 7) & 7))) << 4)) =
                make_float4(v[4 % WPT], v[5 % WPT], v[6 % WPT], v[7 % WPT]);
          } else if (WPT == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1 % WPT], v[2 % WPT], v[3 % WPT]);
          } else if (WPT == 2) {
            *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1 % WPT]);
          } else {
            *reinterpret_cast<float*>(dst) = v[0];
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
  p.kblocks = (N + kGwRows - 1) / kGwRows;
  p.raw_bytes = ((unsigned)(kGwRows * O * 4) + 1023u) & ~1023u;
  p.a_bytes = (unsigned)(p.mtiles * 128 * 128);             // one [128 x 32] fp32 tile per M tile
  p.b_bytes = (unsigned)(kpad * 128);
  p.stage_bytes = (p.a_bytes + p.b_bytes + 1023u) & ~1023u;
  // two MMA stages are enough to keep the tensor core fed; the rest of the shared memory holds raw boxes in
  // flight from HBM
  int stages = 2;
  int raw_stages = (int)((200 * 1024 - (long long)stages * p.stage_bytes) / p.raw_bytes);
  if (raw_stages > kGwMaxStages) raw_stages = kGwMaxStages;
  EXB_REQUIRE(raw_stages >= 2, "grad_weight_from_packed: the pipeline does not fit in shared memory");
  if (raw_stages == kGwMaxStages) {
    stages = (int)((200 * 1024 - (long long)raw_stages * p.raw_bytes) / p.stage_bytes);
    if (stages > kGwMaxStages) stages = kGwMaxStages;
  }
  p.stages = stages; p.raw_stages = raw_stages;
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
    int rc = make_tensor_map_2d_f32(&tm_g, g, (unsigned long long)O, (unsigned long long)N, (unsigned long long)O * 4, (unsigned)O,
                                    kGwRows, /*swizzle128=*/false);
    if (rc) return rc;
    const size_t dyn = (size_t)raw_stages * p.raw_bytes + (size_t)stages * p.stage_bytes + 1024;
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
