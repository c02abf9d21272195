// Slot geometry of compact rows (see crows.cu), shared by the producer and the SpMM that gathers them.
#pragma once

namespace exb {

// Bytes of the column-index region of a slot: K rounded up to 16, so the values behind it are 16-byte aligned.
__host__ __device__ __forceinline__ int crows_cols_bytes(int K) { return (K + 15) & ~15; }
// Bytes of one slot: 16-byte header, the column indices, K fp32 values.
__host__ __device__ __forceinline__ long long crows_stride_bytes(int K) { return 16 + crows_cols_bytes(K) + 4ll * K; }

}  // namespace exb
