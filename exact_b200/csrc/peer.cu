// Device buffers that the ranks of a row-sharded run write into each other: allocation and CUDA IPC mapping.
//
// The compact rows a rank produces before an aggregation (crows.cu) are stored straight into the same slots
// of every rank's buffer, so each rank needs a device pointer to every peer's buffer.  A buffer is a plain
// cudaMalloc allocation of its owner, exported as a 64-byte IPC handle that the other processes of the node
// open; opening enables peer access between the two devices.  These are the only entry points of the
// library that allocate or free device memory, and they do so only when called.
//
// The reference is single-GPU and has no counterpart.
#include <cstring>

#include "common.cuh"
#include "exact_b200.h"

using namespace exb;

extern "C" {

int exact_peer_alloc(int64_t bytes, void** ptr) {
  EXB_REQUIRE(bytes > 0 && ptr != nullptr, "peer_alloc: bad argument");
  *ptr = nullptr;
  EXB_CUDA_OK(cudaMalloc(ptr, (size_t)bytes));
  return EXB_OK;
}

int exact_peer_free(void* ptr) {
  if (ptr == nullptr) return EXB_OK;
  EXB_CUDA_OK(cudaFree(ptr));
  return EXB_OK;
}

int exact_peer_export(const void* ptr, void* handle64) {
  EXB_REQUIRE(ptr != nullptr && handle64 != nullptr, "peer_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == EXACT_PEER_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  EXB_CUDA_OK(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  memcpy(handle64, &h, sizeof(h));
  return EXB_OK;
}

int exact_peer_import(const void* handle64, void** ptr) {
  EXB_REQUIRE(ptr != nullptr && handle64 != nullptr, "peer_import: null pointer");
  *ptr = nullptr;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  EXB_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return EXB_OK;
}

int exact_peer_close(void* ptr) {
  if (ptr == nullptr) return EXB_OK;
  EXB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return EXB_OK;
}

}  // extern "C"
