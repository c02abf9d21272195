// Library-wide pieces of the C ABI: version, error text, device properties.
#include <mutex>

#include "common.cuh"
#include "exact_b200.h"

namespace exb {

char* last_error_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached = n;
    cached_dev = dev;
  }
  return cached;
}

// Library-wide status word: kernels with bounded on-chip waits OR a code into it when a wait expires.
static __device__ int g_status_word;

int* status_word_ptr() {
  static std::mutex mu;
  static int* addr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    addr[dev] = static_cast<int*>(p);
  }
  return addr[dev];
}

}  // namespace exb

extern "C" {

int exact_version(void) { return 200; }

int exact_status(int* status, void* stream) {
  EXB_REQUIRE(status != nullptr, "exact_status: null output");
  int* w = exb::status_word_ptr();
  EXB_REQUIRE(w != nullptr, "exact_status: no CUDA device");
  EXB_CUDA_OK(cudaMemcpyAsync(status, w, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  EXB_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return exb::EXB_OK;
}

int exact_status_async(int* pinned_host_status, void* stream) {
  EXB_REQUIRE(pinned_host_status != nullptr, "exact_status_async: null output");
  int* w = exb::status_word_ptr();
  EXB_REQUIRE(w != nullptr, "exact_status_async: no CUDA device");
  EXB_CUDA_OK(cudaMemcpyAsync(pinned_host_status, w, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return exb::EXB_OK;
}

int exact_clear_status(void* stream) {
  int* w = exb::status_word_ptr();
  EXB_REQUIRE(w != nullptr, "exact_clear_status: no CUDA device");
  EXB_CUDA_OK(cudaMemsetAsync(w, 0, sizeof(int), (cudaStream_t)stream));
  return exb::EXB_OK;
}

int exact_set_status(int code, void* stream) {
  int* w = exb::status_word_ptr();
  EXB_REQUIRE(w != nullptr, "exact_set_status: no CUDA device");
  EXB_CUDA_OK(cudaMemcpyAsync(w, &code, sizeof(int), cudaMemcpyHostToDevice, (cudaStream_t)stream));
  EXB_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return exb::EXB_OK;
}

const char* exact_last_error(void) { return exb::last_error_buf(); }

int64_t exact_packed_bytes(int64_t N, int64_t D, int bits) {
  if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8) || N < 0 || D < 0) return -1;
  const int64_t wpt = 8 / bits;
  return ((N + wpt - 1) / wpt) * D;
}

}  // extern "C"
