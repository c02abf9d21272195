// Library-wide pieces of the C ABI: version, error text, device properties.
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

}  // namespace exb

extern "C" {

int exact_version(void) { return 100; }

const char* exact_last_error(void) { return exb::last_error_buf(); }

int64_t exact_packed_bytes(int64_t N, int64_t D, int bits) {
  if (!(bits == 1 || bits == 2 || bits == 4 || bits == 8) || N < 0 || D < 0) return -1;
  const int64_t wpt = 8 / bits;
  return ((N + wpt - 1) / wpt) * D;
}

}  // extern "C"
