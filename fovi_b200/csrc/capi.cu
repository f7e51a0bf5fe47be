// Status strings, error capture and process-wide counters of the C ABI.
#include "common.cuh"

namespace fovi {
thread_local std::string g_last_cuda_error;
std::atomic<int64_t> g_launch_count{0};

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace fovi

extern "C" const char* fovi_status_string(int status) {
  switch (status) {
    case FOVI_OK: return "ok";
    case FOVI_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FOVI_ERR_UNSUPPORTED: return "unsupported shape, dtype or layout";
    case FOVI_ERR_TABLE_RANGE: return "neighbour or tap table entry out of range";
    case FOVI_ERR_CUDA: return "CUDA call failed";
    case FOVI_ERR_ALIGNMENT: return "pointer or stride not aligned as required";
    case FOVI_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel gave up";
    case FOVI_ERR_NO_DEVICE: return "no sm_100 device is current";
    default: return "unknown status";
  }
}

extern "C" const char* fovi_last_cuda_error(void) { return fovi::g_last_cuda_error.c_str(); }
extern "C" const char* fovi_version(void) { return "0.1"; }
extern "C" int64_t fovi_launch_count(void) { return fovi::g_launch_count.load(); }
