// Error reporting and device queries of the C ABI.
#include "common.cuh"

namespace sglb200 {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace sglb200

extern "C" {

const char* sglb200_last_error(void) { return sglb200::g_err; }

int sglb200_abi_version(void) { return 2; }

int sglb200_check_device(int device) {
  int major = 0;
  SGLB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10)
    return sglb200::fail(SGLB200_E_UNSUPPORTED, "device %d has compute capability %d.x; this library is sm_100a only",
                         device, major);
  return SGLB200_OK;
}
}
