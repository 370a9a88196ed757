// Library-wide plumbing of the C ABI: error strings, device queries.
#include "common.cuh"

namespace b200 {

thread_local int g_last_cuda_error = 0;

namespace {
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
int g_cc_major[kMaxDevices] = {0};

int query_device(int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return B200_ERR_UNSUPPORTED;
  if (g_sm_count[dev] == 0) {
    int sms = 0, major = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    g_cc_major[dev] = major;
    g_sm_count[dev] = sms;
  }
  *dev_out = dev;
  return B200_OK;
}
}  // namespace

namespace {
int g_sm_limit = 0;   // 0 = all SMs
}

int sm_count() {
  int dev = 0;
  if (query_device(&dev) != B200_OK) return -1;
  const int sms = g_sm_count[dev];
  return (g_sm_limit > 0 && g_sm_limit < sms) ? g_sm_limit : sms;
}

int require_sm100() {
  int dev = 0;
  const int rc = query_device(&dev);
  if (rc != B200_OK) return rc;
  return g_cc_major[dev] == 10 ? B200_OK : B200_ERR_NOT_SM100;
}

}  // namespace b200

extern "C" int b200_set_sm_limit(int sms) {
  const int old = b200::g_sm_limit;
  b200::g_sm_limit = sms > 0 ? sms : 0;
  return old;
}

extern "C" const char* b200_strerror(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_NULL_PTR: return "null pointer argument";
    case B200_ERR_BAD_DTYPE: return "unsupported element type";
    case B200_ERR_BAD_SHAPE: return "invalid shape (negative size or size not divisible as required)";
    case B200_ERR_BAD_STRIDE: return "stride not allowed by the layout contract";
    case B200_ERR_MISALIGNED: return "pointer or leading dimension is not 16-byte aligned";
    case B200_ERR_UNSUPPORTED: return "configuration not supported by this build";
    case B200_ERR_CUDA: return "a CUDA call failed (see b200_last_cuda_error)";
    case B200_ERR_NOT_SM100: return "current device is not compute capability 10.x (B200)";
    case B200_ERR_TOO_LARGE: return "size exceeds a stated maximum";
    case B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    default: return "unknown error code";
  }
}

extern "C" int b200_last_cuda_error(void) { return b200::g_last_cuda_error; }

extern "C" int b200_abi_version(void) { return 1; }
