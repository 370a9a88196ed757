// Host-side helpers shared by the GEMM kernels: tensor-map encoding through the driver entry
// point and the per-device status word that bounded device-side waits report into.
#include <atomic>

#include "gemm_common.cuh"

namespace b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// 2-D map over a row-major [rows, cols] matrix of bytes, box = box_rows x 128 bytes, 128-byte swizzle.
int make_map_u8_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return B200_ERR_CUDA;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld)};
  cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return B200_ERR_CUDA;
  }
  return B200_OK;
}

// The status ring (layout in common.cuh).  Set up once per device: the ring's address, a 4-byte mirror of
// the sticky code in pinned mapped host memory, and the mirror's device address stored into the ring.
static __device__ __align__(4096) int g_gemm_status[kStatusRingInts];

namespace {
struct DeviceStatus {
  int* ring = nullptr;        // device address of g_gemm_status on this device
  volatile int* host = nullptr;   // pinned mirror of the sticky code
  std::atomic<unsigned> next{0};
  std::atomic<int> state{0};  // 0 = not set up, 1 = being set up, 2 = ready, -1 = failed
};
DeviceStatus g_status[64];

DeviceStatus* device_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  DeviceStatus& d = g_status[dev];
  int st = d.state.load(std::memory_order_acquire);
  if (st == 2) return &d;
  if (st == -1) return nullptr;
  int expected = 0;
  if (d.state.compare_exchange_strong(expected, 1)) {
    void* ring = nullptr;
    int* host = nullptr;
    int* host_dev = nullptr;
    bool ok = cudaGetSymbolAddress(&ring, g_gemm_status) == cudaSuccess &&
              cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped) == cudaSuccess;
    if (ok) {
      *host = 0;
      ok = cudaHostGetDevicePointer(reinterpret_cast<void**>(&host_dev), host, 0) == cudaSuccess &&
           cudaMemset(ring, 0, kStatusRingInts * sizeof(int)) == cudaSuccess &&
           cudaMemcpy(static_cast<int*>(ring) + 2, &host_dev, sizeof(host_dev), cudaMemcpyHostToDevice) == cudaSuccess;
    }
    if (!ok) {
      d.state.store(-1, std::memory_order_release);
      return nullptr;
    }
    d.ring = static_cast<int*>(ring);
    d.host = host;
    d.state.store(2, std::memory_order_release);
    return &d;
  }
  while ((st = d.state.load(std::memory_order_acquire)) == 1) {}   // another thread is setting this device up
  return st == 2 ? &d : nullptr;
}
}  // namespace

int* gemm_status_ptr() {
  DeviceStatus* d = device_status();
  if (!d) return nullptr;
  const unsigned n = d->next.fetch_add(1, std::memory_order_relaxed);
  return d->ring + kStatusFirstSlot + n % (kStatusRingInts - kStatusFirstSlot);
}

int gemm_sticky_status() {
  DeviceStatus* d = device_status();
  return d ? *d->host : 0;
}

}  // namespace b200

extern "C" int b200_gemm_poll_status(int* status_out) {
  using namespace b200;
  if (!status_out) return B200_ERR_NULL_PTR;
  DeviceStatus* d = device_status();
  if (!d) return B200_ERR_CUDA;
  *status_out = *d->host;
  return B200_OK;
}

extern "C" int b200_gemm_device_status(int* status_out) {
  using namespace b200;
  if (!status_out) return B200_ERR_NULL_PTR;
  DeviceStatus* d = device_status();
  if (!d) return B200_ERR_CUDA;
  B200_CUDA_TRY(cudaDeviceSynchronize());
  B200_CUDA_TRY(cudaMemcpy(status_out, d->ring, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) {
    // clear the sticky word and every slot, keep the mirror's address (words 2..3)
    B200_CUDA_TRY(cudaMemset(d->ring, 0, 2 * sizeof(int)));
    B200_CUDA_TRY(cudaMemset(d->ring + kStatusFirstSlot, 0, (kStatusRingInts - kStatusFirstSlot) * sizeof(int)));
    *d->host = 0;
  }
  return B200_OK;
}
