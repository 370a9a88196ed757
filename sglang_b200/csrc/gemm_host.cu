// Host-side helpers shared by the GEMM kernels: tensor-map encoding through the driver entry
// point and the per-device status word that bounded device-side waits report into.
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

static __device__ int g_gemm_status = 0;

int* gemm_status_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptrs[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_gemm_status) != cudaSuccess) return nullptr;
    ptrs[dev] = static_cast<int*>(ptr);
  }
  return ptrs[dev];
}


}  // namespace b200

extern "C" int b200_gemm_device_status(int* status_out) {
  using namespace b200;
  if (!status_out) return B200_ERR_NULL_PTR;
  int* ptr = gemm_status_ptr();
  if (!ptr) return B200_ERR_CUDA;
  B200_CUDA_TRY(cudaDeviceSynchronize());
  B200_CUDA_TRY(cudaMemcpy(status_out, ptr, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out != 0) B200_CUDA_TRY(cudaMemset(ptr, 0, sizeof(int)));
  return B200_OK;
}
