// Pieces shared by the block-FP8 GEMM kernels: parameter block, output-row stores, tensor-map
// construction and the device status word.
#pragma once
#include "common.cuh"

namespace b200 {

struct GemmParams {
  const float* sa;
  const float* sb;
  void* out;
  int64_t sa_stride_m, sa_stride_g, sb_stride_n, sb_stride_g, ldo;
  int M, N, K;
  int out_dtype;
  int* status;
  // grouped (per-expert) form only: rows [expert_offsets[e], +problem_sizes[3e]) of A/out belong to
  // expert e, whose weights are rows [e*N, (e+1)*N) of B and whose weight scales start at sb + e*sb_stride_e
  const int32_t* expert_offsets;
  const int32_t* problem_sizes;
  int64_t sb_stride_e;
  int num_experts;
  // split-K form (dense, small M): the k-blocks of a tile are divided among split_k CTAs, each writing
  // fp32 partial sums to partial[split][M][N]; a second kernel adds them in split order
  int split_k;
  int kb_per_split;
  float* partial;
  // tail split (dense, large M): tiles [0, tail_first) are whole; each tile from tail_first on -- the ones
  // that would form a mostly empty last wave -- is divided among split_k CTAs, partial sums stored compactly
  // as partial[(tile - tail_first) * split_k + split][128][block_n].  0 = the uniform split above.
  int tail_first;
  // activation scales given as packed UE8M0 exponent bytes (four k-blocks per 32-bit word) instead of fp32:
  // element (m, kb) is byte kb % 4 of the word at sa[(kb / 4) * sa_stride_g + m * sa_stride_m]
  int sa_ue8m0;
};


// A fresh slot of the current device's status ring for one launch, or nullptr on error.
int* gemm_status_ptr();
// The device's sticky error code as mirrored in pinned host memory (0 = none); no synchronisation.
int gemm_sticky_status();
// 2-D tensor map over a row-major [rows, cols] byte matrix with leading dimension ld, box =
// box_rows x 128 bytes, 128-byte swizzle, zero fill outside the matrix.
int make_map_u8_2d(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);

#if defined(__CUDACC__)
// Activation scale of (row, k-block), fp32 or packed UE8M0.  The representation is a template argument so
// that a stager's batch of loads stays a straight line of independent loads: with a run-time test inside
// every load the compiler serialised them and the stager fell behind the tensor pipe.
template <bool UE8M0>
__device__ __forceinline__ float load_sa(const GemmParams& p, int64_t row, int kb) {
  if constexpr (UE8M0) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(p.sa);
    const uint32_t word = __ldg(w + static_cast<int64_t>(kb >> 2) * p.sa_stride_g + row * p.sa_stride_m);
    return __uint_as_float(((word >> (8 * (kb & 3))) & 0xffu) << 23);   // 2 ** (byte - 127); byte 0 -> 0
  } else {
    return __ldg(p.sa + row * p.sa_stride_m + static_cast<int64_t>(kb) * p.sa_stride_g);
  }
}

__device__ __forceinline__ uint32_t pack2(__nv_bfloat16*, float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack2(__half*, float a, float b) {
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ __nv_bfloat16 cvt1(__nv_bfloat16*, float a) { return __float2bfloat16_rn(a); }
__device__ __forceinline__ __half cvt1(__half*, float a) { return __float2half_rn(a); }
__device__ __forceinline__ float cvt1(float*, float a) { return a; }

// Store NCOLS consecutive outputs of one row; `valid` = columns left before N.
template <int NCOLS, typename OutT>
__device__ __forceinline__ void store_row(OutT* dst, const float (&acc)[NCOLS], int valid, bool vec_ok) {
  if (vec_ok && valid >= NCOLS) {
#pragma unroll
    for (int c = 0; c < NCOLS; c += 8) {
      uint4 v;
      v.x = pack2(dst, acc[c + 0], acc[c + 1]);
      v.y = pack2(dst, acc[c + 2], acc[c + 3]);
      v.z = pack2(dst, acc[c + 4], acc[c + 5]);
      v.w = pack2(dst, acc[c + 6], acc[c + 7]);
      *reinterpret_cast<uint4*>(dst + c) = v;
    }
  } else {
#pragma unroll
    for (int c = 0; c < NCOLS; ++c)
      if (c < valid) dst[c] = cvt1(dst, acc[c]);
  }
}
template <int NCOLS>
__device__ __forceinline__ void store_row(float* dst, const float (&acc)[NCOLS], int valid, bool vec_ok) {
  if (vec_ok && valid >= NCOLS) {
#pragma unroll
    for (int c = 0; c < NCOLS; c += 4)
      *reinterpret_cast<float4*>(dst + c) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
  } else {
#pragma unroll
    for (int c = 0; c < NCOLS; ++c)
      if (c < valid) dst[c] = acc[c];
  }
}

#endif  // __CUDACC__

}  // namespace b200
