// Dense block-scaled FP8 GEMM for sm_100a:  out = cast( sum_kb (A_kb * B_kb^T) * sa[:,kb] * sb[nb,kb] ).
//
// Stands in for the reference's fp8_blockwise_scaled_mm
// (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:165-423) and the Triton kernel
// _w8a8_block_fp8_matmul (python/sglang/srt/layers/quantization/fp8_kernel.py:493-575).
//
// One persistent CTA per SM, 18 warps, warp-specialised:
//   warp 0      TMA producer: per 128-wide k-block one A box (128 rows x 128 B) and one B box
//               (BLOCK_N rows x 128 B) into a ring of shared-memory stages (128-byte swizzle).
//   warp 1      MMA issuer: 4 x tcgen05.mma kind::f8f6f4 (M128 x N BLOCK_N x K32) per k-block into
//               a tensor-memory accumulator that is started fresh for every k-block (the fp32
//               scales differ per k-block, so partial sums cannot be chained inside the tensor
//               core); accumulators rotate through 512/BLOCK_N tensor-memory buffers.
//   warps 2..17 promotion + epilogue: each warp owns 32 rows (its tensor-memory lane quadrant)
//               x BLOCK_N/4 columns; per k-block it reads the partial sums with tcgen05.ld,
//               releases the buffer, and does acc += partial * (sa[m,kb] * sb[nb,kb]) in fp32
//               registers; after the last k-block it converts and stores the output row segment.
// All mbarrier waits are bounded; a wait that gives up records a code in a device status word
// and every role drains to a common exit where tensor memory is released.
#include "gemm_common.cuh"

namespace b200 {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;
constexpr int kEpiWarps = 16;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;  // m-blocks per rasterisation group (keeps A and B tiles of a wave in L2)

template <int BLOCK_N>
struct Cfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kABytes = BLOCK_M * BLOCK_K;
  static constexpr int kBBytes = BLOCK_N * BLOCK_K;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNumAcc = kTmemCols / BLOCK_N;
  static constexpr int kColsPerWarp = BLOCK_N / 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int& m_blk, int& n_blk) {
  const int group_size = kGroupM * n_blocks;
  const int group = tile / group_size;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, m_blocks - first_m);
  const int in_group = tile - group * group_size;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

template <int BLOCK_N, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_block_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
  using C = Cfg<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + C::kStages * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* acc_full = bars + 2 * C::kStages;
  uint64_t* acc_empty = acc_full + C::kNumAcc;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::kNumAcc);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int num_tiles = m_blocks * n_blocks;
  const int nkb = (p.K + BLOCK_K - 1) / BLOCK_K;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < C::kNumAcc; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kEpiWarps);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m_blk, n_blk;
        tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, 1);
          if (!ok) break;
          mbar_expect_tx(&full_bar[stage], C::kStageBytes);
          tma_load_2d(smem_a + stage * C::kABytes, &map_a, &full_bar[stage], kb * BLOCK_K, m_blk * BLOCK_M);
          tma_load_2d(smem_b + stage * C::kBBytes, &map_b, &full_bar[stage], kb * BLOCK_K, n_blk * BLOCK_N);
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(BLOCK_M, BLOCK_N);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 2);
          if (!ok) break;
          ok = mbar_wait(&full_bar[stage], phase, p.status, 3);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = umma_desc_k128(smem_u32(smem_a + stage * C::kABytes));
          const uint64_t b_desc = umma_desc_k128(smem_u32(smem_b + stage * C::kBBytes));
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
#pragma unroll
          for (int k = 0; k < BLOCK_K / 32; ++k) {
            // advance 32 bytes along K inside the 128-byte swizzle row: +2 in the (addr >> 4) field
            umma_f8(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                    k > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // stage reusable once these MMAs have read it
          umma_commit(&acc_full[acc]);     // partial sums of this k-block are in tensor memory
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
          if (++acc == C::kNumAcc) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ promotion + epilogue
    constexpr int CPW = C::kColsPerWarp;
    const int quad = warp & 3;          // tensor-memory lane quadrant this warp may read
    const int part = (warp - 2) >> 2;   // which BLOCK_N/4 column slice
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (p.ldo % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    int acc_i = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int m_blk, n_blk;
      tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
      const int m = m_blk * BLOCK_M + quad * 32 + lane;
      const int n0 = n_blk * BLOCK_N + part * CPW;
      const bool row_ok = m < p.M;
      const float* sa_ptr = p.sa + static_cast<int64_t>(row_ok ? m : 0) * p.sa_stride_m;
      const int nb = min(n0, p.N - 1) / 128;
      const float* sb_ptr = p.sb + static_cast<int64_t>(nb) * p.sb_stride_n;
      float acc[CPW];
#pragma unroll
      for (int c = 0; c < CPW; ++c) acc[c] = 0.f;
      float s_next = row_ok ? __ldg(sa_ptr) * __ldg(sb_ptr) : 0.f;
      for (int kb = 0; kb < nkb; ++kb) {
        const float s = s_next;
        if (kb + 1 < nkb) {
          const float a_s = row_ok ? __ldg(sa_ptr + static_cast<int64_t>(kb + 1) * p.sa_stride_g) : 0.f;
          s_next = a_s * __ldg(sb_ptr + static_cast<int64_t>(kb + 1) * p.sb_stride_g);
        }
        ok = mbar_wait(&acc_full[acc_i], acc_phase, p.status, 4);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(acc_i * BLOCK_N + part * CPW);
#pragma unroll
        for (int ch = 0; ch < CPW / 16; ++ch) {
          float v[16];
          tmem_ld16(taddr + ch * 16, v);
          tmem_ld_wait();
          if (ch == CPW / 16 - 1) {
            // all of this warp's reads of the buffer are complete: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc_i]);
          }
#pragma unroll
          for (int c = 0; c < 16; ++c) acc[ch * 16 + c] = fmaf(v[c], s, acc[ch * 16 + c]);
        }
        if (++acc_i == C::kNumAcc) { acc_i = 0; acc_phase ^= 1u; }
      }
      if (ok && row_ok && n0 < p.N) {
        store_row<CPW>(out + static_cast<int64_t>(m) * p.ldo + n0, acc, p.N - n0, vec_ok);
      }
    }
  }

  // ---------------------------------------------------------------------- common exit
  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(p.status) != 0) {
    // a wait gave up: let copies that may still be in flight land before shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------ host
template <int BLOCK_N, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<BLOCK_N>;
  auto kern = gemm_block_fp8_kernel<BLOCK_N, OutT>;
  static bool attr_set[64] = {false};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  const int m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int tiles = m_blocks * n_blocks;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(ma, mb, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <int BLOCK_N>
int launch_dtype(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch<BLOCK_N, __nv_bfloat16>(ma, mb, p, stream);
    case B200_DT_F16: return launch<BLOCK_N, __half>(ma, mb, p, stream);
    case B200_DT_F32: return launch<BLOCK_N, float>(ma, mb, p, stream);
    default: return B200_ERR_BAD_DTYPE;
  }
}

}  // namespace

// Kernel override for experiments and tests: 0 = automatic, 128 / 256 = single-CTA kernel with that
// BLOCK_N, 2 = CTA-pair kernel.
int g_force_block_n = 0;

int launch_gemm_pair(const void* a, int64_t lda, const void* b, int64_t ldb, const GemmParams& p, cudaStream_t stream);

}  // namespace b200

extern "C" int b200_fp8_blockwise_scaled_mm(const void* a, int64_t lda, const void* b, int64_t ldb, const float* sa,
                                            int64_t sa_stride_m, int64_t sa_stride_g, const float* sb,
                                            int64_t sb_stride_n, int64_t sb_stride_g, void* out, int64_t ldo,
                                            int out_dtype, int64_t M, int64_t N, int64_t K, void* stream) {
  using namespace b200;
  if (M < 0 || N < 0 || K <= 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || N == 0) return B200_OK;
  if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa || !sb || !out) return B200_ERR_NULL_PTR;
  if (out_dtype != B200_DT_BF16 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_F32) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldo < N) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || !aligned16(a) || !aligned16(b)) return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_g < 0 || sb_stride_n < 0 || sb_stride_g < 0) return B200_ERR_BAD_STRIDE;
  int rc = require_sm100();
  if (rc != B200_OK) return rc;

  GemmParams p;
  p.sa = sa; p.sb = sb; p.out = out;
  p.sa_stride_m = sa_stride_m; p.sa_stride_g = sa_stride_g;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g;
  p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = out_dtype;
  p.status = gemm_status_ptr();
  if (!p.status) return B200_ERR_CUDA;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // M > 128: CTA-pair kernel (256 x 128 tiles).  Otherwise one CTA per tile:
  // 128 x 256 when that still gives every SM a tile, else 128 x 128.
  if ((M > 128 && g_force_block_n == 0) || g_force_block_n == 2) return launch_gemm_pair(a, lda, b, ldb, p, st);
  const int64_t m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
  int block_n = 256;
  if (m_blocks * ((N + 255) / 256) < sm_count()) block_n = 128;
  if (g_force_block_n == 128 || g_force_block_n == 256) block_n = g_force_block_n;

  CUtensorMap ma, mb;
  rc = make_map_u8_2d(&ma, a, M, K, lda, BLOCK_M);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, N, K, ldb, block_n);
  if (rc != B200_OK) return rc;
  return block_n == 256 ? launch_dtype<256>(ma, mb, p, st) : launch_dtype<128>(ma, mb, p, st);
}

extern "C" int b200_debug_force_block_n(int block_n) {
  b200::g_force_block_n = block_n;
  return B200_OK;
}
