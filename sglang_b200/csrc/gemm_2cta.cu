// Dense block-scaled FP8 GEMM for sm_100a, CTA-pair form (tcgen05 cta_group::2).
//
// Same contract as gemm.cu; used when M > 128.  Two CTAs of a cluster work on one
// 256 x 128 output tile: each CTA TMA-loads its own 128 rows of A and its own 64 rows of B per
// 128-wide k-block (no multicast: halving the B traffic per SM comes from the pair MMA reading
// both halves), the leader CTA issues tcgen05.mma.cta_group::2 (M256 x N128 x K32, four per
// k-block) and each CTA receives its 128 x 128 fp32 partial sums in its own tensor memory.
// Tensor memory holds four such buffers, so the MMA of k-block i+1..i+3 overlaps the promotion
// of k-block i: 8 epilogue warps per CTA read their 32 x 64 slice with tcgen05.ld, hand the
// buffer back at once, and accumulate acc += partial * (sa[m,kb] * sb[nb,kb]) in registers.
// Scales are fetched four k-blocks ahead.  Every wait is bounded (see common.cuh).
#include "gemm_common.cuh"

namespace b200 {
int g_last_max_pairs = 0;  // what the cluster occupancy query returned (diagnostics)
namespace {

constexpr int kPairM = 256;     // rows per CTA pair
constexpr int kCtaM = 128;      // rows per CTA
constexpr int kTileN = 128;     // output columns per tile (= one weight-scale block)
constexpr int kCtaBRows = 64;   // B rows each CTA loads
constexpr int kBlockK = 128;
constexpr int kStages = 8;
constexpr int kABytes = kCtaM * kBlockK;
constexpr int kBBytes = kCtaBRows * kBlockK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kNumAcc = 4;
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;   // 2 per SM sub-partition: fewer, fatter warps amortise the per-k-block handshake
constexpr int kMmaWarpB = 2 + kEpiWarps;   // second MMA-issuing warp (the first is warp 1)
constexpr int kThreads = 32 * (3 + kEpiWarps);
constexpr int kColsPerWarp = kTileN / (kEpiWarps / 4);
constexpr int kGroupM = 8;      // pair-m-blocks per rasterisation group
constexpr int kScaleAhead = 4;  // k-blocks of scale prefetch
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

__device__ __forceinline__ void pair_tile_coords(int tile, int m_blocks, int n_blocks, int& m_blk, int& n_blk) {
  const int group_size = kGroupM * n_blocks;
  const int group = tile / group_size;
  const int first_m = group * kGroupM;
  const int rows = min(kGroupM, m_blocks - first_m);
  const int in_group = tile - group * group_size;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_block_fp8_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                  // operands landed (leader's copy is the live one)
  uint64_t* done_bar = bars + kStages;        // the k-block's MMAs completed: its stage may be refilled
                                              // and its partial sums read (one per CTA)
  uint64_t* acc_empty = bars + 2 * kStages;   // accumulator buffer read out (leader's copy is live)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kNumAcc);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_blocks = (p.M + kPairM - 1) / kPairM;
  const int n_blocks = (p.N + kTileN - 1) / kTileN;
  const int num_tiles = m_blocks * n_blocks;
  const int nkb = (p.K + kBlockK - 1) / kBlockK;

  cluster_sync_all();  // both CTAs of the pair are resident before tensor memory is paired
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full_bar[i], 2);   // one arrival per CTA's producer (+ both CTAs' bytes)
      mbar_init(&done_bar[i], 1);   // the leader's commit, delivered to both CTAs
    }
    for (int i = 0; i < kNumAcc; ++i) mbar_init(&acc_empty[i], 2 * kEpiWarps);  // epilogue warps of both CTAs
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (each CTA)
    if (!(p.debug_mode & 2)) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        int m_blk, n_blk;
        pair_tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
        const int row_a = m_blk * kPairM + static_cast<int>(rank) * kCtaM;
        const int row_b = n_blk * kTileN + static_cast<int>(rank) * kCtaBRows;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait_warp(&done_bar[stage], phase ^ 1u, p.status, 11, p.wait_hint_ns);
          if (!ok) break;
          if (elect_one()) {
            if (leader) mbar_expect_tx(&full_bar[stage], 2 * kStageBytes);
            tma_load_2d_pair(smem_a + stage * kABytes, &map_a, &full_bar[stage], kb * kBlockK, row_a);
            tma_load_2d_pair(smem_b + stage * kBBytes, &map_b, &full_bar[stage], kb * kBlockK, row_b);
            if (!leader) mbar_arrive_cluster(&full_bar[stage], 0);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1 || warp == kMmaWarpB) {
    // ------------------------------------------------------------------ MMA issuers (leader CTA only)
    // Two warps share the issue: warp 1 takes the even k-blocks of the CTA pair's k-block sequence,
    // warp kMmaWarpB the odd ones.  One warp alone spends ~700 cycles per k-block on its two barrier
    // waits plus the issue (measured), which starves the tensor pipe; k-blocks are independent
    // (own stage, own accumulator buffer), so the two issue streams may interleave freely.
    if (leader) {
      constexpr uint32_t idesc = umma_idesc_e4m3(kPairM, kTileN);
      // the whole warp walks the loop so that addresses and descriptors stay warp-uniform; one
      // elected lane issues the MMAs and the commit
      const uint64_t a_desc0 = umma_desc_k128(smem_u32(smem_a));
      const uint64_t b_desc0 = umma_desc_k128(smem_u32(smem_b));
      const int issuer = (warp == 1) ? 0 : 1;
      const bool wait_operands = !(p.debug_mode & 2);
      const long long my_tiles = (num_tiles > pair_id) ? (num_tiles - pair_id + num_pairs - 1) / num_pairs : 0;
      const long long total_kb = my_tiles * nkb;
      bool ok = true;
      for (long long g = issuer; ok && g < total_kb; g += 2) {
        const int stage = static_cast<int>(g % kStages);
        const uint32_t phase = static_cast<uint32_t>((g / kStages) & 1);
        const int acc = static_cast<int>(g % kNumAcc);
        const uint32_t acc_phase = static_cast<uint32_t>((g / kNumAcc) & 1);
        const bool rec = p.debug_buf != nullptr && pair_id == 0 && g < 64;
        if (rec && lane == 0) p.debug_buf[0 * 64 + g] = clock64();   // before the waits
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 12, p.wait_hint_ns);
        if (rec && lane == 0) p.debug_buf[1 * 64 + g] = clock64();   // accumulator free
        if (ok && wait_operands) ok = mbar_wait(&full_bar[stage], phase, p.status, 13, p.wait_hint_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (rec && lane == 0) p.debug_buf[2 * 64 + g] = clock64();   // operands landed, about to issue
        const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kABytes >> 4));
        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage * (kBBytes >> 4));
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * kTileN);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < kBlockK / 32; ++k) {
            umma_f8_pair(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                         k > 0 ? 1u : 0u);
          }
          umma_commit_pair(&done_bar[stage], 3);  // one completion signal, delivered to both CTAs
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ promotion + epilogue (each CTA)
    constexpr int CPW = kColsPerWarp;
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (p.ldo % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    int acc_i = 0, stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      pair_tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
      const int m = m_blk * kPairM + static_cast<int>(rank) * kCtaM + quad * 32 + lane;
      const int n0 = n_blk * kTileN + part * CPW;
      const bool row_ok = m < p.M;
      const float* sa_ptr = p.sa + static_cast<int64_t>(row_ok ? m : 0) * p.sa_stride_m;
      const float* sb_ptr = p.sb + static_cast<int64_t>(n_blk) * p.sb_stride_n;
      float acc[CPW];
#pragma unroll
      for (int c = 0; c < CPW; ++c) acc[c] = 0.f;
      float fa[kScaleAhead], fb[kScaleAhead];
#pragma unroll
      for (int j = 0; j < kScaleAhead; ++j) {
        const bool in = j < nkb;
        fa[j] = in ? __ldg(sa_ptr + static_cast<int64_t>(j) * p.sa_stride_g) : 0.f;
        fb[j] = in ? __ldg(sb_ptr + static_cast<int64_t>(j) * p.sb_stride_g) : 0.f;
      }
      for (int kb0 = 0; ok && kb0 < nkb; kb0 += kScaleAhead) {
#pragma unroll
        for (int j = 0; j < kScaleAhead; ++j) {
          const int kb = kb0 + j;
          if (kb < nkb) {
            const float s = row_ok ? fa[j] * fb[j] : 0.f;
            const int kn = kb + kScaleAhead;
            if (kn < nkb) {
              fa[j] = __ldg(sa_ptr + static_cast<int64_t>(kn) * p.sa_stride_g);
              fb[j] = __ldg(sb_ptr + static_cast<int64_t>(kn) * p.sb_stride_g);
            }
            ok = mbar_wait(&done_bar[stage], phase, p.status, 14, p.wait_hint_ns);
            if (!ok) break;
            const bool rec = p.debug_buf != nullptr && pair_id == 0 && leader && tile == pair_id && kb < 64 &&
                             warp == 2 && lane == 0;
            if (rec) p.debug_buf[3 * 64 + kb] = clock64();   // partial sums visible to the epilogue
            tc_fence_after();
            float v[CPW];
            const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(acc_i * kTileN + part * CPW);
            if (!(p.debug_mode & 1)) {
#pragma unroll
              for (int ch = 0; ch < CPW / 32; ++ch) tmem_ld32(taddr + ch * 32, v + ch * 32);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int c = 0; c < CPW; ++c) v[c] = 0.f;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&acc_empty[acc_i], 0);
            if (rec) p.debug_buf[4 * 64 + kb] = clock64();   // accumulator handed back
            // two fp32 FMAs per instruction (fma.rn.f32x2): the promotion is issue-bound otherwise
            const float2 s2 = make_float2(s, s);
            if (!(p.debug_mode & 17)) {
#pragma unroll
              for (int c = 0; c < CPW; c += 2) {
                const float2 r = __ffma2_rn(make_float2(v[c], v[c + 1]), s2, make_float2(acc[c], acc[c + 1]));
                acc[c] = r.x;
                acc[c + 1] = r.y;
              }
            } else {
              acc[0] += v[0] * s;
            }
            if (++acc_i == kNumAcc) acc_i = 0;
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
      if (ok && row_ok && n0 < p.N) {
        store_row<CPW>(out + static_cast<int64_t>(m) * p.ldo + n0, acc, p.N - n0, vec_ok);
      }
    }
  }

  // ---------------------------------------------------------------------- common exit
  tc_fence_before();
  cluster_sync_all();
  if (*reinterpret_cast<volatile int*>(p.status) != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <typename OutT>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  auto kern = gemm_block_fp8_pair_kernel<OutT>;
  static int max_pairs[64] = {0};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  dev &= 63;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return B200_ERR_UNSUPPORTED;
    max_pairs[dev] = n;
    g_last_max_pairs = n;
  }
  const int m_blocks = (p.M + kPairM - 1) / kPairM;
  const int n_blocks = (p.N + kTileN - 1) / kTileN;
  const int tiles = m_blocks * n_blocks;
  const int pairs = tiles < max_pairs[dev] ? tiles : max_pairs[dev];
  cfg.gridDim = dim3(2 * pairs);
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, p));
  return B200_OK;
}

}  // namespace

// Entry used by the dispatcher in gemm.cu.
int launch_gemm_pair(const void* a, int64_t lda, const void* b, int64_t ldb, const GemmParams& p, cudaStream_t stream) {
  CUtensorMap ma, mb;
  int rc = make_map_u8_2d(&ma, a, p.M, p.K, lda, kCtaM);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, p.N, p.K, ldb, kCtaBRows);
  if (rc != B200_OK) return rc;
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch_pair<__nv_bfloat16>(ma, mb, p, stream);
    case B200_DT_F16: return launch_pair<__half>(ma, mb, p, stream);
    case B200_DT_F32: return launch_pair<float>(ma, mb, p, stream);
    default: return B200_ERR_BAD_DTYPE;
  }
}

}  // namespace b200

extern "C" int b200_debug_pair_kernel_max_clusters(void) { return b200::g_last_max_pairs; }
