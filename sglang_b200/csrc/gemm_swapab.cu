// Weight-streaming form of the block-scaled FP8 GEMM for few tokens per weight matrix (decode-size
// batches, and MoE experts that each see about a hundred rows): the operands are swapped, so the
// 128-row side of the tensor-core instruction holds WEIGHT rows and the narrow side (16..128
// columns, chosen per tile at run time) holds tokens.
//
//   out[m, n] = cast( sum_kb ( sum_{k in kb} a[m,k] * b[n,k] ) * sa[m,kb] * sb[n/128,kb] )
//
// Same arithmetic as gemm_block_fp8_kernel (gemm.cu); it stands in for the swap-AB configurations the
// reference picks for small problems (sgl-kernel/csrc/moe/fp8_blockwise_moe_kernel.cu:342-437,
// sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:321-343).  Why a second kernel:
//   * a tile is 128 weight rows x up to TN tokens, so the tensor-core and read-out work follows the
//     number of tokens (rounded up to 16) instead of whole 128-row token tiles, and an expert's
//     weights are streamed once however its rows fall on 128-row boundaries;
//   * a pipeline stage holds 2 x 16 KB of weights and only 2 x TN x 128 B of activations, so 3 to 5
//     two-k-block stages fit and enough weight bytes are in flight per SM to cover the DRAM latency;
//   * the accumulator of one k-block is TN tensor-memory columns, so 4 to 8 of them rotate.
// Every hand-off (operands landed, MMAs complete, accumulators read) covers TWO k-blocks: the cost of
// a barrier round trip and of the loop around it was the bound with one k-block per hand-off.
// Roles, bounded waits and the common exit are those of gemm.cu.
#include "gemm_common.cuh"

namespace b200 {
namespace {

constexpr int BLOCK_W = 128;     // weight rows per tile = rows of the MMA = tensor-memory lanes
constexpr int BLOCK_K = 128;
constexpr int kTmemCols = 512;
constexpr int kPair = 2;         // k-blocks per pipeline stage and per hand-off
constexpr int kScaleGroup = 8;   // k-blocks per scale-ring slot (8 fp32 scales of a token = one 32-byte sector)
constexpr int kScaleSlots = 4;
constexpr int kEpiWarps = 8;     // 4 lane quadrants x 2 column halves
constexpr int kMaxExperts = 1024;

template <int TN>
struct SwapCfg {
  static_assert(TN == 32 || TN == 64 || TN == 128, "token tile");
  static constexpr int kWBytes = BLOCK_W * BLOCK_K;    // one k-block of weights
  static constexpr int kXBytes = TN * BLOCK_K;         // one k-block of activations
  static constexpr int kStageBytes = kPair * (kWBytes + kXBytes);
  static constexpr int kStages = TN == 128 ? 3 : (TN == 64 ? 4 : 5);
  static constexpr int kAccPairs = (kTmemCols / (kPair * TN)) < 4 ? (kTmemCols / (kPair * TN)) : 4;
  static_assert(kAccPairs <= kStages, "the MMA warp must not lap a stage's completion barrier");
  static constexpr int kColsPerWarp = TN / 2;
  static constexpr int kTmaWarp = kEpiWarps;
  static constexpr int kMmaWarp = kEpiWarps + 1;
  static constexpr int kStagerWarp = kEpiWarps + 2;
  static constexpr int kStagers = 2;   // both stage scale products, taking alternate slot fills
  static constexpr int kThreads = 32 * (kEpiWarps + 4);
  // Register rebalancing for the widest tile (64 accumulators + two 32-register fragments + 32 scale
  // products per read-out thread): the launch gives each of the 384 threads 168 registers; the helper
  // warpgroup hands 88 per thread back and the two read-out warpgroups take 40 more each.
  // setmaxnreg.inc WAITS until the CTA's pool holds what it asks for, so the request must never
  // exceed what the helpers release (and the kernel must really be allocated kLaunchRegs: the build
  // checks the register count ptxas reports).
  static constexpr bool kRebalanceRegs = TN == 128;
  static constexpr int kLaunchRegs = 168;
  static constexpr int kHelperRegs = 80;
  static constexpr int kEpiRegs = 208;
  static_assert(kEpiWarps * (kEpiRegs - kLaunchRegs) <= 4 * (kLaunchRegs - kHelperRegs),
                "read-out warps would wait forever for registers nobody releases");
  static constexpr int kSlotFloats = kScaleGroup * TN;
  static constexpr int kScaleBytes = kScaleSlots * kSlotFloats * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + 1024 /*alignment slack*/ + 512 /*barriers*/ +
                                    (kMaxExperts + 1) * 4;
};

// A tile: 128 weight rows (n-tile) x up to TN tokens.  Dense: token tiles fastest.  Grouped: the
// token tiles of all experts laid end to end (tile_start[e] = first token tile of expert e), n-tiles
// fastest, so that a wave of CTAs streams different slices of one expert's weights and a second
// token tile of the same expert finds them in L2.
struct SwapTile {
  int row0;      // first token row (of A / out)
  int valid;     // tokens of this tile (1..TN)
  int n0;        // first output column = first weight row within the expert
  int w_row0;    // first row of the [E*N, K] weight matrix
  int expert;
};

template <bool GROUPED, int TN>
__device__ __forceinline__ SwapTile get_swap_tile(int tile, const GemmParams& p, int m_tiles, int n_tiles,
                                                  const int* tile_start) {
  SwapTile t;
  if constexpr (!GROUPED) {
    const int nt = tile / m_tiles;
    const int mt = tile - nt * m_tiles;
    t.row0 = mt * TN;
    t.valid = min(TN, p.M - t.row0);
    t.n0 = nt * BLOCK_W;
    t.w_row0 = t.n0;
    t.expert = 0;
  } else {
    const int mt = tile / n_tiles;
    const int nt = tile - mt * n_tiles;
    int lo = 0, hi = p.num_experts;   // last e with tile_start[e] <= mt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_start[mid] <= mt) lo = mid; else hi = mid;
    }
    const int sub = mt - tile_start[lo];
    t.expert = lo;
    // Tables that do not describe the buffers (left over from another batch, never filled) must not send a
    // store outside `out`: the tile is clamped into [0, total rows); what it then computes is meaningless,
    // but so were the tables.
    t.row0 = min(max(p.expert_offsets[lo] + sub * TN, 0), p.M - 1);
    t.valid = max(1, min(min(TN, p.problem_sizes[lo * 3] - sub * TN), p.M - t.row0));
    t.n0 = nt * BLOCK_W;
    t.w_row0 = lo * p.N + t.n0;
  }
  return t;
}

// acc[i] += v[i] * s[col(i)] for one 16-lane fragment: v[4g + 2rp + e] belongs to token column 8g + 2q + e,
// whose scale product is sv[2g + e].
template <int NG>
__device__ __forceinline__ void promote(float* acc, const float* v, const float* sv) {
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int rp = 0; rp < 2; ++rp) {
      const int i = 4 * g + 2 * rp;
      const float2 r = __ffma2_rn(make_float2(v[i], v[i + 1]), make_float2(sv[2 * g], sv[2 * g + 1]),
                                  make_float2(acc[i], acc[i + 1]));
      acc[i] = r.x;
      acc[i + 1] = r.y;
    }
}

template <int TN, bool GROUPED, typename OutT>
__global__ void __launch_bounds__(SwapCfg<TN>::kThreads, 1)
gemm_block_fp8_swapab_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             const GemmParams p) {
  using C = SwapCfg<TN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_w = smem;                                        // [stage][kPair][128 x 128 B]
  uint8_t* smem_x = smem + C::kStages * kPair * C::kWBytes;      // [stage][kPair][TN x 128 B]
  float* smem_scale = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes + C::kScaleBytes);
  uint64_t* full_bar = bars;                     // operands of the stage (two k-blocks) have landed
  uint64_t* done_bar = bars + C::kStages;        // the stage's MMAs completed
  uint64_t* acc_empty = bars + 2 * C::kStages;   // accumulator pair has been read out
  uint64_t* scale_full = acc_empty + C::kAccPairs;
  uint64_t* scale_empty = scale_full + kScaleSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(scale_empty + kScaleSlots);
  int* tile_start = reinterpret_cast<int*>(tmem_slot + 2);   // [num_experts + 1], grouped form only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + TN - 1) / TN;
  const int n_tiles = (p.N + BLOCK_W - 1) / BLOCK_W;
  const int nkb = (p.K + BLOCK_K - 1) / BLOCK_K;

  if constexpr (GROUPED) {
    for (int e = threadIdx.x; e < p.num_experts; e += blockDim.x)
      tile_start[e + 1] = (max(p.problem_sizes[e * 3], 0) + TN - 1) / TN;
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      tile_start[0] = 0;
      for (int e = 1; e <= p.num_experts; ++e) {
        run += tile_start[e];
        tile_start[e] = run;
      }
    }
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&done_bar[i], 1);
    }
    for (int i = 0; i < C::kAccPairs; ++i) mbar_init(&acc_empty[i], kEpiWarps);
    for (int i = 0; i < kScaleSlots; ++i) {
      mbar_init(&scale_full[i], 1);
      mbar_init(&scale_empty[i], kEpiWarps);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kTmaWarp && lane == 0) {
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int num_tiles = GROUPED ? tile_start[p.num_experts] * n_tiles : m_tiles * n_tiles;
  const int split_k = GROUPED ? 1 : p.split_k;
  const int kbps = GROUPED ? nkb : p.kb_per_split;
  const int num_vtiles = num_tiles * split_k;

  if (warp >= kEpiWarps) {
  // ====================================================================== helper warpgroup
  if constexpr (C::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kHelperRegs));
  if (warp == C::kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const SwapTile t = get_swap_tile<GROUPED, TN>(vt / split_k, p, m_tiles, n_tiles, tile_start);
      const int split = vt % split_k;
      const int kb_begin = split * kbps, kb_end = min(nkb, kb_begin + kbps);
      for (int kb = kb_begin; kb < kb_end; kb += kPair) {
        ok = mbar_wait_warp(&done_bar[stage], phase ^ 1u, p.status, 1);
        if (!ok) break;
        if (elect_one()) {
          const int n = min(kPair, kb_end - kb);
          mbar_expect_tx(&full_bar[stage], n * (C::kWBytes + C::kXBytes));
          for (int j = 0; j < n; ++j) {
            tma_load_2d(smem_w + (stage * kPair + j) * C::kWBytes, &map_w, &full_bar[stage], (kb + j) * BLOCK_K,
                        t.w_row0);
            tma_load_2d(smem_x + (stage * kPair + j) * C::kXBytes, &map_x, &full_bar[stage], (kb + j) * BLOCK_K,
                        t.row0);
          }
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == C::kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // D[weight row, token] = W_tile (128 x 128 B, the instruction's M side) x X_tile^T (tn tokens, its
    // N side); tn = tokens of the tile rounded up to 16, encoded in the instruction descriptor.  The two
    // k-blocks of a stage go to the two accumulators of a pair; one commit covers both.
    const uint64_t w_desc0 = umma_desc_k128(smem_u32(smem_w));
    const uint64_t x_desc0 = umma_desc_k128(smem_u32(smem_x));
    int stage = 0, ap = 0;
    uint32_t phase = 0, ap_phase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const SwapTile t = get_swap_tile<GROUPED, TN>(vt / split_k, p, m_tiles, n_tiles, tile_start);
      const int tn = (t.valid + 15) & ~15;
      const uint32_t idesc = umma_idesc_e4m3(BLOCK_W, tn);
      const int split = vt % split_k;
      const int kb_begin = split * kbps, kb_end = min(nkb, kb_begin + kbps);
      for (int kb = kb_begin; kb < kb_end; kb += kPair) {
        ok = mbar_wait(&acc_empty[ap], ap_phase ^ 1u, p.status, 2);
        if (ok) ok = mbar_wait(&full_bar[stage], phase, p.status, 3);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const int n = min(kPair, kb_end - kb);
        if (elect_one()) {
          for (int j = 0; j < n; ++j) {
            const uint64_t w_desc = w_desc0 + static_cast<uint64_t>((stage * kPair + j) * (C::kWBytes >> 4));
            const uint64_t x_desc = x_desc0 + static_cast<uint64_t>((stage * kPair + j) * (C::kXBytes >> 4));
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((ap * kPair + j) * TN);
#pragma unroll
            for (int k = 0; k < BLOCK_K / 32; ++k) {
              umma_f8(d_tmem, w_desc + static_cast<uint64_t>(2 * k), x_desc + static_cast<uint64_t>(2 * k), idesc,
                      k > 0 ? 1u : 0u);
            }
          }
          umma_commit(&done_bar[stage]);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        if (++ap == C::kAccPairs) { ap = 0; ap_phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp >= C::kStagerWarp && warp < C::kStagerWarp + C::kStagers) {
    // ------------------------------------------------------------------ scale stagers
    // A slot holds, per k-block j, the TN products sa[row0 + c, kb0 + j] * sb[n-block, kb0 + j], ordered
    // so that a read-out thread finds its own CPW/4 products contiguous: token c = part*CPW + 8g + 2q + e
    // is stored at j*TN + part*CPW + q*(CPW/4) + 2g + e.
    // Global loads take far longer than a k-block, and with row-major activation scales (the grouped
    // form) every token's scales sit in a different sector, so: a slot covers 8 k-blocks (the whole
    // sector of a token, fetched as two 16-byte loads), the loads are issued before the wait for the
    // slot, and two warps take alternate fills.
    const int which = warp - C::kStagerWarp;
    const bool row_major_vec = !p.sa_ue8m0 && p.sa_stride_g == 1 && (p.sa_stride_m & 3) == 0 &&
                               (reinterpret_cast<uintptr_t>(p.sa) & 15u) == 0;
    int fill = 0;   // running count of slot fills of this CTA; fill % slots is the slot, its quotient the phase
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const SwapTile t = get_swap_tile<GROUPED, TN>(vt / split_k, p, m_tiles, n_tiles, tile_start);
      const float* sb_row = p.sb + static_cast<int64_t>(t.expert) * p.sb_stride_e +
                            static_cast<int64_t>(t.n0 / 128) * p.sb_stride_n;
      const int split = vt % split_k;
      const int kb_begin = split * kbps, kb_end = min(nkb, kb_begin + kbps);
      const bool vec = row_major_vec && (kb_begin & 3) == 0;
      for (int kb0 = kb_begin; kb0 < kb_end; kb0 += kScaleGroup, ++fill) {
        if ((fill & 1) != which) continue;
        const int slot = fill % kScaleSlots;
        const uint32_t sphase = static_cast<uint32_t>(fill / kScaleSlots) & 1u;
        float a[TN / 32][kScaleGroup];
        float bsc[kScaleGroup];
#pragma unroll
        for (int r = 0; r < TN / 32; ++r) {
          const int c = r * 32 + lane;
          const float* src = p.sa + static_cast<int64_t>(t.row0 + c) * p.sa_stride_m;
          if (vec) {
#pragma unroll
            for (int h = 0; h < kScaleGroup / 4; ++h) {
              float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
              if (c < t.valid && kb0 + 4 * h < kb_end) v = __ldg(reinterpret_cast<const float4*>(src + kb0 + 4 * h));
              a[r][4 * h] = v.x; a[r][4 * h + 1] = v.y; a[r][4 * h + 2] = v.z; a[r][4 * h + 3] = v.w;
            }
          } else if (p.sa_ue8m0) {
#pragma unroll
            for (int j = 0; j < kScaleGroup; ++j)
              a[r][j] = (c < t.valid && kb0 + j < kb_end) ? load_sa<true>(p, t.row0 + c, kb0 + j) : 0.f;
          } else {
#pragma unroll
            for (int j = 0; j < kScaleGroup; ++j)
              a[r][j] = (c < t.valid && kb0 + j < kb_end) ? load_sa<false>(p, t.row0 + c, kb0 + j) : 0.f;
          }
        }
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j)
          bsc[j] = kb0 + j < kb_end ? __ldg(sb_row + static_cast<int64_t>(kb0 + j) * p.sb_stride_g) : 0.f;
        ok = mbar_wait_warp(&scale_empty[slot], sphase ^ 1u, p.status, 5);
        if (!ok) break;
        float* dst = smem_scale + slot * C::kSlotFloats;
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j)
#pragma unroll
          for (int r = 0; r < TN / 32; ++r) {
            constexpr int CPW = C::kColsPerWarp;
            const int c = r * 32 + lane, cc = c % CPW;
            const int pos = (c / CPW) * CPW + ((cc & 7) >> 1) * (CPW / 4) + 2 * (cc >> 3) + (cc & 1);
            dst[j * TN + pos] = (kb0 + j < kb_end) ? a[r][j] * bsc[j] : 0.f;
          }
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(&scale_full[slot]);
      }
    }
    __syncwarp();
  }
  } else {
    // ====================================================================== promotion + epilogue warps
    if constexpr (C::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kEpiRegs));
    // The accumulator is read in the 16-lane fragment layout (tcgen05.ld 16x256b): a thread then holds
    // 4 weight rows x CPW/4 tokens instead of 1 row x CPW tokens, so it needs only CPW/4 scale products
    // per k-block.  (With one row per thread every thread reads every token's product, and the
    // shared-memory-to-register path, 128 B/clk per SM, was the bottleneck.)
    // Fragment h (lanes 16h..16h+15 of the quadrant): register 4g + 2rp + e <-> weight row
    // 32*quad + 16h + 8rp + lane/4, token col0 + 8g + 2(lane%4) + e.
    constexpr int CPW = C::kColsPerWarp;
    constexpr int NG = CPW / 8;          // 8-column groups per warp
    constexpr int SPT = CPW / 4;         // scale products per thread per k-block
    constexpr int FR = 4 * NG;           // registers per fragment
    const int quad = warp & 3;
    const int part = warp >> 2;
    const int q = lane & 3;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    OutT* out = static_cast<OutT*>(p.out);
    int stage = 0, ap = 0, slot = 0;
    uint32_t phase = 0, sphase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const SwapTile t = get_swap_tile<GROUPED, TN>(vt / split_k, p, m_tiles, n_tiles, tile_start);
      const int split = vt % split_k;
      const int kb_begin = split * kbps, kb_end = min(nkb, kb_begin + kbps);
      const int col0 = part * CPW;                    // first token column of this warp
      const int my_cols = min(CPW, t.valid - col0);   // <= 0: nothing to read for this warp
      const bool live = my_cols > 0;
      float acc0[FR], acc1[FR];                       // fragment 0 / fragment 1
#pragma unroll
      for (int c = 0; c < FR; ++c) acc0[c] = acc1[c] = 0.f;
      for (int kb0 = kb_begin; ok && kb0 < kb_end; kb0 += kScaleGroup) {
        ok = mbar_wait(&scale_full[slot], sphase, p.status, 6);
        if (!ok) break;
        // this thread's SPT products of k-block j: slot[j][part][q][2g + e]  (see the stagers)
        const float* sc = smem_scale + slot * C::kSlotFloats + col0 + q * SPT;
#pragma unroll 1
        for (int jj = 0; jj < kScaleGroup; jj += kPair) {
          const int kb = kb0 + jj;
          if (kb < kb_end) {
            const bool two = kb + 1 < kb_end;
            ok = mbar_wait(&done_bar[stage], phase, p.status, 4);
            if (!ok) break;
            tc_fence_after();
            if (live) {   // warp-uniform: columns past the tile's tokens hold nothing
              const uint32_t t0 = tmem_base + lane_addr + static_cast<uint32_t>((ap * kPair) * TN + col0);
              const uint32_t t1 = t0 + TN;
              float v0[FR], v1[FR], sv0[SPT], sv1[SPT];
              tmem_ld_16x256b<NG>(t0, v0);
              tmem_ld_16x256b<NG>(t0 + (16u << 16), v1);
              // the scale products are fetched while the tensor-memory reads are in flight
#pragma unroll
              for (int i = 0; i < SPT; i += 4) {
                *reinterpret_cast<float4*>(sv0 + i) = *reinterpret_cast<const float4*>(sc + jj * TN + i);
                *reinterpret_cast<float4*>(sv1 + i) = *reinterpret_cast<const float4*>(sc + (jj + 1) * TN + i);
              }
              tmem_ld_wait();
              if (two) {
                promote<NG>(acc0, v0, sv0);
                tmem_ld_16x256b<NG>(t1, v0);                 // second k-block, fragment 0, while ...
                promote<NG>(acc1, v1, sv0);                  // ... fragment 1 of the first is promoted
                tmem_ld_wait();
                tmem_ld_16x256b<NG>(t1 + (16u << 16), v1);
                promote<NG>(acc0, v0, sv1);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ap]);
                promote<NG>(acc1, v1, sv1);
              } else {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ap]);
                promote<NG>(acc0, v0, sv0);
                promote<NG>(acc1, v1, sv0);
              }
            } else {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[ap]);
            }
            if (++ap == C::kAccPairs) ap = 0;
            if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
          }
        }
        // the slot's products have been consumed by this warp
        __syncwarp();
        if (lane == 0) mbar_arrive(&scale_empty[slot]);
        if (++slot == kScaleSlots) { slot = 0; sphase ^= 1u; }
      }
      // out[token, n]: one store instruction covers 4 tokens x 8 consecutive output columns
      auto for_each_owned = [&](auto&& fn) {   // fn(value, token row, output column) for this thread's elements
        if (my_cols > 0) {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int rp = 0; rp < 2; ++rp) {
              const int n = t.n0 + quad * 32 + 16 * h + 8 * rp + (lane >> 2);
              if (n < p.N) {
#pragma unroll
                for (int g = 0; g < NG; ++g)
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    const int c = 8 * g + 2 * q + e;
                    const float val = h == 0 ? acc0[4 * g + 2 * rp + e] : acc1[4 * g + 2 * rp + e];
                    if (c < my_cols) fn(val, static_cast<int64_t>(t.row0 + col0 + c), n);
                  }
              }
            }
        }
      };
      if (ok && split_k == 1) {
        for_each_owned([&](float val, int64_t tok, int n) {
          OutT* dst = out + tok * p.ldo + n;
          *dst = cvt1(dst, val);
        });
      } else if (ok) {
        for_each_owned([&](float val, int64_t tok, int n) {
          p.partial[(static_cast<int64_t>(split) * p.M + tok) * p.N + n] = val;
        });
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
  if (warp == C::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int TN, bool GROUPED, typename OutT>
int launch_swap(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t stream) {
  using C = SwapCfg<TN>;
  auto kern = gemm_block_fp8_swapab_kernel<TN, GROUPED, OutT>;
  static bool attr_set[64] = {false};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  const long long m_tiles = (p.M + TN - 1) / TN;
  const long long n_tiles = (p.N + BLOCK_W - 1) / BLOCK_W;
  // grouped: the tile count lives on the device; token tiles <= ceil(rows/TN) + experts bounds the grid
  const long long tiles = GROUPED ? (m_tiles + p.num_experts) * n_tiles : m_tiles * n_tiles * p.split_k;
  if (tiles > 0x7fffffffLL) return B200_ERR_TOO_LARGE;   // the kernels count tiles in 32 bits
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(mw, mx, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <int TN, bool GROUPED>
int launch_swap_dtype(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, cudaStream_t stream) {
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch_swap<TN, GROUPED, __nv_bfloat16>(mw, mx, p, stream);
    case B200_DT_F16: return launch_swap<TN, GROUPED, __half>(mw, mx, p, stream);
    case B200_DT_F32: return launch_swap<TN, GROUPED, float>(mw, mx, p, stream);
    default: return B200_ERR_BAD_DTYPE;
  }
}

}  // namespace

// a: tokens [rows, K] (leading dimension lda), b: weights [w_rows, K] (dense: N rows; grouped: E*N rows).
// token_tile: 32, 64 or 128.  In the grouped form N must be a multiple of 128 (a tile must not
// straddle two experts' weight rows).
int launch_gemm_swapab(const void* a, int64_t lda, int64_t a_rows, const void* b, int64_t ldb, int64_t w_rows,
                       const GemmParams& p, bool grouped, int token_tile, cudaStream_t stream) {
  if (token_tile != 32 && token_tile != 64 && token_tile != 128) return B200_ERR_UNSUPPORTED;
  if (grouped && (p.N % BLOCK_W) != 0) return B200_ERR_UNSUPPORTED;
  CUtensorMap mw, mx;
  int rc = make_map_u8_2d(&mw, b, w_rows, p.K, ldb, BLOCK_W);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mx, a, a_rows, p.K, lda, token_tile);
  if (rc != B200_OK) return rc;
  if (grouped) {
    switch (token_tile) {
      case 32: return launch_swap_dtype<32, true>(mw, mx, p, stream);
      case 64: return launch_swap_dtype<64, true>(mw, mx, p, stream);
      default: return launch_swap_dtype<128, true>(mw, mx, p, stream);
    }
  }
  switch (token_tile) {
    case 32: return launch_swap_dtype<32, false>(mw, mx, p, stream);
    case 64: return launch_swap_dtype<64, false>(mw, mx, p, stream);
    default: return launch_swap_dtype<128, false>(mw, mx, p, stream);
  }
}

}  // namespace b200
