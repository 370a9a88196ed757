// Block-scaled FP8 GEMM with POWER-OF-TWO scales on the tensor core's own block-scaling path:
//   out = cast( sum_kb 2^(ea[m,kb] + eb[n/128,kb]) * (A_kb * B_kb^T) )
// where the exponents are UE8M0 bytes (value 2^(byte - 127)).  tcgen05.mma.kind::mxf8f6f4.block_scale applies
// one scale per row (A) and per column (B) for every 32 elements along K inside the MMA, so the products of ALL
// k-blocks accumulate in one tensor-memory accumulator and nothing is read out per k-block: the fp32 promotion
// that bounds gemm.cu (one tensor-memory read-out and 32 K fp32 FMAs per 128 x 256 x 128 k-block) disappears.
// Because the scales are powers of two the scaling is exact, and the result equals the fp32-promotion kernels'
// up to the order of the fp32 additions.
//
// Stands in for the reference's DeepGEMM path with UE8M0 scales -- its default on Blackwell
// (python/sglang/srt/layers/quantization/fp8_utils.py:215-258 deepgemm_w8a8_block_fp8_linear_with_fallback,
//  python/sglang/srt/layers/deep_gemm_wrapper/entrypoint.py:78-93 gemm_nt_f8f8bf16,
//  weights re-quantised to power-of-two scales by requant_weight_ue8m0, fp8_utils.py:370-443).
//
// Three forms: 128 x 256 and 256 x 240 tiles on one CTA per SM (below), and 256 x 256 tiles on a CTA pair
// (cta_group::2, further down).  One persistent CTA per SM, 8 warps:
//   warps 0-3  epilogue: after a tile's last k-block, each reads its rows of the accumulator(s) from tensor memory,
//              converts and stores; then hands the accumulator back.
//   warp 4     TMA producer: A box + B box per k-block, 128-byte swizzle, no multicast.
//   warp 5     MMA issuer: 4 x tcgen05.mma per k-block and 128-row half (K = 32 each).  A row's (column's) 32-bit
//              scale word holds the exponent bytes of FOUR consecutive k-blocks; the instruction's scale-factor id
//              picks the k-block's byte, so the scale tiles are copied from shared to tensor memory
//              (tcgen05.cp 32x128b.warpx4) once per four k-blocks.
//   warp 6     scale stager: builds those tiles in the layout the MMA expects -- per 128 rows a 512-byte tile,
//              row r's word at (r % 32) * 16 + (r / 32) * 4 -- from the packed activation exponents (the
//              quantiser's words, as they are) and the weights' fp32 power-of-two scales (exponent fields).
// Every mbarrier wait is bounded (common.cuh); a wait that gives up records a code and all roles drain.
#include "gemm_common.cuh"

namespace b200 {
namespace {

constexpr int BM = 128, BK = 128;
constexpr int kSfSlots = 3;                             // scale-factor ring: one slot serves four k-blocks
constexpr int kSfaBytes = 512, kSfbBytes = 1024;       // one 512-byte tile per 128 rows of A, two for the (up to 256) columns of B
constexpr int kThreadsMx = 256;
constexpr int kThreadsMxSilu = 384;   // the fused-activation form: four more epilogue warps (warps 8-11)
constexpr int kGroupMMx = 32;

// Tile shapes (rows x columns per CTA) and their tensor-memory maps:
//   128 x 256  one accumulator [0,256), scale factors at [256,268).
//   128 x 240  two accumulators [0,240) and [256,496), scale factors at [240,252): a tile's read-out overlaps the
//              next tile's MMAs.
//   256 x 240  (MSUB = 2) two 128-row halves that share every B stage: accumulators [0,240) and [256,496), scale
//              factors of the two halves and of B at [240,256).  One CTA per SM moves 188 bytes of shared memory per
//              clock at full MMA rate with a 128-row tile (TMA writes plus operand reads); sharing B between two
//              halves brings that to 125.
template <int BN, int MSUB>
struct MxCfg {
  static_assert(MSUB == 1 || BN <= 240, "two 128-row halves need the 240-wide tile");
  static constexpr int kStages = MSUB == 2 ? 3 : (BN <= 192 ? 5 : 4);
  static constexpr int kNumAcc = (BN <= 240 && MSUB == 1) ? 2 : 1;   // accumulator double buffering across tiles
  static constexpr int kABytes = MSUB * BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kSfaCol = BN <= 240 ? 240 : 256;          // 4 columns per 128-row half
  static constexpr uint32_t kSfbCol = kSfaCol + 4 * MSUB;
  static constexpr uint32_t kAccStride = 256;
  static constexpr int kSfBytes = MSUB * kSfaBytes + kSfbBytes;
  static constexpr int kSmem = kStages * kStageBytes + kSfSlots * kSfBytes + 1024 + 256;
  static_assert(kBBytes % 1024 == 0, "stage bases must keep the 1024-byte alignment of the swizzle pattern");
  static_assert(kSmem <= 227 * 1024, "shared memory");
};

struct MxParams {
  const uint32_t* sa;       // packed exponents: word (m, g4) at sa[g4 * sa_stride_pack + m * sa_stride_m]
  const float* sb;          // [N/128, K/128] fp32 powers of two, element (nb, kb) at sb[nb * sb_stride_n + kb * sb_stride_g]
  void* out;
  int64_t sa_stride_m, sa_stride_pack, sb_stride_n, sb_stride_g, ldo;
  int M, N, K;
  int out_dtype;
  int* status;
  // grouped form: problem i multiplies rows [offsets[i], offsets[i] + rows[i * rows_stride]) of A with weight slice
  // experts[i] (i itself when experts is null): weight rows [e * N, (e + 1) * N), scales at sb + e * sb_stride_e.
  const int* offsets;
  const int* rows;
  const int* experts;
  int64_t rows_stride, sb_stride_e;
  // packed activation exponents of problem i: indexed by the GLOBAL row of A (sa_stride_problem < 0; DeepGEMM's
  // contiguous layout), or per problem by the row inside it at sa + i * sa_stride_problem (its masked layout)
  int64_t sa_stride_problem;
  int num_problems, num_weight_experts;
  // SiLU*mul + power-of-two quantisation in the epilogue (grouped form, expert GEMM 1): N is the number of OUTPUT
  // columns (the intermediate size I); weight slice e holds 2 * N rows, gate rows first; `out` receives e4m3 codes
  // [rows, N] (leading dimension ldo bytes) and out_s the packed exponent words (word (row, w) at
  // out_s[w * out_s_stride_pack + row]).
  uint32_t* out_s;
  int64_t out_s_stride_pack;
};

constexpr int kMaxProblems = 2048;

// One output tile: rows [row0, row0 + valid) of A / out, column block n_blk of weight slice e_w.
struct MxTile {
  int row0, valid, n_blk, e_w;
  int64_t sa_base;   // word (row, g4) of the packed exponents sits at sa[sa_base + g4 * sa_stride_pack + row * sa_stride_m]
};

// Shared-memory descriptor of a scale-factor tile for tcgen05.cp: 32 rows x 16 bytes, rows contiguous, no
// swizzle -- four 8-row core matrices 128 bytes apart (stride byte offset), nothing along the other dimension.
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 16;   // leading byte offset (unused for a single 16-byte column)
  d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// Instruction descriptor of the block-scaled kind: b_sf_id [4,6), a/b format e4m3 = 0 at [7,10) / [10,13), both
// K-major, N>>3 at [17,23), scale format UE8M0 = 1 at [23], M>>4 at [24,29), a_sf_id [29,31).  The scale-factor id
// picks one of the four bytes of a row's (column's) 32-bit scale word.
__device__ __forceinline__ uint32_t idesc_mx(int m, int n, uint32_t sf_id) {
  return (sf_id << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(m >> 4) << 24) |
         (sf_id << 29);
}

__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}

// Grouped tile order inside a problem.  Column blocks outermost (the row tiles that share a weight block run side by
// side) for a problem with at least four row tiles -- a problem of a few thousand rows then behaves like the dense
// kernel: activations in L2, every weight block from HBM once -- and for deep reductions (K >= 4096); otherwise
// column blocks fastest.  Measured on the two expert GEMMs of a 256-expert layer with one or two row tiles per
// expert: K = 7168 is 4-5 % faster with the column blocks outermost, K = 2048 is 11 % slower.
constexpr int kRowTilesColumnMajor = 4;
constexpr int kDeepK = 4096;

__device__ __forceinline__ void mx_tile_coords(int tile, int m_blocks, int n_blocks, int& m_blk, int& n_blk) {
  const int group_size = kGroupMMx * n_blocks;
  const int group = tile / group_size;
  const int first_m = group * kGroupMMx;
  const int rows = min(kGroupMMx, m_blocks - first_m);
  const int in_group = tile - group * group_size;
  m_blk = first_m + in_group % rows;
  n_blk = in_group / rows;
}

// Dense: groups of 32 row blocks x all column blocks.  Grouped: the problems laid end to end (prefix table
// `tile_start` of row tiles, built once per CTA), the order inside a problem as described above.  Offsets and counts come from
// device memory and are clamped into the row range: a table that does not match the buffers cannot send a load or a
// store out of bounds.
template <bool GROUPED, int TILE_M>
__device__ __forceinline__ MxTile mx_get_tile(int tile, const MxParams& p, int m_blocks, int n_blocks,
                                              const int* tile_start) {
  MxTile t;
  if constexpr (!GROUPED) {
    int m_blk;
    mx_tile_coords(tile, m_blocks, n_blocks, m_blk, t.n_blk);
    t.row0 = m_blk * TILE_M;
    t.valid = min(TILE_M, p.M - t.row0);
    t.e_w = 0;
    t.sa_base = 0;
  } else {
    int lo = 0, hi = p.num_problems;            // last problem whose first tile is <= tile
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_start[mid] * n_blocks <= tile) lo = mid; else hi = mid;
    }
    const int local = tile - tile_start[lo] * n_blocks;
    const int row_tiles = max(tile_start[lo + 1] - tile_start[lo], 1);
    int sub;
    if (row_tiles >= kRowTilesColumnMajor || p.K >= kDeepK) {
      mx_tile_coords(local, row_tiles, n_blocks, sub, t.n_blk);    // groups of 32 row tiles, like the dense form
    } else {
      sub = local / n_blocks;
      t.n_blk = local - sub * n_blocks;
    }
    const int rows = __ldg(p.rows + static_cast<int64_t>(lo) * p.rows_stride);
    const int off = __ldg(p.offsets + lo);
    t.row0 = min(max(off + sub * TILE_M, 0), p.M - 1);
    t.sa_base = p.sa_stride_problem < 0 ? 0 : lo * p.sa_stride_problem - off * p.sa_stride_m;
    t.valid = max(1, min(min(TILE_M, rows - sub * TILE_M), p.M - t.row0));
    const int e = p.experts ? __ldg(p.experts + lo) : lo;
    t.e_w = min(max(e, 0), p.num_weight_experts - 1);
  }
  return t;
}

template <int BN, int MSUB, bool GROUPED, typename OutT, bool SILU_Q = false>
__global__ void __launch_bounds__((SILU_Q || (BN == 256 && MSUB == 1)) ? kThreadsMxSilu : kThreadsMx, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const MxParams p) {
  using C = MxCfg<BN, MSUB>;
  static_assert(!SILU_Q || (GROUPED && BN == 256 && MSUB == 1), "the fused activation epilogue is built for the grouped 128 x 256 tile");
  // SILU_Q: a tile is 128 rows x (128 gate columns | the 128 up columns of the same outputs); n-blocks count
  // 128 OUTPUT columns
  constexpr int kOutN = SILU_Q ? 128 : BN;
  // the 128 x 256 tile runs with eight epilogue warps (warps 0-3 and 8-11: two per row quadrant, 128 columns each)
  constexpr bool kWide8 = (BN == 256 && MSUB == 1);
  constexpr int kStagesMx = C::kStages;
  constexpr int kABytesMx = C::kABytes;
  constexpr int kSfBytes = C::kSfBytes;
  constexpr int kTileM = BM * MSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStagesMx * kABytesMx;
  uint8_t* smem_sf = smem + kStagesMx * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sf + kSfSlots * kSfBytes);
  uint64_t* full_bar = bars;                        // operands of the stage landed (TMA)
  uint64_t* empty_bar = full_bar + kStagesMx;       // the k-block's MMAs completed: stage reusable
  uint64_t* sf_full = empty_bar + kStagesMx;        // scale-factor slot written (stager)
  uint64_t* sf_empty = sf_full + kSfSlots;          // the slot's four k-blocks completed
  uint64_t* acc_full = sf_empty + kSfSlots;         // the tile's last MMA completed
  uint64_t* acc_empty = acc_full + 2;               // the epilogue has read the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (p.M + kTileM - 1) / kTileM;
  const int n_blocks = (p.N + kOutN - 1) / kOutN;
  const int nkb = (p.K + BK - 1) / BK;
  __shared__ int tile_start[GROUPED ? kMaxProblems + 1 : 1];
  __shared__ float amax_x[SILU_Q ? 2 : 1][2][SILU_Q ? BM : 1];   // fused-activation epilogue: maxima of the two column halves
  __shared__ uint64_t xbar[4];                                    // ... and where the two warps of a row quadrant meet
  if constexpr (GROUPED) {
    // row tiles per problem (none for an empty problem or one whose weight slice does not exist) ...
    for (int i = threadIdx.x; i < p.num_problems; i += blockDim.x) {
      const int rows = __ldg(p.rows + static_cast<int64_t>(i) * p.rows_stride);
      const int e = p.experts ? __ldg(p.experts + i) : i;
      tile_start[i + 1] = (rows > 0 && e >= 0 && e < p.num_weight_experts) ? (min(rows, p.M) + kTileM - 1) / kTileM : 0;
    }
    __syncthreads();
    // ... and their running sum, by one warp
    if (warp == 0) {
      int carry = 0;
      for (int base = 0; base < p.num_problems; base += 32) {
        int v = (base + lane < p.num_problems) ? tile_start[base + lane + 1] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, v, off);
          if (lane >= off) v += u;
        }
        if (base + lane < p.num_problems) tile_start[base + lane + 1] = carry + v;
        carry += __shfl_sync(0xffffffffu, v, 31);
      }
      if (lane == 0) tile_start[0] = 0;
    }
    __syncthreads();
  }
  const int num_tiles = GROUPED ? tile_start[p.num_problems] * n_blocks : m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStagesMx; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < kSfSlots; ++i) {
      mbar_init(&sf_full[i], 1);
      mbar_init(&sf_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], kWide8 ? 8 : 4);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&xbar[i], 2);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const MxTile t = mx_get_tile<GROUPED, kTileM>(tile, p, m_blocks, n_blocks, tile_start);
      // SILU_Q: the weight map's box is 128 rows; the gate rows and the up rows of the tile's 128 outputs land in
      // the two halves of the stage
      const int w_row0 = SILU_Q ? t.e_w * 2 * p.N + t.n_blk * 128 : t.e_w * p.N + t.n_blk * BN;
      for (int kb = 0; kb < nkb; ++kb) {
        ok = mbar_wait_warp(&empty_bar[stage], phase ^ 1u, p.status, 41);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&full_bar[stage], C::kStageBytes);
          tma_load_2d(smem_a + stage * kABytesMx, &map_a, &full_bar[stage], kb * BK, t.row0);
          if constexpr (SILU_Q) {
            tma_load_2d(smem_b + stage * C::kBBytes, &map_b, &full_bar[stage], kb * BK, w_row0);
            tma_load_2d(smem_b + stage * C::kBBytes + 128 * BK, &map_b, &full_bar[stage], kb * BK, w_row0 + p.N);
          } else {
            tma_load_2d(smem_b + stage * C::kBBytes, &map_b, &full_bar[stage], kb * BK, w_row0);
          }
        }
        __syncwarp();
        if (++stage == kStagesMx) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    // Per k-block: four MMAs (K = 32 each) into the tile's accumulator; the scale-factor id of all four is the
    // k-block's position inside its group of four (one byte of every row's / column's scale word per k-block).
    // The barrier test for the NEXT k-block's operands is made between the third and the fourth MMA, so that its
    // latency and the loop's bookkeeping run while queued MMAs keep the tensor pipe busy.
    const uint64_t a_desc0 = umma_desc_k128(smem_u32(smem_a));
    const uint64_t b_desc0 = umma_desc_k128(smem_u32(smem_b));
    int stage = 0, slot = 0, acc = 0;
    uint32_t phase = 0, sphase = 0, acc_phase[2] = {0, 0};
    bool ok = true;
    bool next_ready = false;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      ok = mbar_wait(&acc_empty[acc], acc_phase[acc] ^ 1u, p.status, 42);   // the epilogue has drained this accumulator
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * C::kAccStride;
      // two-half tile of a problem with at most 128 rows left: the second half's MMAs are not issued
      int nh = MSUB;
      if constexpr (GROUPED && MSUB == 2)
        nh = mx_get_tile<GROUPED, kTileM>(tile, p, m_blocks, n_blocks, tile_start).valid > BM ? 2 : 1;
      const int hl = nh - 1;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!next_ready) {
          ok = mbar_wait(&full_bar[stage], phase, p.status, 43);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        const int j = kb & 3;
        if (j == 0) {
          ok = mbar_wait(&sf_full[slot], sphase, p.status, 44);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        tc_fence_after();
        const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kABytesMx >> 4));
        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage * (C::kBBytes >> 4));
        const uint32_t idesc = idesc_mx(BM, BN, static_cast<uint32_t>(j));
        const int nstage = (stage + 1 == kStagesMx) ? 0 : stage + 1;
        const uint32_t nphase = (stage + 1 == kStagesMx) ? (phase ^ 1u) : phase;
        const bool last_kb = (kb == nkb - 1);
        const bool elected = elect_one();
        if (elected) {
          if (j == 0) {
            const uint32_t sf_addr = smem_u32(smem_sf + slot * kSfBytes);
#pragma unroll
            for (int h = 0; h < MSUB; ++h) tmem_cp_sf(tmem_base + C::kSfaCol + 4 * h, sf_desc(sf_addr + h * kSfaBytes));
            tmem_cp_sf(tmem_base + C::kSfbCol, sf_desc(sf_addr + MSUB * kSfaBytes));
            tmem_cp_sf(tmem_base + C::kSfbCol + 4, sf_desc(sf_addr + MSUB * kSfaBytes + 512));
          }
#pragma unroll
          for (int i = 0; i < 4 * MSUB - 1; ++i) {
            const int k = i / MSUB, h = i % MSUB;      // K step, 128-row half
            if (h >= nh || (k == 3 && h == hl)) continue;
            umma_mx(d_tmem + h * C::kAccStride, a_desc + static_cast<uint64_t>(2 * k + h * ((BM * BK) >> 4)),
                    b_desc + static_cast<uint64_t>(2 * k), idesc, tmem_base + C::kSfaCol + 4 * h, tmem_base + C::kSfbCol,
                    (kb > 0 || k > 0) ? 1u : 0u);
          }
        }
        // all lanes test (warp-uniform outcome); a tile's last k-block is followed by another tile's first
        next_ready = mbar_try_wait(&full_bar[nstage], nphase, 1);
        next_ready = __all_sync(0xffffffffu, next_ready);
        if (elected) {
          const int h = hl;
          umma_mx(d_tmem + h * C::kAccStride, a_desc + static_cast<uint64_t>(6 + h * ((BM * BK) >> 4)), b_desc + 6, idesc,
                  tmem_base + C::kSfaCol + 4 * h, tmem_base + C::kSfbCol, 1u);
          umma_commit(&empty_bar[stage]);
          if (j == 3 || last_kb) umma_commit(&sf_empty[slot]);
          if (last_kb) umma_commit(&acc_full[acc]);
        }
        __syncwarp();
        stage = nstage;
        phase = nphase;
        if (j == 3 || last_kb) {
          if (++slot == kSfSlots) { slot = 0; sphase ^= 1u; }
        }
      }
      acc_phase[acc] ^= 1u;
      if (C::kNumAcc == 2) acc ^= 1;
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------------------------ scale-factor stager
    // One slot per group of four k-blocks.  A row's 32-bit word holds the four k-blocks' exponent bytes -- for the
    // activations exactly the packed word the quantiser wrote -- at (row % 32) * 16 + (row / 32) * 4 of the 512-byte
    // tile; a weight column's word is built from the four fp32 scales of its 128 x 128 blocks (exponent fields).
    int slot = 0;
    uint32_t sphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const MxTile t = mx_get_tile<GROUPED, kTileM>(tile, p, m_blocks, n_blocks, tile_start);
      const int row0 = t.row0, n_blk = t.n_blk, row_end = t.row0 + t.valid;
      const float* sb_e = p.sb + (GROUPED ? static_cast<int64_t>(t.e_w) * p.sb_stride_e : 0);
      [[maybe_unused]] const int up_blocks0 = p.N >> 7;     // SILU_Q: first scale block of the up rows
      for (int kb0 = 0; kb0 < nkb; kb0 += 4) {
        uint32_t w[4 * MSUB];
#pragma unroll
        for (int j = 0; j < 4 * MSUB; ++j) {
          const int row = row0 + lane + 32 * j;
          w[j] = (row < row_end) ? __ldg(p.sa + t.sa_base + static_cast<int64_t>(kb0 >> 2) * p.sa_stride_pack + row * p.sa_stride_m) : 0u;
        }
        uint32_t wb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // column (i / 4) * 128 + (i % 4) * 32 + lane of the tile
          const int col = min(n_blk * BN + (i >> 2) * 128 + (i & 3) * 32 + lane, p.N - 1);
          const int wblock = SILU_Q ? ((i >> 2) ? up_blocks0 + n_blk : n_blk) : (col >> 7);
          const float* sp = sb_e + static_cast<int64_t>(wblock) * p.sb_stride_n;
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int kb = min(kb0 + k, nkb - 1);
            word |= ((__float_as_uint(__ldg(sp + static_cast<int64_t>(kb) * p.sb_stride_g)) >> 23) & 0xffu) << (8 * k);
          }
          wb[i] = word;
        }
        ok = mbar_wait_warp(&sf_empty[slot], sphase ^ 1u, p.status, 45);
        if (!ok) break;
        uint8_t* sf = smem_sf + slot * kSfBytes;
#pragma unroll
        for (int h = 0; h < MSUB; ++h)
          *reinterpret_cast<uint4*>(sf + h * kSfaBytes + lane * 16) = make_uint4(w[4 * h], w[4 * h + 1], w[4 * h + 2], w[4 * h + 3]);
        *reinterpret_cast<uint4*>(sf + MSUB * kSfaBytes + lane * 16) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
        *reinterpret_cast<uint4*>(sf + MSUB * kSfaBytes + 512 + lane * 16) = make_uint4(wb[4], wb[5], wb[6], wb[7]);
        fence_proxy_async_smem();     // generic-proxy writes -> visible to the tensor core's copy
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_full[slot]);
        if (++slot == kSfSlots) { slot = 0; sphase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp < 4 || (kWide8 && warp >= 8)) {
    // ------------------------------------------------------------------ epilogue
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (p.ldo % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    [[maybe_unused]] uint32_t xpar = 0;
    int acc = 0;
    uint32_t acc_phase[2] = {0, 0};
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const MxTile t = mx_get_tile<GROUPED, kTileM>(tile, p, m_blocks, n_blocks, tile_start);
      const int n_blk = t.n_blk;
      const int m_end = t.row0 + t.valid;
      ok = mbar_wait(&acc_full[acc], acc_phase[acc], p.status, 46);
      if (!ok) break;
      tc_fence_after();
      if constexpr (SILU_Q) {
        // gate = columns [0, 128), up = [128, 256) of the accumulator: round both to OutT (what GEMM 1 would have
        // stored), SiLU(gate) * up in fp32, round to OutT (what the activation kernel stores), then the power-of-two
        // quantisation of the row's 128 values -- the arithmetic of the unfused sequence, value for value.
        // Two warps share a row quadrant: warps 0-3 take outputs [0, 64), warps 8-11 outputs [64, 128); the halves'
        // maxima meet in shared memory.  The accumulator goes back to the MMA warp as soon as both have read it, and
        // the arithmetic runs under the next tile's MMAs.
        const int quad = warp & 3, half = warp >> 3;
        const int row_in_tile = quad * 32 + lane;
        const int m = t.row0 + row_in_tile;
        const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(acc) * C::kAccStride + half * 64;
        // phase one: the accumulator's values rounded to OutT and packed (64 registers), then the accumulator goes
        // back; phase two: the arithmetic, from registers
        uint32_t gp[32], up[32];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float g[16], u[16];
          tmem_ld16(taddr + ch * 16, g);
          tmem_ld16(taddr + 128 + ch * 16, u);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; c += 2) {
            gp[ch * 8 + c / 2] = pack2(out, g[c], g[c + 1]);
            up[ch * 8 + c / 2] = pack2(out, u[c], u[c + 1]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        auto lo_of = [](uint32_t w) { OutT v; *reinterpret_cast<uint16_t*>(&v) = static_cast<uint16_t>(w & 0xffffu); return static_cast<float>(v); };
        auto hi_of = [](uint32_t w) { OutT v; *reinterpret_cast<uint16_t*>(&v) = static_cast<uint16_t>(w >> 16); return static_cast<float>(v); };
        uint32_t y[32];                       // 64 activations in OutT, packed in pairs
        float amax = 1e-10f;                  // eps of the quantiser
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float g0 = lo_of(gp[i]), g1 = hi_of(gp[i]);
          const float f0 = (g0 / (1.0f + __expf(-g0))) * lo_of(up[i]);
          const float f1 = (g1 / (1.0f + __expf(-g1))) * hi_of(up[i]);
          y[i] = pack2(out, f0, f1);
          amax = fmaxf(amax, fmaxf(fabsf(lo_of(y[i])), fabsf(hi_of(y[i]))));
        }
        // exchange through shared memory, double-buffered by tile parity; the two warps of a quadrant meet at an
        // mbarrier (bounded wait, like every other wait of the kernel)
        amax_x[xpar][half][row_in_tile] = amax;
        __syncwarp();
        if (lane == 0) mbar_arrive(&xbar[quad]);
        ok = mbar_wait(&xbar[quad], xpar, p.status, 47);
        if (!ok) break;
        amax = fmaxf(amax, amax_x[xpar][half ^ 1][row_in_tile]);
        xpar ^= 1u;
        const float scale = exp2f(ceilf(log2f(fmaxf(__fdiv_rn(amax, 448.0f), 1e-10f))));
        const float rinv = __frcp_rn(scale);          // exact: the scale is a power of two
        if (m < m_end) {
          uint8_t* qrow = reinterpret_cast<uint8_t*>(p.out) + static_cast<int64_t>(m) * p.ldo + n_blk * 128 + half * 64;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float q4[4];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const uint32_t packed = y[v * 8 + j * 2 + e];
                OutT lo, hi;
                *reinterpret_cast<uint16_t*>(&lo) = static_cast<uint16_t>(packed & 0xffffu);
                *reinterpret_cast<uint16_t*>(&hi) = static_cast<uint16_t>(packed >> 16);
                q4[2 * e] = fminf(fmaxf(static_cast<float>(lo) * rinv, -448.0f), 448.0f);
                q4[2 * e + 1] = fminf(fmaxf(static_cast<float>(hi) * rinv, -448.0f), 448.0f);
              }
              const uint32_t c01 = __nv_cvt_float2_to_fp8x2(make_float2(q4[0], q4[1]), __NV_SATFINITE, __NV_E4M3);
              const uint32_t c23 = __nv_cvt_float2_to_fp8x2(make_float2(q4[2], q4[3]), __NV_SATFINITE, __NV_E4M3);
              w4[j] = c01 | (c23 << 16);
            }
            *reinterpret_cast<uint4*>(qrow + v * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
          if (half == 0)
            reinterpret_cast<uint8_t*>(p.out_s)[(static_cast<int64_t>(n_blk >> 2) * p.out_s_stride_pack + m) * 4 + (n_blk & 3)] =
                static_cast<uint8_t>(static_cast<int>(log2f(scale)) + 127);
        }
        acc_phase[acc] ^= 1u;
        if (C::kNumAcc == 2) acc ^= 1;
        continue;
      }
      if constexpr (kWide8 && sizeof(OutT) == 2) {
        // 16-bit output: each warp reads its 32 rows x 128 columns out of tensor memory, rounds and packs them into
        // 64 registers, hands the accumulator back at once and only then stores -- the stores (32 rows per
        // instruction, 16 bytes each) run under the next tile's MMAs.
        const int half = warp >> 3;
        const int m = t.row0 + (warp & 3) * 32 + lane;
        const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(acc) * C::kAccStride + half * 128;
        uint32_t pk[64];
#pragma unroll
        for (int ch = 0; ch < 8; ch += 2) {
          float v[32];
          tmem_ld16(taddr + ch * 16, *reinterpret_cast<float(*)[16]>(v));
          tmem_ld16(taddr + (ch + 1) * 16, *reinterpret_cast<float(*)[16]>(v + 16));
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; c += 2) pk[ch * 8 + c / 2] = pack2(out, v[c], v[c + 1]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        const int n0 = n_blk * BN + half * 128;
        if (m < m_end && n0 < p.N) {
          OutT* dst = out + static_cast<int64_t>(m) * p.ldo + n0;
          const int valid = min(p.N - n0, 128);
          if (vec_ok && valid == 128) {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              reinterpret_cast<uint4*>(dst)[c] = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              OutT lo, hi;
              *reinterpret_cast<uint16_t*>(&lo) = static_cast<uint16_t>(pk[c] & 0xffffu);
              *reinterpret_cast<uint16_t*>(&hi) = static_cast<uint16_t>(pk[c] >> 16);
              if (2 * c < valid) dst[2 * c] = lo;
              if (2 * c + 1 < valid) dst[2 * c + 1] = hi;
            }
          }
        }
        acc_phase[acc] ^= 1u;
        if (C::kNumAcc == 2) acc ^= 1;
        continue;
      }
      // (fp32 output, and the 240-wide tiles: chunk by chunk, the accumulator is handed back after the last load)
      constexpr int kChunks = (kWide8 ? 128 : BN) / 16;
      [[maybe_unused]] const int col_half = kWide8 ? (warp >> 3) : 0;
      const int nh = (MSUB == 2 && t.valid <= BM) ? 1 : MSUB;   // halves that hold rows of the problem
#pragma unroll 1
      for (int h = 0; h < nh; ++h) {
        const int m = t.row0 + h * BM + (warp & 3) * 32 + lane;
        const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(MSUB == 2 ? h : acc) * C::kAccStride +
                               col_half * 128;
#pragma unroll 1
        for (int ch = 0; ch < kChunks; ch += 2) {
          float v[32];
          tmem_ld16(taddr + ch * 16, *reinterpret_cast<float(*)[16]>(v));
          if (ch + 1 < kChunks) tmem_ld16(taddr + (ch + 1) * 16, *reinterpret_cast<float(*)[16]>(v + 16));
          tmem_ld_wait();
          if (h == nh - 1 && ch + 2 >= kChunks) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
          }
          const int n0 = n_blk * BN + col_half * 128 + ch * 16;
          const int width = (ch + 1 < kChunks) ? 32 : 16;
          if (m < m_end && n0 < p.N)
            store_row<32>(out + static_cast<int64_t>(m) * p.ldo + n0, v, min(p.N - n0, width), vec_ok && width == 32);
        }
      }
      acc_phase[acc] ^= 1u;
      if (C::kNumAcc == 2) acc ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(p.status) != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int BN, int MSUB, bool GROUPED, typename OutT>
int launch_mx(const CUtensorMap& ma, const CUtensorMap& mb, const MxParams& p, cudaStream_t stream) {
  using C = MxCfg<BN, MSUB>;
  auto kern = gemm_mx_kernel<BN, MSUB, GROUPED, OutT>;
  static bool attr_set[64] = {false};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
    attr_set[dev & 63] = true;
  }
  // grouped: the tile count lives on the device; row tiles <= ceil(rows / tile) + problems bounds the grid
  const long long m_tiles = (p.M + BM * MSUB - 1) / (BM * MSUB) + (GROUPED ? p.num_problems : 0);
  const long long tiles = m_tiles * ((p.N + BN - 1) / BN);
  if (tiles > 0x7fffffffLL) return B200_ERR_TOO_LARGE;   // the kernels count tiles in 32 bits
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  kern<<<grid, (BN == 256 && MSUB == 1) ? kThreadsMxSilu : kThreadsMx, C::kSmem, stream>>>(ma, mb, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <int BN, int MSUB, bool GROUPED = false>
int launch_mx_dtype(const void* a, int64_t lda, const void* b, int64_t ldb, const MxParams& p, cudaStream_t st) {
  CUtensorMap ma, mb;
  int rc = make_map_u8_2d(&ma, a, p.M, p.K, lda, BM * MSUB);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, GROUPED ? static_cast<int64_t>(p.N) * p.num_weight_experts : p.N, p.K, ldb, BN);
  if (rc != B200_OK) return rc;
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch_mx<BN, MSUB, GROUPED, __nv_bfloat16>(ma, mb, p, st);
    case B200_DT_F16: return launch_mx<BN, MSUB, GROUPED, __half>(ma, mb, p, st);
    default: return launch_mx<BN, MSUB, GROUPED, float>(ma, mb, p, st);
  }
}


template <typename OutT>
int launch_mx_silu(const void* a, int64_t lda, const void* b, int64_t ldb, const MxParams& p, cudaStream_t stream) {
  using C = MxCfg<256, 1>;
  CUtensorMap ma, mb;
  int rc = make_map_u8_2d(&ma, a, p.M, p.K, lda, BM);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, static_cast<int64_t>(2) * p.N * p.num_weight_experts, p.K, ldb, 128);
  if (rc != B200_OK) return rc;
  auto kern = gemm_mx_kernel<256, 1, true, OutT, true>;   // 12 warps
  static bool attr_set[64] = {false};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
    attr_set[dev & 63] = true;
  }
  const long long m_tiles = (p.M + BM - 1) / BM + p.num_problems;
  const long long tiles = m_tiles * ((p.N + 127) / 128);
  if (tiles > 0x7fffffffLL) return B200_ERR_TOO_LARGE;   // the kernels count tiles in 32 bits
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  kern<<<grid, kThreadsMxSilu, C::kSmem, stream>>>(ma, mb, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ============================================================================================ CTA-pair form
// Two CTAs of a cluster work on one 256 x 256 tile (tcgen05 cta_group::2): each CTA loads its own 128 rows of A
// and HALF of the weight tile (128 of the 256 columns) per k-block, the leader CTA's elected thread issues
// M256 x N256 x K32 MMAs that both SMs execute, each on its own rows with the weight halves of both.  Per SM and
// k-block that is 32 KB written to and 32 KB read from shared memory and 32 KB fetched from L2 for 512 tensor
// cycles -- the single-CTA form moves 48 + 48 + 48 KB -- so the operand feed no longer sets the pace.
// Scale factors: every CTA's stager builds the tile of its OWN rows and the tile of ALL 256 columns in its own
// shared memory; the leader's tcgen05.cp.cta_group::2 copies, in each CTA, that CTA's tiles into its tensor memory
// (like the MMA, the copy acts on both CTAs with the same shared-memory offset and the same tensor-memory address).
// Barriers: operands -> the leader's full barrier (both CTAs' loads credit it); scale tiles -> the leader's
// sf_full (one arrival per CTA, cluster-scope release); completions are committed to both CTAs at once
// (stage reusable, scale slot reusable, accumulator ready); accumulator drained -> the leader's acc_empty
// (four epilogue warps of each CTA).
constexpr int kPairStages = 6;
constexpr int kPairABytes = BM * BK;            // 128 rows of A per CTA
constexpr int kPairBBytes = 128 * BK;           // 128 of the tile's 256 weight rows per CTA
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairSfBytes = kSfaBytes + kSfbBytes;
constexpr int kPairSmem = kPairStages * kPairStageBytes + kSfSlots * kPairSfBytes + 1024 + 256;
constexpr uint32_t kPairSfaCol = 256, kPairSfbCol = 260;
static_assert(kPairSmem <= 227 * 1024, "shared memory");

__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mx_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
      : "memory");
}
// Arrival on the leader CTA's barrier that publishes this CTA's shared-memory writes to the cluster.
__device__ __forceinline__ void mbar_arrive_leader_release(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, 0;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t}\n"
      ::"r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 0xffu) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        report_wait_failure(status, code);
        return false;
      }
    }
  }
  return true;
}

template <typename OutT>
__global__ void __launch_bounds__(kThreadsMxSilu, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const MxParams p) {
  constexpr int kTileM = 2 * BM, kTileN = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kPairStages * kPairABytes;
  uint8_t* smem_sf = smem + kPairStages * kPairStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_sf + kSfSlots * kPairSfBytes);
  uint64_t* full_bar = bars;                        // leader's copy is live: operands of both CTAs landed
  uint64_t* empty_bar = full_bar + kPairStages;     // per CTA: the k-block's MMAs completed
  uint64_t* sf_full = empty_bar + kPairStages;      // leader's copy is live: both CTAs' scale tiles written
  uint64_t* sf_empty = sf_full + kSfSlots;          // per CTA: the slot's k-blocks completed
  uint64_t* acc_full = sf_empty + kSfSlots;         // per CTA: the tile's last MMA completed
  uint64_t* acc_empty = acc_full + 1;               // leader's copy is live: both CTAs have read their accumulators
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_blocks = (p.M + kTileM - 1) / kTileM;
  const int n_blocks = (p.N + kTileN - 1) / kTileN;
  const int nkb = (p.K + BK - 1) / BK;
  const int num_tiles = m_blocks * n_blocks;

  cluster_sync_all();   // both CTAs are resident before tensor memory is paired
  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(&full_bar[i], 2);    // one arrival per CTA's producer (+ both CTAs' bytes)
      mbar_init(&empty_bar[i], 1);   // the leader's commit, delivered to both CTAs
    }
    for (int i = 0; i < kSfSlots; ++i) {
      mbar_init(&sf_full[i], 2);     // one arrival per CTA's stager
      mbar_init(&sf_empty[i], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 16);        // eight epilogue warps in each CTA
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 5) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer (each CTA)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      mx_tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
      const int row_a = m_blk * kTileM + static_cast<int>(rank) * BM;
      const int row_b = n_blk * kTileN + static_cast<int>(rank) * 128;
      for (int kb = 0; kb < nkb; ++kb) {
        ok = mbar_wait_warp(&empty_bar[stage], phase ^ 1u, p.status, 51);
        if (!ok) break;
        if (elect_one()) {
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * kPairStageBytes);
          tma_load_2d_pair(smem_a + stage * kPairABytes, &map_a, &full_bar[stage], kb * BK, row_a);
          tma_load_2d_pair(smem_b + stage * kPairBBytes, &map_b, &full_bar[stage], kb * BK, row_b);
          if (!leader) mbar_arrive_cluster(&full_bar[stage], 0);
        }
        __syncwarp();
        if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader) {
      const uint64_t a_desc0 = umma_desc_k128(smem_u32(smem_a));
      const uint64_t b_desc0 = umma_desc_k128(smem_u32(smem_b));
      int stage = 0, slot = 0;
      uint32_t phase = 0, sphase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        ok = mbar_wait(acc_empty, acc_phase ^ 1u, p.status, 52);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, p.status, 53);
          const int j = kb & 3;
          if (ok && j == 0) ok = mbar_wait_cluster(&sf_full[slot], sphase, p.status, 54);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (kPairABytes >> 4));
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage * (kPairBBytes >> 4));
          const uint32_t idesc = idesc_mx(kTileM, kTileN, static_cast<uint32_t>(j));
          const bool last_kb = (kb == nkb - 1);
          if (elect_one()) {
            if (j == 0) {
              const uint32_t sf_addr = smem_u32(smem_sf + slot * kPairSfBytes);
              tmem_cp_sf_pair(tmem_base + kPairSfaCol, sf_desc(sf_addr));
              tmem_cp_sf_pair(tmem_base + kPairSfbCol, sf_desc(sf_addr + kSfaBytes));
              tmem_cp_sf_pair(tmem_base + kPairSfbCol + 4, sf_desc(sf_addr + kSfaBytes + 512));
            }
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_mx_pair(tmem_base, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                           tmem_base + kPairSfaCol, tmem_base + kPairSfbCol, (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit_pair(&empty_bar[stage], 3);
            if (j == 3 || last_kb) umma_commit_pair(&sf_empty[slot], 3);
            if (last_kb) umma_commit_pair(acc_full, 3);
          }
          __syncwarp();
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
          if (j == 3 || last_kb) {
            if (++slot == kSfSlots) { slot = 0; sphase ^= 1u; }
          }
        }
        acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------------------------ scale-factor stager (each CTA)
    int slot = 0;
    uint32_t sphase = 0;
    bool ok = true;
    for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      mx_tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
      const int row0 = m_blk * kTileM + static_cast<int>(rank) * BM;
      for (int kb0 = 0; kb0 < nkb; kb0 += 4) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = row0 + lane + 32 * j;
          w[j] = (row < p.M) ? __ldg(p.sa + static_cast<int64_t>(kb0 >> 2) * p.sa_stride_pack + row * p.sa_stride_m) : 0u;
        }
        uint32_t wb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int col = min(n_blk * kTileN + (i >> 2) * 128 + (i & 3) * 32 + lane, p.N - 1);
          const float* sp = p.sb + static_cast<int64_t>(col >> 7) * p.sb_stride_n;
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int kb = min(kb0 + k, nkb - 1);
            word |= ((__float_as_uint(__ldg(sp + static_cast<int64_t>(kb) * p.sb_stride_g)) >> 23) & 0xffu) << (8 * k);
          }
          wb[i] = word;
        }
        ok = mbar_wait_warp(&sf_empty[slot], sphase ^ 1u, p.status, 55);
        if (!ok) break;
        uint8_t* sf = smem_sf + slot * kPairSfBytes;
        *reinterpret_cast<uint4*>(sf + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(sf + kSfaBytes + lane * 16) = make_uint4(wb[0], wb[1], wb[2], wb[3]);
        *reinterpret_cast<uint4*>(sf + kSfaBytes + 512 + lane * 16) = make_uint4(wb[4], wb[5], wb[6], wb[7]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_leader_release(&sf_full[slot]);
        if (++slot == kSfSlots) { slot = 0; sphase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp < 4 || warp >= 8) {
    // ------------------------------------------------------------------ epilogue (each CTA, its own 128 rows; warps
    // 0-3 take columns [0, 128) of their row quadrant, warps 8-11 columns [128, 256))
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (p.ldo % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int half = warp >> 3;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
      int m_blk, n_blk;
      mx_tile_coords(tile, m_blocks, n_blocks, m_blk, n_blk);
      ok = mbar_wait(acc_full, acc_phase, p.status, 56);
      if (!ok) break;
      tc_fence_after();
      const int m = m_blk * kTileM + static_cast<int>(rank) * BM + (warp & 3) * 32 + lane;
      const uint32_t taddr = tmem_base + lane_addr + half * 128;
      const int n_half = n_blk * kTileN + half * 128;
      if constexpr (sizeof(OutT) == 2) {
        // 16-bit output: read, round and pack the warp's 128 columns (64 registers), hand the accumulator back, then
        // store -- the stores run under the next tile's MMAs
        uint32_t pk[64];
#pragma unroll
        for (int ch = 0; ch < 8; ch += 2) {
          float v[32];
          tmem_ld16(taddr + ch * 16, *reinterpret_cast<float(*)[16]>(v));
          tmem_ld16(taddr + (ch + 1) * 16, *reinterpret_cast<float(*)[16]>(v + 16));
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; c += 2) pk[ch * 8 + c / 2] = pack2(out, v[c], v[c + 1]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
        if (m < p.M && n_half < p.N) {
          OutT* dst = out + static_cast<int64_t>(m) * p.ldo + n_half;
          const int valid = min(p.N - n_half, 128);
          if (vec_ok && valid == 128) {
#pragma unroll
            for (int c = 0; c < 16; ++c)
              reinterpret_cast<uint4*>(dst)[c] = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              OutT lo, hi;
              *reinterpret_cast<uint16_t*>(&lo) = static_cast<uint16_t>(pk[c] & 0xffffu);
              *reinterpret_cast<uint16_t*>(&hi) = static_cast<uint16_t>(pk[c] >> 16);
              if (2 * c < valid) dst[2 * c] = lo;
              if (2 * c + 1 < valid) dst[2 * c + 1] = hi;
            }
          }
        }
      } else {
#pragma unroll 1
        for (int ch = 0; ch < 8; ch += 2) {
          float v[32];
          tmem_ld16(taddr + ch * 16, *reinterpret_cast<float(*)[16]>(v));
          tmem_ld16(taddr + (ch + 1) * 16, *reinterpret_cast<float(*)[16]>(v + 16));
          tmem_ld_wait();
          if (ch + 2 >= 8) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);
          }
          const int n0 = n_half + ch * 16;
          if (m < p.M && n0 < p.N) store_row<32>(out + static_cast<int64_t>(m) * p.ldo + n0, v, min(p.N - n0, 32), vec_ok);
        }
      }
      acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  cluster_sync_all();
  if (*reinterpret_cast<volatile int*>(p.status) != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

template <typename OutT>
int launch_mx_pair(const CUtensorMap& ma, const CUtensorMap& mb, const MxParams& p, cudaStream_t stream) {
  auto kern = gemm_mx_pair_kernel<OutT>;
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
  cfg.blockDim = dim3(kThreadsMxSilu);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs[dev] == 0) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem));
    cfg.gridDim = dim3(2 * 74);
    int n = 0;
    B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, kern, &cfg));
    if (n <= 0) return B200_ERR_UNSUPPORTED;
    max_pairs[dev] = n;
  }
  const long long tiles = static_cast<long long>((p.M + 255) / 256) * ((p.N + 255) / 256);
  int pairs = sm_count() / 2;
  if (pairs > max_pairs[dev]) pairs = max_pairs[dev];
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  cfg.gridDim = dim3(2 * pairs);
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, ma, mb, p));
  return B200_OK;
}

int launch_mx_pair_dtype(const void* a, int64_t lda, const void* b, int64_t ldb, const MxParams& p, cudaStream_t st) {
  CUtensorMap ma, mb;
  int rc = make_map_u8_2d(&ma, a, p.M, p.K, lda, BM);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, p.N, p.K, ldb, 128);
  if (rc != B200_OK) return rc;
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch_mx_pair<__nv_bfloat16>(ma, mb, p, st);
    case B200_DT_F16: return launch_mx_pair<__half>(ma, mb, p, st);
    default: return launch_mx_pair<float>(ma, mb, p, st);
  }
}

}  // namespace

extern int g_force_block_n;

}  // namespace b200

extern "C" int b200_fp8_blockwise_scaled_mm_pow2(const void* a, int64_t lda, const void* b, int64_t ldb,
                                                 const uint32_t* sa_packed, int64_t sa_stride_m, int64_t sa_stride_pack,
                                                 const float* sb_pow2, int64_t sb_stride_n, int64_t sb_stride_g, void* out,
                                                 int64_t ldo, int out_dtype, int64_t M, int64_t N, int64_t K,
                                                 void* stream) {
  using namespace b200;
  if (M < 0 || N < 0 || K <= 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || N == 0) return B200_OK;
  if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa_packed || !sb_pow2 || !out) return B200_ERR_NULL_PTR;
  if (out_dtype != B200_DT_BF16 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_F32) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldo < N) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || !aligned16(a) || !aligned16(b)) return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_pack < 0 || sb_stride_n < 0 || sb_stride_g < 0) return B200_ERR_BAD_STRIDE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;   // every k-block carries exactly one exponent per row / column block
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  if (gemm_sticky_status() != 0) return B200_ERR_DEVICE_TIMEOUT;
  MxParams p;
  p.sa = sa_packed; p.sb = sb_pow2; p.out = out;
  p.sa_stride_m = sa_stride_m; p.sa_stride_pack = sa_stride_pack;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g; p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = out_dtype;
  p.offsets = nullptr; p.rows = nullptr; p.experts = nullptr;
  p.rows_stride = 0; p.sb_stride_e = 0; p.sa_stride_problem = -1; p.num_problems = 0; p.num_weight_experts = 1;
  p.out_s = nullptr; p.out_s_stride_pack = 0;
  p.status = gemm_status_ptr();
  if (!p.status) return B200_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Tile choice.  Measured (us; 1024 / 4096 / 16384 x 36864 x 7168, then 1024 / 4096 / 16384 x 7168 x 18432):
  //   128 x 256, one CTA        245 / 857 / 3358    179 / 496 / 1770
  //   256 x 240, one CTA        261 / 883 / 3881    142 / 482 / 1649
  //   256 x 256 on a CTA pair   228 / 858 / 3587    151 / 511 / 2053
  // (128 x 240 with two accumulators: 940 on the second shape, never ahead.)  Long K favours the two-half tile
  // (fewer, longer tiles amortise its unoverlapped read-out), wide N with K up to 8192 the CTA pair (half the
  // operand bytes per SM).  With every SM issuing MMAs back to back and nothing else the chip settles at 1.5 GHz
  // under its power cap (3.7 PFLOP/s); these kernels reach 2.5-2.7 and slow down the longer they run.
  // The test hook selects a form directly: 256 / 240 / 2240 / 2256.
  if (g_force_block_n == 2256) return launch_mx_pair_dtype(a, lda, b, ldb, p, st);
  if (g_force_block_n == 256) return launch_mx_dtype<256, 1>(a, lda, b, ldb, p, st);
  if (g_force_block_n == 240) return launch_mx_dtype<240, 1>(a, lda, b, ldb, p, st);
  if (g_force_block_n == 2240) return launch_mx_dtype<240, 2>(a, lda, b, ldb, p, st);
  if (M >= 1024 && K >= 12288) return launch_mx_dtype<240, 2>(a, lda, b, ldb, p, st);
  if (M >= 512 && M < 4096 && N >= 4096) {
    // a cluster launch can be refused where a plain one is not (no pair of SMs free, a tool that does not support
    // clusters): then the one-CTA form runs instead
    if (launch_mx_pair_dtype(a, lda, b, ldb, p, st) == B200_OK) return B200_OK;
    (void)cudaGetLastError();
  }
  return launch_mx_dtype<256, 1>(a, lda, b, ldb, p, st);
}


// Grouped form (MoE experts; DeepGEMM's contiguous and masked layouts are special cases of the problem table, see
// the header).  Weights are one [num_weight_experts * N, K] matrix, weight scales [expert][N/128][K/128] fp32 powers
// of two with strides (sb_stride_e, sb_stride_n, sb_stride_g); the packed activation exponents are indexed by the
// GLOBAL row of `a` like the codes (sa_stride_problem < 0), or by the row inside the problem with each problem's
// words starting at sa_packed + i * sa_stride_problem.  Everything the tile schedule needs is read on the device.
extern "C" int b200_fp8_blockwise_scaled_grouped_mm_pow2(
    const void* a, int64_t lda, int64_t total_rows, const void* b, int64_t ldb, const uint32_t* sa_packed,
    int64_t sa_stride_m, int64_t sa_stride_pack, int64_t sa_stride_problem, const float* sb_pow2, int64_t sb_stride_e, int64_t sb_stride_n,
    int64_t sb_stride_g, void* out, int64_t ldo, int out_dtype, const int32_t* problem_offsets,
    const int32_t* problem_rows, int64_t problem_rows_stride, const int32_t* problem_experts, int num_problems,
    int num_weight_experts, int64_t N, int64_t K, void* stream) {
  using namespace b200;
  if (total_rows < 0 || N < 0 || K <= 0 || num_problems < 0 || num_weight_experts <= 0) return B200_ERR_BAD_SHAPE;
  if (total_rows == 0 || N == 0 || num_problems == 0) return B200_OK;
  if (num_problems > kMaxProblems) return B200_ERR_TOO_LARGE;
  if (total_rows > 0x7fffff00LL || K > 0x7fffff00LL || N * num_weight_experts > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa_packed || !sb_pow2 || !out || !problem_offsets || !problem_rows) return B200_ERR_NULL_PTR;
  if (out_dtype != B200_DT_BF16 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_F32) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldo < N) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || !aligned16(a) || !aligned16(b)) return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_pack < 0 || sb_stride_e < 0 || sb_stride_n < 0 || sb_stride_g < 0 ||
      problem_rows_stride < 0)
    return B200_ERR_BAD_STRIDE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (N % 128 != 0) return B200_ERR_UNSUPPORTED;   // a column block of scales must not straddle two experts
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  if (gemm_sticky_status() != 0) return B200_ERR_DEVICE_TIMEOUT;
  MxParams p;
  p.sa = sa_packed; p.sb = sb_pow2; p.out = out;
  p.sa_stride_m = sa_stride_m; p.sa_stride_pack = sa_stride_pack;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g; p.ldo = ldo;
  p.M = static_cast<int>(total_rows); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = out_dtype;
  p.offsets = problem_offsets; p.rows = problem_rows; p.experts = problem_experts;
  p.rows_stride = problem_rows_stride; p.sb_stride_e = sb_stride_e; p.sa_stride_problem = sa_stride_problem;
  p.num_problems = num_problems; p.num_weight_experts = num_weight_experts;
  p.out_s = nullptr; p.out_s_stride_pack = 0;
  p.status = gemm_status_ptr();
  if (!p.status) return B200_ERR_CUDA;
  // Tile width.  128 x 256 with one accumulator is the default; the test hook reaches the narrower tiles with two
  // accumulators (a tile's read-out overlaps the next tile's MMAs): 9240 -> 128 x 240, 9192 -> 128 x 192.
  if (g_force_block_n == 9240) return launch_mx_dtype<240, 1, true>(a, lda, b, ldb, p, static_cast<cudaStream_t>(stream));
  if (g_force_block_n == 9192) return launch_mx_dtype<192, 1, true>(a, lda, b, ldb, p, static_cast<cudaStream_t>(stream));
  if (g_force_block_n == 9480) return launch_mx_dtype<240, 2, true>(a, lda, b, ldb, p, static_cast<cudaStream_t>(stream));
  return launch_mx_dtype<256, 1, true>(a, lda, b, ldb, p, static_cast<cudaStream_t>(stream));
}

// Expert GEMM 1 with the activation and the next GEMM's quantisation in its epilogue: for every problem,
//   q, s = quantise_pow2( SiLU(x W_gate^T) * (x W_up^T) )       (128-wide groups, packed exponent words)
// where W = b holds, per weight slice, 2 * N rows (gate rows first) and N is the intermediate size.  The accumulator
// is rounded to `mid_dtype` (bf16 / fp16) before the activation and the product after it, exactly as the unfused
// sequence stores them, so codes and exponents equal b200_fp8_blockwise_scaled_grouped_mm_pow2 followed by
// b200_silu_mul_per_token_group_quant_fp8_ue8m0 bit for bit -- without the [rows, 2N] intermediate ever reaching HBM.
// out_q [total_rows, N] e4m3 (leading dimension ldq bytes); out_s packed words, word (row, w) at
// out_s[w * out_s_stride_pack + row], bytes of groups past N / 128 untouched (pass a zeroed tensor).
// Replaces: the SiLU*mul + quant pass between the two expert GEMMs (python/sglang/srt/layers/moe/cutlass_moe.py:191-194;
// ep_moe/layer.py:606-628) together with the GEMM before it.
extern "C" int b200_fp8_blockwise_scaled_grouped_mm_pow2_silu_quant(
    const void* a, int64_t lda, int64_t total_rows, const void* b, int64_t ldb, const uint32_t* sa_packed,
    int64_t sa_stride_m, int64_t sa_stride_pack, int64_t sa_stride_problem, const float* sb_pow2, int64_t sb_stride_e,
    int64_t sb_stride_n, int64_t sb_stride_g, void* out_q, int64_t ldq, uint32_t* out_s, int64_t out_s_stride_pack,
    int mid_dtype, const int32_t* problem_offsets, const int32_t* problem_rows, int64_t problem_rows_stride,
    const int32_t* problem_experts, int num_problems, int num_weight_experts, int64_t N, int64_t K, void* stream) {
  using namespace b200;
  if (total_rows < 0 || N < 0 || K <= 0 || num_problems < 0 || num_weight_experts <= 0) return B200_ERR_BAD_SHAPE;
  if (total_rows == 0 || N == 0 || num_problems == 0) return B200_OK;
  if (num_problems > kMaxProblems) return B200_ERR_TOO_LARGE;
  if (total_rows > 0x7fffff00LL || K > 0x7fffff00LL || 2 * N * num_weight_experts > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa_packed || !sb_pow2 || !out_q || !out_s || !problem_offsets || !problem_rows) return B200_ERR_NULL_PTR;
  if (mid_dtype != B200_DT_BF16 && mid_dtype != B200_DT_F16) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldq < N || out_s_stride_pack < total_rows) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || (ldq % 16) != 0 || !aligned16(a) || !aligned16(b) || !aligned16(out_q))
    return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_pack < 0 || sb_stride_e < 0 || sb_stride_n < 0 || sb_stride_g < 0 ||
      problem_rows_stride < 0)
    return B200_ERR_BAD_STRIDE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (N % 128 != 0) return B200_ERR_UNSUPPORTED;
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  if (gemm_sticky_status() != 0) return B200_ERR_DEVICE_TIMEOUT;
  MxParams p;
  p.sa = sa_packed; p.sb = sb_pow2; p.out = out_q;
  p.sa_stride_m = sa_stride_m; p.sa_stride_pack = sa_stride_pack;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g; p.ldo = ldq;
  p.M = static_cast<int>(total_rows); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = mid_dtype;
  p.offsets = problem_offsets; p.rows = problem_rows; p.experts = problem_experts;
  p.rows_stride = problem_rows_stride; p.sb_stride_e = sb_stride_e; p.sa_stride_problem = sa_stride_problem;
  p.num_problems = num_problems; p.num_weight_experts = num_weight_experts;
  p.out_s = out_s; p.out_s_stride_pack = out_s_stride_pack;
  p.status = gemm_status_ptr();
  if (!p.status) return B200_ERR_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return mid_dtype == B200_DT_BF16 ? launch_mx_silu<__nv_bfloat16>(a, lda, b, ldb, p, st)
                                    : launch_mx_silu<__half>(a, lda, b, ldb, p, st);
}
