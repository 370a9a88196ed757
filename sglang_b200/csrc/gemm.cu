// Dense block-scaled FP8 GEMM for sm_100a:  out = cast( sum_kb (A_kb * B_kb^T) * sa[:,kb] * sb[nb,kb] ).
//
// Stands in for the reference's fp8_blockwise_scaled_mm
// (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:165-423) and the Triton kernel
// _w8a8_block_fp8_matmul (python/sglang/srt/layers/quantization/fp8_kernel.py:493-575).
//
// One persistent CTA per SM, warp-specialised:
//   TMA warp    producer: per 128-wide k-block one A box (128 rows x 128 B) and one B box
//               (BLOCK_N rows x 128 B) into a ring of shared-memory stages (128-byte swizzle).
//   MMA warp    issuer: 4 x tcgen05.mma kind::f8f6f4 (M128 x N BLOCK_N x K32) per k-block into
//               a tensor-memory accumulator that is started fresh for every k-block (the fp32
//               scales differ per k-block, so partial sums cannot be chained inside the tensor
//               core); accumulators rotate through 512/BLOCK_N tensor-memory buffers.  One
//               tcgen05.commit per k-block signals both "stage reusable" and "partial sums ready".
//   warps 0..E-1 promotion + epilogue: each warp owns 32 rows (its tensor-memory lane quadrant)
//               x CPW columns; per k-block it reads the partial sums with tcgen05.ld in chunks,
//               releases the buffer after the last chunk has landed, and does
//               acc += partial * (sa[m,kb] * sb[nb,kb]) with packed fp32 FMAs; after the last
//               k-block it converts and stores its output row segment.
// The TMA and MMA warps walk their loops with all 32 lanes (warp-uniform addresses and
// descriptors) and one elected lane issues.  All mbarrier waits are bounded; a wait that gives up
// records a code in a device status word and every role drains to a common exit where tensor
// memory is released.
#include "gemm_common.cuh"

namespace b200 {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 32;     // m-blocks per rasterisation group: the group's A rows (<= 4096 x K bytes) stay in L2
                                // while every weight slice is streamed once per group
constexpr int kScaleGroup = 4;   // k-blocks per scale-ring slot
constexpr int kScaleSlots = 4;   // slots in the ring (the stager runs up to 16 k-blocks ahead)

template <int BLOCK_N, int EPI_WARPS, int ISSUERS = 1>
struct Cfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kABytes = BLOCK_M * BLOCK_K;
  static constexpr int kBBytes = BLOCK_N * BLOCK_K;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNumAcc = kTmemCols / BLOCK_N;
  static constexpr int kColsPerWarp = BLOCK_N / (EPI_WARPS / 4);
  // Warp roles: epilogue warps first (whole warpgroups, so their register budget can be raised with
  // setmaxnreg), then one warpgroup of helpers.
  static constexpr int kTmaWarp = EPI_WARPS;
  static constexpr int kMmaWarp = EPI_WARPS + 1;
  static constexpr int kStagerWarp = EPI_WARPS + 2;             // stages the scale products in shared memory
  static constexpr int kMmaWarp2 = EPI_WARPS + 3;               // second MMA issuer (kIssuers == 2)
  // Two MMA-issuing warps take alternate k-blocks: one warp's barrier waits and loop bookkeeping then overlap
  // the other's issue instead of leaving the tensor pipe idle between k-blocks.
  static constexpr int kIssuers = ISSUERS;
  static constexpr int kThreads = 32 * (4 + EPI_WARPS);
  // With 16 epilogue warps the launch gives every thread 96 registers (20 warps); the helper
  // warpgroup hands 32 per thread back and the epilogue warps take 8 more each, enough to hold 64
  // accumulators plus a 32-column chunk.  setmaxnreg.inc WAITS until the CTA's pool holds the
  // registers it asks for, so the request must never exceed what the helpers release.
  static constexpr bool kRebalanceRegs = EPI_WARPS == 16;
  static constexpr int kLaunchRegs = 96;
  static constexpr int kEpiRegs = 104;
  static constexpr int kHelperRegs = 64;
  static_assert(EPI_WARPS * (kEpiRegs - kLaunchRegs) <= 4 * (kLaunchRegs - kHelperRegs),
                "epilogue warps would wait forever for registers nobody releases");
  static constexpr int kHalves = BLOCK_N / 128;                 // weight-scale blocks per tile row
  static constexpr int kSlotFloats = kScaleGroup * kHalves * BLOCK_M;
  static constexpr int kScaleBytes = kScaleSlots * kSlotFloats * 4;
  static constexpr int kMaxExperts = 1024;  // grouped form: m-tile prefix table in shared memory
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + 1024 /*alignment slack*/ +
                                    256 /*barriers*/ + (kMaxExperts + 1) * 4;
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

// Where a tile lives.  Dense: tiles of the [M, N] output, rasterised in groups of kGroupM m-blocks.
// Grouped: the m-tiles of all experts laid end to end (tile_m_start[e] = first m-tile of expert e,
// in shared memory), n-blocks fastest so that neighbouring CTAs stream different slices of the same
// expert's weights while sharing its few activation rows through L2.
struct TileInfo {
  int row0;        // first row of A / out
  int valid_rows;  // rows of this tile that belong to the problem (<= BLOCK_M)
  int n_blk;       // column block
  int b_row0;      // first row of the [E*N, K] weight matrix
  int expert;
};

template <bool GROUPED, int BLOCK_N>
__device__ __forceinline__ TileInfo get_tile(int tile, const GemmParams& p, int m_blocks, int n_blocks,
                                             const int* tile_m_start) {
  TileInfo t;
  if constexpr (!GROUPED) {
    int m_blk;
    tile_coords(tile, m_blocks, n_blocks, m_blk, t.n_blk);
    t.row0 = m_blk * BLOCK_M;
    t.valid_rows = min(BLOCK_M, p.M - t.row0);
    t.b_row0 = t.n_blk * BLOCK_N;
    t.expert = 0;
  } else {
    const int mt = tile / n_blocks;
    t.n_blk = tile - mt * n_blocks;
    int lo = 0, hi = p.num_experts;   // last e with tile_m_start[e] <= mt
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (tile_m_start[mid] <= mt) lo = mid; else hi = mid;
    }
    t.expert = lo;
    const int m_blk = mt - tile_m_start[lo];
    const int m_e = p.problem_sizes[lo * 3];
    // Tables that do not describe the buffers (left over from another batch, never filled) must not send a
    // store outside `out`: the tile is clamped into [0, total rows).
    t.row0 = min(max(p.expert_offsets[lo] + m_blk * BLOCK_M, 0), p.M - 1);
    t.valid_rows = max(0, min(min(BLOCK_M, m_e - m_blk * BLOCK_M), p.M - t.row0));
    t.b_row0 = lo * p.N + t.n_blk * BLOCK_N;
  }
  return t;
}

// One unit of a CTA's work list: a whole tile, or one split of a tile's k-blocks.
struct Work {
  int tile, split, kb_begin, kb_end;
  bool partial;   // the result is a partial sum for the workspace, not an output tile
};
__device__ __forceinline__ Work decode_work(int vt, const GemmParams& p, int nkb, bool grouped) {
  if (grouped || p.split_k == 1) return Work{vt, 0, 0, nkb, false};
  if (vt < p.tail_first) return Work{vt, 0, 0, nkb, false};
  const int r = vt - p.tail_first;
  const int tile = p.tail_first + r / p.split_k, split = r % p.split_k;
  const int kb0 = split * p.kb_per_split;
  return Work{tile, split, kb0, min(nkb, kb0 + p.kb_per_split), true};
}

// ld of 16 columns has landed: the wait carries the destination registers as operands so that no use of
// them can be scheduled before it (the load itself only names them as outputs at issue time).
__device__ __forceinline__ void tmem_ld_wait16(float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// acc[0..15] += v[0..15] * s, two fp32 FMAs per instruction (fma.rn.f32x2)
__device__ __forceinline__ void fma16(float* acc, const float (&v)[16], float2 s2) {
#pragma unroll
  for (int c = 0; c < 16; c += 2) {
    const float2 r = __ffma2_rn(make_float2(v[c], v[c + 1]), s2, make_float2(acc[c], acc[c + 1]));
    acc[c] = r.x;
    acc[c + 1] = r.y;
  }
}

template <int BLOCK_N, int EPI_WARPS, int CHUNK, bool GROUPED, typename OutT, int ISSUERS = 1>
__global__ void __launch_bounds__(Cfg<BLOCK_N, EPI_WARPS, ISSUERS>::kThreads, 1)
gemm_block_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const GemmParams p) {
  using C = Cfg<BLOCK_N, EPI_WARPS, ISSUERS>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128-byte swizzle pattern is a function of address bits [4,10).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + C::kStages * C::kABytes;
  float* smem_scale = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes + C::kScaleBytes);
  uint64_t* full_bar = bars;                    // operands of the stage have landed
  uint64_t* done_bar = bars + C::kStages;       // the k-block's MMAs completed
  uint64_t* acc_empty = bars + 2 * C::kStages;  // accumulator buffer has been read out
  uint64_t* scale_full = acc_empty + C::kNumAcc;     // scale-ring slot written
  uint64_t* scale_empty = scale_full + kScaleSlots;  // scale-ring slot consumed by every epilogue warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(scale_empty + kScaleSlots);

  int* tile_m_start = reinterpret_cast<int*>(tmem_slot + 2);   // [num_experts + 1], grouped form only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int nkb = (p.K + BLOCK_K - 1) / BLOCK_K;

  if constexpr (GROUPED) {
    for (int e = threadIdx.x; e < p.num_experts; e += blockDim.x)
      tile_m_start[e + 1] = (max(p.problem_sizes[e * 3], 0) + BLOCK_M - 1) / BLOCK_M;
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      tile_m_start[0] = 0;
      for (int e = 1; e <= p.num_experts; ++e) {
        run += tile_m_start[e];
        tile_m_start[e] = run;
      }
    }
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&done_bar[i], 1);
    }
    for (int i = 0; i < C::kNumAcc; ++i) mbar_init(&acc_empty[i], EPI_WARPS);
    for (int i = 0; i < kScaleSlots; ++i) {
      mbar_init(&scale_full[i], 1);
      mbar_init(&scale_empty[i], EPI_WARPS);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kTmaWarp && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const int num_tiles = GROUPED ? tile_m_start[p.num_experts] * n_blocks : m_blocks * n_blocks;
  // split-K: every tile from tail_first on becomes split_k work units (split fastest), each covering
  // kb_per_split k-blocks; tail_first = 0 splits all tiles (decode-size M), otherwise only the last wave
  const int split_k = GROUPED ? 1 : p.split_k;
  const int tail_first = (GROUPED || split_k == 1) ? num_tiles : p.tail_first;
  const int num_vtiles = tail_first + (num_tiles - tail_first) * split_k;

  if (warp >= EPI_WARPS) {
  // ====================================================================== helper warpgroup
  if constexpr (C::kRebalanceRegs) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::kHelperRegs));
  if (warp == C::kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const Work w = decode_work(vt, p, nkb, GROUPED);
      const TileInfo t = get_tile<GROUPED, BLOCK_N>(w.tile, p, m_blocks, n_blocks, tile_m_start);
      const int kb_begin = w.kb_begin, kb_end = w.kb_end;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        ok = mbar_wait_warp(&done_bar[stage], phase ^ 1u, p.status, 1);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&full_bar[stage], C::kStageBytes);
          tma_load_2d(smem_a + stage * C::kABytes, &map_a, &full_bar[stage], kb * BLOCK_K, t.row0);
          tma_load_2d(smem_b + stage * C::kBBytes, &map_b, &full_bar[stage], kb * BLOCK_K, t.b_row0);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == C::kMmaWarp || (C::kIssuers == 2 && warp == C::kMmaWarp2)) {
    // ------------------------------------------------------------------ MMA issuer(s)
    // The whole warp walks the loop so that addresses and descriptors stay warp-uniform; one
    // elected lane issues.  With two issuers each warp takes every other k-block of the CTA's sequence
    // (own stage, own accumulator buffer: k-blocks are independent) and only tracks the ring positions
    // of the ones it skips.
    constexpr uint32_t idesc = umma_idesc_e4m3(BLOCK_M, BLOCK_N);
    const uint64_t a_desc0 = umma_desc_k128(smem_u32(smem_a));
    const uint64_t b_desc0 = umma_desc_k128(smem_u32(smem_b));
    const int issuer = (warp == C::kMmaWarp) ? 0 : 1;
    int stage = 0, acc = 0, turn = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const Work w = decode_work(vt, p, nkb, GROUPED);
      const int kb_begin = w.kb_begin, kb_end = w.kb_end;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (C::kIssuers == 2 && turn != issuer) {
          turn ^= 1;
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
          if (++acc == C::kNumAcc) { acc = 0; acc_phase ^= 1u; }
          continue;
        }
        turn ^= 1;
        ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1u, p.status, 2);
        if (ok) ok = mbar_wait(&full_bar[stage], phase, p.status, 3);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint64_t a_desc = a_desc0 + static_cast<uint64_t>(stage * (C::kABytes >> 4));
        const uint64_t b_desc = b_desc0 + static_cast<uint64_t>(stage * (C::kBBytes >> 4));
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BLOCK_N);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BLOCK_K / 32; ++k) {
            // advance 32 bytes along K inside the 128-byte swizzle row: +2 in the (addr >> 4) field
            umma_f8(d_tmem, a_desc + static_cast<uint64_t>(2 * k), b_desc + static_cast<uint64_t>(2 * k), idesc,
                    k > 0 ? 1u : 0u);
          }
          umma_commit(&done_bar[stage]);  // stage reusable and partial sums readable once these MMAs finish
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        if (++acc == C::kNumAcc) { acc = 0; acc_phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == C::kStagerWarp) {
    // ------------------------------------------------------------------ scale stager
    // Global loads of the scales take far longer than a k-block under TMA load (they were the
    // dominant stall when the epilogue warps fetched them a few k-blocks ahead), so one warp
    // runs up to kScaleSlots*kScaleGroup k-blocks ahead and leaves the products
    // sa[m,kb] * sb[nb,kb] in a shared-memory ring: slot layout [kScaleGroup][halves][128 rows].
    int slot = 0;
    uint32_t sphase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const Work w = decode_work(vt, p, nkb, GROUPED);
      const TileInfo t = get_tile<GROUPED, BLOCK_N>(w.tile, p, m_blocks, n_blocks, tile_m_start);
      const float* sb_base = p.sb + static_cast<int64_t>(t.expert) * p.sb_stride_e;
      const int kb_begin = w.kb_begin, kb_end = w.kb_end;
      for (int kb0 = kb_begin; kb0 < kb_end; kb0 += kScaleGroup) {
        float* dst = smem_scale + slot * C::kSlotFloats;
        float a[kScaleGroup][4];
        float bsc[kScaleGroup][C::kHalves];
        // Row-major activation scales (the grouped form): the four k-blocks of a row are 16 contiguous bytes, one
        // load per row instead of four loads that each touch 32 different sectors.
        static_assert(kScaleGroup == 4, "one float4 per row and slot");
        const bool row_vec = !p.sa_ue8m0 && p.sa_stride_g == 1 && (p.sa_stride_m & 3) == 0 && (kb_begin & 3) == 0 &&
                             (reinterpret_cast<uintptr_t>(p.sa) & 15u) == 0 && kb0 + kScaleGroup <= ((nkb + 3) & ~3) &&
                             (p.sa_stride_m >= ((nkb + 3) & ~3));
        if (row_vec) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const int rr = r * 32 + lane;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rr < t.valid_rows)
              v = __ldg(reinterpret_cast<const float4*>(p.sa + static_cast<int64_t>(t.row0 + rr) * p.sa_stride_m + kb0));
            a[0][r] = v.x; a[1][r] = v.y; a[2][r] = v.z; a[3][r] = v.w;
          }
        }
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j) {
          const int kb = kb0 + j;
          const bool kin = kb < kb_end;
          if (row_vec) {
            // loaded above
          } else if (p.sa_ue8m0) {   // warp-uniform; each branch is a batch of independent loads
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int rr = r * 32 + lane;
              a[j][r] = (kin && rr < t.valid_rows) ? load_sa<true>(p, t.row0 + rr, kb) : 0.f;
            }
          } else {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int rr = r * 32 + lane;
              a[j][r] = (kin && rr < t.valid_rows) ? load_sa<false>(p, t.row0 + rr, kb) : 0.f;
            }
          }
#pragma unroll
          for (int h = 0; h < C::kHalves; ++h) {
            const int nb = min(t.n_blk * BLOCK_N + h * 128, p.N - 1) / 128;
            bsc[j][h] = kin ? __ldg(sb_base + static_cast<int64_t>(nb) * p.sb_stride_n +
                                    static_cast<int64_t>(kb) * p.sb_stride_g)
                            : 0.f;
          }
        }
        // the loads above do not depend on the slot: issued first, they are in flight during this wait
        ok = mbar_wait_warp(&scale_empty[slot], sphase ^ 1u, p.status, 5);
        if (!ok) break;
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j)
#pragma unroll
          for (int h = 0; h < C::kHalves; ++h)
#pragma unroll
            for (int r = 0; r < 4; ++r) dst[(j * C::kHalves + h) * BLOCK_M + r * 32 + lane] = a[j][r] * bsc[j][h];
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(&scale_full[slot]);
        if (++slot == kScaleSlots) { slot = 0; sphase ^= 1u; }
      }
    }
    __syncwarp();
  }
  } else {
    // ====================================================================== promotion + epilogue warps
    if constexpr (C::kRebalanceRegs) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::kEpiRegs));
    constexpr int CPW = C::kColsPerWarp;
    constexpr bool kPipe = (CHUNK == 16);
    static_assert(!kPipe || CPW == 64, "the pipelined read-out is written for 64 columns per warp");
    static_assert(CPW % CHUNK == 0 && (CHUNK == 16 || CHUNK == 32 || CHUNK == 64), "chunking");
    static_assert(CPW <= 128, "a warp's columns lie in one weight-scale block");
    const int quad = warp & 3;         // tensor-memory lane quadrant this warp may read
    const int part = warp >> 2;        // which CPW-wide column slice
    const int half = (part * CPW) / 128;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    OutT* out = static_cast<OutT*>(p.out);
    const bool vec_ok = (p.ldo % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
    int acc_i = 0, stage = 0, slot = 0;
    uint32_t phase = 0, sphase = 0;
    bool ok = true;
    for (int vt = blockIdx.x; ok && vt < num_vtiles; vt += gridDim.x) {
      const Work w = decode_work(vt, p, nkb, GROUPED);
      const TileInfo t = get_tile<GROUPED, BLOCK_N>(w.tile, p, m_blocks, n_blocks, tile_m_start);
      const int kb_begin = w.kb_begin, kb_end = w.kb_end;
      const int row_in_tile = quad * 32 + lane;
      const int m = t.row0 + row_in_tile;
      const int n0 = t.n_blk * BLOCK_N + part * CPW;
      float acc[CPW];
#pragma unroll
      for (int c = 0; c < CPW; ++c) acc[c] = 0.f;
      // software-pipelined read-out (kPipe): the last chunk of a k-block is accumulated under the first
      // tensor-memory load of the next one
      [[maybe_unused]] float va[16], vb[16];
      [[maybe_unused]] bool pending = false;
      [[maybe_unused]] float2 s2_pending = make_float2(0.f, 0.f);
      for (int kb0 = kb_begin; ok && kb0 < kb_end; kb0 += kScaleGroup) {
        // the four scale products of this group, then the slot goes straight back to the stager
        ok = mbar_wait(&scale_full[slot], sphase, p.status, 6);
        if (!ok) break;
        float sc[kScaleGroup];
        const float* src = smem_scale + slot * C::kSlotFloats + half * BLOCK_M + quad * 32 + lane;
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j) sc[j] = src[j * C::kHalves * BLOCK_M];
        __syncwarp();
        if (lane == 0) mbar_arrive(&scale_empty[slot]);
        if (++slot == kScaleSlots) { slot = 0; sphase ^= 1u; }
#pragma unroll
        for (int j = 0; j < kScaleGroup; ++j) {
          const int kb = kb0 + j;
          if (kb < kb_end) {
            const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(acc_i * BLOCK_N + part * CPW);
            const float2 s2 = make_float2(sc[j], sc[j]);
            if constexpr (kPipe) {
              // Four 16-column chunks per k-block through two register buffers: while the FMAs of one chunk
              // run, the tensor-memory load of the next is in flight, so neither the load latency nor the
              // FMA pipe (shared by the scheduler's four read-out warps) is waited for on its own.  The
              // buffer goes back to the MMA warps as soon as the last load has landed; that chunk's FMAs
              // are deferred until the next k-block's first load has been issued (or done at once if the
              // next k-block has not completed yet).
              if (!mbar_try_wait(&done_bar[stage], phase)) {
                if (pending) { fma16(acc + 48, vb, s2_pending); pending = false; }
                ok = mbar_wait(&done_bar[stage], phase, p.status, 4);
                if (!ok) break;
              }
              tc_fence_after();
              tmem_ld16(taddr, va);
              if (pending) { fma16(acc + 48, vb, s2_pending); pending = false; }
              tmem_ld_wait16(va);
              tmem_ld16(taddr + 16, vb);
              fma16(acc, va, s2);
              tmem_ld_wait16(vb);
              tmem_ld16(taddr + 32, va);
              fma16(acc + 16, vb, s2);
              tmem_ld_wait16(va);
              tmem_ld16(taddr + 48, vb);
              fma16(acc + 32, va, s2);
              tmem_ld_wait16(vb);
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[acc_i]);
              pending = true;
              s2_pending = s2;
            } else {
            ok = mbar_wait(&done_bar[stage], phase, p.status, 4);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int ch = 0; ch < CPW / CHUNK; ++ch) {
              float v[CHUNK];
              if constexpr (CHUNK == 16) {
                tmem_ld16(taddr + ch * CHUNK, v);
              } else {
#pragma unroll
                for (int q = 0; q < CHUNK / 32; ++q) tmem_ld32(taddr + ch * CHUNK + q * 32, v + q * 32);
              }
              tmem_ld_wait();
              if (ch == CPW / CHUNK - 1) {
                // all of this warp's reads of the buffer are complete: hand it back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc_i]);
              }
              // two fp32 FMAs per instruction (fma.rn.f32x2); the promotion is issue-bound otherwise
#pragma unroll
              for (int c = 0; c < CHUNK; c += 2) {
                const float2 r = __ffma2_rn(make_float2(v[c], v[c + 1]), s2,
                                            make_float2(acc[ch * CHUNK + c], acc[ch * CHUNK + c + 1]));
                acc[ch * CHUNK + c] = r.x;
                acc[ch * CHUNK + c + 1] = r.y;
              }
            }
            }
            if (++acc_i == C::kNumAcc) acc_i = 0;
            if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
          }
        }
      }
      if constexpr (kPipe) {
        if (pending) { fma16(acc + 48, vb, s2_pending); pending = false; }
      }
      if (ok && row_in_tile < t.valid_rows && n0 < p.N) {
        if (w.partial && p.tail_first > 0) {
          // tail split: compact planes of whole tiles, [(tile - tail_first) * split_k + split][128][BLOCK_N]
          float* dst = p.partial +
                       (static_cast<int64_t>(w.tile - p.tail_first) * split_k + w.split) * (BLOCK_M * BLOCK_N) +
                       row_in_tile * BLOCK_N + part * CPW;
          store_row<CPW>(dst, acc, CPW, true);
        } else if (w.partial) {
          float* dst = p.partial + (static_cast<int64_t>(w.split) * p.M + m) * p.N + n0;
          store_row<CPW>(dst, acc, p.N - n0, (p.N % 4) == 0);
        } else {
          store_row<CPW>(out + static_cast<int64_t>(m) * p.ldo + n0, acc, p.N - n0, vec_ok);
        }
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

// Sum of the split-K partial results, added in split order (so the result does not depend on which
// CTA finished first), converted to the output type.  One thread per four consecutive columns.
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ out,
                                                            int M, int N, int64_t ldo, int split_k) {
  const int n4 = N >> 2;
  const int64_t total = static_cast<int64_t>(M) * n4;
  const int64_t plane = static_cast<int64_t>(M) * N;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / n4), c = static_cast<int>(i % n4) * 4;
    const float* src = partial + static_cast<int64_t>(m) * N + c;
    float4 acc = __ldcs(reinterpret_cast<const float4*>(src));
    for (int s = 1; s < split_k; ++s) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src + s * plane));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    OutT* dst = out + static_cast<int64_t>(m) * ldo + c;
    dst[0] = cvt1(dst, acc.x); dst[1] = cvt1(dst, acc.y); dst[2] = cvt1(dst, acc.z); dst[3] = cvt1(dst, acc.w);
  }
}

template <typename OutT>
int launch_reduce(const GemmParams& p, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(p.M) * (p.N >> 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  splitk_reduce_kernel<OutT><<<static_cast<int>(blocks), 256, 0, stream>>>(p.partial, static_cast<OutT*>(p.out), p.M, p.N,
                                                                         p.ldo, p.split_k);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// Sum of the tail tiles' partial planes (tail split), added in split order, converted and written into the
// output tile with its row / column bounds.  grid = (tail tiles, 16 slices of 8 rows): a tile's planes are
// megabytes, so one block per tile would make this kernel longer than the wave it saves.
constexpr int kTailSlices = 16;
template <typename OutT, int BLOCK_N>
__global__ void __launch_bounds__(256) tail_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ out,
                                                          int M, int N, int64_t ldo, int split_k, int tail_first,
                                                          int m_blocks, int n_blocks) {
  int m_blk, n_blk;
  tile_coords(tail_first + blockIdx.x, m_blocks, n_blocks, m_blk, n_blk);
  const float* base = partial + static_cast<int64_t>(blockIdx.x) * split_k * (BLOCK_M * BLOCK_N);
  constexpr int kRows = BLOCK_M / kTailSlices;
  for (int i = threadIdx.x; i < kRows * BLOCK_N / 4; i += blockDim.x) {
    const int r = blockIdx.y * kRows + i / (BLOCK_N / 4), c = (i % (BLOCK_N / 4)) * 4;
    const int m = m_blk * BLOCK_M + r, n = n_blk * BLOCK_N + c;
    if (m >= M || n >= N) continue;
    float4 acc = __ldcs(reinterpret_cast<const float4*>(base + r * BLOCK_N + c));
    for (int s = 1; s < split_k; ++s) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(base + s * (BLOCK_M * BLOCK_N) + r * BLOCK_N + c));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    OutT* dst = out + static_cast<int64_t>(m) * ldo + n;
    const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (n + j < N) dst[j] = cvt1(dst, vals[j]);
  }
}

template <typename OutT>
int launch_tail_reduce(const GemmParams& p, int block_n, cudaStream_t stream) {
  const int m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int n_blocks = (p.N + block_n - 1) / block_n;
  const dim3 grid(m_blocks * n_blocks - p.tail_first, kTailSlices);
  if (block_n == 256)
    tail_reduce_kernel<OutT, 256><<<grid, 256, 0, stream>>>(p.partial, static_cast<OutT*>(p.out), p.M, p.N, p.ldo,
                                                            p.split_k, p.tail_first, m_blocks, n_blocks);
  else
    tail_reduce_kernel<OutT, 128><<<grid, 256, 0, stream>>>(p.partial, static_cast<OutT*>(p.out), p.M, p.N, p.ldo,
                                                            p.split_k, p.tail_first, m_blocks, n_blocks);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ------------------------------------------------------------------------------------ host
template <int BLOCK_N, int EPI_WARPS, int CHUNK, bool GROUPED, typename OutT, int ISSUERS>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<BLOCK_N, EPI_WARPS, ISSUERS>;
  auto kern = gemm_block_fp8_kernel<BLOCK_N, EPI_WARPS, CHUNK, GROUPED, OutT, ISSUERS>;
  static bool attr_set[64] = {false};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev & 63] = true;
  }
  const int m_blocks = (p.M + BLOCK_M - 1) / BLOCK_M;
  const int n_blocks = (p.N + BLOCK_N - 1) / BLOCK_N;
  // grouped: the tile count lives on the device; m-tiles <= ceil(rows/128) + experts bounds the grid
  const long long dense_tiles = static_cast<long long>(m_blocks) * n_blocks;
  const long long split_from = p.split_k == 1 ? dense_tiles : p.tail_first;
  const long long tiles = GROUPED ? static_cast<long long>(m_blocks + p.num_experts) * n_blocks
                                  : split_from + (dense_tiles - split_from) * p.split_k;
  if (tiles > 0x7fffffffLL) return B200_ERR_TOO_LARGE;   // the kernels count tiles in 32 bits
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(ma, mb, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <int BLOCK_N, int EPI_WARPS, int CHUNK, bool GROUPED = false, int ISSUERS = 1>
int launch_dtype(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  switch (p.out_dtype) {
    case B200_DT_BF16: return launch<BLOCK_N, EPI_WARPS, CHUNK, GROUPED, __nv_bfloat16, ISSUERS>(ma, mb, p, stream);
    case B200_DT_F16: return launch<BLOCK_N, EPI_WARPS, CHUNK, GROUPED, __half, ISSUERS>(ma, mb, p, stream);
    case B200_DT_F32: return launch<BLOCK_N, EPI_WARPS, CHUNK, GROUPED, float, ISSUERS>(ma, mb, p, stream);
    default: return B200_ERR_BAD_DTYPE;
  }
}

}  // namespace

// Kernel override for the tests, so that every kernel is reached on every shape: 0 = automatic,
// 128 / 256 = the 128-token-tile kernel with that BLOCK_N, 3 / 3032 / 3064 / 3128 and 4: see below.
int g_force_block_n = 0;

int launch_gemm_swapab(const void* a, int64_t lda, int64_t a_rows, const void* b, int64_t ldb, int64_t w_rows,
                       const GemmParams& p, bool grouped, int token_tile, cudaStream_t stream);

// g_force_block_n values that select the weight-streaming (swapped-operand) kernel: 3 = token tile
// chosen from the shape, 3032 / 3064 / 3128 = that token tile; 4 = never use it.
inline int forced_token_tile() {
  return g_force_block_n == 3032 ? 32 : g_force_block_n == 3064 ? 64 : g_force_block_n == 3128 ? 128 : 0;
}

}  // namespace b200

namespace b200 {
namespace {

// Which kernel a dense problem gets: up to 192 tokens the weight-streaming kernel (gemm_swapab.cu,
// 128 weight rows x up to 64 tokens per tile).  Measured against this file's tiles on the DeepSeek-V3 and
// Llama-3-70B projections: 10-30 % faster up to 64 tokens, 0-25 % faster for 65-192 (two or three token tiles per
// weight tile, the second and third reading the weights from L2), slower from 256 on.
inline bool dense_uses_swapab(int64_t M) { return M <= 192; }
inline int dense_token_tile(int64_t M) { return M <= 32 ? 32 : 64; }

// Split count for small M (up to 512 rows): when the output has too few tiles for the SMs, the k-blocks of
// each tile are spread over several CTAs so that the weights stream through all SMs at once.
int plan_split_k(int64_t M, int64_t N, int64_t K, int sms) {
  if (M > 4 * BLOCK_M || (N % 4) != 0) return 1;   // beyond 512 rows the tile count is never that small
  const int64_t m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
  const int64_t tt = dense_token_tile(M);
  const int64_t tiles = dense_uses_swapab(M) ? ((M + tt - 1) / tt) * ((N + 127) / 128) : m_blocks * ((N + 255) / 256);
  const int64_t nkb = (K + BLOCK_K - 1) / BLOCK_K;
  // measured on DeepSeek-V3 shapes: below 32 k-blocks the launch and pipeline ramp dominate and the
  // extra reduce kernel costs more than the idle SMs
  if (nkb < 32) return 1;
  if (tiles * 2 > sms) {
    // More tiles than half the SMs.  The weight-streaming kernel with two or three token tiles per weight tile can
    // still leave most of its last wave empty (DeepSeek-V3 down projection at 129-192 tokens: 168 tiles on 148 SMs;
    // measured 63.9 us unsplit, 55.5 us split in two): split only to fill such a wave.
    if (!dense_uses_swapab(M)) return 1;
    auto fill = [sms](int64_t t) { return static_cast<double>(t) / static_cast<double>(((t + sms - 1) / sms) * sms); };
    if (fill(tiles) >= 0.7) return 1;
    for (int s2 = 2; s2 <= 4; ++s2)
      if (nkb / s2 >= 8 && fill(tiles * s2) >= 0.75) return s2;
    return 1;
  }
  // (A byte model that picks the count with the best fill of the SMs' wave slots -- 5 for 56 tiles, 3 for 80 -- was
  // measured no better than this rule: 31.5 against 30.1 us on the 56-tile down projection at 64 tokens, 23.8 against
  // 22.5 us on the 80-tile qkv projection; fewer CTAs each pull more than their share of the HBM bandwidth.)
  int64_t s = sms / tiles;
  if (s > nkb / 8) s = nkb / 8;  // at least eight k-blocks per CTA
  if (s > 16) s = 16;
  return s < 2 ? 1 : static_cast<int>(s);
}

// Split-K workspace: split_k fp32 planes of [M, N].  (Folding the sum into the GEMM kernel -- the CTA that
// completes a tile's last split adds the planes -- was measured slower than the second kernel at every M:
// the device-wide fences and the CTA-wide meeting it needs cost more than a launch.)
inline size_t splitk_workspace_bytes(int split_k, int64_t M, int64_t N) {
  return static_cast<size_t>(split_k) * M * N * sizeof(float);
}

// Tile width of the 128-token-tile kernel for a dense problem: 128 x 256 when that fills at least three
// quarters of the SMs in one wave (two waves of half-size tiles take as long), else 128 x 128.
inline int dense_block_n(int64_t M, int64_t N, int sms) {
  const int64_t m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
  return 4 * m_blocks * ((N + 255) / 256) < 3 * sms ? 128 : 256;
}

// Tail split for large M: when the last wave of tiles would occupy at most half of the SMs, those
// tiles' k-blocks are divided among the SMs instead (e.g. 896 tiles on 148 SMs: six full waves, then
// 8 tiles x 18 splits instead of a seventh wave that is 5 % full).
struct TailPlan {
  int tail_first = 0, split_k = 1, kb_per_split = 0;
  size_t bytes = 0;
};
TailPlan plan_tail(int64_t M, int64_t N, int64_t K, int block_n, int sms) {
  TailPlan t;
  const int64_t tiles = ((M + BLOCK_M - 1) / BLOCK_M) * ((N + block_n - 1) / block_n);
  const int64_t nkb = (K + BLOCK_K - 1) / BLOCK_K;
  if (M <= BLOCK_M || tiles <= sms || tiles > 0x3fffffff || nkb < 16) return t;
  const int64_t tail = tiles % sms;
  if (tail == 0 || tail * 2 > sms) return t;   // at least two splits per tail tile
  int64_t s = sms / tail;
  if (s > nkb / 4) s = nkb / 4;   // at least four k-blocks per work unit
  if (s > 32) s = 32;
  if (s < 2) return t;
  t.kb_per_split = static_cast<int>((nkb + s - 1) / s);
  t.split_k = static_cast<int>((nkb + t.kb_per_split - 1) / t.kb_per_split);
  t.tail_first = static_cast<int>(tiles - tail);
  t.bytes = static_cast<size_t>(tail) * t.split_k * BLOCK_M * block_n * sizeof(float);
  return t;
}

int dense_mm(const void* a, int64_t lda, const void* b, int64_t ldb, const float* sa, int64_t sa_stride_m,
             int64_t sa_stride_g, const float* sb, int64_t sb_stride_n, int64_t sb_stride_g, void* out, int64_t ldo,
             int out_dtype, int64_t M, int64_t N, int64_t K, int split_k, void* workspace, size_t workspace_bytes,
             void* stream, int sa_ue8m0 = 0) {
  if (M < 0 || N < 0 || K <= 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || N == 0) return B200_OK;
  if (M > 0x7fffff00LL || N > 0x7fffff00LL || K > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa || !sb || !out) return B200_ERR_NULL_PTR;
  if (out_dtype != B200_DT_BF16 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_F32) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldo < N) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || !aligned16(a) || !aligned16(b)) return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_g < 0 || sb_stride_n < 0 || sb_stride_g < 0) return B200_ERR_BAD_STRIDE;
  const int nkb = static_cast<int>((K + BLOCK_K - 1) / BLOCK_K);
  if (split_k < 0 || split_k > 64) return B200_ERR_BAD_SHAPE;
  if (split_k > 1) {
    if ((N % 4) != 0 || split_k > nkb) return B200_ERR_BAD_SHAPE;
    if (!workspace) return B200_ERR_NULL_PTR;
    if (!aligned16(workspace)) return B200_ERR_MISALIGNED;
    if (workspace_bytes < splitk_workspace_bytes(split_k, M, N)) return B200_ERR_TOO_LARGE;
  }
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  if (gemm_sticky_status() != 0) return B200_ERR_DEVICE_TIMEOUT;   // sticky until b200_gemm_device_status clears it
  TailPlan tail;
  if (split_k == 0) {
    // automatic: split only when the caller gave room for it
    split_k = plan_split_k(M, N, K, sm_count());
    if (split_k > 1 && (!workspace || !aligned16(workspace) || workspace_bytes < splitk_workspace_bytes(split_k, M, N)))
      split_k = 1;
    if (split_k == 1 && M > BLOCK_M && !dense_uses_swapab(M) && g_force_block_n == 0 && workspace && aligned16(workspace)) {
      tail = plan_tail(M, N, K, dense_block_n(M, N, sm_count()), sm_count());
      if (tail.split_k > 1 && workspace_bytes < tail.bytes) tail = TailPlan();
    }
  }

  GemmParams p;
  p.sa = sa; p.sb = sb; p.out = out;
  p.sa_stride_m = sa_stride_m; p.sa_stride_g = sa_stride_g;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g;
  p.ldo = ldo;
  p.M = static_cast<int>(M); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = out_dtype;
  p.status = gemm_status_ptr();
  p.expert_offsets = nullptr; p.problem_sizes = nullptr; p.sb_stride_e = 0; p.num_experts = 0;
  p.split_k = split_k < 1 ? 1 : split_k;
  p.kb_per_split = (nkb + p.split_k - 1) / p.split_k;
  // every split must own at least one k-block (an empty one would store zeros, which is still right,
  // but the count is trimmed so that no CTA is launched for nothing)
  p.split_k = (nkb + p.kb_per_split - 1) / p.kb_per_split;
  p.tail_first = 0;
  if (tail.split_k > 1) {
    p.split_k = tail.split_k;
    p.kb_per_split = tail.kb_per_split;
    p.tail_first = tail.tail_first;
  }
  p.partial = static_cast<float*>(workspace);
  p.sa_ue8m0 = sa_ue8m0;
  if (!p.status) return B200_ERR_CUDA;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // One CTA per tile: 128 x 256 when that fills at least three quarters of the SMs in one wave (two
  // waves of half-size tiles take as long), else 128 x 128.
  if (g_force_block_n == 3 || forced_token_tile() != 0 || (g_force_block_n == 0 && dense_uses_swapab(M))) {
    int tt = forced_token_tile();
    if (tt == 0) tt = dense_token_tile(M);
    rc = launch_gemm_swapab(a, lda, M, b, ldb, N, p, false, tt, st);
    if (rc != B200_OK || p.split_k == 1) return rc;
    switch (out_dtype) {
      case B200_DT_BF16: return launch_reduce<__nv_bfloat16>(p, st);
      case B200_DT_F16: return launch_reduce<__half>(p, st);
      default: return launch_reduce<float>(p, st);
    }
  }
  const int64_t m_blocks = (M + BLOCK_M - 1) / BLOCK_M;
  int block_n = 256;
  if (p.split_k == 1 || p.tail_first > 0) block_n = dense_block_n(M, N, sm_count());
  if (g_force_block_n == 128 || g_force_block_n == 256) block_n = g_force_block_n;
  if (g_force_block_n == 2562) block_n = 256;   // A/B runs: 256-wide tile, two MMA issuers
  if (g_force_block_n == 1282) block_n = 128;   // A/B runs: 128-wide tile, two MMA issuers

  CUtensorMap ma, mb;
  rc = make_map_u8_2d(&ma, a, M, K, lda, BLOCK_M);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, N, K, ldb, block_n);
  if (rc != B200_OK) return rc;
  if (g_force_block_n == 1282) rc = launch_dtype<128, 8, 64, false, 2>(ma, mb, p, st);
  else if (block_n != 256) rc = launch_dtype<128, 8, 64>(ma, mb, p, st);
  else if (g_force_block_n == 2562) rc = launch_dtype<256, 16, 32, false, 2>(ma, mb, p, st);
  else rc = launch_dtype<256, 16, 32, false, 1>(ma, mb, p, st);
  if (rc != B200_OK || p.split_k == 1) return rc;
  if (p.tail_first > 0) {
    switch (out_dtype) {
      case B200_DT_BF16: return launch_tail_reduce<__nv_bfloat16>(p, block_n, st);
      case B200_DT_F16: return launch_tail_reduce<__half>(p, block_n, st);
      default: return launch_tail_reduce<float>(p, block_n, st);
    }
  }
  switch (out_dtype) {
    case B200_DT_BF16: return launch_reduce<__nv_bfloat16>(p, st);
    case B200_DT_F16: return launch_reduce<__half>(p, st);
    default: return launch_reduce<float>(p, st);
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_fp8_blockwise_scaled_mm(const void* a, int64_t lda, const void* b, int64_t ldb, const float* sa,
                                            int64_t sa_stride_m, int64_t sa_stride_g, const float* sb,
                                            int64_t sb_stride_n, int64_t sb_stride_g, void* out, int64_t ldo,
                                            int out_dtype, int64_t M, int64_t N, int64_t K, void* stream) {
  return b200::dense_mm(a, lda, b, ldb, sa, sa_stride_m, sa_stride_g, sb, sb_stride_n, sb_stride_g, out, ldo, out_dtype,
                        M, N, K, 1, nullptr, 0, stream);
}

extern "C" int b200_fp8_blockwise_scaled_mm_splitk(const void* a, int64_t lda, const void* b, int64_t ldb,
                                                   const float* sa, int64_t sa_stride_m, int64_t sa_stride_g,
                                                   const float* sb, int64_t sb_stride_n, int64_t sb_stride_g, void* out,
                                                   int64_t ldo, int out_dtype, int64_t M, int64_t N, int64_t K,
                                                   int split_k, void* workspace, size_t workspace_bytes, void* stream) {
  return b200::dense_mm(a, lda, b, ldb, sa, sa_stride_m, sa_stride_g, sb, sb_stride_n, sb_stride_g, out, ldo, out_dtype,
                        M, N, K, split_k, workspace, workspace_bytes, stream);
}

extern "C" int b200_fp8_blockwise_scaled_mm_ue8m0(const void* a, int64_t lda, const void* b, int64_t ldb,
                                                  const uint32_t* sa_packed, int64_t sa_stride_m, int64_t sa_stride_pack,
                                                  const float* sb, int64_t sb_stride_n, int64_t sb_stride_g, void* out,
                                                  int64_t ldo, int out_dtype, int64_t M, int64_t N, int64_t K,
                                                  void* stream) {
  return b200::dense_mm(a, lda, b, ldb, reinterpret_cast<const float*>(sa_packed), sa_stride_m, sa_stride_pack, sb,
                        sb_stride_n, sb_stride_g, out, ldo, out_dtype, M, N, K, 1, nullptr, 0, stream, 1);
}

extern "C" int b200_fp8_blockwise_scaled_mm_splitk_plan(int64_t M, int64_t N, int64_t K, int sm_count, int* split_k,
                                                        size_t* workspace_bytes) {
  if (M < 0 || N < 0 || K <= 0) return B200_ERR_BAD_SHAPE;
  if (!split_k || !workspace_bytes) return B200_ERR_NULL_PTR;
  const int sms = sm_count > 0 ? sm_count : 148;
  const int s = (M == 0 || N == 0) ? 1 : b200::plan_split_k(M, N, K, sms);
  *split_k = s;
  *workspace_bytes = s > 1 ? b200::splitk_workspace_bytes(s, M, N) : 0;
  if (s == 1 && M > 128 && !b200::dense_uses_swapab(M) && N > 0) {   // large M: split of the last, mostly empty wave of tiles
    const b200::TailPlan t = b200::plan_tail(M, N, K, b200::dense_block_n(M, N, sms), sms);
    if (t.split_k > 1) {
      *split_k = t.split_k;
      *workspace_bytes = t.bytes;
    }
  }
  return B200_OK;
}

extern "C" int b200_fp8_blockwise_scaled_grouped_mm(const void* a, int64_t lda, const void* b, int64_t ldb,
                                                    const float* sa, int64_t sa_stride_m, int64_t sa_stride_g,
                                                    const float* sb, int64_t sb_stride_e, int64_t sb_stride_n,
                                                    int64_t sb_stride_g, void* out, int64_t ldo, int out_dtype,
                                                    const int32_t* expert_offsets, const int32_t* problem_sizes,
                                                    int num_experts, int64_t total_rows, int64_t N, int64_t K,
                                                    void* stream) {
  using namespace b200;
  if (total_rows < 0 || N < 0 || K <= 0 || num_experts <= 0) return B200_ERR_BAD_SHAPE;
  if (total_rows == 0 || N == 0) return B200_OK;
  if (num_experts > Cfg<256, 16>::kMaxExperts) return B200_ERR_TOO_LARGE;
  if (total_rows > 0x7fffff00LL || K > 0x7fffff00LL || N * num_experts > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!a || !b || !sa || !sb || !out || !expert_offsets || !problem_sizes) return B200_ERR_NULL_PTR;
  if (out_dtype != B200_DT_BF16 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_F32) return B200_ERR_BAD_DTYPE;
  if (lda < K || ldb < K || ldo < N) return B200_ERR_BAD_STRIDE;
  if ((lda % 16) != 0 || (ldb % 16) != 0 || !aligned16(a) || !aligned16(b)) return B200_ERR_MISALIGNED;
  if (sa_stride_m < 0 || sa_stride_g < 0 || sb_stride_e < 0 || sb_stride_n < 0 || sb_stride_g < 0)
    return B200_ERR_BAD_STRIDE;
  // an expert's weights are rows [e*N, (e+1)*N) of one matrix and its scales are indexed by 128-row block:
  // with N % 128 != 0 both would straddle experts
  if (N % 128 != 0) return B200_ERR_BAD_SHAPE;
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  if (gemm_sticky_status() != 0) return B200_ERR_DEVICE_TIMEOUT;

  GemmParams p;
  p.sa = sa; p.sb = sb; p.out = out;
  p.sa_stride_m = sa_stride_m; p.sa_stride_g = sa_stride_g;
  p.sb_stride_n = sb_stride_n; p.sb_stride_g = sb_stride_g; p.sb_stride_e = sb_stride_e;
  p.ldo = ldo;
  p.M = static_cast<int>(total_rows); p.N = static_cast<int>(N); p.K = static_cast<int>(K);
  p.out_dtype = out_dtype;
  p.status = gemm_status_ptr();
  p.expert_offsets = expert_offsets; p.problem_sizes = problem_sizes; p.num_experts = num_experts;
  p.split_k = 1; p.kb_per_split = 0; p.partial = nullptr; p.tail_first = 0; p.sa_ue8m0 = 0;
  if (!p.status) return B200_ERR_CUDA;

  // An expert's weights are rows [e*N, (e+1)*N) of one [E*N, K] matrix; a 128 x 256 tile must not
  // straddle two experts' rows, so the wide tile needs N % 256 == 0.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Up to 64 rows per expert on average the weight-streaming kernel is used (measured on the DeepSeek-V3
  // expert shapes, 256 experts: 1.25x at 16-32 rows per expert, level at 64); beyond that an expert fills most
  // of a 128-row token tile and the wider MMAs of this file's kernel win (1.15x at 96 rows, level at 128).
  const int64_t avg_rows = total_rows / num_experts;
  const bool auto_swap = g_force_block_n == 0 && avg_rows <= 64;
  if ((g_force_block_n == 3 || forced_token_tile() != 0 || auto_swap) && N % 128 == 0) {
    int tt = forced_token_tile();
    if (tt == 0) tt = avg_rows <= 20 ? 32 : 64;
    return launch_gemm_swapab(a, lda, total_rows, b, ldb, N * num_experts, p, true, tt, st);
  }
  // Up to 256 rows per expert the 128-wide tile (four accumulators, twice as many tiles to balance over the SMs)
  // measured faster than the 256-wide one: 256 experts x 128 rows, 1.92 / 1.18 ms against 2.29 / 1.28 ms for the
  // two expert GEMMs of the DeepSeek-V3 layer.
  const bool wide = N % 256 == 0 && g_force_block_n != 128 && (avg_rows > 256 || g_force_block_n == 256);
  const int block_n = wide ? 256 : 128;
  CUtensorMap ma, mb;
  rc = make_map_u8_2d(&ma, a, total_rows, K, lda, BLOCK_M);
  if (rc != B200_OK) return rc;
  rc = make_map_u8_2d(&mb, b, N * num_experts, K, ldb, block_n);
  if (rc != B200_OK) return rc;
  return block_n == 256 ? launch_dtype<256, 16, 32, true>(ma, mb, p, st)
                        : launch_dtype<128, 8, 64, true>(ma, mb, p, st);
}

extern "C" int b200_debug_force_block_n(int block_n) {
  b200::g_force_block_n = block_n;
  return B200_OK;
}
