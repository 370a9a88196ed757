// Expert-parallel token exchange over NVLink for the block-FP8 MoE layer: the dispatch of quantised
// token rows to the ranks that own their experts, and the combine of the expert outputs back to the
// ranks that own the tokens.
//
// The reference moves tokens with DeepEP (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:314-480;
// the dispatch sends ALREADY-QUANTISED e4m3 rows + fp32 scales, :328-336) inside DeepEPMoE
// (python/sglang/srt/layers/moe/ep_moe/layer.py:427-489); experts are split contiguously over the ranks
// (python/sglang/srt/layers/moe/fused_moe_triton/layer.py:165-185).  Here the exchange is two kernels over a
// symmetric buffer that every rank has mapped (one process per GPU):
//
//   dispatch   plan (one block): for every (token, choice) slot the destination rank and its position in
//              that rank's receive region for this source -- a stable counting sort over <= 8 destinations.
//              push (whole grid, one warp per row): the row's 16-byte vectors of codes and scales and its
//              (local expert id, source slot) pair are stored straight into the destination's receive
//              region with peer stores; the per-destination counts go into the destination's count table.
//   combine    one warp per received row: the expert output row (bf16) is stored into the source rank's
//              return buffer at the row's original (token, choice) slot.
// The last block of each grid meets the other ranks at a flag barrier (peer_sync.cuh), so nothing on the
// host ever looks at a count: the receive regions have a fixed capacity per source and the rows a rank did
// not receive are marked with expert id -1 for the grouped GEMM's routing tables.  A source that routes more
// rows to one rank than the capacity holds records B200_EP_OVERFLOW in the status word and drops the excess
// (the caller sizes the capacity; capacity = tokens * topk can never overflow).
#include "peer_sync.cuh"

namespace b200 {
namespace {

constexpr int kEpOverflow = 31;

struct EpLayout {
  // byte offsets inside every rank's symmetric buffer (identical on all ranks)
  int64_t recv_q, recv_s, recv_meta, recv_cnt, back;
  int capacity;      // rows per source rank in a receive region
  int H, G;          // row bytes of codes, scale floats per row
};

struct EpParams {
  void* peers[kMaxRanks];
  PeerSync sync;
  EpLayout lay;
  int rank, world;
};

// ---- dispatch: plan
// pos[f] = position of slot f among the slots of the same destination rank (stable), counts[d] = slots for d.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int32_t* __restrict__ topk_ids, int n_slots,
                                                       int experts_per_rank, int world, int capacity,
                                                       int32_t* __restrict__ pos, int32_t* __restrict__ counts,
                                                       EpParams p) {
  __shared__ int warp_tot[32][kMaxRanks];
  __shared__ int base[kMaxRanks];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kMaxRanks) base[threadIdx.x] = 0;
  __syncthreads();
  for (int f0 = 0; f0 < n_slots; f0 += blockDim.x) {
    const int f = f0 + threadIdx.x;
    int d = -1;
    if (f < n_slots) {
      const int e = topk_ids[f];
      d = (e >= 0) ? e / experts_per_rank : -1;
      if (d >= world) d = -1;
    }
    int my_rank_in_warp = 0;
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      const uint32_t m = __ballot_sync(0xffffffffu, d == r);
      if (d == r) my_rank_in_warp = __popc(m & ((1u << lane) - 1u));
      if (lane == 0) warp_tot[warp][r] = __popc(m);
    }
    __syncthreads();
    int before = 0;
    if (d >= 0) {
      for (int w = 0; w < warp; ++w) before += warp_tot[w][d];
      pos[f] = base[d] + before + my_rank_in_warp;
    } else if (f < n_slots) {
      pos[f] = -1;
    }
    __syncthreads();
    if (threadIdx.x < kMaxRanks) {
      int tot = 0;
      for (int w = 0; w < 32; ++w) tot += warp_tot[w][threadIdx.x];
      base[threadIdx.x] += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x < world) {
    int c = base[threadIdx.x];
    if (c > capacity) {
      atomicCAS(p.sync.status, 0, kEpOverflow);
      c = capacity;
    }
    counts[threadIdx.x] = c;
    // the destination's count table: entry [this rank] = rows this rank sends it
    int32_t* cnt = reinterpret_cast<int32_t*>(static_cast<char*>(p.peers[threadIdx.x]) + p.lay.recv_cnt);
    cnt[p.rank] = c;
  }
}

__device__ __forceinline__ void copy16(void* dst, const void* src) {
  *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
}

// The last block of the grid to get here meets the other ranks; `counter` returns to zero for the next launch.
__device__ __forceinline__ void last_block_barrier(const PeerSync& sync, unsigned int* counter, int code) {
  __shared__ bool last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(counter, 1u);
    last = (done == gridDim.x - 1);
    if (last) *counter = 0;
  }
  __syncthreads();
  if (last) {
    __threadfence_system();
    // the barrier's flags are indexed by block: every rank's last block uses index 0
    PeerSync s0 = sync;
    if (threadIdx.x < s0.world) {
      const int peer = threadIdx.x;
      uint32_t* theirs = s0.signals[peer] + s0.flag_base + s0.rank;
      uint32_t* mine = s0.signals[s0.rank] + s0.flag_base + peer;
      const long long t0 = clock64();
      bool ok = true;
      while (cas_release_sys(theirs, 0u, 1u) != 0u) {
        if (clock64() - t0 > kPeerWaitCycles) { ok = false; break; }
      }
      if (ok) {
        while (cas_acquire_sys(mine, 1u, 0u) != 1u) {
          if (clock64() - t0 > kPeerWaitCycles) { ok = false; break; }
        }
      }
      if (!ok) atomicCAS(s0.status, 0, code);
    }
    __syncthreads();
  }
}

// ---- dispatch: push.  One warp per (token, choice) slot.
__global__ void __launch_bounds__(256) ep_push_kernel(const uint8_t* __restrict__ q, const float* __restrict__ s,
                                                      const int32_t* __restrict__ topk_ids,
                                                      const int32_t* __restrict__ pos, int n_slots, int topk,
                                                      int experts_per_rank, unsigned int* counter, EpParams p) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int H = p.lay.H, G = p.lay.G, cap = p.lay.capacity;
  for (int f = blockIdx.x * warps_per_block + (threadIdx.x >> 5); f < n_slots; f += gridDim.x * warps_per_block) {
    const int ps = pos[f];
    if (ps < 0 || ps >= cap) continue;
    const int e = topk_ids[f];
    const int d = e / experts_per_rank;
    const int t = f / topk;
    const int64_t row = static_cast<int64_t>(p.rank) * cap + ps;       // row in the destination's receive regions
    char* dst = static_cast<char*>(p.peers[d]);
    const uint8_t* src_q = q + static_cast<int64_t>(t) * H;
    char* dst_q = dst + p.lay.recv_q + row * H;
    for (int i = lane * 16; i < H; i += 32 * 16) copy16(dst_q + i, src_q + i);
    const char* src_s = reinterpret_cast<const char*>(s + static_cast<int64_t>(t) * G);
    char* dst_s = dst + p.lay.recv_s + row * (G * 4);
    for (int i = lane * 16; i < G * 4; i += 32 * 16) copy16(dst_s + i, src_s + i);
    if (lane == 0) {
      int2 meta = make_int2(e - d * experts_per_rank, f);
      *reinterpret_cast<int2*>(dst + p.lay.recv_meta + row * 8) = meta;
    }
  }
  last_block_barrier(p.sync, counter, 32);
}

// ---- after the dispatch: expert ids of the receive regions (-1 = no row), in region order
__global__ void __launch_bounds__(256) ep_unpack_ids_kernel(const char* __restrict__ local, EpLayout lay, int world,
                                                            int32_t* __restrict__ ids) {
  const int R = world * lay.capacity;
  const int32_t* cnt = reinterpret_cast<const int32_t*>(local + lay.recv_cnt);
  const int2* meta = reinterpret_cast<const int2*>(local + lay.recv_meta);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < R; r += gridDim.x * blockDim.x) {
    const int src = r / lay.capacity, i = r - src * lay.capacity;
    ids[r] = (i < cnt[src]) ? meta[r].x : -1;
  }
}

// ---- combine: one warp per received row; rows[row_of[r]] is the expert output of receive-region row r
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_kernel(const T* __restrict__ rows, const int32_t* __restrict__ row_of,
                                                         int out_cols, unsigned int* counter, EpParams p) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const char* local = static_cast<const char*>(p.peers[p.rank]);
  const int32_t* cnt = reinterpret_cast<const int32_t*>(local + p.lay.recv_cnt);
  const int2* meta = reinterpret_cast<const int2*>(local + p.lay.recv_meta);
  const int cap = p.lay.capacity;
  const int R = p.world * cap;
  const int64_t row_bytes = static_cast<int64_t>(out_cols) * sizeof(T);
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < R; r += gridDim.x * warps_per_block) {
    const int src = r / cap, i = r - src * cap;
    if (i >= cnt[src]) continue;
    const int slot = meta[r].y;
    const char* from = reinterpret_cast<const char*>(rows) + static_cast<int64_t>(row_of ? row_of[r] : r) * row_bytes;
    char* to = static_cast<char*>(p.peers[src]) + p.lay.back + static_cast<int64_t>(slot) * row_bytes;
    for (int64_t b = lane * 16; b < row_bytes; b += 32 * 16) copy16(to + b, from + b);
  }
  last_block_barrier(p.sync, counter, 33);
}

int fill_params(EpParams* p, void* const* peer_buffers, void* const* peer_signal_pads, int rank, int world,
                int64_t flag_base_words, int* status, const int64_t* layout_offsets, int capacity, int H, int G) {
  if (!peer_buffers || !layout_offsets) return B200_ERR_NULL_PTR;
  int rc = make_peer_sync(&p->sync, peer_signal_pads, rank, world, flag_base_words, status);
  if (rc != B200_OK) return rc;
  for (int r = 0; r < kMaxRanks; ++r) {
    p->peers[r] = r < world ? peer_buffers[r] : nullptr;
    if (r < world && !p->peers[r]) return B200_ERR_NULL_PTR;
    if (r < world && !aligned16(p->peers[r])) return B200_ERR_MISALIGNED;
  }
  if (capacity <= 0 || H <= 0 || G <= 0 || H % 16 != 0 || (G * 4) % 16 != 0) return B200_ERR_BAD_SHAPE;
  for (int i = 0; i < 5; ++i)
    if (layout_offsets[i] < 0 || layout_offsets[i] % 16 != 0) return B200_ERR_MISALIGNED;
  p->lay.recv_q = layout_offsets[0];
  p->lay.recv_s = layout_offsets[1];
  p->lay.recv_meta = layout_offsets[2];
  p->lay.recv_cnt = layout_offsets[3];
  p->lay.back = layout_offsets[4];
  p->lay.capacity = capacity;
  p->lay.H = H;
  p->lay.G = G;
  p->rank = rank;
  p->world = world;
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int64_t b200_ep_buffer_bytes(int world_size, int capacity, int hidden, int max_slots, int out_elem_bytes,
                                        int64_t* layout_offsets_5) {
  // regions: codes, scales, (expert, slot) pairs, counts, returned rows; each starts on a 256-byte boundary
  if (world_size < 1 || capacity <= 0 || hidden <= 0 || hidden % 128 != 0 || max_slots <= 0 || !layout_offsets_5) return -1;
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  const int64_t R = static_cast<int64_t>(world_size) * capacity;
  int64_t off = 0;
  layout_offsets_5[0] = off; off = up(off + R * hidden);
  layout_offsets_5[1] = off; off = up(off + R * (hidden / 128) * 4);
  layout_offsets_5[2] = off; off = up(off + R * 8);
  layout_offsets_5[3] = off; off = up(off + static_cast<int64_t>(world_size) * 4);
  layout_offsets_5[4] = off; off = up(off + static_cast<int64_t>(max_slots) * hidden * out_elem_bytes);
  return off;
}

extern "C" int b200_ep_dispatch(const void* q, const void* s, int scale_words_per_row, const int32_t* topk_ids,
                                int64_t num_tokens, int topk, int hidden, int experts_per_rank, void* const* peer_buffers,
                                void* const* peer_signal_pads, const int64_t* layout_offsets_5, int capacity, int rank,
                                int world_size, int64_t flag_base_words, int* status, int32_t* scratch_pos,
                                int32_t* scratch_counts, unsigned int* scratch_counter, void* stream) {
  using namespace b200;
  if (!q || !s || !topk_ids || !scratch_pos || !scratch_counts || !scratch_counter) return B200_ERR_NULL_PTR;
  if (num_tokens < 0 || topk <= 0 || experts_per_rank <= 0 || hidden % 128 != 0) return B200_ERR_BAD_SHAPE;
  const int64_t n_slots = num_tokens * topk;
  if (n_slots > 0x7fffff00LL) return B200_ERR_TOO_LARGE;
  if (!aligned16(q) || !aligned16(s)) return B200_ERR_MISALIGNED;
  // a token's scales are `scale_words_per_row` 32-bit words (0 = one fp32 per 128 codes; 16-byte multiples, and no
  // more than the region holds: hidden / 128 words per row)
  const int G = scale_words_per_row > 0 ? scale_words_per_row : hidden / 128;
  if (G % 4 != 0 || G > hidden / 128) return B200_ERR_BAD_SHAPE;
  EpParams p;
  int rc = fill_params(&p, peer_buffers, peer_signal_pads, rank, world_size, flag_base_words, status, layout_offsets_5,
                       capacity, hidden, G);
  if (rc != B200_OK) return rc;
  rc = require_sm100();
  if (rc != B200_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ep_plan_kernel<<<1, 1024, 0, st>>>(topk_ids, static_cast<int>(n_slots), experts_per_rank, world_size, capacity,
                                     scratch_pos, scratch_counts, p);
  B200_CUDA_TRY(cudaGetLastError());
  const int warps = 8;
  int64_t blocks = (n_slots + warps - 1) / warps;
  const int cap_blocks = 4 * sm_count();
  if (blocks > cap_blocks) blocks = cap_blocks;
  if (blocks < 1) blocks = 1;
  ep_push_kernel<<<static_cast<int>(blocks), 32 * warps, 0, st>>>(static_cast<const uint8_t*>(q),
                                                                 static_cast<const float*>(s), topk_ids, scratch_pos,
                                                                 static_cast<int>(n_slots), topk, experts_per_rank,
                                                                 scratch_counter, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_ep_received_expert_ids(const void* local_buffer, const int64_t* layout_offsets_5, int capacity,
                                           int hidden, int world_size, int32_t* ids_out, void* stream) {
  using namespace b200;
  if (!local_buffer || !layout_offsets_5 || !ids_out) return B200_ERR_NULL_PTR;
  if (capacity <= 0 || world_size < 1 || world_size > kMaxRanks) return B200_ERR_BAD_SHAPE;
  EpLayout lay;
  lay.recv_q = layout_offsets_5[0]; lay.recv_s = layout_offsets_5[1]; lay.recv_meta = layout_offsets_5[2];
  lay.recv_cnt = layout_offsets_5[3]; lay.back = layout_offsets_5[4];
  lay.capacity = capacity; lay.H = hidden; lay.G = hidden / 128;
  const int R = world_size * capacity;
  ep_unpack_ids_kernel<<<(R + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(local_buffer), lay, world_size, ids_out);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_ep_combine(const void* rows, const int32_t* row_of, int dtype, int hidden, void* const* peer_buffers,
                               void* const* peer_signal_pads, const int64_t* layout_offsets_5, int capacity, int rank,
                               int world_size, int64_t flag_base_words, int* status, unsigned int* scratch_counter,
                               void* stream) {
  using namespace b200;
  if (!rows || !scratch_counter) return B200_ERR_NULL_PTR;
  if (dtype != B200_DT_BF16 && dtype != B200_DT_F16) return B200_ERR_BAD_DTYPE;
  if (hidden % 128 != 0 || !aligned16(rows)) return B200_ERR_BAD_SHAPE;
  EpParams p;
  int rc = fill_params(&p, peer_buffers, peer_signal_pads, rank, world_size, flag_base_words, status, layout_offsets_5,
                       capacity, hidden, hidden / 128);
  if (rc != B200_OK) return rc;
  rc = require_sm100();
  if (rc != B200_OK) return rc;
  const int warps = 8;
  int64_t blocks = (static_cast<int64_t>(world_size) * capacity + warps - 1) / warps;
  const int cap_blocks = 4 * sm_count();
  if (blocks > cap_blocks) blocks = cap_blocks;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200_DT_BF16)
    ep_combine_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 32 * warps, 0, st>>>(
        static_cast<const __nv_bfloat16*>(rows), row_of, hidden, scratch_counter, p);
  else
    ep_combine_kernel<__half><<<static_cast<int>(blocks), 32 * warps, 0, st>>>(static_cast<const __half*>(rows), row_of,
                                                                               hidden, scratch_counter, p);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
