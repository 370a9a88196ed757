// moe_align_block_size: sorts the flat (token, choice) indices by expert and pads every expert's run to a
// multiple of the GEMM row block, for MoE kernels that walk fixed-size row blocks.  HBM-bound integer work.
//
// Stands in for sgl-kernel/csrc/moe/moe_align_kernel.cu:28-366 (op `moe_align_block_size`), called from
// python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:558-628.
//
// Conventions kept from the reference: ids are shifted by one, so slot 0 collects id -1 (experts filtered out
// by expert parallelism) and `num_experts` counts the slots (real experts + 1); expert_ids[block] is the
// slot minus one; padding positions hold `numel`.  The reference hands out positions inside an expert with
// atomics (moe_align_kernel.cu:37-41), so its order inside an expert varies from run to run; here it is the
// ascending flat index (a stable counting sort), one of the orders the reference can produce.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kAlignThreads = 256;
constexpr int kAlignChunk = 2048;    // ids per chunk of the three-launch form
constexpr int kAlignSmall = 4096;    // ids handled by the one-block form
constexpr int kMaxSlots = 2048;

__device__ __forceinline__ int load_id(const void* ids, int is64, int64_t i) {
  return is64 ? static_cast<int>(static_cast<const int64_t*>(ids)[i]) : static_cast<const int32_t*>(ids)[i];
}

// Warp 0: exclusive prefix of the padded counts.  In: s_cnt[slots].  Out: s_off[slots + 1].
__device__ __forceinline__ void padded_prefix_warp0(const int32_t* s_cnt, int32_t* s_off, int slots, int block_size) {
  const int lane = threadIdx.x;
  const int per = (slots + 31) / 32;
  const int lo = min(lane * per, slots), hi = min(lo + per, slots);
  int sum = 0;
  for (int e = lo; e < hi; ++e) sum += (s_cnt[e] + block_size - 1) / block_size * block_size;
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  int run = incl - sum;
  for (int e = lo; e < hi; ++e) {
    s_off[e] = run;
    run += (s_cnt[e] + block_size - 1) / block_size * block_size;
  }
  if (lane == 31) s_off[slots] = incl;
}

// Everything that follows from the counts and the padded offsets: cumsum, total, expert id of each row block,
// and (optionally) `numel` in the padding positions.  Called by all threads of a block after a barrier.
__device__ __forceinline__ void write_tables(const int32_t* s_cnt, const int32_t* s_off, int slots, int block_size,
                                             int64_t numel, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                             int32_t* expert_ids, int64_t expert_ids_capacity,
                                             int32_t* num_tokens_post_pad, int32_t* cumsum, int pad) {
  const int total = s_off[slots];
  if (threadIdx.x == 0) *num_tokens_post_pad = total;
  for (int e = threadIdx.x; e <= slots; e += blockDim.x) cumsum[e] = s_off[e];
  for (int e = threadIdx.x; e < slots; e += blockDim.x) {
    for (int i = s_off[e]; i < s_off[e + 1]; i += block_size) {
      const int b = i / block_size;
      if (b < expert_ids_capacity) expert_ids[b] = e - 1;
    }
  }
  if (pad) {
    const int32_t fill = static_cast<int32_t>(numel);
    // padding positions of every slot, then the reference's round-up of the filled range to 4 entries
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int e = warp; e < slots; e += nwarps) {
      const int lo = s_off[e] + s_cnt[e], hi = s_off[e + 1];
      for (int i = lo + lane; i < hi; i += 32)
        if (i < sorted_capacity) sorted_token_ids[i] = fill;
    }
    const int64_t end4 = (static_cast<int64_t>(total) + 3) / 4 * 4;
    const int64_t end = end4 < sorted_capacity ? end4 : sorted_capacity;
    for (int64_t i = total + threadIdx.x; i < end; i += blockDim.x) sorted_token_ids[i] = fill;
  }
}

// Stable placement of `count` ids (held in s_ids) by one warp: 32 ids at a time, equal slots inside the 32
// ranked with a match mask.  s_next[slot] = next free position of the slot.
__device__ __forceinline__ void place_warp0(const int32_t* s_ids, int count, int64_t base, int slots, int32_t* s_next,
                                            int32_t* sorted_token_ids, int64_t sorted_capacity, int first = 0) {
  const int lane = threadIdx.x & 31;
  for (int i0 = first; i0 < count; i0 += 32) {
    const int i = i0 + lane;
    const int slot = i < count ? s_ids[i] + 1 : -1;
    const bool valid = slot >= 0 && slot < slots;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? slot : -1 - lane);
    if (valid) {
      const int pos = s_next[slot] + __popc(peers & ((1u << lane) - 1u));
      if (pos < sorted_capacity) sorted_token_ids[pos] = static_cast<int32_t>(base + i);
    }
    __syncwarp();
    if (valid && (peers >> lane) <= 1u) s_next[slot] += __popc(peers);   // highest lane of each group
    __syncwarp();
  }
}

// ---- one-block form (numel <= kAlignSmall).  `walkers` warps each own a contiguous segment of the ids (a
// multiple of 32 long): per-warp histograms, a scan over the warps per slot, then every warp places its own
// segment, so the order inside a slot still follows the flat index.
__global__ void __launch_bounds__(1024)
align_small_kernel(const void* __restrict__ ids, int is64, int64_t numel, int slots, int block_size, int walkers,
                   int32_t* __restrict__ sorted_token_ids, int64_t sorted_capacity, int32_t* __restrict__ expert_ids,
                   int64_t expert_ids_capacity, int32_t* __restrict__ num_tokens_post_pad, int32_t* __restrict__ cumsum,
                   int pad) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_cnt = s_mem;                  // [slots]
  int32_t* s_off = s_cnt + slots;          // [slots + 1]
  int32_t* s_ids = s_off + slots + 1;      // [kAlignSmall]
  int32_t* s_w = s_ids + kAlignSmall;      // [walkers][slots]
  const int n = static_cast<int>(numel);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = ((n + walkers - 1) / walkers + 31) / 32 * 32;
  for (int i = threadIdx.x; i < walkers * slots; i += blockDim.x) s_w[i] = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s_ids[i] = load_id(ids, is64, i);
  __syncthreads();
  const int seg_lo = min(warp * seg, n), seg_hi = min(seg_lo + seg, n);
  if (warp < walkers) {
    for (int i = seg_lo + lane; i < seg_hi; i += 32) {
      const int slot = s_ids[i] + 1;
      if (slot >= 0 && slot < slots) atomicAdd(&s_w[warp * slots + slot], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < slots; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < walkers; ++w) {
      const int v = s_w[w * slots + e];
      s_w[w * slots + e] = run;
      run += v;
    }
    s_cnt[e] = run;
  }
  __syncthreads();
  if (threadIdx.x < 32) padded_prefix_warp0(s_cnt, s_off, slots, block_size);
  __syncthreads();
  for (int e = threadIdx.x; e < slots; e += blockDim.x) {
    const int off = s_off[e];
    for (int w = 0; w < walkers; ++w) s_w[w * slots + e] += off;
  }
  write_tables(s_cnt, s_off, slots, block_size, numel, sorted_token_ids, sorted_capacity, expert_ids,
               expert_ids_capacity, num_tokens_post_pad, cumsum, pad);
  __syncthreads();
  if (warp < walkers) place_warp0(s_ids, seg_hi, 0, slots, s_w + warp * slots, sorted_token_ids, sorted_capacity, seg_lo);
}

// ---- three-launch form.  Phase 1: per-chunk histogram -> scratch[chunk][slots]
__global__ void __launch_bounds__(kAlignThreads)
align_count_kernel(const void* __restrict__ ids, int is64, int64_t numel, int slots, int32_t* __restrict__ scratch) {
  extern __shared__ int32_t s_mem[];
  for (int e = threadIdx.x; e < slots; e += kAlignThreads) s_mem[e] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kAlignChunk;
  for (int i = threadIdx.x; i < kAlignChunk; i += kAlignThreads) {
    const int64_t idx = base + i;
    if (idx < numel) {
      const int slot = load_id(ids, is64, idx) + 1;
      if (slot >= 0 && slot < slots) atomicAdd(&s_mem[slot], 1);
    }
  }
  __syncthreads();
  int32_t* out = scratch + static_cast<int64_t>(blockIdx.x) * slots;
  for (int e = threadIdx.x; e < slots; e += kAlignThreads) out[e] = s_mem[e];
}

// Phase 2 (one block): totals per slot, padded offsets, tables; scratch[chunk][slot] becomes the first position
// of the slot's ids that live in `chunk`.
__global__ void __launch_bounds__(1024)
align_scan_kernel(int32_t* __restrict__ scratch, int num_chunks, int64_t numel, int slots, int block_size,
                  int32_t* __restrict__ sorted_token_ids, int64_t sorted_capacity, int32_t* __restrict__ expert_ids,
                  int64_t expert_ids_capacity, int32_t* __restrict__ num_tokens_post_pad, int32_t* __restrict__ cumsum,
                  int pad) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_cnt = s_mem;
  int32_t* s_off = s_cnt + slots;
  for (int e = threadIdx.x; e < slots; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < num_chunks; ++c) {
      const int64_t at = static_cast<int64_t>(c) * slots + e;
      const int v = scratch[at];
      scratch[at] = run;
      run += v;
    }
    s_cnt[e] = run;
  }
  __syncthreads();
  if (threadIdx.x < 32) padded_prefix_warp0(s_cnt, s_off, slots, block_size);
  __syncthreads();
  for (int e = threadIdx.x; e < slots; e += blockDim.x) {
    const int off = s_off[e];
    for (int c = 0; c < num_chunks; ++c) scratch[static_cast<int64_t>(c) * slots + e] += off;
  }
  write_tables(s_cnt, s_off, slots, block_size, numel, sorted_token_ids, sorted_capacity, expert_ids,
               expert_ids_capacity, num_tokens_post_pad, cumsum, pad);
}

// Phase 3: stable placement inside each chunk.
__global__ void __launch_bounds__(kAlignThreads)
align_place_kernel(const void* __restrict__ ids, int is64, int64_t numel, int slots, const int32_t* __restrict__ scratch,
                   int32_t* __restrict__ sorted_token_ids, int64_t sorted_capacity) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_next = s_mem;             // [slots]
  int32_t* s_ids = s_mem + slots;      // [kAlignChunk]
  const int32_t* chunk_base = scratch + static_cast<int64_t>(blockIdx.x) * slots;
  for (int e = threadIdx.x; e < slots; e += kAlignThreads) s_next[e] = chunk_base[e];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kAlignChunk;
  const int64_t left = numel - base;
  const int count = left < kAlignChunk ? static_cast<int>(left) : kAlignChunk;
  for (int i = threadIdx.x; i < count; i += kAlignThreads) s_ids[i] = load_id(ids, is64, base + i);
  __syncthreads();
  if (threadIdx.x < 32) place_warp0(s_ids, count, base, slots, s_next, sorted_token_ids, sorted_capacity);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" size_t b200_moe_align_block_size_scratch_bytes(int64_t numel, int num_experts) {
  if (numel <= kAlignSmall) return 0;
  const int64_t chunks = (numel + kAlignChunk - 1) / kAlignChunk;
  return static_cast<size_t>(chunks) * static_cast<size_t>(num_experts) * sizeof(int32_t);
}

extern "C" int b200_moe_align_block_size(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts,
                                         int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                         int32_t* expert_ids, int64_t expert_ids_capacity,
                                         int32_t* num_tokens_post_pad, int32_t* cumsum_buffer,
                                         int pad_sorted_token_ids, void* scratch, size_t scratch_bytes, void* stream) {
  if (numel < 0 || num_experts <= 0 || block_size <= 0) return B200_ERR_BAD_SHAPE;
  if (num_experts > kMaxSlots) return B200_ERR_TOO_LARGE;   // shared-memory tables are sized by the slot count
  if (numel > 0 && !topk_ids) return B200_ERR_NULL_PTR;
  if (!sorted_token_ids || !expert_ids || !num_tokens_post_pad || !cumsum_buffer)
    return B200_ERR_NULL_PTR;
  // worst case the reference's callers size for: every slot padded by block_size - 1
  if (numel + static_cast<int64_t>(num_experts) * (block_size - 1) >= (int64_t{1} << 31))
    return B200_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (numel <= kAlignSmall) {
    // as many walking warps (<= 16) as 48 KB of shared memory holds histograms for
    const int room = 48 * 1024 / 4 - kAlignSmall - (2 * num_experts + 1);
    const int walkers = room / num_experts >= 16 ? 16 : (room / num_experts >= 1 ? room / num_experts : 1);
    const size_t smem = (static_cast<size_t>(2 * num_experts + 1) + kAlignSmall +
                         static_cast<size_t>(walkers) * num_experts) * sizeof(int32_t);
    align_small_kernel<<<1, 1024, smem, st>>>(topk_ids, ids_are_int64, numel, num_experts, block_size, walkers,
                                              sorted_token_ids,
                                              sorted_capacity, expert_ids, expert_ids_capacity, num_tokens_post_pad,
                                              cumsum_buffer, pad_sorted_token_ids);
    B200_CUDA_TRY(cudaGetLastError());
    return 0;
  }
  const int64_t chunks = (numel + kAlignChunk - 1) / kAlignChunk;
  const size_t need = static_cast<size_t>(chunks) * static_cast<size_t>(num_experts) * sizeof(int32_t);
  if (!scratch || scratch_bytes < need) return B200_ERR_NULL_PTR;
  int32_t* sc = static_cast<int32_t*>(scratch);
  align_count_kernel<<<static_cast<unsigned>(chunks), kAlignThreads, num_experts * sizeof(int32_t), st>>>(
      topk_ids, ids_are_int64, numel, num_experts, sc);
  align_scan_kernel<<<1, 1024, (2 * num_experts + 1) * sizeof(int32_t), st>>>(
      sc, static_cast<int>(chunks), numel, num_experts, block_size, sorted_token_ids, sorted_capacity, expert_ids,
      expert_ids_capacity, num_tokens_post_pad, cumsum_buffer, pad_sorted_token_ids);
  align_place_kernel<<<static_cast<unsigned>(chunks), kAlignThreads, (num_experts + kAlignChunk) * sizeof(int32_t), st>>>(
      topk_ids, ids_are_int64, numel, num_experts, sc, sorted_token_ids, sorted_capacity);
  B200_CUDA_TRY(cudaGetLastError());
  return 0;
}
