// Sum of bf16 / fp16 buffers across the GPUs of one NVSwitch domain, for the row-parallel linear's
// partial outputs.  Stands in for the reference's custom all-reduce
// (sgl-kernel/csrc/allreduce/custom_all_reduce.cuh: one-shot and two-shot kernels over IPC peer
// pointers) and for the NCCL all-reduce behind tensor_model_parallel_all_reduce
// (python/sglang/srt/distributed/communication_op.py:11-13).
//
// Every rank passes the same symmetric buffer (same size, same offset on every rank): its own
// address, the peers' addresses of it, and -- where the driver could bind the buffers to an NVLink
// multicast object -- the multicast address.  Two forms:
//   two-shot, in place   rank r owns the r-th slice.  With a multicast address it pulls the slice's sum
//                        out of the switch (multimem.ld_reduce: the switch reads the slice from every
//                        GPU and adds in fp32) and pushes the result to every GPU (multimem.st); without
//                        one it reads the slice from every peer, adds in fp32 in rank order, and stores
//                        the result into every peer's buffer.
//   one-shot, out of place  every rank sums the whole buffer into a local output; one pass and two
//                        barriers, for buffers of a few hundred kilobytes where latency is everything.
// Either way every element is the fp32 sum of all ranks' values rounded once -- the same bits on every
// rank, independent of timing.  (The peer-pointer forms round to nearest-even; the switch's own rounding of
// its fp32 sum differs from that by one unit in the last place now and then.)
//
// Ranks meet at flag barriers in the peers' signal pads (one 32-bit flag per block and peer,
// compare-and-swap 0 -> 1 by the sender, 1 -> 0 by the receiver, so the flags need no epoch).  Every
// spin is bounded; a rank whose peer never arrives records an error code in `status` (a device word of
// the caller) and carries on without waiting, so a missing rank costs wrong data, not a hung GPU.
// These kernels wait for kernels on OTHER GPUs: one process per GPU, never two ranks on one GPU.
#include "peer_sync.cuh"

namespace b200 {
namespace {

constexpr int kArThreads = 512;

struct ArParams {
  void* local;                   // this rank's buffer
  void* peers[kMaxRanks];        // every rank's buffer, as mapped into this process (peers[rank] == local)
  PeerSync sync;                 // signal pads, rank, world, first flag word, status word
  void* mc;                      // multicast address of the buffer, or null
  void* out;                     // one-shot: local output
  int64_t offset_bytes;          // of the reduced range inside the buffer (multiple of 16 * world)
  int64_t bytes;                 // length of the reduced range (multiple of 16 * world for two-shot, 16 for one-shot)
  int rank, world;
};

struct alignas(16) Vec16 { uint32_t w[4]; };

template <typename T> struct Pair2;
template <> struct Pair2<__nv_bfloat16> {
  __device__ static float2 unpack(uint32_t w) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w)); }
  __device__ static uint32_t pack(float2 f) { __nv_bfloat162 t = __float22bfloat162_rn(f); return *reinterpret_cast<uint32_t*>(&t); }
};
template <> struct Pair2<__half> {
  __device__ static float2 unpack(uint32_t w) { return __half22float2(*reinterpret_cast<__half2*>(&w)); }
  __device__ static uint32_t pack(float2 f) { __half2 t = __float22half2_rn(f); return *reinterpret_cast<uint32_t*>(&t); }
};

template <typename T>
__device__ __forceinline__ Vec16 multimem_ld_reduce(const void* mc_addr);
template <>
__device__ __forceinline__ Vec16 multimem_ld_reduce<__nv_bfloat16>(const void* mc_addr) {
  Vec16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc_addr) : "memory");
  return v;
}
template <>
__device__ __forceinline__ Vec16 multimem_ld_reduce<__half>(const void* mc_addr) {
  Vec16 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(void* mc_addr, const Vec16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_addr), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]) : "memory");
}

// Sum over ranks of one 16-byte vector read from every rank's buffer, fp32, rank order.
template <typename T>
__device__ __forceinline__ Vec16 peer_sum(const ArParams& p, int64_t byte_off) {
  float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
  Vec16 v[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.world) v[r] = *reinterpret_cast<const Vec16*>(static_cast<const char*>(p.peers[r]) + byte_off);
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r)
    if (r < p.world) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Pair2<T>::unpack(v[r].w[j]);
        acc[j].x += f.x;
        acc[j].y += f.y;
      }
    }
  Vec16 o;
#pragma unroll
  for (int j = 0; j < 4; ++j) o.w[j] = Pair2<T>::pack(acc[j]);
  return o;
}

// U 16-byte vectors of this rank's slice, summed over the ranks (through the switch or from every peer).
template <typename T, bool MULTIMEM, int U>
__device__ __forceinline__ void twoshot_load(const ArParams& p, int64_t base, int64_t i0, int64_t stride, int64_t nvec,
                                             Vec16 (&v)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = i0 + u * stride;
    if (i < nvec) {
      if constexpr (MULTIMEM) v[u] = multimem_ld_reduce<T>(static_cast<const char*>(p.mc) + base + i * 16);
      else v[u] = peer_sum<T>(p, base + i * 16);
    }
  }
}
// ... and stored to every rank.
template <bool MULTIMEM, int U>
__device__ __forceinline__ void twoshot_store(const ArParams& p, int64_t base, int64_t i0, int64_t stride, int64_t nvec,
                                              const Vec16 (&v)[U]) {
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t i = i0 + u * stride;
    if (i < nvec) {
      if constexpr (MULTIMEM) {
        multimem_st(static_cast<char*>(p.mc) + base + i * 16, v[u]);
      } else {
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
          if (r < p.world) *reinterpret_cast<Vec16*>(static_cast<char*>(p.peers[r]) + base + i * 16) = v[u];
      }
    }
  }
}

// The loads of a rank's slice travel one way over NVLink (every rank SENDS its contribution to the sums), the stores
// the other way (every rank RECEIVES every slice).  A loop that loads, waits and then stores uses the two directions
// in turn -- and all blocks of all ranks leave the opening barrier in step, so the whole machine alternates.  The
// loop is therefore software-pipelined: the loads of batch i+1 are issued before the stores of batch i, and both
// directions carry data at the same time.
template <typename T, bool MULTIMEM>
__global__ void __launch_bounds__(kArThreads) allreduce_twoshot_kernel(const ArParams p) {
  rank_barrier(p.sync, 21);   // every rank's partial values are in its buffer
  const int64_t slice = p.bytes / p.world;
  const int64_t base = p.offset_bytes + slice * p.rank;
  const int64_t nvec = slice / 16;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // 16-byte vectors per batch and thread; two batches are live at a time (the peer form holds one vector per rank
  // for each of them while it sums)
  constexpr int U = MULTIMEM ? 4 : 2;
  const int64_t step = stride * U;
  int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  Vec16 a[U], b[U];
  if (i0 < nvec) twoshot_load<T, MULTIMEM, U>(p, base, i0, stride, nvec, a);
  while (i0 < nvec) {
    if (i0 + step < nvec) twoshot_load<T, MULTIMEM, U>(p, base, i0 + step, stride, nvec, b);
    twoshot_store<MULTIMEM, U>(p, base, i0, stride, nvec, a);
    i0 += step;
    if (i0 >= nvec) break;
    if (i0 + step < nvec) twoshot_load<T, MULTIMEM, U>(p, base, i0 + step, stride, nvec, a);
    twoshot_store<MULTIMEM, U>(p, base, i0, stride, nvec, b);
    i0 += step;
  }
  __threadfence_system();
  rank_barrier(p.sync, 22);   // every slice has reached every rank
}

template <typename T, bool MULTIMEM>
__global__ void __launch_bounds__(kArThreads) allreduce_oneshot_kernel(const ArParams p) {
  rank_barrier(p.sync, 23);
  const int64_t nvec = p.bytes / 16;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    Vec16 v;
    if constexpr (MULTIMEM) v = multimem_ld_reduce<T>(static_cast<const char*>(p.mc) + p.offset_bytes + i * 16);
    else v = peer_sum<T>(p, p.offset_bytes + i * 16);
    *reinterpret_cast<Vec16*>(static_cast<char*>(p.out) + i * 16) = v;
  }
  rank_barrier(p.sync, 24);   // nobody overwrites its buffer while a peer still reads it
}

}  // namespace
}  // namespace b200

extern "C" int b200_allreduce_max_blocks(void) { return 148; }

extern "C" int b200_allreduce_flag_words(int world_size) { return 148 * world_size; }

extern "C" int b200_allreduce(void* const* peer_buffers, void* const* peer_signal_pads, void* multicast_buffer,
                              void* out, int* status, int64_t offset_bytes, int64_t bytes, int dtype, int rank,
                              int world_size, int one_shot, int num_blocks, int64_t flag_base_words, void* stream) {
  using namespace b200;
  if (!peer_buffers || !peer_signal_pads || !status) return B200_ERR_NULL_PTR;
  if (world_size < 2 || world_size > kMaxRanks || rank < 0 || rank >= world_size) return B200_ERR_BAD_SHAPE;
  if (dtype != B200_DT_BF16 && dtype != B200_DT_F16) return B200_ERR_BAD_DTYPE;
  if (bytes < 0 || offset_bytes < 0 || flag_base_words < 0) return B200_ERR_BAD_SHAPE;
  if (bytes == 0) return B200_OK;
  if (one_shot ? (bytes % 16 != 0) : (bytes % (16 * world_size) != 0)) return B200_ERR_BAD_SHAPE;
  if (offset_bytes % 16 != 0) return B200_ERR_MISALIGNED;
  if (one_shot && !out) return B200_ERR_NULL_PTR;
  // Default grid.  Measured at two ranks on 58.7 MB: the multicast form runs at the same speed with 8 and with 64
  // blocks (the switch sets the pace: 166-175 us), the peer-pointer form scales with the blocks (1037 / 563 / 297 /
  // 168 / 133 / 120 us with 8 / 16 / 32 / 64 / 96 / 128; NCCL 135 us): few blocks for the first, so that a GEMM
  // running beside it keeps its SMs, one per SM for the second.
  if (num_blocks <= 0) num_blocks = multicast_buffer ? 32 : b200_allreduce_max_blocks();
  if (num_blocks > b200_allreduce_max_blocks()) num_blocks = b200_allreduce_max_blocks();
  int rc = require_sm100();
  if (rc != B200_OK) return rc;
  ArParams p;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.peers[r] = r < world_size ? peer_buffers[r] : nullptr;
    if (r < world_size && !p.peers[r]) return B200_ERR_NULL_PTR;
    if (r < world_size && !aligned16(p.peers[r])) return B200_ERR_MISALIGNED;
  }
  rc = make_peer_sync(&p.sync, peer_signal_pads, rank, world_size, flag_base_words, status);
  if (rc != B200_OK) return rc;
  p.local = p.peers[rank];
  p.mc = multicast_buffer;
  p.out = out;
  p.offset_bytes = offset_bytes;
  p.bytes = bytes;
  p.rank = rank;
  p.world = world_size;
  // no more blocks than 16-byte vectors of work per rank
  const int64_t vecs = (one_shot ? bytes : bytes / world_size) / 16;
  const int64_t want = (vecs + kArThreads - 1) / kArThreads;
  if (want < num_blocks) num_blocks = static_cast<int>(want < 1 ? 1 : want);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool mm = multicast_buffer != nullptr;
#define B200_AR_LAUNCH(KERN, T)                                                       \
  do {                                                                                \
    if (mm) KERN<T, true><<<num_blocks, kArThreads, 0, st>>>(p);                      \
    else KERN<T, false><<<num_blocks, kArThreads, 0, st>>>(p);                        \
  } while (0)
  if (one_shot) {
    if (dtype == B200_DT_BF16) B200_AR_LAUNCH(allreduce_oneshot_kernel, __nv_bfloat16);
    else B200_AR_LAUNCH(allreduce_oneshot_kernel, __half);
  } else {
    if (dtype == B200_DT_BF16) B200_AR_LAUNCH(allreduce_twoshot_kernel, __nv_bfloat16);
    else B200_AR_LAUNCH(allreduce_twoshot_kernel, __half);
  }
#undef B200_AR_LAUNCH
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
