// Meeting points between the GPUs of one NVSwitch domain, shared by the kernels that exchange data over
// NVLink (all-reduce, expert-parallel dispatch / combine).  One process per GPU: a kernel that waits here
// waits for a kernel on ANOTHER GPU.
//
// Every rank owns a signal pad (zero-initialised 32-bit flags) that every other rank has mapped.  Flag
// [block][peer] of a rank's pad is set (compare-and-swap 0 -> 1, release) by that peer's block with the
// same index and cleared (1 -> 0, acquire) by the owner, so the flags need no epoch and a pad is reused
// call after call.  Every spin is bounded (about ten seconds): a rank whose peer never arrives records a code in its status
// word and carries on, so a missing rank costs wrong data, never a hung GPU.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kMaxRanks = 8;
// Ranks reach a meeting point at different times (one may still be loading a module or running a longer kernel),
// so the limit is generous: about ten seconds of SM clocks.
constexpr long long kPeerWaitCycles = 20000000000LL;

struct PeerSync {
  uint32_t* signals[kMaxRanks];  // every rank's signal pad, as mapped into this process
  int* status;                   // device word of this rank: 0, or the code of the first wait that gave up
  uint32_t flag_base;            // first flag word this call site uses inside the pads
  int rank, world;
};

inline int make_peer_sync(PeerSync* s, void* const* peer_signal_pads, int rank, int world, int64_t flag_base_words,
                          int* status) {
  if (!peer_signal_pads || !status) return B200_ERR_NULL_PTR;
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world || flag_base_words < 0) return B200_ERR_BAD_SHAPE;
  for (int r = 0; r < kMaxRanks; ++r) {
    s->signals[r] = r < world ? static_cast<uint32_t*>(peer_signal_pads[r]) : nullptr;
    if (r < world && !s->signals[r]) return B200_ERR_NULL_PTR;
  }
  s->status = status;
  s->flag_base = static_cast<uint32_t>(flag_base_words);
  s->rank = rank;
  s->world = world;
  return B200_OK;
}

#if defined(__CUDACC__)
__device__ __forceinline__ uint32_t cas_release_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.global.release.sys.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t cas_acquire_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  return old;
}

// All ranks' blocks with the same index meet.  Thread t < world of each block signals rank t's pad and
// waits for rank t's signal in its own pad.  Flags of block b: words [flag_base + b*world, +world).
__device__ __forceinline__ void rank_barrier(const PeerSync& p, int code) {
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    uint32_t* theirs = p.signals[peer] + p.flag_base + blockIdx.x * p.world + p.rank;
    uint32_t* mine = p.signals[p.rank] + p.flag_base + blockIdx.x * p.world + peer;
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
    if (!ok) atomicCAS(p.status, 0, code);
  }
  __syncthreads();
}


#endif  // __CUDACC__

}  // namespace b200
