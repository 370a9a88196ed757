// Shared helpers for the sm_100a kernels: error plumbing and thin PTX wrappers
// (mbarrier, TMA, tcgen05 / tensor memory).  Every device-side wait is bounded.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_block_fp8.h"

namespace b200 {

// ----------------------------------------------------------------------------- host side
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return B200_ERR_CUDA;
}

#define B200_CUDA_TRY(expr)                               \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return ::b200::cuda_fail(_e);  \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();
// 0 if the current device is compute capability 10.x, else B200_ERR_NOT_SM100 / B200_ERR_CUDA.
int require_sm100();

// ----------------------------------------------------------------------------- device side
#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// try_wait with an optional suspend-time hint (ns): with a hint a failed try may keep the thread
// suspended in hardware for up to that long; hint 0 uses the plain form.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns = 0) {
  uint32_t ok;
  if (hint_ns == 1) {
    // non-blocking form: returns at once whether or not the phase has completed
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  } else if (hint_ns != 0) {
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred P;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
  }
  return ok != 0;
}

// Status words of the GEMM kernels: one 4 KB-aligned ring of ints per device.  Word 0 is the device's
// sticky error code, words 2..3 hold the device address of its mirror in pinned host memory, words
// kStatusFirstSlot.. are per-launch slots (a launch watches only its own slot, so a code left by an
// earlier launch cannot make a healthy kernel abandon its waits).
constexpr int kStatusRingInts = 1024;
constexpr int kStatusFirstSlot = 8;

// Records that a wait of this launch gave up: the launch's slot (read by the launch's other waiters),
// the device's sticky word and its host mirror (read by the host without a synchronisation).
__device__ __forceinline__ void report_wait_failure(int* slot, int code) {
  atomicCAS(slot, 0, code);
  int* ring = reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(slot) & ~uintptr_t(kStatusRingInts * 4 - 1));
  if (atomicCAS(ring, 0, code) == 0) {
    int* host = *reinterpret_cast<int* volatile*>(ring + 2);
    if (host != nullptr) {
      *reinterpret_cast<volatile int*>(host) = code;
      __threadfence_system();
    }
  }
}

// Bounded wait: gives up after ~kWaitLimitCycles SM clocks (about a second), records `code`
// (first failure wins) and returns false.  `status` is the launch's slot of the status ring.
// Callers leave their loops on false.
constexpr long long kWaitLimitCycles = 2000000000LL;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          uint32_t hint_ns = 0) {
  if (mbar_try_wait(bar, parity, hint_ns)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity, hint_ns)) {
    if ((++spins & 0xffu) == 0) {
      if (*reinterpret_cast<volatile int*>(status) != 0) return false;  // another wait of this launch gave up
      if (clock64() - t0 > kWaitLimitCycles) {
        report_wait_failure(status, code);
        return false;
      }
    }
  }
  return true;
}

// The same wait for a whole converged warp: lane 0 polls and the outcome is broadcast, so that all
// lanes leave their loop together when a wait gives up.  (32 lanes polling one mbarrier are 32
// operations on one shared-memory word; with several warps spinning, that traffic alone cost hundreds
// of cycles per wait.)  The shuffle orders the other lanes' later accesses after lane 0's acquire.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int code,
                                               uint32_t hint_ns = 0) {
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, status, code, hint_ns);
  return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}

// ---- TMA (tiled bulk tensor copy global -> shared, completion on an mbarrier; no multicast)
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory / tcgen05 (cta_group::1)
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], e4m3 x e4m3 -> fp32, one thread issues.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All previously issued MMAs of this thread arrive on `bar` when complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x (8 * X) consecutive fp32 columns in the accumulator-fragment layout: for column group g
// (8 columns) thread t gets v[4g + 0..1] = lane (base_lane + t/4), columns 8g + 2(t%4) + 0..1 and
// v[4g + 2..3] = lane (base_lane + 8 + t/4), same columns.  base_lane is a multiple of 16 inside the
// warp's own lane quadrant.
template <int X>
__device__ __forceinline__ void tmem_ld_16x256b(uint32_t taddr, float* v);
template <>
__device__ __forceinline__ void tmem_ld_16x256b<2>(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_16x256b<4>(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_16x256b<8>(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- thread-block cluster / CTA-pair (cta_group::2) forms
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {  // every thread of every CTA in the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the same-named mbarrier in CTA `cta` of the cluster.  Default (.release.cta) semantics on
// purpose: a cluster-scope release makes the warp wait for all its outstanding global loads
// (measured as the dominant "membar" stall), and the only thing ordered here is tensor-memory
// reads, which tcgen05.wait::ld + fence::before_thread_sync already cover.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [remote];\n\t}\n"
      ::"r"(smem_u32(bar)), "r"(cta)
      : "memory");
}
// In the shared::cluster window bit 24 of a CTA-pair member's shared address selects the odd CTA;
// clearing it addresses the same offset in the even (leader) CTA.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
// Tiled load issued by either CTA of a pair into its OWN shared memory; the transaction bytes are
// credited to the LEADER CTA's mbarrier.  No multicast: each CTA fetches its own box.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {  // one warp in EACH CTA
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// One thread of the leader CTA issues; both SMs of the pair execute (M = 256 split 128 + 128).
__device__ __forceinline__ void umma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Completion of the pair's MMAs arrives on the same-offset mbarrier in every CTA of `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}

// One k-block of pair MMAs (four K=32 steps, fresh accumulator) plus its completion commit, issued
// by the elected lane, bracketed by the barrier tests for the NEXT k-block: the two try_waits are
// started first and their results are only read after the MMAs have been issued, so their latency
// overlaps the issue instead of preceding it.  All lanes execute the tests (warp-uniform flow).
__device__ __forceinline__ void umma_f8_pair_kblock_with_peek(
    uint32_t elected, uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint64_t* done_bar,
    uint16_t cta_mask, uint64_t* next_acc_bar, uint32_t next_acc_parity, uint64_t* next_full_bar,
    uint32_t next_full_parity, uint32_t& acc_ready, uint32_t& ops_ready) {
  asm volatile(
      "{\n\t"
      ".reg .pred PE, PA, PF, PT, PZ;\n\t"
      ".reg .b64 ad, bd;\n\t"
      "setp.ne.b32 PE, %2, 0;\n\t"
      "setp.eq.b32 PT, 0, 0;\n\t"
      "setp.ne.b32 PZ, 0, 0;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 PA, [%9], %10;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 PF, [%11], %12;\n\t"
      "@PE tcgen05.mma.cta_group::2.kind::f8f6f4 [%3], %4, %5, %6, PZ;\n\t"
      "add.s64 ad, %4, 2;\n\t"
      "add.s64 bd, %5, 2;\n\t"
      "@PE tcgen05.mma.cta_group::2.kind::f8f6f4 [%3], ad, bd, %6, PT;\n\t"
      "add.s64 ad, %4, 4;\n\t"
      "add.s64 bd, %5, 4;\n\t"
      "@PE tcgen05.mma.cta_group::2.kind::f8f6f4 [%3], ad, bd, %6, PT;\n\t"
      "add.s64 ad, %4, 6;\n\t"
      "add.s64 bd, %5, 6;\n\t"
      "@PE tcgen05.mma.cta_group::2.kind::f8f6f4 [%3], ad, bd, %6, PT;\n\t"
      "@PE tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%7], %8;\n\t"
      "selp.b32 %0, 1, 0, PA;\n\t"
      "selp.b32 %1, 1, 0, PF;\n\t"
      "}\n"
      : "=r"(acc_ready), "=r"(ops_ready)
      : "r"(elected), "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(smem_u32(done_bar)), "h"(cta_mask),
        "r"(smem_u32(next_acc_bar)), "r"(next_acc_parity), "r"(smem_u32(next_full_bar)), "r"(next_full_parity)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 128 bytes x R rows with SWIZZLE_128B produces):
// start address >> 4 in bits [0,14); leading byte offset (unused for swizzled K-major) = 1 in
// [16,30); stride byte offset = 1024 B (8 rows x 128 B) >> 4 in [32,46); descriptor version 1 in
// [46,48); layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f8f6f4, A = B = e4m3 (format 0), both K-major, fp32 accumulate:
// c_format = 1 at [4,6); a_format at [7,10); b_format at [10,13); N>>3 at [17,23); M>>4 at [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

#endif  // __CUDACC__

}  // namespace b200
