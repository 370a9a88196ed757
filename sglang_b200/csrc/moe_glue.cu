// MoE glue kernels around the grouped block-FP8 GEMM: routing tables, row gather, SiLU*mul,
// weighted un-permute sum.  All HBM-bound integer/byte work: 128-bit coalesced accesses, no
// tensor cores.
//
// Stand in for (paths in the reference checkout):
//   prepare_moe_input      sgl-kernel/csrc/moe/prepare_moe_input.cu:13-167
//   shuffle_rows           sgl-kernel/csrc/moe/prepare_moe_input.cu:169-256
//   apply_shuffle_mul_sum  sgl-kernel/csrc/moe/prepare_moe_input.cu:258-392
//   silu_and_mul           sgl-kernel/csrc/elementwise/activation.cu (used at
//                          python/sglang/srt/layers/moe/cutlass_moe.py:191-192)
//
// prepare: the reference hands out slots inside an expert with atomics, so its order inside an
// expert changes from run to run; here the order is the ascending flat index of topk_ids
// (a stable counting sort), one of the orders the reference can produce, and reproducible.
// It runs as three launches over chunks of the flat id list and needs a scratch table of
// per-chunk, per-expert counts in global memory.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kPrepThreads = 256;
constexpr int kPrepChunk = 2048;   // ids per chunk

// ---- phase 1: per-chunk histogram -> scratch[chunk][E]
__global__ void __launch_bounds__(kPrepThreads)
prep_count_kernel(const int32_t* __restrict__ topk_ids, int64_t n_ids, int num_experts, int32_t* __restrict__ scratch) {
  extern __shared__ int32_t s_cnt[];
  for (int e = threadIdx.x; e < num_experts; e += kPrepThreads) s_cnt[e] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kPrepChunk;
  for (int i = threadIdx.x; i < kPrepChunk; i += kPrepThreads) {
    const int64_t idx = base + i;
    if (idx < n_ids) {
      const int e = topk_ids[idx];
      if (e >= 0 && e < num_experts) atomicAdd(&s_cnt[e], 1);   // integer adds commute: deterministic totals
    }
  }
  __syncthreads();
  int32_t* out = scratch + static_cast<int64_t>(blockIdx.x) * num_experts;
  for (int e = threadIdx.x; e < num_experts; e += kPrepThreads) out[e] = s_cnt[e];
}

// ---- phase 2 (one block): per expert, exclusive scan over chunks; expert totals -> offsets, sizes.
// After it, scratch[chunk][e] = first slot (global) of expert e's ids that live in `chunk`.
__global__ void __launch_bounds__(1024)
prep_scan_kernel(int32_t* __restrict__ scratch, int num_chunks, int num_experts, int32_t* __restrict__ expert_offsets,
                 int32_t* __restrict__ blockscale_offsets, int32_t* __restrict__ problem_sizes1,
                 int32_t* __restrict__ problem_sizes2, int n, int k) {
  extern __shared__ int32_t s_tot[];   // [num_experts] totals, then exclusive offsets
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < num_chunks; ++c) {
      const int v = scratch[static_cast<int64_t>(c) * num_experts + e];
      scratch[static_cast<int64_t>(c) * num_experts + e] = run;   // offset inside the expert for now
      run += v;
    }
    s_tot[e] = run;
    problem_sizes1[e * 3 + 0] = run;
    problem_sizes1[e * 3 + 1] = 2 * n;
    problem_sizes1[e * 3 + 2] = k;
    problem_sizes2[e * 3 + 0] = run;
    problem_sizes2[e * 3 + 1] = k;
    problem_sizes2[e * 3 + 2] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {   // E is a few hundred at most: a serial prefix is a few microseconds
    int run = 0, run_rounded = 0;
    expert_offsets[0] = 0;
    if (blockscale_offsets) blockscale_offsets[0] = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int c = s_tot[e];
      s_tot[e] = run;
      run += c;
      run_rounded += (c + 127) / 128 * 128;
      expert_offsets[e + 1] = run;
      if (blockscale_offsets) blockscale_offsets[e + 1] = run_rounded;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int off = s_tot[e];
    for (int c = 0; c < num_chunks; ++c) scratch[static_cast<int64_t>(c) * num_experts + e] += off;
  }
}

// ---- phase 3: stable slot assignment inside each chunk.
__global__ void __launch_bounds__(kPrepThreads)
prep_scatter_kernel(const int32_t* __restrict__ topk_ids, int64_t n_ids, int topk, int num_experts,
                    const int32_t* __restrict__ scratch, int32_t* __restrict__ input_permutation,
                    int32_t* __restrict__ output_permutation, int walk_warps) {
  extern __shared__ int32_t s_mem[];
  int32_t* s_ids = s_mem;                          // [kPrepChunk]
  int32_t* s_wnext = s_mem + kPrepChunk;           // [walk_warps][E] next free slot of each expert for each walking warp
  const int kWarps = walk_warps;                   // 1, 2, 4 or 8 (as many as the per-warp tables leave room for)
  const int kSeg = kPrepChunk / kWarps;            // ids per warp: contiguous, so the order stays the flat index
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* chunk_base = scratch + static_cast<int64_t>(blockIdx.x) * num_experts;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kPrepChunk;
  const int64_t left = n_ids - base;
  const int n_here = left < kPrepChunk ? static_cast<int>(left < 0 ? 0 : left) : kPrepChunk;
  for (int i = threadIdx.x; i < kWarps * num_experts; i += kPrepThreads) s_wnext[i] = 0;
  for (int i = threadIdx.x; i < kPrepChunk; i += kPrepThreads) s_ids[i] = i < n_here ? topk_ids[base + i] : -1;
  __syncthreads();
  // per-warp histograms of the warps' segments
  if (warp < kWarps) {
    for (int i = lane; i < kSeg; i += 32) {
      const int e = s_ids[warp * kSeg + i];
      if (e >= 0 && e < num_experts) atomicAdd(&s_wnext[warp * num_experts + e], 1);
    }
  }
  __syncthreads();
  // per expert: exclusive scan over the warps on top of the chunk's first slot
  for (int e = threadIdx.x; e < num_experts; e += kPrepThreads) {
    int run = chunk_base[e];
    for (int w = 0; w < kWarps; ++w) {
      const int c = s_wnext[w * num_experts + e];
      s_wnext[w * num_experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  // Every warp walks its own segment in order, 32 ids at a time; equal experts inside the 32 are ranked with a
  // match mask, so slots follow the ascending flat index exactly.  (One warp walking the whole chunk took 17 us
  // even for a few dozen ids: a match step costs ~650 cycles, so the depth of the walk is what matters.)
  if (warp >= kWarps) return;
  int32_t* my_next = s_wnext + warp * num_experts;
  const int seg_end = min(kSeg, n_here - warp * kSeg);
  for (int i0 = 0; i0 < seg_end; i0 += 32) {
    const int i = warp * kSeg + i0 + lane;
    const int64_t idx = base + i;
    const int e = s_ids[i];
    const bool valid = e >= 0 && e < num_experts;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
    if (valid) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int slot = my_next[e] + rank;
      input_permutation[slot] = static_cast<int32_t>(idx / topk);
      output_permutation[idx] = slot;
    } else if (idx < n_ids) {
      output_permutation[idx] = -1;   // no slot: masked expert (the weighted sum skips it)
    }
    __syncwarp();
    if (valid && (peers >> lane) <= 1u) my_next[e] += __popc(peers);   // highest lane of each group
    __syncwarp();
  }
}

// ---- row gather: out[d] = in[map[d]], rows of row_bytes bytes (multiple of 16)
template <typename V>
__global__ void __launch_bounds__(256)
rows_gather_kernel(const V* __restrict__ in, const int32_t* __restrict__ map, V* __restrict__ out,
                   int64_t num_dst_rows, int vec_per_row) {
  const int rows_per_block = 256 / 32;   // one warp per row
  const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_block + (threadIdx.x >> 5);
  if (row >= num_dst_rows) return;
  const int64_t src = map[row];
  const V* s = in + src * vec_per_row;
  V* d = out + row * vec_per_row;
  for (int v = threadIdx.x & 31; v < vec_per_row; v += 32) d[v] = __ldg(s + v);
}

template <typename T>
struct Pack8;   // 8 elements of T in one uint4
template <>
struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <>
struct Pack8<__half> {
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
};

// ---- out[r, :d] = silu(x[r, :d]) * x[r, d:2d], fp32 math, one rounding
template <typename T>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int d) {
  const int vec_per_row = d / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * 256) {
    const int64_t r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(x + r * 2 * d) + v);
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(x + r * 2 * d + d) + v);
    float fg[8], fu[8], fo[8];
    Pack8<T>::unpack(g, fg);
    Pack8<T>::unpack(u, fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) fo[k] = (fg[k] / (1.0f + __expf(-fg[k]))) * fu[k];
    reinterpret_cast<uint4*>(out + r * d)[v] = Pack8<T>::pack(fo);
  }
}

// ---- out[i] = sum_j factors[i*topk+j] * in[perm[i*topk+j]], j ascending, fp32 accumulate
template <typename T>
__global__ void __launch_bounds__(256)
unpermute_sum_kernel(const T* __restrict__ in, T* __restrict__ out, const int32_t* __restrict__ perm,
                     const T* __restrict__ factors, int m, int topk, int row_len) {
  const int i = blockIdx.x;
  if (i >= m) return;
  const int vec_per_row = row_len / 8;
  for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int j = 0; j < topk; ++j) {
      const int src = perm[i * topk + j];
      if (src < 0) continue;   // masked expert (expert parallel): contributes nothing
      const float w = factors ? Pack8<T>::to_float(factors[i * topk + j]) : 1.0f;
      float f[8];
      Pack8<T>::unpack(__ldg(reinterpret_cast<const uint4*>(in + static_cast<int64_t>(src) * row_len) + v), f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += w * f[k];   // contracted to an fma by nvcc, as the reference's `sum += factor * val` is
    }
    reinterpret_cast<uint4*>(out + static_cast<int64_t>(i) * row_len)[v] = Pack8<T>::pack(acc);
  }
}

}  // namespace

size_t moe_prepare_scratch_bytes(int64_t n_ids, int num_experts) {
  const int64_t chunks = (n_ids + kPrepChunk - 1) / kPrepChunk;
  return static_cast<size_t>(chunks < 1 ? 1 : chunks) * num_experts * sizeof(int32_t);
}

int moe_prepare_launch(const int32_t* topk_ids, int64_t n_ids, int topk, int num_experts, int n, int k,
                       int32_t* expert_offsets, int32_t* blockscale_offsets, int32_t* problem_sizes1,
                       int32_t* problem_sizes2, int32_t* input_permutation, int32_t* output_permutation,
                       int32_t* scratch, cudaStream_t st) {
  const int chunks = static_cast<int>((n_ids + kPrepChunk - 1) / kPrepChunk);
  const int nch = chunks < 1 ? 1 : chunks;
  prep_count_kernel<<<nch, kPrepThreads, num_experts * sizeof(int32_t), st>>>(topk_ids, n_ids, num_experts, scratch);
  prep_scan_kernel<<<1, 1024, num_experts * sizeof(int32_t), st>>>(scratch, nch, num_experts, expert_offsets,
                                                                   blockscale_offsets, problem_sizes1,
                                                                   problem_sizes2, n, k);
  // walking warps: as many (a power of two up to 8) as fit their per-expert tables into 48 KB of shared memory
  int walk_warps = 8;
  while (walk_warps > 1 && (static_cast<size_t>(walk_warps) * num_experts + kPrepChunk) * sizeof(int32_t) > 48 * 1024)
    walk_warps >>= 1;
  prep_scatter_kernel<<<nch, kPrepThreads, (static_cast<size_t>(walk_warps) * num_experts + kPrepChunk) * sizeof(int32_t), st>>>(
      topk_ids, n_ids, topk, num_experts, scratch, input_permutation, output_permutation, walk_warps);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

extern "C" size_t b200_moe_prepare_scratch_bytes(int64_t num_ids, int num_experts) {
  if (num_ids < 0 || num_experts <= 0) return 0;
  return b200::moe_prepare_scratch_bytes(num_ids, num_experts);
}

extern "C" int b200_moe_prepare(const int32_t* topk_ids, int64_t num_tokens, int topk, int num_experts, int n, int k,
                                int32_t* expert_offsets, int32_t* blockscale_offsets, int32_t* problem_sizes1,
                                int32_t* problem_sizes2, int32_t* input_permutation, int32_t* output_permutation,
                                void* scratch, size_t scratch_bytes, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || topk <= 0 || num_experts <= 0 || n < 0 || k < 0) return B200_ERR_BAD_SHAPE;
  if (num_experts > 8192) return B200_ERR_TOO_LARGE;   // shared-memory tables are sized by the expert count
  if (!expert_offsets || !problem_sizes1 || !problem_sizes2) return B200_ERR_NULL_PTR;
  const int64_t n_ids = num_tokens * topk;
  if (n_ids > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  if (n_ids > 0 && (!topk_ids || !input_permutation || !output_permutation)) return B200_ERR_NULL_PTR;
  if (!scratch || scratch_bytes < moe_prepare_scratch_bytes(n_ids, num_experts)) return B200_ERR_NULL_PTR;
  return moe_prepare_launch(topk_ids, n_ids, topk, num_experts, n, k, expert_offsets, blockscale_offsets,
                            problem_sizes1, problem_sizes2, input_permutation, output_permutation,
                            static_cast<int32_t*>(scratch), static_cast<cudaStream_t>(stream));
}

// ---- routing tables without any allocation by anyone
//
// Some callers may not allocate device memory at the point where they build the routing tables: a
// serving process that has handed every free byte of the GPU to its KV-cache pool has nothing left
// for cudaMalloc to give, and a latency-critical section may forbid allocator calls (they can
// synchronise the device) altogether.  For them the chunk-count table lives in a fixed array inside this library
// instead of in caller-provided scratch.  The array costs kStaticScratchInts * 4 bytes on every GPU
// that loads the library, for the life of the process.
constexpr int kStaticScratchInts = 65536;   // 256 KiB: chunks * experts, e.g. 131072 ids x 1024 experts
static __device__ __align__(256) int32_t g_prepare_scratch[kStaticScratchInts];

namespace b200 {
namespace {
// Device address of g_prepare_scratch on the current device.  In host code the array's name is only
// a handle for the runtime, never an address a kernel could use, so the address is asked for once
// per device (with that device current) and cached.
int static_scratch_ptr(int32_t** out) {
  static int32_t* ptrs[64] = {nullptr};
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200_ERR_UNSUPPORTED;
  if (!ptrs[dev]) {
    int32_t* ptr = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_prepare_scratch));
    ptrs[dev] = ptr;
  }
  *out = ptrs[dev];
  return B200_OK;
}
}  // namespace
}  // namespace b200

extern "C" int b200_moe_prepare_noalloc(const int32_t* topk_ids, int64_t num_tokens, int topk, int num_experts,
                                        int n, int k, int32_t* expert_offsets, int32_t* blockscale_offsets,
                                        int32_t* problem_sizes1, int32_t* problem_sizes2,
                                        int32_t* input_permutation, int32_t* output_permutation, void* stream) {
  using namespace b200;
  if (num_tokens < 0 || topk <= 0 || num_experts <= 0 || n < 0 || k < 0) return B200_ERR_BAD_SHAPE;
  if (num_experts > 8192) return B200_ERR_TOO_LARGE;
  if (!expert_offsets || !problem_sizes1 || !problem_sizes2) return B200_ERR_NULL_PTR;
  const int64_t n_ids = num_tokens * topk;
  if (n_ids > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  if (n_ids > 0 && (!topk_ids || !input_permutation || !output_permutation)) return B200_ERR_NULL_PTR;
  // the table needs one int per (chunk of 2048 ids, expert); beyond the built-in array: refuse
  if (moe_prepare_scratch_bytes(n_ids, num_experts) > sizeof(int32_t) * kStaticScratchInts) return B200_ERR_TOO_LARGE;
  int32_t* scratch = nullptr;
  const int rc = static_scratch_ptr(&scratch);
  if (rc != B200_OK) return rc;
  // Nothing in the table has to start at zero: the counting launch overwrites every entry that the
  // later launches read, so whatever an earlier call left behind is harmless.
  return moe_prepare_launch(topk_ids, n_ids, topk, num_experts, n, k, expert_offsets, blockscale_offsets,
                            problem_sizes1, problem_sizes2, input_permutation, output_permutation, scratch,
                            static_cast<cudaStream_t>(stream));
}

namespace b200 {
namespace {
// Column gather of a [words][rows] table: dst[w][r] = src[w][clamp(map[r])].  The packed power-of-two scales are
// stored with the rows contiguous, so copying a token's scale words to the rows of its experts is a gather along
// the contiguous dimension: coalesced stores, reads from a table that sits in L2.
__global__ void __launch_bounds__(256) packed_scales_gather_kernel(const uint32_t* __restrict__ src, int64_t src_ld,
                                                                    int64_t src_rows, const int32_t* __restrict__ map,
                                                                    uint32_t* __restrict__ dst, int64_t dst_ld,
                                                                    int64_t num_dst_rows) {
  const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= num_dst_rows) return;
  const int64_t c = min(max(static_cast<int64_t>(__ldg(map + r)), int64_t(0)), src_rows - 1);
  dst[blockIdx.y * dst_ld + r] = __ldg(src + blockIdx.y * src_ld + c);
}
}  // namespace
}  // namespace b200

extern "C" int b200_shuffle_packed_scales(const uint32_t* input, int64_t input_stride_pack, int64_t num_src_rows,
                                          const int32_t* dst2src_map, uint32_t* output, int64_t output_stride_pack,
                                          int64_t num_dst_rows, int words_per_row, void* stream) {
  using namespace b200;
  if (num_dst_rows < 0 || num_src_rows < 0 || words_per_row < 0) return B200_ERR_BAD_SHAPE;
  if (num_dst_rows == 0 || words_per_row == 0) return B200_OK;
  if (num_src_rows == 0) return B200_ERR_BAD_SHAPE;
  if (!input || !dst2src_map || !output) return B200_ERR_NULL_PTR;
  if (input_stride_pack < num_src_rows || output_stride_pack < num_dst_rows) return B200_ERR_BAD_STRIDE;
  const int64_t blocks = (num_dst_rows + 255) / 256;
  if (blocks > 0x7fffffffLL || words_per_row > 65535) return B200_ERR_TOO_LARGE;
  packed_scales_gather_kernel<<<dim3(static_cast<unsigned>(blocks), static_cast<unsigned>(words_per_row)), 256, 0,
                                static_cast<cudaStream_t>(stream)>>>(input, input_stride_pack, num_src_rows, dst2src_map,
                                                                     output, output_stride_pack, num_dst_rows);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_shuffle_rows(const void* input, const int32_t* dst2src_map, void* output, int64_t num_dst_rows,
                                 int64_t row_bytes, void* stream) {
  using namespace b200;
  if (num_dst_rows < 0 || row_bytes < 0) return B200_ERR_BAD_SHAPE;
  if (num_dst_rows == 0 || row_bytes == 0) return B200_OK;
  if (!input || !dst2src_map || !output) return B200_ERR_NULL_PTR;
  const int64_t blocks = (num_dst_rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  // widest vector that divides the row and both base addresses: 16 bytes for the shapes of the
  // hot path (rows of K codes or K/128 scales with K % 512 == 0), narrower ones otherwise
  const uintptr_t bits = static_cast<uintptr_t>(row_bytes) | reinterpret_cast<uintptr_t>(input) |
                         reinterpret_cast<uintptr_t>(output);
  const unsigned grid = static_cast<unsigned>(blocks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((bits & 15u) == 0) {
    rows_gather_kernel<uint4><<<grid, 256, 0, st>>>(static_cast<const uint4*>(input), dst2src_map,
                                                    static_cast<uint4*>(output), num_dst_rows,
                                                    static_cast<int>(row_bytes / 16));
  } else if ((bits & 7u) == 0) {
    rows_gather_kernel<uint2><<<grid, 256, 0, st>>>(static_cast<const uint2*>(input), dst2src_map,
                                                    static_cast<uint2*>(output), num_dst_rows,
                                                    static_cast<int>(row_bytes / 8));
  } else if ((bits & 3u) == 0) {
    rows_gather_kernel<uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(input), dst2src_map,
                                                       static_cast<uint32_t*>(output), num_dst_rows,
                                                       static_cast<int>(row_bytes / 4));
  } else {
    rows_gather_kernel<uint8_t><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(input), dst2src_map,
                                                      static_cast<uint8_t*>(output), num_dst_rows,
                                                      static_cast<int>(row_bytes));
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_silu_and_mul(const void* x, void* out, int64_t rows, int64_t d, int dtype, void* stream) {
  using namespace b200;
  if (rows < 0 || d < 0) return B200_ERR_BAD_SHAPE;
  if (rows == 0 || d == 0) return B200_OK;
  if (!x || !out) return B200_ERR_NULL_PTR;
  if ((d % 8) != 0 || !aligned16(x) || !aligned16(out)) return B200_ERR_MISALIGNED;
  const int64_t total = rows * (d / 8);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == B200_DT_BF16) {
    silu_and_mul_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), rows, static_cast<int>(d));
  } else if (dtype == B200_DT_F16) {
    silu_and_mul_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const __half*>(x), static_cast<__half*>(out), rows, static_cast<int>(d));
  } else {
    return B200_ERR_BAD_DTYPE;
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_apply_shuffle_mul_sum(const void* input, void* output, const int32_t* permutation,
                                          const void* factors, int64_t m, int64_t topk, int64_t row_len, int dtype,
                                          void* stream) {
  using namespace b200;
  if (m < 0 || topk <= 0 || row_len < 0) return B200_ERR_BAD_SHAPE;
  if (m == 0 || row_len == 0) return B200_OK;
  if (!input || !output || !permutation) return B200_ERR_NULL_PTR;
  if ((row_len % 8) != 0 || !aligned16(input) || !aligned16(output)) return B200_ERR_MISALIGNED;
  if (m > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int threads = static_cast<int>(row_len / 8);
  threads = threads > 256 ? 256 : (threads < 32 ? 32 : (threads + 31) / 32 * 32);
  if (dtype == B200_DT_BF16) {
    unpermute_sum_kernel<__nv_bfloat16><<<static_cast<unsigned>(m), threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(input), static_cast<__nv_bfloat16*>(output), permutation,
        static_cast<const __nv_bfloat16*>(factors), static_cast<int>(m), static_cast<int>(topk),
        static_cast<int>(row_len));
  } else if (dtype == B200_DT_F16) {
    unpermute_sum_kernel<__half><<<static_cast<unsigned>(m), threads, 0, st>>>(
        static_cast<const __half*>(input), static_cast<__half*>(output), permutation,
        static_cast<const __half*>(factors), static_cast<int>(m), static_cast<int>(topk), static_cast<int>(row_len));
  } else {
    return B200_ERR_BAD_DTYPE;
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Router: softmax over the experts, then the top-k probabilities and their expert ids
// (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:502-570; torch form: softmax(logits.float()) -> topk,
// python/sglang/srt/layers/moe/topk.py:284-302).  One warp per token, up to 32 experts per lane in registers;
// ties go to the lower expert id.  With `renormalize` the k weights are divided by their sum.
namespace b200 {
namespace {

constexpr int kRouterMaxPerLane = 32;   // experts <= 1024

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, int PER_LANE>
__global__ void __launch_bounds__(128) topk_softmax_kernel(const T* __restrict__ logits, float* __restrict__ weights,
                                                           int32_t* __restrict__ ids, int64_t num_tokens,
                                                           int num_experts, int topk, int64_t logits_stride,
                                                           int renormalize) {
  const int lane = threadIdx.x & 31;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= num_tokens) return;
  const T* row = logits + token * logits_stride;
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < num_experts ? to_f32<T>(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const bool real = (i * 32 + lane) < num_experts;
    v[i] = real ? expf(v[i] - mx) : -1.f;   // padding can never be picked
    sum += real ? v[i] : 0.f;
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  const float inv = 1.0f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;      // lane j keeps the j-th pick (topk <= 32)
  int my_id = 0;
  for (int j = 0; j < topk; ++j) {
    // lane-local best (value descending, expert id ascending), then the warp's best
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > best) { best = v[i]; best_e = e; }   // equal values keep the earlier (lower) id
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) v[i] = -1.f;   // taken
    }
    const float w = best * inv;
    picked_sum += w;
    if (lane == j) { my_w = w; my_id = best_e; }
  }
  if (lane < topk) {
    weights[token * topk + lane] = renormalize ? my_w / picked_sum : my_w;
    ids[token * topk + lane] = my_id;
  }
}

template <typename T>
int launch_router(const void* logits, float* weights, int32_t* ids, int64_t num_tokens, int num_experts, int topk,
                  int64_t stride, int renormalize, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>((num_tokens + 3) / 4);
  const T* lp = static_cast<const T*>(logits);
  const int per_lane = (num_experts + 31) / 32;
  if (per_lane <= 2) topk_softmax_kernel<T, 2><<<blocks, 128, 0, st>>>(lp, weights, ids, num_tokens, num_experts, topk, stride, renormalize);
  else if (per_lane <= 8) topk_softmax_kernel<T, 8><<<blocks, 128, 0, st>>>(lp, weights, ids, num_tokens, num_experts, topk, stride, renormalize);
  else topk_softmax_kernel<T, kRouterMaxPerLane><<<blocks, 128, 0, st>>>(lp, weights, ids, num_tokens, num_experts, topk, stride, renormalize);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" int b200_topk_softmax(const void* gating_output, int dtype, int64_t row_stride, float* topk_weights,
                                 int32_t* topk_ids, int64_t num_tokens, int num_experts, int topk, int renormalize,
                                 void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_experts <= 0 || topk <= 0) return B200_ERR_BAD_SHAPE;
  if (topk > num_experts || topk > 32) return B200_ERR_BAD_SHAPE;
  if (num_experts > 32 * kRouterMaxPerLane) return B200_ERR_TOO_LARGE;
  if (num_tokens == 0) return B200_OK;
  if (!gating_output || !topk_weights || !topk_ids) return B200_ERR_NULL_PTR;
  if (row_stride < num_experts) return B200_ERR_BAD_STRIDE;
  if (num_tokens > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case B200_DT_F32: return launch_router<float>(gating_output, topk_weights, topk_ids, num_tokens, num_experts, topk, row_stride, renormalize, st);
    case B200_DT_F16: return launch_router<__half>(gating_output, topk_weights, topk_ids, num_tokens, num_experts, topk, row_stride, renormalize, st);
    case B200_DT_BF16: return launch_router<__nv_bfloat16>(gating_output, topk_weights, topk_ids, num_tokens, num_experts, topk, row_stride, renormalize, st);
    default: return B200_ERR_BAD_DTYPE;
  }
}

// ---------------------------------------------------------------------------------------------------------
// DeepSeek-V3 gate: sigmoid scores, a per-expert bias used for the CHOICE only, group-limited top-k
// (sgl-kernel/csrc/moe/moe_fused_gate.cu:56-260; torch form biased_grouped_topk_impl,
// python/sglang/srt/layers/moe/topk.py:462-530):
//   s = sigmoid(x);  c = s + bias;  group score = sum of the two largest c in the group;
//   keep the topk_group best groups;  pick the topk largest c among their experts;
//   weights = s[picked] / sum(s[picked]).
// One warp per token; lane g scores group g (num_expert_group <= 32); ties go to the lower index.
namespace b200 {
namespace {

template <int PER_LANE>
__global__ void __launch_bounds__(128) fused_gate_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                         float* __restrict__ weights, int32_t* __restrict__ ids,
                                                         int64_t num_tokens, int num_experts, int num_groups,
                                                         int topk_group, int topk_all, int64_t logits_stride,
                                                         int num_shared, double routed_scaling_factor) {
  // topk_all output slots per token: the first topk routed choices, then num_shared fused shared experts
  // (ids num_experts, num_experts + 1, ...) whose weight is (sum of the routed scores / routed_scaling_factor)
  // before the common division by that sum (sgl-kernel/csrc/moe/moe_fused_gate.cu:225-252)
  const int topk = topk_all - num_shared;
  extern __shared__ float smem_choice[];   // [warps][num_experts]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t token = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + wib;
  if (token >= num_tokens) return;
  float* choice = smem_choice + wib * num_experts;
  const float* row = logits + token * logits_stride;
  const int group_size = num_experts / num_groups;
  float s[PER_LANE], c[PER_LANE];
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    if (e < num_experts) {
      s[i] = 1.0f / (1.0f + expf(-row[e]));
      c[i] = s[i] + bias[e];
      choice[e] = c[i];
    } else {
      s[i] = 0.f;
      c[i] = -INFINITY;
    }
  }
  __syncwarp();
  // lane g: sum of the two largest choice scores of group g
  float gscore = -INFINITY;
  if (lane < num_groups) {
    float m1 = -INFINITY, m2 = -INFINITY;
    for (int j = 0; j < group_size; ++j) {
      const float x = choice[lane * group_size + j];
      if (x > m1) { m2 = m1; m1 = x; } else if (x > m2) { m2 = x; }
    }
    gscore = m1 + m2;
  }
  // the topk_group best groups -> bit mask
  uint32_t keep = 0;
  for (int j = 0; j < topk_group; ++j) {
    float best = gscore;
    int best_g = lane < num_groups ? lane : 0x7fffffff;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int og = __shfl_xor_sync(0xffffffffu, best_g, off);
      if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
    }
    keep |= 1u << best_g;
    if (lane == best_g) gscore = -INFINITY;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = i * 32 + lane;
    if (e < num_experts && !((keep >> (e / group_size)) & 1u)) c[i] = -INFINITY;
  }
  float picked_sum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < topk; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    float best_s = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = i * 32 + lane;
      if (e < num_experts && c[i] > best) { best = c[i]; best_e = e; best_s = s[i]; }   // equal values keep the lower id
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      const float os = __shfl_xor_sync(0xffffffffu, best_s, off);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) c[i] = -INFINITY;   // taken
    }
    picked_sum += best_s;
    if (lane == j) { my_w = best_s; my_id = best_e; }
  }
  if (lane < topk) {
    weights[token * topk_all + lane] = my_w / picked_sum;
    ids[token * topk_all + lane] = my_id;
  } else if (lane < topk_all) {
    const float shared = static_cast<float>(static_cast<double>(picked_sum) / routed_scaling_factor);
    weights[token * topk_all + lane] = shared / picked_sum;
    ids[token * topk_all + lane] = num_experts + (lane - topk);
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_moe_fused_gate_shared_experts(const float* gating_output, int64_t row_stride, const float* bias,
                                                  float* topk_weights, int32_t* topk_ids, int64_t num_tokens,
                                                  int num_experts, int num_expert_group, int topk_group, int topk,
                                                  int num_fused_shared_experts, double routed_scaling_factor,
                                                  void* stream) {
  using namespace b200;
  if (num_tokens < 0 || num_experts <= 0 || num_expert_group <= 0 || topk_group <= 0 || topk <= 0) return B200_ERR_BAD_SHAPE;
  if (num_experts % num_expert_group != 0 || num_expert_group > 32 || topk_group > num_expert_group) return B200_ERR_BAD_SHAPE;
  if (num_fused_shared_experts < 0 || num_fused_shared_experts >= topk) return B200_ERR_BAD_SHAPE;
  if (num_fused_shared_experts > 0 && !(routed_scaling_factor != 0.0)) return B200_ERR_BAD_SHAPE;
  const int group_size = num_experts / num_expert_group;
  const int routed = topk - num_fused_shared_experts;
  if (group_size < 2 || topk > 32 || routed > topk_group * group_size) return B200_ERR_BAD_SHAPE;
  if (num_experts > 1024) return B200_ERR_TOO_LARGE;
  if (num_tokens == 0) return B200_OK;
  if (!gating_output || !bias || !topk_weights || !topk_ids) return B200_ERR_NULL_PTR;
  if (row_stride < num_experts) return B200_ERR_BAD_STRIDE;
  if (num_tokens > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>((num_tokens + 3) / 4);
  const size_t smem = 4 * static_cast<size_t>(num_experts) * sizeof(float);
  if (num_experts <= 256)
    fused_gate_kernel<8><<<blocks, 128, smem, st>>>(gating_output, bias, topk_weights, topk_ids, num_tokens, num_experts,
                                                   num_expert_group, topk_group, topk, row_stride,
                                                   num_fused_shared_experts, routed_scaling_factor);
  else
    fused_gate_kernel<32><<<blocks, 128, smem, st>>>(gating_output, bias, topk_weights, topk_ids, num_tokens, num_experts,
                                                    num_expert_group, topk_group, topk, row_stride,
                                                    num_fused_shared_experts, routed_scaling_factor);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_moe_fused_gate(const float* gating_output, int64_t row_stride, const float* bias, float* topk_weights,
                                   int32_t* topk_ids, int64_t num_tokens, int num_experts, int num_expert_group,
                                   int topk_group, int topk, void* stream) {
  return b200_moe_fused_gate_shared_experts(gating_output, row_stride, bias, topk_weights, topk_ids, num_tokens,
                                            num_experts, num_expert_group, topk_group, topk, 0, 1.0, stream);
}
