// Per-token-group FP8 (e4m3) quantisation for sm_100a, single pass over the input.
//
// Stands in for the reference kernel per_token_group_quant_8bit_kernel
// (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:19-114) and must reproduce its codes
// and scales bit for bit:
//     amax  = max(eps, max_i |float(x_i)|)            (fmaxf drops NaNs)
//     scale = amax / fp8_max                          (IEEE fp32 division)
//     code  = e4m3_rne_satfinite(fminf(fmaxf(float(x_i) / scale, fp8_min), fp8_max))
//
// Layout of the work: a block of 256 threads owns a tile of ROWS x 1024 elements.  Each thread
// keeps 16 consecutive elements per row-pass in registers (two 128-bit loads for 2-byte
// inputs), so the input is read once; a warp reads 1 KB contiguous and writes 512 B
// contiguous.  GROUP/16 neighbouring lanes reduce the group's amax with xor shuffles.
// Scales of the tile are staged in shared memory and written out along whichever of the two
// scale strides is the contiguous one, so row-major and column-major scale layouts both
// produce full-sector stores.
//
// Division: x/scale is needed correctly rounded.  The default form computes the correctly
// rounded reciprocal r once per group and then, per element, q0 = x*r, rem = fma(-q0, scale, x),
// q = fma(rem, r, q0) -- correctly rounded for every scale whose significand is not all ones
// (Markstein), with no clamp (the saturating conversion does it).  Threads whose group has such a
// scale or a non-finite one, whose 16 elements contain a NaN, or that were given a non-e4m3 range
// evaluate the reference's expression literally (IEEE division, fmaxf, fminf).
// The *_ieee_div entry point always takes the literal form and exists for cross-checking.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kTileW = 1024;  // elements per tile row
constexpr int kVec = 16;      // elements per thread per pass

template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  uint4 v[2];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    v[0] = __ldcs(p4);
    v[1] = __ldcs(p4 + 1);
  }
  __device__ __forceinline__ void zero() { v[0] = v[1] = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void load_cached(const __nv_bfloat16* p) {   // reused data: default caching
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    v[0] = __ldg(p4);
    v[1] = __ldg(p4 + 1);
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    reinterpret_cast<uint4*>(p)[0] = v[0];
    reinterpret_cast<uint4*>(p)[1] = v[1];
  }
  __device__ __forceinline__ float get(int i) const {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(v);
    const uint32_t word = w[i >> 1];
    return __uint_as_float((i & 1) ? (word & 0xffff0000u) : (word << 16));
  }
  __device__ __forceinline__ void from_floats(const float (&f)[16]) {   // round to nearest even, as a bf16 store would
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(v);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <>
struct Vec16<__half> {
  uint4 v[2];
  __device__ __forceinline__ void load(const __half* p) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    v[0] = __ldcs(p4);
    v[1] = __ldcs(p4 + 1);
  }
  __device__ __forceinline__ void zero() { v[0] = v[1] = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void load_cached(const __half* p) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
    v[0] = __ldg(p4);
    v[1] = __ldg(p4 + 1);
  }
  __device__ __forceinline__ void store(__half* p) const {
    reinterpret_cast<uint4*>(p)[0] = v[0];
    reinterpret_cast<uint4*>(p)[1] = v[1];
  }
  __device__ __forceinline__ float get(int i) const {
    const __half2* h = reinterpret_cast<const __half2*>(v);
    const float2 f = __half22float2(h[i >> 1]);
    return (i & 1) ? f.y : f.x;
  }
  __device__ __forceinline__ void from_floats(const float (&f)[16]) {
    __half2* h = reinterpret_cast<__half2*>(v);
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
};
template <>
struct Vec16<float> {
  uint4 v[4];
  __device__ __forceinline__ void load(const float* p) {
    const uint4* p4 = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = __ldcs(p4 + i);
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = make_uint4(0, 0, 0, 0);
  }
  __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(v)[i]; }
  __device__ __forceinline__ void from_floats(const float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) reinterpret_cast<float*>(v)[i] = f[i];
  }
};

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// The 16 codes of one thread: x / scale correctly rounded, clamped, converted (see the file header).
template <typename T, bool IEEE_DIV>
__device__ __forceinline__ uint4 quantise_vec16(const Vec16<T>& data, float scale, float fp8_min, float fp8_max) {
  const bool std_range = (fp8_max == 448.0f) && (fp8_min == -448.0f);
  bool fast = !IEEE_DIV && std_range;
  if (fast) {
    const uint32_t bits = __float_as_uint(scale);
    // all-ones significand or Inf/NaN scale: leave the fast form
    fast = ((bits & 0x007fffffu) != 0x007fffffu) && ((bits & 0x7f800000u) != 0x7f800000u);
  }
  uint4 out;
  bool need_slow = !fast;
  if (fast) {
    // Correctly rounded x/scale from the correctly rounded reciprocal (Markstein): q0 = x*r,
    // t = fma(q0, scale, -x) = -(x - q0*scale) exactly, q = fma(-t, r, q0).  Written with t = -rem so
    // that a zero x keeps its sign through both fmas (-0 stays -0, +0 stays +0), as x/scale does.
    // |q| <= 448*(1 + 2^-23): the saturating conversion clamps that, so no explicit clamp is needed;
    // only a NaN input must become fp8_min (fmaxf(NaN, lo) = lo in the reference): NaN survives the
    // arithmetic and converts to code 0x7f / 0xff, which is detected on the packed codes below.
    const float r = __frcp_rn(scale);
    float y[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const float v = data.get(i);
      const float q0 = __fmul_rn(v, r);
      const float t = __fmaf_rn(q0, scale, -v);
      y[i] = __fmaf_rn(-t, r, q0);
    }
    out.x = pack4_e4m3(y[0], y[1], y[2], y[3]);
    out.y = pack4_e4m3(y[4], y[5], y[6], y[7]);
    out.z = pack4_e4m3(y[8], y[9], y[10], y[11]);
    out.w = pack4_e4m3(y[12], y[13], y[14], y[15]);
    // a byte with all seven low bits set is a NaN code: (b & 0x7f) + 1 carries into bit 7
    const uint32_t m7 = 0x7f7f7f7fu, one = 0x01010101u;
    const uint32_t nan_bits = (((out.x & m7) + one) | ((out.y & m7) + one) | ((out.z & m7) + one) |
                               ((out.w & m7) + one)) & 0x80808080u;
    need_slow = nan_bits != 0;
  }
  if (need_slow) {
    // the reference's expression, literally
    float y[kVec];
#pragma unroll
    for (int i = 0; i < kVec; ++i)
      y[i] = fminf(fmaxf(__fdiv_rn(data.get(i), scale), fp8_min), fp8_max);
    out.x = pack4_e4m3(y[0], y[1], y[2], y[3]);
    out.y = pack4_e4m3(y[4], y[5], y[6], y[7]);
    out.z = pack4_e4m3(y[8], y[9], y[10], y[11]);
    out.w = pack4_e4m3(y[12], y[13], y[14], y[15]);
  }
  return out;
}

// int8 destination (per_token_group_quant_8bit.cu:110-111 with DST_DTYPE = int8_t, :206-207): the clamped quotient is
// converted by truncation toward zero, as the C++ cast does.  Same quotient as above (correctly rounded; the literal
// division where the reciprocal form is not exact); the clamp is explicit here, and fmaxf turns a NaN into q_min.
template <typename T>
__device__ __forceinline__ uint4 quantise_vec16_int8(const Vec16<T>& data, float scale, float q_min, float q_max) {
  const uint32_t bits = __float_as_uint(scale);
  const bool fast = ((bits & 0x007fffffu) != 0x007fffffu) && ((bits & 0x7f800000u) != 0x7f800000u);
  const float r = __frcp_rn(scale);
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int c[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float v = data.get(4 * j + e);
      float q;
      if (fast) {
        const float q0 = __fmul_rn(v, r);
        const float t = __fmaf_rn(q0, scale, -v);
        q = __fmaf_rn(-t, r, q0);
      } else {
        q = __fdiv_rn(v, scale);
      }
      c[e] = __float2int_rz(fminf(fmaxf(q, q_min), q_max));
    }
    // four ints -> four saturated int8 in one word (byte e = c[e])
    uint32_t hi;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(c[3]), "r"(c[2]));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(w[j]) : "r"(c[1]), "r"(c[0]), "r"(hi));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// FUSE_SILU: x is [M, 2K] (gate | up); the row to quantise is silu(gate) * up, computed in fp32 and
// rounded to T exactly as the separate silu_and_mul kernel stores it, so codes and scales equal the
// two-kernel sequence bit for bit while the [M, K] intermediate never touches HBM.
// UE8M0: the scale is rounded up to a power of two, exp2f(ceilf(log2f(max(amax/448, 1e-10)))), and
// stored as its biased exponent byte, four k-groups per int32, column-major: the byte of (row r,
// group g) lives at byte ((g/4) * s_stride_grp + r) * 4 + g%4 of s
// (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:54-61,86-97; rows are
// contiguous; s_stride_row = 1 there).  A caller may ask for other word strides (rows of words contiguous: what an
// expert-parallel dispatch sends per token).  The tile writes whole words; groups past K/GROUP inside the last word
// are zero bytes.
template <typename T, int GROUP, int PASSES, bool IEEE_DIV, bool FUSE_SILU = false, bool UE8M0 = false, bool INT8 = false>
__global__ void __launch_bounds__(kThreads, (PASSES >= 8 || sizeof(T) == 4) ? 2 : 4)   // 4 blocks/SM: <= 64 registers
quant_group_kernel(const T* __restrict__ x, const int32_t* __restrict__ src_rows, int64_t x_rows, uint8_t* __restrict__ q,
                   float* __restrict__ s, int64_t M, int64_t K,
                   int64_t s_stride_row, int64_t s_stride_grp, float eps, float fp8_min, float fp8_max,
                   int tiles_k) {
  constexpr int TPG = GROUP / kVec;              // lanes cooperating on one group
  constexpr int GPT = kTileW / GROUP;            // groups per tile row
  constexpr int SLOTS_PER_ROW = kTileW / kVec;   // 64 threads per tile row
  constexpr int ROWS_PER_PASS = kThreads / SLOTS_PER_ROW;  // 4
  constexpr int ROWS = ROWS_PER_PASS * PASSES;
  static_assert(TPG >= 1 && TPG <= 32, "group size");

  __shared__ float s_tile[ROWS * GPT];

  const int tid = threadIdx.x;
  const int64_t tile_m = blockIdx.x / tiles_k;
  const int tile_k = blockIdx.x % tiles_k;
  const int row_in_pass = tid / SLOTS_PER_ROW;
  const int slot = tid % SLOTS_PER_ROW;
  const int64_t col = static_cast<int64_t>(tile_k) * kTileW + slot * kVec;
  const int64_t row0 = tile_m * ROWS + row_in_pass;
  const bool col_ok = col < K;  // K % GROUP == 0 and GROUP % 16 == 0: a thread's 16 elements never straddle K

  Vec16<T> data[PASSES];
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int64_t row = row0 + p * ROWS_PER_PASS;
    if (col_ok && row < M) {
      // src_rows (optional): output row `row` quantises input row src_rows[row] (a routed copy of a token)
      // (clamped into the input's rows: a table that does not match the buffer cannot send a load out of bounds)
      const int64_t srow = src_rows ? min(max(static_cast<int64_t>(__ldg(src_rows + row)), int64_t(0)), x_rows - 1) : row;
      if constexpr (FUSE_SILU) {
        Vec16<T> gate, up;
        gate.load(x + srow * 2 * K + col);
        up.load(x + srow * 2 * K + K + col);
        float f[kVec];
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          const float gv = gate.get(i);
          f[i] = (gv / (1.0f + __expf(-gv))) * up.get(i);
        }
        data[p].from_floats(f);
      } else {
        data[p].load(x + srow * K + col);
      }
    } else {
      data[p].zero();
    }
  }

#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int64_t row = row0 + p * ROWS_PER_PASS;
    float amax = eps;
#pragma unroll
    for (int i = 0; i < kVec; ++i) amax = fmaxf(amax, fabsf(data[p].get(i)));
#pragma unroll
    for (int off = TPG / 2; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));

    float scale = __fdiv_rn(amax, fp8_max);
    if constexpr (UE8M0) scale = exp2f(ceilf(log2f(fmaxf(scale, 1e-10f))));
    uint4 out;
    if constexpr (INT8) out = quantise_vec16_int8<T>(data[p], scale, fp8_min, fp8_max);
    else out = quantise_vec16<T, IEEE_DIV>(data[p], scale, fp8_min, fp8_max);
    if (col_ok && row < M) *reinterpret_cast<uint4*>(q + row * K + col) = out;
    if ((slot % TPG) == 0) s_tile[(p * ROWS_PER_PASS + row_in_pass) * GPT + slot / TPG] = scale;
  }
  __syncthreads();

  // Write the tile's scales along the contiguous scale dimension.
  const int64_t g0 = static_cast<int64_t>(tile_k) * GPT;
  const int64_t G = K / GROUP;
  const int64_t r0 = tile_m * ROWS;
  if constexpr (UE8M0) {
    static_assert(GPT % 4 == 0, "a tile row must hold whole packed words");
    uint32_t* sp = reinterpret_cast<uint32_t*>(s);
    for (int idx = tid; idx < ROWS * (GPT / 4); idx += kThreads) {
      const int w = idx / ROWS, r = idx % ROWS;   // rows are the contiguous dimension
      if (r0 + r < M && g0 + 4 * w < G) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          if (g0 + 4 * w + b < G) {
            const uint32_t byte = static_cast<uint8_t>(static_cast<int>(log2f(s_tile[r * GPT + 4 * w + b])) + 127);
            word |= byte << (8 * b);
          }
        }
        sp[(g0 / 4 + w) * s_stride_grp + (r0 + r) * s_stride_row] = word;
      }
    }
    return;
  }
  const bool rows_contig = s_stride_row <= s_stride_grp;
  for (int idx = tid; idx < ROWS * GPT; idx += kThreads) {
    int r, g;
    if (rows_contig) {
      g = idx / ROWS;
      r = idx % ROWS;
    } else {
      r = idx / GPT;
      g = idx % GPT;
    }
    if (r0 + r < M && g0 + g < G) s[(r0 + r) * s_stride_row + (g0 + g) * s_stride_grp] = s_tile[r * GPT + g];
  }
}

// ------------------------------------------------------------------------------------------ RMSNorm -> quant
// One block per row: y = T((x * rsqrt(mean(x^2) + eps)) * w), optionally after x += residual (the sum is kept in
// fp32 for the norm and written back rounded, as the reference's fused_add_rmsnorm does), then the 128-group
// quantisation of y -- the arithmetic of RMSNorm.forward_native
// (python/sglang/srt/layers/layernorm.py:135-171) followed by sglang_per_token_group_quant_fp8.  The row stays in
// registers between the three phases (sum of squares, normalise, quantise), so HBM sees one read of x (and of the
// residual) and one write of the codes (and of y when the caller wants it).  WITH_Q = false is the plain norm.
constexpr int kNormMaxVecs = 4;   // 16-element vectors per thread: rows up to 256 * 4 * 16 = 16384 elements

template <typename T, bool WITH_Q, bool UE8M0, int NV, bool HAS_RES>
__global__ void __launch_bounds__(kThreads, NV <= 2 ? (HAS_RES ? 4 : 5) : 2) rmsnorm_quant_kernel(const T* __restrict__ x, T* __restrict__ residual,
                                                                    const T* __restrict__ weight, T* __restrict__ y,
                                                                    uint8_t* __restrict__ q, float* __restrict__ s, int64_t M,
                                                                    int64_t K, int64_t s_stride_row, int64_t s_stride_grp,
                                                                    float norm_eps, float eps, float fp8_min,
                                                                    float fp8_max) {
  __shared__ float red[kThreads / 32];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  const int nvec = static_cast<int>(K / kVec);
  // The row is held PACKED (8 registers per 16 elements; with a residual both addends) and unpacked again in each
  // phase: few registers per thread, so that several blocks share an SM and enough loads are in flight.
  Vec16<T> d[NV];
  [[maybe_unused]] Vec16<T> r[HAS_RES ? NV : 1];
  constexpr bool has_res = HAS_RES;
  float sumsq = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * kThreads;
    if (v < nvec) {
      d[i].load(x + row * K + static_cast<int64_t>(v) * kVec);
      if constexpr (HAS_RES) {
        r[i].load(residual + row * K + static_cast<int64_t>(v) * kVec);
        float f[kVec];
#pragma unroll
        for (int e = 0; e < kVec; ++e) {
          f[e] = d[i].get(e) + r[i].get(e);
          sumsq = fmaf(f[e], f[e], sumsq);
        }
        Vec16<T> o;
        o.from_floats(f);
        o.store(residual + row * K + static_cast<int64_t>(v) * kVec);
      } else {
#pragma unroll
        for (int e = 0; e < kVec; ++e) sumsq = fmaf(d[i].get(e), d[i].get(e), sumsq);
      }
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, off);
  if ((tid & 31) == 0) red[tid >> 5] = sumsq;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) total += red[w];   // same order in every thread
  const float rinv = rsqrtf(total / static_cast<float>(K) + norm_eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = tid + i * kThreads;
    // K % 128 == 0: the eight lanes of a group are inside the row together or not at all
    [[maybe_unused]] const unsigned lanes = __ballot_sync(0xffffffffu, v < nvec);
    if (v < nvec) {
      Vec16<T> w;
      w.load_cached(weight + static_cast<int64_t>(v) * kVec);
      float f[kVec];
#pragma unroll
      for (int e = 0; e < kVec; ++e) {
        float xe = d[i].get(e);
        if constexpr (HAS_RES) xe += r[i].get(e);                              // the same fp32 sum as in phase one
        f[e] = __fmul_rn(__fmul_rn(xe, rinv), w.get(e));
      }
      Vec16<T> o;
      o.from_floats(f);                                          // y in T, exactly what a separate norm kernel stores
      if (y) o.store(y + row * K + static_cast<int64_t>(v) * kVec);
      if constexpr (WITH_Q) {
        // a 128-group is eight consecutive vectors = eight consecutive lanes
        float amax = eps;
#pragma unroll
        for (int e = 0; e < kVec; ++e) amax = fmaxf(amax, fabsf(o.get(e)));
#pragma unroll
        for (int off = 4; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(lanes, amax, off));
        float scale = __fdiv_rn(amax, fp8_max);
        if constexpr (UE8M0) scale = exp2f(ceilf(log2f(fmaxf(scale, 1e-10f))));
        const uint4 codes = quantise_vec16<T, false>(o, scale, fp8_min, fp8_max);
        *reinterpret_cast<uint4*>(q + row * K + static_cast<int64_t>(v) * kVec) = codes;
        if ((v & 7) == 0) {
          const int g = v >> 3;
          if constexpr (UE8M0) {
            // one byte of the packed word of (row, g / 4); the four groups of a word are written by four threads
            reinterpret_cast<uint8_t*>(s)[(static_cast<int64_t>(g >> 2) * s_stride_grp + row) * 4 + (g & 3)] =
                static_cast<uint8_t>(static_cast<int>(log2f(scale)) + 127);
          } else {
            s[row * s_stride_row + g * s_stride_grp] = scale;
          }
        }
      }
    }
  }
}

template <typename T, int GROUP, bool IEEE_DIV, bool FUSE_SILU = false, bool UE8M0 = false, bool INT8 = false>
int launch_group(const void* x, void* q, float* s, int64_t M, int64_t K, int64_t ssr, int64_t ssg, float eps,
                 float fmin_, float fmax_, cudaStream_t stream, const int32_t* src_rows = nullptr, int64_t x_rows = 0) {
  const int tiles_k = static_cast<int>((K + kTileW - 1) / kTileW);
  const int sms = sm_count();
  if (sms <= 0) return B200_ERR_CUDA;
  // 4 passes (16 rows, 64 registers, 4 blocks per SM) measured fastest; 8 is kept for experiments
  constexpr int kMaxPasses = sizeof(T) == 4 ? 4 : 8;
  constexpr int kDefaultPasses = 4;
  auto tiles_for = [&](int passes) { return ((M + 4 * passes - 1) / (4 * passes)) * tiles_k; };
  int passes = kDefaultPasses;
  while (passes > 1 && tiles_for(passes) < 4LL * sms) passes >>= 1;
  const int64_t tiles = tiles_for(passes);
  if (tiles > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  const dim3 grid(static_cast<unsigned>(tiles));
  const T* xp = static_cast<const T*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
#define B200_LAUNCH_Q(P)                                                                                       \
  quant_group_kernel<T, GROUP, P, IEEE_DIV, FUSE_SILU, UE8M0, INT8><<<grid, kThreads, 0, stream>>>(xp, src_rows, x_rows, qp, s, M, K, ssr, ssg, eps, fmin_, \
                                                                           fmax_, tiles_k)
  switch (passes) {
    case 8:
      if constexpr (kMaxPasses >= 8) { B200_LAUNCH_Q(8); }
      break;
    case 4: B200_LAUNCH_Q(4); break;
    case 2: B200_LAUNCH_Q(2); break;
    default: B200_LAUNCH_Q(1); break;
  }
#undef B200_LAUNCH_Q
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <typename T, bool IEEE_DIV, bool INT8 = false>
int dispatch_group(int64_t group, const void* x, void* q, float* s, int64_t M, int64_t K, int64_t ssr, int64_t ssg,
                   float eps, float fmin_, float fmax_, cudaStream_t st) {
  switch (group) {
    case 64: return launch_group<T, 64, IEEE_DIV, false, false, INT8>(x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    case 128: return launch_group<T, 128, IEEE_DIV, false, false, INT8>(x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    case 256: return launch_group<T, 256, IEEE_DIV, false, false, INT8>(x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    case 512: return launch_group<T, 512, IEEE_DIV, false, false, INT8>(x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    default: return B200_ERR_UNSUPPORTED;
  }
}

template <bool IEEE_DIV, bool INT8 = false>
int quant_entry(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K, int64_t group, int64_t ssr,
                int64_t ssg, float eps, float fmin_, float fmax_, void* stream) {
  if (M < 0 || K < 0 || group <= 0) return B200_ERR_BAD_SHAPE;
  if (K % group != 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || K == 0) return B200_OK;
  if (!x || !q || !s) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (ssr < 0 || ssg < 0 || (ssr == 0 && M > 1) || (ssg == 0 && K / group > 1)) return B200_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_DT_BF16:
      return dispatch_group<__nv_bfloat16, IEEE_DIV, INT8>(group, x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    case B200_DT_F16:
      return dispatch_group<__half, IEEE_DIV, INT8>(group, x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    case B200_DT_F32:
      return dispatch_group<float, IEEE_DIV, INT8>(group, x, q, s, M, K, ssr, ssg, eps, fmin_, fmax_, st);
    default:
      return B200_ERR_BAD_DTYPE;
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                                              int64_t group_size, int64_t s_stride_row, int64_t s_stride_grp,
                                              float eps, float fp8_min, float fp8_max, void* stream) {
  return b200::quant_entry<false>(x, x_dtype, q, s, M, K, group_size, s_stride_row, s_stride_grp, eps, fp8_min,
                                  fp8_max, stream);
}

extern "C" int b200_per_token_group_quant_int8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                                               int64_t group_size, int64_t s_stride_row, int64_t s_stride_grp,
                                               float eps, float int8_min, float int8_max, void* stream) {
  return b200::quant_entry<false, true>(x, x_dtype, q, s, M, K, group_size, s_stride_row, s_stride_grp, eps, int8_min,
                                        int8_max, stream);
}

extern "C" int b200_per_token_group_quant_fp8_ieee_div(const void* x, int x_dtype, void* q, float* s, int64_t M,
                                                       int64_t K, int64_t group_size, int64_t s_stride_row,
                                                       int64_t s_stride_grp, float eps, float fp8_min, float fp8_max,
                                                       void* stream) {
  return b200::quant_entry<true>(x, x_dtype, q, s, M, K, group_size, s_stride_row, s_stride_grp, eps, fp8_min,
                                 fp8_max, stream);
}

extern "C" int b200_silu_mul_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M,
                                                       int64_t K, int64_t s_stride_row, int64_t s_stride_grp,
                                                       float eps, float fp8_min, float fp8_max, void* stream) {
  using namespace b200;
  if (M < 0 || K < 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || K == 0) return B200_OK;
  if (!x || !q || !s) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (s_stride_row < 0 || s_stride_grp < 0 || (s_stride_row == 0 && M > 1) || (s_stride_grp == 0 && K / 128 > 1))
    return B200_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case B200_DT_BF16:
      return launch_group<__nv_bfloat16, 128, false, true>(x, q, s, M, K, s_stride_row, s_stride_grp, eps, fp8_min,
                                                           fp8_max, st);
    case B200_DT_F16:
      return launch_group<__half, 128, false, true>(x, q, s, M, K, s_stride_row, s_stride_grp, eps, fp8_min, fp8_max,
                                                    st);
    default:
      return B200_ERR_BAD_DTYPE;
  }
}

extern "C" int b200_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, uint32_t* s_packed, int64_t M,
                                                    int64_t K, int64_t s_stride_pack, float eps, float fp8_min,
                                                    float fp8_max, void* stream) {
  using namespace b200;
  if (M < 0 || K < 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || K == 0) return B200_OK;
  if (!x || !q || !s_packed) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (s_stride_pack < M) return B200_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* s = reinterpret_cast<float*>(s_packed);
  switch (x_dtype) {
    case B200_DT_BF16:
      return launch_group<__nv_bfloat16, 128, false, false, true>(x, q, s, M, K, 1, s_stride_pack, eps, fp8_min, fp8_max, st);
    case B200_DT_F16:
      return launch_group<__half, 128, false, false, true>(x, q, s, M, K, 1, s_stride_pack, eps, fp8_min, fp8_max, st);
    case B200_DT_F32:
      return launch_group<float, 128, false, false, true>(x, q, s, M, K, 1, s_stride_pack, eps, fp8_min, fp8_max, st);
    default:
      return B200_ERR_BAD_DTYPE;
  }
}

// SiLU(gate) * up followed by the power-of-two quantisation, in one pass: what the second expert GEMM of the
// block-scaling path consumes (the reference runs silu_and_mul, then sglang_per_token_group_quant_fp8 with
// scale_ue8m0=True: python/sglang/srt/layers/moe/ep_moe/layer.py:606-628).  x is [M, 2K] (gate | up).
extern "C" int b200_silu_mul_per_token_group_quant_fp8_ue8m0(const void* x, int x_dtype, void* q, uint32_t* s_packed,
                                                             int64_t M, int64_t K, int64_t s_stride_pack, float eps,
                                                             float fp8_min, float fp8_max, void* stream) {
  using namespace b200;
  if (M < 0 || K < 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || K == 0) return B200_OK;
  if (!x || !q || !s_packed) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (s_stride_pack < M) return B200_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* s = reinterpret_cast<float*>(s_packed);
  switch (x_dtype) {
    case B200_DT_BF16:
      return launch_group<__nv_bfloat16, 128, false, true, true>(x, q, s, M, K, 1, s_stride_pack, eps, fp8_min, fp8_max, st);
    case B200_DT_F16:
      return launch_group<__half, 128, false, true, true>(x, q, s, M, K, 1, s_stride_pack, eps, fp8_min, fp8_max, st);
    default:
      return B200_ERR_BAD_DTYPE;
  }
}

// Row gather fused into the quantisation: output row r holds the codes and scale(s) of input row src_rows[r].
// One launch in place of quantise + gather codes + gather scales when every token is copied to the rows of its
// experts (the reference's ep_scatter after the quantisation, python/sglang/srt/layers/moe/ep_moe/kernels.py;
// shuffle_rows in cutlass_moe.py:144-150): same bits as quantising first and gathering afterwards.  x has `x_rows`
// rows; indices are clamped into [0, x_rows).  scale_ue8m0 != 0: s is the packed exponent tensor
// (s_stride_grp = the stride between packed words, s_stride_row ignored).
extern "C" int b200_gather_per_token_group_quant_fp8(const void* x, int x_dtype, int64_t x_rows, const int32_t* src_rows,
                                                     void* q, void* s, int64_t R, int64_t K, int64_t s_stride_row,
                                                     int64_t s_stride_grp, int scale_ue8m0, float eps, float fp8_min,
                                                     float fp8_max, void* stream) {
  using namespace b200;
  if (R < 0 || K < 0 || x_rows < 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (R == 0 || K == 0) return B200_OK;
  if (x_rows == 0) return B200_ERR_BAD_SHAPE;
  if (!x || !q || !s || !src_rows) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (scale_ue8m0) {
    if (s_stride_grp < R) return B200_ERR_BAD_STRIDE;
    s_stride_row = 1;
  } else if (s_stride_row < 0 || s_stride_grp < 0 || (s_stride_row == 0 && R > 1) || (s_stride_grp == 0 && K / 128 > 1)) {
    return B200_ERR_BAD_STRIDE;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* sp = static_cast<float*>(s);
#define B200_GQ(T)                                                                                                  \
  (scale_ue8m0 ? launch_group<T, 128, false, false, true>(x, q, sp, R, K, s_stride_row, s_stride_grp, eps, fp8_min, \
                                                          fp8_max, st, src_rows, x_rows)                           \
               : launch_group<T, 128, false, false, false>(x, q, sp, R, K, s_stride_row, s_stride_grp, eps, fp8_min, \
                                                           fp8_max, st, src_rows, x_rows))
  switch (x_dtype) {
    case B200_DT_BF16: return B200_GQ(__nv_bfloat16);
    case B200_DT_F16: return B200_GQ(__half);
    case B200_DT_F32: return B200_GQ(float);
    default: return B200_ERR_BAD_DTYPE;
  }
#undef B200_GQ
}

// RMSNorm (optionally fused with the residual add) with or without the 128-group FP8 quantisation of its output,
// one pass.  x [M, K] (bf16 / fp16), weight [K]; residual [M, K] or NULL: x + residual is normalised and written back
// to residual; y [M, K] or NULL: the normalised row in x's type; q / s: codes and scales as in
// b200_per_token_group_quant_fp8 (scale_ue8m0 != 0: the packed layout, s_stride_grp = stride between words), or
// both NULL for the norm alone.  K % 128 == 0 and K <= 16384.
extern "C" int b200_rmsnorm_per_token_group_quant_fp8(const void* x, int x_dtype, void* residual, const void* weight,
                                                      float norm_eps, void* y, void* q, void* s, int64_t M, int64_t K,
                                                      int64_t s_stride_row, int64_t s_stride_grp, int scale_ue8m0,
                                                      float eps, float fp8_min, float fp8_max, void* stream) {
  using namespace b200;
  if (M < 0 || K <= 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (K > static_cast<int64_t>(kThreads) * kNormMaxVecs * kVec) return B200_ERR_TOO_LARGE;
  if (M == 0) return B200_OK;
  if (M > 0x7fffffffLL) return B200_ERR_TOO_LARGE;
  if (!x || !weight) return B200_ERR_NULL_PTR;
  const bool with_q = q != nullptr;
  if (with_q != (s != nullptr)) return B200_ERR_NULL_PTR;
  if (!with_q && !y) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(weight) || (residual && !aligned16(residual)) || (y && !aligned16(y)) ||
      (q && !aligned16(q)))
    return B200_ERR_MISALIGNED;
  if (with_q) {
    if (scale_ue8m0) {
      if (s_stride_grp < M) return B200_ERR_BAD_STRIDE;
    } else if (s_stride_row < 0 || s_stride_grp < 0 || (s_stride_row == 0 && M > 1) || (s_stride_grp == 0 && K / 128 > 1)) {
      return B200_ERR_BAD_STRIDE;
    }
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(M));
#define B200_NORM_GO(T, NV, WQ, UE, RES)                                                                              \
  rmsnorm_quant_kernel<T, WQ, UE, NV, RES><<<grid, kThreads, 0, st>>>(                                                \
      static_cast<const T*>(x), static_cast<T*>(residual), static_cast<const T*>(weight), static_cast<T*>(y),         \
      static_cast<uint8_t*>(q), static_cast<float*>(s), M, K, s_stride_row, s_stride_grp, norm_eps, eps, fp8_min,     \
      fp8_max)
#define B200_NORM_NV(T, NV)                                       \
  do {                                                            \
    if (residual) {                                               \
      if (!with_q) B200_NORM_GO(T, NV, false, false, true);       \
      else if (scale_ue8m0) B200_NORM_GO(T, NV, true, true, true); \
      else B200_NORM_GO(T, NV, true, false, true);                \
    } else {                                                      \
      if (!with_q) B200_NORM_GO(T, NV, false, false, false);      \
      else if (scale_ue8m0) B200_NORM_GO(T, NV, true, true, false); \
      else B200_NORM_GO(T, NV, true, false, false);               \
    }                                                             \
  } while (0)
  // vectors per thread: rows up to 4096 / 8192 / 16384 elements
#define B200_NORM(T)                                              \
  do {                                                            \
    if (K <= kThreads * kVec) B200_NORM_NV(T, 1);                 \
    else if (K <= 2 * kThreads * kVec) B200_NORM_NV(T, 2);        \
    else B200_NORM_NV(T, 4);                                      \
  } while (0)
  switch (x_dtype) {
    case B200_DT_BF16: B200_NORM(__nv_bfloat16); break;
    case B200_DT_F16: B200_NORM(__half); break;
    default: return B200_ERR_BAD_DTYPE;
  }
#undef B200_NORM_NV
#undef B200_NORM_GO
#undef B200_NORM
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// The power-of-two quantisation with caller-chosen word strides: word (r, w) at s_packed[r * s_stride_row +
// w * s_stride_pack].  s_stride_row = 1 is b200_per_token_group_quant_fp8_ue8m0; s_stride_pack = 1 with
// s_stride_row >= ceil(K / 512) keeps a token's words together (one contiguous scale row per token, which is what the
// expert-parallel dispatch copies).
extern "C" int b200_per_token_group_quant_fp8_ue8m0_strided(const void* x, int x_dtype, void* q, uint32_t* s_packed,
                                                            int64_t M, int64_t K, int64_t s_stride_row,
                                                            int64_t s_stride_pack, float eps, float fp8_min,
                                                            float fp8_max, void* stream) {
  using namespace b200;
  if (M < 0 || K < 0) return B200_ERR_BAD_SHAPE;
  if (K % 128 != 0) return B200_ERR_BAD_SHAPE;
  if (M == 0 || K == 0) return B200_OK;
  if (!x || !q || !s_packed) return B200_ERR_NULL_PTR;
  if (!aligned16(x) || !aligned16(q)) return B200_ERR_MISALIGNED;
  if (s_stride_row <= 0 || s_stride_pack <= 0) return B200_ERR_BAD_STRIDE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* s = reinterpret_cast<float*>(s_packed);
  switch (x_dtype) {
    case B200_DT_BF16:
      return launch_group<__nv_bfloat16, 128, false, false, true>(x, q, s, M, K, s_stride_row, s_stride_pack, eps, fp8_min, fp8_max, st);
    case B200_DT_F16:
      return launch_group<__half, 128, false, false, true>(x, q, s, M, K, s_stride_row, s_stride_pack, eps, fp8_min, fp8_max, st);
    case B200_DT_F32:
      return launch_group<float, 128, false, false, true>(x, q, s, M, K, s_stride_row, s_stride_pack, eps, fp8_min, fp8_max, st);
    default:
      return B200_ERR_BAD_DTYPE;
  }
}
