// Rowwise e4m3 quantiser: one pass over HBM.  A CTA owns a row, keeps it in registers between
// the absmax reduction and the quantisation, and writes e4m3 bytes plus one fp32 scale.
//
// Two recipes, both bit-exact with the torch expressions they replace:
//   kRecipeOperator   the operator's own `fp8_row_quantize`: every step in the dtype T of x, each
//                     result rounded to T as torch's eager kernels do:
//                        c = max(rowabsmax, T(1e-12));  mult = T(T(1 / c) * 448)   [torch evaluates scalar / tensor
//                        as reciprocal(tensor) * scalar];  (fp16: mult = min(mult, 65504))
//                        q = e4m3( clamp( T(x * mult), +-448 ) );  scale = float( T(1 / mult) )
//   kRecipeFp32       the benchmark recipe on fp32 math:
//                        scale = max(rowabsmax, 1e-12) / 448;  q = e4m3( clamp( x / scale, +-448 ) )
// Divisions and products are IEEE round-to-nearest (no fast-math), conversions to e4m3 round to
// nearest even and cannot overflow after the clamp.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>
#include <type_traits>

#include "kernels.h"
#include "nanmax.cuh"

namespace b200fp8 {
namespace {


constexpr int kThreads = 256;
constexpr int kVec = 8;       // elements per vector load (16 bytes of a 16-bit type; two loads for fp32)
constexpr int kMaxVecs = 8;   // vectors a thread keeps in registers: rows up to 256*8*8 = 16384 elements

template <typename T> struct Conv;
template <> struct Conv<__nv_bfloat16> {
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct Conv<__half> {
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ float rnd(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct Conv<float> {
  static __device__ __forceinline__ float up(float v) { return v; }
  static __device__ __forceinline__ float rnd(float v) { return v; }
};

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float block_max(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max_nan(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = smem[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) r = max_nan(r, smem[w]);
  return r;
}

// eight consecutive elements as loaded (kept packed between the two passes to save registers)
template <typename T>
struct Raw {
  uint4 lo;
  uint4 hi;  // used by 4-byte T only
};

template <typename T>
__device__ __forceinline__ Raw<T> load_raw(const T* p) {
  Raw<T> r;
  r.lo = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 4) r.hi = *reinterpret_cast<const uint4*>(p + 4);
  return r;
}

// absmax of the eight elements, and their eight e4m3 codes.  16-bit types stay packed: two
// elements per instruction for |x|, max, the product (mul.rn of the packed type IS the correctly
// rounded product torch computes) and the e4m3 conversion (cvt.rn.satfinite.e4m3x2.f32; saturation
// to +-448 is the clamp).
template <typename T, int kRecipe>
struct Ops;

template <int kRecipe>
struct Ops<__nv_bfloat16, kRecipe> {
  static __device__ __forceinline__ float absmax(const Raw<__nv_bfloat16>& r) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.lo);
    __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(__habs2(h[0]), __habs2(h[1])), __hmax2_nan(__habs2(h[2]), __habs2(h[3])));
    return max_nan(__low2float(m), __high2float(m));
  }
  static __device__ __forceinline__ uint2 codes(const Raw<__nv_bfloat16>& r, float mult) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r.lo);
    const __nv_bfloat162 m2 = __float2bfloat162_rn(mult);  // mult is a bf16 value already
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 a = __bfloat1622float2(__hmul2(h[2 * i], m2));
      const float2 b = __bfloat1622float2(__hmul2(h[2 * i + 1], m2));
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(a, __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(b, __NV_SATFINITE, __NV_E4M3);
      w[i] = lo | (hi << 16);
    }
    return make_uint2(w[0], w[1]);
  }
};

template <int kRecipe>
struct Ops<__half, kRecipe> {
  static __device__ __forceinline__ float absmax(const Raw<__half>& r) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.lo);
    __half2 m = __hmax2_nan(__hmax2_nan(__habs2(h[0]), __habs2(h[1])), __hmax2_nan(__habs2(h[2]), __habs2(h[3])));
    return max_nan(__low2float(m), __high2float(m));
  }
  static __device__ __forceinline__ uint2 codes(const Raw<__half>& r, float mult) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.lo);
    const __half2 m2 = __float2half2_rn(mult);
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 a = __half22float2(__hmul2(h[2 * i], m2));
      const float2 b = __half22float2(__hmul2(h[2 * i + 1], m2));
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(a, __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(b, __NV_SATFINITE, __NV_E4M3);
      w[i] = lo | (hi << 16);
    }
    return make_uint2(w[0], w[1]);
  }
};

template <int kRecipe>
struct Ops<float, kRecipe> {
  static __device__ __forceinline__ float absmax(const Raw<float>& r) {
    const float* a = reinterpret_cast<const float*>(&r.lo);
    const float* b = reinterpret_cast<const float*>(&r.hi);
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) m = max_nan(m, max_nan(fabsf(a[j]), fabsf(b[j])));
    return m;
  }
  static __device__ __forceinline__ float one(float v, float mult) {
    return kRecipe == kRecipeOperator ? __fmul_rn(v, mult) : __fdiv_rn(v, mult);
  }
  static __device__ __forceinline__ uint2 codes(const Raw<float>& r, float mult) {
    const float* a = reinterpret_cast<const float*>(&r.lo);
    const float* b = reinterpret_cast<const float*>(&r.hi);
    const uint32_t c0 = __nv_cvt_float2_to_fp8x2(make_float2(one(a[0], mult), one(a[1], mult)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t c1 = __nv_cvt_float2_to_fp8x2(make_float2(one(a[2], mult), one(a[3], mult)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t c2 = __nv_cvt_float2_to_fp8x2(make_float2(one(b[0], mult), one(b[1], mult)), __NV_SATFINITE, __NV_E4M3);
    const uint32_t c3 = __nv_cvt_float2_to_fp8x2(make_float2(one(b[2], mult), one(b[3], mult)), __NV_SATFINITE, __NV_E4M3);
    return make_uint2(c0 | (c1 << 16), c2 | (c3 << 16));
  }
};

template <typename T, int kRecipe>
__global__ void __launch_bounds__(kThreads) row_quantize_kernel(const QuantParams p) {
  __shared__ float red[kThreads / 32];
  const long long row = blockIdx.x;
  const T* x = static_cast<const T*>(p.x) + row * p.ldx;
  uint8_t* q = p.q + row * p.ldq;
  const int cols = p.cols;
  const int vec_cols = p.vector_ok ? (cols / kVec) * kVec : 0;  // handled with 16-byte accesses
  const int nvec = vec_cols / kVec;

  // pass 1: absmax; the first kMaxVecs vectors of every thread stay (packed) in registers
  using O = Ops<T, kRecipe>;
  Raw<T> keep[kMaxVecs];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < kMaxVecs; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) keep[i] = load_raw<T>(x + v * kVec);
  }
#pragma unroll
  for (int i = 0; i < kMaxVecs; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) amax = max_nan(amax, O::absmax(keep[i]));
  }
  for (int v = threadIdx.x + kMaxVecs * kThreads; v < nvec; v += kThreads) {  // rows longer than 16384
    amax = max_nan(amax, O::absmax(load_raw<T>(x + v * kVec)));
  }
  for (int c = vec_cols + threadIdx.x; c < cols; c += kThreads) amax = max_nan(amax, fabsf(Conv<T>::up(x[c])));
  amax = block_max(amax, red);

  // the row's multiplier (or divisor) and the scale handed to the GEMM
  float mult, scale;
  if constexpr (kRecipe == kRecipeOperator) {
    const float c = max_nan(amax, Conv<T>::rnd(1e-12f));
    mult = Conv<T>::rnd(__fmul_rn(Conv<T>::rnd(__fdiv_rn(1.0f, c)), 448.0f));
    if constexpr (std::is_same<T, __half>::value) mult = min_nan(mult, 65504.0f);
    scale = Conv<T>::rnd(__fdiv_rn(1.0f, mult));
  } else {
    scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
    mult = scale;  // used as the divisor
  }
  if (threadIdx.x == 0) p.scale[row] = scale;

  // pass 2: quantise from registers (re-reading only what did not fit)
#pragma unroll
  for (int i = 0; i < kMaxVecs; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) *reinterpret_cast<uint2*>(q + v * kVec) = O::codes(keep[i], mult);
  }
  for (int v = threadIdx.x + kMaxVecs * kThreads; v < nvec; v += kThreads) {
    *reinterpret_cast<uint2*>(q + v * kVec) = O::codes(load_raw<T>(x + v * kVec), mult);
  }
  for (int c = vec_cols + threadIdx.x; c < cols; c += kThreads) {
    const float v = Conv<T>::up(x[c]);
    const float y = kRecipe == kRecipeOperator ? Conv<T>::rnd(__fmul_rn(v, mult)) : __fdiv_rn(v, mult);
    q[c] = to_e4m3(y);
  }
}

// Persistent form for aligned rows of 2561 to 16384 elements: a CTA of one warp per 1024 elements (a thread owns four
// vectors of eight, whatever the row length; the CTA size is a compile-time constant) walks over rows blockIdx.x,
// blockIdx.x + gridDim.x, ... and requests the next row before it reduces and writes the current one, so that
// memory latency is paid once per CTA instead of once per row.  One barrier per row: the warps' maxima alternate
// between two buffers by row parity and every warp combines them itself.  Same arithmetic, same bits.
constexpr int kPersistVecs = 4;
constexpr int kPersistMaxWarps = 16;
__host__ __device__ constexpr int pow2_at_least(int n) { return n <= 1 ? 1 : 2 * pow2_at_least((n + 1) / 2); }

template <typename T, int kRecipe, int kWarpsT>
__global__ void __launch_bounds__(32 * kWarpsT) row_quantize_persistent_kernel(const QuantParams p) {
  constexpr int kKeep = kPersistVecs, threads = 32 * kWarpsT;
  __shared__ float red[2][kPersistMaxWarps];
  using O = Ops<T, kRecipe>;
  const int nvec = p.cols / kVec;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Raw<T> cur[kKeep];
  auto load_row = [&](long long r, Raw<T> (&dst)[kKeep]) {
    const T* x = static_cast<const T*>(p.x) + r * p.ldx;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * threads;
      if (v < nvec) {
        dst[i] = load_raw<T>(x + v * kVec);
      } else {
        dst[i].lo = make_uint4(0u, 0u, 0u, 0u);  // zeros: no effect on the absmax, never written
        dst[i].hi = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  };
  long long row = blockIdx.x;
  int parity = 0;
  if (row < p.rows) load_row(row, cur);
  for (; row < p.rows; row += gridDim.x) {
    Raw<T> nxt[kKeep];
    const long long next_row = row + gridDim.x;
    if (next_row < p.rows) load_row(next_row, nxt);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) amax = max_nan(amax, O::absmax(cur[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[parity][warp] = amax;
    __syncthreads();  // the only barrier of the row
    constexpr int kSlots = pow2_at_least(kWarpsT);
    const int src = lane & (kSlots - 1);  // every group of kSlots lanes combines the same slots
    amax = src < kWarpsT ? red[parity][src] : 0.0f;
#pragma unroll
    for (int o = kSlots / 2; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    parity ^= 1;
    float mult, scale;
    if constexpr (kRecipe == kRecipeOperator) {
      const float c = max_nan(amax, Conv<T>::rnd(1e-12f));
      mult = Conv<T>::rnd(__fmul_rn(Conv<T>::rnd(__fdiv_rn(1.0f, c)), 448.0f));
      if constexpr (std::is_same<T, __half>::value) mult = min_nan(mult, 65504.0f);
      scale = Conv<T>::rnd(__fdiv_rn(1.0f, mult));
    } else {
      scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
      mult = scale;  // used as the divisor
    }
    if (threadIdx.x == 0) p.scale[row] = scale;
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * threads;
      if (v < nvec) *reinterpret_cast<uint2*>(q + v * kVec) = O::codes(cur[i], mult);
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) cur[i] = nxt[i];
  }
}

// Short rows (at most 2560 elements, aligned, a multiple of 8 long): one warp per row, eight rows per CTA.
// The absmax is a warp reduction, so no thread ever waits at a block barrier.  Same arithmetic, same bits.
constexpr int kShortRowVecs = 10;  // vectors of 8 elements per lane: 32 * 8 * 10 = 2560 elements
template <typename T, int kRecipe>
__global__ void __launch_bounds__(kThreads) row_quantize_short_rows_kernel(const QuantParams p) {
  using O = Ops<T, kRecipe>;
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
  if (row >= p.rows) return;  // whole warps leave together: no barrier follows
  const T* x = static_cast<const T*>(p.x) + row * p.ldx;
  uint8_t* q = p.q + row * p.ldq;
  const int nvec = p.cols / kVec;
  Raw<T> keep[kShortRowVecs];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < kShortRowVecs; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) keep[i] = load_raw<T>(x + v * kVec);
  }
#pragma unroll
  for (int i = 0; i < kShortRowVecs; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) amax = max_nan(amax, O::absmax(keep[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float mult, scale;
  if constexpr (kRecipe == kRecipeOperator) {
    const float c = max_nan(amax, Conv<T>::rnd(1e-12f));
    mult = Conv<T>::rnd(__fmul_rn(Conv<T>::rnd(__fdiv_rn(1.0f, c)), 448.0f));
    if constexpr (std::is_same<T, __half>::value) mult = min_nan(mult, 65504.0f);
    scale = Conv<T>::rnd(__fdiv_rn(1.0f, mult));
  } else {
    scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
    mult = scale;  // used as the divisor
  }
  if (lane == 0) p.scale[row] = scale;
#pragma unroll
  for (int i = 0; i < kShortRowVecs; ++i) {
    const int v = lane + i * 32;
    if (v < nvec) *reinterpret_cast<uint2*>(q + v * kVec) = O::codes(keep[i], mult);
  }
}

template <typename T, int kRecipe, int kWarpsT>
cudaError_t launch_persistent_t(const QuantParams& p, cudaStream_t stream) {
  static std::atomic<int> ctas_per_device[64] = {};
  constexpr int threads = 32 * kWarpsT;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  int ctas = dev < 64 ? ctas_per_device[dev].load() : 0;
  if (ctas == 0) {
    int sms = 0, per_sm = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, row_quantize_persistent_kernel<T, kRecipe, kWarpsT>,
                                                        threads, 0);
    if (err != cudaSuccess) return err;
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    if (dev < 64) ctas_per_device[dev] = ctas;
  }
  const long long grid = p.rows < ctas ? p.rows : ctas;
  row_quantize_persistent_kernel<T, kRecipe, kWarpsT><<<static_cast<unsigned>(grid), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <typename T, int kRecipe, int kWarpsT = 3>
cudaError_t launch_persistent(int warps, const QuantParams& p, cudaStream_t stream) {
  if constexpr (kWarpsT > kPersistMaxWarps) {
    return cudaErrorInvalidValue;
  } else {
    if (warps == kWarpsT) return launch_persistent_t<T, kRecipe, kWarpsT>(p, stream);
    return launch_persistent<T, kRecipe, kWarpsT + 1>(warps, p, stream);
  }
}

template <typename T, int kRecipe>
cudaError_t launch_recipe(const QuantParams& p, cudaStream_t stream) {
  // rows of 2561..16384 elements, aligned, a multiple of 8 long: the persistent kernel (shorter rows: a warp per row)
  if (p.vector_ok && p.cols % kVec == 0 && p.cols > 2560 && p.cols <= kPersistMaxWarps * 32 * kPersistVecs * kVec) {
    return launch_persistent<T, kRecipe>((p.cols + 1023) / 1024, p, stream);
  }
  if (p.vector_ok && p.cols % kVec == 0 && p.cols <= 32 * kVec * kShortRowVecs && p.rows >= 64) {
    const long long ctas = (p.rows + kThreads / 32 - 1) / (kThreads / 32);
    row_quantize_short_rows_kernel<T, kRecipe><<<static_cast<unsigned>(ctas), kThreads, 0, stream>>>(p);
    return cudaGetLastError();
  }
  const dim3 grid(static_cast<unsigned>(p.rows), 1, 1);
  row_quantize_kernel<T, kRecipe><<<grid, kThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

// 128x128 block quantiser (the operand format of the block-scaled GEMM): one CTA per block, one pass.
//   blockmax = max |x| over the block (rows / columns beyond the matrix count as zeros), clamped below at T(1e-12);
//   mult = (1 / float(blockmax)) * 448 in fp32 (1 where that is infinite);  q = e4m3(float(x) * mult): no clamp is
//   needed, |x * mult| <= 448 (1 + 2^-23) by construction, so the saturating hardware conversion never saturates;
//   the scale handed to the GEMM is 1 / mult.
// Thread t owns the 8 columns [8 (t % 16), +8) of the rows t / 16 + 16 i, i = 0..7, so that a warp reads two
// whole rows of the block (2 x 256 contiguous bytes of a 16-bit type) per instruction; interior, 16-byte aligned
// blocks use vector accesses, edge blocks element accesses.
template <typename T>
__global__ void __launch_bounds__(kThreads) block_quantize_kernel(const BlockQuantParams p) {
  __shared__ float red[kThreads / 32];
  const int bk = blockIdx.x, bm = blockIdx.y;
  const int r0 = threadIdx.x >> 4;
  const int c0 = (threadIdx.x & 15) * kVec;
  const long long row0 = static_cast<long long>(bm) * 128 + r0;
  const long long col = static_cast<long long>(bk) * 128 + c0;
  const bool interior = p.vector_ok && (bm + 1) * 128ll <= p.rows && (bk + 1) * 128ll <= p.cols;
  const T* x = static_cast<const T*>(p.x) + row0 * p.ldx + col;
  uint8_t* q = p.q + row0 * p.ldq + col;

  if constexpr (sizeof(T) == 2) {
    if (interior) {
      // 16-bit input, whole block: the 64 values stay packed (32 registers instead of 64, so twice as many CTAs are
      // resident and in flight), |x| and max work on pairs; same results as the general path below
      Raw<T> raw[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) raw[i] = load_raw<T>(x + 16ll * i * p.ldx);
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_nan(amax, Ops<T, kRecipeFp32>::absmax(raw[i]));
      amax = block_max(amax, red);
      float mult = __fmul_rn(__fdiv_rn(1.0f, max_nan(amax, Conv<T>::rnd(1e-12f))), 448.0f);
      if (isinf(mult)) mult = 1.0f;
      if (threadIdx.x == 0) p.scale[static_cast<long long>(bm) * p.ld_scale + bk] = __fdiv_rn(1.0f, mult);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const T* h = reinterpret_cast<const T*>(&raw[i].lo);
        uint32_t w[2];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(__fmul_rn(Conv<T>::up(h[4 * g]), mult), __fmul_rn(Conv<T>::up(h[4 * g + 1]), mult)), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(__fmul_rn(Conv<T>::up(h[4 * g + 2]), mult), __fmul_rn(Conv<T>::up(h[4 * g + 3]), mult)), __NV_SATFINITE, __NV_E4M3);
          w[g] = lo | (hi << 16);
        }
        *reinterpret_cast<uint2*>(q + 16ll * i * p.ldq) = make_uint2(w[0], w[1]);
      }
      return;
    }
    // 16-bit input, block on the edge of the matrix (or unaligned rows): element accesses, and the second pass reads
    // the block again (from L1 / L2) instead of keeping 64 fp32 values, so that this rare path does not set the
    // kernel's register count
    float amax = 0.0f;
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
      if (row0 + 16 * i < p.rows) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (col + j < p.cols) amax = max_nan(amax, fabsf(Conv<T>::up(x[16ll * i * p.ldx + j])));
        }
      }
    }
    amax = block_max(amax, red);
    float mult = __fmul_rn(__fdiv_rn(1.0f, max_nan(amax, Conv<T>::rnd(1e-12f))), 448.0f);
    if (isinf(mult)) mult = 1.0f;
    if (threadIdx.x == 0) p.scale[static_cast<long long>(bm) * p.ld_scale + bk] = __fdiv_rn(1.0f, mult);
#pragma unroll 1
    for (int i = 0; i < 8; ++i) {
      if (row0 + 16 * i < p.rows) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (col + j < p.cols) {
            q[16ll * i * p.ldq + j] = to_e4m3(__fmul_rn(Conv<T>::up(x[16ll * i * p.ldx + j]), mult));
          }
        }
      }
    }
    return;
  }

  float v[8][8];
  if (interior) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const Raw<T> raw = load_raw<T>(x + 16ll * i * p.ldx);
      if constexpr (sizeof(T) == 4) {
        const float* a = reinterpret_cast<const float*>(&raw.lo);
        const float* b = reinterpret_cast<const float*>(&raw.hi);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[i][j] = a[j];
          v[i][4 + j] = b[j];
        }
      } else {
        const T* h = reinterpret_cast<const T*>(&raw.lo);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = Conv<T>::up(h[j]);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = (row0 + 16 * i < p.rows && col + j < p.cols) ? Conv<T>::up(x[16ll * i * p.ldx + j]) : 0.0f;
      }
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = max_nan(amax, fabsf(v[i][j]));
  }
  amax = block_max(amax, red);
  // torch evaluates `448 / blockmax` as reciprocal(blockmax) * 448: two roundings
  float mult = __fmul_rn(__fdiv_rn(1.0f, max_nan(amax, Conv<T>::rnd(1e-12f))), 448.0f);
  if (isinf(mult)) mult = 1.0f;
  if (threadIdx.x == 0) p.scale[static_cast<long long>(bm) * p.ld_scale + bk] = __fdiv_rn(1.0f, mult);

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (interior) {
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float* a = v[i] + 4 * h;
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[0], mult), __fmul_rn(a[1], mult)), __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(a[2], mult), __fmul_rn(a[3], mult)), __NV_SATFINITE, __NV_E4M3);
        w[h] = lo | (hi << 16);
      }
      *reinterpret_cast<uint2*>(q + 16ll * i * p.ldq) = make_uint2(w[0], w[1]);
    } else if (row0 + 16 * i < p.rows) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (col + j < p.cols) {
          q[16ll * i * p.ldq + j] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fmul_rn(v[i][j], mult), __NV_SATFINITE, __NV_E4M3));
        }
      }
    }
  }
}

template <typename T>
cudaError_t launch_block_t(const BlockQuantParams& p, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>((p.cols + 127) / 128), static_cast<unsigned>((p.rows + 127) / 128), 1);
  block_quantize_kernel<T><<<grid, kThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launch_t(const QuantParams& p, cudaStream_t stream) {
  if (p.recipe == kRecipeOperator) return launch_recipe<T, kRecipeOperator>(p, stream);
  return launch_recipe<T, kRecipeFp32>(p, stream);
}

}  // namespace

cudaError_t launch_row_quantize(const QuantParams& p, cudaStream_t stream) {
  switch (p.dtype) {
    case kQuantBf16: return launch_t<__nv_bfloat16>(p, stream);
    case kQuantFp16: return launch_t<__half>(p, stream);
    case kQuantFp32: return launch_t<float>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_block_quantize(const BlockQuantParams& p, cudaStream_t stream) {
  switch (p.dtype) {
    case kQuantBf16: return launch_block_t<__nv_bfloat16>(p, stream);
    case kQuantFp16: return launch_block_t<__half>(p, stream);
    case kQuantFp32: return launch_block_t<float>(p, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace b200fp8
