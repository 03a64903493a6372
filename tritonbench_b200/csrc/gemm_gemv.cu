// FP8 rowwise GEMM for one to four tokens (M <= 4): a GEMV on the CUDA cores.
//
//   Y[m,n] = bf16( (sum_k X[m,k] * W[n,k]) * x_scale[m] * w_scale[n] (+ bias[n]) )
//
// With so few rows of X the work is reading W once from HBM.  Every warp owns whole rows of W and streams them
// with 128-bit loads, four per lane in flight (512 contiguous bytes per warp and load), 1024 threads per SM:
//   * X is converted once per CTA from e4m3 to fp16 (exact) into shared memory, laid out so that the two
//     16-byte reads a lane makes per W load are free of bank conflicts;
//   * W goes e4m3x2 -> f16x2 (one cvt per pair) and each product is accumulated in fp32 by a mixed-precision
//     fma (fma.rn.f32.f16: the fp16 x fp16 product is exact, the sum is rounded once to fp32, as an fp32 FMA
//     on the converted values would);
//   * a warp-shuffle reduction finishes the row; lane 0 scales, adds the bias, rounds and stores.
// Rows are dealt so that every warp gets the same number of them (the grid is sized from N), because a last
// round with a few busy warps would be latency-bound.
//
// Measured on a B200 at N = 28672, K = 8192: 48.7 / 67.3 / 94.9 us for one / two / four tokens against 42.8-43.1 us
// for the tensor-core decode kernel, although a kernel that only READS W with the same loads takes 36.9 us: the
// conversions (eight cvt per 16 bytes) and the multiply-adds (sixteen per 16 bytes and token, fp32 accumulation)
// need more issue slots than HBM leaves time for - at 6.4 TB/s an SM receives 23 bytes per cycle.  The library's
// `auto` choice therefore never takes this kernel; it stays as variant `gemv`, correct and tested.
#include <cuda_fp8.h>

#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

constexpr int kGemvThreads = 512;   // 16 warps
constexpr int kGemvInFlight = 4;    // 128-bit loads per lane in flight
constexpr int kChunkElems = 16;     // e4m3 values per 128-bit load
constexpr int kBlockElems = 32 * kChunkElems;  // 512 values: what a warp covers with one load

// 16 e4m3 bytes -> 8 packed fp16 pairs, in order
__device__ __forceinline__ void e4m3x16_to_f16(const uint4& v, uint32_t (&h)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xFFFFu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    h[2 * i] = static_cast<uint32_t>(lo.x) | (static_cast<uint32_t>(lo.y) << 16);
    h[2 * i + 1] = static_cast<uint32_t>(hi.x) | (static_cast<uint32_t>(hi.y) << 16);
  }
}

// acc += a.lo * b.lo + a.hi * b.hi with fp32 accumulation (two mixed-precision FMAs on packed fp16 pairs)
__device__ __forceinline__ void fma_f16x2_f32(float& acc, uint32_t a, uint32_t b) {
  asm("{\n"
      ".reg .f16 a0, a1, b0, b1;\n"
      "mov.b32 {a0, a1}, %1;\n"
      "mov.b32 {b0, b1}, %2;\n"
      "fma.rn.f32.f16 %0, a0, b0, %0;\n"
      "fma.rn.f32.f16 %0, a1, b1, %0;\n"
      "}\n"
      : "+f"(acc)
      : "r"(a), "r"(b));
}

template <int kTokens>
__global__ void __launch_bounds__(kGemvThreads, 2) gemm_gemv_kernel(const GemvParams p) {
  // X as fp16 in shared memory: [token][block of 512 values][low / high half of a lane's 16 values][lane] x 16 bytes
  extern __shared__ uint4 x_smem[];
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int blocks_k = (p.K + kBlockElems - 1) / kBlockElems;
  const int chunks = p.K / kChunkElems;  // K is a multiple of 16

  if (p.overlap) {
    griddep_launch_dependents();  // the next kernel may take SMs as they become free
    griddep_wait();               // X (and Y) only after the previous kernel has completed
  }
  for (int i = threadIdx.x; i < kTokens * blocks_k * 32; i += kGemvThreads) {
    const int m = i / (blocks_k * 32);
    const int chunk = i - m * blocks_k * 32;  // 16-value chunk of row m
    uint32_t h[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};  // beyond K (and beyond M): zeros, so that 0 x 0 is added
    if (m < p.M && chunk < chunks) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.xq + static_cast<long long>(m) * p.ldx) + chunk);
      e4m3x16_to_f16(v, h);
    }
    const int block = chunk >> 5, l = chunk & 31;
    uint4* dst = x_smem + (static_cast<size_t>(m) * blocks_k + block) * 64 + l;
    dst[0] = make_uint4(h[0], h[1], h[2], h[3]);
    dst[32] = make_uint4(h[4], h[5], h[6], h[7]);
  }
  __syncthreads();

  const int warps_per_cta = kGemvThreads / 32;
  const long long first_row = (static_cast<long long>(blockIdx.x) * warps_per_cta + warp_in_cta) * p.rows_per_warp;
  for (int r = 0; r < p.rows_per_warp; ++r) {
    const long long n = first_row + r;
    if (n >= p.N) break;  // warp-uniform
    const uint4* w_row = reinterpret_cast<const uint4*>(p.wq + n * p.ldw);
    float acc[kTokens];
#pragma unroll
    for (int m = 0; m < kTokens; ++m) acc[m] = 0.0f;
    for (int c0 = 0; c0 < chunks; c0 += 32 * kGemvInFlight) {
      uint4 v[kGemvInFlight];
#pragma unroll
      for (int u = 0; u < kGemvInFlight; ++u) {
        const int c = c0 + u * 32 + lane;
        v[u] = c < chunks ? __ldg(w_row + c) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < kGemvInFlight; ++u) {
        if (c0 + u * 32 < chunks) {  // warp-uniform: this 512-value block exists
          uint32_t wh[8];
          e4m3x16_to_f16(v[u], wh);
          const int block = (c0 >> 5) + u;
#pragma unroll
          for (int m = 0; m < kTokens; ++m) {
            const uint4* xs = x_smem + (static_cast<size_t>(m) * blocks_k + block) * 64 + lane;
            const uint4 xlo = xs[0], xhi = xs[32];
            fma_f16x2_f32(acc[m], wh[0], xlo.x);
            fma_f16x2_f32(acc[m], wh[1], xlo.y);
            fma_f16x2_f32(acc[m], wh[2], xlo.z);
            fma_f16x2_f32(acc[m], wh[3], xlo.w);
            fma_f16x2_f32(acc[m], wh[4], xhi.x);
            fma_f16x2_f32(acc[m], wh[5], xhi.y);
            fma_f16x2_f32(acc[m], wh[6], xhi.z);
            fma_f16x2_f32(acc[m], wh[7], xhi.w);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kTokens; ++m) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
      const float ws = __ldg(p.w_scale + n);
      const float b = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.0f;
#pragma unroll
      for (int m = 0; m < kTokens; ++m) {
        if (m < p.M) {
          const float y = acc[m] * (__ldg(p.x_scale + m) * ws) + b;
          reinterpret_cast<uint16_t*>(p.y)[static_cast<long long>(m) * p.ldy + n] = to_out16(y, p.out_fp16);
        }
      }
    }
  }
}

template <int kTokens>
cudaError_t launch_t(const GemvParams& p, int ctas, size_t smem, cudaStream_t stream) {
  static size_t configured[64] = {};
  static std::mutex mutex;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (dev < 64 && configured[dev] < smem) {
      err = cudaFuncSetAttribute(gemm_gemv_kernel<kTokens>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kGemvMaxSmemBytes));
      if (err != cudaSuccess) return err;
      configured[dev] = kGemvMaxSmemBytes;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_gemv_kernel<kTokens>, p);
}

}  // namespace

GemvPlan make_gemv_plan(long long M, long long N, long long K, int sm_count) {
  GemvPlan pl = {};
  const long long blocks_k = (K + kBlockElems - 1) / kBlockElems;
  const int tokens = M <= 1 ? 1 : (M <= 2 ? 2 : 4);
  pl.tokens = tokens;
  pl.smem_bytes = static_cast<size_t>(tokens) * blocks_k * 64 * sizeof(uint4);
  pl.ok = M >= 1 && M <= kGemvMaxTokens && K % kChunkElems == 0 && pl.smem_bytes <= kGemvMaxSmemBytes;
  // every warp the same number of rows: the fewest rows per warp that two CTAs per SM can cover
  const long long warps_per_cta = kGemvThreads / 32;
  const long long max_warps = 2ll * sm_count * warps_per_cta;
  long long rows_per_warp = (N + max_warps - 1) / max_warps;
  if (rows_per_warp < 1) rows_per_warp = 1;
  pl.rows_per_warp = static_cast<int>(rows_per_warp);
  pl.ctas = static_cast<int>((N + warps_per_cta * rows_per_warp - 1) / (warps_per_cta * rows_per_warp));
  return pl;
}

cudaError_t launch_gemm_gemv(const GemvParams& p_in, const GemvPlan& plan, cudaStream_t stream) {
  if (!plan.ok) return cudaErrorInvalidValue;
  GemvParams p = p_in;
  p.rows_per_warp = plan.rows_per_warp;
  if (plan.tokens == 1) return launch_t<1>(p, plan.ctas, plan.smem_bytes, stream);
  if (plan.tokens == 2) return launch_t<2>(p, plan.ctas, plan.smem_bytes, stream);
  return launch_t<4>(p, plan.ctas, plan.smem_bytes, stream);
}

}  // namespace b200fp8
