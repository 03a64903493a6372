// CUDA-core FP8 rowwise GEMM: byte loads, software-visible e4m3 decode, fp32 FMA in ascending k.
// It accepts any pointer alignment and any leading dimension, which the TMA-fed tcgen05 kernels
// do not, and it is the on-GPU cross-check for sizes where a host check would take minutes.
// It is two orders of magnitude slower than the tensor-core kernels and is never chosen for a
// shape those kernels accept.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

constexpr int kTile = 64;   // output tile edge per block
constexpr int kStepK = 32;  // k elements staged per iteration

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(__half(h));
}

__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
  __shared__ float xs[kStepK][kTile + 1];
  __shared__ float ws[kStepK][kTile + 1];
  const int tx = threadIdx.x & 15;  // 4 output columns each
  const int ty = threadIdx.x >> 4;  // 4 output rows each
  const int m0 = blockIdx.y * kTile;
  const int n0 = blockIdx.x * kTile;

  float acc[4][4] = {};
  for (int k0 = 0; k0 < p.K; k0 += kStepK) {
    for (int i = threadIdx.x; i < kTile * kStepK; i += 256) {
      const int r = i / kStepK;
      const int k = i - r * kStepK;
      const bool k_ok = k0 + k < p.K;
      xs[k][r] = (k_ok && m0 + r < p.M) ? e4m3_to_float(p.xq[static_cast<long long>(m0 + r) * p.ldx + k0 + k]) : 0.0f;
      ws[k][r] = (k_ok && n0 + r < p.N) ? e4m3_to_float(p.wq[static_cast<long long>(n0 + r) * p.ldw + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kStepK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = xs[k][ty * 4 + i];
        b[i] = ws[k][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    const float sx = p.x_scale[m];
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j] * (sx * p.w_scale[n]);
      if (p.bias != nullptr) v += __bfloat162float(p.bias[n]);
      if (p.out_fp16) {
        reinterpret_cast<__half*>(p.y)[static_cast<long long>(m) * p.ldy + n] = __float2half_rn(v);
      } else {
        p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

// Self-test of the bounded wait every tensor-core kernel is built on: one CTA waits on an mbarrier
// that nothing will ever arrive on.  The wait must run out after `limit_ns`, record its site in the
// status word and let the kernel end normally.
constexpr uint32_t kSiteSelfTest = 0x7E57;

__global__ void wait_timeout_selftest_kernel(uint32_t* status, unsigned long long limit_ns) {
  __shared__ unsigned long long barrier_storage;
  __shared__ uint32_t abort_flag;
  const uint32_t bar = smem_u32(&barrier_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  // every thread waits; the first to run out of time raises the flag, the others leave on seeing it
  mbar_wait<false>(bar, 0u, &abort_flag, status, kSiteSelfTest, limit_ns);
}

}  // namespace

cudaError_t launch_wait_timeout_selftest(uint32_t* status, unsigned long long limit_ns, cudaStream_t stream) {
  wait_timeout_selftest_kernel<<<1, 64, 0, stream>>>(status, limit_ns);
  return cudaGetLastError();
}

cudaError_t launch_gemm_simt(const SimtParams& p, cudaStream_t stream) {
  const dim3 grid((p.N + kTile - 1) / kTile, (p.M + kTile - 1) / kTile, 1);
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace b200fp8
