// Producer + rowwise e4m3 quantiser in one pass over HBM: the activation that feeds the FP8 GEMM is
// computed from its bf16 inputs, quantised and written as e4m3 bytes plus one fp32 scale per row,
// without the bf16 activation ever being stored.  Two producers:
//
//   kProducerRmsNorm   y[k] = x[k] * rsqrt(mean_k(x^2) + eps) * weight[k]
//   kProducerSiluMul   y[k] = x1[k] / (1 + exp(-x1[k])) * x2[k]
//
// All arithmetic is fp32 on the bf16 inputs.  The row statistics (1/rms, the scale and its
// reciprocal) use IEEE divide and square root; per element the SiLU uses the hardware exponential
// and reciprocal (ex2.approx / rcp.approx, about 2 ulp) and the quantisation multiplies by the
// reciprocal scale - the kernel is bandwidth-bound only if it spends a dozen instructions per element.
// With `round_bf16` y is rounded to bf16 before the quantisation, which is what a two-kernel
// pipeline (producer writes bf16, quantiser reads it) computes.  Quantisation:
//   scale = max(rowabsmax(y), 1e-12) / 448;   q = e4m3(clamp(y * (1 / scale), +-448));   scale is returned.
//
// A CTA owns a row; what it read stays in registers between the reductions and the quantisation
// (RMS norm: the packed bf16 row, y is recomputed; SiLU-mul: y in fp32), for rows up to 16384 columns;
// longer rows recompute the overflow from the inputs.  The common RMS-norm case (aligned rows of at most
// 8192 columns, no bf16 rounding) runs a persistent form that keeps the weight vector in registers.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "kernels.h"
#include "nanmax.cuh"

namespace b200fp8 {
namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;      // bf16 elements per 16-byte load

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ float silu_mul(float a, float b) { return __fdividef(a, 1.0f + __expf(-a)) * b; }

template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = kMax ? max_nan(v, other) : v + other;
  }
  __syncthreads();  // the previous reduction's readers are done with smem
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = smem[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) r = kMax ? max_nan(r, smem[w]) : r + smem[w];
  return r;
}

// sum of `s` and max of `m` over the block in one round of barriers
__device__ __forceinline__ void block_reduce_sum_max(float& s, float& m, float* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) {
    smem[threadIdx.x >> 5] = s;
    smem[kThreads / 32 + (threadIdx.x >> 5)] = m;
  }
  __syncthreads();
  s = smem[0];
  m = smem[kThreads / 32];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) {
    s += smem[w];
    m = max_nan(m, smem[kThreads / 32 + w]);
  }
}

__device__ __forceinline__ uint2 codes8(const float (&y)[8], float inv_scale) {
  uint32_t w[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * i] * inv_scale, y[4 * i + 1] * inv_scale),
                                                 __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(y[4 * i + 2] * inv_scale, y[4 * i + 3] * inv_scale),
                                                 __NV_SATFINITE, __NV_E4M3);
    w[i] = lo | (hi << 16);
  }
  return make_uint2(w[0], w[1]);
}

// kKeep: vectors of 8 elements a thread keeps in registers (rows up to 256 * 8 * kKeep columns stay on chip)
template <int kProducer, int kKeep>
__global__ void __launch_bounds__(kThreads) fused_row_quantize_kernel(const FusedQuantParams p) {
  __shared__ float red[2 * (kThreads / 32)];
  const long long row = blockIdx.x;
  const __nv_bfloat16* x1 = static_cast<const __nv_bfloat16*>(p.x1) + row * p.ld1;
  // second operand: the weight vector (RMS norm, shared by all rows) or this row of x2 (SiLU-mul)
  const __nv_bfloat16* x2 = static_cast<const __nv_bfloat16*>(p.x2) + (kProducer == kProducerSiluMul ? row * p.ld2 : 0);
  uint8_t* q = p.q + row * p.ldq;
  const int cols = p.cols;
  const int vec_cols = p.vector_ok ? (cols / kVec) * kVec : 0;
  const int nvec = vec_cols / kVec;
  const bool round_y = p.round_bf16 != 0;

  // what stays in registers: the packed row (RMS norm) or y (SiLU-mul)
  uint4 raw[kProducer == kProducerRmsNorm ? kKeep : 1];
  float keep[kProducer == kProducerSiluMul ? kKeep : 1][8];

  // RMS norm without the bf16 rounding: |y| = |x w| / rms up to the last bit, so the sum of squares and the
  // largest |x w| are reduced together and the row needs two block reductions' worth of waiting less.
  float inv_rms = 1.0f;
  float amax_xw = 0.0f;
  const bool one_pass_stats = kProducer == kProducerRmsNorm && !round_y;
  if constexpr (kProducer == kProducerRmsNorm) {
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nvec) raw[i] = *reinterpret_cast<const uint4*>(x1 + v * kVec);
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nvec) {
        float a[8], b[8];
        unpack8(raw[i], a);
        unpack8(*reinterpret_cast<const uint4*>(x2 + v * kVec), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss = fmaf(a[j], a[j], ss);
          amax_xw = max_nan(amax_xw, fabsf(a[j] * b[j]));
        }
      }
    }
    for (int v = threadIdx.x + kKeep * kThreads; v < nvec; v += kThreads) {
      float a[8], b[8];
      unpack8(*reinterpret_cast<const uint4*>(x1 + v * kVec), a);
      unpack8(*reinterpret_cast<const uint4*>(x2 + v * kVec), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ss = fmaf(a[j], a[j], ss);
        amax_xw = max_nan(amax_xw, fabsf(a[j] * b[j]));
      }
    }
    for (int c = vec_cols + threadIdx.x; c < cols; c += kThreads) {
      const float a = __bfloat162float(x1[c]);
      ss = fmaf(a, a, ss);
      amax_xw = max_nan(amax_xw, fabsf(a * __bfloat162float(x2[c])));
    }
    if (one_pass_stats) {
      block_reduce_sum_max(ss, amax_xw, red);
    } else {
      ss = block_reduce<false>(ss, red);
    }
    inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(ss, static_cast<float>(cols)) + p.eps));
  }

  auto produce = [&](float a, float b) {
    const float y = kProducer == kProducerRmsNorm ? (a * inv_rms) * b : silu_mul(a, b);
    return round_y ? bf16_round(y) : y;
  };
  auto produce8 = [&](const uint4& ra, const uint4& rb, float (&y)[8]) {
    float a[8], b[8];
    unpack8(ra, a);
    unpack8(rb, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = produce(a[j], b[j]);
  };
  auto absmax8 = [](const float (&y)[8], float m) {
#pragma unroll
    for (int j = 0; j < 8; ++j) m = max_nan(m, fabsf(y[j]));
    return m;
  };

  // pass 1: absmax of y
  float amax = 0.0f;
  if (one_pass_stats) {
    amax = amax_xw * inv_rms;
  } else {
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nvec) {
        const uint4 rb = *reinterpret_cast<const uint4*>(x2 + v * kVec);
        if constexpr (kProducer == kProducerRmsNorm) {
          float y[8];
          produce8(raw[i], rb, y);
          amax = absmax8(y, amax);
        } else {
          produce8(*reinterpret_cast<const uint4*>(x1 + v * kVec), rb, keep[i]);
          amax = absmax8(keep[i], amax);
        }
      }
    }
    for (int v = threadIdx.x + kKeep * kThreads; v < nvec; v += kThreads) {  // longer rows: not kept
      float y[8];
      produce8(*reinterpret_cast<const uint4*>(x1 + v * kVec), *reinterpret_cast<const uint4*>(x2 + v * kVec), y);
      amax = absmax8(y, amax);
    }
    for (int c = vec_cols + threadIdx.x; c < cols; c += kThreads) {
      amax = max_nan(amax, fabsf(produce(__bfloat162float(x1[c]), __bfloat162float(x2[c]))));
    }
    amax = block_reduce<true>(amax, red);
  }

  const float scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
  const float inv_scale = __fdiv_rn(1.0f, scale);
  if (threadIdx.x == 0) p.scale[row] = scale;

  // pass 2: quantise from registers (re-reading only what did not fit; the weight vector comes from L1)
#pragma unroll
  for (int i = 0; i < kKeep; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) {
      if constexpr (kProducer == kProducerRmsNorm) {
        float y[8];
        produce8(raw[i], *reinterpret_cast<const uint4*>(x2 + v * kVec), y);
        *reinterpret_cast<uint2*>(q + v * kVec) = codes8(y, inv_scale);
      } else {
        *reinterpret_cast<uint2*>(q + v * kVec) = codes8(keep[i], inv_scale);
      }
    }
  }
  for (int v = threadIdx.x + kKeep * kThreads; v < nvec; v += kThreads) {
    float y[8];
    produce8(*reinterpret_cast<const uint4*>(x1 + v * kVec), *reinterpret_cast<const uint4*>(x2 + v * kVec), y);
    *reinterpret_cast<uint2*>(q + v * kVec) = codes8(y, inv_scale);
  }
  for (int c = vec_cols + threadIdx.x; c < cols; c += kThreads) {
    const float y = produce(__bfloat162float(x1[c]), __bfloat162float(x2[c]));
    q[c] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(y * inv_scale, __NV_SATFINITE, __NV_E4M3));
  }
}

// RMS norm, persistent form: a CTA walks over rows blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its
// slice of the weight vector unpacked in registers for all of them; the next row is requested from memory
// before the current one is reduced.  Same arithmetic as the kernel above without the bf16 rounding of y.
// Needs 16-byte aligned rows, cols a multiple of 8 and at most 256 * 8 * kKeep (kKeep <= 4: the weight slice,
// this row and the next one have to fit in registers).
template <int kKeep>
__global__ void __launch_bounds__(kThreads) rms_norm_quantize_persistent_kernel(const FusedQuantParams p) {
  __shared__ float red[2 * (kThreads / 32)];
  const __nv_bfloat16* wvec = static_cast<const __nv_bfloat16*>(p.x2);
  const int nvec = p.cols / kVec;
  float w[kKeep][8];
#pragma unroll
  for (int i = 0; i < kKeep; ++i) {
    const int v = threadIdx.x + i * kThreads;
    if (v < nvec) {
      unpack8(*reinterpret_cast<const uint4*>(wvec + v * kVec), w[i]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) w[i][j] = 0.0f;
    }
  }
  uint4 cur[kKeep];
  long long row = blockIdx.x;
  if (row < p.rows) {
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x1) + row * p.ld1;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      cur[i] = v < nvec ? *reinterpret_cast<const uint4*>(x + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  for (; row < p.rows; row += gridDim.x) {
    uint4 nxt[kKeep];
    const long long next_row = row + gridDim.x;
    if (next_row < p.rows) {  // in flight while this row is reduced and written
      const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x1) + next_row * p.ld1;
#pragma unroll
      for (int i = 0; i < kKeep; ++i) {
        const int v = threadIdx.x + i * kThreads;
        nxt[i] = v < nvec ? *reinterpret_cast<const uint4*>(x + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    float ss = 0.0f, amax_xw = 0.0f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {  // vectors beyond the row are zeros: they add nothing
      float a[8];
      unpack8(cur[i], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ss = fmaf(a[j], a[j], ss);
        amax_xw = max_nan(amax_xw, fabsf(a[j] * w[i][j]));
      }
    }
    block_reduce_sum_max(ss, amax_xw, red);
    const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(ss, static_cast<float>(p.cols)) + p.eps));
    const float scale = __fdiv_rn(max_nan(amax_xw * inv_rms, 1e-12f), 448.0f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) p.scale[row] = scale;
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nvec) {
        float a[8], y[8];
        unpack8(cur[i], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = (a[j] * inv_rms) * w[i][j];
        *reinterpret_cast<uint2*>(q + v * kVec) = codes8(y, inv_scale);
      }
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) cur[i] = nxt[i];
  }
}

// SiLU-mul, persistent form: the next row of both inputs is in flight while the current one is reduced
// and written.  Same arithmetic as the one-row-per-CTA kernel without the bf16 rounding of y.
template <int kKeep>
__global__ void __launch_bounds__(kThreads) silu_mul_quantize_persistent_kernel(const FusedQuantParams p) {
  __shared__ float red[kThreads / 32];
  const int nvec = p.cols / kVec;
  uint4 cur1[kKeep], cur2[kKeep];
  auto load_row = [&](long long r, uint4 (&a)[kKeep], uint4 (&b)[kKeep]) {
    const __nv_bfloat16* x1 = static_cast<const __nv_bfloat16*>(p.x1) + r * p.ld1;
    const __nv_bfloat16* x2 = static_cast<const __nv_bfloat16*>(p.x2) + r * p.ld2;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      a[i] = v < nvec ? *reinterpret_cast<const uint4*>(x1 + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
      b[i] = v < nvec ? *reinterpret_cast<const uint4*>(x2 + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  long long row = blockIdx.x;
  if (row < p.rows) load_row(row, cur1, cur2);
  for (; row < p.rows; row += gridDim.x) {
    uint4 nxt1[kKeep], nxt2[kKeep];
    const long long next_row = row + gridDim.x;
    if (next_row < p.rows) load_row(next_row, nxt1, nxt2);
    float y[kKeep][8];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {  // vectors beyond the row are zeros: silu(0) * 0 = 0
      float a[8], b[8];
      unpack8(cur1[i], a);
      unpack8(cur2[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        y[i][j] = silu_mul(a[j], b[j]);
        amax = max_nan(amax, fabsf(y[i][j]));
      }
    }
    amax = block_reduce<true>(amax, red);
    const float scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) p.scale[row] = scale;
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * kThreads;
      if (v < nvec) *reinterpret_cast<uint2*>(q + v * kVec) = codes8(y[i], inv_scale);
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      cur1[i] = nxt1[i];
      cur2[i] = nxt2[i];
    }
  }
}

template <typename Kernel>
cudaError_t launch_persistent(Kernel kernel, std::atomic<int>* ctas_per_device, const FusedQuantParams& p, cudaStream_t stream) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  int ctas = dev < 64 ? ctas_per_device[dev].load() : 0;
  if (ctas == 0) {
    int sms = 0, per_sm = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0);
    if (err != cudaSuccess) return err;
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    if (dev < 64) ctas_per_device[dev] = ctas;
  }
  const long long grid = p.rows < ctas ? p.rows : ctas;
  kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int kKeep>
cudaError_t launch_rms_persistent(const FusedQuantParams& p, cudaStream_t stream) {
  static std::atomic<int> ctas_per_device[64] = {};
  return launch_persistent(rms_norm_quantize_persistent_kernel<kKeep>, ctas_per_device, p, stream);
}

template <int kKeep>
cudaError_t launch_silu_persistent(const FusedQuantParams& p, cudaStream_t stream) {
  static std::atomic<int> ctas_per_device[64] = {};
  return launch_persistent(silu_mul_quantize_persistent_kernel<kKeep>, ctas_per_device, p, stream);
}

template <int kProducer>
cudaError_t launch_producer(const FusedQuantParams& p, cudaStream_t stream) {
  const dim3 grid(static_cast<unsigned>(p.rows), 1, 1);
  if (p.cols <= 2 * kThreads * kVec) {
    fused_row_quantize_kernel<kProducer, 2><<<grid, kThreads, 0, stream>>>(p);
  } else if (p.cols <= 4 * kThreads * kVec) {
    fused_row_quantize_kernel<kProducer, 4><<<grid, kThreads, 0, stream>>>(p);
  } else {
    fused_row_quantize_kernel<kProducer, 8><<<grid, kThreads, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fused_row_quantize(const FusedQuantParams& p, cudaStream_t stream) {
  if (p.producer == kProducerRmsNorm && !p.round_bf16 && p.vector_ok && p.cols % kVec == 0) {
    if (p.cols <= 2 * kThreads * kVec) return launch_rms_persistent<2>(p, stream);
    if (p.cols <= 4 * kThreads * kVec) return launch_rms_persistent<4>(p, stream);
  }
  // (rows of up to 2560 columns give a thread too little to do between two block reductions: measured slower)
  if (p.producer == kProducerSiluMul && !p.round_bf16 && p.vector_ok && p.cols % kVec == 0 && p.cols > 2560) {
    if (p.cols <= 2 * kThreads * kVec) return launch_silu_persistent<2>(p, stream);
    if (p.cols <= 4 * kThreads * kVec) return launch_silu_persistent<4>(p, stream);
  }
  if (p.producer == kProducerRmsNorm) return launch_producer<kProducerRmsNorm>(p, stream);
  if (p.producer == kProducerSiluMul) return launch_producer<kProducerSiluMul>(p, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200fp8
