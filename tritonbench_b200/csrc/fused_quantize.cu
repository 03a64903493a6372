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
// longer rows recompute the overflow from the inputs.  Aligned rows of up to 16384 columns run persistent forms,
// described where they are defined.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "kernels.h"
#include "nanmax.cuh"

namespace b200fp8 {
namespace {

// These kernels produce activations, never weights.  A decode GEMM launched behind one of them with programmatic
// stream serialization (B200FP8_FLAG_PDL: it may read W, and only W, before its predecessor has completed) may
// therefore start as soon as every CTA here has passed this point: it prefetches W while the quantiser runs and reads
// what the quantiser wrote only after its own griddepcontrol.wait, i.e. after this grid has completed.  Without such
// a dependent the instruction does nothing.  (The plain row and block quantisers, which also quantise weights, do
// not do this.)
__device__ __forceinline__ void let_dependents_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }


constexpr int kThreads = 256;
constexpr int kVec = 8;      // bf16 elements per 16-byte load

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

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
  let_dependents_start();
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

// ---- persistent forms ----
// A CTA walks over rows blockIdx.x, blockIdx.x + gridDim.x, ...; both need 16-byte aligned rows, cols a multiple
// of 8 and at most 256 * 8 * kKeep.

// Two fp32 values in one 64-bit register, multiplied / fused-multiply-added two per instruction (sm_100 packed
// fp32).  Each half rounds as the scalar instruction does, so results do not change.  The values stay in 64-bit
// registers from the bf16 pair to the e4m3 pair, so that no instruction is spent on packing.
using pair_t = unsigned long long;
__device__ __forceinline__ pair_t pack2(float lo, float hi) {
  pair_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(pair_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ pair_t bf16x2_to_pair(uint32_t h) {  // exact: low half first
  pair_t r;
  asm("{\n"
      ".reg .b32 lo, hi;\n"
      "shl.b32 lo, %1, 16;\n"
      "and.b32 hi, %1, 0xffff0000;\n"
      "mov.b64 %0, {lo, hi};\n"
      "}\n"
      : "=l"(r)
      : "r"(h));
  return r;
}
__device__ __forceinline__ pair_t mul2(pair_t a, pair_t b) {
  pair_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ pair_t fma2(pair_t a, pair_t b, pair_t c) {
  pair_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_of(pair_t v) {  // round to nearest even, low half into the low 16 bits
  uint32_t r;
  asm("{\n"
      ".reg .b32 lo, hi;\n"
      "mov.b64 {lo, hi}, %1;\n"
      "cvt.rn.bf16x2.f32 %0, hi, lo;\n"
      "}\n"
      : "=r"(r)
      : "l"(v));
  return r;
}
__device__ __forceinline__ uint32_t e4m3x2_of(pair_t v) {  // saturating, low half into the low byte
  uint16_t r;
  asm("{\n"
      ".reg .b32 lo, hi;\n"
      "mov.b64 {lo, hi}, %1;\n"
      "cvt.rn.satfinite.e4m3x2.f32 %0, hi, lo;\n"
      "}\n"
      : "=h"(r)
      : "l"(v));
  return r;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

// RMS norm.  At 6.5 TB/s an SM has about 14 issue slots per element, which is what the straightforward kernel
// spends (it measured 72 % issue-slot utilisation and 0.82 of the HBM bandwidth), so this one saves instructions
// and waits:
//   * the rows live in a ring in shared memory instead of registers: each thread copies its own 16-byte vectors
//     with cp.async and reads back only what it copied itself, so the ring needs no barrier (cp.async.wait_group is
//     a hardware wait, like a load's); with the rows out of the register file twice as many CTAs fit on an SM;
//   * multiplications go two per instruction, on values that stay in 64-bit registers;
//   * one barrier per row: the warps' partial sums alternate between two buffers by row parity, every warp combines
//     them itself (in a fixed order) and computes the row's scalars.
// The CTA has one warp per 1024 columns (a thread owns four 16-byte vectors of a row), so a thread's work per row
// is the same for every row length up to 16384; its slice of the weight vector stays unpacked in registers for
// all the rows the CTA walks over.  Same arithmetic per element as the one-row-per-CTA kernel without the bf16
// rounding of y.
constexpr int kRmsStages = 3;       // this row and the two after it
constexpr int kRmsVecs = 4;         // 16-byte vectors of a row per thread
constexpr int kRmsMaxWarps = 16;     // rows of at most 16 * 32 * 4 * 8 = 16384 columns
__host__ __device__ constexpr int silu_ctas_per_sm(int warps) { return warps <= 24 ? 24 / warps : 1; }  // 24 warps of these per SM: 85 registers a thread
__host__ __device__ constexpr int rms_ctas_per_sm(int warps) { return 32 / warps; }                   // 32 warps of these per SM
__host__ __device__ constexpr int rms_pow2_at_least(int n) { return n <= 1 ? 1 : 2 * rms_pow2_at_least((n + 1) / 2); }

template <int kWarpsT>  // the CTA size is a compile-time constant: index arithmetic costs issue slots too
__global__ void __launch_bounds__(32 * kWarpsT, rms_ctas_per_sm(kWarpsT)) rms_norm_quantize_persistent_kernel(const FusedQuantParams p) {
  let_dependents_start();
  extern __shared__ uint4 ring[];              // [kRmsStages][kRmsVecs][threads]
  __shared__ float part[2][2 * kRmsMaxWarps];  // by row parity; per warp: sum of squares, max |x w|
  const __nv_bfloat16* wvec = static_cast<const __nv_bfloat16*>(p.x2);
  const int nvec = p.cols / kVec;
  constexpr int threads = 32 * kWarpsT, warps = kWarpsT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pair_t w[kRmsVecs][4];
#pragma unroll
  for (int k = 0; k < kRmsVecs; ++k) {
    const int v = threadIdx.x + k * threads;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (v < nvec) raw = *reinterpret_cast<const uint4*>(wvec + v * kVec);
    w[k][0] = bf16x2_to_pair(raw.x);
    w[k][1] = bf16x2_to_pair(raw.y);
    w[k][2] = bf16x2_to_pair(raw.z);
    w[k][3] = bf16x2_to_pair(raw.w);
  }
  auto request = [&](long long r, int stage) {  // one group per call, also when there is no such row
    if (r < p.rows) {
      const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x1) + r * p.ld1;
#pragma unroll
      for (int k = 0; k < kRmsVecs; ++k) {
        const int v = threadIdx.x + k * threads;
        if (v < nvec) cp_async_16(smem_addr(&ring[(stage * kRmsVecs + k) * threads + threadIdx.x]), x + v * kVec);
      }
    }
    cp_async_commit();
  };
  long long row = blockIdx.x;
#pragma unroll
  for (int s = 0; s < kRmsStages - 1; ++s) request(row + static_cast<long long>(s) * gridDim.x, s);
  int stage = 0, parity = 0;
  for (; row < p.rows; row += gridDim.x) {
    // refill the stage this thread emptied one row ago, then wait for this row: the newest kRmsStages - 1 groups may
    // still be on their way
    request(row + static_cast<long long>(kRmsStages - 1) * gridDim.x, stage == 0 ? kRmsStages - 1 : stage - 1);
    cp_async_wait<kRmsStages - 1>();
    pair_t ss = pack2(0.0f, 0.0f);
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < kRmsVecs; ++k) {
      const int v = threadIdx.x + k * threads;
      if (v < nvec) {  // vectors beyond the row add nothing
        const uint4 raw = ring[(stage * kRmsVecs + k) * threads + threadIdx.x];
        const uint32_t h[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const pair_t a = bf16x2_to_pair(h[j]);
          ss = fma2(a, a, ss);
          float lo, hi;
          unpack2(mul2(a, w[k][j]), lo, hi);
          amax = max_nan(amax, fabsf(lo));
          amax = max_nan(amax, fabsf(hi));
        }
      }
    }
    float s_lo, s_hi;
    unpack2(ss, s_lo, s_hi);
    float s = s_lo + s_hi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    if (lane == 0) {
      part[parity][warp] = s;
      part[parity][kRmsMaxWarps + warp] = amax;
    }
    __syncthreads();  // the only barrier of the row
    constexpr int kSlots = rms_pow2_at_least(warps);
    const int src = lane & (kSlots - 1);  // every group of kSlots lanes combines the same slots
    float t = src < warps ? part[parity][src] : 0.0f;
    float m = src < warps ? part[parity][kRmsMaxWarps + src] : 0.0f;
#pragma unroll
    for (int o = kSlots / 2; o > 0; o >>= 1) {  // a fixed order: the result does not depend on timing
      t += __shfl_xor_sync(0xffffffffu, t, o);
      m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
    }
    parity ^= 1;
    const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(p.cols)) + p.eps));
    const float scale = __fdiv_rn(max_nan(m * inv_rms, 1e-12f), 448.0f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) p.scale[row] = scale;
    const pair_t inv_rms2 = pack2(inv_rms, inv_rms), inv_scale2 = pack2(inv_scale, inv_scale);
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int k = 0; k < kRmsVecs; ++k) {
      const int v = threadIdx.x + k * threads;
      if (v < nvec) {
        const uint4 raw = ring[(stage * kRmsVecs + k) * threads + threadIdx.x];
        const uint32_t h[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // q = e4m3(((x / rms) * w) / scale), rounded after every multiplication
          c[j] = e4m3x2_of(mul2(mul2(mul2(bf16x2_to_pair(h[j]), inv_rms2), w[k][j]), inv_scale2));
        }
        *reinterpret_cast<uint2*>(q + v * kVec) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
      }
    }
    stage = stage + 1 == kRmsStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();  // nothing of this CTA's is in flight when it leaves
}

// RMS norm with y rounded to bf16 before the quantisation (`round_bf16`: what a producer kernel followed by a quantiser
// computes).  The row's maximum must then be taken over the ROUNDED y, so the row needs two reductions: the sum of
// squares, then max |bf16(y)|; the rounded y is a bf16 value and waits for the second one packed in 16 registers.
// Otherwise the kernel above: rows in a cp.async ring, one warp per 1024 columns, packed multiplies.
template <int kWarpsT>
__global__ void __launch_bounds__(32 * kWarpsT, silu_ctas_per_sm(kWarpsT)) rms_norm_round_quantize_persistent_kernel(const FusedQuantParams p) {
  let_dependents_start();
  extern __shared__ uint4 ring[];  // [kRmsStages][kRmsVecs][threads]
  __shared__ float part_ss[kRmsMaxWarps], part_max[kRmsMaxWarps];
  const __nv_bfloat16* wvec = static_cast<const __nv_bfloat16*>(p.x2);
  const int nvec = p.cols / kVec;
  constexpr int threads = 32 * kWarpsT, warps = kWarpsT;
  constexpr int kSlots = rms_pow2_at_least(warps);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int src = lane & (kSlots - 1);  // every group of kSlots lanes combines the same slots
  pair_t w[kRmsVecs][4];
#pragma unroll
  for (int k = 0; k < kRmsVecs; ++k) {
    const int v = threadIdx.x + k * threads;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (v < nvec) raw = *reinterpret_cast<const uint4*>(wvec + v * kVec);
    w[k][0] = bf16x2_to_pair(raw.x);
    w[k][1] = bf16x2_to_pair(raw.y);
    w[k][2] = bf16x2_to_pair(raw.z);
    w[k][3] = bf16x2_to_pair(raw.w);
  }
  auto request = [&](long long r, int stage) {  // one group per call, also when there is no such row
    if (r < p.rows) {
      const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.x1) + r * p.ld1;
#pragma unroll
      for (int k = 0; k < kRmsVecs; ++k) {
        const int v = threadIdx.x + k * threads;
        if (v < nvec) cp_async_16(smem_addr(&ring[(stage * kRmsVecs + k) * threads + threadIdx.x]), x + v * kVec);
      }
    }
    cp_async_commit();
  };
  long long row = blockIdx.x;
#pragma unroll
  for (int s = 0; s < kRmsStages - 1; ++s) request(row + static_cast<long long>(s) * gridDim.x, s);
  int stage = 0;
  for (; row < p.rows; row += gridDim.x) {
    request(row + static_cast<long long>(kRmsStages - 1) * gridDim.x, stage == 0 ? kRmsStages - 1 : stage - 1);
    cp_async_wait<kRmsStages - 1>();
    // ---- sum of squares
    pair_t ss = pack2(0.0f, 0.0f);
#pragma unroll
    for (int k = 0; k < kRmsVecs; ++k) {
      const int v = threadIdx.x + k * threads;
      if (v < nvec) {
        const uint4 raw = ring[(stage * kRmsVecs + k) * threads + threadIdx.x];
        const uint32_t h[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const pair_t a = bf16x2_to_pair(h[j]);
          ss = fma2(a, a, ss);
        }
      }
    }
    float s_lo, s_hi;
    unpack2(ss, s_lo, s_hi);
    float s = s_lo + s_hi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) part_ss[warp] = s;
    __syncthreads();  // (everybody has also finished reading part_max of the row before)
    float t = src < warps ? part_ss[src] : 0.0f;
#pragma unroll
    for (int o = kSlots / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    const float inv_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fdiv_rn(t, static_cast<float>(p.cols)) + p.eps));
    const pair_t inv_rms2 = pack2(inv_rms, inv_rms);
    // ---- y = bf16((x / rms) * w), kept packed, and its largest magnitude
    uint32_t y[kRmsVecs][4];
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < kRmsVecs; ++k) {
      const int v = threadIdx.x + k * threads;
      const uint4 raw = v < nvec ? ring[(stage * kRmsVecs + k) * threads + threadIdx.x] : make_uint4(0u, 0u, 0u, 0u);
      const uint32_t h[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[k][j] = bf16x2_of(mul2(mul2(bf16x2_to_pair(h[j]), inv_rms2), w[k][j]));
        float lo, hi;
        unpack2(bf16x2_to_pair(y[k][j]), lo, hi);
        amax = max_nan(amax, fabsf(lo));
        amax = max_nan(amax, fabsf(hi));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) part_max[warp] = amax;
    __syncthreads();  // (everybody has also finished reading part_ss of this row)
    float m = src < warps ? part_max[src] : 0.0f;
#pragma unroll
    for (int o = kSlots / 2; o > 0; o >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = __fdiv_rn(max_nan(m, 1e-12f), 448.0f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    const pair_t inv_scale2 = pack2(inv_scale, inv_scale);
    if (threadIdx.x == 0) p.scale[row] = scale;
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int k = 0; k < kRmsVecs; ++k) {
      const int v = threadIdx.x + k * threads;
      if (v < nvec) {
        uint32_t c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = e4m3x2_of(mul2(bf16x2_to_pair(y[k][j]), inv_scale2));
        *reinterpret_cast<uint2*>(q + v * kVec) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
      }
    }
    stage = stage + 1 == kRmsStages ? 0 : stage + 1;
  }
  cp_async_wait<0>();
}

// SiLU-mul, persistent form: the next row of both inputs is in flight (in registers: a shared-memory ring made this
// kernel slower, its exponentials and reciprocals already queue where shared-memory traffic does) while the current
// one is reduced and written.  Multiplications and the addition go two per instruction, the row's maximum needs one
// barrier (the warps' results alternate between two buffers by row parity).  Same arithmetic per element as
// silu_mul(): ex2.approx and rcp.approx, everything else rounded to nearest.
__device__ __forceinline__ pair_t add2(pair_t a, pair_t b) {
  pair_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ pair_t silu_mul2(pair_t a, pair_t b) {
  float t0, t1, e0, e1, d0, d1, r0, r1;
  unpack2(mul2(a, pack2(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);  // exp(-a) = 2^(-a log2 e)
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(t0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(t1));
  unpack2(add2(pack2(e0, e1), pack2(1.0f, 1.0f)), d0, d1);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d0));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d1));
  return mul2(mul2(a, pack2(r0, r1)), b);
}

constexpr int kSiluVecs = 4;  // 16-byte vectors of a row (of each input) per thread: one warp per 1024 columns, as above

template <int kWarpsT, bool kRound>  // kRound: y is rounded to bf16 before the quantisation (`round_bf16`)
__global__ void __launch_bounds__(32 * kWarpsT, silu_ctas_per_sm(kWarpsT)) silu_mul_quantize_persistent_kernel(const FusedQuantParams p) {
  let_dependents_start();
  constexpr int kKeep = kSiluVecs, threads = 32 * kWarpsT;
  __shared__ float red[2][kRmsMaxWarps];
  const int nvec = p.cols / kVec;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint4 cur1[kKeep], cur2[kKeep];
  auto load_row = [&](long long r, uint4 (&a)[kKeep], uint4 (&b)[kKeep]) {
    const __nv_bfloat16* x1 = static_cast<const __nv_bfloat16*>(p.x1) + r * p.ld1;
    const __nv_bfloat16* x2 = static_cast<const __nv_bfloat16*>(p.x2) + r * p.ld2;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * threads;
      a[i] = v < nvec ? *reinterpret_cast<const uint4*>(x1 + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
      b[i] = v < nvec ? *reinterpret_cast<const uint4*>(x2 + v * kVec) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  long long row = blockIdx.x;
  int parity = 0;
  if (row < p.rows) load_row(row, cur1, cur2);
  for (; row < p.rows; row += gridDim.x) {
    uint4 nxt1[kKeep], nxt2[kKeep];
    const long long next_row = row + gridDim.x;
    if (next_row < p.rows) load_row(next_row, nxt1, nxt2);
    pair_t y[kKeep][4];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {  // vectors beyond the row are zeros: silu(0) * 0 = 0
      const uint32_t h1[4] = {cur1[i].x, cur1[i].y, cur1[i].z, cur1[i].w};
      const uint32_t h2[4] = {cur2[i].x, cur2[i].y, cur2[i].z, cur2[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[i][j] = silu_mul2(bf16x2_to_pair(h1[j]), bf16x2_to_pair(h2[j]));
        if constexpr (kRound) y[i][j] = bf16x2_to_pair(bf16x2_of(y[i][j]));
        float lo, hi;
        unpack2(y[i][j], lo, hi);
        amax = max_nan(amax, fabsf(lo));
        amax = max_nan(amax, fabsf(hi));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[parity][warp] = amax;
    __syncthreads();  // the only barrier of the row
    constexpr int kSlots = rms_pow2_at_least(kWarpsT);
    const int src = lane & (kSlots - 1);  // every group of kSlots lanes combines the same slots
    amax = src < kWarpsT ? red[parity][src] : 0.0f;
#pragma unroll
    for (int o = kSlots / 2; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    parity ^= 1;
    const float scale = __fdiv_rn(max_nan(amax, 1e-12f), 448.0f);
    const float inv_scale = __fdiv_rn(1.0f, scale);
    const pair_t inv_scale2 = pack2(inv_scale, inv_scale);
    if (threadIdx.x == 0) p.scale[row] = scale;
    uint8_t* q = p.q + row * p.ldq;
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      const int v = threadIdx.x + i * threads;
      if (v < nvec) {
        uint32_t c[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = e4m3x2_of(mul2(y[i][j], inv_scale2));
        *reinterpret_cast<uint2*>(q + v * kVec) = make_uint2(c[0] | (c[1] << 16), c[2] | (c[3] << 16));
      }
    }
#pragma unroll
    for (int i = 0; i < kKeep; ++i) {
      cur1[i] = nxt1[i];
      cur2[i] = nxt2[i];
    }
  }
}

// one warp per 1024 columns; the grid fills the GPU with as many CTAs as fit (cached per device)
template <int kWarpsT, bool kRound>
cudaError_t launch_rms_persistent_t(const FusedQuantParams& p, cudaStream_t stream) {
  const auto kernel = kRound ? rms_norm_round_quantize_persistent_kernel<kWarpsT> : rms_norm_quantize_persistent_kernel<kWarpsT>;
  static std::atomic<int> ctas_per_device[64] = {};
  constexpr int threads = 32 * kWarpsT;
  constexpr size_t ring_bytes = static_cast<size_t>(kRmsStages) * kRmsVecs * threads * sizeof(uint4);
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  int ctas = ctas_per_device[dev].load();
  if (ctas == 0) {  // first call on this device (two threads may both get here: they compute the same values)
    int sms = 0, per_sm = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(ring_bytes));
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads,
                                                        ring_bytes);
    if (err != cudaSuccess) return err;
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    ctas_per_device[dev] = ctas;
  }
  const long long grid = p.rows < ctas ? p.rows : ctas;
  kernel<<<static_cast<unsigned>(grid), threads, ring_bytes, stream>>>(p);
  return cudaGetLastError();
}

template <int kWarpsT = 1>
cudaError_t launch_rms_persistent(int warps, const FusedQuantParams& p, cudaStream_t stream) {
  if constexpr (kWarpsT > kRmsMaxWarps) {
    return cudaErrorInvalidValue;
  } else {
    if (warps == kWarpsT) {
      return p.round_bf16 ? launch_rms_persistent_t<kWarpsT, true>(p, stream) : launch_rms_persistent_t<kWarpsT, false>(p, stream);
    }
    return launch_rms_persistent<kWarpsT + 1>(warps, p, stream);
  }
}

template <int kWarpsT, bool kRound>
cudaError_t launch_silu_persistent_t(const FusedQuantParams& p, cudaStream_t stream) {
  static std::atomic<int> ctas_per_device[64] = {};
  constexpr int threads = 32 * kWarpsT;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  int ctas = ctas_per_device[dev].load();
  if (ctas == 0) {
    int sms = 0, per_sm = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, silu_mul_quantize_persistent_kernel<kWarpsT, kRound>, threads, 0);
    if (err != cudaSuccess) return err;
    ctas = sms * (per_sm > 0 ? per_sm : 1);
    ctas_per_device[dev] = ctas;
  }
  const long long grid = p.rows < ctas ? p.rows : ctas;
  silu_mul_quantize_persistent_kernel<kWarpsT, kRound><<<static_cast<unsigned>(grid), threads, 0, stream>>>(p);
  return cudaGetLastError();
}

template <int kWarpsT = 1>
cudaError_t launch_silu_persistent(int warps, const FusedQuantParams& p, cudaStream_t stream) {
  if constexpr (kWarpsT > kRmsMaxWarps) {
    return cudaErrorInvalidValue;
  } else {
    if (warps == kWarpsT) {
      return p.round_bf16 ? launch_silu_persistent_t<kWarpsT, true>(p, stream) : launch_silu_persistent_t<kWarpsT, false>(p, stream);
    }
    return launch_silu_persistent<kWarpsT + 1>(warps, p, stream);
  }
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
  if (p.producer == kProducerRmsNorm && p.vector_ok && p.cols % kVec == 0 &&
      p.cols <= kRmsMaxWarps * 32 * kRmsVecs * kVec) {
    return launch_rms_persistent((p.cols + 1023) / 1024, p, stream);
  }
  if (p.producer == kProducerSiluMul && p.vector_ok && p.cols % kVec == 0 &&
      p.cols <= kRmsMaxWarps * 32 * kSiluVecs * kVec) {
    return launch_silu_persistent((p.cols + 1023) / 1024, p, stream);
  }
  if (p.producer == kProducerRmsNorm) return launch_producer<kProducerRmsNorm>(p, stream);
  if (p.producer == kProducerSiluMul) return launch_producer<kProducerSiluMul>(p, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200fp8
