// Skinny-M (decode, M <= 128) FP8 rowwise GEMM for sm_100a.  The work is bound by streaming
// W[N,K] from HBM exactly once, so the kernel is organised around that stream:
//
//   * swap-AB: a tile is 128 rows of W (the MMA M side, one TMEM lane each) against all tokens
//     (MMA N = M rounded up to 16), so the tensor core consumes W at the rate TMA delivers it and
//     CUDA cores never touch the operands;
//   * stream-K: the (tile, k-block) space is cut into equal runs of consecutive
//     units, one run per CTA, so every SM streams the same number of W bytes whatever N/128 is
//     relative to the SM count;
//   * a tile whose K range is split over several CTAs is finished by whichever CTA arrives last:
//     each writes its fp32 partial sums to a slot in the workspace, bumps a per-(tile, lane quarter)
//     counter, and the last one adds the slots in ascending CTA order (a fixed order, so the result
//     does not depend on who is last), applies the scales and writes bf16.  No CTA waits for another.
//
// Warp roles: warp 0 TMA producer, warp 1 TMEM owner + MMA issuer, warps 2-5 drain the accumulators
// (to Y for a whole tile, to a partial-sum slot for a split one), warps 6-9 do the cross-CTA
// additions ("fix-ups") that the draining warps hand them through a small mailbox in shared memory,
// so that a fix-up - a chain of dependent global-memory round trips - never keeps an accumulator
// from being drained.  Split segments are processed first, so fix-ups happen while W still streams.
// All waits are bounded.
//
// Launched with the programmatic-serialization attribute (B200FP8_FLAG_PDL) the kernel may start
// while the kernel before it in the stream is still running.  It then fills its whole pipeline
// with W - weights, which the caller promises nothing in flight is writing - and touches everything
// else (X, scales, bias, Y, workspace) only after griddepcontrol.wait, i.e. after the previous kernel
// has completed.  Back-to-back decode GEMMs thus overlap one kernel's tail, where SMs finish at
// different times, with the next kernel's prologue and first 192 KiB of weights per SM.
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"
#include "streamk.cuh"

namespace b200fp8 {

SkinnyPlan make_skinny_plan(int M, int N, int K, int sm_count) {
  using G = SkinnyGeometry;
  SkinnyPlan pl = {};
  pl.tokens_pad = ((M + 15) / 16) * 16;
  if (pl.tokens_pad < 16) pl.tokens_pad = 16;
  const int stage_bytes = G::kBytesA + pl.tokens_pad * G::kBlockK;
  pl.stages = (G::kSmemBudget - G::kBarBytes - 1024) / stage_bytes;
  if (pl.stages > G::kMaxStages) pl.stages = G::kMaxStages;
  pl.tiles = (N + G::kRowsW - 1) / G::kRowsW;
  pl.kblocks = (K + G::kBlockK - 1) / G::kBlockK;

  // Whole waves of tiles are dealt out one tile per CTA (nothing to add across CTAs); only the
  // remainder, fewer tiles than CTAs, is cut along K into equal runs.  All of it when tiles < CTAs.
  pl.dp_waves = pl.tiles / sm_count;
  pl.sk_tiles = pl.tiles - pl.dp_waves * sm_count;
  const long long sk_units = static_cast<long long>(pl.sk_tiles) * pl.kblocks;
  long long per = (sk_units + sm_count - 1) / sm_count;
  const long long floor_units = pl.kblocks < 4 ? pl.kblocks : 4;  // do not cut K finer than 512 bytes
  if (per < floor_units) per = floor_units;
  pl.units_per_cta = static_cast<int>(per);
  pl.num_ctas = pl.dp_waves > 0 ? sm_count : static_cast<int>((sk_units + per - 1) / per);
  pl.segs_per_cta = (pl.units_per_cta + pl.kblocks - 1) / pl.kblocks + 1;
  pl.smem_bytes = static_cast<size_t>(pl.stages) * stage_bytes + G::kBarBytes + 1024;
  pl.partial_bytes =
      static_cast<size_t>(pl.num_ctas) * pl.segs_per_cta * pl.tokens_pad * G::kRowsW * sizeof(float);
  pl.counter_bytes = G::kCounterRegionBytes;
  return pl;
}

namespace {

enum WaitSite : uint32_t {
  kSiteProducerEmpty = 0x201,
  kSiteMmaTmemEmpty = 0x202,
  kSiteMmaFull = 0x203,
  kSiteEpiTmemFull = 0x204,
  kSiteMailEmpty = 0x205,
  kSiteMailFull = 0x206,
};

constexpr int kMailDepth = 4;      // fix-up requests in flight per lane quarter
constexpr int kMailDone = -1;      // "no more requests" marker

__global__ void __launch_bounds__(SkinnyGeometry::kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const SkinnyParams p, const SkinnyShape sh) {
  using G = SkinnyGeometry;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const int stages = sh.stages;
  const int kblocks = sh.kblocks;
  const int bytes_b = sh.tokens_pad * G::kBlockK;
  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + stages * G::kBytesA;
  const uint32_t bars = smem_b + stages * bytes_b;
  const uint32_t bar_full = bars;                                   // [stages]
  const uint32_t bar_empty = bars + 8 * stages;                     // [stages]
  const uint32_t bar_tmem_full = bars + 16 * stages;                // [2]
  const uint32_t bar_tmem_empty = bar_tmem_full + 16;               // [2]
  const uint32_t bar_mail_full = bar_tmem_empty + 16;               // [4 quarters][kMailDepth]
  const uint32_t bar_mail_empty = bar_mail_full + 8 * 4 * kMailDepth;  // [4 quarters][kMailDepth]
  const uint32_t tmem_slot = bar_mail_empty + 8 * 4 * kMailDepth;
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);
  volatile int* mail_tile = reinterpret_cast<volatile int*>(tail_ptr + 8);  // [4 quarters][kMailDepth]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const size_t slot_floats = static_cast<size_t>(sh.tokens_pad) * G::kRowsW;
  // this CTA's work: a run of the K-split region first, then its whole tiles
  const CtaWork work = make_cta_work(static_cast<int>(blockIdx.x), static_cast<int>(gridDim.x), sh.tiles, sh.sk_tiles,
                                     kblocks, sh.units_per_cta, sh.segs_per_cta);
  const int seg_count = work.count;
  auto segment_at = [&](int i) { return work_segment(work, i); };

  // Producer state that survives the set-up barrier: thread 0 starts streaming W as soon as it has
  // initialised the barriers, without waiting for the TMEM allocation or the other warps.
  const uint32_t tx_bytes = static_cast<uint32_t>(G::kBytesA + bytes_b);
  int first_pass_kb[G::kMaxStages];  // k-block held by each stage after the first pass over the ring
  int issued = 0, resume_i = 0, resume_kb = 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tmem_full + 8 * b, 1);
      mbar_init(bar_tmem_empty + 8 * b, 4);
    }
    for (int s = 0; s < 4 * kMailDepth; ++s) {
      mbar_init(bar_mail_full + 8 * s, 1);
      mbar_init(bar_mail_empty + 8 * s, 1);
    }
    *abort_flag = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
    // First pass over the ring: W only (weights; every stage is free, nothing to wait for).  X joins
    // after griddepcontrol.wait below, because the kernel before this one may still be producing it.
    for (int i = 0; i < seg_count && issued < stages; ++i) {
      const Segment sg = segment_at(i);
      int kb = sg.kb0;
      for (; kb < sg.kb1 && issued < stages; ++kb) {
        const uint32_t full = bar_full + 8 * issued;
        mbar_arrive_expect_tx(full, tx_bytes);
        tma_load_2d(smem_a + issued * G::kBytesA, &tm_w, full, kb * G::kBlockK, sg.tile * G::kRowsW);
        first_pass_kb[issued] = kb;
        ++issued;
      }
      resume_i = i;
      resume_kb = kb;
    }
  }
  // two accumulators of tokens_pad columns; the allocation is a power of two of at least 32
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * static_cast<uint32_t>(sh.tokens_pad)) tmem_cols <<= 1;
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, tmem_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) griddep_launch_dependents();  // the next kernel does its own waiting

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t stage = static_cast<uint32_t>(issued % stages);
      uint32_t phase = static_cast<uint32_t>(issued / stages) & 1u;
      bool ok = true;
      // the kernels before this one are done from here on: add the X boxes of the first-pass stages
      griddep_wait();
      for (int s = 0; s < issued; ++s) {
        tma_load_2d(smem_b + s * bytes_b, &tm_x, bar_full + 8 * s, first_pass_kb[s] * G::kBlockK, 0);
      }
      for (int i = resume_i; i < seg_count && ok; ++i) {
        const Segment sg = segment_at(i);
        for (int kb = (i == resume_i ? resume_kb : sg.kb0); kb < sg.kb1; ++kb) {
          ok = mbar_wait<false>(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          mbar_arrive_expect_tx(full, tx_bytes);
          tma_load_2d(smem_a + stage * G::kBytesA, &tm_w, full, kb * G::kBlockK, sg.tile * G::kRowsW);
          tma_load_2d(smem_b + stage * bytes_b, &tm_x, full, kb * G::kBlockK, 0);
          if (++stage == static_cast<uint32_t>(stages)) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------- MMA issuer --------------------------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc_e4m3(G::kRowsW, static_cast<uint32_t>(sh.tokens_pad));
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = 0; i < seg_count && ok; ++i) {
        const Segment sg = segment_at(i);
        const uint32_t buf = static_cast<uint32_t>(i) & 1u;
        const uint32_t use = (static_cast<uint32_t>(i) >> 1) & 1u;
        ok = mbar_wait<false>(bar_tmem_empty + 8 * buf, use ^ 1u, abort_flag, p.status, kSiteMmaTmemEmpty);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * static_cast<uint32_t>(sh.tokens_pad);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          ok = mbar_wait<false>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = smem_desc_k_sw128(smem_a + stage * G::kBytesA);
          const uint64_t b_desc = smem_desc_k_sw128(smem_b + stage * bytes_b);
#pragma unroll
          for (int k = 0; k < G::kBlockK / 32; ++k) {
            tc_mma_f8<1>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * stage);
          if (++stage == static_cast<uint32_t>(stages)) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(bar_tmem_full + 8 * buf);
      }
    }
  } else if (warp < 6) {
    // ------------------------- drain: TMEM -> Y or partial-sum slot -------------------------
    const int quarter = warp & 3;
    const int lane_row = quarter * 32 + lane;  // row of the 128-row W tile = TMEM lane
    griddep_wait();  // scales, bias, Y and the workspace belong to the previous kernel until it is done
    uint32_t mail_no = 0;
    bool ok = true;
    // hand one tile (or the end marker) to this quarter's fix-up warp
    auto post = [&](int tile) {
      const uint32_t ring = mail_no % kMailDepth;
      const uint32_t use = (mail_no / kMailDepth) & 1u;
      ++mail_no;
      const uint32_t idx = quarter * kMailDepth + ring;
      bool free_slot = true;
      if (lane == 0) {
        free_slot = mbar_wait<false>(bar_mail_empty + 8 * idx, use ^ 1u, abort_flag, p.status, kSiteMailEmpty);
        if (free_slot) {
          mail_tile[idx] = tile;
          mbar_arrive(bar_mail_full + 8 * idx);  // release: the entry is visible to the waiter
        }
      }
      return __all_sync(0xffffffffu, free_slot) != 0;
    };

    for (int i = 0; i < seg_count && ok; ++i) {
      const Segment sg = segment_at(i);
      const uint32_t buf = static_cast<uint32_t>(i) & 1u;
      const uint32_t use = (static_cast<uint32_t>(i) >> 1) & 1u;
      const int n = sg.tile * G::kRowsW + lane_row;  // output column
      const bool full_k = sg.kb0 == 0 && sg.kb1 == kblocks;
      const bool n_ok = n < p.N;
      const float ws = n_ok ? __ldg(p.w_scale + n) : 0.0f;
      const float bias = (n_ok && p.bias != nullptr) ? __bfloat162float(p.bias[n]) : 0.0f;
      float* slot = p.partials + static_cast<size_t>(sg.slot) * slot_floats;

      ok = mbar_wait<false>(bar_tmem_full + 8 * buf, use, abort_flag, p.status, kSiteEpiTmemFull);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * static_cast<uint32_t>(sh.tokens_pad);

      for (int c = 0; c < sh.tokens_pad; c += 16) {
        uint32_t acc[16];
        tmem_ld_32x16(t_addr + c, acc);
        tmem_ld_wait();
        if (full_k) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            if (m < p.M && n_ok) {
              const float v = __uint_as_float(acc[j]) * (__ldg(p.x_scale + m) * ws) + bias;
              reinterpret_cast<uint16_t*>(p.y)[static_cast<long long>(m) * p.ldy + n] = to_out16(v, p.out_fp16);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            if (m < p.M) slot[static_cast<size_t>(m) * G::kRowsW + lane_row] = __uint_as_float(acc[j]);
          }
        }
      }
      // accumulator read: hand the TMEM buffer back
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tmem_empty + 8 * buf);
      if (full_k) continue;

      // Publish this warp's part of the slot; if every other part of the tile is already there,
      // this CTA finishes the tile: its fix-up warp does, this warp goes back to draining.
      int first_part, last_part;
      tile_parts(sg.tile, kblocks, sh.units_per_cta, &first_part, &last_part);
      const uint32_t parts = static_cast<uint32_t>(last_part - first_part + 1);
      __threadfence();
      __syncwarp();
      uint32_t seen = 0;
      if (lane == 0) seen = atomicAdd(p.counters + sg.tile * 4 + quarter, 1u);
      seen = __shfl_sync(0xffffffffu, seen, 0);
      if (seen == parts - 1u) ok = post(sg.tile);
    }
    post(kMailDone);
  } else {
    // ------------------- fix-up: add the parts of a split tile, scale, write Y -------------------
    const int quarter = warp & 3;
    const int lane_row = quarter * 32 + lane;
    griddep_wait();
    for (uint32_t mail_no = 0;; ++mail_no) {
      const uint32_t ring = mail_no % kMailDepth;
      const uint32_t use = (mail_no / kMailDepth) & 1u;
      const uint32_t idx = quarter * kMailDepth + ring;
      bool ok = mbar_wait<false>(bar_mail_full + 8 * idx, use, abort_flag, p.status, kSiteMailFull);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      const int tile = mail_tile[idx];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_mail_empty + 8 * idx);
      if (tile == kMailDone) break;

      const int n = tile * G::kRowsW + lane_row;
      const bool n_ok = n < p.N;
      const float ws = n_ok ? __ldg(p.w_scale + n) : 0.0f;
      const float bias = (n_ok && p.bias != nullptr) ? __bfloat162float(p.bias[n]) : 0.0f;
      int first_part, last_part;
      tile_parts(tile, kblocks, sh.units_per_cta, &first_part, &last_part);
      __threadfence();  // the counter said every part is published; order our reads after that
      // 16 tokens x up to 4 parts = up to 64 independent loads in flight per thread; the parts of an
      // element are added in ascending CTA order whatever CTA does the adding.
      for (int m0 = 0; m0 < p.M; m0 += 16) {
        float sum[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) sum[j] = 0.0f;
        for (int part0 = first_part; part0 <= last_part; part0 += 4) {
          float v[4][16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int part = part0 + q <= last_part ? part0 + q : last_part;
            const size_t their_slot = part_slot(part, tile, kblocks, sh.units_per_cta, sh.segs_per_cta);
            const float* src =
                p.partials + their_slot * slot_floats + static_cast<size_t>(m0) * G::kRowsW + lane_row;
#pragma unroll
            for (int j = 0; j < 16; ++j) v[q][j] = __ldcg(src + j * G::kRowsW);  // rows >= M: unused padding
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (part0 + q <= last_part) {
#pragma unroll
              for (int j = 0; j < 16; ++j) sum[j] += v[q][j];
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int m = m0 + j;
          if (m < p.M && n_ok) {
            const float v = sum[j] * (__ldg(p.x_scale + m) * ws) + bias;
            reinterpret_cast<uint16_t*>(p.y)[static_cast<long long>(m) * p.ldy + n] = to_out16(v, p.out_fp16);
          }
        }
      }
      __syncwarp();
      if (lane == 0) p.counters[tile * 4 + quarter] = 0u;  // leave the workspace zero
    }
  }

  // ------------------------------------ common exit ------------------------------------
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    tmem_dealloc<1>(tmem_base, tmem_cols);
  }
}

}  // namespace

// Scratch of the no-allocation entry point.  In host code this name is only a handle for the
// runtime: its device address comes from cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

cudaError_t skinny_static_scratch(void** device_ptr, size_t* bytes) {
  static void* address_on_device[64] = {};
  static std::mutex mutex;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mutex);
  if (address_on_device[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return err;
    address_on_device[dev] = ptr;
  }
  *device_ptr = address_on_device[dev];
  *bytes = kStaticScratchBytes;
  return cudaSuccess;
}

cudaError_t launch_gemm_skinny(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const SkinnyParams& p,
                               const SkinnyPlan& plan, cudaStream_t stream) {
  static size_t configured_bytes[64] = {};
  static std::mutex mutex;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (dev < 64 && configured_bytes[dev] < plan.smem_bytes) {
      err = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SkinnyGeometry::kSmemBudget);
      if (err != cudaSuccess) return err;
      configured_bytes[dev] = SkinnyGeometry::kSmemBudget;
    }
  }
  SkinnyShape sh = {};
  sh.tokens_pad = plan.tokens_pad;
  sh.stages = plan.stages;
  sh.kblocks = plan.kblocks;
  sh.units_per_cta = plan.units_per_cta;
  sh.segs_per_cta = plan.segs_per_cta;
  sh.sk_units = static_cast<long long>(plan.sk_tiles) * plan.kblocks;
  sh.sk_tiles = plan.sk_tiles;
  sh.tiles = plan.tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.num_ctas), 1, 1);
  cfg.blockDim = dim3(SkinnyGeometry::kThreads, 1, 1);
  cfg.dynamicSmemBytes = plan.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = plan.overlap_previous_kernel ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_skinny_kernel, tm_w, tm_x, p, sh);
}

}  // namespace b200fp8
