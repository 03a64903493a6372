// Skinny-M (decode, M <= 128) FP8 rowwise GEMM for sm_100a.  The work is bound by streaming
// W[N,K] from HBM exactly once, so the kernel is organised around that stream:
//
//   * swap-AB: a tile is 128 rows of W (the MMA M side, one TMEM lane each) against all tokens
//     (MMA N = M rounded up to 16), so the tensor core consumes W at the rate TMA delivers it and
//     CUDA cores never touch the operands;
//   * stream-K: the (tile, k-block) space is cut into equal runs of consecutive units, one run per
//     CTA, so every SM streams the same number of W bytes whatever N/128 is relative to the SM count;
//   * a tile whose K range is split over several CTAs is finished by whichever CTA arrives last:
//     each writes its fp32 partial sums to a slot in the workspace, bumps a per-(tile, lane quarter)
//     counter, and the last one adds the slots in ascending CTA order (a fixed order, so the result
//     does not depend on who is last), applies the scales and writes bf16.  No CTA waits for another.
//
// Warp roles are those of the large-M kernel: warp 0 TMA producer, warp 1 TMEM owner + MMA issuer,
// warps 2-5 epilogue.  All mbarrier waits are bounded.
#include "kernels.h"
#include "ptx.cuh"

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
  const long long total = static_cast<long long>(pl.tiles) * pl.kblocks;
  long long per = (total + sm_count - 1) / sm_count;
  const long long floor_units = pl.kblocks < 4 ? pl.kblocks : 4;  // do not cut K finer than 512 bytes
  if (per < floor_units) per = floor_units;
  pl.units_per_cta = static_cast<int>(per);
  pl.num_ctas = static_cast<int>((total + per - 1) / per);
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
};

struct Segment {
  int tile;
  int slot;  // index of the segment inside this CTA's run (selects the partial-sum slot)
  int kb0;
  int kb1;
};

// One CTA's run of consecutive units [u_begin, u_stop) cut at tile boundaries.  Segments that
// cover only part of a tile's K range are processed FIRST (the one at the end of the run, then
// the one at its start), the whole tiles after them: the cross-CTA fix-up of a split tile then
// happens early, hidden behind the streaming of the remaining tiles, instead of at the very end
// of the kernel where nothing overlaps it.
struct Run {
  long long u_begin;
  long long u_stop;
  int kblocks;
  int first_tile;
  int count;
  bool tail_first;  // last segment is partial and goes first
  bool head_next;   // first segment is partial (and is not that same segment)
};

__device__ __forceinline__ Run make_run(long long u_begin, long long u_stop, int kblocks) {
  Run r;
  r.u_begin = u_begin;
  r.u_stop = u_stop;
  r.kblocks = kblocks;
  r.first_tile = static_cast<int>(u_begin / kblocks);
  r.count = u_stop > u_begin ? static_cast<int>((u_stop - 1) / kblocks) - r.first_tile + 1 : 0;
  r.tail_first = r.count > 0 && (u_stop % kblocks) != 0;
  r.head_next = r.count > 0 && (u_begin % kblocks) != 0 && !(r.tail_first && r.count == 1);
  return r;
}

// i-th segment in processing order
__device__ __forceinline__ Segment run_segment(const Run& r, int i) {
  int j;  // position in the run
  int pos = 0;
  if (r.tail_first && i == 0) {
    j = r.count - 1;
  } else {
    pos += r.tail_first ? 1 : 0;
    if (r.head_next && i == pos) {
      j = 0;
    } else {
      pos += r.head_next ? 1 : 0;
      j = (r.head_next ? 1 : 0) + (i - pos);
    }
  }
  Segment s;
  s.slot = j;
  s.tile = r.first_tile + j;
  const long long tile_u0 = static_cast<long long>(s.tile) * r.kblocks;
  s.kb0 = r.u_begin > tile_u0 ? static_cast<int>(r.u_begin - tile_u0) : 0;
  s.kb1 = r.u_stop < tile_u0 + r.kblocks ? static_cast<int>(r.u_stop - tile_u0) : r.kblocks;
  return s;
}

__global__ void __launch_bounds__(SkinnyGeometry::kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                   const SkinnyParams p, const int tokens_pad, const int stages, const int kblocks,
                   const int units_per_cta, const int segs_per_cta, const long long total_units) {
  using G = SkinnyGeometry;

#ifdef B200FP8_DEBUG_KNOBS
#define SK_TRACE(i) do { if (p.trace) p.trace[blockIdx.x * 8 + (i)] = globaltimer_ns(); } while (0)
#else
#define SK_TRACE(i) do {} while (0)
#endif
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);
  if (threadIdx.x == 0) SK_TRACE(0);

  const int bytes_b = tokens_pad * G::kBlockK;
  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + stages * G::kBytesA;
  const uint32_t bars = smem_b + stages * bytes_b;
  const uint32_t bar_full = bars;                       // [stages]
  const uint32_t bar_empty = bars + 8 * stages;         // [stages]
  const uint32_t bar_tmem_full = bars + 16 * stages;    // [2]
  const uint32_t bar_tmem_empty = bar_tmem_full + 16;   // [2]
  const uint32_t tmem_slot = bar_tmem_empty + 16;
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const long long u_begin = static_cast<long long>(blockIdx.x) * units_per_cta;
  const long long u_stop = u_begin + units_per_cta < total_units ? u_begin + units_per_cta : total_units;
  const Run run = make_run(u_begin, u_stop, kblocks);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tmem_full + 8 * b, 1);
      mbar_init(bar_tmem_empty + 8 * b, 4);
    }
    *abort_flag = 0u;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_w);
    prefetch_tensormap(&tm_x);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 256);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) SK_TRACE(1);

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      const uint32_t tx_bytes = static_cast<uint32_t>(G::kBytesA + bytes_b);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = 0; i < run.count && ok; ++i) {
        const Segment sg = run_segment(run, i);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
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
      const uint32_t idesc = instr_desc_e4m3(G::kRowsW, static_cast<uint32_t>(tokens_pad));
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int i = 0; i < run.count && ok; ++i) {
        const Segment sg = run_segment(run, i);
        const uint32_t buf = static_cast<uint32_t>(i) & 1u;
        const uint32_t use = (static_cast<uint32_t>(i) >> 1) & 1u;
        ok = mbar_wait<false>(bar_tmem_empty + 8 * buf, use ^ 1u, abort_flag, p.status, kSiteMmaTmemEmpty);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * G::kMaxTokens;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          ok = mbar_wait<false>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
          if (!ok) break;
          if (i == 0 && kb == sg.kb0) SK_TRACE(2);
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
      SK_TRACE(3);
    }
  } else {
    // ---------------------------------- epilogue ---------------------------------
    const int quarter = warp & 3;
    const int lane_row = quarter * 32 + lane;  // row of the 128-row W tile = TMEM lane
    const size_t slot_floats = static_cast<size_t>(tokens_pad) * G::kRowsW;
    bool ok = true;
    for (int i = 0; i < run.count && ok; ++i) {
      const Segment sg = run_segment(run, i);
      const uint32_t buf = static_cast<uint32_t>(i) & 1u;
      const uint32_t use = (static_cast<uint32_t>(i) >> 1) & 1u;
      const int n = sg.tile * G::kRowsW + lane_row;  // output column
      const bool full_k = sg.kb0 == 0 && sg.kb1 == kblocks;
      const bool n_ok = n < p.N;
      const float ws = n_ok ? __ldg(p.w_scale + n) : 0.0f;
      const float bias = (n_ok && p.bias != nullptr) ? __bfloat162float(p.bias[n]) : 0.0f;
      float* slot = p.partials + (static_cast<size_t>(blockIdx.x) * segs_per_cta + sg.slot) * slot_floats;

      ok = mbar_wait<false>(bar_tmem_full + 8 * buf, use, abort_flag, p.status, kSiteEpiTmemFull);
      ok = __all_sync(0xffffffffu, ok) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * G::kMaxTokens;

      for (int c = 0; c < tokens_pad; c += 16) {
        uint32_t acc[16];
        tmem_ld_32x16(t_addr + c, acc);
        tmem_ld_wait();
        if (full_k) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = c + j;
            if (m < p.M && n_ok) {
              const float v = __uint_as_float(acc[j]) * (__ldg(p.x_scale + m) * ws) + bias;
              p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16_rn(v);
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

      if (!full_k) {
        // publish this warp's part of the slot, then see whether every other part is already there
        const long long tile_u0 = static_cast<long long>(sg.tile) * kblocks;
        const int cta_first = static_cast<int>(tile_u0 / units_per_cta);
        const int cta_last = static_cast<int>((tile_u0 + kblocks - 1) / units_per_cta);
        const uint32_t parts = static_cast<uint32_t>(cta_last - cta_first + 1);
        __threadfence();
        __syncwarp();
        uint32_t seen = 0;
        if (lane == 0) seen = atomicAdd(p.counters + sg.tile * 4 + quarter, 1u);
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (seen == parts - 1u) {
          __threadfence();
          // Eight tokens at a time, so that eight independent loads per part are in flight; the
          // parts of one element are still added in ascending CTA order.
          for (int m0 = 0; m0 < p.M; m0 += 8) {
            float sum[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] = 0.0f;
            for (int cta = cta_first; cta <= cta_last; ++cta) {
              const long long their_first = static_cast<long long>(cta) * units_per_cta / kblocks;
              const float* src = p.partials +
                                 (static_cast<size_t>(cta) * segs_per_cta + (sg.tile - their_first)) * slot_floats +
                                 static_cast<size_t>(m0) * G::kRowsW + lane_row;
              float part[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) part[j] = __ldcg(src + j * G::kRowsW);  // rows >= M: unused padding
#pragma unroll
              for (int j = 0; j < 8; ++j) sum[j] += part[j];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int m = m0 + j;
              if (m < p.M && n_ok) {
                const float v = sum[j] * (__ldg(p.x_scale + m) * ws) + bias;
                p.y[static_cast<long long>(m) * p.ldy + n] = __float2bfloat16_rn(v);
              }
            }
          }
          __syncwarp();
          if (lane == 0) p.counters[sg.tile * 4 + quarter] = 0u;  // leave the workspace zero
        }
      }
    }
    if (quarter == 0 && lane == 0) SK_TRACE(4);
  }

  // ------------------------------------ common exit ------------------------------------
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    tmem_dealloc<1>(tmem_base, 256);
  }
  if (threadIdx.x == 32) SK_TRACE(5);
}

}  // namespace

// Scratch of the no-allocation entry point.  In host code this name is only a handle for the
// runtime: its device address comes from cudaGetSymbolAddress, once per device, below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

cudaError_t skinny_static_scratch(void** device_ptr, size_t* bytes) {
  static void* address_on_device[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
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
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 64 && configured_bytes[dev] < plan.smem_bytes) {
    err = cudaFuncSetAttribute(gemm_skinny_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               SkinnyGeometry::kSmemBudget);
    if (err != cudaSuccess) return err;
    configured_bytes[dev] = SkinnyGeometry::kSmemBudget;
  }
  const long long total = static_cast<long long>(plan.tiles) * plan.kblocks;
  gemm_skinny_kernel<<<plan.num_ctas, SkinnyGeometry::kThreads, plan.smem_bytes, stream>>>(
      tm_w, tm_x, p, plan.tokens_pad, plan.stages, plan.kblocks, plan.units_per_cta, plan.segs_per_cta, total);
  return cudaGetLastError();
}

}  // namespace b200fp8
