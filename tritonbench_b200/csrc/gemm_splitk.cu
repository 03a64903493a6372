// FP8 rowwise GEMM for problems with few output tiles and a long K: split-K inside a thread-block
// cluster, reduced over distributed shared memory.
//
// A cluster of S CTAs (S = 2 or 4) owns one 128x256 tile of Y.  CTA r multiplies the r-th slice of K
// with the usual pipeline (TMA -> 128B-swizzled ring -> tcgen05.mma -> TMEM).  Then
//   (A) cluster barrier: every CTA's MMAs have finished, so every operand ring is free;
//   exchange: each CTA writes its fp32 partial tile, column slice j (256/S columns) to CTA j,
//   into CTA j's (now idle) operand ring through shared::cluster stores - a reduce-scatter;
//   (B) cluster barrier: all partials have landed;
//   each CTA adds the S partials of its column slice in CTA order (fixed, deterministic),
//   applies the scales, rounds and stores its 128 x 256/S part of the tile.
// Partial sums never leave the SMs, and the epilogue is spread over the S CTAs.
//
// Every mbarrier wait is bounded; a CTA that gives up still arrives at both cluster barriers so
// that its peers are never left waiting.
#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

using Geo = TcGeometry;
constexpr int kStages = 4;
constexpr int kBytesA = Geo::kBlockM * Geo::kBlockK;   // 16 KiB
constexpr int kBytesB = Geo::kBlockN * Geo::kBlockK;   // 32 KiB
constexpr int kRingBytes = kStages * (kBytesA + kBytesB);            // 192 KiB, reused for the exchange
constexpr int kExchangeBytes = Geo::kBlockM * Geo::kBlockN * 4;      // 128 KiB of fp32 partials per CTA
constexpr int kEpiBytes = 4 * 2 * Geo::kStoreRows * Geo::kStoreCols * 2;
constexpr int kBarBytes = 256;
static_assert(kExchangeBytes <= kRingBytes, "the exchange buffer lives in the operand ring");

enum WaitSite : uint32_t {
  kSiteProducerEmpty = 0x301,
  kSiteMmaFull = 0x302,
  kSiteEpiTmemFull = 0x303,
};

__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

__device__ __forceinline__ float4 ld_shared_v4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// Exchange buffer of a CTA: [sender][group of 4 columns of its slice][row][4 columns] fp32, so that a warp
// (32 consecutive rows) moves 512 contiguous bytes per instruction.
__device__ __forceinline__ uint32_t exchange_offset(int sender, int slice_cols, int col_in_slice, int row) {
  return static_cast<uint32_t>((((sender * (slice_cols / 4) + col_in_slice / 4) * Geo::kBlockM) + row) * 16);
}

__global__ void __launch_bounds__(Geo::kThreads, 1)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_y, const TcParams p, const int split) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + kStages * kBytesA;
  const uint32_t smem_epi = base + kRingBytes;
  const uint32_t bars = smem_epi + kEpiBytes;
  const uint32_t bar_full = bars;                  // [kStages]
  const uint32_t bar_empty = bars + 8 * kStages;   // [kStages]
  const uint32_t bar_tmem_full = bars + 16 * kStages;
  const uint32_t tmem_slot = bar_tmem_full + 8;
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.x / split;
  const int tiles_m = (p.M + Geo::kBlockM - 1) / Geo::kBlockM;
  const int m_tile = tile % tiles_m;
  const int n_tile = tile / tiles_m;
  const int row_base = m_tile * Geo::kBlockM;
  const int col_base = n_tile * Geo::kBlockN;

  const int num_kb = (p.K + Geo::kBlockK - 1) / Geo::kBlockK;
  const int kb_per = (num_kb + split - 1) / split;
  const int kb0 = rank * kb_per < num_kb ? rank * kb_per : num_kb;
  const int kb1 = kb0 + kb_per < num_kb ? kb0 + kb_per : num_kb;
  const bool has_work = kb1 > kb0;
  const int slice_cols = Geo::kBlockN / split;  // columns of the tile this CTA finishes

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tmem_full, 1);
    *abort_flag = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    if (p.use_tma_store) prefetch_tensormap(&tm_y);
    // the first pass over the ring needs no waiting: start it before the set-up barrier
    for (int kb = kb0; kb < kb1 && kb < kb0 + kStages; ++kb) {
      const int stage = kb - kb0;
      const uint32_t full = bar_full + 8 * stage;
      mbar_arrive_expect_tx(full, kBytesA + kBytesB);
      tma_load_2d(smem_a + stage * kBytesA, &tm_x, full, kb * Geo::kBlockK, row_base);
      tma_load_2d(smem_b + stage * kBytesB, &tm_w, full, kb * Geo::kBlockK, col_base);
    }
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 256);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 1;  // the first kStages k-blocks were issued before the set-up barrier
      for (int kb = kb0 + kStages; kb < kb1; ++kb) {
        ok = mbar_wait<false>(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty);
        if (!ok) break;
        const uint32_t full = bar_full + 8 * stage;
        mbar_arrive_expect_tx(full, kBytesA + kBytesB);
        tma_load_2d(smem_a + stage * kBytesA, &tm_x, full, kb * Geo::kBlockK, row_base);
        tma_load_2d(smem_b + stage * kBytesB, &tm_w, full, kb * Geo::kBlockK, col_base);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      constexpr uint32_t idesc = instr_desc_e4m3(Geo::kBlockM, Geo::kBlockN);
      uint32_t stage = 0, phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = mbar_wait<false>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t a_desc = smem_desc_k_sw128(smem_a + stage * kBytesA);
        const uint64_t b_desc = smem_desc_k_sw128(smem_b + stage * kBytesB);
#pragma unroll
        for (int k = 0; k < Geo::kBlockK / 32; ++k) {
          tc_mma_f8<1>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar_empty + 8 * stage);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tc_commit(bar_tmem_full);
    }
  } else if (has_work) {
    // the accumulator is complete (and this CTA's operand ring idle) once the last commit arrives
    ok = mbar_wait<false>(bar_tmem_full, 0u, abort_flag, p.status, kSiteEpiTmemFull);
    tc_fence_after_sync();
  }
  __syncwarp();
  // a CTA that gave up neither sends nor adds (its output is garbage and the status word says so)
  const bool cta_ok = __all_sync(0xffffffffu, *abort_flag == 0u) != 0;

  // ---- (A) every CTA of the cluster has finished reading its operand ring ----
  cluster_sync_all();

  const int quarter = warp & 3;
  const int tile_row = quarter * 32 + lane;  // row inside the 128-row tile = TMEM lane
  if (warp >= 2 && cta_ok) {
    // exchange: columns [j*slice_cols, (j+1)*slice_cols) of this CTA's partial go to CTA j
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < Geo::kBlockN; c0 += 32) {
      uint32_t acc[32];
      if (has_work) {
        tmem_ld_32x32(t_addr + c0, acc);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = 0u;  // K shorter than the split: an empty slice adds nothing
      }
      const int dest = c0 / slice_cols;  // 32 | slice_cols: one destination per chunk
      const int c_in_slice = c0 - dest * slice_cols;
      const uint32_t local = smem_a + exchange_offset(rank, slice_cols, c_in_slice, tile_row);
      const uint32_t remote = mapa_cluster(local, static_cast<uint32_t>(dest));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        st_cluster_v4(remote + j * Geo::kBlockM * 16, acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
      }
    }
    tc_fence_before_sync();
  }

  // ---- (B) all partial sums have landed ----
  cluster_sync_all();

  if (warp >= 2 && cta_ok) {
    const int row0 = row_base + quarter * 32;
    const int row = row0 + lane;
    const float xs = row < p.M ? __ldg(p.x_scale + row) : 0.0f;
    const uint32_t stage_buf = smem_epi + quarter * (2 * Geo::kStoreRows * Geo::kStoreCols * 2);
    uint32_t store_count = 0;
#pragma unroll 1
    for (int box = 0; box < slice_cols / Geo::kStoreCols; ++box) {
      const int box_col = col_base + rank * slice_cols + box * Geo::kStoreCols;
      const uint32_t sbuf = stage_buf + (store_count & 1u) * (Geo::kStoreRows * Geo::kStoreCols * 2);
      if (p.use_tma_store) {
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
      }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int c_in_slice = box * Geo::kStoreCols + half * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.0f;
        for (int sender = 0; sender < split; ++sender) {  // CTA order: the sum does not depend on timing
          const uint32_t src = smem_a + exchange_offset(sender, slice_cols, c_in_slice, tile_row);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 t = ld_shared_v4(src + j * Geo::kBlockM * 16);
            v[4 * j + 0] += t.x;
            v[4 * j + 1] += t.y;
            v[4 * j + 2] += t.z;
            v[4 * j + 3] += t.w;
          }
        }
        const int c_first = box_col + half * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float ws = (c_first + j < p.N) ? __ldg(p.w_scale + c_first + j) : 0.0f;
          v[j] *= xs * ws;
          if (p.bias != nullptr && c_first + j < p.N) v[j] += __bfloat162float(p.bias[c_first + j]);
        }
        if (p.use_tma_store) {
          const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t chunk = static_cast<uint32_t>((half * 4 + j) ^ (lane & 7));
            if (p.out_fp16) {
              st_shared_v4(row_addr + chunk * 16, pack_f16x2(v[8 * j + 0], v[8 * j + 1]),
                           pack_f16x2(v[8 * j + 2], v[8 * j + 3]), pack_f16x2(v[8 * j + 4], v[8 * j + 5]),
                           pack_f16x2(v[8 * j + 6], v[8 * j + 7]));
            } else {
              st_shared_v4(row_addr + chunk * 16, pack_bf16x2(v[8 * j + 0], v[8 * j + 1]),
                           pack_bf16x2(v[8 * j + 2], v[8 * j + 3]), pack_bf16x2(v[8 * j + 4], v[8 * j + 5]),
                           pack_bf16x2(v[8 * j + 6], v[8 * j + 7]));
            }
          }
        } else if (row < p.M) {
          uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + static_cast<long long>(row) * p.ldy + c_first;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c_first + j < p.N) dst[j] = to_out16(v[j], p.out_fp16);
          }
        }
      }
      if (p.use_tma_store) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.M && box_col < p.N) tma_store_2d(&tm_y, sbuf, box_col, row0);
        if (lane == 0) tma_store_commit();
        ++store_count;
      }
    }
    if (p.use_tma_store && lane == 0) tma_store_wait_all();
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc<1>(tmem_base, 256);
}

}  // namespace

cudaError_t launch_gemm_splitk(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                               const TcParams& p, int tiles, int split, cudaStream_t stream) {
  constexpr int kSmemBytes = kRingBytes + kEpiBytes + kBarBytes + 1024;
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 64 && !configured[dev]) {
    err = cudaFuncSetAttribute(gemm_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return err;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * split), 1, 1);
  cfg.blockDim = dim3(Geo::kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_splitk_kernel, tm_x, tm_w, tm_y, p, split);
}

}  // namespace b200fp8
