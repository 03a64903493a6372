// Large-M FP8 rowwise GEMM for sm_100a: persistent, warp-specialised tcgen05 kernel.
//
//   Y[m,n] = bf16( (sum_k X[m,k] * W[n,k]) * x_scale[m] * w_scale[n] (+ bias[n]) )
//
// One CTA (kCtaGroup = 1) or a CTA pair of one cluster (kCtaGroup = 2, tcgen05 cta_group::2)
// owns a tile of 128*kCtaGroup rows by 256 columns of Y at a time and walks a static list of
// tiles (tile = cluster index + i * number of clusters).
//
//   warp 0     TMA producer: X box {128 B of K, 128 rows} and W box {128 B of K, 256/kCtaGroup rows}
//              per k-block into a ring of 128-byte-swizzled stages (no cluster multicast anywhere);
//   warp 1     allocates TMEM (512 columns = two 256-column fp32 accumulators); one lane of the
//              leader CTA issues 4 x tcgen05.mma (K = 32 each) per stage and commits to mbarriers;
//   warps 2-5  epilogue: tcgen05.ld one TMEM lane quarter each, multiply by x_scale[m]*w_scale[n],
//              add bias, round to bf16, stage 32x64 boxes in swizzled shared memory, TMA-store.
//
// Grouped mode (both variants; a mixture-of-experts layer): the rows of X are partitioned into
// groups by a device array of group sizes, group g multiplies rows g*N..(g+1)*N of the stacked W.
// The tile list is then built on the device from the group sizes (no host round trip); a tile never
// writes rows of the next group: boxes that straddle a group's end are stored with plain predicated
// stores instead of TMA.
//
// Gathered output (the sharded run): a tile's boxes are TMA-stored not only into Y but into up to seven more
// buffers - the other GPUs' copies of the gathered matrix, reached through peer mappings - so the all-gather of
// Y travels over NVLink from inside the epilogue, tile by tile, while the tensor cores multiply the next tile.
//
// The accumulator is double buffered in TMEM, so the epilogue of tile i overlaps the main loop
// of tile i+1.  Every mbarrier wait is bounded (ptx.cuh: mbar_wait); on a time-out the kernel
// records a status word and all roles fall through to the common exit, which frees TMEM.
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

enum WaitSite : uint32_t {
  kSiteProducerEmpty = 0x101,
  kSiteMmaTmemEmpty = 0x102,
  kSiteMmaFull = 0x103,
  kSiteEpiTmemFull = 0x104,
  kSiteDrain = 0x105,
};

struct TileCoord {
  int m_tile;
  int n_tile;
};

// Grouped rasterisation: tiles are numbered down a column of `group_m` row-tiles, then across
// N, then to the next group, so that the tiles in flight at one time share X and W panels in L2.
__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n, int group_m) {
  const int per_group = group_m * tiles_n;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int rows = min(group_m, tiles_m - first_m);
  const int r = t - g * per_group;
  TileCoord c;
  c.m_tile = first_m + r % rows;
  c.n_tile = r / rows;
  return c;
}

// Everything a role needs to know about one tile.
struct TileInfo {
  int row0;       // first row of X / Y of the CTA's 128-row block
  int row_limit;  // rows >= row_limit are not this tile's to write (end of M, or end of the group)
  int col0;       // first column of Y
  int w_row0;     // first row of W of the CTA's share
  int scale_col0; // index of w_scale / bias of column col0 (differs from col0 in grouped mode)
};

struct TileSpace {
  int M, N, tiles_n, group_m;
  int num_groups;         // 0: plain GEMM
  const int* group_rows;  // [num_groups] rows of X per group (device memory)
  int plain_tiles_m;
};

__device__ __forceinline__ int count_tiles(const TileSpace& ts, int tile_m) {
  if (ts.num_groups == 0) return ts.plain_tiles_m * ts.tiles_n;
  int total = 0;
  for (int g = 0; g < ts.num_groups; ++g) total += ((__ldg(ts.group_rows + g) + tile_m - 1) / tile_m) * ts.tiles_n;
  return total;
}

template <int kCtaGroup>
__device__ __forceinline__ TileInfo tile_info(const TileSpace& ts, int t, uint32_t cta_rank) {
  using Cfg = TcConfig<kCtaGroup>;
  TileInfo ti;
  if (ts.num_groups == 0) {
    const TileCoord tc = tile_coord(t, ts.plain_tiles_m, ts.tiles_n, ts.group_m);
    ti.row0 = tc.m_tile * Cfg::kTileM + static_cast<int>(cta_rank) * Cfg::kBlockM;
    ti.row_limit = ts.M;
    ti.col0 = tc.n_tile * Cfg::kBlockN;
    ti.w_row0 = ti.col0 + static_cast<int>(cta_rank) * Cfg::kRowsW;
    ti.scale_col0 = ti.col0;
    return ti;
  }
  int first_tile = 0, first_row = 0;
  int g = 0, rows = 0, tiles_m = 0;
  for (; g < ts.num_groups; ++g) {
    rows = __ldg(ts.group_rows + g);
    tiles_m = (rows + Cfg::kTileM - 1) / Cfg::kTileM;
    if (t < first_tile + tiles_m * ts.tiles_n) break;
    first_tile += tiles_m * ts.tiles_n;
    first_row += rows;
  }
  const TileCoord tc = tile_coord(t - first_tile, tiles_m, ts.tiles_n, ts.group_m);
  ti.row0 = first_row + tc.m_tile * Cfg::kTileM + static_cast<int>(cta_rank) * Cfg::kBlockM;
  ti.row_limit = min(first_row + rows, ts.M);
  ti.col0 = tc.n_tile * Cfg::kBlockN;
  ti.w_row0 = g * ts.N + ti.col0 + static_cast<int>(cta_rank) * Cfg::kRowsW;
  ti.scale_col0 = g * ts.N + ti.col0;
  return ti;
}

template <int kCtaGroup>
__global__ void __launch_bounds__(TcGeometry::kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_y, const TcParams p, const __grid_constant__ ExtraOutputs extra) {
  using Cfg = TcConfig<kCtaGroup>;
  constexpr bool kPair = kCtaGroup == 2;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + kStages * Cfg::kBytesA;
  const uint32_t smem_epi = smem_b + kStages * Cfg::kBytesB;
  const uint32_t bars = smem_epi + Cfg::kEpiBytes;
  const uint32_t bar_full = bars;                          // [kStages]
  const uint32_t bar_empty = bars + 8 * kStages;           // [kStages]
  const uint32_t bar_tmem_full = bars + 16 * kStages;      // [2]
  const uint32_t bar_tmem_empty = bar_tmem_full + 16;      // [2]
  const uint32_t tmem_slot = bar_tmem_empty + 16;          // u32 written by tcgen05.alloc
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kPair ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / kCtaGroup;
  const int num_clusters = gridDim.x / kCtaGroup;

  TileSpace ts;
  ts.M = p.M;
  ts.N = p.N;
  ts.tiles_n = (p.N + Cfg::kBlockN - 1) / Cfg::kBlockN;
  ts.group_m = p.group_m;
  ts.num_groups = p.num_groups;
  ts.group_rows = p.group_rows;
  ts.plain_tiles_m = (p.M + Cfg::kTileM - 1) / Cfg::kTileM;
  const int num_tiles = count_tiles(ts, Cfg::kTileM);
  const int num_kb = (p.K + Cfg::kBlockK - 1) / Cfg::kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tmem_full + 8 * b, 1);
      mbar_init(bar_tmem_empty + 8 * b, 4 * kCtaGroup);  // one arrival per epilogue warp of the pair
    }
    *abort_flag = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    if (p.use_tma_store) prefetch_tensormap(&tm_y);
    for (int e = 0; e < p.num_extra; ++e) prefetch_tensormap(&extra.tm[e]);
    if constexpr (!kPair) {
      // Single CTA: the first pass over the ring needs no waiting, so it starts before the set-up barrier
      // (a CTA pair cannot: the peer's loads credit the leader's barriers, which must exist first).
      if (cluster_id < num_tiles) {
        const TileInfo ti = tile_info<kCtaGroup>(ts, cluster_id, 0u);
        for (int kb = 0; kb < num_kb && kb < kStages; ++kb) {
          const uint32_t full = bar_full + 8 * kb;
          mbar_arrive_expect_tx(full, Cfg::kStageTxBytes);
          tma_load_2d(smem_a + kb * Cfg::kBytesA, &tm_x, full, kb * Cfg::kBlockK, ti.row0);
          tma_load_2d(smem_b + kb * Cfg::kBytesB, &tm_w, full, kb * Cfg::kBlockK, ti.w_row0);
        }
      }
    }
  }
  if (warp == 1) {
    tmem_alloc<kCtaGroup>(tmem_slot, 512);
    tmem_relinquish<kCtaGroup>();
  }
  tc_fence_before_sync();
  if constexpr (kPair) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      // k-blocks of the first tile already issued before the set-up barrier (single CTA only)
      const int pre = kPair ? 0 : (num_kb < kStages ? num_kb : kStages);
      uint32_t stage = static_cast<uint32_t>(pre % kStages), phase = static_cast<uint32_t>(pre / kStages) & 1u;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        const TileInfo ti = tile_info<kCtaGroup>(ts, t, cta_rank);
        const int row_x = ti.row0;
        const int row_w = ti.w_row0;
        for (int kb = (t == cluster_id ? pre : 0); kb < num_kb; ++kb) {
          ok = mbar_wait<kPair>(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty);
          if (!ok) break;
          const uint32_t dst_a = smem_a + stage * Cfg::kBytesA;
          const uint32_t dst_b = smem_b + stage * Cfg::kBytesB;
          if constexpr (kPair) {
            // both CTAs credit the leader's barrier; the leader alone announces the byte total
            const uint32_t full = mapa_cluster(bar_full + 8 * stage, 0);
            if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, Cfg::kStageTxBytes);
            tma_load_2d_pair(dst_a, &tm_x, full, kb * Cfg::kBlockK, row_x);
            tma_load_2d_pair(dst_b, &tm_w, full, kb * Cfg::kBlockK, row_w);
          } else {
            const uint32_t full = bar_full + 8 * stage;
            mbar_arrive_expect_tx(full, Cfg::kStageTxBytes);
            tma_load_2d(dst_a, &tm_x, full, kb * Cfg::kBlockK, row_x);
            tma_load_2d(dst_b, &tm_w, full, kb * Cfg::kBlockK, row_w);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Gave up: give the loads this thread already issued a bounded time to land before the
        // CTA leaves (the consumer of a full barrier is gone, so just watch the clock).
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------- MMA issuer --------------------------------
    if (cta_rank == 0 && lane == 0) {
      constexpr uint32_t idesc = instr_desc_e4m3(Cfg::kTileM, Cfg::kBlockN);
      uint32_t stage = 0, phase = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
        const uint32_t buf = local_tile & 1u;
        const uint32_t use = (local_tile >> 1) & 1u;
        ok = mbar_wait<kPair>(bar_tmem_empty + 8 * buf, use ^ 1u, abort_flag, p.status, kSiteMmaTmemEmpty);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * Cfg::kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait<kPair>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t a_desc = smem_desc_k_sw128(smem_a + stage * Cfg::kBytesA);
          const uint64_t b_desc = smem_desc_k_sw128(smem_b + stage * Cfg::kBytesB);
#pragma unroll
          for (int k = 0; k < Cfg::kBlockK / 32; ++k) {
            // +2 in the address field = +32 bytes = the next K=32 slice inside the swizzled row
            tc_mma_f8<kCtaGroup>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if constexpr (kPair) {
            tc_commit_pair(bar_empty + 8 * stage, 0x3);
          } else {
            tc_commit(bar_empty + 8 * stage);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if constexpr (kPair) {
          tc_commit_pair(bar_tmem_full + 8 * buf, 0x3);
        } else {
          tc_commit(bar_tmem_full + 8 * buf);
        }
      }
    }
  } else {
    // ---------------------------------- epilogue ---------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const uint32_t stage_buf = smem_epi + quarter * (2 * Cfg::kStoreRows * Cfg::kStoreCols * 2);
    const uint32_t tmem_empty_remote = kPair ? mapa_cluster(bar_tmem_empty, 0) : bar_tmem_empty;
    const uint64_t y_policy = l2_policy_evict_first();
    uint32_t local_tile = 0;
    uint32_t store_count = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local_tile) {
      const TileInfo ti = tile_info<kCtaGroup>(ts, t, cta_rank);
      const uint32_t buf = local_tile & 1u;
      const uint32_t use = (local_tile >> 1) & 1u;
      const int row0 = ti.row0 + quarter * 32;
      const int row = row0 + lane;
      const int col0 = ti.col0;
      const int row_limit = ti.row_limit;
      const float* w_scale = p.w_scale + (ti.scale_col0 - col0);  // w_scale[column] for this tile's group
      const __nv_bfloat16* bias = p.bias != nullptr ? p.bias + (ti.scale_col0 - col0) : nullptr;
      // a box whose 32 rows straddle the end of a group must not be stored whole
      const bool box_rows_whole = ts.num_groups == 0 || row0 + Cfg::kStoreRows <= row_limit;
      const bool tma_box = p.use_tma_store && box_rows_whole;
      const float xs = row < row_limit ? __ldg(p.x_scale + row) : 0.0f;

      ok = mbar_wait<kPair>(bar_tmem_full + 8 * buf, use, abort_flag, p.status, kSiteEpiTmemFull);
      ok = __all_sync(0xffffffffu, ok) != 0;  // the whole warp leaves together
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * Cfg::kBlockN;

      // The common case - whole tile inside Y, bf16, no bias, TMA boxes - runs a loop of its own that is a fraction of
      // the general loop's code: the four epilogue warps of a short-K problem are otherwise held up fetching
      // instructions (the general loop is unrolled over every combination of edge, bias and output type).
      const bool lean = tma_box && bias == nullptr && !p.out_fp16 && col0 + Cfg::kBlockN <= p.N &&
                        (reinterpret_cast<uintptr_t>(w_scale + col0) & 15u) == 0;
      if (lean) {
#pragma unroll 1
        for (int box = 0; box < Cfg::kBlockN / Cfg::kStoreCols; ++box) {
          const int box_col = col0 + box * Cfg::kStoreCols;
          const uint32_t sbuf = stage_buf + (store_count & 1u) * (Cfg::kStoreRows * Cfg::kStoreCols * 2);
          // both 32-column reads of the box and its 64 column scales are requested before anything is waited for
          uint32_t acc[Cfg::kStoreCols];
          tmem_ld_32x32(t_addr + box * Cfg::kStoreCols, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
          tmem_ld_32x32(t_addr + box * Cfg::kStoreCols + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
          const float4* ws4 = reinterpret_cast<const float4*>(w_scale + box_col);
          float4 ws[Cfg::kStoreCols / 4];
#pragma unroll
          for (int j = 0; j < Cfg::kStoreCols / 4; ++j) ws[j] = __ldg(ws4 + j);
          if (lane == 0) tma_store_wait_read<1>();  // the buffer about to be rewritten: source of the store before last
          __syncwarp();
          const uint32_t row_addr = sbuf + lane * 128;
          tmem_ld_wait();
          if (box == Cfg::kBlockN / Cfg::kStoreCols - 1) {
            tc_fence_before_sync();  // accumulator fully read: hand the TMEM buffer back to the MMA issuer
            __syncwarp();
            if (lane == 0) {
              if constexpr (kPair) {
                mbar_arrive_cluster(tmem_empty_remote + 8 * buf);
              } else {
                mbar_arrive(bar_tmem_empty + 8 * buf);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < Cfg::kStoreCols / 8; ++j) {
            const float4 wa = ws[2 * j], wb = ws[2 * j + 1];
            const uint32_t chunk = static_cast<uint32_t>(j ^ (lane & 7));
            st_shared_v4(row_addr + chunk * 16,
                         pack_bf16x2(__uint_as_float(acc[8 * j + 0]) * (xs * wa.x), __uint_as_float(acc[8 * j + 1]) * (xs * wa.y)),
                         pack_bf16x2(__uint_as_float(acc[8 * j + 2]) * (xs * wa.z), __uint_as_float(acc[8 * j + 3]) * (xs * wa.w)),
                         pack_bf16x2(__uint_as_float(acc[8 * j + 4]) * (xs * wb.x), __uint_as_float(acc[8 * j + 5]) * (xs * wb.y)),
                         pack_bf16x2(__uint_as_float(acc[8 * j + 6]) * (xs * wb.z), __uint_as_float(acc[8 * j + 7]) * (xs * wb.w)));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (row0 < row_limit) {
              if (p.y_evict_first) {
                tma_store_2d_hint(&tm_y, sbuf, box_col, row0, y_policy);
              } else {
                tma_store_2d(&tm_y, sbuf, box_col, row0);
              }
              for (int e = 0; e < p.num_extra; ++e) tma_store_2d(&extra.tm[e], sbuf, box_col, row0);
            }
            tma_store_commit();
          }
          ++store_count;
        }
        continue;
      }

#pragma unroll 1
      for (int box = 0; box < Cfg::kBlockN / Cfg::kStoreCols; ++box) {
        const int box_col = col0 + box * Cfg::kStoreCols;
        const uint32_t sbuf = stage_buf + (store_count & 1u) * (Cfg::kStoreRows * Cfg::kStoreCols * 2);
        if (tma_box) {
          // the buffer about to be rewritten was the source of the store before last
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t acc[32];
          tmem_ld_32x32(t_addr + box * Cfg::kStoreCols + half * 32, acc);
          tmem_ld_wait();
          if (box == Cfg::kBlockN / Cfg::kStoreCols - 1 && half == 1) {
            // accumulator fully read: hand the TMEM buffer back to the MMA issuer
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if constexpr (kPair) {
                mbar_arrive_cluster(tmem_empty_remote + 8 * buf);
              } else {
                mbar_arrive(bar_tmem_empty + 8 * buf);
              }
            }
          }
          const int c_first = box_col + half * 32;
          float v[32];
          const bool vec_ok = (c_first + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(w_scale + c_first) & 15u) == 0);
          if (vec_ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 ws = __ldg(reinterpret_cast<const float4*>(w_scale + c_first) + j);
              v[4 * j + 0] = __uint_as_float(acc[4 * j + 0]) * (xs * ws.x);
              v[4 * j + 1] = __uint_as_float(acc[4 * j + 1]) * (xs * ws.y);
              v[4 * j + 2] = __uint_as_float(acc[4 * j + 2]) * (xs * ws.z);
              v[4 * j + 3] = __uint_as_float(acc[4 * j + 3]) * (xs * ws.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float ws = (c_first + j < p.N) ? __ldg(w_scale + c_first + j) : 0.0f;
              v[j] = __uint_as_float(acc[j]) * (xs * ws);
            }
          }
          if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c_first + j < p.N) v[j] += __bfloat162float(bias[c_first + j]);
            }
          }
          if (tma_box) {
            // row `lane` of the box is 128 bytes; 16-byte chunk j sits at chunk (j ^ (lane & 7))
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
          } else if (row < row_limit) {
            uint16_t* dst = reinterpret_cast<uint16_t*>(p.y) + static_cast<long long>(row) * p.ldy + c_first;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c_first + j < p.N) dst[j] = to_out16(v[j], p.out_fp16);
            }
          }
        }
        if (tma_box) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < row_limit && box_col < p.N) {
            if (p.y_evict_first) {
              tma_store_2d_hint(&tm_y, sbuf, box_col, row0, y_policy);
            } else {
              tma_store_2d(&tm_y, sbuf, box_col, row0);
            }
            // gathered output: the same box into every other copy of Y (peer GPUs' memory over NVLink); the
            // stores share this box's bulk group, so the staging buffer is reused only when all have read it
            for (int e = 0; e < p.num_extra; ++e) tma_store_2d(&extra.tm[e], sbuf, box_col, row0);
          }
          if (lane == 0) tma_store_commit();
          ++store_count;
        }
      }
    }
    if (p.use_tma_store && lane == 0) tma_store_wait_all();
  }

  // ------------------------------------ common exit ------------------------------------
  __syncwarp();  // single-lane roles rejoin their warp before the aligned barriers below
  tc_fence_before_sync();
  if constexpr (kPair) {
    cluster_sync_all();
  } else {
    __syncthreads();
  }
  tc_fence_after_sync();
  if (warp == 1) {
    tmem_dealloc<kCtaGroup>(tmem_base, 512);
  }
}

}  // namespace

template <int kCtaGroup>
cudaError_t launch_gemm_tc(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                           const TcParams& p, int num_ctas, cudaStream_t stream, const ExtraOutputs* extra) {
  static const ExtraOutputs no_extra = {};
  if (extra == nullptr) {
    if (p.num_extra != 0) return cudaErrorInvalidValue;
    extra = &no_extra;
  }
  using Cfg = TcConfig<kCtaGroup>;
  auto kernel = gemm_tc_kernel<kCtaGroup>;
  // Opt in to the large dynamic shared-memory size once per device.
  static bool configured[64] = {};
  static std::mutex mutex;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (dev < 64 && !configured[dev]) {
      err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
      if (err != cudaSuccess) return err;
      configured[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(num_ctas), 1, 1);
  cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtaGroup;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, tm_x, tm_w, tm_y, p, *extra);
}

template cudaError_t launch_gemm_tc<1>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&,
                                       int, cudaStream_t, const ExtraOutputs*);
template cudaError_t launch_gemm_tc<2>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const TcParams&,
                                       int, cudaStream_t, const ExtraOutputs*);

}  // namespace b200fp8
