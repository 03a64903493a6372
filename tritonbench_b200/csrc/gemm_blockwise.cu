// FP8 GEMM with 128x128 block scales for sm_100a:
//
//   Y[m,n] = bf16( sum_kb ( sum_{k in block kb} X[m,k] * W[n,k] ) * x_scale[m/128, kb] * w_scale[n/128, kb] )
//
// The scales change with the k-block, so the tensor core cannot accumulate across k-blocks: every
// k-block's 128x256 product is accumulated on its own in TMEM (4 x tcgen05.mma, K = 32 each), read back
// by the epilogue warps, multiplied by that block's scale and added to fp32 accumulators in registers
// ("promotion").  Two TMEM buffers alternate per k-block, so the tensor core multiplies block kb+1
// while the CUDA cores promote block kb.
//
//   warp 0      TMA producer (X box 128x128 B, W box 256x128 B per k-block, 4-stage ring, 128B swizzle)
//   warp 1      TMEM owner + MMA issuer
//   warps 2-3   idle (they complete the first warpgroup, which gives its registers away)
//   warps 4-11  promotion + epilogue: warp w owns TMEM lane quarter w%4 (32 rows) and column half
//               (w-4)/4 (128 columns = one scale block of W): 128 fp32 accumulators per thread
//
// A promotion thread holds 128 accumulators plus two 32-column read buffers, two TMEM reads in flight at a
// time, and folds the products in with packed fp32 FMAs (fma.rn.f32x2); that needs about 210 registers.  The kernel
// starts with 168 per thread (384 threads) and moves registers from the first warpgroup (40 each)
// to the two promotion warpgroups (232 each) with setmaxnreg.
//
// Persistent over a static tile list; every mbarrier wait is bounded.
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

using Geo = TcGeometry;
constexpr int kThreadsBw = 384;
constexpr int kFirstEpiWarp = 4;
constexpr int kRegsRoles = 40;
constexpr int kRegsPromotion = 232;  // 128 * 40 + 256 * 232 == 384 * 168
constexpr int kStages = 4;
constexpr int kBytesA = Geo::kBlockM * Geo::kBlockK;  // 16 KiB
constexpr int kBytesB = Geo::kBlockN * Geo::kBlockK;  // 32 KiB
constexpr int kEpiWarps = 8;
constexpr int kEpiBytes = kEpiWarps * Geo::kStoreRows * Geo::kStoreCols * 2;  // one 4 KiB box per warp
constexpr int kBarBytes = 256;
constexpr int kSmemBytesBw = kStages * (kBytesA + kBytesB) + kEpiBytes + kBarBytes + 1024;
constexpr int kScaleBlock = 128;

enum WaitSite : uint32_t {
  kSiteProducerEmpty = 0x401,
  kSiteMmaAccEmpty = 0x402,
  kSiteMmaFull = 0x403,
  kSiteEpiAccFull = 0x404,
};

struct TileCoord {
  int m_tile;
  int n_tile;
};

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

__global__ void __launch_bounds__(kThreadsBw, 1)
gemm_blockwise_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_y, const BlockwiseParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + kStages * kBytesA;
  const uint32_t smem_epi = smem_b + kStages * kBytesB;
  const uint32_t bars = smem_epi + kEpiBytes;
  const uint32_t bar_full = bars;                       // [kStages]
  const uint32_t bar_empty = bars + 8 * kStages;        // [kStages]
  const uint32_t bar_acc_full = bars + 16 * kStages;    // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;     // [2]
  const uint32_t tmem_slot = bar_acc_empty + 16;
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = static_cast<int>(blockIdx.x);
  const int num_ctas = static_cast<int>(gridDim.x);

  const int tiles_m = (p.M + Geo::kBlockM - 1) / Geo::kBlockM;
  const int tiles_n = (p.N + Geo::kBlockN - 1) / Geo::kBlockN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + Geo::kBlockK - 1) / Geo::kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
    }
    *abort_flag = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    if (p.use_tma_store) prefetch_tensormap(&tm_y);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp < kFirstEpiWarp) {
    setmaxnreg_dec<kRegsRoles>();
  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += num_ctas) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n, p.group_m);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait<false>(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty);
          if (!ok) break;
          const uint32_t full = bar_full + 8 * stage;
          mbar_arrive_expect_tx(full, kBytesA + kBytesB);
          tma_load_2d(smem_a + stage * kBytesA, &tm_x, full, kb * Geo::kBlockK, tc.m_tile * Geo::kBlockM);
          tma_load_2d(smem_b + stage * kBytesB, &tm_w, full, kb * Geo::kBlockK, tc.n_tile * Geo::kBlockN);
          if (++stage == kStages) {
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
      constexpr uint32_t idesc = instr_desc_e4m3(Geo::kBlockM, Geo::kBlockN);
      uint32_t stage = 0, phase = 0;
      uint32_t block_no = 0;  // k-blocks issued so far, over all tiles: selects the TMEM buffer
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += num_ctas) {
        for (int kb = 0; kb < num_kb; ++kb, ++block_no) {
          const uint32_t buf = block_no & 1u;
          const uint32_t use = (block_no >> 1) & 1u;
          ok = mbar_wait<false>(bar_acc_empty + 8 * buf, use ^ 1u, abort_flag, p.status, kSiteMmaAccEmpty);
          if (!ok) break;
          ok = mbar_wait<false>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * Geo::kBlockN;
          const uint64_t a_desc = smem_desc_k_sw128(smem_a + stage * kBytesA);
          const uint64_t b_desc = smem_desc_k_sw128(smem_b + stage * kBytesB);
#pragma unroll
          for (int k = 0; k < Geo::kBlockK / 32; ++k) {
            tc_mma_f8<1>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k > 0 ? 1u : 0u);  // one k-block per buffer
          }
          tc_commit(bar_empty + 8 * stage);
          tc_commit(bar_acc_full + 8 * buf);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  }
  } else {
    // ------------------------------ promotion + epilogue -----------------------------
    setmaxnreg_inc<kRegsPromotion>();
    const int epi = warp - kFirstEpiWarp;
    const int quarter = warp & 3;      // TMEM lanes [32*quarter, +32)
    const int half = epi >> 2;         // columns [128*half, +128) of the tile: one scale block of W
    const uint32_t sbuf = smem_epi + epi * (Geo::kStoreRows * Geo::kStoreCols * 2);
    const int scale_rows_x = (p.M + kScaleBlock - 1) / kScaleBlock;
    const int scale_rows_w = (p.N + kScaleBlock - 1) / kScaleBlock;
    uint32_t block_no = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += num_ctas) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n, p.group_m);
      const int row0 = tc.m_tile * Geo::kBlockM + quarter * 32;
      const int row = row0 + lane;
      const int col0 = tc.n_tile * Geo::kBlockN + half * 128;
      const int xb = min(tc.m_tile, scale_rows_x - 1);               // the tile's 128 rows are one scale block of X
      const int wb = min(col0 / kScaleBlock, scale_rows_w - 1);
      const float* xs = p.x_scale + static_cast<long long>(xb) * p.ld_xs;
      const float* ws = p.w_scale + static_cast<long long>(wb) * p.ld_ws;

      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.0f;

      for (int kb = 0; kb < num_kb; ++kb, ++block_no) {
        const uint32_t buf = block_no & 1u;
        const uint32_t use = (block_no >> 1) & 1u;
        const float s = __ldg(xs + kb) * __ldg(ws + kb);  // issued before the wait below; measured: not on the critical path
        ok = mbar_wait<false>(bar_acc_full + 8 * buf, use, abort_flag, p.status, kSiteEpiAccFull);
        ok = __all_sync(0xffffffffu, ok) != 0;
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * Geo::kBlockN + half * 128;
        // four 32-column reads through two 32-register buffers, two reads in flight at a time; the products are
        // folded in with packed fp32 FMAs (two per instruction), so that from "buffer full" to "buffer free" a
        // warp spends two read latencies and 32 instructions
        uint32_t part0[32], part1[32];
        tmem_ld_32x32(t_addr, part0);
        tmem_ld_32x32(t_addr + 32, part1);
        tmem_ld_wait_for(part0);
        keep_below(part1);
#pragma unroll
        for (int j = 0; j < 32; j += 2) fma2(acc[j], acc[j + 1], part0[j], part0[j + 1], s);
        tmem_ld_32x32(t_addr + 64, part0);
#pragma unroll
        for (int j = 0; j < 32; j += 2) fma2(acc[32 + j], acc[33 + j], part1[j], part1[j + 1], s);
        tmem_ld_32x32(t_addr + 96, part1);
        tmem_ld_wait_for(part0);
        keep_below(part1);
        // the whole buffer is in registers: hand it back before the second half of the arithmetic
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
#pragma unroll
        for (int j = 0; j < 32; j += 2) fma2(acc[64 + j], acc[65 + j], part0[j], part0[j + 1], s);
#pragma unroll
        for (int j = 0; j < 32; j += 2) fma2(acc[96 + j], acc[97 + j], part1[j], part1[j + 1], s);
      }
      if (!ok) break;

      // the tile is complete: round and store this warp's 32 x 128 part as two 32 x 64 boxes
#pragma unroll
      for (int box = 0; box < 2; ++box) {
        const int box_col = col0 + box * Geo::kStoreCols;
        if (p.use_tma_store) {
          if (lane == 0) tma_store_wait_read<0>();  // single staging box per warp
          __syncwarp();
          const uint32_t row_addr = sbuf + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float* v = acc + box * 64 + j * 8;
            const uint32_t chunk = static_cast<uint32_t>(j ^ (lane & 7));
            st_shared_v4(row_addr + chunk * 16, pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                         pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M && box_col < p.N) tma_store_2d(&tm_y, sbuf, box_col, row0);
          if (lane == 0) tma_store_commit();
        } else if (row < p.M) {
          __nv_bfloat16* dst = p.y + static_cast<long long>(row) * p.ldy + box_col;
#pragma unroll
          for (int j = 0; j < 64; ++j) {
            if (box_col + j < p.N) dst[j] = __float2bfloat16_rn(acc[box * 64 + j]);
          }
        }
      }
    }
    if (p.use_tma_store && lane == 0) tma_store_wait_all();
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc<1>(tmem_base, 512);
}

}  // namespace

cudaError_t launch_gemm_blockwise(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                                  const BlockwiseParams& p, int num_ctas, cudaStream_t stream) {
  static bool configured[64] = {};
  static std::mutex mutex;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (dev < 64 && !configured[dev]) {
      err = cudaFuncSetAttribute(gemm_blockwise_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesBw);
      if (err != cudaSuccess) return err;
      configured[dev] = true;
    }
  }
  gemm_blockwise_kernel<<<num_ctas, kThreadsBw, kSmemBytesBw, stream>>>(tm_x, tm_w, tm_y, p);
  return cudaGetLastError();
}

}  // namespace b200fp8
