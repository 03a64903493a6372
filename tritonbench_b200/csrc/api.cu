// C ABI of the library (declared in include/b200fp8.h): argument checks, the choice of kernel
// variant, TMA descriptor encoding, workspace layout, and the host-buffer context.
#include <cudaTypedefs.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <new>

#include "../../include/b200fp8.h"
#include "kernels.h"

namespace {

using namespace b200fp8;

thread_local int g_last_cuda_error = 0;

struct DeviceInfo {
  bool known = false;
  int cc_major = 0;
  int sm_count = 0;
  int max_pair_clusters = 0;
  int split_clusters[4] = {0, 0, 0, 0};  // resident clusters of 1, 2, 4, 8 CTAs of the one-tile-per-cluster kernel
};

std::mutex g_mutex;
DeviceInfo g_devices[64];
PFN_cuTensorMapEncodeTiled g_encode = nullptr;

int note_cuda(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return e == cudaSuccess ? B200FP8_OK : B200FP8_LAUNCH_FAILED;
}

int device_info(DeviceInfo* out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return note_cuda(e);
  if (dev < 0 || dev >= 64) return B200FP8_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_devices[dev];
  if (!d.known) {
    e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return note_cuda(e);
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return note_cuda(e);
    d.max_pair_clusters = d.sm_count / 2;
    d.split_clusters[0] = d.sm_count;
    for (int i = 1; i < 4; ++i) {
      d.split_clusters[i] = d.cc_major == 10 ? splitk_resident_clusters(1 << i, &e) : 0;
      if (d.split_clusters[i] <= 0) d.split_clusters[i] = (d.sm_count * 7 / 8) >> i;  // query unavailable: a guess
    }
    d.known = true;
  }
  if (g_encode == nullptr) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return note_cuda(e);
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr) {
      g_last_cuda_error = static_cast<int>(cudaErrorSymbolNotFound);
      return B200FP8_LAUNCH_FAILED;
    }
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
  }
  *out = d;
  return B200FP8_OK;
}

// 2-D row-major tensor [rows, cols] with row pitch `pitch_bytes`; box {box_cols, box_rows};
// 128-byte swizzle (box_cols * elem_bytes must be 128); out-of-range elements read as zero.
int encode_2d(CUtensorMap* tm, CUtensorMapDataType dtype, int elem_bytes, const void* ptr, uint64_t rows,
              uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols, uint32_t box_rows) {
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  (void)elem_bytes;
  const CUresult r = g_encode(tm, dtype, 2, const_cast<void*>(ptr), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return B200FP8_LAUNCH_FAILED;
  }
  return B200FP8_OK;
}

// Height of a rasterisation group of the persistent kernels, in row tiles: the tiles of a group are walked down
// its rows first, so one column panel of W serves the whole group from L2 and W is read from HBM once per group.
// 16 row tiles when their X panel (16 x tile_m x K bytes) still leaves room in L2 for the W panels in flight and
// the problem has at least one full group; 8 otherwise.  Measured, microseconds per launch for heights 8 / 16:
// 8192^3 377.6 / 370.9, 4096x14336x4096 177.7 / 174.2 (sustained 8192^3 439 / 429); 16384x8192x13312 1225 / 1235,
// 16384x4096x16384 765 / 770, 3000x7168x2048 41.8 / 42.4 (fewer than 16 row tiles); 24 and more lose everywhere.
int choose_group_m(int64_t M, int64_t K, int tile_m) {
  const int64_t tiles_m = (M + tile_m - 1) / tile_m;
  return tiles_m >= 16 && 16.0 * tile_m * static_cast<double>(K) <= 36.0e6 ? 16 : 8;
}

// An output of 64 MB and more cannot stay in the 126 MB L2 next to the operand panels anyway: its stores carry the
// evict-first hint, so that they push out each other rather than the X and W panels the next tiles re-read
// (8192^3: 370.7 -> 369.7 us per launch, sustained 422.8 -> 419.8 us).  A smaller Y is left alone: the kernel that
// consumes it may find it in L2.
bool y_streams_past_l2(int64_t M, int64_t N) { return 2.0 * static_cast<double>(M) * static_cast<double>(N) >= 64.0e6; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct Plan {
  uint32_t variant;
  bool tma_store;
  int num_ctas;      // tcgen05 variants
  int group_m;
  SplitPlan splitk;  // one-tile-per-cluster variant
  SkinnyPlan skinny;  // skinny variant
  GemvPlan gemv;      // GEMV variant
  size_t workspace_bytes;
};

// The tcgen05 kernels read X and W through TMA: rows must start on 16-byte boundaries.
bool tma_loadable(int64_t K, int64_t ldx, int64_t ldw, const void* xq, const void* wq) {
  (void)K;
  return ldx % 16 == 0 && ldw % 16 == 0 && aligned16(xq) && aligned16(wq);
}

}  // namespace

namespace b200fp8 {

// Cost model of the one-tile-per-cluster kernel, in microseconds, fitted to graph-replay timings of every
// (block_n, split) on 45 shapes (mean regret of the model's pick against the best measured: 2 %, worst 14 %).
// A CTA's main loop is the slowest of: its bytes at the rate its ring sustains (bytes in flight / latency),
// its MMAs, and the whole wave's bytes at chip bandwidth (L2 for re-read operands, HBM for the unique bytes).
// Then the DSMEM exchange and the epilogue; all of it once per wave of resident clusters.
double split_plan_cost_us(long long M, long long N, long long K, int block_n, int split, int resident_clusters) {
  const double kLaunch = 1.0, kLatency = 2.17, kRingLatency = 0.81, kMmaPerColumn = 0.9e-3, kPerKBlock = 0.151;
  const double kL2BytesPerUs = 13.5e6, kHbmBytesPerUs = 6.0e6, kL2ResidentBytes = 120.0e6;
  const double kHbmBytesPerUsPerSm = 0.058e6;
  const double kExchangeFixed = 0.93, kExchangePerByte = 41.5e-6, kEpilogue = 0.11;
  const long long tiles = ((M + 127) / 128) * ((N + block_n - 1) / block_n);
  const long long kb = (K + TcGeometry::kBlockK - 1) / TcGeometry::kBlockK;
  const long long kb_per = (kb + split - 1) / split;
  const long long rows_a = M >= 128 ? 128 : (M + 7) / 8 * 8;
  const long long waves = (tiles + resident_clusters - 1) / resident_clusters;
  const double stage_bytes = static_cast<double>((rows_a + block_n) * TcGeometry::kBlockK);
  long long stages = SplitGeometry::kRingBytes / static_cast<long long>(stage_bytes);
  if (stages > SplitGeometry::kMaxStages) stages = SplitGeometry::kMaxStages;
  if (stages > kb_per) stages = kb_per;
  const double cta_bytes = static_cast<double>(kb_per) * stage_bytes;
  const double per_kb = kPerKBlock * static_cast<double>(kb_per);  // issue and hand-over cost of a k-block
  const double ring = kLatency + per_kb + cta_bytes / (static_cast<double>(stages) * stage_bytes / kRingLatency);
  const double mma = kLatency + per_kb + static_cast<double>(kb_per * block_n) * kMmaPerColumn;
  const long long concurrent = (tiles < resident_clusters ? tiles : resident_clusters) * split;
  const double unique_bytes = static_cast<double>(M + N) * static_cast<double>(K);
  double chip = static_cast<double>(concurrent) * cta_bytes / kL2BytesPerUs;
  // operands beyond what L2 can hold between calls come from HBM whatever the access pattern
  // one SM draws about 58 GB/s from HBM with 32 KiB boxes of W however deep its ring (46 with 16 KiB
  // boxes, 29 with 8 KiB): few CTAs cannot saturate the memory
  const double box_factor = block_n >= 128 ? 0.8 + 0.2 * (block_n - 128) / 128.0
                                           : (block_n >= 64 ? 0.5 + 0.3 * (block_n - 64) / 64.0 : 0.5 * block_n / 64.0);
  double hbm_rate = static_cast<double>(concurrent) * kHbmBytesPerUsPerSm * box_factor;
  if (hbm_rate > kHbmBytesPerUs) hbm_rate = kHbmBytesPerUs;
  const double hbm = unique_bytes / static_cast<double>(waves) / hbm_rate;
  if (unique_bytes > kL2ResidentBytes && hbm > chip) chip = hbm;
  chip += kLatency;
  double main_loop = ring > mma ? ring : mma;
  if (chip > main_loop) main_loop = chip;
  const long long rows_sent = M < 128 ? M : 128;
  const double exchange =
      split > 1 ? kExchangeFixed + kExchangePerByte * static_cast<double>(rows_sent * block_n * 4 * (split - 1) / split)
                : 0.0;
  return kLaunch + static_cast<double>(waves) * (main_loop + exchange + kEpilogue);
}

// forced_block_n / forced_split: 0 = choose by the cost model.  Candidate widths: 256, 128, 64, and for
// each cluster size the narrowest tile that still gives one wave (every SM, or as many as can hold a
// cluster, gets exactly one tile).
// Shared-memory layout of one (block_n, split) configuration: stages, ring, dynamic shared memory.
static void size_split_plan(long long M, long long K, SplitPlan* p) {
  const long long kb = (K + TcGeometry::kBlockK - 1) / TcGeometry::kBlockK;
  p->rows_a = M >= 128 ? 128 : static_cast<int>((M + 7) / 8 * 8);
  const int bytes_a = p->rows_a * TcGeometry::kBlockK, bytes_b = p->block_n * TcGeometry::kBlockK;
  const long long kb_per = (kb + p->split - 1) / p->split;
  p->stages = SplitGeometry::kRingBytes / (bytes_a + bytes_b);
  if (p->stages > SplitGeometry::kMaxStages) p->stages = SplitGeometry::kMaxStages;
  if (p->stages > kb_per) p->stages = static_cast<int>(kb_per > 0 ? kb_per : 1);
  p->staged_stores = M > 64 ? 1 : 0;  // short outputs leave in 16-byte stores straight from registers
  for (;; --p->stages) {
    // the ring: the stages; room for the MMA's 128-row read of the last X stage; the exchange buffer
    int ring = p->stages * (bytes_a + bytes_b);
    const int a_overread = p->stages * bytes_a + TcGeometry::kBlockM * TcGeometry::kBlockK;
    if (ring < a_overread) ring = a_overread;
    const int exchange = p->split > 1 ? p->block_n * p->rows_a * 4 : 0;
    if (ring < exchange) ring = exchange;
    p->ring_bytes = (ring + 1023) / 1024 * 1024;
    p->smem_bytes = p->ring_bytes + (p->staged_stores ? 32 * 1024 : 0) + split_scale_bytes(p->block_n) + 256 + 1024;
    if (p->smem_bytes <= SplitGeometry::kMaxSmemBytes || p->stages == 1) break;  // a wide tile's third stage may not fit
  }
  // Tensor memory: an SM has 512 columns and this kernel's CTAs take tmem_cols each with a tcgen05.alloc that
  // blocks until the columns are free.  CTAs that block there while their cluster peers wait at a cluster
  // barrier would never be released, so no more CTAs may be resident on an SM than its tensor memory holds.
  // Shared memory is the limit the launch controls: ask for enough of it that floor(227 KiB / smem_bytes)
  // CTAs need at most 512 columns (76 KiB for 256 columns: two CTAs; 46 KiB for 128: four; ...).
  const int min_smem = SplitGeometry::min_smem_bytes_for_tmem(split_tmem_cols(p->block_n));
  if (p->smem_bytes < min_smem) p->smem_bytes = min_smem;
}

// Fewer stages (never fewer than three) until two CTAs fit on an SM by shared memory.
static void shrink_ring_for_two_ctas(SplitPlan* p) {
  const int half_sm = SplitGeometry::kSmemPerSm / 2 - 1024;
  const int bytes_a = p->rows_a * TcGeometry::kBlockK, bytes_b = p->block_n * TcGeometry::kBlockK;
  while (p->smem_bytes > half_sm && p->stages > 3) {
    --p->stages;
    int ring = p->stages * (bytes_a + bytes_b);
    const int a_overread = p->stages * bytes_a + TcGeometry::kBlockM * TcGeometry::kBlockK;
    if (ring < a_overread) ring = a_overread;
    const int exchange = p->split > 1 ? p->block_n * p->rows_a * 4 : 0;
    if (ring < exchange) ring = exchange;
    p->ring_bytes = (ring + 1023) / 1024 * 1024;
    p->smem_bytes = p->ring_bytes + (p->staged_stores ? 32 * 1024 : 0) + split_scale_bytes(p->block_n) + 256 + 1024;
    const int min_smem = SplitGeometry::min_smem_bytes_for_tmem(split_tmem_cols(p->block_n));
    if (p->smem_bytes < min_smem) p->smem_bytes = min_smem;
  }
}

// CTAs of a configuration that share an SM: by shared memory, and never more than two (168 registers x 192
// threads).  resident_clusters[] was measured with the largest shared-memory request, one CTA per SM.
static int split_ctas_per_sm(const SplitPlan& p) {
  const int by_smem = SplitGeometry::kSmemPerSm / (p.smem_bytes + 1024);
  return by_smem >= 2 ? 2 : 1;
}

SplitPlan make_split_plan(long long M, long long N, long long K, const int* resident_clusters, int forced_block_n,
                          int forced_split) {
  SplitPlan best = {};
  best.block_n = 256;
  best.split = 1;
  double best_cost = 1e30;
  const long long kb = (K + TcGeometry::kBlockK - 1) / TcGeometry::kBlockK;
  const long long tiles_m = (M + 127) / 128;
  for (int split = 1, log2_split = 0; split <= 8; split *= 2, ++log2_split) {
    if (forced_split != 0 && split != forced_split) continue;
    if (forced_split == 0 && split > 1 && kb / split < 2) break;
    const int resident = resident_clusters[log2_split];
    const int step = 16 * split;  // a CTA finishes block_n / split columns, a multiple of 16
    int candidates[4] = {256, 128, 64, 0};
    if (resident >= tiles_m) {
      const long long tiles_n = resident / tiles_m;                  // tiles along N that fit in one wave
      // narrowest width that needs no more, in whole 32-column steps: MMAs of 144, 176 or 208 columns were measured
      // at about half the rate of their neighbours of 160, 192 and 224
      const int fit_step = step < 32 ? 32 : step;
      long long fit = ((N + tiles_n - 1) / tiles_n + fit_step - 1) / fit_step * fit_step;
      // beyond 256 columns a single CTA multiplies the tile as two halves, no K split then.  Halves that are
      // multiples of 32 columns: an MMA of 144 or 176 columns was measured at half the rate of one of 160.
      if (fit > 256 && split == 1) fit = (fit + 63) / 64 * 64;
      const long long widest = split == 1 ? SplitGeometry::kMaxBlockN : 256;
      if (fit <= widest && fit != 256 && fit != 128 && fit != 64) candidates[3] = static_cast<int>(fit);
    }
    for (int i = 0; i < 4; ++i) {
      const int block_n = forced_block_n != 0 ? forced_block_n : candidates[i];
      if (block_n == 0 || block_n % step != 0) continue;
      SplitPlan cand = {};
      cand.block_n = block_n;
      cand.split = split;
      size_split_plan(M, K, &cand);
      const int resident_here = resident * split_ctas_per_sm(cand);  // short rings: two CTAs per SM
      const double cost = split_plan_cost_us(M, N, K, block_n, split, resident_here);
      if (cost < best_cost) {
        best_cost = cost;
        best = cand;
        best.waves = static_cast<int>((tiles_m * ((N + block_n - 1) / block_n) + resident_here - 1) / resident_here);
      }
      if (forced_block_n != 0) break;
    }
  }
  if (best.smem_bytes == 0) size_split_plan(M, K, &best);  // nothing was eligible: the default 256 x 1
  best.tiles = static_cast<int>(tiles_m * ((N + best.block_n - 1) / best.block_n));
  return best;
}

}  // namespace b200fp8

namespace {

int make_plan(int64_t M, int64_t N, int64_t K, uint32_t flags, bool operands_tma_ok, bool y_tma_ok,
              const DeviceInfo& dev, Plan* out) {
  Plan pl = {};
  uint32_t v = flags & B200FP8_VARIANT_MASK;
  if (v > B200FP8_VARIANT_GEMV) return B200FP8_BAD_ARG;
  const GemvPlan gemv = make_gemv_plan(M, N, K, dev.sm_count);
  if (v == B200FP8_VARIANT_AUTO) {
    if (!operands_tma_ok) {
      v = B200FP8_VARIANT_SIMT;
    } else if (M <= SkinnyGeometry::kMaxTokens) {
      // one tile per cluster while the output is narrow enough for a wave or two of clusters; beyond
      // that a persistent kernel: stream-K for a handful of tokens, whole tiles otherwise
      const SplitPlan sp = make_split_plan(M, N, K, dev.split_clusters, 0, 0);
      v = sp.waves <= 2 ? B200FP8_VARIANT_TC_SPLITK : (M <= 32 ? B200FP8_VARIANT_SKINNY : B200FP8_VARIANT_TC_1CTA);
    } else {
      // a CTA pair per 256x256 tile halves the shared-memory fill per flop; keep single CTAs when
      // the pair tiles could not occupy the SMs anyway
      const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
      v = pair_tiles >= dev.sm_count / 2 ? B200FP8_VARIANT_TC_2CTA : B200FP8_VARIANT_TC_1CTA;
      if (v == B200FP8_VARIANT_TC_1CTA && ((M + 127) / 128) * ((N + 255) / 256) < dev.sm_count) {
        v = B200FP8_VARIANT_TC_SPLITK;
      }
      // The persistent kernels run whole waves of 256-column tiles.  With one to two waves, most of the last
      // wave's SMs idle; if tiles widened to at most 512 columns cover the output in ONE wave of single CTAs,
      // compare that plan's modelled time with the waves of the pair kernel (a 256x256 tile takes 0.30 us per
      // k-block at the clock these short launches see, plus 5 us of launch, pipeline fill and epilogue).
      if (v == B200FP8_VARIANT_TC_2CTA && pair_tiles <= 2 * (dev.sm_count / 2)) {
        const SplitPlan sp = make_split_plan(M, N, K, dev.split_clusters, 0, 1);
        if (sp.waves == 1) {
          const int64_t waves = (pair_tiles + dev.sm_count / 2 - 1) / (dev.sm_count / 2);
          const double kb = static_cast<double>((K + TcGeometry::kBlockK - 1) / TcGeometry::kBlockK);
          const double pair_us = 5.0 + static_cast<double>(waves) * kb * 0.30;
          if (split_plan_cost_us(M, N, K, sp.block_n, 1, dev.split_clusters[0]) < pair_us) v = B200FP8_VARIANT_TC_SPLITK;
        }
      }
    }
  } else if (v != B200FP8_VARIANT_SIMT && !operands_tma_ok) {
    return B200FP8_UNSUPPORTED_ALIGNMENT;
  }
  if (v == B200FP8_VARIANT_GEMV) {
    if (M > kGemvMaxTokens) return B200FP8_BAD_ARG;
    if (!gemv.ok) return K % 16 != 0 ? B200FP8_UNSUPPORTED_ALIGNMENT : B200FP8_TOO_LARGE;
  }
  if (v == B200FP8_VARIANT_SKINNY && M > SkinnyGeometry::kMaxTokens) return B200FP8_BAD_ARG;
  if (v == B200FP8_VARIANT_SKINNY && (N + SkinnyGeometry::kRowsW - 1) / SkinnyGeometry::kRowsW > SkinnyGeometry::kMaxTiles) {
    if ((flags & B200FP8_VARIANT_MASK) != B200FP8_VARIANT_AUTO) return B200FP8_TOO_LARGE;
    v = B200FP8_VARIANT_TC_1CTA;  // wider than the counter region covers: use the large-M kernel
  }
  pl.variant = v;
  pl.tma_store = y_tma_ok && (flags & B200FP8_FLAG_NO_TMA_STORE) == 0;
  pl.group_m = choose_group_m(M, K, v == B200FP8_VARIANT_TC_2CTA ? 256 : 128);
  pl.workspace_bytes = B200FP8_WORKSPACE_HEADER_BYTES;
  if (v == B200FP8_VARIANT_TC_1CTA) {
    const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
    pl.num_ctas = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
  } else if (v == B200FP8_VARIANT_TC_2CTA) {
    const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t clusters = tiles < dev.max_pair_clusters ? tiles : dev.max_pair_clusters;
    pl.num_ctas = static_cast<int>(2 * clusters);
  } else if (v == B200FP8_VARIANT_TC_SPLITK) {
    const int forced_block_n = static_cast<int>((flags >> 8) & 0x1Fu) * 16;
    const int forced_split = static_cast<int>((flags >> 13) & 0xFu);
    if (forced_block_n > SplitGeometry::kMaxBlockN ||
        (forced_split != 0 && forced_split != 1 && forced_split != 2 && forced_split != 4 && forced_split != 8) ||
        (forced_block_n != 0 && forced_block_n % (16 * (forced_split != 0 ? forced_split : 1)) != 0) ||
        (forced_block_n > 256 && (forced_split > 1 || forced_block_n % 64 != 0))) {
      return B200FP8_BAD_ARG;
    }
    // a forced wide tile implies no K split
    pl.splitk = make_split_plan(M, N, K, dev.split_clusters, forced_block_n, forced_block_n > 256 ? 1 : forced_split);
    pl.splitk.overlap_previous_kernel = (flags & B200FP8_FLAG_PDL) != 0;
    // Overlapped launches of a problem whose W stays in L2 between calls: a ring short enough for two CTAs per
    // SM lets the next launch's CTAs move in and prefetch W while this launch's CTAs finish (measured, CUDA-graph
    // replay: 4x13312x2048 8.5 -> 8.0 us, 128x8192x2304 8.1 -> 7.6, 16x4096x6656 8.6 -> 7.6).  When W has to come
    // from HBM the deep ring matters more (32x8192x13312: 22.7 us deep, 25.3 shallow).
    if (pl.splitk.overlap_previous_kernel && static_cast<double>(N) * static_cast<double>(K) <= 48.0e6) {
      shrink_ring_for_two_ctas(&pl.splitk);
    }
  } else if (v == B200FP8_VARIANT_GEMV) {
    pl.gemv = gemv;
  } else if (v == B200FP8_VARIANT_SKINNY) {
    pl.skinny = make_skinny_plan(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), dev.sm_count);
    pl.skinny.overlap_previous_kernel = (flags & B200FP8_FLAG_PDL) != 0;
    pl.workspace_bytes += pl.skinny.counter_bytes;
    pl.workspace_bytes = (pl.workspace_bytes + 255) & ~static_cast<size_t>(255);
    pl.workspace_bytes += pl.skinny.partial_bytes;
  }
  *out = pl;
  return B200FP8_OK;
}

int check_sizes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0) return B200FP8_BAD_ARG;
  if (M > 0x7FFFFF00ll || N > 0x7FFFFF00ll || K > 0x7FFFFF00ll) return B200FP8_TOO_LARGE;
  return B200FP8_OK;
}

}  // namespace

extern "C" {


int b200fp8_abi_version(void) { return B200FP8_ABI_VERSION; }

const char* b200fp8_status_string(int status) {
  switch (status) {
    case B200FP8_OK: return "ok";
    case B200FP8_BAD_ARG: return "bad argument";
    case B200FP8_UNSUPPORTED_ARCH: return "device is not compute capability 10.x (B200)";
    case B200FP8_UNSUPPORTED_ALIGNMENT: return "operand rows are not 16-byte aligned for the requested variant";
    case B200FP8_WORKSPACE_TOO_SMALL: return "workspace too small";
    case B200FP8_LAUNCH_FAILED: return "CUDA call failed";
    case B200FP8_DEVICE_TIMEOUT: return "a bounded wait inside the kernel timed out";
    case B200FP8_TOO_LARGE: return "size exceeds the supported maximum";
    default: return "unknown status";
  }
}

int b200fp8_last_cuda_error(void) { return g_last_cuda_error; }

size_t b200fp8_workspace_bytes(int64_t M, int64_t N, int64_t K, uint32_t flags) {
  if (check_sizes(M, N, K) != B200FP8_OK) return 0;
  DeviceInfo dev;
  if (device_info(&dev) != B200FP8_OK) {
    // no usable device: size for the largest B200 configuration so that callers can still plan
    dev.sm_count = 148;
    dev.max_pair_clusters = 74;
    dev.split_clusters[0] = 148;
    dev.split_clusters[1] = 74;
    dev.split_clusters[2] = 33;
    dev.split_clusters[3] = 15;
  }
  Plan pl;
  if (make_plan(M, N, K, flags, true, true, dev, &pl) != B200FP8_OK) return 0;
  return pl.workspace_bytes;
}

int b200fp8_workspace_init(void* workspace, size_t workspace_bytes, void* cuda_stream) {
  if (workspace == nullptr || workspace_bytes < B200FP8_WORKSPACE_HEADER_BYTES) return B200FP8_BAD_ARG;
  return note_cuda(cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_gemm_rowwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                         const void* bias_bf16, void* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldx,
                         int64_t ldw, int64_t ldy, void* workspace, size_t workspace_bytes, uint32_t flags,
                         void* cuda_stream) {
  if (xq == nullptr || wq == nullptr || x_scale == nullptr || w_scale == nullptr || y_bf16 == nullptr ||
      workspace == nullptr) {
    return B200FP8_BAD_ARG;
  }
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  if (ldx < K || ldw < K || ldy < N) return B200FP8_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return B200FP8_BAD_ARG;

  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;

  const bool operands_ok = tma_loadable(K, ldx, ldw, xq, wq);
  const bool y_ok = (ldy % 8 == 0) && aligned16(y_bf16);
  Plan pl;
  st = make_plan(M, N, K, flags, operands_ok, y_ok, dev, &pl);
  if (st != B200FP8_OK) return st;
  if (workspace_bytes < pl.workspace_bytes) return B200FP8_WORKSPACE_TOO_SMALL;

  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  uint32_t* status_word = static_cast<uint32_t*>(workspace);
  const __nv_bfloat16* bias = static_cast<const __nv_bfloat16*>(bias_bf16);
  __nv_bfloat16* y = static_cast<__nv_bfloat16*>(y_bf16);

  if (pl.variant == B200FP8_VARIANT_SIMT) {
    SimtParams sp = {static_cast<const uint8_t*>(xq), static_cast<const uint8_t*>(wq), x_scale, w_scale, bias, y,
                     static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldx, ldw, ldy,
                     (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0};
    return note_cuda(launch_gemm_simt(sp, stream));
  }

  if (pl.variant == B200FP8_VARIANT_GEMV) {
    GemvParams gp = {static_cast<const uint8_t*>(xq), static_cast<const uint8_t*>(wq), x_scale, w_scale, bias, y,
                     static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldx, ldw, ldy,
                     (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0, (flags & B200FP8_FLAG_PDL) ? 1 : 0, 0};
    return note_cuda(launch_gemm_gemv(gp, pl.gemv, stream));
  }

  if (pl.variant == B200FP8_VARIANT_SKINNY) {
    CUtensorMap tm_w, tm_x;
    st = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, K, ldw, SkinnyGeometry::kBlockK,
                   SkinnyGeometry::kRowsW);
    if (st != B200FP8_OK) return st;
    st = encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, K, ldx, SkinnyGeometry::kBlockK,
                   static_cast<uint32_t>(pl.skinny.tokens_pad));
    if (st != B200FP8_OK) return st;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    size_t off = B200FP8_WORKSPACE_HEADER_BYTES;
    SkinnyParams kp = {};
    kp.x_scale = x_scale;
    kp.w_scale = w_scale;
    kp.bias = bias;
    kp.y = y;
    kp.M = static_cast<int>(M);
    kp.N = static_cast<int>(N);
    kp.K = static_cast<int>(K);
    kp.ldy = ldy;
    kp.out_fp16 = (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0;
    kp.counters = reinterpret_cast<uint32_t*>(ws + off);
    off = (off + pl.skinny.counter_bytes + 255) & ~static_cast<size_t>(255);
    kp.partials = reinterpret_cast<float*>(ws + off);
    kp.status = status_word;
    return note_cuda(launch_gemm_skinny(tm_w, tm_x, kp, pl.skinny, stream));
  }

  const int cta_group = pl.variant == B200FP8_VARIANT_TC_2CTA ? 2 : 1;
  CUtensorMap tm_x, tm_w, tm_y;
  memset(&tm_y, 0, sizeof(tm_y));
  const int x_box_rows = pl.variant == B200FP8_VARIANT_TC_SPLITK ? pl.splitk.rows_a : TcGeometry::kBlockM;
  st = encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, K, ldx, TcGeometry::kBlockK, x_box_rows);
  if (st != B200FP8_OK) return st;
  const int w_box_rows =
      pl.variant == B200FP8_VARIANT_TC_SPLITK ? split_first_half(pl.splitk.block_n) : TcGeometry::kBlockN / cta_group;
  st = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, K, ldw, TcGeometry::kBlockK, w_box_rows);
  if (st != B200FP8_OK) return st;
  if (pl.tma_store) {
    st = encode_2d(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y, M, N, ldy * 2, TcGeometry::kStoreCols,
                   TcGeometry::kStoreRows);
    if (st != B200FP8_OK) return st;
  }
  TcParams tp = {};
  tp.x_scale = x_scale;
  tp.w_scale = w_scale;
  tp.bias = bias;
  tp.y = y;
  tp.M = static_cast<int>(M);
  tp.N = static_cast<int>(N);
  tp.K = static_cast<int>(K);
  tp.ldy = ldy;
  tp.use_tma_store = pl.tma_store ? 1 : 0;
  tp.out_fp16 = (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0;
  tp.group_m = pl.group_m;
  tp.y_evict_first = y_streams_past_l2(M, N) ? 1 : 0;
  tp.status = status_word;
  if (pl.variant == B200FP8_VARIANT_TC_SPLITK) {
    return note_cuda(launch_gemm_splitk(tm_x, tm_w, tm_y, tp, pl.splitk, stream));
  }
  if (cta_group == 2) return note_cuda(launch_gemm_tc<2>(tm_x, tm_w, tm_y, tp, pl.num_ctas, stream));
  return note_cuda(launch_gemm_tc<1>(tm_x, tm_w, tm_y, tp, pl.num_ctas, stream));
}

int b200fp8_gemm_rowwise_gather(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                const void* bias_bf16, void* const* y_copies, int num_copies, int64_t M, int64_t N,
                                int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, void* workspace,
                                size_t workspace_bytes, uint32_t flags, void* cuda_stream) {
  if (xq == nullptr || wq == nullptr || x_scale == nullptr || w_scale == nullptr || y_copies == nullptr ||
      workspace == nullptr) {
    return B200FP8_BAD_ARG;
  }
  if (num_copies < 1 || num_copies > 1 + kMaxExtraOutputs) return B200FP8_BAD_ARG;
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  if (ldx < K || ldw < K || ldy < N) return B200FP8_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || workspace_bytes < B200FP8_WORKSPACE_HEADER_BYTES) {
    return B200FP8_BAD_ARG;
  }
  uint32_t variant = flags & B200FP8_VARIANT_MASK;
  if (variant != B200FP8_VARIANT_AUTO && variant != B200FP8_VARIANT_TC_1CTA && variant != B200FP8_VARIANT_TC_2CTA) {
    return B200FP8_BAD_ARG;
  }
  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;
  // every copy is written with TMA stores only: all of them need 16-byte aligned rows
  if (!tma_loadable(K, ldx, ldw, xq, wq) || ldy % 8 != 0) return B200FP8_UNSUPPORTED_ALIGNMENT;
  for (int i = 0; i < num_copies; ++i) {
    if (y_copies[i] == nullptr) return B200FP8_BAD_ARG;
    if (!aligned16(y_copies[i])) return B200FP8_UNSUPPORTED_ALIGNMENT;
  }
  if (variant == B200FP8_VARIANT_AUTO) {
    const int64_t pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    variant = pair_tiles >= dev.sm_count / 2 ? B200FP8_VARIANT_TC_2CTA : B200FP8_VARIANT_TC_1CTA;
  }
  const int cta_group = variant == B200FP8_VARIANT_TC_2CTA ? 2 : 1;
  CUtensorMap tm_x, tm_w, tm_y;
  st = encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, K, ldx, TcGeometry::kBlockK, TcGeometry::kBlockM);
  if (st != B200FP8_OK) return st;
  st = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, K, ldw, TcGeometry::kBlockK,
                 TcGeometry::kBlockN / cta_group);
  if (st != B200FP8_OK) return st;
  st = encode_2d(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_copies[0], M, N, ldy * 2, TcGeometry::kStoreCols,
                 TcGeometry::kStoreRows);
  if (st != B200FP8_OK) return st;
  ExtraOutputs extra;
  memset(&extra, 0, sizeof(extra));
  for (int i = 1; i < num_copies; ++i) {
    st = encode_2d(&extra.tm[i - 1], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_copies[i], M, N, ldy * 2,
                   TcGeometry::kStoreCols, TcGeometry::kStoreRows);
    if (st != B200FP8_OK) return st;
  }
  TcParams tp = {};
  tp.x_scale = x_scale;
  tp.w_scale = w_scale;
  tp.bias = static_cast<const __nv_bfloat16*>(bias_bf16);
  tp.y = static_cast<__nv_bfloat16*>(y_copies[0]);
  tp.M = static_cast<int>(M);
  tp.N = static_cast<int>(N);
  tp.K = static_cast<int>(K);
  tp.ldy = ldy;
  tp.use_tma_store = 1;
  tp.out_fp16 = (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0;
  tp.group_m = choose_group_m(M, K, cta_group == 2 ? 256 : 128);
  tp.y_evict_first = y_streams_past_l2(M, N) ? 1 : 0;
  tp.num_extra = num_copies - 1;
  tp.status = static_cast<uint32_t*>(workspace);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (cta_group == 2) {
    const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const int64_t clusters = tiles < dev.max_pair_clusters ? tiles : dev.max_pair_clusters;
    return note_cuda(launch_gemm_tc<2>(tm_x, tm_w, tm_y, tp, static_cast<int>(2 * clusters), stream, &extra));
  }
  const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
  const int ctas = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
  return note_cuda(launch_gemm_tc<1>(tm_x, tm_w, tm_y, tp, ctas, stream, &extra));
}

// ---- device buffers that other processes of the node can map (CUDA IPC): where the gathered Y lives ----
int b200fp8_shared_buffer_create(size_t bytes, void** device_ptr, void* handle_out, size_t handle_bytes) {
  if (bytes == 0 || device_ptr == nullptr || handle_out == nullptr) return B200FP8_BAD_ARG;
  if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return B200FP8_BAD_ARG;
  *device_ptr = nullptr;
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  if (e != cudaSuccess) return note_cuda(e);
  cudaIpcMemHandle_t handle;
  e = cudaIpcGetMemHandle(&handle, ptr);
  if (e != cudaSuccess) {
    cudaFree(ptr);
    return note_cuda(e);
  }
  memcpy(handle_out, &handle, sizeof(handle));
  *device_ptr = ptr;
  return B200FP8_OK;
}

int b200fp8_shared_buffer_open(const void* handle_in, size_t handle_bytes, void** device_ptr) {
  if (handle_in == nullptr || device_ptr == nullptr || handle_bytes < sizeof(cudaIpcMemHandle_t)) return B200FP8_BAD_ARG;
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle_in, sizeof(handle));
  *device_ptr = nullptr;
  return note_cuda(cudaIpcOpenMemHandle(device_ptr, handle, cudaIpcMemLazyEnablePeerAccess));
}

int b200fp8_shared_buffer_close(void* device_ptr) {
  if (device_ptr == nullptr) return B200FP8_BAD_ARG;
  return note_cuda(cudaIpcCloseMemHandle(device_ptr));
}

int b200fp8_shared_buffer_destroy(void* device_ptr) {
  if (device_ptr == nullptr) return B200FP8_BAD_ARG;
  return note_cuda(cudaFree(device_ptr));
}

int b200fp8_gemm_rowwise_noalloc(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                 const void* bias_bf16, void* y_bf16, int64_t M, int64_t N, int64_t K, int64_t ldx,
                                 int64_t ldw, int64_t ldy, void* cuda_stream) {
  if (xq == nullptr || wq == nullptr || x_scale == nullptr || w_scale == nullptr || y_bf16 == nullptr) {
    return B200FP8_BAD_ARG;
  }
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  if (ldx < K || ldw < K || ldy < N) return B200FP8_BAD_ARG;
  if (M > SkinnyGeometry::kMaxTokens) return B200FP8_TOO_LARGE;
  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;
  if (!tma_loadable(K, ldx, ldw, xq, wq)) return B200FP8_UNSUPPORTED_ALIGNMENT;
  Plan pl;
  st = make_plan(M, N, K, B200FP8_VARIANT_SKINNY, true, true, dev, &pl);
  if (st != B200FP8_OK) return st;
  if (pl.workspace_bytes > kStaticScratchBytes) return B200FP8_TOO_LARGE;  // partial sums would not fit

  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  cudaError_t e = skinny_static_scratch(&scratch, &scratch_bytes);  // first call on a device: symbol look-up
  if (e != cudaSuccess) return note_cuda(e);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The array keeps whatever the last call left.  What must start at zero is the status word and
  // the arrival counters of the tiles this call uses; the partial-sum slots are written before read.
  const size_t clear_bytes =
      B200FP8_WORKSPACE_HEADER_BYTES + static_cast<size_t>(pl.skinny.tiles) * 4 * sizeof(uint32_t);
  e = cudaMemsetAsync(scratch, 0, clear_bytes, stream);
  if (e != cudaSuccess) return note_cuda(e);
  return b200fp8_gemm_rowwise(xq, wq, x_scale, w_scale, bias_bf16, y_bf16, M, N, K, ldx, ldw, ldy, scratch,
                              scratch_bytes, B200FP8_VARIANT_SKINNY, cuda_stream);
}

int b200fp8_noalloc_status(uint32_t* device_status) {
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  const cudaError_t e = skinny_static_scratch(&scratch, &scratch_bytes);
  if (e != cudaSuccess) return note_cuda(e);
  return b200fp8_query_status(scratch, device_status);
}

int b200fp8_gemm_rowwise_grouped(const void* xq, const void* wq, const float* x_scale, const float* w_scale,
                                 const int32_t* group_rows, int64_t num_groups, void* y_bf16, int64_t M_total,
                                 int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, void* workspace,
                                 size_t workspace_bytes, uint32_t flags, void* cuda_stream) {
  if (xq == nullptr || wq == nullptr || x_scale == nullptr || w_scale == nullptr || y_bf16 == nullptr ||
      workspace == nullptr || group_rows == nullptr) {
    return B200FP8_BAD_ARG;
  }
  int st = check_sizes(M_total, N, K);
  if (st != B200FP8_OK) return st;
  if (num_groups <= 0 || num_groups > 4096) return B200FP8_BAD_ARG;
  if (num_groups * N > 0x7FFFFF00ll) return B200FP8_TOO_LARGE;
  if (ldx < K || ldw < K || ldy < N) return B200FP8_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || workspace_bytes < B200FP8_WORKSPACE_HEADER_BYTES) {
    return B200FP8_BAD_ARG;
  }
  const uint32_t variant = flags & B200FP8_VARIANT_MASK;
  if (variant != B200FP8_VARIANT_AUTO && variant != B200FP8_VARIANT_TC_1CTA && variant != B200FP8_VARIANT_TC_2CTA) {
    return B200FP8_BAD_ARG;
  }
  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;
  if (!tma_loadable(K, ldx, ldw, xq, wq)) return B200FP8_UNSUPPORTED_ALIGNMENT;

  CUtensorMap tm_x, tm_w, tm_y;
  memset(&tm_y, 0, sizeof(tm_y));
  st = encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M_total, K, ldx, TcGeometry::kBlockK, TcGeometry::kBlockM);
  if (st != B200FP8_OK) return st;
  // a CTA pair per 256-row tile of a group when the problem has enough such tiles for the pairs the device runs at once
  // (the group sizes live on the device: the estimate uses M_total as if it were one group)
  const int64_t tiles_n = (N + 255) / 256;
  int cta_group = variant == B200FP8_VARIANT_TC_2CTA ? 2 : 1;
  if (variant == B200FP8_VARIANT_AUTO && (M_total / 256) * tiles_n >= dev.sm_count / 2) cta_group = 2;
  st = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, num_groups * N, K, ldw, TcGeometry::kBlockK,
                 TcGeometry::kBlockN / cta_group);
  if (st != B200FP8_OK) return st;
  const bool tma_store = (ldy % 8 == 0) && aligned16(y_bf16) && (flags & B200FP8_FLAG_NO_TMA_STORE) == 0;
  if (tma_store) {
    st = encode_2d(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_bf16, M_total, N, ldy * 2, TcGeometry::kStoreCols,
                   TcGeometry::kStoreRows);
    if (st != B200FP8_OK) return st;
  }
  TcParams tp = {};
  tp.x_scale = x_scale;
  tp.w_scale = w_scale;
  tp.bias = nullptr;
  tp.y = static_cast<__nv_bfloat16*>(y_bf16);
  tp.M = static_cast<int>(M_total);
  tp.N = static_cast<int>(N);
  tp.K = static_cast<int>(K);
  tp.ldy = ldy;
  tp.use_tma_store = tma_store ? 1 : 0;
  tp.out_fp16 = (flags & B200FP8_FLAG_OUT_FP16) ? 1 : 0;
  tp.group_m = 8;
  tp.num_groups = static_cast<int>(num_groups);
  tp.group_rows = group_rows;
  tp.status = static_cast<uint32_t*>(workspace);
  // the group sizes live on the device, so the tile count is not known here: one CTA (pair) per SM (pair), each
  // walks the tile list it derives from the sizes
  if (cta_group == 2) {
    const int64_t max_tiles = ((M_total + 255) / 256 + num_groups) * tiles_n;
    const int clusters = static_cast<int>(max_tiles < dev.max_pair_clusters ? max_tiles : dev.max_pair_clusters);
    return note_cuda(launch_gemm_tc<2>(tm_x, tm_w, tm_y, tp, 2 * clusters, static_cast<cudaStream_t>(cuda_stream)));
  }
  const int64_t max_tiles = ((M_total + 127) / 128 + num_groups) * tiles_n;
  const int ctas = static_cast<int>(max_tiles < dev.sm_count ? max_tiles : dev.sm_count);
  return note_cuda(launch_gemm_tc<1>(tm_x, tm_w, tm_y, tp, ctas, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_gemm_blockwise(const void* xq, const void* wq, const float* x_scale, const float* w_scale, void* y_bf16,
                           int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldw, int64_t ldy, int64_t ld_xs,
                           int64_t ld_ws, void* workspace, size_t workspace_bytes, uint32_t flags, void* cuda_stream) {
  if (xq == nullptr || wq == nullptr || x_scale == nullptr || w_scale == nullptr || y_bf16 == nullptr ||
      workspace == nullptr) {
    return B200FP8_BAD_ARG;
  }
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  const int64_t kb = (K + 127) / 128;
  if (ldx < K || ldw < K || ldy < N || ld_xs < kb || ld_ws < kb) return B200FP8_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || workspace_bytes < B200FP8_WORKSPACE_HEADER_BYTES) {
    return B200FP8_BAD_ARG;
  }
  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;
  if (!tma_loadable(K, ldx, ldw, xq, wq)) return B200FP8_UNSUPPORTED_ALIGNMENT;
  CUtensorMap tm_x, tm_w, tm_y;
  memset(&tm_y, 0, sizeof(tm_y));
  st = encode_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, M, K, ldx, TcGeometry::kBlockK, TcGeometry::kBlockM);
  if (st != B200FP8_OK) return st;
  st = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, N, K, ldw, TcGeometry::kBlockK, TcGeometry::kBlockN);
  if (st != B200FP8_OK) return st;
  const bool tma_store = (ldy % 8 == 0) && aligned16(y_bf16) && (flags & B200FP8_FLAG_NO_TMA_STORE) == 0;
  if (tma_store) {
    st = encode_2d(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, y_bf16, M, N, ldy * 2, TcGeometry::kStoreCols,
                   TcGeometry::kStoreRows);
    if (st != B200FP8_OK) return st;
  }
  BlockwiseParams bp = {};
  bp.x_scale = x_scale;
  bp.w_scale = w_scale;
  bp.y = static_cast<__nv_bfloat16*>(y_bf16);
  bp.M = static_cast<int>(M);
  bp.N = static_cast<int>(N);
  bp.K = static_cast<int>(K);
  bp.ldy = ldy;
  bp.ld_xs = ld_xs;
  bp.ld_ws = ld_ws;
  bp.use_tma_store = tma_store ? 1 : 0;
  bp.group_m = choose_group_m(M, K, 128);
  bp.status = static_cast<uint32_t*>(workspace);
  const int64_t tiles = ((M + 127) / 128) * ((N + 255) / 256);
  const int ctas = static_cast<int>(tiles < dev.sm_count ? tiles : dev.sm_count);
  return note_cuda(launch_gemm_blockwise(tm_x, tm_w, tm_y, bp, ctas, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_row_quantize(const void* x, int x_dtype, int recipe, int64_t rows, int64_t cols, int64_t ldx, void* q,
                         int64_t ldq, float* scale, void* cuda_stream) {
  if (x == nullptr || q == nullptr || scale == nullptr) return B200FP8_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ldx < cols || ldq < cols) return B200FP8_BAD_ARG;
  if (rows > 0x7FFFFFFFll || cols > 0x7FFFFF00ll) return B200FP8_TOO_LARGE;
  if (x_dtype < kQuantBf16 || x_dtype > kQuantFp32) return B200FP8_BAD_ARG;
  if (recipe != kRecipeOperator && recipe != kRecipeFp32) return B200FP8_BAD_ARG;
  if (recipe == kRecipeFp32 && x_dtype != kQuantFp32) return B200FP8_BAD_ARG;
  const int64_t elem = x_dtype == kQuantFp32 ? 4 : 2;
  QuantParams p = {};
  p.x = x;
  p.q = static_cast<uint8_t*>(q);
  p.scale = scale;
  p.rows = rows;
  p.cols = static_cast<int>(cols);
  p.ldx = ldx;
  p.ldq = ldq;
  p.dtype = x_dtype;
  p.recipe = recipe;
  p.vector_ok = aligned16(x) && (ldx * elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && ldq % 8 == 0;
  return note_cuda(launch_row_quantize(p, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_block_quantize(const void* x, int x_dtype, int64_t rows, int64_t cols, int64_t ldx, void* q, int64_t ldq,
                           float* scale, int64_t ld_scale, void* cuda_stream) {
  if (x == nullptr || q == nullptr || scale == nullptr) return B200FP8_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ldx < cols || ldq < cols || ld_scale < (cols + 127) / 128) return B200FP8_BAD_ARG;
  if (rows > 0x7FFFFF00ll || cols > 0x7FFFFF00ll || (rows + 127) / 128 > 65535) return B200FP8_TOO_LARGE;
  if (x_dtype < kQuantBf16 || x_dtype > kQuantFp32) return B200FP8_BAD_ARG;
  const int64_t elem = x_dtype == kQuantFp32 ? 4 : 2;
  BlockQuantParams p = {};
  p.x = x;
  p.q = static_cast<uint8_t*>(q);
  p.scale = scale;
  p.rows = rows;
  p.cols = cols;
  p.ldx = ldx;
  p.ldq = ldq;
  p.ld_scale = ld_scale;
  p.dtype = x_dtype;
  p.vector_ok = aligned16(x) && (ldx * elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && ldq % 8 == 0;
  return note_cuda(launch_block_quantize(p, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_fused_row_quantize(int producer, const void* x1, const void* x2, int64_t rows, int64_t cols, int64_t ld1,
                               int64_t ld2, float eps, int round_bf16, void* q, int64_t ldq, float* scale,
                               void* cuda_stream) {
  if (x1 == nullptr || x2 == nullptr || q == nullptr || scale == nullptr) return B200FP8_BAD_ARG;
  if (producer != kProducerRmsNorm && producer != kProducerSiluMul) return B200FP8_BAD_ARG;
  if (rows <= 0 || cols <= 0 || ld1 < cols || ldq < cols) return B200FP8_BAD_ARG;
  if (producer == kProducerSiluMul && ld2 < cols) return B200FP8_BAD_ARG;
  if (producer == kProducerRmsNorm && !(eps >= 0.0f)) return B200FP8_BAD_ARG;
  if (rows > 0x7FFFFFFFll || cols > 0x7FFFFF00ll) return B200FP8_TOO_LARGE;
  FusedQuantParams p = {};
  p.x1 = x1;
  p.x2 = x2;
  p.q = static_cast<uint8_t*>(q);
  p.scale = scale;
  p.rows = rows;
  p.cols = static_cast<int>(cols);
  p.ld1 = ld1;
  p.ld2 = producer == kProducerSiluMul ? ld2 : 0;
  p.ldq = ldq;
  p.producer = producer;
  p.round_bf16 = round_bf16 ? 1 : 0;
  p.eps = eps;
  p.vector_ok = aligned16(x1) && aligned16(x2) && (ld1 * 2) % 16 == 0 && (p.ld2 * 2) % 16 == 0 &&
                (reinterpret_cast<uintptr_t>(q) & 7u) == 0 && ldq % 8 == 0;
  return note_cuda(launch_fused_row_quantize(p, static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_selftest_wait_timeout(void* workspace, uint32_t limit_us, void* cuda_stream) {
  if (workspace == nullptr || limit_us == 0 || limit_us > 1000000u) return B200FP8_BAD_ARG;
  return note_cuda(launch_wait_timeout_selftest(static_cast<uint32_t*>(workspace),
                                                static_cast<unsigned long long>(limit_us) * 1000ull,
                                                static_cast<cudaStream_t>(cuda_stream)));
}

int b200fp8_query_status(const void* workspace, uint32_t* device_status) {
  if (workspace == nullptr) return B200FP8_BAD_ARG;
  uint32_t word = 0;
  const cudaError_t e = cudaMemcpy(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return note_cuda(e);
  if (device_status != nullptr) *device_status = word;
  return (word >> 24) == kDevTimeout ? B200FP8_DEVICE_TIMEOUT : B200FP8_OK;
}

int b200fp8_describe_plan(int64_t M, int64_t N, int64_t K, uint32_t flags, char* buf, size_t n) {
  if (buf == nullptr || n == 0) return B200FP8_BAD_ARG;
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  DeviceInfo dev;
  if (device_info(&dev) != B200FP8_OK) {
    dev.sm_count = 148;
    dev.max_pair_clusters = 74;
    dev.split_clusters[0] = 148;
    dev.split_clusters[1] = 74;
    dev.split_clusters[2] = 33;
    dev.split_clusters[3] = 15;
  }
  Plan pl;
  st = make_plan(M, N, K, flags, true, true, dev, &pl);
  if (st != B200FP8_OK) return st;
  switch (pl.variant) {
    case B200FP8_VARIANT_TC_1CTA:
      snprintf(buf, n, "tc_1cta tile=128x256x128 stages=%d ctas=%d group_m=%d smem=%d workspace=%zu",
               TcConfig<1>::kStages, pl.num_ctas, pl.group_m, TcConfig<1>::kSmemBytes, pl.workspace_bytes);
      break;
    case B200FP8_VARIANT_TC_2CTA:
      snprintf(buf, n, "tc_2cta tile=256x256x128 stages=%d ctas=%d group_m=%d smem=%d workspace=%zu",
               TcConfig<2>::kStages, pl.num_ctas, pl.group_m, TcConfig<2>::kSmemBytes, pl.workspace_bytes);
      break;
    case B200FP8_VARIANT_TC_SPLITK:
      snprintf(buf, n,
               "tc_splitk tile=128x%dx128 cluster=%d (K split, DSMEM reduce-scatter) x_rows=%d stages=%d ctas=%d "
               "waves=%d smem=%d resident_clusters=%d/%d/%d/%d workspace=%zu",
               pl.splitk.block_n, pl.splitk.split, pl.splitk.rows_a, pl.splitk.stages,
               pl.splitk.tiles * pl.splitk.split, pl.splitk.waves, pl.splitk.smem_bytes, dev.split_clusters[0],
               dev.split_clusters[1], dev.split_clusters[2], dev.split_clusters[3], pl.workspace_bytes);
      break;
    case B200FP8_VARIANT_GEMV:
      snprintf(buf, n, "gemv tokens=%d rows_per_warp=%d ctas=%d threads=512 loads_in_flight=4x16B smem=%zu workspace=%zu",
               pl.gemv.tokens, pl.gemv.rows_per_warp, pl.gemv.ctas, pl.gemv.smem_bytes, pl.workspace_bytes);
      break;
    case B200FP8_VARIANT_SKINNY:
      snprintf(buf, n,
               "skinny swap-AB stream-K tile=128(W rows)x%d(tokens)x128 stages=%d ctas=%d units_per_cta=%d "
               "whole_tiles_per_cta=%d k_split_tiles=%d smem=%zu workspace=%zu",
               pl.skinny.tokens_pad, pl.skinny.stages, pl.skinny.num_ctas, pl.skinny.units_per_cta,
               pl.skinny.dp_waves, pl.skinny.sk_tiles, pl.skinny.smem_bytes, pl.workspace_bytes);
      break;
    default:
      snprintf(buf, n, "simt tile=64x64x32 workspace=%zu", pl.workspace_bytes);
      break;
  }
  return B200FP8_OK;
}

// ------------------------------------ host-buffer context ------------------------------------
// One call = copy in, GEMM, copy out.  The copies are what the call costs (PCIe), so the problem is cut into
// panels that flow through three streams - uploads, GEMMs, downloads - with both PCIe directions busy at once.
//
// An element of Y needs its row of X and its row of W.  When W comes from the host with every call, sending all
// of W before the first X panel would keep the download direction idle for the first third of the call; instead
// row panels of X and of W go up alternately, and after every upload the strip of Y that has just become
// computable - the new X panel against all of W that is on the device, or all of X that is on the device against
// the new W panel - is multiplied by one GEMM and sent down by one copy (a pitched copy into the host array when
// the strip is narrower than Y).  The part of Y ready for download grows with the square of the bytes uploaded.
// When W stays on the device (b200fp8_host_ctx_set_weights) only X goes up and every strip is a full-width row
// panel (contiguous copies).
namespace {
constexpr int kMaxPanels = 64;       // per dimension
constexpr int kMaxCalls = 2 * kMaxPanels;  // GEMMs (= strips of Y) per call
constexpr int64_t kPanelRows = 1024;
constexpr int64_t kPanelCols = 2048;  // pitched downloads of narrower strips (2 KiB rows and less) were measured slower

struct HostStep {
  int kind;   // 0: upload X panel `index`, then the strip rows(panel) x [0, cols uploaded); 1: the same for W
  int index;
};
}  // namespace

struct b200fp8_host_ctx {
  int device;
  int64_t M, N, K;
  uint32_t flags;
  int64_t panel_rows, panel_cols;  // as configured; W resident: whole rows of Y (one column panel)
  cudaStream_t s_in, s_compute, s_out;
  cudaEvent_t ev_up[kMaxCalls];  // upload of step s has completed
  cudaEvent_t ev_y[kMaxCalls];   // GEMM of step s has completed
  uint8_t* d_x;
  uint8_t* d_w;
  float* d_xs;
  float* d_ws;
  __nv_bfloat16* d_bias;
  __nv_bfloat16* d_y;
  uint8_t* d_workspace;    // one workspace per GEMM in flight when the plan needs more than the status word
  size_t workspace_bytes;  // per GEMM
  size_t workspace_total;
  uint32_t* h_status;      // pinned, one word per GEMM
  bool weights_resident;
  bool bias_resident;
};

namespace {

struct DeviceGuard {  // the context's device is current inside the call, the caller's afterwards
  int previous = -1;
  cudaError_t enter(int device) {
    cudaError_t e = cudaGetDevice(&previous);
    if (e != cudaSuccess) return e;
    return previous == device ? cudaSuccess : cudaSetDevice(device);
  }
  ~DeviceGuard() {
    int now = -1;
    if (previous >= 0 && cudaGetDevice(&now) == cudaSuccess && now != previous) cudaSetDevice(previous);
  }
};

int panels_of(int64_t extent, int64_t panel) { return static_cast<int>((extent + panel - 1) / panel); }

// Largest workspace any strip of the context's panel grid can need: strips are (one row panel) x (1..pn column
// panels) or (1..pm row panels) x (one column panel); every such shape is asked for.
size_t strip_workspace_bytes(const b200fp8_host_ctx* c, int64_t panel_rows, int64_t panel_cols) {
  const int pm = panels_of(c->M, panel_rows), pn = panels_of(c->N, panel_cols);
  const int64_t last_rows = c->M - (pm - 1) * panel_rows, last_cols = c->N - (pn - 1) * panel_cols;
  size_t need = 0;
  auto ask = [&](int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return true;
    const size_t b = b200fp8_workspace_bytes(rows < c->M ? rows : c->M, cols < c->N ? cols : c->N, c->K, c->flags);
    if (b == 0) return false;
    if (b > need) need = b;
    return true;
  };
  for (int j = 1; j <= pn; ++j) {
    const int64_t cols = j < pn ? j * panel_cols : c->N;
    if (!ask(panel_rows, cols) || !ask(last_rows, cols)) return 0;
  }
  for (int i = 1; i <= pm; ++i) {
    const int64_t rows = i < pm ? i * panel_rows : c->M;
    if (!ask(rows, panel_cols) || !ask(rows, last_cols)) return 0;
  }
  return (need + 255) / 256 * 256;
}

// Upload order: always the operand of which the smaller fraction is on the device (X on a tie).
int build_schedule(int pm, int pn, bool weights_resident, HostStep* steps) {
  int n = 0, up_x = 0, up_w = weights_resident ? pn : 0;
  while (up_x < pm || up_w < pn) {
    const bool send_x = up_w >= pn || (up_x < pm && up_x * pn <= up_w * pm);
    if (send_x) {
      steps[n++] = {0, up_x++};
    } else {
      steps[n++] = {1, up_w++};
    }
  }
  return n;
}

void sync_all(b200fp8_host_ctx* c) {
  cudaStreamSynchronize(c->s_in);
  cudaStreamSynchronize(c->s_compute);
  cudaStreamSynchronize(c->s_out);
}

}  // namespace

int b200fp8_host_ctx_destroy(b200fp8_host_ctx* c) {
  if (c == nullptr) return B200FP8_OK;
  DeviceGuard guard;
  guard.enter(c->device);
  if (c->s_in) cudaStreamSynchronize(c->s_in);
  if (c->s_compute) cudaStreamSynchronize(c->s_compute);
  if (c->s_out) cudaStreamSynchronize(c->s_out);
  cudaFree(c->d_x);
  cudaFree(c->d_w);
  cudaFree(c->d_xs);
  cudaFree(c->d_ws);
  cudaFree(c->d_bias);
  cudaFree(c->d_y);
  cudaFree(c->d_workspace);
  if (c->h_status) cudaFreeHost(c->h_status);
  for (int i = 0; i < kMaxCalls; ++i) {
    if (c->ev_up[i]) cudaEventDestroy(c->ev_up[i]);
    if (c->ev_y[i]) cudaEventDestroy(c->ev_y[i]);
  }
  if (c->s_in) cudaStreamDestroy(c->s_in);
  if (c->s_compute) cudaStreamDestroy(c->s_compute);
  if (c->s_out) cudaStreamDestroy(c->s_out);
  delete c;
  return B200FP8_OK;
}

int b200fp8_host_ctx_set_panels(b200fp8_host_ctx* c, int64_t panel_rows, int64_t panel_cols) {
  if (c == nullptr || panel_rows <= 0 || panel_cols <= 0) return B200FP8_BAD_ARG;
  if (panel_rows > c->M) panel_rows = c->M;
  if (panel_cols > c->N) panel_cols = c->N;
  // interior panels must keep every block's pointers aligned for TMA: whole 128-row / 256-column tiles
  if (panel_rows < c->M && panel_rows % 128 != 0) return B200FP8_BAD_ARG;
  if (panel_cols < c->N && panel_cols % 256 != 0) return B200FP8_BAD_ARG;
  const int pm = panels_of(c->M, panel_rows), pn = panels_of(c->N, panel_cols);
  if (pm > kMaxPanels || pn > kMaxPanels) return B200FP8_TOO_LARGE;
  DeviceGuard guard;
  cudaError_t e = guard.enter(c->device);
  if (e != cudaSuccess) return note_cuda(e);
  const size_t per = strip_workspace_bytes(c, panel_rows, panel_cols);  // covers the full-width strips of resident weights
  if (per == 0) return B200FP8_BAD_ARG;
  // kernels that need only the status word share one workspace; the others get one per GEMM of a call
  const size_t total = per == B200FP8_WORKSPACE_HEADER_BYTES ? per : per * static_cast<size_t>(pm + pn);
  if (total > c->workspace_total) {
    sync_all(c);
    cudaFree(c->d_workspace);
    c->d_workspace = nullptr;
    c->workspace_total = 0;
    e = cudaMalloc(&c->d_workspace, total);
    if (e != cudaSuccess) return note_cuda(e);
    c->workspace_total = total;
    e = cudaMemsetAsync(c->d_workspace, 0, total, c->s_compute);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->s_compute);
    if (e != cudaSuccess) return note_cuda(e);
  }
  c->workspace_bytes = per;
  c->panel_rows = panel_rows;
  c->panel_cols = panel_cols;
  return B200FP8_OK;
}

int b200fp8_host_ctx_create(int64_t M, int64_t N, int64_t K, uint32_t flags, b200fp8_host_ctx** out) {
  if (out == nullptr) return B200FP8_BAD_ARG;
  *out = nullptr;
  int st = check_sizes(M, N, K);
  if (st != B200FP8_OK) return st;
  DeviceInfo dev;
  st = device_info(&dev);
  if (st != B200FP8_OK) return st;
  if (dev.cc_major != 10) return B200FP8_UNSUPPORTED_ARCH;
  b200fp8_host_ctx* c = new (std::nothrow) b200fp8_host_ctx();
  if (c == nullptr) return B200FP8_BAD_ARG;
  memset(c, 0, sizeof(*c));
  c->M = M;
  c->N = N;
  c->K = K;
  c->flags = flags;
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_compute, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking);
  for (int i = 0; i < kMaxCalls && e == cudaSuccess; ++i) {
    e = cudaEventCreateWithFlags(&c->ev_up[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev_y[i], cudaEventDisableTiming);
  }
  if (e == cudaSuccess) e = cudaMalloc(&c->d_x, static_cast<size_t>(M) * K);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_w, static_cast<size_t>(N) * K);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_xs, static_cast<size_t>(M) * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&c->d_ws, static_cast<size_t>(N) * sizeof(float));
  if (e == cudaSuccess) e = cudaMalloc(&c->d_bias, static_cast<size_t>(N) * sizeof(__nv_bfloat16));
  if (e == cudaSuccess) e = cudaMalloc(&c->d_y, static_cast<size_t>(M) * N * sizeof(__nv_bfloat16));
  if (e == cudaSuccess) e = cudaMallocHost(&c->h_status, sizeof(uint32_t) * kMaxCalls);
  if (e != cudaSuccess) {
    b200fp8_host_ctx_destroy(c);
    return note_cuda(e);
  }
  // Panels once a dimension holds at least two of them; one panel otherwise.  Small problems (a few MB in
  // all) are not worth cutting: a panel's copy should last much longer than the ~10 us a copy costs to start.
  int64_t rows = M >= 2 * kPanelRows ? kPanelRows : M;
  int64_t cols = N >= 2 * kPanelCols ? kPanelCols : N;
  if (static_cast<double>(M + N) * static_cast<double>(K) < 8.0e6) {
    rows = M;
    cols = N;
  }
  while (panels_of(M, rows) > 16) rows *= 2;
  while (panels_of(N, cols) > 16) cols *= 2;
  st = b200fp8_host_ctx_set_panels(c, rows, cols);
  if (st != B200FP8_OK) {
    b200fp8_host_ctx_destroy(c);
    return st;
  }
  *out = c;
  return B200FP8_OK;
}

int b200fp8_host_ctx_set_weights(b200fp8_host_ctx* c, const void* wq, const float* w_scale, const void* bias_bf16) {
  if (c == nullptr) return B200FP8_BAD_ARG;
  DeviceGuard guard;
  cudaError_t e = guard.enter(c->device);
  if (e != cudaSuccess) return note_cuda(e);
  if (wq == nullptr) {  // forget the resident copy: later calls take W from the host again
    c->weights_resident = false;
    c->bias_resident = false;
    return B200FP8_OK;
  }
  if (w_scale == nullptr) return B200FP8_BAD_ARG;
  const size_t N = static_cast<size_t>(c->N), K = static_cast<size_t>(c->K);
  e = cudaMemcpyAsync(c->d_w, wq, N * K, cudaMemcpyHostToDevice, c->s_in);
  if (e == cudaSuccess) e = cudaMemcpyAsync(c->d_ws, w_scale, N * sizeof(float), cudaMemcpyHostToDevice, c->s_in);
  if (e == cudaSuccess && bias_bf16 != nullptr) {
    e = cudaMemcpyAsync(c->d_bias, bias_bf16, N * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice, c->s_in);
  }
  const cudaError_t e2 = cudaStreamSynchronize(c->s_in);
  if (e == cudaSuccess) e = e2;
  if (e != cudaSuccess) return note_cuda(e);
  c->weights_resident = true;
  c->bias_resident = bias_bf16 != nullptr;
  return B200FP8_OK;
}

int b200fp8_gemm_rowwise_host(b200fp8_host_ctx* c, const void* xq, const void* wq, const float* x_scale,
                              const float* w_scale, const void* bias_bf16, void* y_bf16) {
  if (c == nullptr || xq == nullptr || x_scale == nullptr || y_bf16 == nullptr) return B200FP8_BAD_ARG;
  const bool resident = wq == nullptr;  // reuse the W, w_scale and bias of the last upload
  if (resident ? !c->weights_resident : w_scale == nullptr) return B200FP8_BAD_ARG;
  DeviceGuard guard;
  cudaError_t e = guard.enter(c->device);
  if (e != cudaSuccess) return note_cuda(e);

  const size_t M = static_cast<size_t>(c->M), N = static_cast<size_t>(c->N), K = static_cast<size_t>(c->K);
  const int64_t panel_rows = c->panel_rows;
  const int64_t panel_cols = resident ? c->N : c->panel_cols;
  const int pm = panels_of(c->M, panel_rows), pn = panels_of(c->N, panel_cols);
  const bool shared_workspace = c->workspace_bytes == B200FP8_WORKSPACE_HEADER_BYTES;
  const bool use_bias = resident ? c->bias_resident : bias_bf16 != nullptr;
  HostStep steps[kMaxCalls];
  const int num_steps = build_schedule(pm, pn, resident, steps);

  // the scales and the bias are a few KB: all of them first
  e = cudaMemcpyAsync(c->d_xs, x_scale, M * sizeof(float), cudaMemcpyHostToDevice, c->s_in);
  if (!resident) {
    if (e == cudaSuccess) e = cudaMemcpyAsync(c->d_ws, w_scale, N * sizeof(float), cudaMemcpyHostToDevice, c->s_in);
    if (e == cudaSuccess && bias_bf16 != nullptr) {
      e = cudaMemcpyAsync(c->d_bias, bias_bf16, N * sizeof(__nv_bfloat16), cudaMemcpyHostToDevice, c->s_in);
    }
  }
  if (!resident) c->weights_resident = false;  // until this call's upload has completed
  const uint8_t* x_host = static_cast<const uint8_t*>(xq);
  const uint8_t* w_host = static_cast<const uint8_t*>(wq);
  __nv_bfloat16* y_host = static_cast<__nv_bfloat16*>(y_bf16);
  int status = B200FP8_OK;
  int calls = 0;
  size_t rows_up = 0, cols_up = resident ? N : 0;  // rows of X / rows of W on the device so far
  for (int s = 0; s < num_steps && e == cudaSuccess && status == B200FP8_OK; ++s) {
    const HostStep& step = steps[s];
    size_t r0, rows, c0, cols;  // the strip of Y this upload makes computable
    if (step.kind == 0) {
      r0 = static_cast<size_t>(step.index) * panel_rows;
      rows = r0 + panel_rows <= M ? static_cast<size_t>(panel_rows) : M - r0;
      e = cudaMemcpyAsync(c->d_x + r0 * K, x_host + r0 * K, rows * K, cudaMemcpyHostToDevice, c->s_in);
      rows_up = r0 + rows;
      c0 = 0;
      cols = cols_up;
    } else {
      c0 = static_cast<size_t>(step.index) * panel_cols;
      cols = c0 + panel_cols <= N ? static_cast<size_t>(panel_cols) : N - c0;
      e = cudaMemcpyAsync(c->d_w + c0 * K, w_host + c0 * K, cols * K, cudaMemcpyHostToDevice, c->s_in);
      cols_up = c0 + cols;
      r0 = 0;
      rows = rows_up;
    }
    if (e == cudaSuccess) e = cudaEventRecord(c->ev_up[s], c->s_in);
    if (e != cudaSuccess || rows == 0 || cols == 0) continue;  // nothing computable yet (the very first upload)
    // uploads are ordered on one stream: waiting for this one covers every earlier panel and the scales
    e = cudaStreamWaitEvent(c->s_compute, c->ev_up[s], 0);
    if (e != cudaSuccess) break;
    uint8_t* ws = c->d_workspace + (shared_workspace ? 0 : static_cast<size_t>(calls) * c->workspace_bytes);
    status = b200fp8_gemm_rowwise(c->d_x + r0 * K, c->d_w + c0 * K, c->d_xs + r0, c->d_ws + c0,
                                  use_bias ? c->d_bias + c0 : nullptr, c->d_y + r0 * N + c0,
                                  static_cast<int64_t>(rows), static_cast<int64_t>(cols), c->K, c->K, c->K, c->N, ws,
                                  c->workspace_bytes, c->flags, c->s_compute);
    if (status != B200FP8_OK) break;
    e = cudaEventRecord(c->ev_y[calls], c->s_compute);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->s_out, c->ev_y[calls], 0);
    if (e == cudaSuccess) {
      if (cols == N) {
        e = cudaMemcpyAsync(y_host + r0 * N, c->d_y + r0 * N, rows * N * sizeof(__nv_bfloat16), cudaMemcpyDeviceToHost,
                            c->s_out);
      } else {
        e = cudaMemcpy2DAsync(y_host + r0 * N + c0, N * sizeof(__nv_bfloat16), c->d_y + r0 * N + c0,
                              N * sizeof(__nv_bfloat16), cols * sizeof(__nv_bfloat16), rows, cudaMemcpyDeviceToHost,
                              c->s_out);
      }
    }
    if (e == cudaSuccess && !shared_workspace) {
      e = cudaMemcpyAsync(c->h_status + calls, ws, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->s_out);
    }
    ++calls;
  }
  if (e == cudaSuccess && status == B200FP8_OK && shared_workspace) {
    e = cudaMemcpyAsync(c->h_status, c->d_workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->s_out);
  }
  // Whatever happened, the caller gets its host buffers back only when no copy is in flight on them: all
  // three streams are waited for.
  const cudaError_t e_in = cudaStreamSynchronize(c->s_in);
  const cudaError_t e_compute = cudaStreamSynchronize(c->s_compute);
  const cudaError_t e_out = cudaStreamSynchronize(c->s_out);
  if (status != B200FP8_OK) return status;
  if (e == cudaSuccess) e = e_in;
  if (e == cudaSuccess) e = e_compute;
  if (e == cudaSuccess) e = e_out;
  if (e != cudaSuccess) return note_cuda(e);
  if (!resident) {
    c->weights_resident = true;
    c->bias_resident = bias_bf16 != nullptr;
  }
  const int words = shared_workspace ? 1 : calls;
  for (int i = 0; i < words; ++i) {
    if ((c->h_status[i] >> 24) == kDevTimeout) {
      // leave the workspace clean for the next call
      cudaMemsetAsync(c->d_workspace, 0, c->workspace_total, c->s_compute);
      cudaStreamSynchronize(c->s_compute);
      return B200FP8_DEVICE_TIMEOUT;
    }
  }
  return B200FP8_OK;
}

}  // extern "C"
