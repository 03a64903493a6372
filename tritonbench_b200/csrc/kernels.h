// Internal launch interface between the C-ABI layer (api.cu) and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200fp8 {

// Device status word (first word of every workspace): code << 24 | site of the wait that gave up.
constexpr uint32_t kDevOk = 0u;
constexpr uint32_t kDevTimeout = 1u;

// --------------------------- large-M tcgen05 kernel (gemm_tc.cu) ---------------------------
struct TcGeometry {
  static constexpr int kBlockM = 128;    // rows of X per CTA (TMEM lanes)
  static constexpr int kBlockN = 256;    // columns of Y per tile (MMA N)
  static constexpr int kBlockK = 128;    // bytes (= e4m3 elements) of K per pipeline stage
  static constexpr int kStoreCols = 64;  // bf16 columns per TMA-store box (128 bytes)
  static constexpr int kStoreRows = 32;  // rows per TMA-store box (one epilogue warp)
  static constexpr int kThreads = 192;   // warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 epilogue
};

template <int kCtaGroup>
struct TcConfig : TcGeometry {
  static constexpr int kRowsW = kBlockN / kCtaGroup;                  // W rows each CTA loads per stage
  static constexpr int kBytesA = kBlockM * kBlockK;                   // 16 KiB
  static constexpr int kBytesB = kRowsW * kBlockK;                    // 32 KiB / 16 KiB
  static constexpr int kStages = kCtaGroup == 1 ? 4 : 6;              // 192 KiB of operand ring either way
  static constexpr int kStageTxBytes = (kBytesA + kBytesB) * kCtaGroup;  // bytes credited to one full barrier
  static constexpr int kEpiBytes = 4 * 2 * kStoreRows * kStoreCols * 2;  // 4 warps x 2 buffers x 4 KiB
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * (kBytesA + kBytesB) + kEpiBytes + kBarBytes + 1024;
  static constexpr int kTileM = kBlockM * kCtaGroup;  // rows of Y per (cluster) tile
};

struct TcParams {
  const float* x_scale;
  const float* w_scale;
  const __nv_bfloat16* bias;  // may be null
  __nv_bfloat16* y;
  int M, N, K;
  long long ldy;       // elements
  int use_tma_store;   // 0: plain predicated stores
  int out_fp16;        // 0: Y holds bf16, 1: Y holds IEEE fp16
  int group_m;         // tile-rasterisation group height (tiles)
  int num_groups;      // 0: plain GEMM.  >0: rows of X are partitioned into groups (single-CTA variant)
  const int* group_rows;  // [num_groups] rows per group, device memory; group g uses W rows [g*N, (g+1)*N)
  int num_extra;       // copies of Y to write besides `y` (TMA stores only; 0 for the plain GEMM)
  int y_evict_first;   // TMA stores of Y carry the L2 evict-first hint
  uint32_t* status;    // device status word
};

// Extra destinations of every tile of Y: the same rows inside other buffers - in the sharded run, the copies
// of the gathered [M_total, N] matrix that live on the other GPUs, mapped into this process.  Each map covers
// the [M, N] slice of its buffer where this rank's rows belong, so a box has the same coordinates in all of them.
constexpr int kMaxExtraOutputs = 7;
struct alignas(64) ExtraOutputs {
  CUtensorMap tm[kMaxExtraOutputs];
};

template <int kCtaGroup>
cudaError_t launch_gemm_tc(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                           const TcParams& p, int num_ctas, cudaStream_t stream, const ExtraOutputs* extra = nullptr);

// One 128 x block_n tile per cluster of `split` CTAs, K split over the cluster and reduced over distributed
// shared memory (gemm_splitk.cu).  split is 1, 2, 4 or 8; block_n a multiple of 16 * split, at most 256 - or, with
// split 1 only, a multiple of 64 up to 512: a wide tile, multiplied as two column halves, for outputs whose
// 256-column tiles would need a second, mostly empty wave of CTAs.
struct SplitGeometry {
  static constexpr int kRingBytes = 192 * 1024;
  static constexpr int kMaxStages = 14;
  static constexpr int kMaxBlockN = 512;     // split 1; 256 with a K split
  // most dynamic shared memory a CTA asks for: ring, store staging (32 KiB), scales (1 KiB), barriers, alignment
  static constexpr int kMaxSmemBytes = kRingBytes + 32 * 1024 + 1024 + 256 + 1024;
  static constexpr int kSmemPerSm = 227 * 1024;  // shared memory the CTAs of one SM can hold together
  static constexpr int kTmemColsPerSm = 512;
  // Smallest dynamic shared-memory request with which the CTAs that fit on one SM by shared memory
  // (floor(kSmemPerSm / request)) hold at most the SM's 512 tensor-memory columns between them.
  static constexpr int min_smem_bytes_for_tmem(int tmem_cols) {
    const int max_ctas = kTmemColsPerSm / tmem_cols;
    return (kSmemPerSm / (max_ctas + 1) / 1024 + 1) * 1024;
  }
};
// tensor-memory columns a CTA of the one-tile-per-cluster kernel allocates for a tile of block_n columns
__host__ __device__ constexpr int split_tmem_cols(int block_n) {
  return block_n <= 32 ? 32 : (block_n <= 64 ? 64 : (block_n <= 128 ? 128 : (block_n <= 256 ? 256 : 512)));
}
// a tile wider than 256 columns is multiplied as two halves: columns [0, first) and [first, block_n)
__host__ __device__ constexpr int split_first_half(int block_n) { return block_n <= 256 ? block_n : block_n / 2; }
// shared memory for the W scales of a CTA's column slice
__host__ __device__ constexpr int split_scale_bytes(int block_n) { return block_n <= 256 ? 1024 : 2048; }
struct SplitPlan {
  int block_n;
  int split;
  int rows_a;                    // rows of X per stage: M rounded up to 8, at most 128
  int stages;                    // operand stages in the ring
  int ring_bytes;                // ring (operands, then the split-K exchange), a multiple of 1024, at most 192 KiB
  int staged_stores;             // 1: Y leaves through TMA boxes staged in shared memory (tall outputs)
  int smem_bytes;                // dynamic shared memory of a CTA
  int tiles;                     // clusters
  int waves;                     // tiles / clusters resident at once, rounded up
  bool overlap_previous_kernel;  // programmatic stream serialization: W is prefetched under the previous kernel
};
// resident_clusters[i]: clusters of 2^i CTAs of this kernel the device runs at once (i = 0..3)
SplitPlan make_split_plan(long long M, long long N, long long K, const int* resident_clusters, int forced_block_n,
                          int forced_split);
double split_plan_cost_us(long long M, long long N, long long K, int block_n, int split, int resident_clusters);
// Clusters of `split` CTAs the current device can run at once (a cluster must fit inside one GPC, so this
// is less than SMs / split); 0 with the error left in *err when the query fails.
int splitk_resident_clusters(int split, cudaError_t* err);
cudaError_t launch_gemm_splitk(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                               const TcParams& p, const SplitPlan& plan, cudaStream_t stream);

// ------------------------ 128x128 block-scaled GEMM (gemm_blockwise.cu) ------------------------
struct BlockwiseParams {
  const float* x_scale;  // [ceil(M/128)][ld_xs >= ceil(K/128)]
  const float* w_scale;  // [ceil(N/128)][ld_ws >= ceil(K/128)]
  __nv_bfloat16* y;
  int M, N, K;
  long long ldy, ld_xs, ld_ws;  // elements
  int use_tma_store;
  int group_m;
  uint32_t* status;
};

cudaError_t launch_gemm_blockwise(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                                  const BlockwiseParams& p, int num_ctas, cudaStream_t stream);

// ------------------------ skinny-M stream-K kernel (gemm_skinny.cu) ------------------------
struct SkinnyGeometry {
  static constexpr int kRowsW = 128;   // W rows per tile (MMA M, TMEM lanes)
  static constexpr int kBlockK = 128;  // bytes of K per stage
  static constexpr int kMaxTokens = 128;
  static constexpr int kThreads = 320;  // producer, MMA issuer, 4 drain warps, 4 fix-up warps
  static constexpr int kBytesA = kRowsW * kBlockK;  // 16 KiB of W per stage
  static constexpr int kBarBytes = 1024;
  static constexpr int kMaxStages = 12;
  // The arrival counters occupy a region of fixed size right after the workspace header, whatever
  // N is, so that a workspace left zero by one problem size is still zero where the next size
  // (with a different number of tiles) looks for its counters.
  static constexpr int kMaxTiles = 16384;  // N <= 2,097,152
  static constexpr size_t kCounterRegionBytes = static_cast<size_t>(kMaxTiles) * 4 * sizeof(uint32_t);
  static constexpr int kSmemBudget = 220 * 1024;
};

struct SkinnyPlan {
  int tokens_pad;    // M rounded up to 16: MMA N and rows of the X box
  int stages;        // pipeline depth
  int num_ctas;      // grid
  int tiles;         // ceil(N / 128)
  int kblocks;       // ceil(K / 128)
  int units_per_cta; // consecutive (tile, k-block) units each CTA owns
  int segs_per_cta;  // upper bound on tile segments per CTA (partial-sum slots)
  int dp_waves;      // whole tiles per CTA (tiles / CTAs)
  int sk_tiles;      // remaining tiles, cut along K into equal runs
  bool overlap_previous_kernel;  // launch with programmatic stream serialization
  size_t smem_bytes;
  size_t partial_bytes;  // fp32 partial sums
  size_t counter_bytes;  // fixed-size region of per (tile, lane quarter) arrival counters
};

SkinnyPlan make_skinny_plan(int M, int N, int K, int sm_count);

// what the kernel needs of the plan
struct SkinnyShape {
  int tokens_pad, stages, kblocks;
  int units_per_cta, segs_per_cta;
  long long sk_units;  // units of the K-split region = sk_tiles * kblocks
  int sk_tiles, tiles;
};

struct SkinnyParams {
  const float* x_scale;
  const float* w_scale;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  int M, N, K;
  long long ldy;
  int out_fp16;
  float* partials;     // [num_ctas * segs_per_cta][tokens_pad][128] fp32
  uint32_t* counters;  // [tiles * 4], zero on entry, zero again on exit
  uint32_t* status;
};

cudaError_t launch_gemm_skinny(const CUtensorMap& tm_w, const CUtensorMap& tm_x, const SkinnyParams& p,
                               const SkinnyPlan& plan, cudaStream_t stream);

// Library-owned scratch for the entry point that allocates nothing: a fixed-size array in device
// global memory that is part of the loaded module.  Returns its device address for the CURRENT
// device (looked up once per device) and its size.
constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB per GPU that loads the library
cudaError_t skinny_static_scratch(void** device_ptr, size_t* bytes);

// ------------------------ GEMV for one to four tokens (gemm_gemv.cu) ------------------------
constexpr int kGemvMaxTokens = 4;
constexpr size_t kGemvMaxSmemBytes = 112 * 1024;  // X as fp16 in shared memory, two CTAs per SM
struct GemvParams {
  const uint8_t* xq;
  const uint8_t* wq;
  const float* x_scale;
  const float* w_scale;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  int M, N, K;
  long long ldx, ldw, ldy;
  int out_fp16;
  int overlap;        // launched with programmatic stream serialization
  int rows_per_warp;  // filled in from the plan
};
struct GemvPlan {
  bool ok;            // M <= 4, K a multiple of 16, X fits in shared memory
  int tokens;         // kernel instance: 1, 2 or 4 rows of X
  int rows_per_warp;  // rows of W per warp, the same for every warp
  int ctas;
  size_t smem_bytes;
};
GemvPlan make_gemv_plan(long long M, long long N, long long K, int sm_count);
cudaError_t launch_gemm_gemv(const GemvParams& p, const GemvPlan& plan, cudaStream_t stream);

// ------------------------------ CUDA-core kernel (gemm_simt.cu) -----------------------------
struct SimtParams {
  const uint8_t* xq;
  const uint8_t* wq;
  const float* x_scale;
  const float* w_scale;
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;
  int M, N, K;
  long long ldx, ldw, ldy;
  int out_fp16;
};

cudaError_t launch_gemm_simt(const SimtParams& p, cudaStream_t stream);

// one CTA waits `limit_ns` on a barrier nothing arrives on, then records a time-out in *status
cudaError_t launch_wait_timeout_selftest(uint32_t* status, unsigned long long limit_ns, cudaStream_t stream);

// ------------------------------ rowwise quantiser (quantize.cu) -----------------------------
constexpr int kQuantBf16 = 0, kQuantFp16 = 1, kQuantFp32 = 2;  // dtype of x
constexpr int kRecipeOperator = 0;  // the operator's fp8_row_quantize: arithmetic in x's dtype, multiplier 448/max
constexpr int kRecipeFp32 = 1;      // benchmark recipe: scale = max(absmax, 1e-12) / 448 in fp32, q = x / scale

struct QuantParams {
  const void* x;
  uint8_t* q;
  float* scale;
  long long rows;
  int cols;
  long long ldx;  // elements
  long long ldq;  // bytes
  int dtype;
  int recipe;
  int vector_ok;  // rows of x start on 16-byte boundaries and rows of q on 8-byte boundaries
};

cudaError_t launch_row_quantize(const QuantParams& p, cudaStream_t stream);

// 128x128 block quantiser (quantize.cu): q [rows, cols] e4m3, scale [ceil(rows/128)][ld_scale >= ceil(cols/128)] fp32
struct BlockQuantParams {
  const void* x;
  uint8_t* q;
  float* scale;
  long long rows, cols;
  long long ldx;       // elements
  long long ldq;       // bytes
  long long ld_scale;  // elements
  int dtype;
  int vector_ok;  // rows of x start on 16-byte boundaries and rows of q on 8-byte boundaries
};
cudaError_t launch_block_quantize(const BlockQuantParams& p, cudaStream_t stream);

// ------------------------ producer + quantiser in one pass (fused_quantize.cu) ------------------------
constexpr int kProducerRmsNorm = 1;  // y = x1 * rsqrt(mean(x1^2) + eps) * x2[k]   (x2: weight vector [cols])
constexpr int kProducerSiluMul = 2;  // y = silu(x1) * x2                          (x2: [rows, cols])
struct FusedQuantParams {
  const void* x1;  // bf16 [rows, cols]
  const void* x2;  // bf16: weight [cols] or second operand [rows, cols]
  uint8_t* q;
  float* scale;
  long long rows;
  int cols;
  long long ld1, ld2;  // elements
  long long ldq;       // bytes
  int producer;
  int round_bf16;  // round y to bf16 before quantising (what a producer kernel followed by a quantiser computes)
  float eps;       // RMS norm only
  int vector_ok;   // rows of x1, x2 start on 16-byte boundaries, rows of q on 8-byte boundaries
};
cudaError_t launch_fused_row_quantize(const FusedQuantParams& p, cudaStream_t stream);

}  // namespace b200fp8
