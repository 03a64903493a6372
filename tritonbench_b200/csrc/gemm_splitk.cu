// FP8 rowwise GEMM for problems whose output has too few 128x256 tiles to occupy the GPU with the
// persistent kernels: narrower tiles, and split-K inside a thread-block cluster, reduced over
// distributed shared memory.
//
// A cluster of S CTAs (S = 1, 2, 4 or 8) owns one 128 x BN tile of Y (BN a multiple of 16 S, at most 256:
// the host picks the width that gives every SM a tile where it can).  CTA r multiplies the r-th slice of K
// with the usual pipeline (TMA -> 128B-swizzled ring -> tcgen05.mma -> TMEM); the ring is deep enough that
// a short slice is requested from memory all at once.  Then, S > 1:
//   (A) cluster barrier: every CTA's MMAs have finished, so every operand ring is free;
//   exchange: each CTA writes its fp32 partial tile, column slice j (BN/S columns) to CTA j,
//   into CTA j's (now idle) operand ring through shared::cluster stores - a reduce-scatter;
//   (B) cluster barrier: all partials have landed;
//   each CTA adds the S partials of its column slice in CTA order (fixed, deterministic),
//   applies the scales, rounds and stores its 128 x BN/S part of the tile.
// Partial sums never leave the SMs, and the epilogue is spread over the S CTAs.  With S = 1 the
// epilogue reads the accumulator straight from TMEM.  Rows of the tile beyond M are neither exchanged
// nor stored, so a decode-sized M costs a decode-sized epilogue.
//
// With `overlap_previous_kernel` the kernel is launched with programmatic stream serialization: its
// set-up and its first W loads run while the previous kernel on the stream drains; X is read, and Y
// written, only after that kernel has completed.
//
// Every mbarrier wait is bounded; a CTA that gives up still arrives at both cluster barriers so
// that its peers are never left waiting.
#include <mutex>
#include <type_traits>

#include "kernels.h"
#include "ptx.cuh"

namespace b200fp8 {
namespace {

using Geo = TcGeometry;

// The operand ring holds at most 192 KiB: a stage is `rows_a` rows of X (M rounded up to 8, at most 128;
// the MMA reads 128 rows, the rows never loaded only feed output rows that do not exist) and block_n rows
// of W, and as many stages as fit (and as the CTA has k-blocks) are kept in flight - for a decode-sized M
// almost all of them W.  A CTA with few k-blocks asks for a small ring, and two CTAs then fit on an SM:
// with overlapped launches the next kernel's CTA loads its W while this one is still in its epilogue.
struct C {
  static constexpr int kRingBytes = SplitGeometry::kRingBytes;  // reused for the exchange
  static constexpr int kExchangeBytes = Geo::kBlockM * 256 * 4;  // fp32 partials a CTA receives, widest tile
  static constexpr int kEpiBytes = 4 * 2 * Geo::kStoreRows * Geo::kStoreCols * 2;
  static constexpr int kScaleBytes = 256 * 4;  // w_scale of the CTA's column slice (twice that for a wide tile, whose ring is short)
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kRingBytes + kEpiBytes + kScaleBytes + kBarBytes + 1024;
  static_assert(kExchangeBytes <= kRingBytes, "the exchange buffer lives in the operand ring");
  static_assert(16 * SplitGeometry::kMaxStages + 16 <= kBarBytes, "barrier block");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
  static_assert(kSmemBytes == SplitGeometry::kMaxSmemBytes, "the host plans against the same limit");
};

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

template <int kCols>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[kCols]) {
  if constexpr (kCols == 64) {  // two reads in flight, one wait
    tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
  } else if constexpr (kCols == 32) {
    tmem_ld_32x32(taddr, r);
  } else {
    tmem_ld_32x16(taddr, r);
  }
}

// Exchange buffer of a CTA: [sender][group of 4 columns of its slice][row][4 columns] fp32 with `rows` rows
// (the rows of the tile that exist, rounded up to 8), so that a warp (32 consecutive rows) moves 512
// contiguous bytes per instruction.
__device__ __forceinline__ uint32_t exchange_offset(int sender, int slice_cols, int col_in_slice, int row, int rows) {
  return static_cast<uint32_t>((((sender * (slice_cols / 4) + col_in_slice / 4) * rows) + row) * 16);
}

// Everything one epilogue warp needs to finish columns of its 32 rows, by value: a pointer to the
// kernel's parameter block would turn every field access into a load the compiler cannot keep in a register.
struct Finish {
  uint16_t* y_row;         // &Y[row][first column of this CTA's slice]
  uint32_t scales;         // shared address: w_scale of the slice, zero beyond N
  const __nv_bfloat16* bias;  // bias of the slice's first column, or null
  uint32_t exchange_base;  // shared address of the exchange buffer (split > 1)
  uint32_t t_addr;         // TMEM address of this warp's lanes at the slice's first column (split == 1)
  int split, slice_cols, tile_row, lane;
  int exchange_rows;       // rows per column group in the exchange buffer
  int cols_valid;          // columns of the slice that exist in Y
  float xs;
  bool row_valid;
  bool out_fp16;
  bool boxed;              // slice is a multiple of 64 columns and Y can take TMA stores
  bool vector_ok;          // rows of Y start on 16-byte boundaries
};

// Sum (or read), scale and round `kCols` columns starting at `c_in_slice`, then store them: into the
// staging box (flushed by the caller every 64 columns), or straight to Y.
// kSplitK / kBoxed / kPlain (no bias, bf16 output) are compile-time: a launch runs this code once, cold, so every
// instruction of a path it does not take still costs instruction-cache lines on the way.
template <int kCols, bool kSplitK, bool kBoxed, bool kPlain>
__device__ __forceinline__ void finish_columns(const Finish& f, int c_in_slice, uint32_t sbuf) {
  float v[kCols];
  if constexpr (!kSplitK) {
    uint32_t raw[kCols];
    tmem_ld_cols<kCols>(f.t_addr + c_in_slice, raw);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < kCols; ++j) v[j] = __uint_as_float(raw[j]);
  } else {
#pragma unroll
    for (int j = 0; j < kCols; ++j) v[j] = 0.0f;
    for (int sender = 0; sender < f.split; ++sender) {  // CTA order: the sum does not depend on timing
      const uint32_t src =
          f.exchange_base + exchange_offset(sender, f.slice_cols, c_in_slice, f.tile_row, f.exchange_rows);
#pragma unroll
      for (int j = 0; j < kCols / 4; ++j) {
        const float4 t = ld_shared_v4(src + j * f.exchange_rows * 16);
        v[4 * j + 0] += t.x;
        v[4 * j + 1] += t.y;
        v[4 * j + 2] += t.z;
        v[4 * j + 3] += t.w;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kCols / 4; ++j) {  // columns beyond N carry a zero scale
    const float4 ws = ld_shared_v4(f.scales + (c_in_slice + 4 * j) * 4);
    v[4 * j + 0] *= f.xs * ws.x;
    v[4 * j + 1] *= f.xs * ws.y;
    v[4 * j + 2] *= f.xs * ws.z;
    v[4 * j + 3] *= f.xs * ws.w;
  }
  if constexpr (!kPlain) {
    if (f.bias != nullptr) {
#pragma unroll
      for (int j = 0; j < kCols; ++j) {
        if (c_in_slice + j < f.cols_valid) v[j] += __bfloat162float(f.bias[c_in_slice + j]);
      }
    }
  }
  uint32_t packed[kCols / 2];
#pragma unroll
  for (int j = 0; j < kCols / 2; ++j) {
    if constexpr (kPlain) {
      packed[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    } else {
      packed[j] = f.out_fp16 ? pack_f16x2(v[2 * j], v[2 * j + 1]) : pack_bf16x2(v[2 * j], v[2 * j + 1]);
    }
  }
  if constexpr (kBoxed) {
    const uint32_t row_addr = sbuf + f.lane * 128;
    const int chunk0 = (c_in_slice % Geo::kStoreCols) / 8;  // 16-byte chunk inside the 128-byte box row
#pragma unroll
    for (int j = 0; j < kCols / 8; ++j) {
      const uint32_t chunk = static_cast<uint32_t>((chunk0 + j) ^ (f.lane & 7));
      st_shared_v4(row_addr + chunk * 16, packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    }
  } else if (f.row_valid) {
    uint16_t* dst = f.y_row + c_in_slice;
    if (f.vector_ok && c_in_slice + kCols <= f.cols_valid) {
#pragma unroll
      for (int j = 0; j < kCols / 8; ++j) {
        *reinterpret_cast<uint4*>(dst + 8 * j) =
            make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < kCols; ++j) {
        if (c_in_slice + j < f.cols_valid) dst[j] = static_cast<uint16_t>(packed[j / 2] >> (16 * (j & 1)));
      }
    }
  }
}

// Two or more CTAs of small problems share an SM.  How many is bounded on the host: the plan asks for at least
// SplitGeometry::min_smem_bytes_for_tmem(columns) of shared memory, so that the CTAs resident on one SM never
// need more than its 512 tensor-memory columns (a tcgen05.alloc that had to wait for a peer stuck at a cluster
// barrier would never return).  With the 168 registers per thread ptxas reports, 192 threads x 168 registers
// already hold an SM to two CTAs; the shared-memory floor keeps the rule true whatever the compiler does.
template <bool kSplitK, bool kBoxed, bool kPlain>
__global__ void __launch_bounds__(Geo::kThreads, 2)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                   const __grid_constant__ CUtensorMap tm_y, const TcParams p, const SplitPlan plan) {
  constexpr int kMaxStages = SplitGeometry::kMaxStages;
  const int split = kSplitK ? plan.split : 1;
  const int stages = plan.stages;
  const int block_n = plan.block_n;
  const bool overlap = plan.overlap_previous_kernel;
  const int bytes_a = plan.rows_a * Geo::kBlockK;  // multiples of 1024: whole 8-row swizzle atoms
  const int bytes_b = block_n * Geo::kBlockK;
  const uint32_t stage_tx = static_cast<uint32_t>(bytes_a + bytes_b);
  const int n_first = split_first_half(block_n);  // a tile wider than 256 columns: two MMAs and two W boxes per step
  const int n_second = block_n - n_first;
  const uint32_t tmem_cols = static_cast<uint32_t>(split_tmem_cols(block_n));
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw_addr);

  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + stages * bytes_a;  // the MMA's 128-row reads of a short X stage end in here
  const uint32_t smem_epi = base + plan.ring_bytes;
  const uint32_t smem_scales = smem_epi + (plan.staged_stores ? C::kEpiBytes : 0);
  const uint32_t bars = smem_scales + split_scale_bytes(block_n);
  const uint32_t bar_full = bars;                     // [stages]
  const uint32_t bar_empty = bars + 8 * kMaxStages;   // [stages]
  const uint32_t bar_tmem_full = bars + 16 * kMaxStages;
  const uint32_t tmem_slot = bar_tmem_full + 8;
  uint8_t* tail_ptr = base_ptr + (tmem_slot - base);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(tail_ptr);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tail_ptr + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rank = split > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int tile = blockIdx.x / split;
  const int tiles_m = (p.M + Geo::kBlockM - 1) / Geo::kBlockM;
  const int m_tile = tile % tiles_m;
  const int n_tile = tile / tiles_m;
  const int row_base = m_tile * Geo::kBlockM;
  const int col_base = n_tile * block_n;

  const int num_kb = (p.K + Geo::kBlockK - 1) / Geo::kBlockK;
  const int kb_per = (num_kb + split - 1) / split;
  const int kb0 = rank * kb_per < num_kb ? rank * kb_per : num_kb;
  const int kb1 = kb0 + kb_per < num_kb ? kb0 + kb_per : num_kb;
  const bool has_work = kb1 > kb0;
  // Tiles of one row of tiles read the same X boxes.  Each starts its K slice at a different k-block and
  // wraps around, so that at any moment the CTAs ask different L2 lines for X instead of all the same one.
  const int kb_len = kb1 - kb0;
  const int kb_rot = has_work ? (n_tile * 5) % kb_len : 0;
  auto kb_at = [&](int i) {  // the i-th k-block this CTA multiplies
    const int j = i + kb_rot;
    return kb0 + (j >= kb_len ? j - kb_len : j);
  };
  const int slice_cols = block_n / split;  // columns of the tile this CTA finishes: a multiple of 16

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tmem_full, 1);
    *abort_flag = 0u;
    fence_mbar_init();
    prefetch_tensormap(&tm_x);
    prefetch_tensormap(&tm_w);
    if (p.use_tma_store && plan.staged_stores) prefetch_tensormap(&tm_y);
    // the first pass over the ring needs no waiting: start it before the set-up barrier.  W (weights) may
    // be read while the previous kernel still runs; X only after it has completed.
    for (int i = 0; i < kb_len && i < stages; ++i) {
      const uint32_t full = bar_full + 8 * i;
      mbar_arrive_expect_tx(full, stage_tx);
      tma_load_2d(smem_b + i * bytes_b, &tm_w, full, kb_at(i) * Geo::kBlockK, col_base);
      if (n_second > 0) {
        tma_load_2d(smem_b + i * bytes_b + n_first * Geo::kBlockK, &tm_w, full, kb_at(i) * Geo::kBlockK, col_base + n_first);
      }
    }
    if (overlap) griddep_wait();
    for (int i = 0; i < kb_len && i < stages; ++i) {
      tma_load_2d(smem_a + i * bytes_a, &tm_x, bar_full + 8 * i, kb_at(i) * Geo::kBlockK, row_base);
    }
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, tmem_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (overlap) {
    griddep_launch_dependents();
    griddep_wait();  // thread 0 has passed it already: everything below may touch X, the scales and Y
  }

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 1;  // the first `stages` k-blocks were issued before the set-up barrier
      for (int i = stages; i < kb_len; ++i) {
        const int kb = kb_at(i);
        ok = mbar_wait<false>(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty);
        if (!ok) break;
        const uint32_t full = bar_full + 8 * stage;
        mbar_arrive_expect_tx(full, stage_tx);
        tma_load_2d(smem_a + stage * bytes_a, &tm_x, full, kb * Geo::kBlockK, row_base);
        tma_load_2d(smem_b + stage * bytes_b, &tm_w, full, kb * Geo::kBlockK, col_base);
        if (n_second > 0) {
          tma_load_2d(smem_b + stage * bytes_b + n_first * Geo::kBlockK, &tm_w, full, kb * Geo::kBlockK, col_base + n_first);
        }
        if (++stage == static_cast<uint32_t>(stages)) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      const uint32_t idesc = instr_desc_e4m3(Geo::kBlockM, static_cast<uint32_t>(n_first));
      const uint32_t idesc2 = instr_desc_e4m3(Geo::kBlockM, static_cast<uint32_t>(n_second > 0 ? n_second : 16));
      uint32_t stage = 0, phase = 0;
      for (int i = 0; i < kb_len; ++i) {
        ok = mbar_wait<false>(bar_full + 8 * stage, phase, abort_flag, p.status, kSiteMmaFull);
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t a_desc = smem_desc_k_sw128(smem_a + stage * bytes_a);
        const uint64_t b_desc = smem_desc_k_sw128(smem_b + stage * bytes_b);
#pragma unroll
        for (int k = 0; k < Geo::kBlockK / 32; ++k) {
          tc_mma_f8<1>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        if (n_second > 0) {
          const uint64_t b2_desc = smem_desc_k_sw128(smem_b + stage * bytes_b + n_first * Geo::kBlockK);
#pragma unroll
          for (int k = 0; k < Geo::kBlockK / 32; ++k) {
            tc_mma_f8<1>(tmem_base + n_first, a_desc + 2 * k, b2_desc + 2 * k, idesc2, (i > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(bar_empty + 8 * stage);
        if (++stage == static_cast<uint32_t>(stages)) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) tc_commit(bar_tmem_full);
    }
  } else {
    // while the main loop runs: the W scales of this CTA's column slice go to shared memory, zero
    // beyond N, so that the tail of the kernel waits on nothing but the accumulator
    const int first = col_base + rank * slice_cols;
    for (int c = static_cast<int>(threadIdx.x) - 64; c < slice_cols; c += Geo::kThreads - 64) {
      st_shared_f32(smem_scales + c * 4, first + c < p.N ? __ldg(p.w_scale + first + c) : 0.0f);
    }
    if (has_work) {
      // the accumulator is complete (and this CTA's operand ring idle) once the last commit arrives
      ok = mbar_wait<false>(bar_tmem_full, 0u, abort_flag, p.status, kSiteEpiTmemFull);
      tc_fence_after_sync();
    }
    named_barrier_sync(1, Geo::kThreads - 64);  // the four epilogue warps: the scales are in place
  }
  __syncwarp();
  // a CTA that gave up neither sends nor adds (its output is garbage and the status word says so)
  const bool cta_ok = __all_sync(0xffffffffu, *abort_flag == 0u) != 0;

  const int quarter = warp & 3;
  const int tile_row = quarter * 32 + lane;  // row inside the 128-row tile = TMEM lane
  const int row0 = row_base + quarter * 32;
  const int row = row0 + lane;
  const bool warp_has_rows = row0 < p.M;  // warp-uniform: the whole 32-row group lies beyond M otherwise
  const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);

  if constexpr (kSplitK) {
    // ---- (A) every CTA of the cluster has finished reading its operand ring ----
    cluster_sync_all();

    if (warp >= 2 && cta_ok && warp_has_rows) {
      // exchange: columns [j*slice_cols, (j+1)*slice_cols) of this CTA's partial go to CTA j
      auto send = [&](auto cols_tag, int dest, int c_in_slice) {
        constexpr int kCols = decltype(cols_tag)::value;
        uint32_t acc[kCols];
        if (has_work) {
          tmem_ld_cols<kCols>(t_addr + dest * slice_cols + c_in_slice, acc);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < kCols; ++j) acc[j] = 0u;  // K shorter than the split: an empty slice adds nothing
        }
        const uint32_t local = smem_a + exchange_offset(rank, slice_cols, c_in_slice, tile_row, plan.rows_a);
        const uint32_t remote = mapa_cluster(local, static_cast<uint32_t>(dest));
        if (row < p.M) {
#pragma unroll
          for (int j = 0; j < kCols / 4; ++j) {
            st_cluster_v4(remote + j * plan.rows_a * 16, acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          }
        }
      };
#pragma unroll 1
      for (int dest = 0; dest < split; ++dest) {  // 32 columns at a time, a last 16 where the slice ends on them
        int c = 0;
#pragma unroll 1
        for (; c + 32 <= slice_cols; c += 32) send(std::integral_constant<int, 32>{}, dest, c);
        if (c < slice_cols) send(std::integral_constant<int, 16>{}, dest, c);
      }
      tc_fence_before_sync();
    }

    // ---- (B) all partial sums have landed ----
    cluster_sync_all();
  }

  if (warp >= 2 && cta_ok && warp_has_rows) {
    const int col_first = col_base + rank * slice_cols;
    Finish f;
    f.y_row = reinterpret_cast<uint16_t*>(p.y) + static_cast<long long>(row) * p.ldy + col_first;
    f.scales = smem_scales;
    f.exchange_base = smem_a;
    f.t_addr = t_addr + rank * slice_cols;
    f.split = split;
    f.slice_cols = slice_cols;
    f.tile_row = tile_row;
    f.lane = lane;
    f.exchange_rows = plan.rows_a;
    f.cols_valid = p.N - col_first < slice_cols ? p.N - col_first : slice_cols;
    f.xs = row < p.M ? __ldg(p.x_scale + row) : 0.0f;
    f.row_valid = row < p.M;
    f.bias = p.bias != nullptr ? p.bias + col_first : nullptr;
    f.out_fp16 = p.out_fp16 != 0;
    f.boxed = kBoxed;  // the host picks the instantiation: TMA stores allowed, staged stores planned, slices of whole boxes
    f.vector_ok = p.use_tma_store != 0;  // same condition: 16-byte aligned rows of Y
    const uint32_t stage_buf = smem_epi + quarter * (2 * Geo::kStoreRows * Geo::kStoreCols * 2);

    {
      uint32_t store_count = 0;
      int c = 0;
#pragma unroll 1
      for (; c + 64 <= slice_cols; c += 64) {  // 64 columns = one box of the TMA store, when Y leaves in boxes
        const uint32_t sbuf = stage_buf + (store_count & 1u) * (Geo::kStoreRows * Geo::kStoreCols * 2);
        if constexpr (kBoxed) {
          if (lane == 0) tma_store_wait_read<1>();  // the box used two stores ago has been read
          __syncwarp();
        }
        finish_columns<64, kSplitK, kBoxed, kPlain>(f, c, sbuf);
        if constexpr (kBoxed) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && col_first + c < p.N) tma_store_2d(&tm_y, sbuf, col_first + c, row0);
          if (lane == 0) tma_store_commit();
          ++store_count;
        }
      }
      // what is left of a slice that is not a multiple of 64 columns (never boxed)
      if (c + 32 <= slice_cols) {
        finish_columns<32, kSplitK, false, kPlain>(f, c, 0u);
        c += 32;
      }
      if (c < slice_cols) finish_columns<16, kSplitK, false, kPlain>(f, c, 0u);  // never boxed: a boxed slice is a multiple of 64 columns
      // the CTA may end once the boxes have been read out of shared memory; the writes complete with the kernel
      if (kBoxed && lane == 0) tma_store_wait_read<0>();
    }
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc<1>(tmem_base, tmem_cols);
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const TcParams, const SplitPlan);

// [split-K][boxed stores][plain: no bias, bf16]
KernelFn kernel_for(bool split_k, bool boxed, bool plain) {
  static const KernelFn table[2][2][2] = {
      {{gemm_splitk_kernel<false, false, false>, gemm_splitk_kernel<false, false, true>},
       {gemm_splitk_kernel<false, true, false>, gemm_splitk_kernel<false, true, true>}},
      {{gemm_splitk_kernel<true, false, false>, gemm_splitk_kernel<true, false, true>},
       {gemm_splitk_kernel<true, true, false>, gemm_splitk_kernel<true, true, true>}}};
  return table[split_k ? 1 : 0][boxed ? 1 : 0][plain ? 1 : 0];
}

cudaError_t configure(int dev) {
  static bool configured[64] = {};
  static std::mutex mutex;
  std::lock_guard<std::mutex> lock(mutex);
  if (dev >= 0 && dev < 64 && configured[dev]) return cudaSuccess;
  for (int i = 0; i < 8; ++i) {
    const cudaError_t err = cudaFuncSetAttribute(kernel_for((i & 4) != 0, (i & 2) != 0, (i & 1) != 0),
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (err != cudaSuccess) return err;
  }
  if (dev >= 0 && dev < 64) configured[dev] = true;
  return cudaSuccess;
}

}  // namespace

int splitk_resident_clusters(int split, cudaError_t* err) {
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return 0;
  *err = configure(dev);
  if (*err != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(split * 64), 1, 1);
  cfg.blockDim = dim3(Geo::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(split);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  *err = cudaOccupancyMaxActiveClusters(&clusters, kernel_for(split > 1, true, false), &cfg);
  return *err == cudaSuccess ? clusters : 0;
}

cudaError_t launch_gemm_splitk(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_y,
                               const TcParams& p, const SplitPlan& plan, cudaStream_t stream) {
  if (plan.block_n < 16 || plan.block_n > SplitGeometry::kMaxBlockN || plan.split < 1 ||
      plan.block_n % (16 * plan.split) != 0 || (plan.block_n > 256 && (plan.split != 1 || plan.block_n % 64 != 0)) ||
      plan.smem_bytes > C::kSmemBytes ||
      plan.smem_bytes < SplitGeometry::min_smem_bytes_for_tmem(split_tmem_cols(plan.block_n))) {
    return cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  err = configure(dev);
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.tiles * plan.split), 1, 1);
  cfg.blockDim = dim3(Geo::kThreads, 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned num_attrs = 0;
  if (plan.split > 1) {
    attr[num_attrs].id = cudaLaunchAttributeClusterDimension;
    attr[num_attrs].val.clusterDim.x = static_cast<unsigned>(plan.split);
    attr[num_attrs].val.clusterDim.y = 1;
    attr[num_attrs].val.clusterDim.z = 1;
    ++num_attrs;
  }
  if (plan.overlap_previous_kernel) {
    attr[num_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[num_attrs].val.programmaticStreamSerializationAllowed = 1;
    ++num_attrs;
  }
  cfg.attrs = attr;
  cfg.numAttrs = num_attrs;
  const int slice_cols = plan.block_n / plan.split;
  const bool boxed = p.use_tma_store != 0 && plan.staged_stores != 0 && slice_cols % Geo::kStoreCols == 0;
  const bool plain = p.bias == nullptr && p.out_fp16 == 0;
  return cudaLaunchKernelEx(&cfg, kernel_for(plan.split > 1, boxed, plain), tm_x, tm_w, tm_y, p, plan);
}

}  // namespace b200fp8
