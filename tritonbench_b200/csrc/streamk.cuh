// Work decomposition shared by the stream-K kernels: a CTA's work is a run of consecutive
// (tile, k-block) units of the K-split region, cut at tile boundaries into segments, followed by
// the whole tiles dealt to it.  Device-only, header-only.
#pragma once

#include <stdint.h>

namespace b200fp8 {

struct Segment {
  int tile;
  int slot;  // partial-sum slot (global index)
  int kb0;
  int kb1;
};

// One CTA's run of consecutive units [u_begin, u_stop) cut at tile boundaries.  Segments that
// cover only part of a tile's K range are processed FIRST (the one at the end of the run, then
// the one at its start), the whole tiles after them: the cross-CTA fix-up of a split tile then
// happens early, hidden behind the streaming of the remaining tiles.
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

// i-th segment of the run in processing order; `slot_base` is this CTA's first partial-sum slot
__device__ __forceinline__ Segment run_segment(const Run& r, int i, int slot_base) {
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
  s.slot = slot_base + j;
  s.tile = r.first_tile + j;
  const long long tile_u0 = static_cast<long long>(s.tile) * r.kblocks;
  s.kb0 = r.u_begin > tile_u0 ? static_cast<int>(r.u_begin - tile_u0) : 0;
  s.kb1 = r.u_stop < tile_u0 + r.kblocks ? static_cast<int>(r.u_stop - tile_u0) : r.kblocks;
  return s;
}

// The whole plan of one CTA: the segments of its run of the K-split region (in the order above),
// then its whole tiles  sk_tiles + cta, sk_tiles + cta + num_ctas, ...  Whole tiles carry slot -1.
struct CtaWork {
  Run run;
  int slot_base;
  int first_whole;
  int whole_stride;
  int count;
  int kblocks;
};

__device__ __forceinline__ CtaWork make_cta_work(int cta, int num_ctas, int tiles, int sk_tiles, int kblocks,
                                                 int units_per_cta, int segs_per_cta) {
  CtaWork w;
  const long long sk_units = static_cast<long long>(sk_tiles) * kblocks;
  long long u_begin = static_cast<long long>(cta) * units_per_cta;
  if (u_begin > sk_units) u_begin = sk_units;
  const long long u_stop = u_begin + units_per_cta < sk_units ? u_begin + units_per_cta : sk_units;
  w.run = make_run(u_begin, u_stop, kblocks);
  w.slot_base = cta * segs_per_cta;
  w.first_whole = sk_tiles + cta;
  w.whole_stride = num_ctas;
  const int whole = w.first_whole < tiles ? (tiles - w.first_whole + num_ctas - 1) / num_ctas : 0;
  w.count = w.run.count + whole;
  w.kblocks = kblocks;
  return w;
}

__device__ __forceinline__ Segment work_segment(const CtaWork& w, int i) {
  if (i < w.run.count) return run_segment(w.run, i, w.slot_base);
  Segment s;
  s.tile = w.first_whole + (i - w.run.count) * w.whole_stride;
  s.slot = -1;
  s.kb0 = 0;
  s.kb1 = w.kblocks;
  return s;
}

// CTAs whose runs touch K-split tile `tile`: [first, last]
__device__ __forceinline__ void tile_parts(int tile, int kblocks, int units_per_cta, int* first, int* last) {
  const long long tile_u0 = static_cast<long long>(tile) * kblocks;
  *first = static_cast<int>(tile_u0 / units_per_cta);
  *last = static_cast<int>((tile_u0 + kblocks - 1) / units_per_cta);
}

// partial-sum slot that CTA `part` uses for K-split tile `tile`
__device__ __forceinline__ size_t part_slot(int part, int tile, int kblocks, int units_per_cta, int segs_per_cta) {
  const long long their_first = static_cast<long long>(part) * units_per_cta / kblocks;
  return static_cast<size_t>(part) * segs_per_cta + static_cast<size_t>(tile - their_first);
}

}  // namespace b200fp8
