// Static work list of the int8 CTA-pair kernel.  T output tiles (256 x 256) of KB K-blocks (128 values
// of K) each are dealt to P persistent CTA pairs.  The first floor(T / P) * P tiles go round-robin, a
// whole tile at a time.  The T mod P tiles left over (the "tail") would keep only some of the pairs
// busy for one more whole tile; instead their K-blocks, taken as one run of (T mod P) * KB units, are
// cut into P nearly equal ranges, one per pair.  A range that ends inside a tile leaves a *partial*
// accumulator (int32 sums over the K-blocks it covered) in scratch memory; the pair whose range holds a
// tile's last K-block *owns* the tile, adds the partial accumulators of the pairs before it and writes
// C.  int32 addition is associative, so the result does not depend on the cut.
//
// A pair's partial piece (at most one: the end of its range) is always its first item; partial pieces wait
// for nothing, so every owner's wait for its contributors ends.  The rest of the order keeps the adding of
// partial sums off the critical path:
//   * a pair with a partial piece and whole tiles runs  partial, whole tiles, owned tail tiles.  Its owned
//     tile that has contributors is *preloaded*: while the whole tile before it is being multiplied, the
//     epilogue warps add the contributors' sums and write them into the (idle) accumulator, and the MMAs of
//     the owned piece then accumulate on top;
//   * a pair without a partial piece runs  owned tail tiles, whole tiles,  and a pair without whole tiles
//     partial, owned tail tiles: there the contributors' sums are added in the epilogue of the owned tile
//     (overlapping the whole tile after it, where there is one).
//
// A second way to share the tail ("equal split") keeps the pairs walking K in step, which the L2 rewards:
// when the tail has at most half as many tiles as there are pairs, every tail tile is cut into
// s = floor(P / tail) equal K pieces (at most 4), piece k of tile j goes to pair j * s + k, and every pair runs
// its piece *last*, after its whole tiles, so that all pieces start together.  The pair with the last piece owns
// the tile and adds the others' sums in its epilogue; their partial sums are the last thing those pairs do, and
// nobody waits for anything else, so the owners' waits end.  The merge is then exposed at the end of the launch
// (a few microseconds) in exchange for (1 - 1/s) of a tile's time.
#pragma once

#include <stdint.h>

namespace vt {

constexpr int PAIR_MIN_PIECE = 4;   // cuts closer than this to a tile boundary snap to it (K-blocks)

struct PairSched {
  int pairs;        // P
  int tiles;        // T
  int kblocks;      // KB
  int whole_waves;  // whole tiles per pair
  int tail;         // tiles whose K-blocks are shared (0: every tile is computed whole by one pair)
  int split;        // 0: the tail's K-blocks are cut into one range per pair; s >= 2: every tail tile into s equal pieces
};

enum : int { PAIR_SHARE_NONE = 0, PAIR_SHARE_RANGES = 1, PAIR_SHARE_EQUAL_SPLIT = 2 };

enum : int { PAIR_ITEM_TO_C = 0, PAIR_ITEM_PARTIAL = 1 };

struct PairItem {
  int tile;            // output tile index (raster order)
  int kb0, kb1;        // K-blocks [kb0, kb1)
  int kind;            // PAIR_ITEM_TO_C: finish the tile and write C; PAIR_ITEM_PARTIAL: leave sums in this pair's slot
  int contrib0;        // PAIR_ITEM_TO_C: pairs [contrib0, contrib0 + ncontrib) left partial sums of this tile
  int ncontrib;
  int preload;         // the contributors' sums go into the accumulator before the MMAs (else: added in the epilogue)
};

// Whether sharing the tail pays: the idle part of the last wave must be worth more than the extra
// epilogues and the merge (about ten K-blocks' time per pair), and ranges must not be slivers.
__host__ __device__ inline PairSched make_pair_sched(int pairs, int tiles, int kblocks, int share) {
  PairSched s;
  s.pairs = pairs;
  s.tiles = tiles;
  s.kblocks = kblocks;
  s.whole_waves = tiles / pairs;
  s.tail = 0;
  s.split = 0;
  const int tail = tiles - s.whole_waves * pairs;
  if (share == PAIR_SHARE_EQUAL_SPLIT && tail > 0) {
    int pieces = pairs / tail;
    if (pieces > 4) pieces = 4;                       // more contributors cost the owner more than they save
    while (pieces >= 2 && kblocks / pieces < 8) --pieces;   // no slivers
    if (pieces >= 2) {
      s.tail = tail;
      s.split = pieces;
    }
  }
  if (share == PAIR_SHARE_RANGES && tail > 0) {
    const long long units = (long long)tail * kblocks;
    const long long per = units / pairs;
    const long long idle = (long long)(pairs - tail) * kblocks;   // pair-K-blocks the whole-tile order leaves unused
    // units * pairs < 2^31 keeps the device-side arithmetic in 32 bits
    if (per >= 16 && per * 8 >= kblocks && idle >= 12LL * pairs && units * pairs < 0x7fffffffLL) s.tail = tail;
  }
  if (s.tail == 0) s.whole_waves = (tiles + pairs - 1) / pairs;   // upper bound; items past `tiles` do not exist
  return s;
}

// First unit of pair p's range (units: tail tile j, K-block kb -> j * KB + kb).
__host__ __device__ inline int pair_range_begin(const PairSched& s, int p) {
  const int units = s.tail * s.kblocks;
  if (p <= 0) return 0;
  if (p >= s.pairs) return units;
  int b = int(unsigned(p * units) / unsigned(s.pairs));
  const int r = b % s.kblocks;
  if (r < PAIR_MIN_PIECE) b -= r;
  else if (s.kblocks - r < PAIR_MIN_PIECE) b += s.kblocks - r;
  return b;
}

// Range begins as a function object, so that the kernel can read them from a table its warps fill in parallel
// while the host-side check computes them directly.
struct PairRangeDirect {
  const PairSched& s;
  __host__ __device__ int operator()(int p) const { return pair_range_begin(s, p); }
};

// Number of items of pair `pair` that lie in the shared tail (they come first): at most one partial piece and
// the tail tiles whose last K-block is in the pair's range.
template <class RangeBegin>
__host__ __device__ inline int pair_tail_items(const PairSched& s, int pair, const RangeBegin& begin) {
  if (s.tail == 0) return 0;
  if (s.split) return pair < s.tail * s.split ? 1 : 0;
  const int u0 = begin(pair), u1 = begin(pair + 1);
  if (u1 <= u0) return 0;
  const int j_end = u1 / s.kblocks;
  return (u1 - j_end * s.kblocks != 0 ? 1 : 0) + j_end - u0 / s.kblocks;
}
__host__ __device__ inline int pair_tail_items(const PairSched& s, int pair) {
  return pair_tail_items(s, pair, PairRangeDirect{s});
}

// The t-th item of pair `pair` inside the shared tail, in range order: the partial piece (if any), then the
// owned tiles; t < pair_tail_items().
template <class RangeBegin>
__host__ __device__ inline void pair_tail_item(const PairSched& s, int pair, int t, PairItem& out, const RangeBegin& begin) {
  const int KB = s.kblocks;
  const int first_tail_tile = s.whole_waves * s.pairs;
  out.contrib0 = 0;
  out.ncontrib = 0;
  out.preload = 0;
  if (s.split) {
    const int j = pair / s.split, part = pair - j * s.split;
    out.tile = first_tail_tile + j;
    out.kb0 = part * KB / s.split;
    out.kb1 = (part + 1) * KB / s.split;
    if (part + 1 < s.split) {
      out.kind = PAIR_ITEM_PARTIAL;
    } else {
      out.kind = PAIR_ITEM_TO_C;
      out.contrib0 = j * s.split;
      out.ncontrib = s.split - 1;
    }
    return;
  }
  const int u0 = begin(pair), u1 = begin(pair + 1);
  const int j_first = u0 / KB, j_end = u1 / KB;                // tail tiles [j_first, j_end) end inside the range
  const bool has_partial = u1 > u0 && u1 != j_end * KB;
  if (has_partial) {
    if (t == 0) {
      const int base = j_end * KB;
      out.tile = first_tail_tile + j_end;
      out.kb0 = (u0 > base ? u0 : base) - base;
      out.kb1 = u1 - base;
      out.kind = PAIR_ITEM_PARTIAL;
      return;
    }
    --t;
  }
  const int j = j_first + t;
  const int base = j * KB;
  out.tile = first_tail_tile + j;
  out.kb0 = (u0 > base ? u0 : base) - base;
  out.kb1 = KB;
  out.kind = PAIR_ITEM_TO_C;
  if (out.kb0 > 0) {
    // The pairs before this one whose ranges reach into tile j, nearest first.
    int n = 0;
    for (int q = pair - 1; q >= 0 && begin(q + 1) > base; --q) {
      ++n;
      if (begin(q) <= base) break;
    }
    out.ncontrib = n;
    out.contrib0 = pair - n;
    out.preload = (has_partial && s.whole_waves > 0) ? 1 : 0;
  }
}

// Position of the whole tiles in a pair's order.  Ranges: after the partial piece when the pair has one, else
// after its tail items.  Equal split: first.
__host__ __device__ inline int pair_whole_first(const PairSched& s, int tail_items, bool first_is_partial) {
  if (s.split) return 0;
  return first_is_partial ? 1 : tail_items;
}

// The idx-th item of pair `pair` in execution order; false when it has no more.
template <class RangeBegin>
__host__ __device__ inline bool pair_item(const PairSched& s, int pair, int idx, PairItem& out, const RangeBegin& begin) {
  out.contrib0 = 0;
  out.ncontrib = 0;
  out.preload = 0;
  out.kb0 = 0;
  out.kb1 = s.kblocks;
  out.kind = PAIR_ITEM_TO_C;
  if (s.tail == 0) {
    const long long t = (long long)pair + (long long)idx * s.pairs;
    if (t >= s.tiles) return false;
    out.tile = int(t);
    return true;
  }
  const int n_tail = pair_tail_items(s, pair, begin);
  bool first_is_partial = false;
  if (n_tail > 0) {
    PairItem first;
    pair_tail_item(s, pair, 0, first, begin);
    first_is_partial = first.kind == PAIR_ITEM_PARTIAL;
  }
  const int w0 = pair_whole_first(s, n_tail, first_is_partial);
  if (idx >= w0 && idx < w0 + s.whole_waves) {
    out.tile = pair + (idx - w0) * s.pairs;
    return true;
  }
  const int t = idx < w0 ? idx : idx - s.whole_waves;
  if (t >= n_tail) return false;
  pair_tail_item(s, pair, t, out, begin);
  return true;
}
__host__ __device__ inline bool pair_item(const PairSched& s, int pair, int idx, PairItem& out) {
  return pair_item(s, pair, idx, out, PairRangeDirect{s});
}

}  // namespace vt
