// Static work list of the int8 CTA-pair kernel.  T output tiles (256 x 256) of KB K-blocks (128 values
// of K) each are dealt to P persistent CTA pairs.  The first floor(T / P) * P tiles go round-robin, a
// whole tile at a time.  The T mod P tiles left over (the "tail") would keep only some of the pairs
// busy for one more whole tile; instead their K-blocks, taken as one run of (T mod P) * KB units, are
// cut into P nearly equal ranges, one per pair.  A range that ends inside a tile leaves a *partial*
// accumulator (int32 sums over the K-blocks it covered) in scratch memory; the pair whose range holds a
// tile's last K-block *owns* the tile, adds the partial accumulators of the pairs before it and writes
// C.  int32 addition is associative, so the result does not depend on the cut.
//
// A pair runs its items in this order: its partial piece (at most one: the end of its range), the tail
// tiles it owns, then its whole tiles.  Partial pieces wait for nothing, so every owner's wait for its
// contributors ends; the owner's merge overlaps the MMAs of the whole tile after it.
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
};

enum : int { PAIR_ITEM_TO_C = 0, PAIR_ITEM_PARTIAL = 1 };

struct PairItem {
  int tile;            // output tile index (raster order)
  int kb0, kb1;        // K-blocks [kb0, kb1)
  int kind;            // PAIR_ITEM_TO_C: finish the tile and write C; PAIR_ITEM_PARTIAL: leave sums in this pair's slot
  int contrib0;        // PAIR_ITEM_TO_C: pairs [contrib0, contrib0 + ncontrib) left partial sums of this tile
  int ncontrib;
};

// Whether sharing the tail pays: the idle part of the last wave must be worth more than the extra
// epilogues and the merge (about ten K-blocks' time per pair), and ranges must not be slivers.
__host__ __device__ inline PairSched make_pair_sched(int pairs, int tiles, int kblocks, bool share_tail) {
  PairSched s;
  s.pairs = pairs;
  s.tiles = tiles;
  s.kblocks = kblocks;
  s.whole_waves = tiles / pairs;
  s.tail = 0;
  const int tail = tiles - s.whole_waves * pairs;
  if (share_tail && tail > 0) {
    const long long units = (long long)tail * kblocks;
    const long long per = units / pairs;
    const long long idle = (long long)(pairs - tail) * kblocks;   // pair-K-blocks the whole-tile order leaves unused
    if (per >= 16 && per * 8 >= kblocks && idle >= 12LL * pairs) s.tail = tail;
  }
  if (s.tail == 0) s.whole_waves = (tiles + pairs - 1) / pairs;   // upper bound; items past `tiles` do not exist
  return s;
}

// First unit of pair p's range (units: tail tile j, K-block kb -> j * KB + kb).
__host__ __device__ inline long long pair_range_begin(const PairSched& s, int p) {
  const long long units = (long long)s.tail * s.kblocks;
  if (p <= 0) return 0;
  if (p >= s.pairs) return units;
  long long b = (long long)p * units / s.pairs;
  const int r = int(b % s.kblocks);
  if (r < PAIR_MIN_PIECE) b -= r;
  else if (s.kblocks - r < PAIR_MIN_PIECE) b += s.kblocks - r;
  return b;
}

// The idx-th item of pair `pair`; false when it has no more.
__host__ __device__ inline bool pair_item(const PairSched& s, int pair, int idx, PairItem& out) {
  out.contrib0 = 0;
  out.ncontrib = 0;
  if (s.tail == 0) {
    const long long t = (long long)pair + (long long)idx * s.pairs;
    if (t >= s.tiles) return false;
    out.tile = int(t);
    out.kb0 = 0;
    out.kb1 = s.kblocks;
    out.kind = PAIR_ITEM_TO_C;
    return true;
  }
  const int KB = s.kblocks;
  const int first_tail_tile = s.whole_waves * s.pairs;
  const long long u0 = pair_range_begin(s, pair), u1 = pair_range_begin(s, pair + 1);
  const int j_first = int(u0 / KB), j_end = int(u1 / KB);      // tail tiles [j_first, j_end) end inside the range
  const bool has_partial = u1 > u0 && (u1 % KB) != 0;
  const int owned = u1 > u0 ? j_end - j_first : 0;
  if (has_partial) {
    if (idx == 0) {
      const long long base = (long long)j_end * KB;
      out.tile = first_tail_tile + j_end;
      out.kb0 = int((u0 > base ? u0 : base) - base);
      out.kb1 = int(u1 - base);
      out.kind = PAIR_ITEM_PARTIAL;
      return true;
    }
    --idx;
  }
  if (idx < owned) {
    const int j = j_first + idx;
    const long long base = (long long)j * KB;
    out.tile = first_tail_tile + j;
    out.kb0 = int((u0 > base ? u0 : base) - base);
    out.kb1 = KB;
    out.kind = PAIR_ITEM_TO_C;
    if (out.kb0 > 0) {
      // The pairs before this one whose ranges reach into tile j, nearest first.
      int n = 0;
      for (int q = pair - 1; q >= 0 && pair_range_begin(s, q + 1) > base; --q) {
        ++n;
        if (pair_range_begin(s, q) <= base) break;
      }
      out.ncontrib = n;
      out.contrib0 = pair - n;
    }
    return true;
  }
  idx -= owned;
  if (idx >= s.whole_waves) return false;
  out.tile = pair + idx * s.pairs;
  out.kb0 = 0;
  out.kb1 = KB;
  out.kind = PAIR_ITEM_TO_C;
  return true;
}

}  // namespace vt
