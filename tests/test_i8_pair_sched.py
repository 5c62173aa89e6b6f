"""The static work list of the int8 CTA-pair kernel (veritac_b200/csrc/i8_pair_sched.cuh), checked on the host.

The header is compiled into a small program that prints every pair's items.  Every (tile, K-block) must be
computed exactly once; every tile must be finished (written to C) by exactly one pair, which must name as
contributors exactly the pairs that left a partial sum of that tile; a pair leaves at most one partial sum
(it has one scratch slot), and leaves it before anything it could have to wait for; an owned tile whose
contributors' sums are written into the accumulator ahead of its MMAs comes right after a whole tile."""
import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PROGRAM = r'''
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "i8_pair_sched.cuh"
int main(int argc, char** argv) {
  const int pairs = atoi(argv[1]), tiles = atoi(argv[2]), kb = atoi(argv[3]), share = atoi(argv[4]);
  vt::PairSched s = vt::make_pair_sched(pairs, tiles, kb, share);
  if (s.tail == 0) s = vt::make_pair_sched(tiles < pairs ? tiles : pairs, tiles, kb, vt::PAIR_SHARE_NONE);
  printf("S %d %d %d %d\n", s.pairs, s.whole_waves, s.tail, s.split);
  for (int p = 0; p < s.pairs; ++p) {
    vt::PairItem it;
    for (int i = 0; vt::pair_item(s, p, i, it); ++i)
      printf("I %d %d %d %d %d %d %d %d %d\n", p, i, it.tile, it.kb0, it.kb1, it.kind, it.contrib0, it.ncontrib, it.preload);
  }
  return 0;
}
'''


@pytest.fixture(scope="module")
def sched_program(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).is_file():
        pytest.skip("nvcc not available")
    d = tmp_path_factory.mktemp("pairsched")
    src = d / "sched.cu"
    src.write_text(PROGRAM)
    exe = d / "sched"
    r = subprocess.run([nvcc, "-O1", "-std=c++17", "-I", str(REPO / "veritac_b200" / "csrc"), "-o", str(exe), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def run(exe, pairs, tiles, kb, share=1):
    out = subprocess.run([str(exe), str(pairs), str(tiles), str(kb), str(share)], capture_output=True, text=True,
                         check=True).stdout.splitlines()
    head = [int(x) for x in out[0].split()[1:]]
    items = [[int(x) for x in line.split()[1:]] for line in out[1:]]
    return head, items


def check(head, items, tiles, kb):
    grid_pairs, whole_waves, tail, split = head
    last_index = {}
    for p, i, *_rest in items:
        last_index[p] = max(last_index.get(p, 0), i)
    covered = {}
    finished = {}
    partial_of = {}
    for p, i, tile, kb0, kb1, kind, c0, nc, pre in items:
        assert 0 <= tile < tiles and 0 <= kb0 < kb1 <= kb
        if pre:
            # sums written into an accumulator ahead of the MMAs: the accumulator must have been used and drained
            # before (two items earlier), and the item right before must be a whole tile that hides the work
            assert kind == 0 and nc > 0 and i >= 2
            before = [x for x in items if x[0] == p and x[1] == i - 1][0]
            assert before[3] == 0 and before[4] == kb and before[5] == 0
        for k in range(kb0, kb1):
            assert (tile, k) not in covered, "K block computed twice"
            covered[(tile, k)] = p
        if kind == 1:
            if split:     # equal split: every piece is its pair's last item, so all pieces start together
                assert i == last_index[p] and kb1 - kb0 in (kb // split, kb // split + 1)
            else:
                assert i == 0, "a partial sum must be the pair's first item"
            assert p not in partial_of, "one scratch slot per pair"
            assert kb1 < kb, "the piece that holds a tile's last K block finishes the tile"
            partial_of[p] = tile
        else:
            assert kb1 == kb
            assert tile not in finished
            finished[tile] = (p, kb0, c0, nc)
    assert len(covered) == tiles * kb
    assert sorted(finished) == list(range(tiles))
    for tile, (p, kb0, c0, nc) in finished.items():
        if split and nc:
            assert nc == split - 1 and [x for x in items if x[0] == p][-1][2] == tile   # the owner's piece is its last item
        contributors = sorted(q for q, t in partial_of.items() if t == tile)
        assert contributors == list(range(c0, c0 + nc)) if nc else contributors == []
        assert (kb0 > 0) == (nc > 0)
        assert all(q < p for q in contributors)
    # per-pair K blocks: nobody does more than a whole-tile schedule would give the busiest pair
    work = {}
    for p, i, tile, kb0, kb1, kind, c0, nc, pre in items:
        work[p] = work.get(p, 0) + kb1 - kb0
    return max(work.values()), tail


CASES = [(74, 128, 64), (74, 256, 64), (74, 1024, 64), (74, 54, 64), (74, 1, 64), (74, 74, 64), (74, 75, 64),
         (74, 147, 64), (74, 148, 64), (74, 100, 8), (74, 100, 1024), (74, 37, 512), (74, 20, 256), (74, 73, 33),
         (66, 128, 64), (3, 7, 5), (74, 111, 17), (74, 4096, 32), (74, 129, 2)]


@pytest.mark.parametrize("share", [1, 2, 0])
def test_every_k_block_once_and_every_tile_finished_once(sched_program, share):
    for pairs, tiles, kb in CASES + [(74, 256, 64), (74, 90, 64), (74, 108, 96), (74, 37 + 74, 33), (74, 10, 256)]:
        head, items = run(sched_program, pairs, tiles, kb, share)
        busiest, tail = check(head, items, tiles, kb)
        whole = -(-tiles // pairs) * kb
        assert busiest <= whole
        if not share:
            assert tail == 0 and busiest == whole


def test_equal_split_of_a_short_tail(sched_program):
    """2048 rows of an 8192-wide C: 256 tiles on 74 pairs, 34 left over: each is cut in two halves that 68 pairs
    compute last, so the busiest pair does three and a half tiles instead of four.  A tail of more than half the
    pairs is not split."""
    head, items = run(sched_program, 74, 256, 64, 2)
    busiest, tail = check(head, items, 256, 64)
    assert head[3] == 2 and tail == 34 and busiest == 3 * 64 + 32
    head, items = run(sched_program, 74, 128, 64, 2)
    assert head[2] == 0 and head[3] == 0
    head, items = run(sched_program, 74, 74 + 10, 64, 2)
    assert head[3] == 4 and check(head, items, 84, 64)[0] == 64 + 16


def test_shared_tail_balances_the_strong_scaling_shards(sched_program):
    """1024 and 2048 rows of an 8192-wide C: 128 and 256 tiles on 74 pairs; the busiest pair gets within a
    few K blocks of the mean instead of a whole extra tile."""
    for tiles in (128, 256):
        head, items = run(sched_program, 74, tiles, 64, 1)
        busiest, tail = check(head, items, tiles, 64)
        assert tail == tiles % 74
        assert busiest <= tiles * 64 / 74 + 6
