"""The static work split of the skinny fp32 kernels (veritac_b200/csrc/skinny_sched.cuh), checked on the
host: the header is compiled into a small program that prints every CTA's pieces, and the pieces must tile
(slab, chunk) space exactly once with consistent part numbers, for grids of one and of three CTAs per SM."""
import shutil
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PROGRAM = r'''
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "skinny_sched.cuh"
int main(int argc, char** argv) {
  const long long N = atoll(argv[1]), K = atoll(argv[2]);
  const int sms = atoi(argv[3]), per_sm = atoi(argv[4]), overhead = atoi(argv[5]);
  int ctas = 0;
  const vt::SkinnySched sc = vt::make_skinny_sched(N, K, sms, per_sm, overhead, &ctas);
  printf("S %d %d %d %d\n", sc.slabs, sc.chunks, ctas, vt::skinny_max_parts(sc));
  for (int c = 0; c < ctas; ++c) {
    vt::SkinnySegment seg;
    for (int i = 0; vt::sched_segment(sc, c, i, seg); ++i)
      printf("P %d %d %d %d %d %d\n", c, seg.slab, seg.chunk_beg, seg.chunk_end, seg.part, seg.parts);
  }
  return 0;
}
'''


@pytest.fixture(scope="module")
def sched_program(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).is_file():
        pytest.skip("nvcc not available")
    d = tmp_path_factory.mktemp("sched")
    src = d / "sched.cu"
    src.write_text(PROGRAM)
    exe = d / "sched"
    r = subprocess.run([nvcc, "-O1", "-std=c++17", "-I", str(REPO / "veritac_b200" / "csrc"), "-o", str(exe), str(src)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


SHAPES = [(8192, 8192), (16384, 4096), (4096, 16384), (32768, 8192), (2048, 2048), (1024, 8192), (60000, 512),
          (516, 100), (128, 32), (132, 31), (4, 7), (260, 8), (56832, 4096), (70000, 64), (18944, 4096), (18948, 4096)]


@pytest.mark.parametrize("per_sm,overhead", [(1, 10), (3, 3), (3, 0)])
def test_pieces_tile_the_matrix_once(sched_program, per_sm, overhead):
    for (n, k) in SHAPES:
        out = subprocess.run([str(sched_program), str(n), str(k), "148", str(per_sm), str(overhead)],
                             capture_output=True, text=True, check=True).stdout.split("\n")
        head = out[0].split()
        slabs, chunks, ctas, max_parts = (int(x) for x in head[1:])
        assert slabs == -(-n // 128) and chunks == -(-k // 32)
        assert 1 <= ctas <= max(148 * per_sm, slabs)
        cover, parts_seen, parts_of, work = set(), set(), {}, {}
        for line in out[1:]:
            if not line:
                continue
            _, c, slab, beg, end, part, parts = line.split()
            c, slab, beg, end, part, parts = int(c), int(slab), int(beg), int(end), int(part), int(parts)
            assert 0 <= slab < slabs and 0 <= beg < end <= chunks, (n, k, line)
            assert 0 <= part < parts <= max_parts
            assert parts_of.setdefault(slab, parts) == parts          # every piece of a slab agrees on the count
            assert (slab, part) not in parts_seen
            parts_seen.add((slab, part))
            for ch in range(beg, end):
                assert (slab, ch) not in cover
                cover.add((slab, ch))
            work[c] = work.get(c, 0) + end - beg
        assert len(cover) == slabs * chunks, (n, k)
        for slab, parts in parts_of.items():
            assert sum(1 for (s, _) in parts_seen if s == slab) == parts   # the ticket count is reached exactly
        if ctas == 148 * per_sm and chunks * slabs >= 16 * ctas:
            assert max(work.values()) <= 1.5 * (slabs * chunks / ctas) + 2   # no CTA far above its share
