// Work split shared by the skinny fp32 kernels (M <= 16): B is cut into 128-column slabs and 32-row
// chunks.  With G CTAs and S slabs, floor(G/S) "regular" CTAs per slab split the upper rows of the
// slab evenly (CTA c -> slab c mod S, so neighbours read neighbouring 512-byte segments of the same
// rows); the G mod S CTAs left over share the bottom rows of all slabs in equal pieces, a piece
// running on from one slab into the next.  The row where the bottom part starts is chosen so that
// every CTA gets the same number of chunks.  Every piece of a slab leaves a partial tile in scratch
// memory; the CTA that finishes a slab's last piece (a ticket per slab) sums the pieces in a
// fixed order, so results do not depend on which CTA that is.
#pragma once

#include <stdint.h>

namespace vt {

constexpr int SKINNY_COLS = 128;   // columns per slab
constexpr int SKINNY_KC = 32;      // rows of B per chunk

// All quantities in chunks / slabs / CTAs.
struct SkinnySched {
  int slabs;      // S
  int chunks;     // chunks per slab (C)
  int regular;    // regular CTAs per slab (p); 0 when there are more slabs than CTAs
  int extras;     // CTAs left over (R = G - S * p)
  int bottom;     // chunks per slab left to the extras (L); the regular CTAs share [0, C - L)
};
struct SkinnySegment {
  int slab, chunk_beg, chunk_end, part, parts;
};

// Extra CTA that owns bottom unit `u` (units: slab-major, `bottom` per slab), and the first unit of extra e.
__host__ __device__ inline int sched_extra_of(const SkinnySched& sc, long long u) {
  return int(((u + 1) * sc.extras - 1) / ((long long)sc.slabs * sc.bottom));
}
__host__ __device__ inline long long sched_extra_begin(const SkinnySched& sc, int e) {
  return (long long)e * sc.slabs * sc.bottom / sc.extras;
}
__host__ __device__ inline int sched_parts(const SkinnySched& sc, int slab) {
  if (sc.extras == 0 || sc.bottom == 0) return sc.regular;
  const int first = sched_extra_of(sc, (long long)slab * sc.bottom);
  const int last = sched_extra_of(sc, (long long)(slab + 1) * sc.bottom - 1);
  return sc.regular + last - first + 1;
}
// The idx-th piece of work of CTA `cta`; false when it has no more.
__host__ __device__ inline bool sched_segment(const SkinnySched& sc, int cta, int idx, SkinnySegment& out) {
  const int n_regular = sc.slabs * sc.regular;
  if (cta < n_regular) {
    if (idx > 0) return false;
    const int upper = sc.chunks - sc.bottom;
    const int i = cta / sc.slabs;
    out.slab = cta % sc.slabs;
    out.chunk_beg = int((long long)upper * i / sc.regular);
    out.chunk_end = int((long long)upper * (i + 1) / sc.regular);
    out.part = i;
    out.parts = sched_parts(sc, out.slab);
    return true;
  }
  if (sc.bottom == 0) return false;
  const int e = cta - n_regular;
  const long long u0 = sched_extra_begin(sc, e), u1 = sched_extra_begin(sc, e + 1);
  long long u = u0;
  for (int k = 0; u < u1; ++k) {
    const int slab = int(u / sc.bottom);
    const long long slab_end = (long long)(slab + 1) * sc.bottom;
    const long long stop = u1 < slab_end ? u1 : slab_end;
    if (k == idx) {
      const int upper = sc.chunks - sc.bottom;
      out.slab = slab;
      out.chunk_beg = upper + int(u - (long long)slab * sc.bottom);
      out.chunk_end = upper + int(stop - (long long)slab * sc.bottom);
      out.part = sc.regular + e - sched_extra_of(sc, (long long)slab * sc.bottom);
      out.parts = sched_parts(sc, slab);
      return true;
    }
    u = stop;
  }
  return false;
}

// piece_overhead: what ending one piece and starting the next costs a CTA, in chunks; a left-over CTA
// works through about S / R + 1 pieces, a regular one through one, so it is given that much less.
inline SkinnySched make_skinny_sched(int64_t N, int64_t K, int sm_count, int ctas_per_sm, int piece_overhead,
                                     int* ctas) {
  SkinnySched sc;
  const int64_t S = (N + SKINNY_COLS - 1) / SKINNY_COLS;
  const int64_t Cn = (K + SKINNY_KC - 1) / SKINNY_KC;
  int64_t G = int64_t(sm_count) * ctas_per_sm;
  // At least four chunks per CTA, or the ramp of the ring is all a CTA ever does.
  const int64_t most = S * (Cn / 4 > 0 ? Cn / 4 : 1);
  if (G > most) G = most;
  sc.slabs = int(S);
  sc.chunks = int(Cn);
  if (S == G) {
    sc.regular = 1;
    sc.extras = 0;
    sc.bottom = 0;
  } else if (S > G) {
    // More slabs than CTAs: no regular CTAs at all; every CTA takes an equal run of chunks in
    // slab-major order (a slab and a part of the next, or several slabs), so there is no second wave.
    sc.regular = 0;
    sc.extras = int(G);
    sc.bottom = int(Cn);
  } else {
    sc.regular = int(G / S);
    sc.extras = int(G - S * sc.regular);
    // Equal time: (C - L) / p == S * L / R + overhead * S / R  =>  L = (C * R - overhead * S * p) / G.
    const int64_t num = Cn * sc.extras - int64_t(piece_overhead) * S * sc.regular;
    sc.bottom = (sc.extras && num > 0) ? int((num + G / 2) / G) : 0;
    if (sc.extras && sc.bottom == 0) {   // too little left over to be worth a CTA
      G = S * sc.regular;
      sc.extras = 0;
    }
  }
  *ctas = int(G);
  return sc;
}


inline int skinny_max_parts(const SkinnySched& sc) {
  int most = 1;
  for (int s = 0; s < sc.slabs; ++s) {
    const int p = sched_parts(sc, s);
    if (p > most) most = p;
  }
  return most;
}

#ifdef __CUDACC__
// Called by the kThreads threads (tid 0..kThreads-1, named barrier `bar_id`) that have just stored
// a piece's partial tile: takes a ticket for the slab and, in the CTA that holds the last one, sums
// the slab's partial tiles in piece order into C and returns the ticket counter to zero.  The
// loads of several pieces are in flight together; the additions keep piece order.
template <int kThreads, int kRows = 16>
__device__ __forceinline__ void skinny_finish_piece(const SkinnySegment& seg, int tid, int bar_id, int* last_flag,
                                                    int* __restrict__ tickets, const float* __restrict__ partials,
                                                    float* __restrict__ C, int M, int N) {
  __threadfence();
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");
  if (tid == 0) {
    const int arrived = atomicAdd(&tickets[seg.slab], 1);
    *last_flag = (arrived == seg.parts - 1) ? 1 : 0;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");
  if (*last_flag) {
    __threadfence();
    const int n0 = seg.slab * SKINNY_COLS;
    const size_t piece = size_t(M) * size_t(N);
    constexpr int kSlots = 16 * SKINNY_COLS / 4 / kThreads;   // float4 per thread and block of 16 rows: rows of 512 bytes
    constexpr int kBatch = kSlots <= 2 ? 4 : 2;               // pieces loaded together
    for (int row0 = 0; row0 < kRows && row0 < M; row0 += 16) {
      size_t off[kSlots];
      bool live[kSlots];
      float4 sum[kSlots];
#pragma unroll
      for (int i = 0; i < kSlots; ++i) {
        const int v = tid + kThreads * i;
        const int m = row0 + (v >> 5), col = n0 + (v & 31) * 4;
        live[i] = m < M && col < N;
        off[i] = size_t(m) * N + col;
        sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      for (int p0 = 0; p0 < seg.parts; p0 += kBatch) {
        float4 x[kSlots][kBatch];
#pragma unroll
        for (int i = 0; i < kSlots; ++i)
#pragma unroll
          for (int q = 0; q < kBatch; ++q)
            x[i][q] = (live[i] && p0 + q < seg.parts)
                          ? __ldcg(reinterpret_cast<const float4*>(partials + size_t(p0 + q) * piece + off[i]))
                          : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < kSlots; ++i)
#pragma unroll
          for (int q = 0; q < kBatch; ++q) {
            sum[i].x += x[i][q].x;
            sum[i].y += x[i][q].y;
            sum[i].z += x[i][q].z;
            sum[i].w += x[i][q].w;
          }
      }
#pragma unroll
      for (int i = 0; i < kSlots; ++i)
        if (live[i]) *reinterpret_cast<float4*>(C + off[i]) = sum[i];
    }
    if (tid == 0) tickets[seg.slab] = 0;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");   // last_flag is rewritten by the next piece
}

// The same for a slab whose tile is whole rows of C (the tall form): `rows` rows from row `row0`, `width` columns
// (a multiple of 4); the pieces' copies have row pitch `width`, C has row pitch `c_pitch`.
template <int kThreads>
__device__ __forceinline__ void skinny_finish_block(const SkinnySegment& seg, int tid, int bar_id, int* last_flag,
                                                    int* __restrict__ tickets, const float* __restrict__ partials,
                                                    float* __restrict__ C, size_t piece, int row0, int rows, int width,
                                                    int c_pitch) {
  __threadfence();
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");
  if (tid == 0) {
    const int arrived = atomicAdd(&tickets[seg.slab], 1);
    *last_flag = (arrived == seg.parts - 1) ? 1 : 0;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");
  if (*last_flag) {
    __threadfence();
    constexpr int kBatch = 4;   // pieces loaded together
    const int per_row = width / 4;
    for (int v = tid; v < rows * per_row; v += kThreads) {
      const int r = v / per_row, q4 = v - r * per_row;
      const size_t off = size_t(row0 + r) * width + size_t(q4) * 4;
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p0 = 0; p0 < seg.parts; p0 += kBatch) {
        float4 x[kBatch];
#pragma unroll
        for (int q = 0; q < kBatch; ++q)
          x[q] = p0 + q < seg.parts ? __ldcg(reinterpret_cast<const float4*>(partials + size_t(p0 + q) * piece + off))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < kBatch; ++q) {
          sum.x += x[q].x;
          sum.y += x[q].y;
          sum.z += x[q].z;
          sum.w += x[q].w;
        }
      }
      *reinterpret_cast<float4*>(C + size_t(row0 + r) * c_pitch + size_t(q4) * 4) = sum;
    }
    if (tid == 0) tickets[seg.slab] = 0;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(kThreads) : "memory");   // last_flag is rewritten by the next piece
}
#endif

}  // namespace vt
