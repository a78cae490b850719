// How the persistent decode kernel deals its work, as plain integer functions usable on the
// host and on the device.
//
// The (virtual head, request, 16-token tile) space is one line, head-major: head vh occupies
// the tiles [vh*Tb, (vh+1)*Tb), request b of a head the tiles [prefix[b], prefix[b+1]) of it.
// CTA c owns the share [ga, gb) of the line, which touches at most two heads ("phases" 0
// and 1); inside a phase the share is split evenly over the NW warps of the CTA ("ranges",
// range index (c*2+ph)*NW + w).  A request that is not contained in one warp's run is CUT:
// every warp whose run meets it leaves a partial result in one of the two slots of its range
// (slot 1 when the part begins the request, else slot 0), except that a CTA whose whole
// phase-span lies inside the request merges its warps first and leaves ONE partial, in the
// slots of its first range.  The functions below give the share of a CTA, the runs of its
// warps, and - for the warp that finds itself the last to finish a cut request - the list of
// all the parts of that request, without reading anything another CTA wrote.
#pragma once

#include <stdint.h>

#ifdef __CUDACC__
#define BKV_HD __host__ __device__ __forceinline__
#else
#define BKV_HD inline
#endif

namespace bkv {
namespace part {

struct Plan {
  int C;        // CTAs of the grid
  int NW;       // warps per CTA
  int hv;       // virtual heads: kv heads x query-head quads
  int Tb;       // tiles of one head (all requests)
  int aligned;  // 1: every share lies inside one head (heads get floor or ceil of C / hv CTAs)
  int gap;      // equal-cost shares: tiles by which a share that straddles two heads is shortened
};

// share [ga, gb) of CTA `cta` on the tile line
BKV_HD void share_of(const Plan& pl, int cta, int64_t* ga, int64_t* gb) {
  const int64_t Tb = pl.Tb;
  if (pl.aligned) {
    // heads 0..extra-1 are served by base+1 CTAs, the others by base
    const int base = pl.C / pl.hv, extra = pl.C - base * pl.hv;
    int h, idx, cnt;
    if (cta < extra * (base + 1)) {
      h = cta / (base + 1);
      idx = cta - h * (base + 1);
      cnt = base + 1;
    } else {
      const int c2 = cta - extra * (base + 1);
      h = extra + c2 / base;
      idx = c2 - (c2 / base) * base;
      cnt = base;
    }
    *ga = h * Tb + Tb * idx / cnt;
    *gb = h * Tb + Tb * (idx + 1) / cnt;
    return;
  }
  // Equal shares of COST: the cost line is the tile line with a gap of `gap` tiles at every
  // head boundary (a CTA whose share straddles two heads sets up twice).  A share that contains
  // a gap is that much shorter in tiles; one that ends inside a gap ends at the head boundary.
  const int64_t gap = pl.gap;
  const int64_t L = static_cast<int64_t>(pl.hv) * Tb + (pl.hv - 1) * gap;
  const int64_t xs[2] = {L * cta / pl.C, L * (cta + 1) / pl.C};
  int64_t out[2];
  for (int i = 0; i < 2; ++i) {
    const int64_t x = xs[i];
    // the gap of head boundary h covers [h*Tb + (h-1)*gap, h*(Tb + gap)) of the cost line
    int64_t passed = Tb + gap > 0 ? x / (Tb + gap) : 0;  // gaps that lie wholly before x
    if (passed > pl.hv - 1) passed = pl.hv - 1;
    int64_t y = x - passed * gap;
    const int64_t h = passed + 1;
    if (h <= pl.hv - 1 && x > h * Tb + (h - 1) * gap) y = h * Tb;  // inside the next gap
    out[i] = y;
  }
  *ga = out[0];
  *gb = out[1];
}

struct Span {
  int vh;     // virtual head of the phase
  int first;  // first tile of the span inside the head
  int span;   // tiles (0: the share has no such phase)
};

BKV_HD Span phase_span(const Plan& pl, int64_t ga, int64_t gb, int ph) {
  Span s = {0, 0, 0};
  if (pl.Tb <= 0 || gb <= ga) return s;
  s.vh = static_cast<int>(ga / pl.Tb) + ph;
  const int64_t h0 = static_cast<int64_t>(s.vh) * pl.Tb;
  const int64_t a = ga > h0 ? ga : h0;
  const int64_t e = gb < h0 + pl.Tb ? gb : h0 + pl.Tb;
  s.span = e > a ? static_cast<int>(e - a) : 0;
  s.first = static_cast<int>(a - h0);
  return s;
}

BKV_HD int run_begin(const Span& s, int NW, int w) {
  // (the same value either way; the 32-bit form is what the merging warp's loop over the warps runs)
  if (s.span < (1 << 26)) return s.first + static_cast<int>(static_cast<uint32_t>(s.span) * static_cast<uint32_t>(w) / static_cast<uint32_t>(NW));
  return s.first + static_cast<int>(static_cast<int64_t>(s.span) * w / NW);
}

// CTAs [*c_lo, *c_hi] (inclusive) outside of which no share touches head vh: a bound, not exact.
BKV_HD void ctas_near_head(const Plan& pl, int vh, int* c_lo, int* c_hi) {
  if (pl.aligned) {
    const int base = pl.C / pl.hv, extra = pl.C - base * pl.hv;
    const int lo = vh < extra ? vh * (base + 1) : extra * (base + 1) + (vh - extra) * base;
    *c_lo = lo;
    *c_hi = lo + (vh < extra ? base : base - 1);
    return;
  }
  // on the cost line head vh, with the gap in front of it, covers [vh*(Tb+gap) - gap, vh*(Tb+gap) + Tb)
  const int64_t Tb = pl.Tb, gap = pl.gap;
  const int64_t L = static_cast<int64_t>(pl.hv) * Tb + (pl.hv - 1) * gap;
  const int64_t lo_cost = vh * (Tb + gap) - gap, hi_cost = vh * (Tb + gap) + Tb;
  int64_t lo = L > 0 ? lo_cost * pl.C / L - 1 : 0, hi = L > 0 ? hi_cost * pl.C / L + 1 : pl.C - 1;
  if (lo < 0) lo = 0;
  if (hi > pl.C - 1) hi = pl.C - 1;
  *c_lo = static_cast<int>(lo);
  *c_hi = static_cast<int>(hi);
}

// The parts of the request with tiles [pb, pe) of head vh that CTA `cta` leaves.
struct CtaParts {
  uint32_t mask;  // bit w: warp w leaves a part (solo: bit 0 only)
  int ph;         // phase of the CTA that meets the request
  int solo;       // 1: one partial for the whole CTA
  int starts;     // 1: the lowest part of the mask begins the request (slot 1 instead of slot 0)
};

// (ga, gb: the share of the CTA, from share_of or from a table of the share boundaries; NWT: the
// warps per CTA when known at compile time, which turns the divisions of the loop into multiplications)
template <int NWT = 0>
BKV_HD CtaParts cta_parts(const Plan& pl, int64_t ga, int64_t gb, int vh, int pb, int pe) {
  const int NW = NWT > 0 ? NWT : pl.NW;
  CtaParts r = {0u, 0, 0, 0};
  // the span of this share inside head vh, and which of the share's (at most two) heads that is:
  // the first one unless the share begins before the head (no division needed for either)
  const int64_t h0 = static_cast<int64_t>(vh) * pl.Tb;
  const int64_t a64 = ga > h0 ? ga : h0, e64 = gb < h0 + pl.Tb ? gb : h0 + pl.Tb;
  if (e64 <= a64) return r;
  Span s;
  s.vh = vh;
  s.first = static_cast<int>(a64 - h0);
  s.span = static_cast<int>(e64 - a64);
  const int a = s.first > pb ? s.first : pb;
  const int e = s.first + s.span < pe ? s.first + s.span : pe;
  if (e <= a) return r;
  r.ph = ga < h0 ? 1 : 0;
  if (pb <= s.first && s.first + s.span <= pe) {
    r.solo = 1;
    r.mask = 1u;
    r.starts = s.first == pb;
    return r;
  }
  int wa = s.first;
  for (int w = 0; w < NW; ++w) {
    const int wb = run_begin(s, NW, w + 1);
    const int i0 = wa > pb ? wa : pb, i1 = wb < pe ? wb : pe;
    if (i1 > i0) {
      if (r.mask == 0u) r.starts = i0 == pb;
      r.mask |= 1u << w;
    }
    wa = wb;
  }
  return r;
}

BKV_HD int part_slot(const Plan& pl, int cta, int ph, int w, int starts) {
  return 2 * ((cta * 2 + ph) * pl.NW + w) + (starts ? 1 : 0);
}

}  // namespace part
}  // namespace bkv
