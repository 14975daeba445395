// Bit-parallel latest-longest suffix matcher for symbols of at most 8 bits, shared by the
// training forward (hard_forward.cu) and the streaming runtime (stream_runtime.cu).
//
// The key stream of a head is kept as one occurrence bitmap per symbol: bit g of E[s] is set
// iff the key symbol at position g is s.  For a query row i the positions whose last L symbols
// agree with the query's are
//     B_1 = E[q_i],      B_{L+1} = B_L & (E[q_{i-L}] << L).
// A position's match length is the number of levels it survives, so every 32-position word is
// evaluated on its own: levels are ANDed in until the word dies, the survivors of the last
// level carry the word's longest match and the highest of them is the latest.  Work per row is
// (levels survived) x (row length / 32) instead of one compare per causal pair; a level costs
// two coalesced loads, a funnel shift and an AND per 32 candidate positions.
// Semantics: reference rosa_soft/soft_reference.py:197-231 (capped suffix length, latest among
// the longest), rosa_soft/csrc/rosa_runtime.cpp:103-133 for the streaming form.
#pragma once

#include <cstdint>

namespace rosa {

// One warp evaluates one query row.  `q[p]` is the query symbol p positions after the
// sequence start (p <= i readable), `e` the bitmaps of this head, row s at e + s * mask_words,
// over an axis on which the sequence starts at bit `start`; the candidates of the row are key
// positions start .. start + i - 1 (i >= 1).  Returns (match length << 32 | route) with route
// the winning key position + 1 relative to the sequence start, or 0 for no match; every lane
// returns the same value.  All 32 lanes must call.
//
// A lane holds kBitSpan words at once (the warp covers 32 * 32 * kBitSpan key positions per
// pass, newest first) and advances all of them level by level, so the loads of one level are
// in flight together instead of one dependent load chain per word.
#ifndef ROSA_BIT_SPAN
#define ROSA_BIT_SPAN 1
#endif
constexpr int kBitSpan = ROSA_BIT_SPAN;

template <typename Sym>
__device__ __forceinline__ unsigned long long bit_match_row(const Sym* __restrict__ q,
                                                            const uint32_t* __restrict__ e,
                                                            int64_t mask_words, int start, int i,
                                                            int W, int lane) {
  const int g_lo = start, g_hi = start + i - 1;
  const int w_lo = g_lo >> 5, w_hi = g_hi >> 5;
  const int q_first = lane <= i ? (int)q[i - lane] : 0;   // lane l: query symbol l rows back
  // every warp-wide primitive below is executed by all 32 lanes, never under a per-lane
  // condition
  const int sym_first = __shfl_sync(0xffffffffu, q_first, 0);
  const uint32_t* __restrict__ first_row = e + (int64_t)sym_first * mask_words;
  int best_len = 0, best_route = 0;

  for (int wtop = w_hi; wtop >= w_lo; wtop -= 32 * kBitSpan) {   // newest positions first
    uint32_t cur[kBitSpan];
    int length[kBitSpan];
    unsigned alive = 0u;                                  // bit c: word c can still extend
#pragma unroll
    for (int c = 0; c < kBitSpan; ++c) {
      const int w = wtop - 32 * c - lane;
      uint32_t bits = w >= w_lo ? first_row[w] : 0u;
      if (w == w_hi) bits &= 0xffffffffu >> (31 - (g_hi & 31));
      if (w == w_lo) bits &= 0xffffffffu << (g_lo & 31);
      cur[c] = bits;
      length[c] = bits ? 1 : 0;
      alive |= bits ? 1u << c : 0u;
    }
    int qv = q_first;
    for (int lev = 1; lev < W && __any_sync(0xffffffffu, alive != 0u); ++lev) {
      if ((lev & 31) == 0) qv = lev + lane <= i ? (int)q[i - lev - lane] : 0;
      const int sym = __shfl_sync(0xffffffffu, qv, lev & 31);
      const uint32_t* __restrict__ row = e + (int64_t)sym * mask_words;
      const int sh = lev & 31;
#pragma unroll
      for (int c = 0; c < kBitSpan; ++c) {
        if (alive >> c & 1u) {
          // bit g of the shifted bitmap is bit g - lev of E[sym]; it may only extend a match
          // that still has a predecessor inside the sequence: g - lev >= start
          const int w = wtop - 32 * c - lane;
          const int hi_w = w - (lev >> 5);
          const uint32_t hi = hi_w >= w_lo ? row[hi_w] : 0u;
          const uint32_t lo = (sh != 0 && hi_w - 1 >= w_lo) ? row[hi_w - 1] : 0u;
          uint32_t m = __funnelshift_l(lo, hi, sh);
          const int lim = start + lev - 32 * w;           // bits below lim have no predecessor
          if (lim > 0) m = lim >= 32 ? 0u : m & (0xffffffffu << lim);
          const uint32_t next = cur[c] & m;
          if (next != 0u) {
            cur[c] = next;
            length[c] = lev + 1;
          } else {
            alive &= ~(1u << c);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < kBitSpan; ++c) {
      if (length[c] > 0) {
        const int w = wtop - 32 * c - lane;
        const int pos = 32 * w + 31 - __clz(cur[c]);      // latest position of the longest match
        const int route = pos - start + 1;
        if (length[c] > best_len || (length[c] == best_len && route > best_route)) {
          best_len = length[c];
          best_route = route;
        }
      }
    }
    // newer positions were examined first: nothing older can beat a match at the horizon
    if (__reduce_max_sync(0xffffffffu, best_len) >= W) break;
  }
  const int row_len = __reduce_max_sync(0xffffffffu, best_len);
  const int row_route = __reduce_max_sync(0xffffffffu, best_len == row_len ? best_route : 0);
  return row_len > 0 ? ((unsigned long long)(unsigned)row_len << 32) | (unsigned)row_route : 0ull;
}

}  // namespace rosa
