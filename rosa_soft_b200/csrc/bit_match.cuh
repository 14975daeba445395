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
// positions start .. start + i - 1 (i >= 1).  `queue` is kBitQueue entries of shared memory
// private to the calling warp.  Returns (match length << 32 | route) with route the winning key
// position + 1 relative to the sequence start, or 0 for no match; every lane returns the same
// value.  All 32 lanes must call.
//
// Two stages.  The scan reads the level-1 word of 32 x 32 key positions per step (newest first)
// and appends the non-empty ones to the queue (ballot + prefix count).  Whenever 32 words are
// queued, or the scan ends, one batch is extended level by level with every lane holding one
// word, so the level loop runs on full warps instead of on the few words of a step that have
// a candidate at all.  Random candidates die within a level or two; when only a couple of
// words are left they are finished with the lanes spread over 32 levels at once, so a match
// of length L costs about L / 32 steps instead of L.
constexpr int kBitQueue = 64;
constexpr int kBitFewWords = 2;   // at most this many live words: switch to level-parallel

struct BitCandidate {
  int word;         // word index on the bitmap axis
  uint32_t bits;    // level-1 candidates inside it
};

template <typename Sym>
__device__ __forceinline__ unsigned long long bit_match_row(const Sym* __restrict__ q,
                                                            const uint32_t* __restrict__ e,
                                                            int64_t mask_words, int start, int i,
                                                            int W, int lane,
                                                            BitCandidate* __restrict__ queue) {
  const int g_lo = start, g_hi = start + i - 1;
  const int w_lo = g_lo >> 5, w_hi = g_hi >> 5;
  // every warp-wide primitive below is executed by all 32 lanes, never under a per-lane
  // condition
  const int sym_first = (int)q[i];
  const uint32_t* __restrict__ first_row = e + (int64_t)sym_first * mask_words;
  const unsigned lanes_below = (1u << lane) - 1u;
  int best_len = 0, best_route = 0;
  int queued = 0;                                         // same value in every lane
  bool done = false;                                      // a match reached the horizon

  // Extends the first min(queued, 32) queue entries to their full match length, keeps the best,
  // and moves the rest of the queue to the front.
  auto extend_batch = [&]() {
    __syncwarp();
    const bool mine = lane < queued;
    const int w = mine ? queue[lane].word : 0;
    uint32_t cur = mine ? queue[lane].bits : 0u;
    const int spill_w = lane + 32 < queued ? queue[lane + 32].word : 0;
    const uint32_t spill_bits = lane + 32 < queued ? queue[lane + 32].bits : 0u;
    int length = mine ? 1 : 0;
    bool alive = mine;
    // Shifted bitmap word of one level: bit g of it is bit g - lev of E[q_{i-lev}]; a bit may
    // only extend a match that still has a predecessor inside the sequence (g - lev >= start).
    auto level_mask = [&](int lev, int word) -> uint32_t {
      const uint32_t* __restrict__ row = e + (int64_t)q[i - lev] * mask_words;
      const int sh = lev & 31, hi_w = word - (lev >> 5);
      const uint32_t hi = hi_w >= w_lo ? row[hi_w] : 0u;
      const uint32_t lo = (sh != 0 && hi_w - 1 >= w_lo) ? row[hi_w - 1] : 0u;
      uint32_t m = __funnelshift_l(lo, hi, sh);
      const int lim = start + lev - 32 * word;            // bits below lim have no predecessor
      if (lim > 0) m = lim >= 32 ? 0u : m & (0xffffffffu << lim);
      return m;
    };
    // `lev` symbols are matched by every word still alive (its length equals lev).
    for (int lev = 1; lev < W && lev <= i; ++lev) {
      const unsigned alive_lanes = __ballot_sync(0xffffffffu, alive);
      if (alive_lanes == 0u) break;
      if (__popc(alive_lanes) <= kBitFewWords) {
        // Few words left, possibly with long matches: finish them one by one with the LANES
        // spread over 32 consecutive levels.  An inclusive AND scan of the level masks gives the
        // survivors after each level; the matches end at the first level with none.
        for (unsigned rest = alive_lanes; rest != 0u; rest &= rest - 1u) {
          const int src = __ffs(rest) - 1;
          const int word = __shfl_sync(0xffffffffu, w, src);
          uint32_t word_bits = __shfl_sync(0xffffffffu, cur, src);
          int word_len = lev;
          for (int base = lev; base < W && base <= i; base += 32) {
            const int level = base + lane;
            uint32_t m = (level < W && level <= i) ? level_mask(level, word) : 0u;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
              const uint32_t up = __shfl_up_sync(0xffffffffu, m, d);
              if (lane >= d) m &= up;
            }
            const uint32_t left = word_bits & m;           // survivors after level base + lane
            const unsigned ok = __ballot_sync(0xffffffffu, left != 0u);   // a prefix of ones
            const int passed = ok == 0xffffffffu ? 32 : __ffs(~ok) - 1;
            if (passed > 0) {
              word_bits = __shfl_sync(0xffffffffu, left, passed - 1);
              word_len = base + passed;
            }
            if (passed < 32) break;
          }
          if (lane == src) {
            cur = word_bits;
            length = word_len;
          }
        }
        break;
      }
      if (alive) {
        const uint32_t next = cur & level_mask(lev, w);
        if (next != 0u) {
          cur = next;
          length = lev + 1;
        } else {
          alive = false;
        }
      }
    }
    if (length > 0) {
      const int pos = 32 * w + 31 - __clz(cur);           // latest position of the longest match
      const int route = pos - start + 1;
      if (length > best_len || (length == best_len && route > best_route)) {
        best_len = length;
        best_route = route;
      }
    }
    __syncwarp();
    if (lane + 32 < queued) {
      queue[lane].word = spill_w;
      queue[lane].bits = spill_bits;
    }
    queued = queued > 32 ? queued - 32 : 0;
    // newer positions are queued first: nothing later in the queue or older on the axis can
    // beat a match at the horizon
    done = __any_sync(0xffffffffu, best_len >= W);
  };

  for (int wb = w_hi; wb >= w_lo && !done; wb -= 32) {    // newest positions first
    const int w = wb - lane;
    uint32_t bits = w >= w_lo ? first_row[w] : 0u;
    if (w == w_hi) bits &= 0xffffffffu >> (31 - (g_hi & 31));
    if (w == w_lo) bits &= 0xffffffffu << (g_lo & 31);
    const unsigned hit = __ballot_sync(0xffffffffu, bits != 0u);
    if (bits != 0u) {
      const int slot = queued + __popc(hit & lanes_below);
      queue[slot].word = w;
      queue[slot].bits = bits;
    }
    queued += __popc(hit);
    if (queued >= 32) extend_batch();
  }
  while (queued > 0 && !done) extend_batch();
  const int row_len = __reduce_max_sync(0xffffffffu, best_len);
  const int row_route = __reduce_max_sync(0xffffffffu, best_len == row_len ? best_route : 0);
  return row_len > 0 ? ((unsigned long long)(unsigned)row_len << 32) | (unsigned)row_route : 0ull;
}

}  // namespace rosa
