// Register-tiled sweeps of the dense surrogate VJP (same math and schedule as
// surrogate_vjp.cu: evidence recurrence along diagonals, online softmax with the analytic
// reference, dropout counter, checkpoints every 16 rows).
//
// One thread owns FOUR consecutive diagonals and walks them down the rows together.  On block
// row r the four cells of a thread sit on four consecutive key columns, and one row further
// down the same four diagonals sit one column to the right, so the key-side tables (key
// symbol, the symbol leaving the horizon window, value sign bits, first dropout hash round) of
// a group of four rows are seven consecutive columns: two aligned 128-bit shared-memory loads
// per table and sixteen cells, kept in registers and indexed at compile time.  Everything that
// depends on the row only (query symbols, hash word of the query position, utility table base)
// is loaded once per row and thread and shared by four cells; the row sums of four cells are
// added in registers before the warp reduction.  Rows of a block always start at a multiple of
// 16 (rows that do not exist are masked), interior blocks -- every cell active and past the
// horizon -- run without any per-cell predicate.
#include "common.cuh"
#include "vjp_shared.cuh"
#include "vjp_tiled.cuh"

namespace rosa {

namespace {

constexpr int kTR = 4;                          // diagonals per thread
constexpr int kTBand = kVjpBand;                // diagonals per band
constexpr int kTThreads = kTBand / kTR;         // threads per CTA
constexpr int kTWarps = kTThreads / 32;
constexpr int kTRows = kVjpRows;                // rows per checkpointed block
constexpr int kTWin = kTBand + kTRows;          // window columns of a block
// The column tables of a block (key symbols, symbols leaving the horizon, first hash round of the
// route, value sign nibbles) cover 272 key positions; the next block of the band needs the same
// positions moved by 16.  The tables therefore SLIDE inside a longer buffer: a block computes
// only its 16 entering columns and moves the base up; every 17th block the surviving 256 columns
// go back to the start (source [272, 528), destination [0, 256) and the entering columns
// [256, 272) are pairwise disjoint, so the step needs no barrier of its own).
constexpr int kTSlide = kTBand;
constexpr int kTTab = kTWin + kTSlide;          // entries per table
static_assert(kTRows == 16 && kTBand % 128 == 0, "geometry assumed by the register windows");

struct S1Smem {
  int* s_k;          // [kTWin] key symbols of the column window
  int* s_kold;       // [kTWin] key symbols W + 1 columns earlier
  uint32_t* s_h1;    // [kTWin] first dropout hash round of route j + 1
  uint32_t* s_vb0;   // [kTWin] spread value sign nibbles, groups 0..3
  uint32_t* s_vb1;   // [kTWin] groups 4..7
  int* s_q;          // [kTRows]
  int* s_qold;       // [kTRows]
  float* glut;       // [64] gate per mismatch count
  float2* wstat;     // [kTRows][kTWarps] per-warp (sum e, sum e d u)
  float* ulut;       // [kTRows][NG][16]
};

__host__ __device__ constexpr int s1_smem_words(int ng) {
  return 5 * kTTab + 2 * kTRows + 64 + 2 * kTRows * kTWarps + kTRows * ng * 16;
}

__device__ __forceinline__ S1Smem s1_carve(float* base, int ng) {
  S1Smem s;
  int* w = reinterpret_cast<int*>(base);
  s.s_k = w;                                        w += kTTab;
  s.s_kold = w;                                     w += kTTab;
  s.s_h1 = reinterpret_cast<uint32_t*>(w);          w += kTTab;
  s.s_vb0 = reinterpret_cast<uint32_t*>(w);         w += kTTab;
  s.s_vb1 = reinterpret_cast<uint32_t*>(w);         w += kTTab;
  s.s_q = w;                                        w += kTRows;
  s.s_qold = w;                                     w += kTRows;
  s.glut = reinterpret_cast<float*>(w);             w += 64;
  s.wstat = reinterpret_cast<float2*>(w);           w += 2 * kTRows * kTWarps;
  s.ulut = reinterpret_cast<float*>(w);
  (void)ng;
  return s;
}

// The column windows of one group of four rows: eight consecutive table entries per table,
// cell (row rr, diagonal e) reads entry rr + 3 - e.
template <int NG, bool kWindowed, bool kDropout>
struct ColWindow {
  int k[8];
  int kold[kWindowed ? 8 : 1];
  uint32_t h1[kDropout ? 8 : 1];
  uint32_t v0[8];
  uint32_t v1[NG > 4 ? 8 : 1];
};

template <int NG, bool kWindowed, bool kDropout>
__device__ __forceinline__ void load_quad(ColWindow<NG, kWindowed, kDropout>& cw, const S1Smem& sm,
                                          int col, int at) {
  const int4 kq = *reinterpret_cast<const int4*>(sm.s_k + col);
  cw.k[at] = kq.x; cw.k[at + 1] = kq.y; cw.k[at + 2] = kq.z; cw.k[at + 3] = kq.w;
  if (kWindowed) {
    const int4 ko = *reinterpret_cast<const int4*>(sm.s_kold + col);
    cw.kold[at] = ko.x; cw.kold[at + 1] = ko.y; cw.kold[at + 2] = ko.z; cw.kold[at + 3] = ko.w;
  }
  if (kDropout) {
    const uint4 hq = *reinterpret_cast<const uint4*>(sm.s_h1 + col);
    cw.h1[at] = hq.x; cw.h1[at + 1] = hq.y; cw.h1[at + 2] = hq.z; cw.h1[at + 3] = hq.w;
  }
  const uint4 va = *reinterpret_cast<const uint4*>(sm.s_vb0 + col);
  cw.v0[at] = va.x; cw.v0[at + 1] = va.y; cw.v0[at + 2] = va.z; cw.v0[at + 3] = va.w;
  if (NG > 4) {
    const uint4 vb = *reinterpret_cast<const uint4*>(sm.s_vb1 + col);
    cw.v1[at] = vb.x; cw.v1[at + 1] = vb.y; cw.v1[at + 2] = vb.z; cw.v1[at + 3] = vb.w;
  }
}

struct S1Params {
  int W, hs_cut, len;
  float neg_md, mul2, bias2;
};

// Sixteen cells: rows r0 .. r0 + 3 of the block, the thread's four diagonals.  kEdge adds the
// predicates of blocks that touch the start of a diagonal, the first W + 1 key columns or the
// end of the sequence.  Returns the keep flags as 16 bits (row rr, diagonal e at bit 4 rr + e)
// and adds the row sums to es / eds.
template <int NG, bool kWindowed, bool kDropout, bool kEdge>
__device__ __forceinline__ uint32_t s1_group(const ColWindow<NG, kWindowed, kDropout>& cw,
                                             const S1Smem& sm, const S1Params& p,
                                             const DropoutKey& dkey, int r0, int i0, int j_first,
                                             uint32_t qword0, float (&S)[kTR], int (&hs)[kTR],
                                             float (&es)[4], float (&eds)[4]) {
  int q[4], qo[4];
  {
    const int4 q4 = *reinterpret_cast<const int4*>(sm.s_q + r0);
    q[0] = q4.x; q[1] = q4.y; q[2] = q4.z; q[3] = q4.w;
    if (kWindowed) {
      const int4 o4 = *reinterpret_cast<const int4*>(sm.s_qold + r0);
      qo[0] = o4.x; qo[1] = o4.y; qo[2] = o4.z; qo[3] = o4.w;
    }
  }
  // mismatch counts and the sliding window sums of all sixteen cells first: whether any window
  // product of the warp survives flush-to-zero is decided once per group
  int ham[4][kTR];
  int hsv[4][kTR];
  bool alive = false;
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
#pragma unroll
    for (int e = 0; e < kTR; ++e) {
      const int idx = rr + 3 - e;
      ham[rr][e] = __popc(q[rr] ^ cw.k[idx]);
      if (kWindowed) {
        const int old = __popc(qo[rr] ^ cw.kold[idx]);
        if (kEdge) {
          const int j = j_first + rr - e;        // key column of the cell
          const bool act = j >= 0 && i0 + r0 + rr <= p.len - 1;
          hs[e] += act ? ham[rr][e] - (j > p.W ? old : 0) : 0;
          alive |= j >= p.W && hs[e] <= p.hs_cut;
        } else {
          hs[e] += ham[rr][e] - old;
          alive |= hs[e] <= p.hs_cut;
        }
        hsv[rr][e] = hs[e];
      }
    }
  }
  float P[4][kTR];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr)
#pragma unroll
    for (int e = 0; e < kTR; ++e) P[rr][e] = 0.0f;
  if (kWindowed && __any_sync(0xffffffffu, alive)) {
#pragma unroll
    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
      for (int e = 0; e < kTR; ++e) {
        bool on = hsv[rr][e] <= p.hs_cut;
        if (kEdge) on = on && (j_first + rr - e) >= p.W;
        P[rr][e] = on ? __expf(p.neg_md * (float)hsv[rr][e]) : 0.0f;
      }
  }
  uint32_t keepbits = 0;
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const float* lut = sm.ulut + (r0 + rr) * NG * 16;
    const uint32_t qword = qword0 ^ (uint32_t)(r0 + rr);   // block rows start at a multiple of 16
#pragma unroll
    for (int e = 0; e < kTR; ++e) {
      const int idx = rr + 3 - e;
      const float x = sm.glut[ham[rr][e]];
      const float Sn = x * (1.0f + S[e]) - P[rr][e];
      bool act = true;
      if (kEdge) act = (j_first + rr - e) >= 0 && i0 + r0 + rr <= p.len - 1;
      S[e] = act ? Sn : 0.0f;
      // the log i term cancels in the softmax, so the fixed reference drops it too
      float ex = exp2f(fmaf(sqrtf(1.0f + S[e]), p.mul2, p.bias2));
      if (kEdge) ex = act ? ex : 0.0f;
      const float du = tiled_utility<NG>(lut, cw.v0[idx], NG > 4 ? cw.v1[idx] : 0u);
      es[rr] += ex;
      if (kDropout) {
        const bool keep = act && dropout_keep_open(dkey, cw.h1[idx], qword);
        if (keep) {     // predicated: one logic operation and one fused multiply-add
          keepbits |= 1u << (4 * rr + e);
          eds[rr] = fmaf(ex, du, eds[rr]);
        }
      } else {
        eds[rr] = fmaf(ex, du, eds[rr]);
      }
    }
  }
  return keepbits;
}

// Sweep 1, four diagonals per thread.  Writes the same checkpoints and per-item row partials as
// vjp_sweep1_kernel<NG, true, ...> (analytic softmax reference only); the dropout keep flags go
// out as one 64-bit word per thread and block, the layout vjp_sweep2_tiled_kernel reads.
template <int NG, bool kWindowed, bool kDropout>
__global__ void __launch_bounds__(kTThreads, 8) vjp_sweep1_tiled_kernel(VjpArgs a) {
  extern __shared__ float4 smem_raw[];
  const S1Smem sm = s1_carve(reinterpret_cast<float*>(smem_raw), NG);
  Item it;
  if (!load_item_1d(a, &it)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool dense = a.plan.cu_seqlens == nullptr;
  const int64_t sym_base = (int64_t)it.seq * a.sym_seq_stride + (int64_t)it.h * a.sym_head_stride +
                           (dense ? 0 : it.start);
  const int32_t* __restrict__ q = a.qsym + sym_base;
  const int32_t* __restrict__ k = a.ksym + sym_base;
  const int vh = it.h / a.group;
  const uint32_t* __restrict__ vb = a.vbits + ((int64_t)vh * a.N + it.start) * a.vwords;
  const int W = a.W;
  S1Params p;
  p.W = W;
  p.len = it.len;
  p.neg_md = -a.mismatch_scale / (float)a.D;
  p.hs_cut = window_sum_cutoff(p.neg_md);
  const float logit_mul = kSqrtScale * a.scale;
  const float ref_top = a.scale * kSqrtScale * (sqrtf(1.0f + (float)W) - 1.0f);
  p.mul2 = logit_mul * 1.4426950408889634f;
  p.bias2 = -(logit_mul + ref_top) * 1.4426950408889634f;
  const DropoutKey dkey = make_dropout_key((uint32_t)it.h + a.head_offset,
                                           (uint32_t)it.seq + a.batch_offset, a.seed, a.dropout_p);
  if (tid <= a.D) sm.glut[tid] = expf(p.neg_md * (float)tid);
  const int vslot = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);

  for (int w = it.w_begin; w < it.w_end; ++w) {
    const int dmin = 1 + w * kTBand;
    const int dmax = dmin + kTBand - 1;
    float S[kTR];
    int hs[kTR];
#pragma unroll
    for (int e = 0; e < kTR; ++e) {
      S[e] = 0.0f;
      hs[e] = 0;
    }
    const int rb_lo = dmin / kTRows, rb_hi = (it.len - 1) / kTRows;
    int tab_base = 0;                           // window column 0 inside the table buffers
    const int64_t ck_band = it.ck_base + vjp_ck_before(it.len, w);
    for (int rb = rb_lo; rb <= rb_hi; ++rb) {
      const int i0 = rb * kTRows;                 // rows i0 .. i0 + 15, masked where absent
      const int jwin0 = i0 - dmax;                // key column of window index 0
      const int first_row = max(i0, dmin);        // rows below it belong to no cell of the band
      const int skew = first_row - i0;
      const int64_t ck_idx = ck_band + (rb - rb_lo);
      // No barrier here: every warp has passed the barrier that closes the previous block (all
      // table reads done), and the threads that still read the per-warp row sums after it are
      // through before they reach the barrier below, ahead of which nobody writes new sums.
      // ---- block tables: entry `at` of the buffers describes window column c.  Every global
      // load of the block (entering columns, row symbols, grad_output of the utility tables) is
      // issued before the first result is used, so the section costs one round trip to L2, not
      // three in a row.
      struct ColRaw { int k, kold; uint32_t bits; };
      auto load_col = [&](int c) {
        const int j = jwin0 + c;
        const bool in = j >= 0 && j < it.len - 1;
        const int jo = j - W - 1;
        ColRaw r;
        r.k = in ? __ldg(k + j) : 0;
        r.kold = (kWindowed && jo >= 0 && jo < it.len) ? __ldg(k + jo) : 0;
        r.bits = in ? __ldg(vb + j + 1) : 0u;
        return r;
      };
      auto store_col = [&](int at, int c, const ColRaw& r) {
        sm.s_k[at] = r.k;
        sm.s_kold[at] = r.kold;
        if (kDropout) sm.s_h1[at] = dropout_route_open((uint32_t)(jwin0 + c + 1));
        sm.s_vb0[at] = spread_nibbles(r.bits & 0xffffu);
        if (NG > 4) sm.s_vb1[at] = spread_nibbles(r.bits >> 16);
      };
      // raw grad_output element (converted after all loads are under way)
      auto go_raw = [&](int64_t idx) -> uint32_t {
        return a.dtype == ROSA_B200_F32 ? __ldg(static_cast<const uint32_t*>(a.go) + idx)
                                        : (uint32_t)__ldg(static_cast<const uint16_t*>(a.go) + idx);
      };
      auto go_value = [&](uint32_t bits) {
        if (a.dtype == ROSA_B200_F32) return __uint_as_float(bits);
        if (a.dtype == ROSA_B200_F16) return __half2float(__ushort_as_half((unsigned short)bits));
        return __uint_as_float(bits << 16);
      };
      // utility table of (row, value group) e from its four raw elements
      auto store_ulut = [&](int e, const uint32_t (&raw)[4]) {
        float gv[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) gv[b] = go_value(raw[b]);
        float4* dst = reinterpret_cast<float4*>(sm.ulut + e * 16);
#pragma unroll
        for (int n4 = 0; n4 < 4; ++n4) {
          // nibbles 4 n4 .. 4 n4 + 3: bits 2 and 3 fixed by n4, bits 0 and 1 vary
          const float hi = ((n4 & 1) ? gv[2] : -gv[2]) + ((n4 & 2) ? gv[3] : -gv[3]);
          dst[n4] = make_float4(hi - gv[0] - gv[1], hi + gv[0] - gv[1], hi - gv[0] + gv[1],
                                hi + gv[0] + gv[1]);
        }
      };
      auto load_go4 = [&](int e, uint32_t (&raw)[4]) {
        const int r = e / NG, g = e - r * NG;
        const int i = i0 + r;
#pragma unroll
        for (int b = 0; b < 4; ++b) raw[b] = 0u;     // +0.0 in every dtype
        if (e < kTRows * NG && i >= first_row && i <= it.len - 1) {
          const int64_t base = (((int64_t)it.start + i) * a.H + it.h) * a.Dv + 4 * g;
#pragma unroll
          for (int b = 0; b < 4; ++b)
            if (4 * g + b < a.Dv) raw[b] = go_raw(base + b);
        }
      };
      // -- loads
      ColRaw entering{0, 0, 0u};
      int q_new = 0, qold_new = 0;
      if (tid < kTRows) {
        if (rb != rb_lo) entering = load_col(kTBand + tid);
        const int i = i0 + tid;
        const bool in = i >= first_row && i <= it.len - 1;
        q_new = in ? __ldg(q + i) : 0;
        qold_new = (kWindowed && in && i - W - 1 >= 0) ? __ldg(q + i - W - 1) : 0;
      }
      uint32_t go_first[4];
      // the per-block chores are spread over both warps: warp 0 fetches the entering columns and
      // the row symbols, warp 1 builds the utility tables and closes the block's row sums
      const int ue = (tid + kTThreads / 2) & (kTThreads - 1);
      load_go4(ue, go_first);
      // -- shared-memory side
      if (rb == rb_lo) {                          // a band starts: the whole window
        tab_base = 0;
        for (int c = tid; c < kTWin; c += kTThreads) store_col(c, c, load_col(c));
      } else {                                    // the window moved up by 16 columns
        if (tab_base < kTSlide) {
          tab_base += kTRows;
        } else {
          for (int e = tid; e < kTWin - kTRows; e += kTThreads) {
            const int from = kTSlide + kTRows + e;
            sm.s_k[e] = sm.s_k[from];
            if (kWindowed) sm.s_kold[e] = sm.s_kold[from];
            if (kDropout) sm.s_h1[e] = sm.s_h1[from];
            sm.s_vb0[e] = sm.s_vb0[from];
            if (NG > 4) sm.s_vb1[e] = sm.s_vb1[from];
          }
          tab_base = 0;
        }
        if (tid < kTRows) store_col(tab_base + kTBand + tid, kTBand + tid, entering);
      }
      S1Smem win = sm;                            // the tables as the block's window sees them
      win.s_k += tab_base;
      win.s_kold += tab_base;
      win.s_h1 += tab_base;
      win.s_vb0 += tab_base;
      win.s_vb1 += tab_base;
      if (tid < kTRows) {
        sm.s_q[tid] = q_new;
        sm.s_qold[tid] = qold_new;
      }
      // nibble tables: one thread per (row, value group) builds its sixteen signed sums
      if (ue < kTRows * NG) store_ulut(ue, go_first);
      for (int e = ue + kTThreads; e < kTRows * NG; e += kTThreads) {
        uint32_t raw[4];
        load_go4(e, raw);
        store_ulut(e, raw);
      }
      __syncthreads();
      // ---- checkpoint of the thread's four diagonals
      {
        int4* ck = reinterpret_cast<int4*>(a.ckpt + ck_idx * kTBand + kTR * tid);
        ck[0] = make_int4(__float_as_int(S[0]), hs[0], __float_as_int(S[1]), hs[1]);
        ck[1] = make_int4(__float_as_int(S[2]), hs[2], __float_as_int(S[3]), hs[3]);
      }
      const bool interior = jwin0 >= (kWindowed ? W + 1 : 0) && i0 + kTRows - 1 <= it.len - 1;
      const uint32_t qword0 = dropout_query_word((uint32_t)i0);
      // window column of (row 0, diagonal 3 of this thread); a multiple of 4
      const int col0 = kTBand - kTR - kTR * tid;
      ColWindow<NG, kWindowed, kDropout> cw;
      load_quad<NG, kWindowed, kDropout>(cw, win, col0, 0);
      uint32_t keep_lo = 0u, keep_hi = 0u;
#pragma unroll 1
      for (int r0 = 0; r0 < kTRows; r0 += 4) {
        load_quad<NG, kWindowed, kDropout>(cw, win, col0 + r0 + 4 < kTWin ? col0 + r0 + 4 : col0 + r0, 4);
        float es[4] = {0.0f, 0.0f, 0.0f, 0.0f}, eds[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // key column of (row r0, diagonal 0 of this thread)
        const int j_first = jwin0 + col0 + r0 + 3;
        uint32_t keep;
        if (interior)
          keep = s1_group<NG, kWindowed, kDropout, false>(cw, sm, p, dkey, r0, i0, j_first, qword0, S,
                                                          hs, es, eds);
        else
          keep = s1_group<NG, kWindowed, kDropout, true>(cw, sm, p, dkey, r0, i0, j_first, qword0, S,
                                                         hs, es, eds);
        if (kDropout) {
          // 16 keep flags of this group: bit 4 r + e of the thread's 64-bit word of the block
          if (r0 < 8) keep_lo |= keep << (4 * r0);
          else keep_hi |= keep << (4 * (r0 - 8));
        }
        float v[8];
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          v[2 * rr] = es[rr];
          v[2 * rr + 1] = eds[rr];
        }
        const float total = warp_reduce8(v, lane);
        if ((lane & 3) == 0)
          reinterpret_cast<float*>(sm.wstat + (r0 + (vslot >> 1)) * kTWarps + warp)[vslot & 1] = total;
        // the upper quad becomes the lower one of the next group
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          cw.k[x] = cw.k[x + 4];
          if (kWindowed) cw.kold[x] = cw.kold[x + 4];
          if (kDropout) cw.h1[x] = cw.h1[x + 4];
          cw.v0[x] = cw.v0[x + 4];
          if (NG > 4) cw.v1[x] = cw.v1[x + 4];
        }
      }
      // keep flags of the block: one 64-bit word per thread (row r, diagonal e at bit 4 r + e)
      if (kDropout)
        reinterpret_cast<uint2*>(a.keepbits)[ck_idx * kTThreads + tid] = make_uint2(keep_lo, keep_hi);
      __syncthreads();
      const int tr = tid - kTThreads / 2;         // row of the tail, on warp 1
      if (tr >= 0 && tr < kTRows) {
        const int i = i0 + tr;
        if (i >= first_row && i <= it.len - 1) {
          float m = ref_top - logf((float)i), z = 0.0f, e = 0.0f;
#pragma unroll
          for (int ww = 0; ww < kTWarps; ++ww) {
            const float2 part = sm.wstat[tr * kTWarps + ww];
            z += part.x;
            e += part.y;
          }
          e *= a.inv_keep;
          const int64_t slot = it.rowslot + i;
          if (w > it.w_begin) {
            const float4 prev = a.stat_part[slot];
            merge_stats(m, z, e, prev.x, prev.y, prev.z);
          }
          a.stat_part[slot] = make_float4(m, z, e, 0.0f);
        }
      }
    }
  }
}

template <int NG>
int launch_s1_tiled(const VjpArgs& a, unsigned grid, cudaStream_t stream) {
  const size_t smem = (size_t)s1_smem_words(NG) * sizeof(float);
  const bool windowed = a.ring_slots > 0;
  const bool dropout = a.dropout_p > 0.0f;
  if (windowed && dropout)
    vjp_sweep1_tiled_kernel<NG, true, true><<<grid, kTThreads, smem, stream>>>(a);
  else if (windowed)
    vjp_sweep1_tiled_kernel<NG, true, false><<<grid, kTThreads, smem, stream>>>(a);
  else if (dropout)
    vjp_sweep1_tiled_kernel<NG, false, true><<<grid, kTThreads, smem, stream>>>(a);
  else
    vjp_sweep1_tiled_kernel<NG, false, false><<<grid, kTThreads, smem, stream>>>(a);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

bool vjp_tiled_applies(const VjpArgs& a) {
  // value rows of up to 32 components (nibble tables), symbols of up to 16 bits (one MMA N of the
  // second sweep), the analytic softmax reference, and not the testing flag that selects the
  // one-diagonal-per-thread kernels
  const float top = a.scale * kSqrtScale * (sqrtf(1.0f + (float)a.W) - 1.0f);
  return a.Dv <= 32 && a.D <= 16 && top <= 80.0f && !a.force_cuda_core_contraction;
}

int launch_vjp_sweep1_tiled(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  const unsigned grid = (unsigned)((int64_t)items_upper * a.H);
  if (a.Dv <= 8) return launch_s1_tiled<2>(a, grid, stream);
  if (a.Dv <= 16) return launch_s1_tiled<4>(a, grid, stream);
  return launch_s1_tiled<8>(a, grid, stream);
}

}  // namespace rosa
