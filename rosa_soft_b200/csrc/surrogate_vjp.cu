// Dense surrogate VJP of the rosa_soft operator.  Replaces local_match_gate,
// raw_suffix_score, transform_suffix_score, the online softmax helpers, the dropout
// counter, scan_route_value, the per-step adjoint loop, accumulate_local_match_qk_vjp,
// surrogate_vjp_kernel and finalize_surrogate_vjp_kernel of the reference
// (rosa_soft/csrc/cuda/rosa_soft_kernels.cu:534-1731) with an O(1)-per-cell scheme.
//
// Math (per sequence and head; cell = (row i, key column j), route a = j + 1, diagonal
// delta = i - j, n = j the position along the diagonal):
//   gate      x_n  = exp(-m * popc(q_i ^ k_j) / D)
//   evidence  S_n  = x_n (1 + S_{n-1}) - P_n,  P_n = prod_{u=0..W} x_{n-u} (0 if n < W)
//             which equals the reference's sum of prefix products over min(W, a) steps;
//             P_n is rebuilt from a sliding integer sum of mismatch counts, so nothing
//             but S itself is carried in floating point.
//   logits    l(i,a) = c (sqrt(1+S) - 1) scale - log i ;  null logit 0.5 scale
//   softmax   p, dropout multiplier d in {0, 1/(1-p_drop)}, u = gO(i) . sign(V[a])
//   dlogit    = p (d u - E_i),  E_i = sum_a p d u ;  dS = scale dlogit c / (2 sqrt(1+S))
//   adjoint   Sbar_n = dS_n + x_{n+1} Sbar_{n+1}
//             Y_n    = sum_{n' = n..n+W} Sbar_{n'} P_{n'}           (sliding window)
//             C_n    = (S_n + P_n) Sbar_n - Y_n
//             C is the adjoint of log x_n: dQz[i] += m/(2D) C k_z[j], dKz[j] += m/(2D) C q_z[i]
//   values    dVz[a] += p d gO(i)
// Sbar and Y are kept in float64 because Y is a difference of long running sums when
// exact matches are longer than the horizon (the tensor-core kernel runs Sbar in float32
// inside a row block while no window product is alive: the recurrence is a contraction then).
//
// Schedule: sweep 1 walks every band top-down (rows ascending), produces per-row
// online-softmax partials and a checkpoint (S, mismatch-window sum) every kVjpRows rows;
// a tiny kernel merges the partials into row statistics; sweep 2 walks the bands
// bottom-up one row block at a time: re-runs the forward recurrence of the block from
// its checkpoint into shared memory, runs the adjoint recurrence backwards over it, then
// contracts the block's C and p*d tiles into per-item partial gradients.  A last kernel
// sums the partials in a fixed order and applies the softsign Jacobian: no floating
// point atomics anywhere.
#include <math_constants.h>

#include "common.cuh"
#include "tcgen05.cuh"
#include "vjp_shared.cuh"

namespace rosa {

namespace {

// ------------------------------------------------------------ value sign bits
template <typename T>
__global__ void pack_value_bits_kernel(const T* __restrict__ v, int64_t N, int Hv, int Dv,
                                       uint32_t* __restrict__ vbits, int vwords) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * Hv * vwords) return;
  const int wd = (int)(idx % vwords);
  const int64_t tv = idx / vwords;
  const int64_t token = tv / Hv;
  const int vh = (int)(tv - token * Hv);
  const T* row = v + tv * Dv;
  uint32_t bits = 0;
  const int d0 = wd * 32, d1 = min(Dv, d0 + 32);
  for (int d = d0; d < d1; ++d) bits |= (uint32_t)((float)row[d] > 0.0f) << (d - d0);
  vbits[((int64_t)vh * N + token) * vwords + wd] = bits;
}

// Builds, for the rows [i0, i0 + nrows) of one head, the nibble tables
//   ulut[r][g][nib] = sum_{b<4} (nib bit b ? +1 : -1) * gO[i0 + r][4 g + b]
// so that u(i, a) is a sum of Dv/4 table lookups keyed by the value sign bits.
__device__ __forceinline__ void build_ulut(const VjpArgs& a, const Item& it, int i0, int nrows,
                                           int ngroups, float* ulut) {
  const int total = nrows * ngroups * 16;
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    const int nib = e & 15;
    const int g = (e >> 4) % ngroups;
    const int r = (e >> 4) / ngroups;
    const int64_t base = (((int64_t)it.start + i0 + r) * a.H + it.h) * a.Dv;
    float s = 0.0f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int d = 4 * g + b;
      if (d < a.Dv) {
        const float gv = load_as_float(a.go, base + d, a.dtype);
        s += (nib >> b & 1) ? gv : -gv;
      }
    }
    ulut[(r * ngroups + g) * 16 + nib] = s;
  }
}

// u(i, a) = gO(i) . sign(V[a])
template <bool kSmallDv>
__device__ __forceinline__ float route_utility(const VjpArgs& a, const Item& it,
                                               const uint32_t* __restrict__ vb, int i, int r,
                                               int route, int ngroups, const float* ulut) {
  if (kSmallDv) {
    const uint32_t bits = __ldg(vb + route);
    float u = 0.0f;
    for (int g = 0; g < ngroups; ++g) u += ulut[(r * ngroups + g) * 16 + ((bits >> (4 * g)) & 15u)];
    return u;
  } else {
    const int64_t base = (((int64_t)it.start + i) * a.H + it.h) * a.Dv;
    float u = 0.0f;
    for (int wd = 0; wd < a.vwords; ++wd) {
      const uint32_t bits = __ldg(vb + (int64_t)route * a.vwords + wd);
      const int d1 = min(32, a.Dv - wd * 32);
      for (int b = 0; b < d1; ++b) {
        const float gv = load_as_float(a.go, base + wd * 32 + b, a.dtype);
        u += (bits >> b & 1u) ? gv : -gv;
      }
    }
    return u;
  }
}

// ------------------------------------------------------------ block tables
// Every row block of a band touches the query rows [i0, i0 + nrows) and the key columns
// [jwin0, jwin0 + nrows + kVjpBand - 1), jwin0 = i0 - dmax.  Thread `tid` (diagonal
// dmin + tid) on block row r sits on column index c = r + kVjpBand - 1 - tid of that
// window, so everything a cell needs is one shared-memory read away and the inner loops
// carry no global loads, no bounds branches and no 64-bit address arithmetic.
constexpr int kWinCols = kVjpRows + kVjpBand;  // window columns (one spare)

struct SweepSmem {
  float4* rstat;     // [kVjpRows] (max, 1/Z, E, log i); sweep 1 only uses .w
  float4* wstat;     // [kVjpRows * kVjpWarps] per-warp softmax partials (sweep 1)
  uint32_t* s_keep;  // [kVjpRows * kVjpWarps] dropout keep ballots of the block (sweep 2)
  float* ulut;       // [kVjpRows * ngroups * 16] nibble tables of gO . sign(V)
  float* glut;       // [64] gate per mismatch count
  int* s_q;          // [kVjpRows] query symbols of the block rows
  int* s_qold;       // [kVjpRows] query symbols W + 1 rows earlier (window tail)
  int* s_k;          // [kWinCols] key symbols of the column window
  int* s_kold;       // [kWinCols] key symbols W + 1 columns earlier
  uint32_t* s_vb;    // [kWinCols] value sign bits of route j + 1 (Dv <= 32)
  uint32_t* s_h1;    // [kWinCols] first dropout hash round of route j + 1 (sweep 1)
  float* rest;       // first float after the common part
};

__host__ __device__ inline int sweep_common_floats(int ngroups) {
  return 4 * kVjpRows + 4 * kVjpRows * kVjpWarps + kVjpRows * ngroups * 16 + 64 + 2 * kVjpRows +
         4 * kWinCols;
}

__device__ __forceinline__ SweepSmem carve_common(float* base, int ngroups) {
  SweepSmem s;
  s.rstat = reinterpret_cast<float4*>(base);
  s.wstat = s.rstat + kVjpRows;
  s.s_keep = reinterpret_cast<uint32_t*>(s.wstat);  // the two are never live together
  float* f = reinterpret_cast<float*>(s.wstat + kVjpRows * kVjpWarps);
  s.ulut = f;            f += kVjpRows * ngroups * 16;
  s.glut = f;            f += 64;
  s.s_q = reinterpret_cast<int*>(f);        f += kVjpRows;
  s.s_qold = reinterpret_cast<int*>(f);     f += kVjpRows;
  s.s_k = reinterpret_cast<int*>(f);        f += kWinCols;
  s.s_kold = reinterpret_cast<int*>(f);     f += kWinCols;
  s.s_vb = reinterpret_cast<uint32_t*>(f);  f += kWinCols;
  s.s_h1 = reinterpret_cast<uint32_t*>(f);  f += kWinCols;
  s.rest = f;
  return s;
}

// Fills the symbol / value-bit / hash windows of one block.  Out-of-range entries are 0.
template <bool kSmallDv>
__device__ __forceinline__ void fill_block_windows(const SweepSmem& sm, const Item& it,
                                                   const int32_t* __restrict__ q,
                                                   const int32_t* __restrict__ k,
                                                   const uint32_t* __restrict__ vb, int i0,
                                                   int nrows, int jwin0, int ncols, bool windowed,
                                                   int W, bool want_hash) {
  const int tid = threadIdx.x;
  if (tid < nrows) {
    const int i = i0 + tid;
    sm.s_q[tid] = __ldg(q + i);
    sm.s_qold[tid] = (windowed && i - W - 1 >= 0) ? __ldg(q + i - W - 1) : 0;
  }
  for (int c = tid; c < ncols; c += kVjpBand) {
    const int j = jwin0 + c;
    const bool in = j >= 0 && j < it.len - 1;  // a key column of some cell
    sm.s_k[c] = in ? __ldg(k + j) : 0;
    const int jo = j - W - 1;
    sm.s_kold[c] = (windowed && jo >= 0 && jo < it.len) ? __ldg(k + jo) : 0;
    if (kSmallDv) sm.s_vb[c] = in ? __ldg(vb + j + 1) : 0u;
    if (want_hash) sm.s_h1[c] = dropout_route_open((uint32_t)(j + 1));
  }
}

// Forward step of one diagonal: gate, window product, evidence.  Inactive cells (before the
// diagonal starts) leave S and hs at zero.  With kSkipDeadWindow the exponential of the window
// product is skipped when no lane of the warp has a sum small enough to survive flush-to-zero
// (all lanes of the warp must then call together); that pays where the special-function unit
// is loaded (sweep 2) and costs where integer issue binds (sweep 1).
template <bool kSkipDeadWindow>
__device__ __forceinline__ float forward_cell(float& S, int& hs, bool act, int qi, int kj,
                                              int qold, int kold, int j, const float* glut,
                                              bool windowed, int W, float neg_md, int hs_cut) {
  const int ham = __popc(qi ^ kj);
  const float x = glut[ham];
  float P = 0.0f;
  if (windowed) {
    hs += act ? ham : 0;
    hs -= (j > W) ? __popc(qold ^ kold) : 0;
    if (!kSkipDeadWindow || __any_sync(0xffffffffu, j >= W && hs <= hs_cut)) {
      const float pw = __expf(neg_md * (float)hs);
      P = (j >= W) ? pw : 0.0f;
    }
  }
  const float Sn = x * (1.0f + S) - P;
  S = act ? Sn : 0.0f;
  return P;
}

template <bool kSmallDv>
__device__ __forceinline__ float cell_utility(const VjpArgs& a, const Item& it,
                                              const SweepSmem& sm,
                                              const uint32_t* __restrict__ vb, bool act, int i,
                                              int j, int r, int c, int ngroups) {
  if (kSmallDv) {
    const uint32_t bits = sm.s_vb[c];
    const float* lut = sm.ulut + r * ngroups * 16;
    float u = 0.0f;
    for (int g = 0; g < ngroups; ++g) u += lut[g * 16 + ((bits >> (4 * g)) & 15u)];
    return u;
  } else {
    return act ? route_utility<false>(a, it, vb, i, r, j + 1, ngroups, sm.ulut) : 0.0f;
  }
}

// ------------------------------------------------------------------- sweep 1
// kFixedRef: the row reference of the online softmax is the analytic upper bound of the
// logits (valid while scale * c * (sqrt(1 + W) - 1) stays far inside the float exponent
// range), so no maximum has to be reduced and four rows share one transposing reduction.
// NG: number of 4-wide value groups (compile time) when Dv <= 32, 0 for the generic path.
template <int NG, bool kFixedRef, bool kWindowed, bool kDropout>
__global__ void __launch_bounds__(kVjpBand) vjp_sweep1_kernel(VjpArgs a) {
  constexpr bool kSmallDv = NG > 0;
  extern __shared__ float4 smem_raw[];
  const int ngroups = NG;
  SweepSmem sm = carve_common(reinterpret_cast<float*>(smem_raw), ngroups);
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
  const float scale = a.scale, inv_keep = a.inv_keep;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const int hs_cut = window_sum_cutoff(neg_md);
  constexpr bool windowed = kWindowed;
  constexpr bool use_dropout = kDropout;
  const DropoutKey dkey = make_dropout_key((uint32_t)it.h + a.head_offset,
                                           (uint32_t)it.seq + a.batch_offset, a.seed, a.dropout_p);
  const float ref_top = scale * kSqrtScale * (sqrtf(1.0f + (float)W) - 1.0f);
  const float logit_mul = kSqrtScale * scale;
  // exp(logit - ref_top) as one fused multiply-add and a base-2 exponential of sqrt(1 + S)
  const float mul2 = logit_mul * 1.4426950408889634f;
  const float bias2 = -(logit_mul + ref_top) * 1.4426950408889634f;
  if (tid <= a.D) sm.glut[tid] = expf(neg_md * (float)tid);

  // one cell of the forward sweep: returns (e, e * d * u) and, with dropout, the keep flag
  auto cell = [&](bool act, int r, int c, int j, int i, uint32_t qword, float& S, int& hs,
                  float& e, float& edu, bool& keep) {
    forward_cell<false>(S, hs, act, sm.s_q[r], sm.s_k[c], sm.s_qold[r], sm.s_kold[c], j, sm.glut,
                        windowed, W, neg_md, hs_cut);
    // the log i term cancels in the softmax, so the fixed reference drops it too
    const float ex = exp2f(fmaf(sqrtf(1.0f + S), mul2, bias2));
    e = act ? ex : 0.0f;
    float du;
    if (kSmallDv) {
      const uint32_t bits = sm.s_vb[c];
      const float* lut = sm.ulut + r * NG * 16;
      du = 0.0f;
#pragma unroll
      for (int g = 0; g < NG; ++g) du += lut[g * 16 + ((bits >> (4 * g)) & 15u)];
    } else {
      du = act ? route_utility<false>(a, it, vb, i, r, j + 1, ngroups, sm.ulut) : 0.0f;
    }
    keep = true;
    if (kDropout) {
      keep = act && dropout_keep_open(dkey, sm.s_h1[c], qword);
      du = keep ? du * inv_keep : 0.0f;
    }
    edu = e * du;
  };

  for (int w = it.w_begin; w < it.w_end; ++w) {
    const int dmin = 1 + w * kVjpBand;
    const int dmax = dmin + kVjpBand - 1;
    const int delta = dmin + tid;
    const bool valid = delta <= it.len - 1;
    float S = 0.0f;
    int hs = 0;
    const int rb_lo = dmin / kVjpRows, rb_hi = (it.len - 1) / kVjpRows;
    const int64_t ck_band = it.ck_base + vjp_ck_before(it.len, w);
    for (int rb = rb_lo; rb <= rb_hi; ++rb) {
      const int i0 = max(rb * kVjpRows, dmin), i1 = min(rb * kVjpRows + kVjpRows - 1, it.len - 1);
      const int nrows = i1 - i0 + 1;
      const int jwin0 = i0 - dmax;
      const int64_t ck_idx = ck_band + (rb - rb_lo);
      __syncthreads();
      fill_block_windows<kSmallDv>(sm, it, q, k, vb, i0, nrows, jwin0, nrows + kVjpBand - 1, windowed, W,
                                   use_dropout);
      if (tid < nrows) sm.rstat[tid].w = logf((float)(i0 + tid));
      if (kSmallDv) build_ulut(a, it, i0, nrows, ngroups, sm.ulut);
      __syncthreads();
      a.ckpt[ck_idx * kVjpBand + tid] = make_int2(__float_as_int(S), hs);
      uint32_t* keep_out = a.keepbits + (ck_idx * kVjpRows) * kVjpWarps + warp;
      // first row of the block on which this diagonal exists
      const int r_first = valid ? max(0, delta - i0) : nrows;
      const int cbase = kVjpBand - 1 - tid;   // column window index on block row 0
      const int jbase = i0 - delta;           // key column on block row 0
      const int vslot = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
      const uint32_t qword0 = dropout_query_word((uint32_t)i0);

      if (kFixedRef && nrows == kVjpRows) {
        // full block: four rows per transposing reduction, no tail handling
#pragma unroll 1
        for (int r0 = 0; r0 < kVjpRows; r0 += 4) {
          float v[8];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r = r0 + rr;
            bool keep;
            // a full block starts on a multiple of kVjpRows, so the row index xors in
            cell(r >= r_first, r, cbase + r, jbase + r, i0 + r, qword0 ^ (uint32_t)r, S, hs,
                 v[2 * rr], v[2 * rr + 1], keep);
            if (kDropout) {
              const uint32_t bits = __ballot_sync(0xffffffffu, keep);
              if (lane == 0) keep_out[r * kVjpWarps] = bits;
            }
          }
          const float total = warp_reduce8(v, lane);
          if ((lane & 3) == 0)
            reinterpret_cast<float*>(sm.wstat + (r0 + (vslot >> 1)) * kVjpWarps + warp)[1 + (vslot & 1)] =
                total;
        }
      } else if (kFixedRef) {
        for (int r0 = 0; r0 < nrows; r0 += 4) {
          float v[8];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int r = min(r0 + rr, nrows - 1);       // clamped: the tail repeats a row, masked
            const bool in = r0 + rr < nrows;
            bool keep = false;
            float e = 0.0f, edu = 0.0f;
            if (in)
              cell(r >= r_first, r, cbase + r, jbase + r, i0 + r,
                   dropout_query_word((uint32_t)(i0 + r)), S, hs, e, edu, keep);
            if (kDropout) {
              const uint32_t bits = __ballot_sync(0xffffffffu, in && keep);
              if (lane == 0 && in) keep_out[r * kVjpWarps] = bits;
            }
            v[2 * rr] = e;
            v[2 * rr + 1] = edu;
          }
          const float total = warp_reduce8(v, lane);
          if ((lane & 3) == 0) {
            const int r = r0 + (vslot >> 1);
            if (r < nrows)
              reinterpret_cast<float*>(sm.wstat + r * kVjpWarps + warp)[1 + (vslot & 1)] = total;
          }
        }
      } else {
        for (int r = 0; r < nrows; ++r) {
          const bool act = r >= r_first;
          const int c = cbase + r, j = jbase + r, i = i0 + r;
          forward_cell<false>(S, hs, act, sm.s_q[r], sm.s_k[c], sm.s_qold[r], sm.s_kold[c], j,
                              sm.glut, windowed, W, neg_md, hs_cut);
          const float logit = act ? kSqrtScale * (sqrtf(1.0f + S) - 1.0f) * scale - sm.rstat[r].w
                                  : -CUDART_INF_F;
          float du = cell_utility<kSmallDv>(a, it, sm, vb, act, i, j, r, c, ngroups);
          if (use_dropout) {
            const bool keep =
                act && dropout_keep_open(dkey, sm.s_h1[c], dropout_query_word((uint32_t)i));
            const uint32_t bits = __ballot_sync(0xffffffffu, keep);
            if (lane == 0) keep_out[r * kVjpWarps] = bits;
            du = keep ? du * inv_keep : 0.0f;
          }
          const float mw = warp_max(logit);
          const float e = act ? __expf(logit - mw) : 0.0f;
          const float zw = warp_sum(e);
          const float ew = warp_sum(e * du);
          if (lane == 0) sm.wstat[r * kVjpWarps + warp] = make_float4(mw, zw, ew, 0.0f);
        }
      }
      __syncthreads();
      if (tid < nrows) {
        float m = -CUDART_INF_F, z = 0.0f, e = 0.0f;
        if (kFixedRef) {
          m = ref_top - sm.rstat[tid].w;
#pragma unroll
          for (int ww = 0; ww < kVjpWarps; ++ww) {
            const float4 p = sm.wstat[tid * kVjpWarps + ww];
            z += p.y;
            e += p.z;
          }
        } else {
#pragma unroll
          for (int ww = 0; ww < kVjpWarps; ++ww) {
            const float4 p = sm.wstat[tid * kVjpWarps + ww];
            merge_stats(m, z, e, p.x, p.y, p.z);
          }
        }
        const int64_t slot = it.rowslot + i0 + tid;
        if (w > it.w_begin) {
          const float4 prev = a.stat_part[slot];
          merge_stats(m, z, e, prev.x, prev.y, prev.z);
        }
        a.stat_part[slot] = make_float4(m, z, e, 0.0f);
      }
    }
  }
}

// --------------------------------------------------------------- row statistics
// One thread per (token, head): merges the per-item partials with the null route.
__global__ void vjp_rowstats_kernel(VjpArgs a) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.N * a.H) return;
  const int h = (int)(idx / a.N);
  const int64_t token = idx - (int64_t)h * a.N;
  int start, len;
  const int seq = find_segment(a.plan, token, &start, &len);
  float4 out = make_float4(0.5f * a.scale, 1.0f, 0.0f, 0.0f);
  if (seq >= 0) {
    const int i = (int)(token - start);
    if (i >= 1) {
      const int nitems = a.plan.item_prefix[seq + 1] - a.plan.item_prefix[seq];
      const int64_t base = a.plan.row_prefix[seq] * a.H + (int64_t)h * nitems * (int64_t)len;
      float m = 0.5f * a.scale, z = 1.0f, e = 0.0f;  // the null route
      for (int t = 0; t < nitems && 1 + (int64_t)t * a.plan.item_diagonals <= i; ++t) {
        const float4 p = a.stat_part[base + (int64_t)t * len + i];
        merge_stats(m, z, e, p.x, p.y, p.z);
      }
      out = make_float4(m, 1.0f / z, e / z, logf((float)i));
    }
  }
  a.rowstat[idx] = out;
}

// ------------------------------------------------------------------- sweep 2
// The per-cell work that does not depend on the adjoint chain: probability, dropout
// multiplier, utility, dS.  Returns dS and writes p*d.  Inactive cells give zeros.
template <bool kSmallDv>
__device__ __forceinline__ float cell_adjoint_seed(const VjpArgs& a, const Item& it,
                                                   const SweepSmem& sm,
                                                   const uint32_t* __restrict__ vb, bool act,
                                                   int i, int j, int r, int c, int lane, int warp,
                                                   int ngroups, bool use_dropout, float scale,
                                                   float inv_keep, float Sv, float* pd_out) {
  const float4 st = sm.rstat[r];
  const float sq = sqrtf(1.0f + Sv);
  const float logit = kSqrtScale * (sq - 1.0f) * scale - st.w;
  const float pr = act ? __expf(logit - st.x) * st.y : 0.0f;
  float dmul = 1.0f;
  if (use_dropout) dmul = (sm.s_keep[r * kVjpWarps + warp] >> lane & 1u) ? inv_keep : 0.0f;
  const float u = cell_utility<kSmallDv>(a, it, sm, vb, act, i, j, r, c, ngroups);
  const float pd = pr * dmul;
  *pd_out = pd;
  const float dlogit = pd * u - pr * st.z;
  return scale * dlogit * (0.5f * kSqrtScale) * __frcp_rn(sq);
}

template <int DPAD, int DVPAD, bool kSmallDv>
__global__ void __launch_bounds__(kVjpBand, 2) vjp_sweep2_kernel(VjpArgs a) {
  extern __shared__ float4 smem_raw[];
  const int ngroups = kSmallDv ? (a.Dv + 3) / 4 : 0;
  SweepSmem sm = carve_common(reinterpret_cast<float*>(smem_raw), ngroups);
  float* Cbuf = sm.rest;                               // [kVjpRows][kVjpBand]; S, then C
  float* Pbuf = Cbuf + kVjpRows * kVjpBand;            // [kVjpRows][kVjpBand]; P, then p*d
  float* kz = Pbuf + kVjpRows * kVjpBand;              // [kWinCols][DPAD]
  float* qz = kz + kWinCols * DPAD;                    // [kVjpRows][DPAD]
  float* gob = qz + kVjpRows * DPAD;                   // [kVjpRows][DVPAD]

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
  const int W = a.W, D = a.D, mask = a.mask, ring_slots = a.ring_slots;
  const float scale = a.scale, inv_keep = a.inv_keep;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const int hs_cut = window_sum_cutoff(neg_md);
  const bool windowed = W <= it.len - 2;
  const bool use_dropout = a.dropout_p > 0.0f;
  const float4* __restrict__ rowstat = a.rowstat + (int64_t)it.h * a.N + it.start;
  float* ring = ring_slots ? a.ring + it.item_linear * (int64_t)ring_slots * kVjpBand + tid
                           : nullptr;
  if (tid <= D) sm.glut[tid] = expf(neg_md * (float)tid);

  for (int w = it.w_begin; w < it.w_end; ++w) {
    const int dmin = 1 + w * kVjpBand;
    const int dmax = dmin + kVjpBand - 1;
    const int delta = dmin + tid;
    const bool valid = delta <= it.len - 1;
    const int rb_lo = dmin / kVjpRows, rb_hi = (it.len - 1) / kVjpRows;
    const int64_t ck_band = it.ck_base + vjp_ck_before(it.len, w);
    double Sbar = 0.0, Y = 0.0;
    float xnext = 0.0f;
    int live = 0;
    bool ring_dirty = false;
    int slot = (valid && ring_slots) ? (it.len - 1 - delta) % ring_slots : 0;

    for (int rb = rb_hi; rb >= rb_lo; --rb) {
      const int i0 = max(rb * kVjpRows, dmin), i1 = min(rb * kVjpRows + kVjpRows - 1, it.len - 1);
      const int nrows = i1 - i0 + 1;
      const int jwin0 = i0 - dmax;  // first key column of the block's column window
      const int64_t ck_idx = ck_band + (rb - rb_lo);
      __syncthreads();
      // ---- block tables
      fill_block_windows<kSmallDv>(sm, it, q, k, vb, i0, nrows, jwin0, nrows + kVjpBand - 1, windowed, W,
                                   false);
      if (tid < nrows) sm.rstat[tid] = rowstat[i0 + tid];
      if (use_dropout && tid < nrows * kVjpWarps)
        sm.s_keep[tid] = a.keepbits[(ck_idx * kVjpRows) * kVjpWarps + tid];
      if (kSmallDv) build_ulut(a, it, i0, nrows, ngroups, sm.ulut);
      const int2 ck = a.ckpt[ck_idx * kVjpBand + tid];
      __syncthreads();
      if (mask & 2)
        for (int e = tid; e < nrows * DPAD; e += kVjpBand) {
          const int r = e / DPAD, d = e - r * DPAD;
          qz[e] = d < D ? ((sm.s_q[r] >> d & 1) ? 1.0f : -1.0f) : 0.0f;
        }
      if (mask & 1)
        for (int e = tid; e < (nrows + kVjpBand - 1) * DPAD; e += kVjpBand) {
          const int c = e / DPAD, d = e - c * DPAD;
          const int j = jwin0 + c;
          kz[e] = (d < D && j >= 0 && j < it.len - 1) ? ((sm.s_k[c] >> d & 1) ? 1.0f : -1.0f)
                                                      : 0.0f;
        }
      // ---- phase A: forward recurrence of the block from its checkpoint
      float S = __int_as_float(ck.x);
      int hs = ck.y;
      const int r_first = valid ? max(0, delta - i0) : nrows;
      const int cbase = kVjpBand - 1 - tid, jbase = i0 - delta;
      bool has_p = false;
#pragma unroll 4
      for (int r = 0; r < nrows; ++r) {
        const int c = cbase + r;
        const float P = forward_cell<true>(S, hs, r >= r_first, sm.s_q[r], sm.s_k[c], sm.s_qold[r],
                                           sm.s_kold[c], jbase + r, sm.glut, windowed, W, neg_md,
                                           hs_cut);
        has_p |= P != 0.0f;
        Cbuf[r * kVjpBand + tid] = S;
        Pbuf[r * kVjpBand + tid] = P;
      }
      // ---- phase B: adjoint recurrence, rows descending
      const bool warp_p = ring != nullptr && __any_sync(0xffffffffu, has_p);
      if (!warp_p && live == 0) {
        // no window product is alive in this warp: P = 0, T = 0, Y = 0, C = S * Sbar
#pragma unroll 4
        for (int r = nrows - 1; r >= 0; --r) {
          const bool act = r >= r_first;
          const int c = cbase + r;
          const float Sv = Cbuf[r * kVjpBand + tid];
          const float x = sm.glut[__popc(sm.s_q[r] ^ sm.s_k[c])];
          float pd;
          const float dS = cell_adjoint_seed<kSmallDv>(a, it, sm, vb, act, i0 + r, jbase + r, r, c,
                                                       lane, warp, ngroups, use_dropout, scale,
                                                       inv_keep, Sv, &pd);
          Sbar = (double)dS + (double)xnext * Sbar;     // inactive: dS = 0 above the diagonal
          Cbuf[r * kVjpBand + tid] = act ? (float)((double)Sv * Sbar) : 0.0f;
          Pbuf[r * kVjpBand + tid] = pd;
          xnext = x;
        }
        if (valid && ring_slots) {  // keep the ring cursor in step with the rows walked
          slot -= (nrows - r_first) % ring_slots;
          if (slot < 0) slot += ring_slots;
        }
      } else {
        for (int r = nrows - 1; r >= 0; --r) {
          const bool act = r >= r_first;
          const int c = cbase + r;
          const float Sv = Cbuf[r * kVjpBand + tid];
          const float P = Pbuf[r * kVjpBand + tid];
          const float x = sm.glut[__popc(sm.s_q[r] ^ sm.s_k[c])];
          float pd;
          const float dS = cell_adjoint_seed<kSmallDv>(a, it, sm, vb, act, i0 + r, jbase + r, r, c,
                                                       lane, warp, ngroups, use_dropout, scale,
                                                       inv_keep, Sv, &pd);
          float Cv = 0.0f;
          double T = 0.0;
          if (act) {
            Sbar = (double)dS + (double)xnext * Sbar;
            T = Sbar * (double)P;
          }
          const bool any_p = __any_sync(0xffffffffu, P != 0.0f);
          if (any_p) {
            live = W + 2;
            ring_dirty = true;
          }
          if (live > 0) {
            if (act) {
              const float tf = (float)T;
              const float old = ring[(int64_t)slot * kVjpBand];
              ring[(int64_t)slot * kVjpBand] = tf;
              Y += (double)tf - (double)old;
            }
            if (--live == 0) Y = 0.0;
          }
          if (act) {
            Cv = (float)((double)(Sv + P) * Sbar - Y);
            xnext = x;
            slot = slot == 0 ? ring_slots - 1 : slot - 1;
          }
          Cbuf[r * kVjpBand + tid] = Cv;
          Pbuf[r * kVjpBand + tid] = pd;
        }
      }
      __syncthreads();
      // ---- phase C: contract the block tiles
      if (mask & 1) {  // dQz[i] += sum_j C(i, j) kz[j]
        for (int r = warp; r < nrows; r += kVjpWarps) {
          float acc[DPAD < 8 ? 8 : DPAD];
#pragma unroll
          for (int d = 0; d < (DPAD < 8 ? 8 : DPAD); ++d) acc[d] = 0.0f;
#pragma unroll
          for (int cc = 0; cc < kVjpBand / 32; ++cc) {
            const int t = lane + 32 * cc;
            const float cv = Cbuf[r * kVjpBand + t];
            const float4* kr =
                reinterpret_cast<const float4*>(kz + (r + kVjpBand - 1 - t) * DPAD);
#pragma unroll
            for (int d4 = 0; d4 < DPAD / 4; ++d4) {
              const float4 kk = kr[d4];
              acc[4 * d4 + 0] += cv * kk.x;
              acc[4 * d4 + 1] += cv * kk.y;
              acc[4 * d4 + 2] += cv * kk.z;
              acc[4 * d4 + 3] += cv * kk.w;
            }
          }
          const int slot8 = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
#pragma unroll
          for (int d0 = 0; d0 < (DPAD < 8 ? 8 : DPAD); d0 += 8) {
            float v[8];
#pragma unroll
            for (int d = 0; d < 8; ++d) v[d] = acc[d0 + d];
            const float total = warp_reduce8(v, lane);
            const int d = d0 + slot8;
            if ((lane & 3) == 0 && d < D) {
              float* dst = a.dq_part + (it.rowslot + i0 + r) * D + d;
              *dst = (w == it.w_begin) ? total : *dst + total;
            }
          }
        }
      }
      if (mask & 6) {  // column sums: dKz[j] += sum_i C(i,j) qz[i];  dVz[j+1] += sum_i pd gO(i)
        const int ncols = nrows + kVjpBand - 1;
        for (int dv0 = 0; dv0 < ((mask & 4) ? a.Dv : 1); dv0 += DVPAD) {
          if (mask & 4) {
            if (dv0 > 0) __syncthreads();
            for (int e = tid; e < nrows * DVPAD; e += kVjpBand) {
              const int r = e / DVPAD, d = e - r * DVPAD;
              gob[e] = (dv0 + d < a.Dv)
                           ? load_as_float(a.go,
                                           (((int64_t)it.start + i0 + r) * a.H + it.h) * a.Dv +
                                               dv0 + d,
                                           a.dtype)
                           : 0.0f;
            }
            __syncthreads();
          }
          const bool do_k = (mask & 2) && dv0 == 0, do_v = (mask & 4) != 0;
          for (int c = tid; c < ncols; c += kVjpBand) {
            const int j = jwin0 + c;
            if (j < 0 || j > it.len - 1 - dmin) continue;
            float acck[DPAD], accv[DVPAD];
#pragma unroll
            for (int d = 0; d < DPAD; ++d) acck[d] = 0.0f;
#pragma unroll
            for (int d = 0; d < DVPAD; ++d) accv[d] = 0.0f;
            // every thread walks the same rows so that a warp reads one tile row at a
            // time (consecutive columns = consecutive diagonals, no bank conflicts);
            // cells outside the band are masked to zero instead of branched around
            const int tbase = kVjpBand - 1 - c;   // diagonal slot of (row 0, column j)
#pragma unroll 4
            for (int r = 0; r < nrows; ++r) {
              const int t = tbase + r;
              const bool in = (unsigned)t < (unsigned)kVjpBand;
              const int off = r * kVjpBand + (in ? t : 0);
              if (do_k) {
                const float cv = in ? Cbuf[off] : 0.0f;
                const float4* qr = reinterpret_cast<const float4*>(qz + r * DPAD);
#pragma unroll
                for (int d4 = 0; d4 < DPAD / 4; ++d4) {
                  const float4 qq = qr[d4];
                  acck[4 * d4 + 0] += cv * qq.x;
                  acck[4 * d4 + 1] += cv * qq.y;
                  acck[4 * d4 + 2] += cv * qq.z;
                  acck[4 * d4 + 3] += cv * qq.w;
                }
              }
              if (do_v) {
                const float pv = in ? Pbuf[off] : 0.0f;
                const float4* gr = reinterpret_cast<const float4*>(gob + r * DVPAD);
#pragma unroll
                for (int d4 = 0; d4 < DVPAD / 4; ++d4) {
                  const float4 gg = gr[d4];
                  accv[4 * d4 + 0] += pv * gg.x;
                  accv[4 * d4 + 1] += pv * gg.y;
                  accv[4 * d4 + 2] += pv * gg.z;
                  accv[4 * d4 + 3] += pv * gg.w;
                }
              }
            }
            // the first block (from the bottom) that touches column j writes, later ones add
            const int i_top = min(j + dmax, it.len - 1);
            const bool first = (w == it.w_begin) && (rb == i_top / kVjpRows);
            if (do_k) {
              float* dst = a.dk_part + (it.rowslot + j) * D;
#pragma unroll
              for (int d = 0; d < DPAD; ++d)
                if (d < D) accumulate_row1(dst + d, first, acck[d]);
            }
            if (do_v) {
              float* dst = a.dv_part + (it.rowslot + j + 1) * a.Dv + dv0;
#pragma unroll
              for (int d = 0; d < DVPAD; ++d)
                if (dv0 + d < a.Dv) accumulate_row1(dst + d, first, accv[d]);
            }
          }
        }
      }
    }
    // leave the ring zeroed for the next band of this item
    if (ring != nullptr && ring_dirty && w + 1 < it.w_end) {
      for (int s = 0; s < ring_slots; ++s) ring[(int64_t)s * kVjpBand] = 0.0f;
    }
  }
}

// ------------------------------------------------- sweep 2 on the tensor core
// Same schedule as vjp_sweep2_kernel, but the three block contractions
//     dKz[j] += sum_i C(i,j) qz[i]      dVz[j+1] += sum_i (p d)(i,j) gO(i)      dQz[i] += sum_j C(i,j) kz[j]
// run as tcgen05.mma with fp32 accumulators in tensor memory.  The adjoint phase writes C as
// three bf16 terms (24 mantissa bits) and p*d as two (the +-1 operands are exact) into one
// un-skewed [row][window column] operand area made of 8x16-byte core matrices.  The same bytes
// are read MN-major (M = 128 window columns, K = the 16 block rows) for the column sums and
// K-major (M = rows, K = window columns) for the row sums.  The 271-column window is covered by
// the chunks [0,128), [128,256) and [144,272); only columns >= 256 of the last chunk are used.
namespace tcl {
// Core matrices are ordered [column group][term][row group]: each of the 34 column groups holds
// ten 8-row core matrices -- C high, C low, C third term, p*d high, p*d low, two row groups each
// -- 144 bytes apart (128-byte core + 16 bytes of skew against bank conflicts).  Read K-major
// with M = 64, the first six of them are the 48 rows (hi; lo; third term) of ONE row-sum
// operand: a single MMA per k-step multiplies all three terms of C by kz, the three 16-row
// slices of the accumulator are added on read-back.  (Rows 48-63 alias the p*d cores: finite
// values in accumulator rows nobody reads.)
constexpr int kRowGroupBytes = 144;
constexpr int kTermBytes = (kVjpRows / 8) * kRowGroupBytes;          // one term of one column group
// 16 bytes of padding make the column-group stride 364 words = 12 (mod 32): a warp's row of 32
// consecutive columns touches up to five column groups, whose 16-byte rows then fall into
// five disjoint sets of four banks
constexpr int kColGroupBytes = 5 * kTermBytes + 16;
constexpr int kOperandBytes = (kWinCols / 8) * kColGroupBytes;       // all five terms
__host__ __device__ constexpr int chunk_start(int ch) { return ch == 0 ? 0 : ch == 1 ? 128 : kWinCols - 128; }
static_assert(kVjpRows == 16, "one MMA k-step spans exactly the 16 rows of a block");
__device__ __forceinline__ int tile_off(int r, int c) {
  return (r >> 3) * kRowGroupBytes + (c >> 3) * kColGroupBytes + (r & 7) * 16 + (c & 7) * 2;
}
// B operand tiles, K-major: element (n, k) of an N x K matrix
__device__ __forceinline__ int b_off(int n, int k, int N) {
  return (k >> 3) * (N / 8 * 128) + (n >> 3) * 128 + (n & 7) * 16 + (k & 7) * 2;
}
__device__ __forceinline__ void store_split(unsigned char* hi, unsigned char* lo, int off,
                                            float v) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
  *reinterpret_cast<__nv_bfloat16*>(hi + off) = h;
  *reinterpret_cast<__nv_bfloat16*>(lo + off) = l;
}
// three-term split: v = hi + lo + lo2 to 24 mantissa bits.  The row sums dQz = C kz add
// thousands of terms that largely cancel (the logit adjoints of a row sum to zero), so their
// operand keeps full float32 precision; the column sums use the first two terms.
__device__ __forceinline__ void store_split3(unsigned char* hi, unsigned char* lo,
                                             unsigned char* lo2, int off, float v) {
  const __nv_bfloat16 h = __float2bfloat16_rn(v);
  const float r1 = v - __bfloat162float(h);
  const __nv_bfloat16 l = __float2bfloat16_rn(r1);
  const __nv_bfloat16 l2 = __float2bfloat16_rn(r1 - __bfloat162float(l));
  *reinterpret_cast<__nv_bfloat16*>(hi + off) = h;
  *reinterpret_cast<__nv_bfloat16*>(lo + off) = l;
  *reinterpret_cast<__nv_bfloat16*>(lo2 + off) = l2;
}
}  // namespace tcl

// floats of one set of block tables of the tensor-core kernel: the common tables, the block's
// grad_output rows as float [kVjpRows][NV] and its checkpoints as int2 [kVjpBand]
__host__ __device__ constexpr int tc_table_floats(int ngroups, int NV) {
  return 4 * kVjpRows + 4 * kVjpRows * kVjpWarps + kVjpRows * ngroups * 16 + 64 + 2 * kVjpRows +
         4 * kWinCols + kVjpRows * NV + 2 * kVjpBand;
}

constexpr bool kSkipTc = true;   // forward phase of the tensor-core kernel skips dead windows

// Shared-memory plan of the tensor-core kernel (bytes from the start of dynamic smem).
template <int NK, int NV>
struct TcSmem {
  static constexpr int kKzSlots = kWinCols / 16 + 2;            // circular k-steps of kz^T
  static constexpr int kKzSlotBytes = NK * 32;                  // [NK][16] bf16
  static constexpr int kQzBytes = NK * kVjpRows * 2;
  static constexpr int kGBytes = NV * kVjpRows * 2;
  static constexpr int oQz = tcl::kOperandBytes;                // two buffers
  static constexpr int oGhi = oQz + 2 * kQzBytes;               // two buffers
  static constexpr int oGlo = oGhi + 2 * kGBytes;               // two buffers
  static constexpr int oKz = oGlo + 2 * kGBytes;
  static constexpr int oBar = oKz + kKzSlots * kKzSlotBytes;
  static constexpr int oDq = oBar + 16;                         // row-sum terms of two warps
  static constexpr int kDqFloats = 2 * kVjpRows * 16;
  static constexpr int kBytes = oDq + kDqFloats * 4;
};

// Software pipeline per CTA: the MMAs of block b run on the tensor core while the CUDA
// cores fill the tables and run the forward recurrence of block b+1; the accumulators of
// block b are read back just before the adjoint phase of block b+1 overwrites the operand
// tiles.  B operands are double buffered, kz^T is a ring of k-steps keyed by the absolute
// key-column group (consecutive blocks share all but one group).
template <int NK, int NV, int NG, bool kWindowed, bool kDropout>
__global__ void __launch_bounds__(kVjpBand, 2) vjp_sweep2_tc_kernel(VjpArgs a) {
  using L = TcSmem<NK, NV>;
  extern __shared__ float4 smem_raw[];
  unsigned char* sbase = reinterpret_cast<unsigned char*>(smem_raw);
  unsigned char* tChi = sbase;                         // C = hi + lo + lo2 (24 mantissa bits)
  unsigned char* tClo = tChi + tcl::kTermBytes;
  unsigned char* tCl2 = tClo + tcl::kTermBytes;        // third term of C, row sums only
  unsigned char* tPhi = tCl2 + tcl::kTermBytes;        // p*d = hi + lo
  unsigned char* tPlo = tPhi + tcl::kTermBytes;
  float* s_dq = reinterpret_cast<float*>(sbase + L::oDq);
  unsigned char* bKz = sbase + L::oKz;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(sbase + L::oBar);
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(mbar + 1);
  // two sets of block tables (the set of block b+1 is filled while block b computes), then S
  float* tab_base = reinterpret_cast<float*>(sbase + L::kBytes);
  constexpr int kTabFloats = tc_table_floats(NG, NV);
  float* Sbuf = tab_base + 2 * kTabFloats;             // [kVjpRows][kVjpBand] evidence S

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
  const int W = a.W, D = a.D, Dv = a.Dv, mask = a.mask, ring_slots = a.ring_slots;
  const float scale = a.scale, inv_keep = a.inv_keep;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const int hs_cut = window_sum_cutoff(neg_md);
  const bool has_glo = a.dtype != ROSA_B200_BF16;   // bf16 grad_output is exact in one term
  const float4* __restrict__ rowstat = a.rowstat + (int64_t)it.h * a.N + it.start;
  float* ring = ring_slots ? a.ring + it.item_linear * (int64_t)ring_slots * kVjpBand + tid
                           : nullptr;
  // row-sum k-loop: split over NQ issuing threads, one accumulator each (summed on read-back)
  constexpr int NQ = 2;
  constexpr uint32_t kTmemCols = ((3 + NQ) * NK + 3 * NV) <= 128 ? 128 : 256;
  constexpr uint32_t kColK = 0, kColV = 3 * NK, kColQ = 3 * NK + 3 * NV;

  // ---- one-time set-up
  for (int e = tid; e < tcl::kOperandBytes / 16; e += kVjpBand)
    reinterpret_cast<uint4*>(tChi)[e] = make_uint4(0, 0, 0, 0);
  if (tid <= D) {
    const float gate = expf(neg_md * (float)tid);
    carve_common(tab_base, NG).glut[tid] = gate;
    carve_common(tab_base + kTabFloats, NG).glut[tid] = gate;
  }
  if (warp == 0) tc::tmem_alloc(tmem_ptr, kTmemCols);
  if (tid == 0) tc::mbar_init(mbar, 4);   // four issuing threads commit per block
  tc::fence_before_thread_sync();
  __syncthreads();
  tc::fence_after_thread_sync();
  const uint32_t tmem = *tmem_ptr;
  uint32_t mma_phase = 0;
  bool mma_timed_out = false;
  int buf = 0;                       // B-operand buffer of the block being built
  // ---- the blocks of this CTA as one flat sequence: bands ascending, row blocks descending
  struct Geom {
    int w, rb, rb_lo, i0, nrows, jwin, dmin, dmax;
    int64_t ck_idx;
  };
  auto geom_of = [&](int w, int rb) {
    Geom g;
    g.w = w;
    g.rb = rb;
    g.dmin = 1 + w * kVjpBand;
    g.dmax = g.dmin + kVjpBand - 1;
    g.rb_lo = g.dmin / kVjpRows;
    g.i0 = max(rb * kVjpRows, g.dmin);
    g.nrows = min(rb * kVjpRows + kVjpRows - 1, it.len - 1) - g.i0 + 1;
    g.jwin = rb * kVjpRows - g.dmax;             // window start, a multiple of 16
    g.ck_idx = it.ck_base + vjp_ck_before(it.len, w) + (rb - g.rb_lo);
    return g;
  };
  // the block whose MMAs are in flight; its geometry is recomputed when they are collected
  int prev_w = 0, prev_rb = 0;
  bool prev_pending = false;

  // Reads the accumulators of a finished block and adds them to the per-item partials.
  auto epilogue = [&](int block_w, int block_rb) {
    const Geom b = geom_of(block_w, block_rb);
    // A wait that gave up ends this warp's use of the tensor core: nothing accumulated may be
    // trusted, so it issues, waits for and reads back nothing more (its partial rows stay
    // incomplete and the status word tells the host).  The decision is taken per warp (a vote),
    // because the accumulator loads below are warp-wide instructions; the named barriers of the
    // row-sum part are still joined so that no warp waits for one that gave up.
    if (!mma_timed_out && !__all_sync(0xffffffffu, tc::mbar_wait(mbar, mma_phase, 1u << 24)))
      mma_timed_out = true;
    if (mma_timed_out) {
      if ((mask & 1) && warp >= 4 && warp < 7)
        for (int n0 = 0; n0 < NK; n0 += 16) {
          asm volatile("bar.sync 1, 96;" ::: "memory");
          if (n0 + 16 < NK) asm volatile("bar.sync 1, 96;" ::: "memory");
        }
      return;
    }
    mma_phase ^= 1u;
    tc::fence_after_thread_sync();
    const int quarter = warp & 3;
    const uint32_t lane_base = (uint32_t)(32 * quarter) << 16;
    const bool k_half = warp < 4;
    const int ncols = b.nrows + kVjpBand - 1 + (b.i0 - b.rb * kVjpRows);
    if (k_half ? (mask & 2) != 0 : (mask & 4) != 0) {
      const int ncol = k_half ? NK : NV;
      const int dim = k_half ? D : Dv;
      float* part = k_half ? a.dk_part + it.rowslot * D : a.dv_part + (it.rowslot + 1) * Dv;
      const bool vec4 = (dim & 3) == 0;
      if (vec4 && dim <= 8) {
        // Rows of at most 8 components (the common shapes): the partial rows of all chunks are
        // read first, so their latencies overlap instead of chaining load -> add -> store three
        // times.
        float4 prior[3][2];
        float* dst3[3];
        bool use3[3];
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          const int c = tcl::chunk_start(ch) + 32 * quarter + lane;
          const int j = b.jwin + c;
          use3[ch] = (ch < 2 || (quarter == 3 && c >= 256)) && c < ncols && j >= 0 &&
                     j <= it.len - 1 - b.dmin;
          const int i_top = min(j + b.dmax, it.len - 1);
          const bool first = (b.w == it.w_begin) && (b.rb == i_top / kVjpRows);
          dst3[ch] = part + (int64_t)j * dim;
#pragma unroll
          for (int d4 = 0; d4 < 2; ++d4) {
            prior[ch][d4] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (use3[ch] && !first && 4 * d4 < dim)
              prior[ch][d4] = reinterpret_cast<const float4*>(dst3[ch])[d4];
          }
        }
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          if (ch == 2 && quarter < 3) continue;
          float v[16];
          tc::tmem_ld16(tmem + lane_base + (k_half ? kColK + ch * NK : kColV + ch * NV), v);
          if (use3[ch]) {
#pragma unroll
            for (int d4 = 0; d4 < 2; ++d4) {
              if (4 * d4 < dim) {
                float4 o = prior[ch][d4];
                o.x += v[4 * d4 + 0];
                o.y += v[4 * d4 + 1];
                o.z += v[4 * d4 + 2];
                o.w += v[4 * d4 + 3];
                reinterpret_cast<float4*>(dst3[ch])[d4] = o;
              }
            }
          }
        }
      } else
#pragma unroll
      for (int ch = 0; ch < 3; ++ch) {
        // only window columns >= 256 of the last chunk are new: they sit in the last quarter
        if (ch == 2 && quarter < 3) continue;
        const int c = tcl::chunk_start(ch) + 32 * quarter + lane;
        const int j = b.jwin + c;
        const bool use =
            (ch < 2 || c >= 256) && c < ncols && j >= 0 && j <= it.len - 1 - b.dmin;
        const int i_top = min(j + b.dmax, it.len - 1);
        const bool first = (b.w == it.w_begin) && (b.rb == i_top / kVjpRows);
        for (int n0 = 0; n0 < ncol && n0 < dim; n0 += 16) {
          float v[16];
          tc::tmem_ld16(tmem + lane_base + (k_half ? kColK + ch * NK : kColV + ch * NV) + n0, v);
          if (use) {
            float* dst = part + (int64_t)j * dim + n0;
            if (vec4) {
#pragma unroll
              for (int d4 = 0; d4 < 4; ++d4) {
                if (n0 + 4 * d4 < dim) {
                  accumulate_row4(reinterpret_cast<float4*>(dst) + d4, first, v[4 * d4 + 0],
                                  v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
                }
              }
            } else {
#pragma unroll
              for (int d = 0; d < 16; ++d)
                if (n0 + d < dim) accumulate_row1(dst + d, first, v[d]);
            }
          }
        }
      }
    }
    if ((mask & 1) && warp >= 4 && warp < 7) {
      // accumulator rows 0-15 / 16-31 / 32-47 (the three terms of C) sit in lanes 0-15 of the
      // lane quarters 0 / 1 / 2: warps 4, 5, 6 read one each, warp 4 adds them up
      const int term = warp - 4;
      const uint32_t term_base = (uint32_t)(32 * term) << 16;
      for (int n0 = 0; n0 < NK; n0 += 16) {
        float v[16];
        tc::tmem_ld16(tmem + term_base + kColQ + n0, v);
#pragma unroll
        for (int part = 1; part < NQ; ++part) {
          float v2[16];
          tc::tmem_ld16(tmem + term_base + kColQ + part * NK + n0, v2);
#pragma unroll
          for (int d = 0; d < 16; ++d) v[d] += v2[d];
        }
        if (term > 0 && lane < kVjpRows) {
          float4* dst4 = reinterpret_cast<float4*>(s_dq + ((term - 1) * kVjpRows + lane) * 16);
#pragma unroll
          for (int d4 = 0; d4 < 4; ++d4)
            dst4[d4] = make_float4(v[4 * d4], v[4 * d4 + 1], v[4 * d4 + 2], v[4 * d4 + 3]);
        }
        asm volatile("bar.sync 1, 96;" ::: "memory");
        if (term == 0 && lane < b.nrows) {
          const float* lo = s_dq + lane * 16;
          const float* l2 = s_dq + (kVjpRows + lane) * 16;
          float* dst = a.dq_part + (it.rowslot + b.i0 + lane) * D + n0;
#pragma unroll
          for (int d = 0; d < 16; ++d) {
            const float sum = v[d] + lo[d] + l2[d];
            if (n0 + d < D) dst[d] = (b.w == it.w_begin) ? sum : dst[d] + sum;
          }
        }
        if (n0 + 16 < NK) asm volatile("bar.sync 1, 96;" ::: "memory");
      }
    }
    tc::fence_before_thread_sync();
  };

  const int rb_top = (it.len - 1) / kVjpRows;    // bottom row block of every band
  // The route probability of a cell is exp(logit - log i - max) / Z with
  // logit = c * scale * (sqrt(1 + S) - 1); the tables keep it ready for one fused
  // multiply-add and a base-2 exponential: p = exp2(sqrt(1 + S) * mul2 + bias) / Z,
  // bias = -(log i + max) * log2(e) - mul2 stored in place of the row maximum.
  constexpr float kLog2e = 1.4426950408889634f;
  const float mul2 = kSqrtScale * scale * kLog2e;
  auto exponent_bias = [&](float row_max, float log_i) {
    return -(log_i + row_max) * kLog2e - mul2;
  };
  auto go_value = [&](const Geom& g, int e) {
    const int r = e / NV, d = e - r * NV;
    return (d < Dv && r < g.nrows)
               ? load_as_float(a.go, (((int64_t)it.start + g.i0 + r) * a.H + it.h) * Dv + d, a.dtype)
               : 0.0f;
  };
  // The same element as raw bits (zero for padding): the prefetch keeps loads free of dependent
  // instructions, so a warp does not sit on the load latency while it still has work to issue;
  // the conversion happens where the value is stored.
  auto go_bits = [&](const Geom& g, int e) -> uint32_t {
    const int r = e / NV, d = e - r * NV;
    if (!(d < Dv && r < g.nrows)) return 0u;
    const int64_t idx = (((int64_t)it.start + g.i0 + r) * a.H + it.h) * Dv + d;
    return a.dtype == ROSA_B200_F32 ? static_cast<const uint32_t*>(a.go)[idx]
                                    : (uint32_t) static_cast<const uint16_t*>(a.go)[idx];
  };
  auto go_from_bits = [&](uint32_t bits) {
    if (a.dtype == ROSA_B200_F32) return __uint_as_float(bits);
    if (a.dtype == ROSA_B200_F16) return __half2float(__ushort_as_half((unsigned short)bits));
    return __uint_as_float(bits << 16);          // bf16 is the upper half of a float
  };
  // straight global -> shared fill of one table set (first block of a band)
  auto fill_direct = [&](const Geom& g, const SweepSmem& t) {
    fill_block_windows<true>(t, it, q, k, vb, g.i0, g.nrows, g.jwin, kWinCols, kWindowed, W, false);
    if (tid < g.nrows) {
      float4 st = rowstat[g.i0 + tid];
      st.x = exponent_bias(st.x, st.w);
      t.rstat[tid] = st;
    }
    if (kDropout && tid < g.nrows * kVjpWarps)
      t.s_keep[tid] = a.keepbits[(g.ck_idx * kVjpRows) * kVjpWarps + tid];
    for (int e = tid; e < kVjpRows * NV; e += kVjpBand) t.rest[e] = go_value(g, e);
    reinterpret_cast<int2*>(t.rest + kVjpRows * NV)[tid] = a.ckpt[g.ck_idx * kVjpBand + tid];
  };

  int w = it.w_begin, rb = rb_top;               // the block being computed
  int tb = 0;                                    // its table set
  fill_direct(geom_of(w, rb), carve_common(tab_base, NG));
  __syncthreads();

  // per-band state of this thread's diagonal
  int delta = 0, live = 0, slot = 0;
  bool valid = false, ring_dirty = false, band_start = true;
  double Sbar = 0.0, Y = 0.0;
  float xnext = 0.0f;

  while (true) {
    const SweepSmem sm = carve_common(tab_base + tb * kTabFloats, NG);
    const SweepSmem nx = carve_common(tab_base + (tb ^ 1) * kTabFloats, NG);
    const float* s_go = sm.rest;                                     // [kVjpRows][NV]
    const int2* s_ck = reinterpret_cast<const int2*>(sm.rest + kVjpRows * NV);
    const Geom g = geom_of(w, rb);
    const int i0 = g.i0, nrows = g.nrows, jwin = g.jwin;
    const int dmin = g.dmin, dmax = g.dmax;
    const int skew = i0 - rb * kVjpRows;         // 1 on the top block of a band, else 0
    if (band_start) {
      delta = dmin + tid;
      valid = delta <= it.len - 1;
      Sbar = 0.0;
      Y = 0.0;
      xnext = 0.0f;
      live = 0;
      ring_dirty = false;
      slot = (valid && ring_slots) ? (it.len - 1 - delta) % ring_slots : 0;
      // the bottom block of a band refills the whole kz^T ring: the last block of the
      // previous band must have released it
      if (prev_pending) {
        epilogue(prev_w, prev_rb);
        prev_pending = false;
      }
    }
    // the block after this one
    const bool next_same = rb > g.rb_lo;
    const bool has_next = next_same || w + 1 < it.w_end;

    unsigned char* bQz = sbase + L::oQz + buf * L::kQzBytes;
    unsigned char* bGhi = sbase + L::oGhi + buf * L::kGBytes;
    unsigned char* bGlo = sbase + L::oGlo + buf * L::kGBytes;

    // ---- prefetch, part 1: the next block of the same band shares all but 16 window columns
    // with this one; its new columns, rows, row statistics, keep ballots, grad_output rows and
    // checkpoints are loaded into registers now and stored after the forward phase, so no
    // global-memory latency is exposed.  One word per thread:
    //   tid   0-15  key symbol            16-31 key symbol leaving the horizon   32-47 value bits
    //        48-63  query symbol          64-127 row statistics (16 x float4)    128-255 keep ballots
    uint32_t pf0 = 0u, pf1 = 0u;
    constexpr int kGoRegs = (kVjpRows * NV + kVjpBand - 1) / kVjpBand;
    uint32_t pgo[kGoRegs];
    int2 pck = make_int2(0, 0);
    if (next_same) {
      const Geom gn = geom_of(w, rb - 1);
      if (tid < 16) {
        const int j = gn.jwin + tid;
        pf0 = (j >= 0 && j < it.len - 1) ? (uint32_t)__ldg(k + j) : 0u;
        const int io = gn.i0 + tid - W - 1;
        pf1 = (kWindowed && tid < gn.nrows && io >= 0) ? (uint32_t)__ldg(q + io) : 0u;
      } else if (tid < 32) {
        const int jo = gn.jwin + (tid - 16) - W - 1;
        pf0 = (kWindowed && jo >= 0 && jo < it.len) ? (uint32_t)__ldg(k + jo) : 0u;
      } else if (tid < 48) {
        const int j = gn.jwin + (tid - 32);
        pf0 = (j >= 0 && j < it.len - 1) ? __ldg(vb + j + 1) : 0u;
      } else if (tid < 64) {
        const int r = tid - 48;
        pf0 = r < gn.nrows ? (uint32_t)__ldg(q + gn.i0 + r) : 0u;
      } else if (tid < 128) {
        // component e & 3 of row e >> 2 (turned into the exponent bias when it is stored)
        const int e = tid - 64;
        if ((e >> 2) < gn.nrows)
          pf0 = __float_as_uint(reinterpret_cast<const float*>(rowstat + gn.i0)[e]);
      } else if (kDropout) {
        const int e = tid - 128;
        if (e < gn.nrows * kVjpWarps) pf0 = a.keepbits[(gn.ck_idx * kVjpRows) * kVjpWarps + e];
      }
#pragma unroll
      for (int x = 0; x < kGoRegs; ++x) {
        const int e = tid + x * kVjpBand;
        pgo[x] = e < kVjpRows * NV ? go_bits(gn, e) : 0u;
      }
      pck = a.ckpt[gn.ck_idx * kVjpBand + tid];
    }

    // ---- B operands and utility tables of this block (shared memory only)
    if (mask & 2)
      for (int e = tid; e < NK * kVjpRows; e += kVjpBand) {
        const int d = e / kVjpRows, r = e - d * kVjpRows;
        const float v = (d < D && r < nrows) ? ((sm.s_q[r] >> d & 1) ? 1.0f : -1.0f) : 0.0f;
        *reinterpret_cast<__nv_bfloat16*>(bQz + tcl::b_off(d, r, NK)) = __float2bfloat16_rn(v);
      }
    if (mask & 4)
      for (int e = tid; e < NV * kVjpRows; e += kVjpBand) {
        const int d = e / kVjpRows, r = e - d * kVjpRows;
        tcl::store_split(bGhi, bGlo, tcl::b_off(d, r, NV), s_go[r * NV + d]);
      }
    if (mask & 1) {
      // kz^T ring: the bottom block of a band fills every k-step, later blocks only the
      // one key-column group that entered the window
      const int g0 = (jwin + (1 << 20)) >> 4;           // absolute group of window column 0
      const int nfill = band_start ? kWinCols / 16 : 1;
      for (int e = tid; e < nfill * NK * 16; e += kVjpBand) {
        const int ks = e / (NK * 16), rem = e - ks * (NK * 16);
        const int d = rem >> 4, cc = rem & 15;
        const int c = ks * 16 + cc;
        const int j = jwin + c;
        const float v = (d < D && j >= 0 && j < it.len - 1)
                            ? ((sm.s_k[c] >> d & 1) ? 1.0f : -1.0f)
                            : 0.0f;
        const int sl = (g0 + ks) % L::kKzSlots;
        *reinterpret_cast<__nv_bfloat16*>(bKz + sl * L::kKzSlotBytes + tcl::b_off(d, cc, NK)) =
            __float2bfloat16_rn(v);
      }
    }
    // nibble tables ulut[r][g][nib] = sum_b (nib bit b ? +1 : -1) * gO[i0 + r][4 g + b]
    for (int e = tid; e < nrows * NG * 16; e += kVjpBand) {
      const int nib = e & 15, rg = e >> 4;
      const int r = rg / NG, gq = rg - r * NG;
      const float* gv = s_go + r * NV + 4 * gq;
      float sum = 0.0f;
#pragma unroll
      for (int b = 0; b < 4; ++b) sum += (nib >> b & 1) ? gv[b] : -gv[b];
      sm.ulut[e] = sum;
    }

    // ---- phase A: forward recurrence of the block from its checkpoint
    const int2 ck = s_ck[tid];
    float S = __int_as_float(ck.x);
    int hs = ck.y;
    const int r_first = valid ? max(0, delta - i0) : nrows;
    const int cbase = kVjpBand - 1 - tid + skew, jbase = i0 - delta;
    bool has_p = false;
#pragma unroll 4
    for (int r = 0; r < nrows; ++r) {
      const int c = cbase + r;
      const float P = forward_cell<kSkipTc>(S, hs, r >= r_first, sm.s_q[r], sm.s_k[c], sm.s_qold[r],
                                            sm.s_kold[c], jbase + r, sm.glut, kWindowed, W, neg_md,
                                            hs_cut);
      has_p |= P != 0.0f;
      Sbuf[r * kVjpBand + tid] = S;
    }

    // ---- prefetch, part 2: build the next block's tables in the other set
    if (next_same) {
      const int c = tid + 16;                    // the 256 window columns both blocks share
      nx.s_k[c] = sm.s_k[tid];
      nx.s_kold[c] = sm.s_kold[tid];
      nx.s_vb[c] = sm.s_vb[tid];
      if (tid < 16) {
        nx.s_k[tid] = (int)pf0;
        nx.s_qold[tid] = (int)pf1;
      } else if (tid < 32) {
        nx.s_kold[tid - 16] = (int)pf0;
      } else if (tid < 48) {
        nx.s_vb[tid - 32] = pf0;
      } else if (tid < 64) {
        nx.s_q[tid - 48] = (int)pf0;
      } else if (tid < 128) {
        // the maximum (component 0) becomes the exponent bias, which needs log i (component 3)
        // from three lanes up; done here, where the loaded words have arrived
        float comp = __uint_as_float(pf0);
        const float log_i = __shfl_down_sync(0xffffffffu, comp, 3);
        if (((tid - 64) & 3) == 0) comp = exponent_bias(comp, log_i);
        reinterpret_cast<float*>(nx.rstat)[tid - 64] = comp;
      } else if (kDropout) {
        nx.s_keep[tid - 128] = pf0;
      }
#pragma unroll
      for (int x = 0; x < kGoRegs; ++x) {
        const int e = tid + x * kVjpBand;
        if (e < kVjpRows * NV) nx.rest[e] = go_from_bits(pgo[x]);
      }
      reinterpret_cast<int2*>(nx.rest + kVjpRows * NV)[tid] = pck;
    } else if (has_next) {
      fill_direct(geom_of(w + 1, rb_top), nx);
    }

    // ---- the previous block's MMAs have had the whole table/forward phase to finish
    if (prev_pending) epilogue(prev_w, prev_rb);
    // rows of a partial block that do not exist contribute nothing
    for (int r = nrows; r < kVjpRows; ++r) {
      const int off = tcl::tile_off(r, cbase + r);
      tcl::store_split3(tChi, tClo, tCl2, off, 0.0f);
      tcl::store_split(tPhi, tPlo, off, 0.0f);
    }
    __syncthreads();                             // sync 1: the utility tables are complete

    // ---- phase B: adjoint recurrence, rows descending; C and p*d go to the operand tiles
    const bool warp_p = kWindowed && ring != nullptr && __any_sync(0xffffffffu, has_p);
    const float ds_mul = scale * (0.5f * kSqrtScale);
    auto seed = [&](bool act, int r, int c, float Sv, float* pd) {
      const float4 st = sm.rstat[r];                  // (exponent bias, 1/Z, E, log i)
      const float t = 1.0f + Sv;
      const float rs = rsqrtf(t);                     // R'(S) = c / (2 sqrt(1 + S))
      const float pr = act ? exp2f(fmaf(t * rs, mul2, st.x)) * st.y : 0.0f;
      float dmul = 1.0f;
      if (kDropout) dmul = (sm.s_keep[r * kVjpWarps + warp] >> lane & 1u) ? inv_keep : 0.0f;
      const uint32_t bits = sm.s_vb[c];
      const float* lut = sm.ulut + r * NG * 16;
      float u = 0.0f;
#pragma unroll
      for (int gq = 0; gq < NG; ++gq) u += lut[gq * 16 + ((bits >> (4 * gq)) & 15u)];
      *pd = pr * dmul;
      const float dlogit = *pd * u - pr * st.z;
      return ds_mul * dlogit * rs;
    };
    if (!warp_p && live == 0) {
      // No window product is alive in this warp: P = 0, T = 0, Y = 0, C = S * Sbar.  The adjoint
      // recurrence Sbar <- dS + x * Sbar is a contraction here and runs in float32 inside the
      // block; the tile offset walks down the diagonal incrementally.
      float sb = (float)Sbar;
      int c = cbase + nrows - 1;
      int off = tcl::tile_off(nrows - 1, c);
#pragma unroll 4
      for (int r = nrows - 1; r >= 0; --r) {
        const bool act = r >= r_first;
        const float Sv = Sbuf[r * kVjpBand + tid];
        const float x = sm.glut[__popc(sm.s_q[r] ^ sm.s_k[c])];
        float pd;
        const float dS = seed(act, r, c, Sv, &pd);
        sb = fmaf(xnext, sb, dS);
        const float Cv = act ? Sv * sb : 0.0f;
        tcl::store_split3(tChi, tClo, tCl2, off, Cv);
        tcl::store_split(tPhi, tPlo, off, pd);
        xnext = x;
        // one row up, one column left: -16 - 2 inside a core matrix, else hop to the previous
        // row group (-144 + 7 * 16) / column group (-kColGroupBytes + 7 * 2)
        off -= ((r & 7) ? 16 : tcl::kRowGroupBytes - 112) + ((c & 7) ? 2 : tcl::kColGroupBytes - 14);
        --c;
      }
      Sbar = (double)sb;
      if (valid && ring_slots) {
        slot -= (nrows - r_first) % ring_slots;
        if (slot < 0) slot += ring_slots;
      }
    } else {
      // The window product is rebuilt from the mismatch-count sum, walked backwards: hs holds
      // the sum of the window that ends at the current cell (it ended phase A at the last row).
      for (int r = nrows - 1; r >= 0; --r) {
        const bool act = r >= r_first;
        const int c = cbase + r, j = jbase + r;
        const float Sv = Sbuf[r * kVjpBand + tid];
        const int ham = __popc(sm.s_q[r] ^ sm.s_k[c]);
        const float P = (act && j >= W) ? __expf(neg_md * (float)hs) : 0.0f;
        hs += ((act && j > W) ? __popc(sm.s_qold[r] ^ sm.s_kold[c]) : 0) - (act ? ham : 0);
        const float x = sm.glut[ham];
        float pd;
        const float dS = seed(act, r, c, Sv, &pd);
        float Cv = 0.0f;
        double T = 0.0;
        if (act) {
          Sbar = (double)dS + (double)xnext * Sbar;
          T = Sbar * (double)P;
        }
        const bool any_p = __any_sync(0xffffffffu, P != 0.0f);
        if (any_p) {
          live = W + 2;
          ring_dirty = true;
        }
        if (live > 0) {
          if (act) {
            const float tf = (float)T;
            const float old = ring[(int64_t)slot * kVjpBand];
            ring[(int64_t)slot * kVjpBand] = tf;
            Y += (double)tf - (double)old;
          }
          if (--live == 0) Y = 0.0;
        }
        if (act) {
          Cv = (float)((double)(Sv + P) * Sbar - Y);
          xnext = x;
          slot = slot == 0 ? ring_slots - 1 : slot - 1;
        }
        const int off = tcl::tile_off(r, c);
        tcl::store_split3(tChi, tClo, tCl2, off, Cv);
        tcl::store_split(tPhi, tPlo, off, pd);
      }
    }
    // ---- phase C: hand the tiles to the tensor core
    tc::fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();                             // sync 2: tiles, B operands, next tables
    // Four issuing threads (lane 0 of warps 0..3) share the work so that no single warp
    // falls behind the others at the next barrier: warp 0 adds the column sums of C, warp 1
    // those of p*d, and the row-sum k-loop is sliced over the issuers (one accumulator per
    // slice, added in the epilogue).  Each issuer commits once; the mbarrier expects four
    // arrivals.
    if (lane == 0 && warp < 4 && !mma_timed_out) {
      tc::fence_after_thread_sync();
      constexpr uint32_t idK = tc::idesc_bf16_f32(128, NK, true, false);
      constexpr uint32_t idV = tc::idesc_bf16_f32(128, NV, true, false);
      // the row sums need 48 accumulator rows (three terms x 16 block rows): M = 64, whose row r
      // lands in lane 32 * (r / 16) + r % 16
      constexpr uint32_t idQ = tc::idesc_bf16_f32(64, NK, false, false);
      if (warp == 0 && (mask & 2)) {
        const uint64_t dQz = tc::smem_desc(tc::smem_addr(bQz), NK / 8 * 128, 128);
        // MN-major view (column sums): K direction = row groups, M direction = column groups
        const uint64_t mnChi = tc::smem_desc(tc::smem_addr(tChi), tcl::kRowGroupBytes, tcl::kColGroupBytes);
        const uint64_t mnClo = tc::smem_desc(tc::smem_addr(tClo), tcl::kRowGroupBytes, tcl::kColGroupBytes);
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          // advancing the 14-bit start-address field by whole 16-byte units
          const uint64_t shift = (uint64_t)(((tcl::chunk_start(ch) >> 3) * tcl::kColGroupBytes) >> 4);
          tc::mma_bf16(tmem + kColK + ch * NK, mnChi + shift, dQz, idK, false);
          tc::mma_bf16(tmem + kColK + ch * NK, mnClo + shift, dQz, idK, true);
        }
      }
      if (warp == 1 && (mask & 4)) {
        const uint64_t dGhi = tc::smem_desc(tc::smem_addr(bGhi), NV / 8 * 128, 128);
        const uint64_t dGlo = tc::smem_desc(tc::smem_addr(bGlo), NV / 8 * 128, 128);
        const uint64_t mnPhi = tc::smem_desc(tc::smem_addr(tPhi), tcl::kRowGroupBytes, tcl::kColGroupBytes);
        const uint64_t mnPlo = tc::smem_desc(tc::smem_addr(tPlo), tcl::kRowGroupBytes, tcl::kColGroupBytes);
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) {
          const uint64_t shift = (uint64_t)(((tcl::chunk_start(ch) >> 3) * tcl::kColGroupBytes) >> 4);
          tc::mma_bf16(tmem + kColV + ch * NV, mnPhi + shift, dGhi, idV, false);
          tc::mma_bf16(tmem + kColV + ch * NV, mnPlo + shift, dGhi, idV, true);
          if (has_glo) tc::mma_bf16(tmem + kColV + ch * NV, mnPhi + shift, dGlo, idV, true);
        }
      }
      if (warp >= 4 - NQ && (mask & 1)) {
        // K-major view (row sums): K direction = column groups, M direction = the six row
        // groups hi0 hi1 lo0 lo1 l20 l21 of a column group (M = 64: two more alias p*d)
        const uint64_t kC = tc::smem_desc(tc::smem_addr(tChi), tcl::kColGroupBytes, tcl::kRowGroupBytes);
        const uint64_t dKz0 = tc::smem_desc(tc::smem_addr(bKz), NK / 8 * 128, 128);
        constexpr int kSteps = kWinCols / 16;
        const int part = warp - (4 - NQ);                       // this issuer's slice of the k-loop
        const int ks0 = part * kSteps / NQ, ks1 = (part + 1) * kSteps / NQ;
        const uint32_t acc = tmem + kColQ + part * NK;
        const int g0 = (jwin + (1 << 20)) >> 4;
        int sl = (g0 + ks0) % L::kKzSlots;
#pragma unroll 1
        for (int ks = ks0; ks < ks1; ++ks) {
          const uint64_t dKz = dKz0 + (uint64_t)((sl * L::kKzSlotBytes) >> 4);
          const uint64_t shift = (uint64_t)((ks * 2 * tcl::kColGroupBytes) >> 4);
          tc::mma_bf16(acc, kC + shift, dKz, idQ, ks > ks0);
          sl = sl + 1 == L::kKzSlots ? 0 : sl + 1;
        }
      }
      tc::mma_commit(mbar);
    }
    prev_w = w;
    prev_rb = rb;
    prev_pending = true;
    buf ^= 1;
    // leave the ring zeroed for the next band of this item
    if (!next_same && ring != nullptr && ring_dirty && has_next) {
      for (int s = 0; s < ring_slots; ++s) ring[(int64_t)s * kVjpBand] = 0.0f;
    }
    if (!has_next) break;
    band_start = !next_same;
    if (next_same) {
      --rb;
    } else {
      ++w;
      rb = rb_top;
    }
    tb ^= 1;
  }
  if (prev_pending) epilogue(prev_w, prev_rb);
  __syncthreads();
  if (mma_timed_out && lane == 0) atomicExch(a.plan.status + 1, 1);
  if (warp == 0) tc::tmem_dealloc(tmem, kTmemCols);
}

// ------------------------------------------------------------------ finalize
// Sums the per-item partials in item order and applies the softsign Jacobian.
// which: 0 = query, 1 = key, 2 = value.  VEC = 4: a thread owns four consecutive components
// (128-bit loads of the partial rows); VEC = 1 for rows that are not a multiple of four.
template <int VEC>
__global__ void vjp_finalize_kernel(VjpArgs a, int which) {
  const int dim = which == 2 ? a.Dv : a.D;
  const int heads = which == 2 ? a.Hv : a.H;
  const int dimv = dim / VEC;
  // Threads run head-major over (head, token, component): the partial rows of one head and item
  // are contiguous over (token, component), so the reads of a warp coalesce; only the final
  // element access is strided by the head count.
  const int64_t lin = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (lin >= a.N * heads * dimv) return;
  const int hh = (int)(lin / (a.N * dimv));
  const int64_t rem = lin - (int64_t)hh * a.N * dimv;
  const int64_t token = rem / dimv;
  const int d = (int)(rem - token * dimv) * VEC;
  const int64_t idx = (token * heads + hh) * dim + d;
  int start, len;
  const int seq = find_segment(a.plan, token, &start, &len);
  float sum[VEC];
#pragma unroll
  for (int x = 0; x < VEC; ++x) sum[x] = 0.0f;
  // adds `count` partial rows `stride` floats apart, in order, a few loads in flight at a time
  auto add_rows = [&](const float* base, int count, int64_t stride) {
#pragma unroll 4
    for (int t = 0; t < count; ++t) {
      if (VEC == 4) {
        const float4 p = *reinterpret_cast<const float4*>(base + t * stride);
        sum[0] += p.x; sum[VEC > 1 ? 1 : 0] += p.y; sum[VEC > 2 ? 2 : 0] += p.z;
        sum[VEC > 3 ? 3 : 0] += p.w;
      } else {
        sum[0] += base[t * stride];
      }
    }
  };
  if (seq >= 0 && len >= 2) {
    const int i = (int)(token - start);
    const int nitems = a.plan.item_prefix[seq + 1] - a.plan.item_prefix[seq];
    const int64_t seq_base = a.plan.row_prefix[seq] * a.H;
    const int64_t id = a.plan.item_diagonals;
    // item t covers diagonals 1 + t id ..: query row i meets it iff 1 + t id <= i, key / value
    // row iff t id <= len - 2 - i (value rows are shifted by one)
    if (which == 0) {
      const int count = i >= 1 ? (int)min((int64_t)nitems, (i - 1) / id + 1) : 0;
      add_rows(a.dq_part + (seq_base + (int64_t)hh * nitems * len + i) * a.D + d, count,
               (int64_t)len * a.D);
    } else if (which == 1) {
      const int64_t room = (int64_t)len - 2 - i;
      const int count = room >= 0 ? (int)min((int64_t)nitems, room / id + 1) : 0;
      add_rows(a.dk_part + (seq_base + (int64_t)hh * nitems * len + i) * a.D + d, count,
               (int64_t)len * a.D);
    } else if (i >= 1) {
      const int64_t room = (int64_t)len - 1 - i;
      const int count = room >= 0 ? (int)min((int64_t)nitems, room / id + 1) : 0;
      for (int g = 0; g < a.group; ++g) {
        const int h = hh * a.group + g;
        add_rows(a.dv_part + (seq_base + (int64_t)h * nitems * len + i) * a.Dv + d, count,
                 (int64_t)len * a.Dv);
      }
    }
  }
  const void* src = which == 0 ? a.q : which == 1 ? a.k : a.v;
  const float coef = which == 2 ? 1.0f : a.mismatch_scale / (2.0f * (float)a.D);
  float* dst = which == 0 ? a.dq : which == 1 ? a.dk : a.dv;
  // the last position of a sequence is never a key: exact zero, whatever the input holds
  const bool never_key = which == 1 && seq >= 0 && token - start == len - 1;
  float out[VEC];
#pragma unroll
  for (int x = 0; x < VEC; ++x) {
    const float xv = load_as_float(src, idx + x, a.dtype);
    const float den = 1.0f + fabsf(xv);
    out[x] = never_key ? 0.0f : coef * sum[x] / (den * den);
  }
  if (VEC == 4) {
    *reinterpret_cast<float4*>(dst + idx) = make_float4(out[0], out[VEC > 1 ? 1 : 0],
                                                        out[VEC > 2 ? 2 : 0], out[VEC > 3 ? 3 : 0]);
  } else {
    dst[idx] = out[0];
  }
}

template <int DPAD, int DVPAD>
int launch_sweep2_t(const VjpArgs& a, int items_upper, bool small_dv, cudaStream_t stream) {
  const int ngroups = small_dv ? (a.Dv + 3) / 4 : 0;
  const size_t floats = sweep_common_floats(ngroups) + 2 * kVjpRows * kVjpBand +
                        (size_t)kWinCols * DPAD + kVjpRows * DPAD + kVjpRows * DVPAD;
  const size_t bytes = floats * sizeof(float);
  const unsigned grid = (unsigned)((int64_t)items_upper * a.H);
  if (small_dv) {
    ROSA_CUDA_OK(cudaFuncSetAttribute(vjp_sweep2_kernel<DPAD, DVPAD, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    vjp_sweep2_kernel<DPAD, DVPAD, true><<<grid, kVjpBand, bytes, stream>>>(a);
  } else {
    ROSA_CUDA_OK(cudaFuncSetAttribute(vjp_sweep2_kernel<DPAD, DVPAD, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    vjp_sweep2_kernel<DPAD, DVPAD, false><<<grid, kVjpBand, bytes, stream>>>(a);
  }
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int NK, int NV, int NG, bool kWindowed, bool kDropout>
int launch_sweep2_tc_t(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  size_t bytes = TcSmem<NK, NV>::kBytes +
                 (2 * tc_table_floats(NG, NV) + kVjpRows * kVjpBand) * sizeof(float);
  const unsigned grid = (unsigned)((int64_t)items_upper * a.H);
  auto kernel = vjp_sweep2_tc_kernel<NK, NV, NG, kWindowed, kDropout>;
  ROSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  kernel<<<grid, kVjpBand, bytes, stream>>>(a);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

template <int NK, int NV, int NG>
int launch_sweep2_tc_n(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  // the window product can only be non-zero when some sequence is longer than the horizon
  const bool windowed = a.ring_slots > 0;
  const bool dropout = a.dropout_p > 0.0f;
  if (windowed && dropout) return launch_sweep2_tc_t<NK, NV, NG, true, true>(a, items_upper, stream);
  if (windowed) return launch_sweep2_tc_t<NK, NV, NG, true, false>(a, items_upper, stream);
  if (dropout) return launch_sweep2_tc_t<NK, NV, NG, false, true>(a, items_upper, stream);
  return launch_sweep2_tc_t<NK, NV, NG, false, false>(a, items_upper, stream);
}

template <int NK>
int launch_sweep2_tc(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  if (a.Dv <= 8) return launch_sweep2_tc_n<NK, 16, 2>(a, items_upper, stream);
  if (a.Dv <= 16) return launch_sweep2_tc_n<NK, 16, 4>(a, items_upper, stream);
  return launch_sweep2_tc_n<NK, 32, 8>(a, items_upper, stream);
}

template <int DPAD>
int launch_sweep2_d(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  const bool small_dv = a.Dv <= 32;
  if (a.Dv <= 8) return launch_sweep2_t<DPAD, 8>(a, items_upper, small_dv, stream);
  if (a.Dv <= 16) return launch_sweep2_t<DPAD, 16>(a, items_upper, small_dv, stream);
  return launch_sweep2_t<DPAD, 32>(a, items_upper, small_dv, stream);
}

}  // namespace

int launch_pack_value_bits(const void* v, int dtype, int64_t N, int Hv, int Dv, uint32_t* vbits,
                           int vwords, cudaStream_t stream) {
  ProfileScope prof("pack_value_bits", stream);
  const int threads = 256;
  const int64_t total = N * Hv * vwords;
  const int64_t blocks = (total + threads - 1) / threads;
  if (dtype == ROSA_B200_F32)
    pack_value_bits_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>((const float*)v, N, Hv,
                                                                            Dv, vbits, vwords);
  else if (dtype == ROSA_B200_F16)
    pack_value_bits_kernel<__half><<<(unsigned)blocks, threads, 0, stream>>>((const __half*)v, N,
                                                                             Hv, Dv, vbits, vwords);
  else
    pack_value_bits_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)v, N, Hv, Dv, vbits, vwords);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_vjp_sweep1(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  if (items_upper <= 0) return 0;
  ProfileScope prof("vjp_sweep1", stream);
  if (vjp_tiled_applies(a)) return launch_vjp_sweep1_tiled(a, items_upper, stream);
  const bool small_dv = a.Dv <= 32;
  const size_t bytes = sweep_common_floats(small_dv ? (a.Dv + 3) / 4 : 0) * sizeof(float);
  const unsigned grid = (unsigned)((int64_t)items_upper * a.H);
  // the analytic logit bound is a safe softmax reference while it stays far inside the
  // float exponent range; otherwise every row reduces its own maximum
  const float top = a.scale * kSqrtScale * (sqrtf(1.0f + (float)a.W) - 1.0f);
  const bool fixed_ref = top <= 80.0f;
  const bool windowed = a.ring_slots > 0;     // some sequence may be longer than the horizon
  const bool dropout = a.dropout_p > 0.0f;
  const int ng = !small_dv ? 0 : a.Dv <= 8 ? 2 : a.Dv <= 16 ? 4 : 8;
  const size_t smem = sweep_common_floats(ng) * sizeof(float);
#define ROSA_SWEEP1(NGV, FR, WI, DO)                                                        \
  vjp_sweep1_kernel<NGV, FR, WI, DO><<<grid, kVjpBand, smem, stream>>>(a)
#define ROSA_SWEEP1_FLAGS(NGV)                                                              \
  do {                                                                                      \
    if (fixed_ref) {                                                                        \
      if (windowed) { if (dropout) ROSA_SWEEP1(NGV, true, true, true); else ROSA_SWEEP1(NGV, true, true, false); } \
      else          { if (dropout) ROSA_SWEEP1(NGV, true, false, true); else ROSA_SWEEP1(NGV, true, false, false); } \
    } else {                                                                                \
      if (windowed) { if (dropout) ROSA_SWEEP1(NGV, false, true, true); else ROSA_SWEEP1(NGV, false, true, false); } \
      else          { if (dropout) ROSA_SWEEP1(NGV, false, false, true); else ROSA_SWEEP1(NGV, false, false, false); } \
    }                                                                                       \
  } while (0)
  if (ng == 0) ROSA_SWEEP1_FLAGS(0);
  else if (ng == 2) ROSA_SWEEP1_FLAGS(2);
  else if (ng == 4) ROSA_SWEEP1_FLAGS(4);
  else ROSA_SWEEP1_FLAGS(8);
#undef ROSA_SWEEP1_FLAGS
#undef ROSA_SWEEP1
  (void)bytes;
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_vjp_rowstats(const VjpArgs& a, cudaStream_t stream) {
  ProfileScope prof("vjp_rowstats", stream);
  const int threads = 256;
  const int64_t blocks = (a.N * a.H + threads - 1) / threads;
  vjp_rowstats_kernel<<<(unsigned)blocks, threads, 0, stream>>>(a);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_vjp_sweep2(const VjpArgs& a, int items_upper, cudaStream_t stream) {
  if (items_upper <= 0) return 0;
  ProfileScope prof("vjp_sweep2", stream);
  if (vjp_tiled_applies(a)) return launch_vjp_sweep2_tiled(a, items_upper, stream);
  if (a.Dv <= 32 && !a.force_cuda_core_contraction) {
    // tensor-core contraction (tcgen05): operand N is 16 or 32 for both symbol and value dims
    if (a.D <= 16) return launch_sweep2_tc<16>(a, items_upper, stream);
    return launch_sweep2_tc<32>(a, items_upper, stream);
  }
  if (a.D <= 4) return launch_sweep2_d<4>(a, items_upper, stream);
  if (a.D <= 8) return launch_sweep2_d<8>(a, items_upper, stream);
  if (a.D <= 16) return launch_sweep2_d<16>(a, items_upper, stream);
  return launch_sweep2_d<32>(a, items_upper, stream);
}

int launch_vjp_finalize(const VjpArgs& a, cudaStream_t stream) {
  ProfileScope prof("vjp_finalize", stream);
  const int threads = 256;
  for (int which = 0; which < 3; ++which) {
    if (!(a.mask >> which & 1)) continue;
    const int dim = which == 2 ? a.Dv : a.D;
    float* dst = which == 0 ? a.dq : which == 1 ? a.dk : a.dv;
    const float* part = which == 0 ? a.dq_part : which == 1 ? a.dk_part : a.dv_part;
    // whole float4 groups and 16-byte aligned rows on both sides: four components per thread
    const bool vec = dim % 4 == 0 && ((reinterpret_cast<uintptr_t>(dst) |
                                       reinterpret_cast<uintptr_t>(part)) & 15) == 0;
    const int64_t total = a.N * (which == 2 ? (int64_t)a.Hv : (int64_t)a.H) * (vec ? dim / 4 : dim);
    const int64_t blocks = (total + threads - 1) / threads;
    if (vec)
      vjp_finalize_kernel<4><<<(unsigned)blocks, threads, 0, stream>>>(a, which);
    else
      vjp_finalize_kernel<1><<<(unsigned)blocks, threads, 0, stream>>>(a, which);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace rosa
