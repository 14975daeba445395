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
// exact matches are longer than the horizon.
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

namespace rosa {

namespace {

constexpr float kSqrtScale = 2.41421356237309504880f;  // sqrt(2) + 1

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

// ------------------------------------------------------------- item geometry
struct Item {
  int seq, it, h, start, len;
  int nitems;            // items of this sequence (per head)
  int w_begin, w_end;    // bands walked by this CTA
  int64_t rowslot;       // first partial-row slot of this (item, head)
  int64_t ck_base;       // first checkpoint block of this (sequence, head)
  int64_t item_linear;   // dense index over (sequence, head, item)
};

__device__ __forceinline__ bool load_item(const VjpArgs& a, Item* o) {
  if (!find_item(a.plan, blockIdx.x, &o->seq, &o->it)) return false;
  o->h = blockIdx.y;
  o->start = a.plan.seg_start[o->seq];
  o->len = a.plan.seg_len[o->seq];
  o->nitems = a.plan.item_prefix[o->seq + 1] - a.plan.item_prefix[o->seq];
  const int nbands = (int)vjp_bands(o->len);
  o->w_begin = o->it * a.bands_per_item;
  o->w_end = min(nbands, o->w_begin + a.bands_per_item);
  o->rowslot = a.plan.row_prefix[o->seq] * a.H +
               ((int64_t)o->h * o->nitems + o->it) * (int64_t)o->len;
  o->ck_base = a.plan.ck_prefix[o->seq] * a.H + (int64_t)o->h * vjp_ck_count(o->len);
  o->item_linear = (int64_t)a.plan.item_prefix[o->seq] * a.H + (int64_t)o->h * o->nitems + o->it;
  return true;
}

__device__ __forceinline__ void merge_stats(float& m, float& z, float& e, float m2, float z2,
                                            float e2) {
  if (m2 == -CUDART_INF_F) return;
  if (m == -CUDART_INF_F) {
    m = m2; z = z2; e = e2;
    return;
  }
  const float mm = fmaxf(m, m2);
  const float s1 = __expf(m - mm), s2 = __expf(m2 - mm);
  z = z * s1 + z2 * s2;
  e = e * s1 + e2 * s2;
  m = mm;
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
    ulut[(r * 8 + g) * 16 + nib] = s;
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
    for (int g = 0; g < ngroups; ++g) u += ulut[(r * 8 + g) * 16 + ((bits >> (4 * g)) & 15u)];
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

// shared-memory carve-up common to both sweeps (float units)
struct SweepSmem {
  float* glut;    // [33] gate per mismatch count
  int* s_q;       // [kVjpRows] query symbols of the block rows
  float4* rstat;  // [kVjpRows] (max, 1/Z, E, log i); sweep 1 only uses .w
  float4* wstat;  // [kVjpRows * kVjpWarps] per-warp online-softmax partials (sweep 1)
  float* ulut;    // [kVjpRows * 8 * 16]
};

constexpr int kSweepCommonFloats =
    64 + kVjpRows + 4 * kVjpRows + 4 * kVjpRows * kVjpWarps + kVjpRows * 8 * 16;

__device__ __forceinline__ SweepSmem carve_common(float* base) {
  SweepSmem s;
  s.rstat = reinterpret_cast<float4*>(base);
  s.wstat = s.rstat + kVjpRows;
  float* f = reinterpret_cast<float*>(s.wstat + kVjpRows * kVjpWarps);
  s.ulut = f;
  f += kVjpRows * 8 * 16;
  s.glut = f;
  f += 64;
  s.s_q = reinterpret_cast<int*>(f);
  return s;
}

// ------------------------------------------------------------------- sweep 1
template <bool kSmallDv>
__global__ void __launch_bounds__(kVjpBand) vjp_sweep1_kernel(VjpArgs a) {
  extern __shared__ float4 smem_raw[];
  SweepSmem sm = carve_common(reinterpret_cast<float*>(smem_raw));
  Item it;
  if (!load_item(a, &it)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool dense = a.plan.cu_seqlens == nullptr;
  const int64_t sym_base = (int64_t)it.seq * a.sym_seq_stride + (int64_t)it.h * a.sym_head_stride +
                           (dense ? 0 : it.start);
  const int32_t* __restrict__ q = a.qsym + sym_base;
  const int32_t* __restrict__ k = a.ksym + sym_base;
  const int vh = it.h / a.group;
  const uint32_t* __restrict__ vb = a.vbits + ((int64_t)vh * a.N + it.start) * a.vwords;
  const int ngroups = kSmallDv ? (a.Dv + 3) / 4 : 0;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const bool windowed = a.W <= it.len - 2;
  const bool use_dropout = a.dropout_p > 0.0f;
  const DropoutKey dkey = make_dropout_key((uint32_t)it.h + a.head_offset,
                                           (uint32_t)it.seq + a.batch_offset, a.seed, a.dropout_p);
  if (tid <= a.D) sm.glut[tid] = expf(neg_md * (float)tid);

  for (int w = it.w_begin; w < it.w_end; ++w) {
    const int dmin = 1 + w * kVjpBand;
    const int delta = dmin + tid;
    const bool valid = delta <= it.len - 1;
    float S = 0.0f;
    int hs = 0;
    const int rb_lo = dmin / kVjpRows, rb_hi = (it.len - 1) / kVjpRows;
    const int64_t ck_band = it.ck_base + vjp_ck_before(it.len, w);
    for (int rb = rb_lo; rb <= rb_hi; ++rb) {
      const int i0 = max(rb * kVjpRows, dmin), i1 = min(rb * kVjpRows + kVjpRows - 1, it.len - 1);
      const int nrows = i1 - i0 + 1;
      __syncthreads();
      if (tid < nrows) {
        sm.s_q[tid] = __ldg(q + i0 + tid);
        sm.rstat[tid].w = logf((float)(i0 + tid));
      }
      if (kSmallDv) build_ulut(a, it, i0, nrows, ngroups, sm.ulut);
      __syncthreads();
      a.ckpt[(ck_band + (rb - rb_lo)) * kVjpBand + tid] = make_int2(__float_as_int(S), hs);

      for (int r = 0; r < nrows; ++r) {
        const int i = i0 + r;
        const int j = i - delta;
        const bool act = valid && j >= 0;
        float logit = -CUDART_INF_F, du = 0.0f;
        if (act) {
          const int qi = sm.s_q[r];
          const int ham = __popc(qi ^ __ldg(k + j));
          const float x = sm.glut[ham];
          float P = 0.0f;
          if (windowed) {
            hs += ham;
            if (j > a.W) hs -= __popc(__ldg(q + i - a.W - 1) ^ __ldg(k + j - a.W - 1));
            if (j >= a.W) P = __expf(neg_md * (float)hs);
          }
          S = x * (1.0f + S) - P;
          logit = kSqrtScale * (sqrtf(1.0f + S) - 1.0f) * a.scale - sm.rstat[r].w;
          du = route_utility<kSmallDv>(a, it, vb, i, r, j + 1, ngroups, sm.ulut);
          if (use_dropout)
            du = dropout_keep(dkey, (uint32_t)(j + 1), (uint32_t)i) ? du * a.inv_keep : 0.0f;
        }
        const float mw = warp_max(logit);
        const float e = act ? __expf(logit - mw) : 0.0f;
        const float zw = warp_sum(e);
        const float ew = warp_sum(e * du);
        if (lane == 0) sm.wstat[r * kVjpWarps + warp] = make_float4(mw, zw, ew, 0.0f);
      }
      __syncthreads();
      if (tid < nrows) {
        float m = -CUDART_INF_F, z = 0.0f, e = 0.0f;
#pragma unroll
        for (int ww = 0; ww < kVjpWarps; ++ww) {
          const float4 p = sm.wstat[tid * kVjpWarps + ww];
          merge_stats(m, z, e, p.x, p.y, p.z);
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
template <int DPAD, int DVPAD, bool kSmallDv>
__global__ void __launch_bounds__(kVjpBand) vjp_sweep2_kernel(VjpArgs a) {
  extern __shared__ float4 smem_raw[];
  float* fbase = reinterpret_cast<float*>(smem_raw);
  SweepSmem sm = carve_common(fbase);
  float* Cbuf = fbase + kSweepCommonFloats;            // [kVjpRows][kVjpBand]; S, then C
  float* Pbuf = Cbuf + kVjpRows * kVjpBand;            // [kVjpRows][kVjpBand]; P, then p*d
  float* kz = Pbuf + kVjpRows * kVjpBand;              // [kVjpRows + kVjpBand][DPAD]
  float* qz = kz + (kVjpRows + kVjpBand) * DPAD;       // [kVjpRows][DPAD]
  float* gob = qz + kVjpRows * DPAD;                   // [kVjpRows][DVPAD]

  Item it;
  if (!load_item(a, &it)) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool dense = a.plan.cu_seqlens == nullptr;
  const int64_t sym_base = (int64_t)it.seq * a.sym_seq_stride + (int64_t)it.h * a.sym_head_stride +
                           (dense ? 0 : it.start);
  const int32_t* __restrict__ q = a.qsym + sym_base;
  const int32_t* __restrict__ k = a.ksym + sym_base;
  const int vh = it.h / a.group;
  const uint32_t* __restrict__ vb = a.vbits + ((int64_t)vh * a.N + it.start) * a.vwords;
  const int ngroups = kSmallDv ? (a.Dv + 3) / 4 : 0;
  const float neg_md = -a.mismatch_scale / (float)a.D;
  const bool windowed = a.W <= it.len - 2;
  const bool use_dropout = a.dropout_p > 0.0f;
  const DropoutKey dkey = make_dropout_key((uint32_t)it.h + a.head_offset,
                                           (uint32_t)it.seq + a.batch_offset, a.seed, a.dropout_p);
  const float4* __restrict__ rowstat = a.rowstat + (int64_t)it.h * a.N + it.start;
  float* ring = a.ring_slots ? a.ring + it.item_linear * (int64_t)a.ring_slots * kVjpBand + tid
                             : nullptr;
  if (tid <= a.D) sm.glut[tid] = expf(neg_md * (float)tid);

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
    int slot = (valid && a.ring_slots) ? (it.len - 1 - delta) % a.ring_slots : 0;

    for (int rb = rb_hi; rb >= rb_lo; --rb) {
      const int i0 = max(rb * kVjpRows, dmin), i1 = min(rb * kVjpRows + kVjpRows - 1, it.len - 1);
      const int nrows = i1 - i0 + 1;
      const int jwin0 = i0 - dmax;  // first key column of the block's column window
      __syncthreads();
      // ---- block tables
      if (tid < nrows) {
        sm.s_q[tid] = __ldg(q + i0 + tid);
        sm.rstat[tid] = rowstat[i0 + tid];
      }
      if (kSmallDv) build_ulut(a, it, i0, nrows, ngroups, sm.ulut);
      if (a.mask & 2)
        for (int e = tid; e < nrows * DPAD; e += kVjpBand) {
          const int r = e / DPAD, d = e - r * DPAD;
          qz[e] = d < a.D ? ((__ldg(q + i0 + r) >> d & 1) ? 1.0f : -1.0f) : 0.0f;
        }
      if (a.mask & 1)
        for (int e = tid; e < (nrows + kVjpBand - 1) * DPAD; e += kVjpBand) {
          const int c = e / DPAD, d = e - c * DPAD;
          const int j = jwin0 + c;
          kz[e] = (d < a.D && j >= 0 && j < it.len) ? ((__ldg(k + j) >> d & 1) ? 1.0f : -1.0f)
                                                    : 0.0f;
        }
      // ---- phase A: forward recurrence of the block from its checkpoint
      const int2 ck = a.ckpt[(ck_band + (rb - rb_lo)) * kVjpBand + tid];
      float S = __int_as_float(ck.x);
      int hs = ck.y;
      __syncthreads();
      for (int r = 0; r < nrows; ++r) {
        const int i = i0 + r;
        const int j = i - delta;
        float P = 0.0f, Sv = 0.0f;
        if (valid && j >= 0) {
          const int ham = __popc(sm.s_q[r] ^ __ldg(k + j));
          if (windowed) {
            hs += ham;
            if (j > a.W) hs -= __popc(__ldg(q + i - a.W - 1) ^ __ldg(k + j - a.W - 1));
            if (j >= a.W) P = __expf(neg_md * (float)hs);
          }
          S = sm.glut[ham] * (1.0f + S) - P;
          Sv = S;
        }
        Cbuf[r * kVjpBand + tid] = Sv;
        Pbuf[r * kVjpBand + tid] = P;
      }
      // ---- phase B: adjoint recurrence, rows descending
      for (int r = nrows - 1; r >= 0; --r) {
        const int i = i0 + r;
        const int j = i - delta;
        const bool act = valid && j >= 0;
        float Cv = 0.0f, pd = 0.0f, P = 0.0f;
        double T = 0.0;
        float x = 0.0f, Sv = 0.0f;
        if (act) {
          Sv = Cbuf[r * kVjpBand + tid];
          P = Pbuf[r * kVjpBand + tid];
          const float4 st = sm.rstat[r];
          x = sm.glut[__popc(sm.s_q[r] ^ __ldg(k + j))];
          const float sq = sqrtf(1.0f + Sv);
          const float logit = kSqrtScale * (sq - 1.0f) * a.scale - st.w;
          const float pr = __expf(logit - st.x) * st.y;
          float dmul = 1.0f;
          if (use_dropout)
            dmul = dropout_keep(dkey, (uint32_t)(j + 1), (uint32_t)i) ? a.inv_keep : 0.0f;
          const float u = route_utility<kSmallDv>(a, it, vb, i, r, j + 1, ngroups, sm.ulut);
          pd = pr * dmul;
          const float dlogit = pd * u - pr * st.z;
          const float dS = a.scale * dlogit * kSqrtScale / (2.0f * sq);
          Sbar = (double)dS + (double)xnext * Sbar;
          T = Sbar * (double)P;
        }
        if (ring != nullptr) {
          const bool any_p = __any_sync(0xffffffffu, P != 0.0f);
          if (any_p) {
            live = a.W + 2;
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
        }
        if (act) {
          Cv = (float)((double)(Sv + P) * Sbar - Y);
          xnext = x;
          slot = slot == 0 ? a.ring_slots - 1 : slot - 1;
        }
        Cbuf[r * kVjpBand + tid] = Cv;
        Pbuf[r * kVjpBand + tid] = pd;
      }
      __syncthreads();
      // ---- phase C: contract the block tiles
      if (a.mask & 1) {  // dQz[i] += sum_j C(i, j) kz[j]
        for (int r = warp; r < nrows; r += kVjpWarps) {
          float acc[DPAD];
#pragma unroll
          for (int d = 0; d < DPAD; ++d) acc[d] = 0.0f;
#pragma unroll
          for (int c = 0; c < kVjpBand / 32; ++c) {
            const int t = lane + 32 * c;
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
          float mine = 0.0f;
#pragma unroll
          for (int d = 0; d < DPAD; ++d) {
            const float s = warp_sum(acc[d]);
            if (lane == d) mine = s;
          }
          if (lane < a.D) {
            float* dst = a.dq_part + (it.rowslot + i0 + r) * a.D + lane;
            *dst = (w == it.w_begin) ? mine : *dst + mine;
          }
        }
      }
      if (a.mask & 6) {  // column sums: dKz[j] += sum_i C(i,j) qz[i];  dVz[j+1] += sum_i pd gO(i)
        const int ncols = nrows + kVjpBand - 1;
        for (int dv0 = 0; dv0 < ((a.mask & 4) ? a.Dv : 1); dv0 += DVPAD) {
          if (a.mask & 4) {
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
          for (int c = tid; c < ncols; c += kVjpBand) {
            const int j = jwin0 + c;
            if (j < 0 || j > it.len - 1 - dmin) continue;
            float acck[DPAD], accv[DVPAD];
#pragma unroll
            for (int d = 0; d < DPAD; ++d) acck[d] = 0.0f;
#pragma unroll
            for (int d = 0; d < DVPAD; ++d) accv[d] = 0.0f;
            // every thread walks the same rows so that a warp reads one tile row at a
            // time (consecutive columns = consecutive diagonals, no bank conflicts)
            for (int r = 0; r < nrows; ++r) {
              const int t = i0 + r - j - dmin;  // diagonal of cell (row, column j) in the band
              if (t < 0 || t >= kVjpBand) continue;
              if ((a.mask & 2) && dv0 == 0) {
                const float cv = Cbuf[r * kVjpBand + t];
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
              if (a.mask & 4) {
                const float pv = Pbuf[r * kVjpBand + t];
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
            if ((a.mask & 2) && dv0 == 0) {
              float* dst = a.dk_part + (it.rowslot + j) * a.D;
#pragma unroll
              for (int d = 0; d < DPAD; ++d)
                if (d < a.D) dst[d] = first ? acck[d] : dst[d] + acck[d];
            }
            if (a.mask & 4) {
              float* dst = a.dv_part + (it.rowslot + j + 1) * a.Dv + dv0;
#pragma unroll
              for (int d = 0; d < DVPAD; ++d)
                if (dv0 + d < a.Dv) dst[d] = first ? accv[d] : dst[d] + accv[d];
            }
          }
        }
      }
    }
    // leave the ring zeroed for the next band of this item
    if (ring != nullptr && ring_dirty && w + 1 < it.w_end) {
      for (int s = 0; s < a.ring_slots; ++s) ring[(int64_t)s * kVjpBand] = 0.0f;
    }
  }
}

// ------------------------------------------------------------------ finalize
// Sums the per-item partials in item order and applies the softsign Jacobian.
// which: 0 = query, 1 = key, 2 = value.
__global__ void vjp_finalize_kernel(VjpArgs a, int which) {
  const int dim = which == 2 ? a.Dv : a.D;
  const int heads = which == 2 ? a.Hv : a.H;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= a.N * heads * dim) return;
  const int d = (int)(idx % dim);
  const int64_t th = idx / dim;
  const int64_t token = th / heads;
  const int hh = (int)(th - token * heads);
  int start, len;
  const int seq = find_segment(a.plan, token, &start, &len);
  float sum = 0.0f;
  if (seq >= 0 && len >= 2) {
    const int i = (int)(token - start);
    const int nitems = a.plan.item_prefix[seq + 1] - a.plan.item_prefix[seq];
    const int64_t seq_base = a.plan.row_prefix[seq] * a.H;
    const int64_t id = a.plan.item_diagonals;
    if (which == 0) {
      for (int t = 0; t < nitems && 1 + t * id <= i; ++t)
        sum += a.dq_part[(seq_base + ((int64_t)hh * nitems + t) * len + i) * a.D + d];
    } else if (which == 1) {
      for (int t = 0; t < nitems && t * id <= (int64_t)len - 2 - i; ++t)
        sum += a.dk_part[(seq_base + ((int64_t)hh * nitems + t) * len + i) * a.D + d];
    } else if (i >= 1) {
      for (int g = 0; g < a.group; ++g) {
        const int h = hh * a.group + g;
        for (int t = 0; t < nitems && t * id <= (int64_t)len - 1 - i; ++t)
          sum += a.dv_part[(seq_base + ((int64_t)h * nitems + t) * len + i) * a.Dv + d];
      }
    }
  }
  const void* src = which == 0 ? a.q : which == 1 ? a.k : a.v;
  const float xv = load_as_float(src, idx, a.dtype);
  const float den = 1.0f + fabsf(xv);
  const float coef = which == 2 ? 1.0f : a.mismatch_scale / (2.0f * (float)a.D);
  float* dst = which == 0 ? a.dq : which == 1 ? a.dk : a.dv;
  dst[idx] = coef * sum / (den * den);
}

template <int DPAD, int DVPAD>
int launch_sweep2_t(const VjpArgs& a, int items_upper, bool small_dv, cudaStream_t stream) {
  const size_t floats = kSweepCommonFloats + 2 * kVjpRows * kVjpBand +
                        (size_t)(kVjpRows + kVjpBand) * DPAD + kVjpRows * DPAD + kVjpRows * DVPAD;
  const size_t bytes = floats * sizeof(float);
  dim3 grid((unsigned)items_upper, (unsigned)a.H);
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
  const size_t bytes = kSweepCommonFloats * sizeof(float);
  dim3 grid((unsigned)items_upper, (unsigned)a.H);
  if (a.Dv <= 32)
    vjp_sweep1_kernel<true><<<grid, kVjpBand, bytes, stream>>>(a);
  else
    vjp_sweep1_kernel<false><<<grid, kVjpBand, bytes, stream>>>(a);
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
    const int64_t total = a.N * (which == 2 ? (int64_t)a.Hv * a.Dv : (int64_t)a.H * a.D);
    const int64_t blocks = (total + threads - 1) / threads;
    vjp_finalize_kernel<<<(unsigned)blocks, threads, 0, stream>>>(a, which);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace rosa
