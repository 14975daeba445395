/*
 * CPU restatement of the rosa_soft operator family.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker for the CUDA path, never the thing that ships:
 * only the test-suite, the smoke check and the benchmark's CPU-baseline leg
 * load it.  The product library has no CPU path.
 *
 * Every routine follows the equations of the reference's pure-PyTorch oracle
 * and evaluates them by their *definition* (explicit prefix products over the
 * suffix window, explicit tail sums for the adjoint), in double precision.
 * The CUDA kernels use O(1)-per-cell diagonal recurrences instead, so the two
 * implementations share no algorithmic shortcut.
 *
 * Parity is pinned: tests/test_oracle_golden.py checks these routines against
 * the known-answer vectors of the reference's own tests and against fixtures
 * produced by importing the reference's rosa_soft_reference (float64 and
 * float32) with the generator committed beside the fixtures.
 *
 * Reference citations (paths inside the reference project):
 *   symbols / softsign VJP        rosa_soft/soft_reference.py:87-105
 *   causal routes                 rosa_soft/soft_reference.py:108-113
 *   exact symbol match            rosa_soft/soft_reference.py:116-132
 *   soft gates                    rosa_soft/soft_reference.py:135-164
 *   suffix prefix products        rosa_soft/soft_reference.py:167-186
 *   sqrt utility                  rosa_soft/soft_reference.py:189-194
 *   latest-longest selection      rosa_soft/soft_reference.py:197-231
 *   null score / probabilities    rosa_soft/soft_reference.py:234-271
 *   value gather                  rosa_soft/soft_reference.py:274-333
 *   carrier                       rosa_soft/soft_reference.py:336-359
 *   dropout counter hash          rosa_soft/soft_reference.py:362-447
 *   varlen segment loop           rosa_soft/soft_reference.py:682-701
 *   runtime match semantics       rosa_soft/csrc/rosa_runtime.cpp:41-45,103-133,455-467
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- symbols */

/* bit d of the word is set iff x[d] > 0 (zero, -0 and NaN give 0);
 * rosa_soft/soft_reference.py:87-88, rosa_soft/csrc/cuda/rosa_soft_kernels.cu:229-240 */
ORACLE_API void oracle_pack_symbols(const float* x, int64_t rows, int dim, uint32_t* out) {
  for (int64_t r = 0; r < rows; ++r) {
    uint32_t w = 0;
    for (int d = 0; d < dim; ++d)
      if (x[r * dim + d] > 0.0f) w |= (uint32_t)1u << d;
    out[r] = w;
  }
}

/* ----------------------------------------------------------- dropout hash */

/* rosa_soft/soft_reference.py:383-391 */
static inline uint32_t avalanche(uint32_t s) {
  s ^= s >> 16;
  s *= 0x7FEB352Du;
  s ^= s >> 15;
  s *= 0x846CA68Bu;
  s ^= s >> 16;
  return s;
}

ORACLE_API uint32_t oracle_hash_counter(uint32_t s) { return avalanche(s); }

/* rosa_soft/soft_reference.py:394-447: coordinates are chained route ->
 * query position -> head -> batch -> seed low -> seed high. */
static inline int dropout_keep(uint32_t route, uint32_t query, uint32_t head, uint32_t batch,
                               uint64_t seed, float p) {
  uint32_t st = avalanche(route ^ 0x68E31DA4u);
  st = avalanche(st ^ query ^ 0xB5297A4Du);
  st = avalanche(st ^ head ^ 0x63D83595u);
  st = avalanche(st ^ batch ^ 0xA511E9B3u);
  st = avalanche(st ^ (uint32_t)(seed & 0xFFFFFFFFu));
  st = avalanche(st ^ (uint32_t)(seed >> 32) ^ 0x9E3779B9u);
  const float uniform = (float)(st >> 8) * (1.0f / 16777216.0f);
  return uniform >= p;
}

ORACLE_API void oracle_dropout_keep_mask(int batch, int batch_offset, int heads, int queries,
                                         int routes, uint64_t seed, float p, uint8_t* keep) {
  for (int b = 0; b < batch; ++b)
    for (int h = 0; h < heads; ++h)
      for (int q = 0; q < queries; ++q)
        for (int r = 0; r < routes; ++r)
          keep[(((int64_t)b * heads + h) * queries + q) * routes + r] =
              (uint8_t)dropout_keep((uint32_t)r, (uint32_t)q, (uint32_t)h,
                                    (uint32_t)(b + batch_offset), seed, p);
}

/* ------------------------------------------------------------ hard routes */

/* Latest-longest causal suffix match for one sequence of one head.
 * route[i] in [0, i]; 0 is the null route.  Route a compares the query suffix
 * ending at i with the key suffix ending at a-1, length capped at min(W, a).
 * rosa_soft/soft_reference.py:295-317, 197-231. */
static void hard_routes_one(const uint32_t* q, const uint32_t* k, int64_t q_stride,
                            int64_t k_stride, int64_t len, int64_t W, int32_t* route,
                            int32_t* match_len) {
  int32_t* run = (int32_t*)calloc((size_t)len + 1, sizeof(int32_t));
  /* run[a] = suffix length of (row, route a); updated in place walking a downward
   * so run[a-1] still holds the previous row's value. */
  for (int64_t i = 0; i < len; ++i) {
    int32_t best_len = 0, best_route = 0;
    const uint32_t qi = q[i * q_stride];
    for (int64_t a = i; a >= 1; --a) {
      int32_t l = 0;
      if (qi == k[(a - 1) * k_stride]) {
        l = run[a - 1] + 1;
        if (l > W) l = (int32_t)W;
      }
      run[a] = l;
      if (l > best_len) { /* walking a downward: strict > keeps the latest on ties */
        best_len = l;
        best_route = (int32_t)a;
      }
    }
    run[0] = 0;
    route[i] = best_route;
    if (match_len) match_len[i] = best_len;
  }
  free(run);
}

/* Packed-symbol entry: symbols laid out [tokens][heads] (token-major), cu_seqlens[S+1].
 * Writes route (local index, 0 = null) and optionally the match length, [tokens][heads]. */
ORACLE_API void oracle_hard_routes(const uint32_t* qsym, const uint32_t* ksym,
                                   const int64_t* cu_seqlens, int64_t num_seq, int heads,
                                   int64_t W, int32_t* route, int32_t* match_len) {
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t s = 0; s < num_seq; ++s)
    for (int h = 0; h < heads; ++h) {
      const int64_t start = cu_seqlens[s], len = cu_seqlens[s + 1] - cu_seqlens[s];
      if (len <= 0) continue;
      const int64_t Weff = W < len ? W : len;
      int32_t* r = (int32_t*)malloc(sizeof(int32_t) * (size_t)len);
      int32_t* m = (int32_t*)malloc(sizeof(int32_t) * (size_t)len);
      hard_routes_one(qsym + start * heads + h, ksym + start * heads + h, heads, heads, len, Weff,
                      r, m);
      for (int64_t i = 0; i < len; ++i) {
        route[(start + i) * heads + h] = r[i];
        if (match_len) match_len[(start + i) * heads + h] = m[i];
      }
      free(r);
      free(m);
    }
}

/* Hard forward on logits: q,k [N,H,D], v [N,Hv,Dv], out [N,H,Dv] in {-1,0,+1};
 * route [N,H] (may be NULL).  rosa_soft/soft_reference.py:295-333. */
ORACLE_API void oracle_hard_forward(const float* q, const float* k, const float* v,
                                    const int64_t* cu_seqlens, int64_t num_seq, int64_t N, int H,
                                    int D, int Hv, int Dv, int64_t W, float* out,
                                    int32_t* route_out) {
  uint32_t* qs = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(N * H));
  uint32_t* ks = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(N * H));
  int32_t* route = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N * H));
  oracle_pack_symbols(q, N * H, D, qs);
  oracle_pack_symbols(k, N * H, D, ks);
  oracle_hard_routes(qs, ks, cu_seqlens, num_seq, H, W, route, NULL);
  const int group = H / Hv;
  for (int64_t s = 0; s < num_seq; ++s) {
    const int64_t start = cu_seqlens[s], end = cu_seqlens[s + 1];
    for (int64_t t = start; t < end; ++t)
      for (int h = 0; h < H; ++h) {
        const int32_t a = route[t * H + h];
        float* o = out + (t * H + h) * Dv;
        if (a == 0) {
          for (int d = 0; d < Dv; ++d) o[d] = 0.0f;
        } else {
          const float* src = v + ((start + a) * Hv + h / group) * Dv;
          for (int d = 0; d < Dv; ++d) o[d] = src[d] > 0.0f ? 1.0f : -1.0f;
        }
      }
  }
  if (route_out) memcpy(route_out, route, sizeof(int32_t) * (size_t)(N * H));
  free(qs);
  free(ks);
  free(route);
}

/* Batched hard inference on packed symbols (up to 32 bits): matched key end
 * position (route - 1, or -1 for null) and the payload at matched_end + 1.
 * Equals RosaRuntime.update_packed fed each stream in one call:
 * rosa_soft/csrc/rosa_runtime.cpp:41-45 (match, then extend), :120-131 (cap),
 * :455-467 (successor payload).  payload [N,Hp,Dp] float, out [N,H,Dp]. */
ORACLE_API void oracle_hard_inference(const uint32_t* qsym, const uint32_t* ksym,
                                      const float* payload, const int64_t* cu_seqlens,
                                      int64_t num_seq, int64_t N, int H, int Hp, int Dp, int64_t W,
                                      float* out, int64_t* matched_end) {
  int32_t* route = (int32_t*)malloc(sizeof(int32_t) * (size_t)(N * H));
  oracle_hard_routes(qsym, ksym, cu_seqlens, num_seq, H, W, route, NULL);
  const int group = H / Hp;
  for (int64_t s = 0; s < num_seq; ++s) {
    const int64_t start = cu_seqlens[s], end = cu_seqlens[s + 1];
    for (int64_t t = start; t < end; ++t)
      for (int h = 0; h < H; ++h) {
        const int32_t a = route[t * H + h];
        matched_end[t * H + h] = (int64_t)a - 1;
        if (out) {
          float* o = out + (t * H + h) * Dp;
          if (a == 0)
            for (int d = 0; d < Dp; ++d) o[d] = 0.0f;
          else
            memcpy(o, payload + ((start + a) * Hp + h / group) * Dp, sizeof(float) * (size_t)Dp);
        }
      }
  }
  free(route);
}

/* ---------------------------------------------------------- surrogate VJP */

/* bit count without a library call (the build does not assume a popcnt instruction) */
static inline int popcount32(uint32_t x) {
  x = x - ((x >> 1) & 0x55555555u);
  x = (x & 0x33333333u) + ((x >> 2) & 0x33333333u);
  x = (x + (x >> 4)) & 0x0F0F0F0Fu;
  return (int)((x * 0x01010101u) >> 24);
}

/* One (segment, head): accumulates dQz, dKz for this head and dVz for its value
 * head.  All arrays are local to the segment (index 0 = first token).
 * rosa_soft/soft_reference.py:484-541 evaluated by definition. */
static void vjp_one(const uint32_t* qs, const uint32_t* ks, /* [len] symbols of this head */
                    const float* v,  /* [len][Dv] value rows of the value head (strided) */
                    int64_t v_stride, const float* go, /* [len][Dv] grad rows (strided) */
                    int64_t go_stride, int64_t len, int D, int Dv, int64_t W, double scale,
                    double dropout_p, double m, uint64_t seed, uint32_t head, uint32_t batch,
                    double* dQz, /* [len][D] */
                    double* dKz, /* [len][D] */
                    double* dVz /* [len][Dv], shared by the group: caller serialises */) {
  const double c = sqrt(2.0) + 1.0;
  /* the keep test compares a float32 uniform with float32(p); the kept weight is
   * divided by (1 - p) in the working precision (soft_reference.py:441-447) */
  const float p = (float)dropout_p;
  const double inv_keep = (dropout_p > 0.0) ? 1.0 / (1.0 - dropout_p) : 1.0;
  double lut[33];
  for (int h = 0; h <= D; ++h) lut[h] = exp(-m * (double)h / (double)D);

  double* S = (double*)malloc(sizeof(double) * (size_t)len);     /* one row of suffix sums */
  double* prob = (double*)malloc(sizeof(double) * (size_t)len);
  double* dS = (double*)malloc(sizeof(double) * (size_t)len);
  double* pref = (double*)malloc(sizeof(double) * (size_t)(W + 1));
  /* cell adjoints, stored diagonal-major (cell (p, j) at [(p - j) * len + j]): a route's
   * window walks one diagonal, so its updates touch consecutive memory */
  double* C = (double*)calloc((size_t)len * (size_t)len, sizeof(double));
  double* u = (double*)malloc(sizeof(double) * (size_t)len);
  double* dmul = (double*)malloc(sizeof(double) * (size_t)len);

  for (int64_t i = 1; i < len; ++i) {
    /* S(i, j) for key position j = a-1 in [0, i-1] */
    double maxlogit = 0.5 * scale; /* null route, rosa_soft/soft_contract.py:15 */
    for (int64_t j = 0; j < i; ++j) {
      const int64_t steps = (W < j + 1) ? W : j + 1;
      double prod = 1.0, sum = 0.0;
      for (int64_t s = 0; s < steps; ++s) {
        prod *= lut[popcount32(qs[i - s] ^ ks[j - s])];
        sum += prod;
      }
      S[j] = sum;
      const double logit = c * (sqrt(1.0 + sum) - 1.0) * scale - log((double)i);
      prob[j] = logit;
      if (logit > maxlogit) maxlogit = logit;
    }
    double Z = exp(0.5 * scale - maxlogit);
    for (int64_t j = 0; j < i; ++j) {
      prob[j] = exp(prob[j] - maxlogit);
      Z += prob[j];
    }
    double E = 0.0;
    for (int64_t j = 0; j < i; ++j) {
      prob[j] /= Z;
      const int64_t a = j + 1;
      double dot = 0.0;
      const float* vr = v + a * v_stride;
      const float* gr = go + i * go_stride;
      for (int d = 0; d < Dv; ++d) dot += (vr[d] > 0.0f ? 1.0 : -1.0) * (double)gr[d];
      u[j] = dot;
      dmul[j] = 1.0;
      if (p > 0.0f)
        dmul[j] = dropout_keep((uint32_t)a, (uint32_t)i, head, batch, seed, p) ? inv_keep : 0.0;
      E += prob[j] * dmul[j] * dot;
    }
    for (int64_t j = 0; j < i; ++j) {
      const int64_t a = j + 1;
      const double w = prob[j] * dmul[j];
      if (dVz) {
        const float* gr = go + i * go_stride;
        double* dv = dVz + a * Dv;
        for (int d = 0; d < Dv; ++d) dv[d] += w * (double)gr[d];
      }
      const double dlogit = prob[j] * (dmul[j] * u[j] - E);
      dS[j] = scale * dlogit * c / (2.0 * sqrt(1.0 + S[j]));
    }
    if (!dQz && !dKz) continue;
    /* adjoint of the prefix-product sum: cell (i-s, j-s) receives dS * tail_s,
     * tail_s = sum_{s' >= s} prod_{u <= s'} g   (rosa_soft_kernels.cu:1530-1596) */
    for (int64_t j = 0; j < i; ++j) {
      if (dS[j] == 0.0) continue;
      const int64_t steps = (W < j + 1) ? W : j + 1;
      double prod = 1.0;
      for (int64_t s = 0; s < steps; ++s) {
        prod *= lut[popcount32(qs[i - s] ^ ks[j - s])];
        pref[s] = prod;
      }
      double tail = 0.0;
      double* diag = C + (i - j) * len + j; /* cell (i - s, j - s) is diag[-s] */
      for (int64_t s = steps - 1; s >= 0; --s) {
        tail += pref[s];
        diag[-s] += dS[j] * tail;
      }
    }
  }
  if (dQz || dKz) {
    const double coef = m / (2.0 * (double)D);
    for (int64_t i = 1; i < len; ++i)
      for (int64_t j = 0; j < i; ++j) {
        const double cc = coef * C[(i - j) * len + j];
        if (cc == 0.0) continue;
        for (int d = 0; d < D; ++d) {
          const double kz = ((ks[j] >> d) & 1u) ? 1.0 : -1.0;
          const double qz = ((qs[i] >> d) & 1u) ? 1.0 : -1.0;
          if (dQz) dQz[i * D + d] += cc * kz;
          if (dKz) dKz[j * D + d] += cc * qz;
        }
      }
  }
  free(S);
  free(prob);
  free(dS);
  free(pref);
  free(C);
  free(u);
  free(dmul);
}

/* Full surrogate VJP over packed sequences.
 * q,k [N,H,D]; v [N,Hv,Dv]; go [N,H,Dv] (all float32 values of the input dtype);
 * outputs double [N,H,D], [N,H,D], [N,Hv,Dv]; pass NULL to skip one.
 * Dropout "batch" coordinate = sequence ordinal counting empty sequences
 * (rosa_soft/soft_reference.py:683-699) plus batch_offset; head_offset shifts the head
 * coordinate the same way (both are zero for an unsharded problem). */
ORACLE_API void oracle_surrogate_vjp(const float* q, const float* k, const float* v,
                                     const float* go, const int64_t* cu_seqlens, int64_t num_seq,
                                     int64_t N, int H, int D, int Hv, int Dv, int64_t W,
                                     double scale, double dropout_p, double mismatch_scale,
                                     int64_t seed, int64_t batch_offset, int64_t head_offset,
                                     double* dq, double* dk, double* dv) {
  const int group = H / Hv;
  uint32_t* qs = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(N * H));
  uint32_t* ks = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(N * H));
  oracle_pack_symbols(q, N * H, D, qs);
  oracle_pack_symbols(k, N * H, D, ks);
  if (dq) memset(dq, 0, sizeof(double) * (size_t)(N * H * D));
  if (dk) memset(dk, 0, sizeof(double) * (size_t)(N * H * D));
  if (dv) memset(dv, 0, sizeof(double) * (size_t)(N * Hv * Dv));

  /* parallel over (sequence, value head); the heads of one group run serially so
   * the shared dVz rows are accumulated in a fixed order. */
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t s = 0; s < num_seq; ++s)
    for (int vh = 0; vh < Hv; ++vh) {
      const int64_t start = cu_seqlens[s], len = cu_seqlens[s + 1] - cu_seqlens[s];
      if (len <= 1) continue;
      const int64_t Weff = W < len ? W : len;
      uint32_t* ql = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)len);
      uint32_t* kl = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)len);
      double* dQz = dq ? (double*)malloc(sizeof(double) * (size_t)(len * D)) : NULL;
      double* dKz = dk ? (double*)malloc(sizeof(double) * (size_t)(len * D)) : NULL;
      double* dVz = dv ? (double*)calloc((size_t)(len * Dv), sizeof(double)) : NULL;
      for (int g = 0; g < group; ++g) {
        const int h = vh * group + g;
        for (int64_t t = 0; t < len; ++t) {
          ql[t] = qs[(start + t) * H + h];
          kl[t] = ks[(start + t) * H + h];
        }
        if (dQz) memset(dQz, 0, sizeof(double) * (size_t)(len * D));
        if (dKz) memset(dKz, 0, sizeof(double) * (size_t)(len * D));
        vjp_one(ql, kl, v + (start * Hv + vh) * Dv, (int64_t)Hv * Dv,
                go + (start * H + h) * Dv, (int64_t)H * Dv, len, D, Dv, Weff, scale, dropout_p,
                mismatch_scale, (uint64_t)seed, (uint32_t)(h + head_offset),
                (uint32_t)(s + batch_offset), dQz,
                dKz, dVz);
        for (int64_t t = 0; t < len; ++t)
          for (int d = 0; d < D; ++d) {
            const int64_t idx = ((start + t) * H + h) * D + d;
            if (dq) {
              const double den = 1.0 + fabs((double)q[idx]);
              dq[idx] = dQz[t * D + d] / (den * den);
            }
            if (dk) {
              /* the last position of a sequence is never a key (routes end at a - 1 = len - 2):
               * the reference slices it away before the sign function, so its gradient is an
               * exact zero whatever the input holds, NaN included */
              const double den = 1.0 + fabs((double)k[idx]);
              dk[idx] = (t == len - 1) ? 0.0 : dKz[t * D + d] / (den * den);
            }
          }
      }
      if (dv)
        for (int64_t t = 0; t < len; ++t)
          for (int d = 0; d < Dv; ++d) {
            const int64_t idx = ((start + t) * Hv + vh) * Dv + d;
            const double den = 1.0 + fabs((double)v[idx]);
            dv[idx] = dVz[t * Dv + d] / (den * den);
          }
      free(ql);
      free(kl);
      free(dQz);
      free(dKz);
      free(dVz);
    }
  free(qs);
  free(ks);
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; a timed baseline asks for the cores. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
