// Hard forward of the rosa_soft operator: sign-binarise Q/K into packed symbols, find the
// latest among the longest causal suffix matches within the horizon, gather the sign of
// the routed value row.  Replaces pack_sign_bits_pair_kernel, exact_suffix_length,
// merge_hard_route and hard_forward_kernel of the reference
// (rosa_soft/csrc/cuda/rosa_soft_kernels.cu:202-241, 311-531).
//
// Matching uses the exact diagonal run-length recurrence
//     len(i, a) = (q_i == k_{a-1}) ? min(len(i-1, a-1) + 1, W) : 0
// instead of re-walking every suffix: one thread owns several diagonals, a warp sits
// on one query row at a time, the per-row winner is reduced with redux.sync and merged
// across bands with one 64-bit integer atomicMax (order independent, hence exact and
// deterministic).
#include "common.cuh"
#include "bit_match.cuh"

namespace rosa {

namespace {

// ------------------------------------------------------------------ packing
template <typename T>
__device__ __forceinline__ bool positive(T x);
template <>
__device__ __forceinline__ bool positive<float>(float x) { return x > 0.0f; }
template <>
__device__ __forceinline__ bool positive<__half>(__half x) { return __half2float(x) > 0.0f; }
template <>
__device__ __forceinline__ bool positive<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x) > 0.0f;
}

// Sign bits of one D-vector.  When the vector is a whole number of 16-byte words (and the tensor
// base is 16-byte aligned) it is read with 128-bit loads; bit d of the word is set iff
// component d is strictly positive (zero, -0 and NaN give 0).
template <typename T>
__device__ __forceinline__ uint32_t sign_word(const T* __restrict__ row, int D, bool vec) {
  uint32_t w = 0;
  if (vec) {
    constexpr int kPer = 16 / (int)sizeof(T);
    const uint4* p = reinterpret_cast<const uint4*>(row);
    for (int c = 0; c < D / kPer; ++c) {
      const uint4 raw = __ldg(p + c);
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int x = 0; x < kPer; ++x) w |= (uint32_t)positive<T>(e[x]) << (c * kPer + x);
    }
  } else {
    for (int d = 0; d < D; ++d) w |= (uint32_t)positive<T>(row[d]) << d;
  }
  return w;
}

// One thread per (token, head); threads of a warp read consecutive D-vectors.
template <typename T>
__global__ void pack_symbols_kernel(const T* __restrict__ q, const T* __restrict__ k, int64_t N,
                                    int H, int D, int dense, int64_t uniform_len, int vec,
                                    int32_t* __restrict__ pq, int32_t* __restrict__ pk) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * H) return;
  const int64_t token = idx / H;
  const int h = (int)(idx - token * H);
  const uint32_t wq = sign_word<T>(q + idx * D, D, vec != 0);
  const uint32_t wk = k != nullptr ? sign_word<T>(k + idx * D, D, vec != 0) : 0u;
  int64_t dst;
  if (dense) {
    const int64_t b = token / uniform_len, t = token - b * uniform_len;
    dst = (b * H + h) * uniform_len + t;
  } else {
    dst = (int64_t)h * N + token;
  }
  pq[dst] = (int32_t)wq;
  if (k != nullptr) pk[dst] = (int32_t)wk;
}

// token-major [N, H] symbols -> head-major [H, N]
__global__ void transpose_symbols_kernel(const uint32_t* __restrict__ q,
                                         const uint32_t* __restrict__ k, int64_t N, int H,
                                         int32_t* __restrict__ qt, int32_t* __restrict__ kt) {
  __shared__ uint32_t tq[32][33], tk[32][33];
  const int64_t t0 = (int64_t)blockIdx.x * 32;
  const int h0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int64_t t = t0 + r;
    const int h = h0 + threadIdx.x;
    if (t < N && h < H) {
      tq[r][threadIdx.x] = q[t * H + h];
      tk[r][threadIdx.x] = k[t * H + h];
    }
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int h = h0 + r;
    const int64_t t = t0 + threadIdx.x;
    if (t < N && h < H) {
      qt[(int64_t)h * N + t] = (int32_t)tq[threadIdx.x][r];
      kt[(int64_t)h * N + t] = (int32_t)tk[threadIdx.x][r];
    }
  }
}

// ------------------------------------------------------------------ matching
// grid = (work items, heads); a work item is kFwdBand consecutive diagonals of one
// sequence; every warp of the CTA walks its own 256 diagonals independently.
__global__ void __launch_bounds__(kFwdWarps * 32)
    hard_match_kernel(Plan plan, const int32_t* __restrict__ qsym,
                      const int32_t* __restrict__ ksym, int64_t sym_seq_stride,
                      int64_t sym_head_stride, int H, int W,
                      unsigned long long* __restrict__ best, const int32_t* __restrict__ run_flag) {
  if (run_flag != nullptr && *run_flag == 0) return;   // only needed when the prefilter gave up
  int seq, local;
  if (!find_item(plan, blockIdx.x, &seq, &local)) return;
  const int h = blockIdx.y;
  const int start = plan.seg_start[seq];
  const int len = plan.seg_len[seq];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int delta0 = 1 + local * kFwdBand + warp * (32 * kFwdPerLane);
  if (delta0 > len - 1) return;
  const bool dense = plan.cu_seqlens == nullptr;
  const int64_t sym_base =
      (int64_t)seq * sym_seq_stride + (int64_t)h * sym_head_stride + (dense ? 0 : start);
  const int32_t* __restrict__ q = qsym + sym_base;
  const int32_t* __restrict__ k = ksym + sym_base;

  int run[kFwdPerLane];
#pragma unroll
  for (int r = 0; r < kFwdPerLane; ++r) run[r] = 0;

  for (int i = delta0; i < len; ++i) {
    const int qi = __ldg(q + i);
    int best_len = 0, best_route = 0;
    const int jbase = i - delta0 - lane;
#pragma unroll
    for (int r = 0; r < kFwdPerLane; ++r) {
      const int j = jbase - r * 32;
      int l = 0;
      if (j >= 0) {
        const int kj = __ldg(k + j);
        l = (kj == qi) ? min(run[r] + 1, W) : 0;
      }
      run[r] = l;
      if (l > best_len) {  // r ascending = route descending: strict > keeps the latest
        best_len = l;
        best_route = j + 1;
      }
    }
    const int row_len = __reduce_max_sync(0xffffffffu, best_len);
    if (row_len > 0) {
      const int row_route =
          __reduce_max_sync(0xffffffffu, best_len == row_len ? best_route : 0);
      if (lane == 0) {
        const unsigned long long key =
            ((unsigned long long)(unsigned)row_len << 32) | (unsigned)row_route;
        unsigned long long* slot = best + ((int64_t)(start + i) * H + h);
        if (*reinterpret_cast<volatile unsigned long long*>(slot) < key) atomicMax(slot, key);
      }
    }
  }
}

// Fast matcher for horizons below 2048 and sequences below 2^21 tokens: the candidate of a
// cell is one 32-bit key (run length << 21 | route), so the row winner is a plain integer
// max.  A CTA of 256 threads owns kFwdBand diagonals (four per thread), stages the key
// symbols of a 32-row block in shared memory, reduces the winner of a row with one
// redux.sync per warp, merges the warps through a shared-memory atomicMax and issues at most
// one global 64-bit atomicMax per row and block.
constexpr int kMatchRows = 32;
constexpr int kMatchThreads = 256;
constexpr int kMatchPerThread = kFwdBand / kMatchThreads;   // 4
constexpr int kMatchWin = kFwdBand + kMatchRows;

template <bool kRamp>
__device__ __forceinline__ void match_rows(int nrows, int tid, int lane, int W, int cmin,
                                           const int* s_q, const int* s_k, unsigned* s_best,
                                           int (&run)[kMatchPerThread], int abase) {
  for (int r = 0; r < nrows; ++r) {
    const int qi = s_q[r];
    unsigned best = 0;
#pragma unroll
    for (int u = 0; u < kMatchPerThread; ++u) {
      const int c = kFwdBand - 1 - tid - u * kMatchThreads + r;   // window column of this cell
      bool eq = s_k[c] == qi;
      if (kRamp) eq = eq && c >= cmin;                            // columns before the sequence
      const int l = eq ? min(run[u] + 1, W) : 0;
      run[u] = l;
      const unsigned key = ((unsigned)l << 21) + (unsigned)(abase + c);   // route = jwin0 + c + 1
      if (eq) best = max(best, key);
    }
    const unsigned wbest = __reduce_max_sync(0xffffffffu, best);
    if (lane == 0 && wbest > 0) atomicMax(s_best + r, wbest);
  }
}

__global__ void __launch_bounds__(kMatchThreads)
    hard_match_fast_kernel(Plan plan, const int32_t* __restrict__ qsym,
                           const int32_t* __restrict__ ksym, int64_t sym_seq_stride,
                           int64_t sym_head_stride, int H, int W,
                           unsigned long long* __restrict__ best,
                           const int32_t* __restrict__ run_flag) {
  if (run_flag != nullptr && *run_flag == 0) return;   // only needed when the prefilter gave up
  __shared__ int s_k[kMatchWin];
  __shared__ int s_q[kMatchRows];
  __shared__ unsigned s_best[kMatchRows];
  const int slot = blockIdx.x / H;
  int seq, local;
  if (!find_item(plan, slot, &seq, &local)) return;
  const int h = blockIdx.x - slot * H;
  const int start = plan.seg_start[seq];
  const int len = plan.seg_len[seq];
  const int tid = threadIdx.x, lane = tid & 31;
  const int dmin = 1 + local * kFwdBand, dmax = dmin + kFwdBand - 1;
  const bool dense = plan.cu_seqlens == nullptr;
  const int64_t sym_base =
      (int64_t)seq * sym_seq_stride + (int64_t)h * sym_head_stride + (dense ? 0 : start);
  const int32_t* __restrict__ q = qsym + sym_base;
  const int32_t* __restrict__ k = ksym + sym_base;
  int run[kMatchPerThread];
#pragma unroll
  for (int u = 0; u < kMatchPerThread; ++u) run[u] = 0;

  for (int i0 = dmin; i0 < len; i0 = (i0 / kMatchRows + 1) * kMatchRows) {
    const int i1 = min((i0 / kMatchRows + 1) * kMatchRows - 1, len - 1);
    const int nrows = i1 - i0 + 1;
    const int jwin0 = i0 - dmax;   // key column of window index 0
    __syncthreads();
    for (int c = tid; c < nrows + kFwdBand - 1; c += kMatchThreads) {
      const int j = jwin0 + c;
      s_k[c] = (j >= 0 && j < len - 1) ? __ldg(k + j) : 0;
    }
    if (tid < nrows) {
      s_q[tid] = __ldg(q + i0 + tid);
      s_best[tid] = 0;
    }
    __syncthreads();
    if (jwin0 < 0)
      match_rows<true>(nrows, tid, lane, W, -jwin0, s_q, s_k, s_best, run, jwin0 + 1);
    else
      match_rows<false>(nrows, tid, lane, W, 0, s_q, s_k, s_best, run, jwin0 + 1);
    __syncthreads();
    if (tid < nrows && s_best[tid] > 0) {
      const unsigned key = s_best[tid];
      const unsigned long long wide =
          ((unsigned long long)(key >> 21) << 32) | (unsigned long long)(key & 0x1FFFFFu);
      atomicMax(best + ((int64_t)(start + i0 + tid) * H + h), wide);
    }
  }
}

// ------------------------------------------------- bit-parallel matcher (D <= 8)
// The matcher itself is bit_match_row (bit_match.cuh).  Here: the occurrence bitmaps of the
// key symbols over the packed token axis, [H][2^D][mask_words], and the kernel that gives one
// warp to every (token, head) and writes the row winner without atomics.

// Occurrence bitmaps: one warp per 32 consecutive tokens of one head; the lanes that share a
// symbol are found with match.any and the lowest of them stores the word.
__global__ void build_match_masks_kernel(Plan plan, const int32_t* __restrict__ ksym, int64_t N,
                                         int H, int D, int64_t sym_seq_stride,
                                         int64_t sym_head_stride, uint32_t* __restrict__ masks,
                                         int64_t mask_words) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t words = (N + 31) >> 5;
  if (warp_id >= words * H) return;
  const int h = (int)(warp_id / words);
  const int64_t word = warp_id - (int64_t)h * words;
  const int64_t g = word * 32 + lane;
  // lanes past the end get distinct out-of-range symbols so that they match nobody
  unsigned sym = 0x80000000u | (unsigned)lane;
  if (g < N) {
    int start = 0, len = 0;
    const int seq = find_segment(plan, g, &start, &len);
    if (seq >= 0) {
      const bool dense = plan.cu_seqlens == nullptr;
      const int64_t idx = (int64_t)seq * sym_seq_stride + (int64_t)h * sym_head_stride +
                          (dense ? g - start : g);
      sym = (unsigned)ksym[idx];
    }
  }
  const unsigned peers = __match_any_sync(0xffffffffu, sym);
  if (sym < (1u << D) && lane == __ffs(peers) - 1)
    masks[(((int64_t)h << D) + sym) * mask_words + word] = peers;
}

constexpr int kBitsWarps = 8;

__global__ void __launch_bounds__(kBitsWarps * 32)
    hard_match_bits_kernel(Plan plan, const int32_t* __restrict__ qsym,
                           const uint32_t* __restrict__ masks, int64_t N, int H, int D, int W,
                           int64_t mask_words, int64_t sym_seq_stride, int64_t sym_head_stride,
                           unsigned long long* __restrict__ best) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kBitsWarps + (threadIdx.x >> 5);
  if (row >= N * H) return;
  // head-major order: neighbouring warps work on neighbouring rows of one head's bitmaps
  const int h = (int)(row / N);
  const int64_t g = row - (int64_t)h * N;
  unsigned long long* out = best + g * H + h;
  int start = 0, len = 0;
  const int seq = find_segment(plan, g, &start, &len);
  const int i = (int)(g - start);
  if (seq < 0 || i == 0) {
    if (lane == 0) *out = 0ull;
    return;
  }
  const bool dense = plan.cu_seqlens == nullptr;
  const int32_t* __restrict__ q = qsym + (int64_t)seq * sym_seq_stride +
                                  (int64_t)h * sym_head_stride + (dense ? 0 : start);
  __shared__ BitCandidate queues[kBitsWarps][kBitQueue];
  const unsigned long long key = bit_match_row(q, masks + ((int64_t)h << D) * mask_words, mask_words,
                                               start, i, W, lane, queues[threadIdx.x >> 5]);
  if (lane == 0) *out = key;
}

// --------------------------------------- hashed prefilter for wide symbols (D > 8)
// Symbols of up to 32 bits are hashed to 8 bits and the key stream is indexed by the same
// occurrence bitmaps as above.  The level-1 word of a row then holds every true candidate plus
// about 1/256 of the other positions; each set bit is verified against the real symbols and
// extended backwards exactly.  Rows with more than kHashTrueLimit genuine candidates (periodic or
// constant streams) would cost O(candidates x horizon): they raise a flag instead, and the
// run-length matcher, whose cost does not depend on the data, then redoes the launch (its
// atomicMax merges the same exact winners, so rows already resolved keep their value).
constexpr int kHashTrueLimit = 48;

__device__ __forceinline__ unsigned hash8(unsigned sym) { return (sym * 0x9E3779B1u) >> 24; }

__global__ void build_hash_masks_kernel(Plan plan, const int32_t* __restrict__ ksym, int64_t N,
                                        int H, int64_t sym_seq_stride, int64_t sym_head_stride,
                                        uint32_t* __restrict__ masks, int64_t mask_words) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t words = (N + 31) >> 5;
  if (warp_id >= words * H) return;
  const int h = (int)(warp_id / words);
  const int64_t word = warp_id - (int64_t)h * words;
  const int64_t g = word * 32 + lane;
  unsigned sym = 0x80000000u | (unsigned)lane;   // lanes past the end match nobody
  if (g < N) {
    int start = 0, len = 0;
    const int seq = find_segment(plan, g, &start, &len);
    if (seq >= 0) {
      const bool dense = plan.cu_seqlens == nullptr;
      sym = hash8((unsigned)ksym[(int64_t)seq * sym_seq_stride + (int64_t)h * sym_head_stride +
                                 (dense ? g - start : g)]);
    }
  }
  const unsigned peers = __match_any_sync(0xffffffffu, sym);
  if (sym < 256u && lane == __ffs(peers) - 1)
    masks[(((int64_t)h << 8) + sym) * mask_words + word] = peers;
}

__global__ void __launch_bounds__(kBitsWarps * 32)
    hard_match_hashed_kernel(Plan plan, const int32_t* __restrict__ qsym,
                             const int32_t* __restrict__ ksym, const uint32_t* __restrict__ masks,
                             int64_t N, int H, int W, int64_t mask_words, int64_t sym_seq_stride,
                             int64_t sym_head_stride, unsigned long long* __restrict__ best,
                             int32_t* __restrict__ overflow_flag) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kBitsWarps + (threadIdx.x >> 5);
  if (row >= N * H) return;
  const int h = (int)(row / N);
  const int64_t g_row = row - (int64_t)h * N;
  unsigned long long* out = best + g_row * H + h;
  int start = 0, len = 0;
  const int seq = find_segment(plan, g_row, &start, &len);
  const int i = (int)(g_row - start);
  if (seq < 0 || i == 0) {
    if (lane == 0) *out = 0ull;
    return;
  }
  const bool dense = plan.cu_seqlens == nullptr;
  const int64_t base = (int64_t)seq * sym_seq_stride + (int64_t)h * sym_head_stride +
                       (dense ? 0 : start);
  const int32_t* __restrict__ q = qsym + base;       // q[p], k[p]: position p of this sequence
  const int32_t* __restrict__ k = ksym + base;
  const int q_i = q[i];
  const uint32_t* __restrict__ e = masks + (((int64_t)h << 8) + hash8((unsigned)q_i)) * mask_words;
  const int g_lo = start, g_hi = start + i - 1;
  const int w_lo = g_lo >> 5, w_hi = g_hi >> 5;
  int best_len = 0, best_route = 0, genuine = 0;
  bool stop = false;                                  // uniform: set from votes only
  for (int wb = w_hi; wb >= w_lo && !stop; wb -= 32) {    // newest positions first
    const int w = wb - lane;
    uint32_t bits = w >= w_lo ? e[w] : 0u;
    if (w == w_hi) bits &= 0xffffffffu >> (31 - (g_hi & 31));
    if (w == w_lo) bits &= 0xffffffffu << (g_lo & 31);
    // every lane walks the set bits of its own word, newest first (no warp primitive inside)
    while (bits != 0u) {
      const int bit = 31 - __clz(bits);
      bits &= ~(1u << bit);
      const int j = 32 * w + bit - start;             // key position inside the sequence
      if (k[j] != q_i) continue;                      // hash collision
      if (++genuine > kHashTrueLimit) break;          // bounded work per lane and row
      int length = 1;
      const int cap = min(W, j + 1);                  // a match cannot start before the sequence
      while (length < cap && k[j - length] == q[i - length]) ++length;
      if (length > best_len || (length == best_len && j + 1 > best_route)) {
        best_len = length;
        best_route = j + 1;
      }
    }
    const bool over = __any_sync(0xffffffffu, genuine > kHashTrueLimit);
    // newer positions were examined first: nothing older can beat a match at the horizon
    stop = over || __reduce_max_sync(0xffffffffu, best_len) >= W;
    if (over) best_len = 0;
  }
  const bool over = __any_sync(0xffffffffu, genuine > kHashTrueLimit);
  const int row_len = over ? 0 : __reduce_max_sync(0xffffffffu, best_len);
  const int row_route =
      over ? 0 : __reduce_max_sync(0xffffffffu, best_len == row_len ? best_route : 0);
  if (lane == 0) {
    *out = row_len > 0 ? ((unsigned long long)(unsigned)row_len << 32) | (unsigned)row_route : 0ull;
    if (over) atomicExch(overflow_flag, 1);
  }
}

// ------------------------------------------------------------------- gather
// One thread per (token, head, chunk of value components): 16 bytes of output per thread when
// the rows allow it (128-bit loads of the value row, one 128-bit store), else element by element.
// OutT = T writes the operator's output in the input dtype; OutT = int8_t writes -1 / 0 / +1
// bytes for a consumer that takes the routed signs as integers.
template <typename T, typename OutT>
__global__ void gather_output_kernel(Plan plan, const unsigned long long* __restrict__ best,
                                     const T* __restrict__ v, int64_t N, int H, int Hv, int Dv,
                                     int chunk, int vec, OutT* __restrict__ out,
                                     int32_t* __restrict__ route_token) {
  const int chunks = (Dv + chunk - 1) / chunk;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= N * H * chunks) return;
  const int c = (int)(idx % chunks);
  const int64_t th = idx / chunks;
  const int64_t token = th / H;
  const int h = (int)(th - token * H);
  const int route = (int)(best[th] & 0xffffffffull);
  int start = 0, len = 0;
  int64_t src_token = -1;
  if (route > 0 && find_segment(plan, token, &start, &len) >= 0) src_token = (int64_t)start + route;
  if (c == 0 && route_token) route_token[th] = (int32_t)src_token;
  OutT* o = out + th * Dv;
  const int d0 = c * chunk, d1 = min(Dv, d0 + chunk);
  const T* src = src_token < 0 ? nullptr : v + (src_token * Hv + h / (H / Hv)) * Dv;
  if (vec) {
    // `chunk` components: 16 bytes of OutT; the value row is read in 16-byte words
    constexpr int kOutPer = 16 / (int)sizeof(OutT);
    constexpr int kInPer = 16 / (int)sizeof(T);
    alignas(16) OutT vals[kOutPer];
#pragma unroll
    for (int x = 0; x < kOutPer; ++x) vals[x] = (OutT)0;
    if (src != nullptr) {
#pragma unroll
      for (int wd = 0; wd < kOutPer / kInPer; ++wd) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + d0) + wd);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int x = 0; x < kInPer; ++x)
          vals[wd * kInPer + x] = positive<T>(e[x]) ? (OutT)1.0f : (OutT)-1.0f;
      }
    }
    *reinterpret_cast<uint4*>(o + d0) = *reinterpret_cast<const uint4*>(vals);
    return;
  }
  for (int d = d0; d < d1; ++d)
    o[d] = src == nullptr ? (OutT)0 : positive<T>(src[d]) ? (OutT)1.0f : (OutT)-1.0f;
}

__global__ void inference_finish_kernel(Plan plan, const unsigned long long* __restrict__ best,
                                        const float* __restrict__ payload, int64_t N, int H,
                                        int Hp, int Dp, float* __restrict__ out,
                                        int64_t* __restrict__ matched_end) {
  const int64_t th = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (th >= N * H) return;
  const int64_t token = th / H;
  const int h = (int)(th - token * H);
  const int route = (int)(best[th] & 0xffffffffull);
  int start = 0, len = 0;
  const bool hit = route > 0 && find_segment(plan, token, &start, &len) >= 0;
  matched_end[th] = hit ? (int64_t)route - 1 : -1;
  if (out) {
    float* o = out + th * Dp;
    if (hit) {
      const float* src = payload + (((int64_t)start + route) * Hp + h / (H / Hp)) * Dp;
      for (int d = 0; d < Dp; ++d) o[d] = src[d];
    } else {
      for (int d = 0; d < Dp; ++d) o[d] = 0.0f;
    }
  }
}

// Splits the winners into the selected route (local index a, 0 = null) and its match length.
__global__ void route_inspect_kernel(const unsigned long long* __restrict__ best, int64_t count,
                                     int32_t* __restrict__ route, int32_t* __restrict__ length) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= count) return;
  const unsigned long long key = best[idx];
  if (route) route[idx] = (int32_t)(key & 0xffffffffull);
  if (length) length[idx] = (int32_t)(key >> 32);
}

}  // namespace

int launch_route_inspect(const unsigned long long* best, int64_t count, int32_t* route,
                         int32_t* length, cudaStream_t stream) {
  ProfileScope prof("route_inspect", stream);
  const int threads = 256;
  route_inspect_kernel<<<(unsigned)((count + threads - 1) / threads), threads, 0, stream>>>(
      best, count, route, length);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_pack_symbols(const void* q, const void* k, int dtype, int64_t N, int H, int D,
                        int dense, int64_t uniform_len, int32_t* pq, int32_t* pk,
                        cudaStream_t stream) {
  ProfileScope prof("pack_symbols", stream);
  const int threads = 256;
  const int64_t blocks = (N * H + threads - 1) / threads;
  const int esize = dtype == ROSA_B200_F32 ? 4 : 2;
  const auto aligned = [](const void* p) { return p == nullptr || ((uintptr_t)p & 15u) == 0; };
  const int vec = (D * esize) % 16 == 0 && aligned(q) && aligned(k);
  if (dtype == ROSA_B200_F32)
    pack_symbols_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        (const float*)q, (const float*)k, N, H, D, dense, uniform_len, vec, pq, pk);
  else if (dtype == ROSA_B200_F16)
    pack_symbols_kernel<__half><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __half*)q, (const __half*)k, N, H, D, dense, uniform_len, vec, pq, pk);
  else
    pack_symbols_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, N, H, D, dense, uniform_len, vec, pq, pk);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_transpose_symbols(const uint32_t* q, const uint32_t* k, int64_t N, int H, int32_t* qt,
                             int32_t* kt, cudaStream_t stream) {
  ProfileScope prof("transpose_symbols", stream);
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((H + 31) / 32)), block(32, 8);
  transpose_symbols_kernel<<<grid, block, 0, stream>>>(q, k, N, H, qt, kt);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

int launch_hard_match(const FwdArgs& a, int items_upper, cudaStream_t stream) {
  if (a.match_masks != nullptr) {
    if (a.N == 0) return 0;
    {
      ProfileScope prof("build_match_masks", stream);
      ROSA_CUDA_OK(cudaMemsetAsync(a.match_masks, 0,
                                   ((size_t)a.H << a.D) * (size_t)a.mask_words * sizeof(uint32_t),
                                   stream));
      const int64_t warps = ((a.N + 31) >> 5) * a.H;
      build_match_masks_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
          a.plan, a.packed_k, a.N, a.H, a.D, a.sym_seq_stride, a.sym_head_stride, a.match_masks,
          a.mask_words);
      ROSA_CUDA_OK(cudaGetLastError());
    }
    ProfileScope prof("hard_match", stream);
    const int64_t rows = a.N * a.H;
    hard_match_bits_kernel<<<(unsigned)((rows + kBitsWarps - 1) / kBitsWarps), kBitsWarps * 32, 0,
                             stream>>>(a.plan, a.packed_q, a.match_masks, a.N, a.H, a.D, a.W,
                                       a.mask_words, a.sym_seq_stride, a.sym_head_stride, a.best);
    ROSA_CUDA_OK(cudaGetLastError());
    return 0;
  }
  if (items_upper <= 0) return 0;
  const int32_t* run_flag = nullptr;
  if (a.hash_masks != nullptr && a.N > 0) {
    // wide symbols: hashed prefilter first; the run-length matcher below then only runs when
    // some row had too many genuine candidates (flag in the plan's status words)
    int32_t* flag = a.plan.status + 2;
    {
      ProfileScope prof("build_match_masks", stream);
      ROSA_CUDA_OK(cudaMemsetAsync(a.hash_masks, 0,
                                   ((size_t)a.H << 8) * (size_t)a.mask_words * sizeof(uint32_t),
                                   stream));
      const int64_t warps = ((a.N + 31) >> 5) * a.H;
      build_hash_masks_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
          a.plan, a.packed_k, a.N, a.H, a.sym_seq_stride, a.sym_head_stride, a.hash_masks,
          a.mask_words);
      ROSA_CUDA_OK(cudaGetLastError());
    }
    {
      ProfileScope prof("hard_match_hashed", stream);
      const int64_t rows = a.N * a.H;
      hard_match_hashed_kernel<<<(unsigned)((rows + kBitsWarps - 1) / kBitsWarps), kBitsWarps * 32,
                                 0, stream>>>(a.plan, a.packed_q, a.packed_k, a.hash_masks, a.N, a.H,
                                              a.W, a.mask_words, a.sym_seq_stride,
                                              a.sym_head_stride, a.best, flag);
      ROSA_CUDA_OK(cudaGetLastError());
    }
    run_flag = flag;
  }
  ProfileScope prof("hard_match", stream);
  const int64_t max_len = a.plan.cu_seqlens == nullptr ? a.plan.uniform_len : a.N;
  if (a.W < 2048 && max_len < (1 << 21)) {
    // 32-bit candidate keys: run length in the top 11 bits, route in the low 21
    hard_match_fast_kernel<<<(unsigned)((int64_t)items_upper * a.H), kMatchThreads, 0, stream>>>(
        a.plan, a.packed_q, a.packed_k, a.sym_seq_stride, a.sym_head_stride, a.H, a.W, a.best,
        run_flag);
    ROSA_CUDA_OK(cudaGetLastError());
    return 0;
  }
  dim3 grid((unsigned)items_upper, (unsigned)a.H);
  hard_match_kernel<<<grid, kFwdWarps * 32, 0, stream>>>(a.plan, a.packed_q, a.packed_k,
                                                        a.sym_seq_stride, a.sym_head_stride, a.H,
                                                        a.W, a.best, run_flag);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

namespace {
template <typename T, typename OutT>
int launch_gather_t(const FwdArgs& a, OutT* out, cudaStream_t stream) {
  // vector path: a thread writes 16 bytes of output, i.e. 16 / sizeof(OutT) components, and
  // reads as many value components in 16-byte words
  constexpr int kOutPer = 16 / (int)sizeof(OutT);
  const auto aligned = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
  const bool vec = a.Dv % kOutPer == 0 && aligned(a.v) && aligned(out) &&
                   (a.Dv * (int)sizeof(T)) % 16 == 0 && kOutPer >= 16 / (int)sizeof(T);
  const int chunk = vec ? kOutPer : 8;
  const int chunks = (a.Dv + chunk - 1) / chunk;
  const int threads = 256;
  const int64_t blocks = (a.N * a.H * chunks + threads - 1) / threads;
  gather_output_kernel<T, OutT><<<(unsigned)blocks, threads, 0, stream>>>(
      a.plan, a.best, (const T*)a.v, a.N, a.H, a.Hv, a.Dv, chunk, vec ? 1 : 0, out, a.route_token);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}
}  // namespace

int launch_gather_output(const FwdArgs& a, cudaStream_t stream) {
  ProfileScope prof("gather_output", stream);
  if (a.out_i8 != nullptr) {
    if (a.dtype == ROSA_B200_F32) return launch_gather_t<float, int8_t>(a, a.out_i8, stream);
    if (a.dtype == ROSA_B200_F16) return launch_gather_t<__half, int8_t>(a, a.out_i8, stream);
    return launch_gather_t<__nv_bfloat16, int8_t>(a, a.out_i8, stream);
  }
  if (a.dtype == ROSA_B200_F32) return launch_gather_t<float, float>(a, (float*)a.out, stream);
  if (a.dtype == ROSA_B200_F16) return launch_gather_t<__half, __half>(a, (__half*)a.out, stream);
  return launch_gather_t<__nv_bfloat16, __nv_bfloat16>(a, (__nv_bfloat16*)a.out, stream);
}

int launch_inference_finish(const Plan& plan, const unsigned long long* best, const float* payload,
                            int64_t N, int H, int Hp, int Dp, float* out, int64_t* matched_end,
                            cudaStream_t stream) {
  ProfileScope prof("inference_finish", stream);
  const int threads = 256;
  const int64_t blocks = (N * H + threads - 1) / threads;
  inference_finish_kernel<<<(unsigned)blocks, threads, 0, stream>>>(plan, best, payload, N, H, Hp,
                                                                   Dp, out, matched_end);
  ROSA_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace rosa
