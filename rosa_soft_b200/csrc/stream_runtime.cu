// Streaming hard inference with the per-slot state resident on the GPU: the chunked
// `update_packed` of the reference runtime (rosa_soft/csrc/rosa_runtime.cpp:333-482; per-token
// automaton step :103-133, successor payload :455-467, slot-count fixing :531-556).
//
// The reference keeps one finite-horizon suffix automaton per (slot, head) on the host.  Here
// the state of a (slot, head) is its key-symbol history plus one capped run length per
// diagonal: run[delta] = number of trailing positions p <= last with q[p] == k[p - delta],
// capped at the horizon.  A new query row i extends every diagonal by one cell, so a chunk of n
// tokens on a history of L tokens costs n * (L + n) symbol compares, independent of how the
// stream was chunked before, and the result equals a one-shot pass over the whole stream.
#include "common.cuh"

namespace rosa {

namespace {

constexpr int kStreamThreads = 256;
constexpr int kStreamPer = 4;                                  // diagonals per thread
constexpr int kStreamBand = kStreamThreads * kStreamPer;       // diagonals per CTA
constexpr int kStreamRows = 32;                                // rows per staged block
constexpr int kStreamWin = kStreamBand + kStreamRows;

// slot containing chunk token `token`: the last s with offsets[s] <= token
__device__ __forceinline__ int stream_slot(const int32_t* __restrict__ offsets, int slots,
                                           int64_t token) {
  int lo = 0, hi = slots;
  while (lo + 1 < hi) {
    const int mid = (lo + hi) >> 1;
    if ((int64_t)offsets[mid] <= token) lo = mid; else hi = mid;
  }
  return lo;
}

// Validates the chunk offsets and the capacity; one CTA.  status[0] != 0 makes every later
// kernel of the call a no-op, so a bad call leaves the state untouched.
__global__ void stream_prepare_kernel(const int32_t* __restrict__ offsets, int slots,
                                      int64_t chunk_tokens, const int32_t* __restrict__ lengths,
                                      int64_t capacity, int32_t* status) {
  __shared__ int s_status;
  if (threadIdx.x == 0) s_status = ROSA_B200_STATUS_OK;
  __syncthreads();
  for (int s = threadIdx.x; s <= slots; s += blockDim.x) {
    const int cur = offsets[s];
    if (s == 0 && cur != 0) atomicMax(&s_status, (int)ROSA_B200_STATUS_BAD_FIRST_OFFSET);
    if (s > 0 && cur < offsets[s - 1]) atomicMax(&s_status, (int)ROSA_B200_STATUS_NOT_MONOTONE);
    if (s == slots && (int64_t)cur != chunk_tokens)
      atomicMax(&s_status, (int)ROSA_B200_STATUS_BAD_LAST_OFFSET);
    if (s > 0 && cur >= offsets[s - 1] &&
        (int64_t)lengths[s - 1] + (cur - offsets[s - 1]) > capacity)
      atomicMax(&s_status, (int)ROSA_B200_STATUS_CAPACITY);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    status[0] = s_status;
    status[1] = status[2] = status[3] = 0;
  }
}

// Appends the chunk's key and payload symbols to the histories and clears the winners.
__global__ void stream_append_kernel(const uint8_t* __restrict__ key,
                                     const uint8_t* __restrict__ payload,
                                     const int32_t* __restrict__ offsets, int slots,
                                     int64_t chunk_tokens, int H, int Hp, int qk_mask,
                                     int payload_mask, const int32_t* __restrict__ lengths,
                                     int64_t capacity, uint8_t* __restrict__ key_history,
                                     uint8_t* __restrict__ payload_history,
                                     unsigned long long* __restrict__ best,
                                     const int32_t* __restrict__ status) {
  if (status[0] != 0) return;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int heads = H + Hp;
  if (idx >= chunk_tokens * heads) return;
  const int64_t token = idx / heads;
  const int hh = (int)(idx - token * heads);
  const int s = stream_slot(offsets, slots, token);
  const int64_t pos = (int64_t)lengths[s] + (token - offsets[s]);
  if (hh < H) {
    key_history[((int64_t)s * H + hh) * capacity + pos] = key[token * H + hh] & qk_mask;
    best[token * H + hh] = 0ull;
  } else {
    const int hp = hh - H;
    payload_history[((int64_t)s * Hp + hp) * capacity + pos] =
        payload[token * Hp + hp] & payload_mask;
  }
}

// Candidate of a cell.  Narrow: run << 21 | route in 32 bits (horizon < 2048, history < 2^21).
template <bool kWide>
struct StreamKey;
template <>
struct StreamKey<false> {
  using type = unsigned;
  static __device__ __forceinline__ unsigned make(int run, int route) {
    return ((unsigned)run << 21) + (unsigned)route;
  }
  static __device__ __forceinline__ unsigned warp_max(unsigned v) {
    return __reduce_max_sync(0xffffffffu, v);
  }
  static __device__ __forceinline__ unsigned long long widen(unsigned v) {
    return ((unsigned long long)(v >> 21) << 32) | (unsigned long long)(v & 0x1FFFFFu);
  }
};
template <>
struct StreamKey<true> {
  using type = unsigned long long;
  static __device__ __forceinline__ unsigned long long make(int run, int route) {
    return ((unsigned long long)(unsigned)run << 32) | (unsigned)route;
  }
  static __device__ __forceinline__ unsigned long long warp_max(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
      v = other > v ? other : v;
    }
    return v;
  }
  static __device__ __forceinline__ unsigned long long widen(unsigned long long v) { return v; }
};

// One CTA = kStreamBand diagonals of one (slot, head); rows are the chunk's new positions.
template <bool kWide>
__global__ void __launch_bounds__(kStreamThreads)
    stream_match_kernel(const uint8_t* __restrict__ query, const int32_t* __restrict__ offsets,
                        int slots, int H, int qk_mask, int W,
                        const int32_t* __restrict__ lengths, int64_t capacity,
                        const uint8_t* __restrict__ key_history, uint16_t* __restrict__ run_state,
                        unsigned long long* __restrict__ best,
                        const int32_t* __restrict__ status) {
  using KeyT = typename StreamKey<kWide>::type;
  __shared__ int s_k[kStreamWin];
  __shared__ int s_q[kStreamRows];
  __shared__ KeyT s_best[kStreamRows];
  if (status[0] != 0) return;
  // heads fastest, then slots, then bands: neighbouring CTAs carry the same amount of work
  const int h = blockIdx.x % H;
  const int s = (blockIdx.x / H) % slots;
  const int band = blockIdx.x / (H * slots);
  const int L = lengths[s];
  const int n = offsets[s + 1] - offsets[s];
  const int Ln = L + n;
  const int dmin = 1 + band * kStreamBand, dmax = dmin + kStreamBand - 1;
  if (n == 0 || dmin > Ln - 1) return;
  const int tid = threadIdx.x, lane = tid & 31;
  const uint8_t* __restrict__ kh = key_history + ((int64_t)s * H + h) * capacity;
  uint16_t* __restrict__ rs = run_state + ((int64_t)s * H + h) * capacity;
  const uint8_t* __restrict__ qc = query + (int64_t)offsets[s] * H + h;

  int run[kStreamPer];
#pragma unroll
  for (int u = 0; u < kStreamPer; ++u) {
    const int delta = dmin + tid + u * kStreamThreads;
    run[u] = delta <= L - 1 ? (int)rs[delta] : 0;   // diagonals that had a cell before this chunk
  }

  for (int i0 = max(L, dmin); i0 < Ln; i0 = (i0 / kStreamRows + 1) * kStreamRows) {
    const int i1 = min((i0 / kStreamRows + 1) * kStreamRows - 1, Ln - 1);
    const int nrows = i1 - i0 + 1;
    const int jwin0 = i0 - dmax;                    // key position of window index 0
    __syncthreads();
    for (int c = tid; c < nrows + kStreamBand - 1; c += kStreamThreads) {
      const int j = jwin0 + c;
      s_k[c] = (j >= 0 && j < Ln) ? (int)kh[j] : 0;
    }
    if (tid < nrows) {
      s_q[tid] = (int)(qc[(int64_t)(i0 + tid - L) * H] & qk_mask);
      s_best[tid] = 0;
    }
    __syncthreads();
    const int cmin = jwin0 < 0 ? -jwin0 : 0;        // window indices before the stream's start
    for (int r = 0; r < nrows; ++r) {
      const int qi = s_q[r];
      KeyT top = 0;
#pragma unroll
      for (int u = 0; u < kStreamPer; ++u) {
        const int c = kStreamBand - 1 - tid - u * kStreamThreads + r;
        const bool eq = s_k[c] == qi && c >= cmin;
        const int l = eq ? min(run[u] + 1, W) : 0;
        run[u] = l;
        const KeyT key = StreamKey<kWide>::make(l, jwin0 + c + 1);   // route = key position + 1
        if (eq && key > top) top = key;
      }
      const KeyT wtop = StreamKey<kWide>::warp_max(top);
      if (lane == 0 && wtop > 0) atomicMax(s_best + r, wtop);
    }
    __syncthreads();
    if (tid < nrows && s_best[tid] > 0)
      atomicMax(best + ((int64_t)(offsets[s] + i0 + tid - L) * H + h),
                StreamKey<kWide>::widen(s_best[tid]));
  }
#pragma unroll
  for (int u = 0; u < kStreamPer; ++u) {
    const int delta = dmin + tid + u * kStreamThreads;
    if (delta <= Ln - 1) rs[delta] = (uint16_t)run[u];
  }
}

__global__ void stream_finish_kernel(const unsigned long long* __restrict__ best,
                                     const int32_t* __restrict__ offsets, int slots,
                                     int64_t chunk_tokens, int H, int Hp, int64_t capacity,
                                     const uint8_t* __restrict__ payload_history,
                                     uint8_t* __restrict__ output,
                                     int64_t* __restrict__ matched_end,
                                     const int32_t* __restrict__ status) {
  if (status[0] != 0) return;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= chunk_tokens * H) return;
  const int64_t token = idx / H;
  const int h = (int)(idx - token * H);
  const int s = stream_slot(offsets, slots, token);
  const int64_t route = (int64_t)(best[idx] & 0xffffffffull);   // successor position, 0 = null
  matched_end[idx] = route - 1;
  output[idx] = route > 0 ? payload_history[((int64_t)s * Hp + h / (H / Hp)) * capacity + route]
                          : (uint8_t)0;
}

__global__ void stream_commit_kernel(const int32_t* __restrict__ offsets, int slots,
                                     int32_t* __restrict__ lengths,
                                     const int32_t* __restrict__ status) {
  if (status[0] != 0) return;
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < slots) lengths[s] += offsets[s + 1] - offsets[s];
}

}  // namespace

int launch_stream_update(const StreamArgs& a, cudaStream_t stream) {
  {
    ProfileScope prof("stream_prepare", stream);
    stream_prepare_kernel<<<1, 256, 0, stream>>>(a.offsets, a.slots, a.chunk_tokens, a.lengths,
                                                 a.capacity, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  if (a.chunk_tokens == 0) return 0;
  const int threads = 256;
  {
    ProfileScope prof("stream_append", stream);
    const int64_t total = a.chunk_tokens * (a.H + a.Hp);
    stream_append_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
        a.key, a.payload, a.offsets, a.slots, a.chunk_tokens, a.H, a.Hp, a.qk_mask, a.payload_mask,
        a.lengths, a.capacity, a.key_history, a.payload_history, a.best, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  {
    ProfileScope prof("stream_match", stream);
    const int64_t bands = std::max<int64_t>(1, (a.max_length_after - 1 + kStreamBand - 1) / kStreamBand);
    const int64_t grid = bands * a.slots * a.H;
    if (a.W < 2048 && a.capacity < (1 << 21))
      stream_match_kernel<false><<<(unsigned)grid, kStreamThreads, 0, stream>>>(
          a.query, a.offsets, a.slots, a.H, a.qk_mask, a.W, a.lengths, a.capacity, a.key_history,
          a.run_state, a.best, a.status);
    else
      stream_match_kernel<true><<<(unsigned)grid, kStreamThreads, 0, stream>>>(
          a.query, a.offsets, a.slots, a.H, a.qk_mask, a.W, a.lengths, a.capacity, a.key_history,
          a.run_state, a.best, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  {
    ProfileScope prof("stream_finish", stream);
    const int64_t total = a.chunk_tokens * a.H;
    stream_finish_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, stream>>>(
        a.best, a.offsets, a.slots, a.chunk_tokens, a.H, a.Hp, a.capacity, a.payload_history,
        a.output, a.matched_end, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
    stream_commit_kernel<<<(a.slots + threads - 1) / threads, threads, 0, stream>>>(
        a.offsets, a.slots, a.lengths, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  return 0;
}

}  // namespace rosa
