// Streaming hard inference with the per-slot state resident on the GPU: the chunked
// `update_packed` of the reference runtime (rosa_soft/csrc/rosa_runtime.cpp:333-482; per-token
// automaton step :103-133, successor payload :455-467, slot-count fixing :531-556).
//
// The reference keeps one finite-horizon suffix automaton per (slot, head) on the host.  Here
// the state of a (slot, head) is the query history plus one occurrence bitmap per key symbol
// (bit p of bitmap s set iff the key symbol at position p is s; symbols have at most 8 bits).
// A new row is resolved by the bit-parallel matcher of bit_match.cuh: per 32 key positions it
// costs as many AND steps as the longest match in that word is long, so a chunk of n tokens on
// a history of L tokens costs about n * (L / 32) * (a few levels) word operations, and the
// result equals a one-shot pass over the whole stream however it was chunked.
#include "common.cuh"
#include "bit_match.cuh"

namespace rosa {

namespace {

constexpr int kStreamWarps = 8;   // rows per CTA of the matcher

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

// Appends the chunk to the state: query and payload symbols to their histories, every key
// symbol as one bit of its occurrence bitmap (atomic OR: several tokens of a chunk share a word).
__global__ void stream_append_kernel(const uint8_t* __restrict__ query,
                                     const uint8_t* __restrict__ key,
                                     const uint8_t* __restrict__ payload,
                                     const int32_t* __restrict__ offsets, int slots,
                                     int64_t chunk_tokens, int H, int Hp, int qk_bits, int qk_mask,
                                     int payload_mask, const int32_t* __restrict__ lengths,
                                     int64_t capacity, uint32_t* __restrict__ key_masks,
                                     uint8_t* __restrict__ query_history,
                                     uint8_t* __restrict__ payload_history,
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
    const int64_t sh = (int64_t)s * H + hh;
    query_history[sh * capacity + pos] = query[token * H + hh] & qk_mask;
    const int sym = key[token * H + hh] & qk_mask;
    atomicOr(key_masks + ((sh << qk_bits) + sym) * (capacity >> 5) + (pos >> 5), 1u << (pos & 31));
  } else {
    const int hp = hh - H;
    payload_history[((int64_t)s * Hp + hp) * capacity + pos] =
        payload[token * Hp + hp] & payload_mask;
  }
}

// One warp per (chunk token, head), head-major so that neighbouring warps read the same
// bitmaps.  Writes (match length << 32 | successor position) or 0.
__global__ void __launch_bounds__(kStreamWarps * 32)
    stream_match_kernel(const int32_t* __restrict__ offsets, int slots, int64_t chunk_tokens,
                        int H, int qk_bits, int W, const int32_t* __restrict__ lengths,
                        int64_t capacity, const uint32_t* __restrict__ key_masks,
                        const uint8_t* __restrict__ query_history,
                        unsigned long long* __restrict__ best,
                        const int32_t* __restrict__ status) {
  __shared__ BitCandidate queues[kStreamWarps][kBitQueue];
  if (status[0] != 0) return;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kStreamWarps + (threadIdx.x >> 5);
  if (row >= chunk_tokens * H) return;
  const int h = (int)(row / chunk_tokens);
  const int64_t token = row - (int64_t)h * chunk_tokens;
  const int s = stream_slot(offsets, slots, token);
  const int i = lengths[s] + (int)(token - offsets[s]);    // position of the row in its stream
  unsigned long long key = 0ull;
  if (i > 0) {
    const int64_t sh = (int64_t)s * H + h;
    key = bit_match_row(query_history + sh * capacity,
                        key_masks + (sh << qk_bits) * (capacity >> 5), capacity >> 5, 0, i, W,
                        lane, queues[threadIdx.x >> 5]);
  }
  if (lane == 0) best[token * H + h] = key;
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
        a.query, a.key, a.payload, a.offsets, a.slots, a.chunk_tokens, a.H, a.Hp, a.qk_bits,
        a.qk_mask, a.payload_mask, a.lengths, a.capacity, a.key_masks, a.query_history,
        a.payload_history, a.status);
    ROSA_CUDA_OK(cudaGetLastError());
  }
  {
    ProfileScope prof("stream_match", stream);
    const int64_t rows = a.chunk_tokens * a.H;
    stream_match_kernel<<<(unsigned)((rows + kStreamWarps - 1) / kStreamWarps), kStreamWarps * 32,
                          0, stream>>>(a.offsets, a.slots, a.chunk_tokens, a.H, a.qk_bits, a.W,
                                       a.lengths, a.capacity, a.key_masks, a.query_history, a.best,
                                       a.status);
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
