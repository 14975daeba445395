// Shared declarations of the rosa_soft_b200 CUDA library (sm_100a only).
//
// Geometry used by every kernel
// -----------------------------
// One sequence of one head is a lower-triangular problem over cells (i, j):
// query row i in [1, L), key column j in [0, i); route index a = j + 1.  All
// recurrences of the operator run along diagonals delta = i - j >= 1, so a cell
// is addressed as (delta, n = j).  Work is split into *bands* of consecutive
// diagonals; one thread owns one diagonal and all threads of a warp sit on the
// same row i at the same time, which makes every symbol / value / scratch access
// of a warp contiguous.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rosa_soft_b200.h"

namespace rosa {

// ------------------------------------------------------------------ constants
constexpr int kVjpBand = 256;      // diagonals per surrogate-VJP band (= CTA threads)
constexpr int kVjpRows = 16;       // rows per checkpointed block of the VJP sweeps
constexpr int kVjpWarps = kVjpBand / 32;
constexpr int kFwdWarps = 4;       // warps per hard-forward CTA
constexpr int kFwdPerLane = 8;     // diagonals per lane in the hard-forward matcher
constexpr int kFwdBand = kFwdWarps * 32 * kFwdPerLane;  // 1024 diagonals per CTA

// --------------------------------------------------------------- segment plan
// Written by build_plan_kernel from cu_seqlens (or from the uniform description
// of a dense batch); read by every other kernel.  `band` is the number of
// diagonals one work item covers (band * group for grouped VJP items).
struct Plan {
  int32_t* status;        // [4]  status[0] = rosa_b200_status
  int32_t* seg_start;     // [S]  first token of each sequence
  int32_t* seg_len;       // [S]  length of each sequence (0 for all when invalid)
  int32_t* item_prefix;   // [S+1] exclusive prefix of work items per sequence (per head)
  int64_t* row_prefix;    // [S+1] exclusive prefix of items_s * len_s  (partial-row slots)
  int64_t* ck_prefix;     // [S+1] exclusive prefix of checkpoint blocks per (sequence, head)
  const int32_t* cu_seqlens;  // nullptr for the dense description
  int64_t N;
  int32_t S;
  int32_t uniform_len;
  int32_t item_diagonals;  // diagonals per work item
  int32_t keep_mma_status; // non-zero: status[1] of an earlier slice of the same call survives
};

struct PlanLayout {
  size_t status_off, seg_start_off, seg_len_off, item_prefix_off, row_prefix_off, ck_prefix_off;
  size_t bytes;
};

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

inline PlanLayout plan_layout(size_t base, int64_t S) {
  PlanLayout l;
  size_t off = base;
  l.status_off = off;       off = align_up(off + 4 * sizeof(int32_t));
  l.seg_start_off = off;    off = align_up(off + (size_t)S * sizeof(int32_t));
  l.seg_len_off = off;      off = align_up(off + (size_t)S * sizeof(int32_t));
  l.item_prefix_off = off;  off = align_up(off + (size_t)(S + 1) * sizeof(int32_t));
  l.row_prefix_off = off;   off = align_up(off + (size_t)(S + 1) * sizeof(int64_t));
  l.ck_prefix_off = off;    off = align_up(off + (size_t)(S + 1) * sizeof(int64_t));
  l.bytes = off - base;
  return l;
}

inline Plan make_plan(void* ws, const PlanLayout& l, const int32_t* cu, int64_t N, int64_t S,
                      int64_t uniform_len, int item_diagonals) {
  char* b = static_cast<char*>(ws);
  Plan p;
  p.status = reinterpret_cast<int32_t*>(b + l.status_off);
  p.seg_start = reinterpret_cast<int32_t*>(b + l.seg_start_off);
  p.seg_len = reinterpret_cast<int32_t*>(b + l.seg_len_off);
  p.item_prefix = reinterpret_cast<int32_t*>(b + l.item_prefix_off);
  p.row_prefix = reinterpret_cast<int64_t*>(b + l.row_prefix_off);
  p.ck_prefix = reinterpret_cast<int64_t*>(b + l.ck_prefix_off);
  p.cu_seqlens = cu;
  p.N = N;
  p.S = (int32_t)S;
  p.uniform_len = (int32_t)uniform_len;
  p.item_diagonals = item_diagonals;
  p.keep_mma_status = 0;
  return p;
}

// number of VJP bands / checkpoint blocks of one sequence (host and device)
__host__ __device__ inline int64_t vjp_bands(int64_t len) {
  return len >= 2 ? (len - 1 + kVjpBand - 1) / kVjpBand : 0;
}
// checkpoint blocks before band w inside one (sequence, head)
__host__ __device__ inline int64_t vjp_ck_before(int64_t len, int64_t w) {
  const int64_t per = (len - 1) / kVjpRows + 1;
  return w * per - (kVjpBand / kVjpRows) * (w * (w - 1) / 2);
}
__host__ __device__ inline int64_t vjp_ck_count(int64_t len) {
  return len >= 2 ? vjp_ck_before(len, vjp_bands(len)) : 0;
}

void launch_build_plan(const Plan& plan, cudaStream_t stream);

// --------------------------------------------------------------- device utils
__device__ __forceinline__ float load_as_float(const void* p, int64_t idx, int dtype) {
  if (dtype == ROSA_B200_F32) return static_cast<const float*>(p)[idx];
  if (dtype == ROSA_B200_F16) return __half2float(static_cast<const __half*>(p)[idx]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

// Sequence containing `token`: returns its ordinal, or -1 when the plan is invalid or the
// token lies outside every sequence.  Dense plans divide; packed plans bisect cu_seqlens.
__device__ __forceinline__ int find_segment(const Plan& plan, int64_t token, int* start,
                                            int* len) {
  if (plan.status[0] != 0) return -1;
  int s;
  if (plan.cu_seqlens == nullptr) {
    s = (int)(token / plan.uniform_len);
  } else {
    int lo = 0, hi = plan.S;  // largest s with seg_start[s] <= token and non-empty
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (plan.seg_start[mid] <= token) lo = mid; else hi = mid;
    }
    s = lo;
  }
  *start = plan.seg_start[s];
  *len = plan.seg_len[s];
  if (token < *start || token >= (int64_t)*start + *len) return -1;
  return s;
}

// Work item -> (sequence, item index inside the sequence); false when the slot is unused.
__device__ __forceinline__ bool find_item(const Plan& plan, int slot, int* seq, int* local) {
  const int total = plan.item_prefix[plan.S];
  if (slot >= total) return false;
  int lo = 0, hi = plan.S;  // largest s with item_prefix[s] <= slot
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (plan.item_prefix[mid] <= slot) lo = mid; else hi = mid;
  }
  // skip sequences without items that share the same prefix value
  while (lo + 1 < plan.S && plan.item_prefix[lo + 1] <= slot) ++lo;
  *seq = lo;
  *local = slot - plan.item_prefix[lo];
  return true;
}

// Dropout counter hash of the operator (reference rosa_soft/soft_reference.py:383-447,
// rosa_soft/csrc/cuda/rosa_soft_kernels.cu:549-586).  One round is
//   s ^= s >> 16;  s *= 0x7FEB352D;  s ^= s >> 15;  s *= 0x846CA68B;  s ^= s >> 16
// and the chain is route -> query position -> head -> batch -> seed low -> seed high, each
// link xor-ing its salted word into the state before the next round.
//
// fold16(x) = x ^ (x >> 16) is linear over xor and its own inverse, so the fold that closes one
// round, the xor of the next word w and the fold that opens the next round collapse into a
// single xor: fold16(fold16(s) ^ w) = s ^ fold16(w).  The kernels therefore carry the state
// *open* (before the closing fold), pre-fold the words once, and run only the middle of each
// round (two multiplies, one shift, two xors) per causal pair.  The first round depends on the
// route only and is hashed once per key column (dropout_route_open).  The keep test
// `float(st >> 8) * 2^-24 >= p` is evaluated exactly on integers: the 24-bit value and the
// power-of-two scaling are exact in float32, so it equals `(st >> 8) >= ceil(p * 2^24)`, i.e.
// `st >= ceil(p * 2^24) << 8` (the threshold is below 2^24 for every float32 p < 1).
constexpr uint32_t kQuerySalt = 0xB5297A4Du;

__device__ __forceinline__ uint32_t fold16(uint32_t s) { return s ^ (s >> 16); }

__device__ __forceinline__ uint32_t round_core(uint32_t s) {
  s *= 0x7FEB352Du;
  s ^= s >> 15;
  s *= 0x846CA68Bu;
  return s;
}

struct DropoutKey {
  uint32_t head_word;   // fold16(head ^ salt)
  uint32_t batch_word;  // fold16(batch ^ salt)
  uint32_t seed_lo_word;
  uint32_t seed_hi_word;
  uint32_t threshold;   // ceil(float32(p) * 2^24) << 8
};

// Open state of the route round (its closing fold is absorbed by the query round).
__device__ __forceinline__ uint32_t dropout_route_open(uint32_t route) {
  return round_core(fold16(route ^ 0x68E31DA4u));
}

// Pre-folded query word.  For a query position i0 + r with i0 a multiple of 2^k and r < 2^k
// <= 2^16 it equals dropout_query_word(i0) ^ r.
__device__ __forceinline__ uint32_t dropout_query_word(uint32_t query) {
  return fold16(query ^ kQuerySalt);
}

__device__ __forceinline__ bool dropout_keep_open(const DropoutKey& k, uint32_t route_open,
                                                  uint32_t query_word) {
  uint32_t st = round_core(route_open ^ query_word);
  st = round_core(st ^ k.head_word);
  st = round_core(st ^ k.batch_word);
  st = round_core(st ^ k.seed_lo_word);
  st = round_core(st ^ k.seed_hi_word);
  return fold16(st) >= k.threshold;
}

__device__ __forceinline__ bool dropout_keep(const DropoutKey& k, uint32_t route, uint32_t query) {
  return dropout_keep_open(k, dropout_route_open(route), dropout_query_word(query));
}

__device__ __forceinline__ DropoutKey make_dropout_key(uint32_t head, uint32_t batch,
                                                       const int64_t* seed_ptr, float p) {
  DropoutKey k;
  const uint64_t seed = seed_ptr ? (uint64_t)(*seed_ptr) : 0ull;
  k.head_word = fold16(head ^ 0x63D83595u);
  k.batch_word = fold16(batch ^ 0xA511E9B3u);
  k.seed_lo_word = fold16((uint32_t)(seed & 0xFFFFFFFFull));
  k.seed_hi_word = fold16((uint32_t)(seed >> 32) ^ 0x9E3779B9u);
  k.threshold = (uint32_t)ceil((double)p * 16777216.0) << 8;
  return k;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// -------------------------------------------------------------- error plumbing
void set_error(const char* fmt, ...);

// ------------------------------------------------------------------- profiling
// Optional per-kernel CUDA-event timing (off by default, see rosa_b200_profile_enable):
// a scope records an event pair on the launching stream around one kernel launch.
struct ProfileScope {
  ProfileScope(const char* name, cudaStream_t stream);
  ~ProfileScope();
  int slot_;
  cudaStream_t stream_;
};

#define ROSA_REQUIRE(cond, ...)   \
  do {                            \
    if (!(cond)) {                \
      rosa::set_error(__VA_ARGS__); \
      return 1;                   \
    }                             \
  } while (0)

#define ROSA_CUDA_OK(expr)                                                        \
  do {                                                                            \
    cudaError_t err__ = (expr);                                                   \
    if (err__ != cudaSuccess) {                                                   \
      rosa::set_error("%s failed: %s", #expr, cudaGetErrorString(err__));         \
      return 2;                                                                   \
    }                                                                             \
  } while (0)

// ------------------------------------------------------- kernel entry points
struct FwdArgs {
  Plan plan;
  const void* q;
  const void* k;
  const void* v;
  int dtype;
  int64_t N;
  int H, D, Hv, Dv;
  int W;
  void* out;
  int8_t* out_i8;      // when set, the routed signs are written as -1 / 0 / +1 bytes instead
  int32_t* packed_q;   // head-major symbols (operator output)
  int32_t* packed_k;
  int32_t* route_token;           // optional
  unsigned long long* best;       // [N*H] (match length << 32 | local route)
  int64_t sym_seq_stride, sym_head_stride;  // packed symbol addressing
  // Per-symbol occurrence bitmaps of the key symbols, [H][2^D][mask_words] over the packed
  // token axis (bit g of row (h, s) set iff key symbol of token g, head h is s); null selects
  // the run-length matcher.
  uint32_t* match_masks;
  int64_t mask_words;
  // Bitmaps over symbols hashed to 8 bits, [H][256][mask_words]: prefilter of the matcher for
  // wide symbols (batched inference); null when not provided.
  uint32_t* hash_masks;
};

int launch_pack_symbols(const void* q, const void* k, int dtype, int64_t N, int H, int D,
                        int dense, int64_t uniform_len, int32_t* packed_q, int32_t* packed_k,
                        cudaStream_t stream);
int launch_hard_match(const FwdArgs& a, int items_upper, cudaStream_t stream);
int launch_gather_output(const FwdArgs& a, cudaStream_t stream);
int launch_route_inspect(const unsigned long long* best, int64_t count, int32_t* route,
                         int32_t* length, cudaStream_t stream);
int launch_inference_finish(const Plan& plan, const unsigned long long* best, const float* payload,
                            int64_t N, int H, int Hp, int Dp, float* out, int64_t* matched_end,
                            cudaStream_t stream);
int launch_transpose_symbols(const uint32_t* q, const uint32_t* k, int64_t N, int H, int32_t* qt,
                             int32_t* kt, cudaStream_t stream);

// One chunked update of the streaming runtime (stream_runtime.cu).
struct StreamArgs {
  const uint8_t* query;        // [chunk_tokens, H] packed symbols of the chunk
  const uint8_t* key;          // [chunk_tokens, H]
  const uint8_t* payload;      // [chunk_tokens, Hp]
  const int32_t* offsets;      // [slots + 1] chunk offsets per slot
  int64_t chunk_tokens;
  int slots, H, Hp, qk_bits, qk_mask, payload_mask, W;
  uint32_t* key_masks;         // [slots, H, 2^qk_bits, capacity / 32] occurrence bitmaps
  uint8_t* query_history;      // [slots, H, capacity]
  uint8_t* payload_history;    // [slots, Hp, capacity]
  int32_t* lengths;            // [slots] tokens held per slot, advanced by the call
  int64_t capacity;
  int64_t max_length_after;    // upper bound of lengths[s] + chunk length over the slots
  uint8_t* output;             // [chunk_tokens, H]
  int64_t* matched_end;        // [chunk_tokens, H]
  unsigned long long* best;    // [chunk_tokens, H] scratch
  int32_t* status;             // 4 words
};
int launch_stream_update(const StreamArgs& a, cudaStream_t stream);

struct VjpArgs {
  Plan plan;
  const void* q;
  const void* k;
  const void* v;
  const void* go;
  int dtype;
  int64_t N;
  int H, D, Hv, Dv;
  int W;
  int group;                       // H / Hv
  int bands_per_item;              // bands a CTA walks one after another
  const int32_t* qsym;
  const int32_t* ksym;
  int64_t sym_seq_stride, sym_head_stride;
  uint32_t* vbits;                 // [Hv][N][vwords] sign bits of the value rows
  int vwords;
  const int64_t* seed;
  float scale, dropout_p, inv_keep, mismatch_scale;
  int mask;
  int force_cuda_core_contraction;  // debugging aid: contract on CUDA cores even when tcgen05 applies
  uint32_t batch_offset, head_offset;
  // scratch
  int2* ckpt;                      // (S bits, window mismatch sum) per (block, diagonal)
  uint32_t* keepbits;              // dropout keep ballots: [ckpt block][row][warp]
  float4* stat_part;               // (max, sum, weighted sum) per (item, row)
  float4* rowstat;                 // [H][N] (max, 1/Z, E, log i)
  float* ring;                     // [items][W+1][band] (0 when the window never closes)
  int ring_slots;
  float* dq_part;                  // [item rows][D]
  float* dk_part;
  float* dv_part;                  // [item rows][Dv]
  float* dq;
  float* dk;
  float* dv;
};

int launch_pack_value_bits(const void* v, int dtype, int64_t N, int Hv, int Dv, uint32_t* vbits,
                           int vwords, cudaStream_t stream);
int launch_vjp_sweep1(const VjpArgs& a, int items_upper, cudaStream_t stream);
// register-tiled sweeps (vjp_tiled.cu): four diagonals per thread
bool vjp_tiled_applies(const VjpArgs& a);
int launch_vjp_sweep1_tiled(const VjpArgs& a, int items_upper, cudaStream_t stream);
int launch_vjp_sweep2_tiled(const VjpArgs& a, int items_upper, cudaStream_t stream);
int launch_vjp_rowstats(const VjpArgs& a, cudaStream_t stream);
int launch_vjp_sweep2(const VjpArgs& a, int items_upper, cudaStream_t stream);
int launch_vjp_finalize(const VjpArgs& a, cudaStream_t stream);

}  // namespace rosa
