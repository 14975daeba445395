// C ABI of librosa_soft_b200.so: argument checks, workspace carve-up and kernel
// sequencing.  No allocation, no synchronisation (except rosa_b200_read_status).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <limits>

#include "common.cuh"

namespace rosa {
const char* get_error();
int static_scratch_for_current_device(void** out);
void profile_enable(bool on);
int profile_collect(const char** names, float* total_ms, int* launches, int capacity);
}

using namespace rosa;

namespace {

// Target size of the VJP partial buffers (per-item partial gradient rows + window ring): items
// grow (more bands per CTA) until they fit.  ROSA_B200_PARTIAL_BUDGET_MB overrides it for
// experiments; the sizing function and the call read the same value.
size_t partial_budget_bytes() {
  static const size_t bytes = [] {
    const char* v = std::getenv("ROSA_B200_PARTIAL_BUDGET_MB");
    const long mb = v != nullptr ? std::atol(v) : 0;
    return mb > 0 ? (size_t)mb << 20 : (size_t)6 << 30;
  }();
  return bytes;
}

struct FwdLayout {
  PlanLayout plan;
  size_t best_off, qt_off, kt_off, masks_off;
  int64_t mask_words;
  size_t bytes;
};

constexpr int kMaskSymbolBits = 8;   // widest symbol served by the bit-parallel matcher

int64_t fwd_items_upper(int64_t N, int64_t S, int64_t uniform_len, bool dense) {
  if (dense) return S * (uniform_len >= 2 ? (uniform_len - 1 + kFwdBand - 1) / kFwdBand : 0);
  return N / kFwdBand + S;
}

FwdLayout fwd_layout(int64_t N, int H, int64_t S, bool transposed_symbols) {
  FwdLayout l;
  l.plan = plan_layout(0, S);
  size_t off = l.plan.bytes;
  l.best_off = off;
  off = align_up(off + (size_t)N * H * sizeof(unsigned long long));
  l.qt_off = l.kt_off = 0;
  if (transposed_symbols) {
    l.qt_off = off;
    off = align_up(off + (size_t)N * H * sizeof(int32_t));
    l.kt_off = off;
    off = align_up(off + (size_t)N * H * sizeof(int32_t));
    // bitmaps over the symbols hashed to 8 bits (prefilter of the wide-symbol matcher)
    l.mask_words = (N + 31) / 32 + 1;
    l.masks_off = off;
    off = align_up(off + ((size_t)H << kMaskSymbolBits) * (size_t)l.mask_words * sizeof(uint32_t));
  } else {
    // occurrence bitmaps of the bit-parallel matcher, sized for the widest symbol it serves
    // (the sizing function does not know D): H * 2^8 rows of ceil(N / 32) + 1 words
    l.mask_words = (N + 31) / 32 + 1;
    l.masks_off = off;
    off = align_up(off + ((size_t)H << kMaskSymbolBits) * (size_t)l.mask_words * sizeof(uint32_t));
  }
  l.bytes = off;
  return l;
}

struct VjpLayout {
  PlanLayout plan;
  size_t vbits_off, ckpt_off, keep_off, stat_off, rowstat_off, ring_off, dq_off, dk_off, dv_off;
  size_t ring_bytes;
  size_t bytes;
  int bands_per_item;
  int vwords;
  int ring_slots;
  int64_t items_upper;  // per head
};

// Upper bounds that depend on shapes only (the packed path never reads cu_seqlens on
// the host): items, partial-row slots and checkpoint blocks per head.
void vjp_bounds(int64_t N, int64_t S, int64_t uniform_len, bool dense, int64_t item_diag,
                int64_t* items, int64_t* rows, int64_t* cks) {
  if (dense) {
    const int64_t per = uniform_len >= 2 ? (uniform_len - 1 + item_diag - 1) / item_diag : 0;
    *items = S * per;
    *rows = S * per * uniform_len;
    *cks = S * vjp_ck_count(uniform_len);
  } else {
    // sum_s ceil((L_s-1)/id) <= N/id + S ; sum_s items_s L_s <= N^2/id + N
    *items = N / item_diag + S;
    *rows = (N / item_diag + 1) * N;
    // the per-sequence count is super-additive up to rounding: sum_s ck(L_s) <= ck(N) + slack
    *cks = vjp_ck_count(N) + 2 * (N / kVjpRows) + 4 * S + 8;
  }
}

VjpLayout vjp_layout(int64_t N, int H, int D, int Hv, int Dv, int64_t S, int64_t uniform_len,
                     bool dense, int64_t W, int mask) {
  VjpLayout l;
  l.plan = plan_layout(0, S);
  l.vwords = (Dv + 31) / 32;
  const int64_t max_len = dense ? uniform_len : N;
  l.ring_slots = (W <= max_len - 2) ? (int)(W + 1) : 0;
  const size_t per_row = sizeof(float4) + sizeof(float) * ((mask & 1 ? D : 0) + (mask & 2 ? D : 0) +
                                                            (mask & 4 ? Dv : 0));
  int g = 1;
  int64_t items = 0, rows = 0, cks = 0;
  for (;; g *= 2) {
    vjp_bounds(N, S, uniform_len, dense, (int64_t)g * kVjpBand, &items, &rows, &cks);
    // the window ring (one line of kVjpBand floats per horizon step and item) counts against
    // the same budget: fewer, longer items shrink it together with the partial rows
    const size_t ring = (size_t)items * H * l.ring_slots * kVjpBand * sizeof(float);
    if ((size_t)rows * H * per_row + ring <= partial_budget_bytes() ||
        (int64_t)g * kVjpBand >= max_len)
      break;
  }
  l.bands_per_item = g;
  l.items_upper = items;
  size_t off = l.plan.bytes;
  l.vbits_off = off;
  off = align_up(off + (size_t)N * Hv * l.vwords * sizeof(uint32_t));
  l.ckpt_off = off;
  off = align_up(off + (size_t)cks * H * kVjpBand * sizeof(int2));
  l.keep_off = off;
  off = align_up(off + (size_t)cks * H * kVjpRows * kVjpWarps * sizeof(uint32_t));
  l.stat_off = off;
  off = align_up(off + (size_t)rows * H * sizeof(float4));
  l.rowstat_off = off;
  off = align_up(off + (size_t)N * H * sizeof(float4));
  l.ring_off = off;
  l.ring_bytes = (size_t)items * H * l.ring_slots * kVjpBand * sizeof(float);
  off = align_up(off + l.ring_bytes);
  l.dq_off = off;
  if (mask & 1) off = align_up(off + (size_t)rows * H * D * sizeof(float));
  l.dk_off = off;
  if (mask & 2) off = align_up(off + (size_t)rows * H * D * sizeof(float));
  l.dv_off = off;
  if (mask & 4) off = align_up(off + (size_t)rows * H * Dv * sizeof(float));
  l.bytes = off;
  return l;
}

// A dense batch whose partial rows would not fit the budget at one band per work item is run in
// slices of whole sequences, one after the other on the caller's stream, each slice with the
// finest work items and all of them in the same workspace: sequences never interact, so the
// results are those of one call, the workspace stops growing with the batch, and the finer items
// balance better than longer items over the whole batch would.  Returns the number of slices;
// slice i holds S / n + (i < S % n) sequences.
int64_t vjp_dense_slices(int H, int D, int Dv, int64_t S, int64_t uniform_len, int64_t W, int mask) {
  if (uniform_len < 2 || S <= 1) return 1;
  const size_t per_row = sizeof(float4) + sizeof(float) * ((mask & 1 ? D : 0) + (mask & 2 ? D : 0) +
                                                            (mask & 4 ? Dv : 0));
  const int64_t items = (uniform_len - 1 + kVjpBand - 1) / kVjpBand;      // per sequence, g = 1
  const int ring_slots = (W <= uniform_len - 2) ? (int)(W + 1) : 0;
  const size_t one = (size_t)items * uniform_len * H * per_row +
                     (size_t)items * H * ring_slots * kVjpBand * sizeof(float);
  const int64_t fit = std::max<int64_t>(1, (int64_t)(partial_budget_bytes() / one));
  return fit >= S ? 1 : (S + fit - 1) / fit;
}
inline int64_t slice_sequences(int64_t S, int64_t n, int64_t i) { return S / n + (i < S % n ? 1 : 0); }

int check_problem(int64_t N, int H, int D, int Hv, int Dv, const int32_t* cu, int64_t S,
                  int64_t uniform_len, int64_t W, int dtype) {
  ROSA_REQUIRE(dtype >= ROSA_B200_F32 && dtype <= ROSA_B200_BF16,
               "dtype must be float32, float16 or bfloat16");
  ROSA_REQUIRE(N > 0 && H > 0 && Hv > 0 && Dv > 0, "N, H, Hv and Dv must be positive");
  ROSA_REQUIRE(D >= 1 && D <= 32, "query/key bit dimension must be in [1, 32]");
  ROSA_REQUIRE(H % Hv == 0, "query heads must be divisible by value heads");
  ROSA_REQUIRE(H <= 65535, "head count exceeds the CUDA grid limit");
  ROSA_REQUIRE(S >= 1, "at least one sequence is required");
  ROSA_REQUIRE(N * H <= std::numeric_limits<int32_t>::max(), "N * H must fit in int32");
  ROSA_REQUIRE(W >= 1, "max_suffix_length must be >= 1");
  if (cu == nullptr)
    ROSA_REQUIRE(uniform_len >= 1 && S * uniform_len == N,
                 "dense description needs num_seq * uniform_len == N");
  return 0;
}

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// The plan's problem (bad offsets, capacity) comes first: it explains everything after it.
inline int decode_status_words(int plan_word, int mma_word) {
  if (plan_word != ROSA_B200_STATUS_OK) return plan_word;
  return mma_word != 0 ? ROSA_B200_STATUS_MMA_TIMEOUT : ROSA_B200_STATUS_OK;
}

}  // namespace

extern "C" {

ROSA_B200_API int rosa_b200_abi_version(void) { return ROSA_B200_ABI_VERSION; }

ROSA_B200_API const char* rosa_b200_last_error(void) { return rosa::get_error(); }

ROSA_B200_API size_t rosa_b200_hard_forward_workspace_bytes(int64_t N, int H, int64_t num_seq) {
  return fwd_layout(N, H, num_seq, false).bytes;
}

namespace {
// Shared driver of the two forward entry points.  `query` / `key` null: the packed symbols are
// inputs (already produced by the caller, e.g. by the epilogue of its projection GEMM) and the
// packing kernel is skipped.  `output_i8` non-null: the routed signs go out as int8.
int run_hard_forward(const void* query, const void* key, const void* value, int dtype, int64_t N,
                     int H, int D, int Hv, int Dv, const int32_t* cu_seqlens, int64_t num_seq,
                     int64_t uniform_len, int64_t max_suffix_length, void* output,
                     int8_t* output_i8, int32_t* packed_query, int32_t* packed_key,
                     int32_t* route_token, void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_problem(N, H, D, Hv, Dv, cu_seqlens, num_seq, uniform_len, max_suffix_length,
                             dtype))
    return rc;
  ROSA_REQUIRE(value && (output || output_i8) && packed_query && packed_key && workspace,
               "null pointer argument");
  ROSA_REQUIRE((query == nullptr) == (key == nullptr), "query and key go together");
  const bool dense = cu_seqlens == nullptr;
  const FwdLayout l = fwd_layout(N, H, num_seq, false);
  ROSA_REQUIRE(workspace_bytes >= l.bytes, "workspace too small: need %zu bytes, got %zu", l.bytes,
               workspace_bytes);
  const int64_t items = fwd_items_upper(N, num_seq, uniform_len, dense);
  ROSA_REQUIRE(items * (int64_t)H <= std::numeric_limits<int32_t>::max(),
               "too many work items: items * heads exceeds the CUDA grid limit");
  cudaStream_t st = as_stream(stream);
  char* ws = static_cast<char*>(workspace);

  FwdArgs a{};
  a.plan = make_plan(workspace, l.plan, cu_seqlens, N, num_seq, uniform_len, kFwdBand);
  a.q = query; a.k = key; a.v = value; a.dtype = dtype;
  a.N = N; a.H = H; a.D = D; a.Hv = Hv; a.Dv = Dv;
  a.W = (int)std::min<int64_t>(max_suffix_length, dense ? uniform_len : N);
  a.out = output; a.out_i8 = output_i8;
  a.packed_q = packed_query; a.packed_k = packed_key;
  a.route_token = route_token;
  a.best = reinterpret_cast<unsigned long long*>(ws + l.best_off);
  a.sym_seq_stride = dense ? (int64_t)H * uniform_len : 0;
  a.sym_head_stride = dense ? uniform_len : N;
  // symbols of up to 8 bits index the bitmaps directly; wider ones go through the hashed
  // prefilter (same 2^8 rows per head)
  if (D <= kMaskSymbolBits)
    a.match_masks = reinterpret_cast<uint32_t*>(ws + l.masks_off);
  else
    a.hash_masks = reinterpret_cast<uint32_t*>(ws + l.masks_off);
  a.mask_words = l.mask_words;

  launch_build_plan(a.plan, st);
  ROSA_CUDA_OK(cudaGetLastError());
  ROSA_CUDA_OK(cudaMemsetAsync(a.best, 0, (size_t)N * H * sizeof(unsigned long long), st));
  if (query != nullptr)
    if (int rc = launch_pack_symbols(query, key, dtype, N, H, D, dense, uniform_len, packed_query,
                                     packed_key, st))
      return rc;
  if (int rc = launch_hard_match(a, (int)items, st)) return rc;
  return launch_gather_output(a, st);
}
}  // namespace

ROSA_B200_API int rosa_b200_hard_forward(const void* query, const void* key, const void* value, int dtype,
                           int64_t N, int H, int D, int Hv, int Dv, const int32_t* cu_seqlens,
                           int64_t num_seq, int64_t uniform_len, int64_t max_suffix_length,
                           void* output, int32_t* packed_query, int32_t* packed_key,
                           int32_t* route_token, void* workspace, size_t workspace_bytes,
                           void* stream) {
  if (int rc = check_problem(N, H, D, Hv, Dv, cu_seqlens, num_seq, uniform_len, max_suffix_length,
                             dtype))
    return rc;
  ROSA_REQUIRE(query && key && output, "null pointer argument");
  return run_hard_forward(query, key, value, dtype, N, H, D, Hv, Dv, cu_seqlens, num_seq,
                          uniform_len, max_suffix_length, output, nullptr, packed_query, packed_key,
                          route_token, workspace, workspace_bytes, stream);
}

ROSA_B200_API int rosa_b200_pack_symbols(const void* logits, int dtype, int64_t N, int H, int D,
                                         int64_t num_seq, int64_t uniform_len, int32_t* packed,
                                         void* stream) {
  ROSA_REQUIRE(dtype >= ROSA_B200_F32 && dtype <= ROSA_B200_BF16,
               "dtype must be float32, float16 or bfloat16");
  ROSA_REQUIRE(logits && packed, "null pointer argument");
  ROSA_REQUIRE(N > 0 && H > 0 && D >= 1 && D <= 32, "invalid problem size");
  const bool dense = uniform_len > 0;
  if (dense)
    ROSA_REQUIRE(num_seq * uniform_len == N, "dense description needs num_seq * uniform_len == N");
  return launch_pack_symbols(logits, nullptr, dtype, N, H, D, dense, uniform_len, packed, nullptr,
                             as_stream(stream));
}

ROSA_B200_API int rosa_b200_hard_forward_packed(
    const int32_t* packed_query, const int32_t* packed_key, const void* value, int dtype, int64_t N,
    int H, int D, int Hv, int Dv, const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
    int64_t max_suffix_length, int8_t* output, int32_t* route_token, void* workspace,
    size_t workspace_bytes, void* stream) {
  ROSA_REQUIRE(packed_query && packed_key && output, "null pointer argument");
  return run_hard_forward(nullptr, nullptr, value, dtype, N, H, D, Hv, Dv, cu_seqlens, num_seq,
                          uniform_len, max_suffix_length, nullptr, output,
                          const_cast<int32_t*>(packed_query), const_cast<int32_t*>(packed_key),
                          route_token, workspace, workspace_bytes, stream);
}

ROSA_B200_API int rosa_b200_hard_forward_routes(const void* workspace, size_t workspace_bytes,
                                                int64_t N, int H, int64_t num_seq,
                                                int32_t* selected_route, int32_t* match_length,
                                                void* stream) {
  ROSA_REQUIRE(workspace != nullptr, "null pointer argument");
  ROSA_REQUIRE(N >= 0 && H >= 1 && num_seq >= 1, "invalid problem size");
  const FwdLayout l = fwd_layout(N, H, num_seq, false);
  ROSA_REQUIRE(workspace_bytes >= l.bytes, "workspace too small: need %zu bytes, got %zu", l.bytes,
               workspace_bytes);
  if (N == 0 || (selected_route == nullptr && match_length == nullptr)) return 0;
  const unsigned long long* best = reinterpret_cast<const unsigned long long*>(
      static_cast<const char*>(workspace) + l.best_off);
  return launch_route_inspect(best, N * (int64_t)H, selected_route, match_length, as_stream(stream));
}

ROSA_B200_API size_t rosa_b200_hard_inference_workspace_bytes(int64_t N, int H, int64_t num_seq) {
  return fwd_layout(N, H, num_seq, true).bytes;
}

ROSA_B200_API int rosa_b200_hard_inference(const uint32_t* query_symbols, const uint32_t* key_symbols,
                             const float* payload, int64_t N, int H, int Hp, int Dp,
                             const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
                             int64_t max_suffix_length, float* out, int64_t* matched_end,
                             void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_problem(N, H, 32, Hp, Dp, cu_seqlens, num_seq, uniform_len,
                             max_suffix_length, ROSA_B200_F32))
    return rc;
  ROSA_REQUIRE(query_symbols && key_symbols && matched_end && workspace, "null pointer argument");
  ROSA_REQUIRE(out == nullptr || payload != nullptr, "payload is required when out is given");
  const bool dense = cu_seqlens == nullptr;
  const FwdLayout l = fwd_layout(N, H, num_seq, true);
  ROSA_REQUIRE(workspace_bytes >= l.bytes, "workspace too small: need %zu bytes, got %zu", l.bytes,
               workspace_bytes);
  cudaStream_t st = as_stream(stream);
  char* ws = static_cast<char*>(workspace);

  FwdArgs a{};
  // symbols are transposed to [H, N] whatever the sequence description: the matcher
  // only needs a per-sequence base and a head stride
  a.plan = make_plan(workspace, l.plan, cu_seqlens, N, num_seq, uniform_len, kFwdBand);
  a.N = N; a.H = H; a.D = 32; a.Hv = Hp; a.Dv = Dp;
  a.W = (int)std::min<int64_t>(max_suffix_length, dense ? uniform_len : N);
  a.packed_q = reinterpret_cast<int32_t*>(ws + l.qt_off);
  a.packed_k = reinterpret_cast<int32_t*>(ws + l.kt_off);
  a.best = reinterpret_cast<unsigned long long*>(ws + l.best_off);
  a.sym_seq_stride = dense ? uniform_len : 0;  // [H, N] with sequence s starting at s * T
  a.sym_head_stride = N;
  a.hash_masks = reinterpret_cast<uint32_t*>(ws + l.masks_off);
  a.mask_words = l.mask_words;

  launch_build_plan(a.plan, st);
  ROSA_CUDA_OK(cudaGetLastError());
  ROSA_CUDA_OK(cudaMemsetAsync(a.best, 0, (size_t)N * H * sizeof(unsigned long long), st));
  if (int rc = launch_transpose_symbols(query_symbols, key_symbols, N, H, a.packed_q, a.packed_k,
                                        st))
    return rc;
  if (int rc = launch_hard_match(a, (int)fwd_items_upper(N, num_seq, uniform_len, dense), st))
    return rc;
  return launch_inference_finish(a.plan, a.best, payload, N, H, Hp, Dp, out, matched_end, st);
}

ROSA_B200_API size_t rosa_b200_stream_workspace_bytes(int64_t chunk_tokens, int num_heads) {
  if (chunk_tokens < 0 || num_heads < 1) return 0;
  return 256 + (size_t)chunk_tokens * (size_t)num_heads * sizeof(unsigned long long);
}

ROSA_B200_API int rosa_b200_stream_update(
    const uint8_t* query, const uint8_t* key, const uint8_t* payload,
    const int32_t* chunk_offsets, int64_t chunk_tokens, int slots, int num_heads,
    int num_payload_heads, int qk_bits, int payload_bits, int64_t max_suffix_length,
    uint32_t* key_masks, uint8_t* query_history, uint8_t* payload_history, int32_t* lengths,
    int64_t capacity, int64_t max_length_after, uint8_t* output, int64_t* matched_key_end,
    void* workspace, size_t workspace_bytes, void* stream) {
  ROSA_REQUIRE(slots >= 1, "slot count must be >= 1");
  ROSA_REQUIRE(num_heads >= 1 && num_payload_heads >= 1, "head counts must be >= 1");
  ROSA_REQUIRE(num_heads % num_payload_heads == 0,
               "num_heads must be divisible by num_payload_heads");
  ROSA_REQUIRE(qk_bits >= 1 && qk_bits <= 8, "qk_bits must be in [1, 8]");
  ROSA_REQUIRE(payload_bits >= 1 && payload_bits <= 8, "payload_bits must be in [1, 8]");
  ROSA_REQUIRE(max_suffix_length >= 1, "max_suffix_length must be >= 1");
  ROSA_REQUIRE(chunk_tokens >= 0, "chunk token count must be non-negative");
  ROSA_REQUIRE(capacity >= 32 && capacity % 32 == 0 &&
                   capacity <= std::numeric_limits<int32_t>::max() - 31,
               "history capacity must be a multiple of 32 in [32, 2^31)");
  ROSA_REQUIRE(max_length_after >= 0 && max_length_after <= capacity,
               "max_length_after exceeds the history capacity");
  ROSA_REQUIRE(chunk_tokens * (int64_t)num_heads <= std::numeric_limits<int32_t>::max(),
               "chunk_tokens * num_heads exceeds the int32 range");
  ROSA_REQUIRE(chunk_offsets && key_masks && query_history && payload_history && lengths && workspace,
               "null pointer argument");
  ROSA_REQUIRE(chunk_tokens == 0 || (query && key && payload && output && matched_key_end),
               "null pointer argument");
  const size_t need = rosa_b200_stream_workspace_bytes(chunk_tokens, num_heads);
  ROSA_REQUIRE(workspace_bytes >= need, "workspace too small: need %zu bytes, got %zu", need,
               workspace_bytes);
  StreamArgs a{};
  a.query = query; a.key = key; a.payload = payload;
  a.offsets = chunk_offsets;
  a.chunk_tokens = chunk_tokens;
  a.slots = slots; a.H = num_heads; a.Hp = num_payload_heads;
  a.qk_bits = qk_bits;
  a.qk_mask = (1 << qk_bits) - 1;
  a.payload_mask = (1 << payload_bits) - 1;
  a.W = (int)std::min<int64_t>(max_suffix_length, capacity);
  a.key_masks = key_masks; a.query_history = query_history; a.payload_history = payload_history;
  a.lengths = lengths;
  a.capacity = capacity;
  a.max_length_after = max_length_after;
  a.output = output; a.matched_end = matched_key_end;
  a.status = static_cast<int32_t*>(workspace);
  a.best = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + 256);
  return launch_stream_update(a, as_stream(stream));
}

namespace {
struct VjpCall {
  const void *query, *key, *value, *grad_output;
  int dtype, H, D, Hv, Dv;
  const int32_t* cu_seqlens;
  int64_t uniform_len, W;
  const int32_t *packed_query, *packed_key;
  const int64_t* dropout_seed;
  float scale, dropout_p, mismatch_scale;
  int gradient_mask;
  bool force_cuda_cores;
  int64_t batch_offset, head_offset;
  float *grad_query, *grad_key, *grad_value;
  void* workspace;
  size_t workspace_bytes;
  cudaStream_t stream;
};

// The backward of `S` whole sequences (`N` tokens) starting at sequence `first_seq` of the call
// (`first_seq` > 0 only for dense layouts, where it is also the token and dropout batch offset).
int run_vjp_slice(const VjpCall& c, int64_t first_seq, int64_t N, int64_t S, bool later_slice) {
  const bool dense = c.cu_seqlens == nullptr;
  const int H = c.H, D = c.D, Hv = c.Hv, Dv = c.Dv;
  const VjpLayout l = vjp_layout(N, H, D, Hv, Dv, S, c.uniform_len, dense, c.W, c.gradient_mask);
  ROSA_REQUIRE(c.workspace_bytes >= l.bytes, "workspace too small: need %zu bytes, got %zu",
               l.bytes, c.workspace_bytes);
  ROSA_REQUIRE(l.items_upper * (int64_t)H <= std::numeric_limits<int32_t>::max(),
               "too many work items: items * heads exceeds the CUDA grid limit");
  cudaStream_t st = c.stream;
  char* ws = static_cast<char*>(c.workspace);
  const size_t esz = c.dtype == ROSA_B200_F32 ? 4 : 2;
  const int64_t tok = first_seq * c.uniform_len;          // first token of the slice
  auto at = [](const void* p, size_t bytes) { return static_cast<const char*>(p) + bytes; };

  VjpArgs a{};
  a.plan = make_plan(c.workspace, l.plan, c.cu_seqlens, N, S, c.uniform_len,
                     l.bands_per_item * kVjpBand);
  a.plan.keep_mma_status = later_slice ? 1 : 0;
  a.q = at(c.query, (size_t)tok * H * D * esz);
  a.k = at(c.key, (size_t)tok * H * D * esz);
  a.v = at(c.value, (size_t)tok * Hv * Dv * esz);
  a.go = at(c.grad_output, (size_t)tok * H * Dv * esz);
  a.dtype = c.dtype;
  a.N = N; a.H = H; a.D = D; a.Hv = Hv; a.Dv = Dv;
  a.W = (int)c.W;
  a.group = H / Hv;
  a.bands_per_item = l.bands_per_item;
  a.qsym = c.packed_query + tok * H;                      // dense symbols: [sequence][head][token]
  a.ksym = c.packed_key + tok * H;
  a.sym_seq_stride = dense ? (int64_t)H * c.uniform_len : 0;
  a.sym_head_stride = dense ? c.uniform_len : N;
  a.vbits = reinterpret_cast<uint32_t*>(ws + l.vbits_off);
  a.vwords = l.vwords;
  a.seed = c.dropout_seed;
  a.scale = c.scale;
  a.dropout_p = c.dropout_p;
  a.inv_keep = 1.0f / (1.0f - c.dropout_p);
  a.mismatch_scale = c.mismatch_scale;
  a.mask = c.gradient_mask;
  a.force_cuda_core_contraction = c.force_cuda_cores;
  a.batch_offset = (uint32_t)(c.batch_offset + first_seq);
  a.head_offset = (uint32_t)c.head_offset;
  a.ckpt = reinterpret_cast<int2*>(ws + l.ckpt_off);
  a.keepbits = reinterpret_cast<uint32_t*>(ws + l.keep_off);
  a.stat_part = reinterpret_cast<float4*>(ws + l.stat_off);
  a.rowstat = reinterpret_cast<float4*>(ws + l.rowstat_off);
  a.ring = reinterpret_cast<float*>(ws + l.ring_off);
  a.ring_slots = l.ring_slots;
  a.dq_part = reinterpret_cast<float*>(ws + l.dq_off);
  a.dk_part = reinterpret_cast<float*>(ws + l.dk_off);
  a.dv_part = reinterpret_cast<float*>(ws + l.dv_off);
  a.dq = c.grad_query ? c.grad_query + tok * H * D : nullptr;
  a.dk = c.grad_key ? c.grad_key + tok * H * D : nullptr;
  a.dv = c.grad_value ? c.grad_value + tok * Hv * Dv : nullptr;

  launch_build_plan(a.plan, st);
  ROSA_CUDA_OK(cudaGetLastError());
  if (l.ring_bytes) ROSA_CUDA_OK(cudaMemsetAsync(a.ring, 0, l.ring_bytes, st));
  if (int rc = launch_pack_value_bits(a.v, c.dtype, N, Hv, Dv, a.vbits, a.vwords, st)) return rc;
  if (int rc = launch_vjp_sweep1(a, (int)l.items_upper, st)) return rc;
  if (int rc = launch_vjp_rowstats(a, st)) return rc;
  if (int rc = launch_vjp_sweep2(a, (int)l.items_upper, st)) return rc;
  return launch_vjp_finalize(a, st);
}
}  // namespace

ROSA_B200_API size_t rosa_b200_surrogate_vjp_workspace_bytes(int64_t N, int H, int D, int Hv, int Dv,
                                               int64_t num_seq, int64_t uniform_len,
                                               int64_t max_suffix_length, int gradient_mask) {
  const bool dense = uniform_len > 0;
  const int64_t W = std::min<int64_t>(max_suffix_length, dense ? uniform_len : N);
  gradient_mask &= ~ROSA_B200_MASK_CUDA_CORE_CONTRACTION;
  if (dense) {
    // the largest slice (slice 0) sizes the workspace that all slices share
    const int64_t n = vjp_dense_slices(H, D, Dv, num_seq, uniform_len, W, gradient_mask);
    const int64_t s0 = slice_sequences(num_seq, n, 0);
    return vjp_layout(s0 * uniform_len, H, D, Hv, Dv, s0, uniform_len, true, W, gradient_mask).bytes;
  }
  return vjp_layout(N, H, D, Hv, Dv, num_seq, uniform_len, dense, W, gradient_mask).bytes;
}

ROSA_B200_API int rosa_b200_surrogate_vjp(const void* query, const void* key, const void* value,
                            const void* grad_output, int dtype, int64_t N, int H, int D, int Hv,
                            int Dv, const int32_t* cu_seqlens, int64_t num_seq,
                            int64_t uniform_len, int64_t max_suffix_length,
                            const int32_t* packed_query, const int32_t* packed_key,
                            const int64_t* dropout_seed, float scale, float dropout_p,
                            float mismatch_scale, int gradient_mask,
                            int64_t dropout_batch_offset, int64_t dropout_head_offset,
                            float* grad_query, float* grad_key, float* grad_value, void* workspace,
                            size_t workspace_bytes, void* stream) {
  if (int rc = check_problem(N, H, D, Hv, Dv, cu_seqlens, num_seq, uniform_len, max_suffix_length,
                             dtype))
    return rc;
  const int force_cuda_cores = gradient_mask & ROSA_B200_MASK_CUDA_CORE_CONTRACTION;
  gradient_mask &= ~ROSA_B200_MASK_CUDA_CORE_CONTRACTION;
  ROSA_REQUIRE(gradient_mask >= 1 && gradient_mask <= 7,
               "gradient_mask must be an integer bit mask in [1, 7]");
  ROSA_REQUIRE(query && key && value && grad_output && packed_query && packed_key && workspace,
               "null pointer argument");
  ROSA_REQUIRE(!(gradient_mask & 1) || grad_query, "grad_query is required by gradient_mask");
  ROSA_REQUIRE(!(gradient_mask & 2) || grad_key, "grad_key is required by gradient_mask");
  ROSA_REQUIRE(!(gradient_mask & 4) || grad_value, "grad_value is required by gradient_mask");
  ROSA_REQUIRE(scale > 0.0f && std::isfinite(scale), "scale must be finite and > 0");
  ROSA_REQUIRE(mismatch_scale > 0.0f && std::isfinite(mismatch_scale),
               "mismatch_scale must be finite and > 0");
  ROSA_REQUIRE(dropout_p >= 0.0f && dropout_p < 1.0f, "dropout_p must be in [0, 1)");
  ROSA_REQUIRE((dropout_p > 0.0f) == (dropout_seed != nullptr),
               "dropout_seed must be given exactly when dropout_p > 0");
  const bool dense = cu_seqlens == nullptr;
  if (!dense) uniform_len = 0;
  const int64_t W = std::min<int64_t>(max_suffix_length, dense ? uniform_len : N);
  VjpCall c{query, key, value, grad_output, dtype, H, D, Hv, Dv, cu_seqlens, uniform_len, W,
            packed_query, packed_key, dropout_seed, scale, dropout_p, mismatch_scale,
            gradient_mask, force_cuda_cores != 0, dropout_batch_offset, dropout_head_offset,
            grad_query, grad_key, grad_value, workspace, workspace_bytes, as_stream(stream)};
  if (!dense) return run_vjp_slice(c, 0, N, num_seq, false);
  // dense: slices of whole sequences (one slice unless the partial rows exceed their budget)
  const int64_t n = vjp_dense_slices(H, D, Dv, num_seq, uniform_len, W, gradient_mask);
  int64_t first = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t count = slice_sequences(num_seq, n, i);
    if (int rc = run_vjp_slice(c, first, count * uniform_len, count, i > 0)) return rc;
    first += count;
  }
  return 0;
}

ROSA_B200_API void rosa_b200_profile_enable(int on) { rosa::profile_enable(on != 0); }

ROSA_B200_API int rosa_b200_profile_collect(const char** names, float* total_ms, int* launches,
                                            int capacity) {
  return rosa::profile_collect(names, total_ms, launches, capacity);
}

ROSA_B200_API int rosa_b200_read_status(const void* workspace, void* stream, int* status) {
  ROSA_REQUIRE(status != nullptr, "null pointer argument");
  if (workspace == nullptr) {
    // the scratch of the workspace-free forward: its plan (status words first) opens the array
    void* scratch = nullptr;
    if (int rc = rosa::static_scratch_for_current_device(&scratch)) return rc;
    workspace = scratch;
  }
  // word 0: offsets / capacity check of the plan; word 1: a tensor-core wait gave up
  int32_t host[2] = {0, 0};
  ROSA_CUDA_OK(cudaMemcpyAsync(host, workspace, sizeof(host), cudaMemcpyDeviceToHost,
                               as_stream(stream)));
  ROSA_CUDA_OK(cudaStreamSynchronize(as_stream(stream)));
  *status = decode_status_words(host[0], host[1]);
  return 0;
}

// Host-side decoding of the two status words, exported for tests of the decoding itself.
ROSA_B200_API int rosa_b200_decode_status(int plan_word, int mma_word) {
  return decode_status_words(plan_word, mma_word);
}

}  // extern "C"
