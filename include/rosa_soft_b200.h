/*
 * rosa_soft_b200 -- C ABI of the sm_100a implementation of the rosa_soft operator
 * family (hard ROSA suffix routing forward, dense surrogate VJP backward, the packed
 * variable-length variant and batched hard inference).
 *
 * Conventions
 *   - All data pointers are DEVICE pointers on the current CUDA device unless a
 *     parameter says otherwise.  `stream` is a cudaStream_t passed as void*.
 *   - The library allocates nothing: every entry point that needs scratch takes a
 *     caller-owned `workspace` of at least `*_workspace_bytes(...)` bytes
 *     (256-byte aligned).  Workspace contents are undefined between calls.
 *   - Every entry point only enqueues work on `stream`; none synchronises.
 *   - Return value 0 = success; non-zero = argument error, nothing was enqueued and
 *     rosa_b200_last_error() describes the problem (thread-local string).
 *   - Sequences: either `cu_seqlens == NULL` (dense: `num_seq` sequences of
 *     `uniform_len` tokens, N = num_seq * uniform_len, packed symbols laid out
 *     [num_seq, H, uniform_len]) or a device int32 array of num_seq + 1 offsets
 *     (packed: symbols laid out [H, N]).  Offsets are validated on the device; an
 *     inconsistent array makes every kernel a no-op for the call (outputs zero) and
 *     sets the status word that rosa_b200_read_status() returns.  Nothing traps.
 *   - Layouts: query/key [N, H, D], value [N, Hv, Dv], output / grad_output
 *     [N, H, Dv], all contiguous, element type given by `dtype`.
 */
#ifndef ROSA_SOFT_B200_H_
#define ROSA_SOFT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ROSA_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define ROSA_B200_API __attribute__((visibility("default")))
#else
#define ROSA_B200_API
#endif

enum rosa_b200_dtype { ROSA_B200_F32 = 0, ROSA_B200_F16 = 1, ROSA_B200_BF16 = 2 };

/* Testing aid: OR-ed into gradient_mask, makes the backward contract its tiles on CUDA cores
 * instead of the tensor core (both paths compute the same sums; tests compare them). */
#define ROSA_B200_MASK_CUDA_CORE_CONTRACTION 0x100

/* status word values reported by rosa_b200_read_status */
enum rosa_b200_status {
  ROSA_B200_STATUS_OK = 0,
  ROSA_B200_STATUS_BAD_FIRST_OFFSET = 1, /* cu_seqlens[0] != 0            */
  ROSA_B200_STATUS_NOT_MONOTONE = 2,     /* cu_seqlens decreases somewhere */
  ROSA_B200_STATUS_BAD_LAST_OFFSET = 3,  /* cu_seqlens[-1] != N            */
  ROSA_B200_STATUS_CAPACITY = 4,         /* a slot would outgrow the history capacity */
  ROSA_B200_STATUS_MMA_TIMEOUT = 5       /* a bounded wait on the tensor core gave up: the
                                            gradients of that call are incomplete */
};

ROSA_B200_API int rosa_b200_abi_version(void);
ROSA_B200_API const char* rosa_b200_last_error(void);

/* ---------------------------------------------------------------- hard forward
 * Replaces hard_forward_cuda / hard_forward_varlen_cuda
 * (reference rosa_soft/csrc/rosa_soft.cpp:11-24, kernels
 * rosa_soft/csrc/cuda/rosa_soft_kernels.cu:202-241, 311-531, 1766-1920).
 * Writes the hard output (sign of the routed value row, or exact zero), the two
 * packed symbol tensors that are part of the operator's return contract, and --
 * optionally -- the global token index of the routed value row per (token, head)
 * (-1 = null route; local route index = route_token - sequence start). */
ROSA_B200_API size_t rosa_b200_hard_forward_workspace_bytes(int64_t N, int H, int64_t num_seq);

ROSA_B200_API int rosa_b200_hard_forward(const void* query, const void* key, const void* value, int dtype,
                           int64_t N, int H, int D, int Hv, int Dv, const int32_t* cu_seqlens,
                           int64_t num_seq, int64_t uniform_len, int64_t max_suffix_length,
                           void* output, int32_t* packed_query, int32_t* packed_key,
                           int32_t* route_token /* nullable, [N, H] */, void* workspace,
                           size_t workspace_bytes, void* stream);

/* The two halves of the forward for a caller that fuses its neighbours (the Q/K projections
 * that feed the operator and the output projection that consumes it, reference
 * examples/fit_soft_reference.py:374-415).
 * rosa_b200_pack_symbols is the contract of the projection epilogue: bit d of the int32 word of
 * (token, head) is set iff logit d is strictly positive (+0, -0 and NaN give 0; reference
 * rosa_soft/csrc/cuda/rosa_soft_kernels.cu:229-240), words laid out [num_seq, H, uniform_len]
 * (dense, uniform_len > 0) or [H, N] (packed, uniform_len = 0).  A GEMM epilogue that writes
 * these words never has to materialise the logits; this entry point does the same from logits
 * in memory, for one tensor.
 * rosa_b200_hard_forward_packed then runs matching and gathering on symbols the caller already
 * holds (no packing pass, the symbol tensors are inputs) and writes the routed signs as int8
 * -1 / 0 / +1 [N, H, Dv] for a consumer that takes them as integers.  Same workspace size, status
 * word and route_token output as rosa_b200_hard_forward; `D` is the symbol width in bits. */
ROSA_B200_API int rosa_b200_pack_symbols(const void* logits, int dtype, int64_t N, int H, int D,
                                         int64_t num_seq, int64_t uniform_len, int32_t* packed,
                                         void* stream);

ROSA_B200_API int rosa_b200_hard_forward_packed(
    const int32_t* packed_query, const int32_t* packed_key, const void* value, int dtype, int64_t N,
    int H, int D, int Hv, int Dv, const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
    int64_t max_suffix_length, int8_t* output, int32_t* route_token /* nullable, [N, H] */,
    void* workspace, size_t workspace_bytes, void* stream);

/* Hard forward without a workspace argument (no counterpart in the reference, whose
 * operators always allocate through the framework).  For hosts that cannot allocate device
 * memory at call time -- a server that gave all of it to its own arena and keeps the CUDA
 * allocator out of its request loop, or an embedding host without a device-memory manager.
 * Same inputs, outputs and results as rosa_b200_hard_forward; the scratch lives in a fixed
 * array inside the library's device image (8 MiB + 128 KiB held by every GPU that loads the
 * library, until the process exits).  Limits: N * H <= 1,048,576 token-heads and
 * num_seq <= 4096; larger problems are rejected with an error and nothing is enqueued.
 * The entry point calls no allocation routine.  The first call on a device resolves the
 * array's device address (cudaGetSymbolAddress, with that device current); make that first
 * call before starting any stream capture.  All calls on one GPU share the array, which
 * keeps the previous call's contents: the parts that must start at zero are cleared on
 * `stream` by each call, and calls that overlap on the same GPU race -- order them.
 * An inconsistent `cu_seqlens` makes the call a no-op with zero outputs, like the workspace
 * variant; rosa_b200_read_status(NULL, stream, &status) reports it.  The variant always uses
 * the run-length matcher (one symbol compare per causal pair): it has no room for the
 * occurrence bitmaps of the bit-parallel matchers, so on symbols of up to 8 bits it is several
 * times slower than rosa_b200_hard_forward; results are identical. */
ROSA_B200_API int rosa_b200_hard_forward_static(
    const void* query, const void* key, const void* value, int dtype, int64_t N, int H, int D,
    int Hv, int Dv, const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
    int64_t max_suffix_length, void* output, int32_t* packed_query, int32_t* packed_key,
    int32_t* route_token /* nullable, [N, H] */, void* stream);

/* ------------------------------------------------------------- surrogate VJP
 * Replaces surrogate_vjp_cuda / surrogate_vjp_varlen_cuda
 * (reference rosa_soft/csrc/rosa_soft.cpp:26-55, kernels
 * rosa_soft/csrc/cuda/rosa_soft_kernels.cu:534-1731, planners :1923-2638).
 * gradient_mask: bit0 query, bit1 key, bit2 value; outputs whose bit is clear may
 * be NULL.  Gradients are float32 in the layout of the corresponding input and
 * include the softsign Jacobian 1/(1+|x|)^2.  `dropout_seed` is a device int64
 * scalar, required iff dropout_p > 0.  `dropout_batch_offset` / `dropout_head_offset`
 * are added to the sequence ordinal / head index inside the dropout counter so a
 * shard of a larger problem reproduces the masks of the unsharded run.
 * Reduction order is fixed: results are bitwise reproducible run to run.
 * The workspace is sized for exactly the shape AND gradient_mask given to the sizing function
 * (a dense batch whose partial gradient rows would pass 6 GiB is run in slices of whole
 * sequences inside that one workspace, and the slice size follows the mask); a call with other
 * arguments than the ones sized for is refused with "workspace too small" when it needs more. */
ROSA_B200_API size_t rosa_b200_surrogate_vjp_workspace_bytes(int64_t N, int H, int D, int Hv, int Dv,
                                               int64_t num_seq, int64_t uniform_len,
                                               int64_t max_suffix_length, int gradient_mask);

ROSA_B200_API int rosa_b200_surrogate_vjp(const void* query, const void* key, const void* value,
                            const void* grad_output, int dtype, int64_t N, int H, int D, int Hv,
                            int Dv, const int32_t* cu_seqlens, int64_t num_seq,
                            int64_t uniform_len, int64_t max_suffix_length,
                            const int32_t* packed_query, const int32_t* packed_key,
                            const int64_t* dropout_seed, float scale, float dropout_p,
                            float mismatch_scale, int gradient_mask,
                            int64_t dropout_batch_offset, int64_t dropout_head_offset,
                            float* grad_query, float* grad_key, float* grad_value, void* workspace,
                            size_t workspace_bytes, void* stream);

/* Inspection of the routing decided by the preceding rosa_b200_hard_forward call on the same
 * `workspace` (same N, H, num_seq) and stream: per token-head the selected route as a position
 * local to its sequence (a in [1, i]; 0 = null route) and the exact match length that won
 * (0 for null).  These are `selected_route_indices` and the winning entry of
 * `exact_suffix_lengths` of the reference's inspect_rosa_soft (rosa_soft/testing.py:49-117,
 * rosa_soft/soft_reference.py:295-333) without its [B, H, T, T + 1] tensors: the winners are
 * already in the workspace, so no matching pass is repeated.  Either output may be NULL. */
ROSA_B200_API int rosa_b200_hard_forward_routes(const void* workspace, size_t workspace_bytes,
                                                int64_t N, int H, int64_t num_seq,
                                                int32_t* selected_route, int32_t* match_length,
                                                void* stream);

/* --------------------------------------------------------- hard inference batch
 * GPU equivalent of feeding whole streams to RosaRuntime.update_packed
 * (reference rosa_soft/csrc/rosa_runtime.cpp:333-482; match semantics :41-45,
 * :103-133; successor payload :455-467).  Symbols are token-major [N, H] words of up
 * to 32 bits; payload [N, Hp, Dp] float32.  Writes the payload row following the
 * match (zeros for null) to out [N, H, Dp] (nullable) and the matched key end
 * position local to its stream (-1 = null) to matched_end [N, H]. */
ROSA_B200_API size_t rosa_b200_hard_inference_workspace_bytes(int64_t N, int H, int64_t num_seq);

ROSA_B200_API int rosa_b200_hard_inference(const uint32_t* query_symbols, const uint32_t* key_symbols,
                             const float* payload, int64_t N, int H, int Hp, int Dp,
                             const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
                             int64_t max_suffix_length, float* out, int64_t* matched_end,
                             void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------ streaming hard inference
 * Chunked update with the per-slot state kept on the GPU: the device form of
 * RosaRuntime::update_packed (reference rosa_soft/csrc/rosa_runtime.cpp:333-482; the
 * automaton step it replaces :103-133; successor payload :455-467; reset :492-498).
 * The caller owns the state and passes it to every call (capacity a multiple of 32):
 *   key_masks       uint32 [slots, num_heads, 2^qk_bits, capacity/32]  one occurrence bitmap per
 *                                                     key symbol: bit p set iff key[p] == symbol
 *   query_history   uint8  [slots, num_heads, capacity]
 *   payload_history uint8  [slots, num_payload_heads, capacity]
 *   lengths         int32  [slots]                    tokens held per slot
 * A fresh or reset runtime is `lengths` = 0 and `key_masks` = 0; the histories need no
 * initialisation.  The chunk is token-major: query/key [chunk_tokens, num_heads], payload
 * [chunk_tokens, num_payload_heads], `chunk_offsets` int32 [slots + 1] on the device
 * (slot s owns chunk tokens [offsets[s], offsets[s+1]); empty slots allowed).  Symbols are
 * masked to qk_bits / payload_bits (1..8).  For every chunk token and head the call writes
 * the payload symbol that followed the latest-longest match (0 for no match) to `output`
 * and the matched key end position inside the slot's whole history (-1 for no match) to
 * `matched_key_end`, appends the chunk to the state and advances `lengths`.
 * `max_length_after` is a host-side upper bound of lengths[s] + chunk length over the slots
 * (the host knows it because it chose the chunk); it must not exceed `capacity`.  The result
 * does not depend on how a stream was cut into chunks.
 * A bad `chunk_offsets` or a slot that would outgrow `capacity` leaves the state untouched
 * and is reported through rosa_b200_read_status (ROSA_B200_STATUS_CAPACITY for the latter).
 * Calls that share a state must be ordered on one stream. */
ROSA_B200_API size_t rosa_b200_stream_workspace_bytes(int64_t chunk_tokens, int num_heads);

ROSA_B200_API int rosa_b200_stream_update(
    const uint8_t* query, const uint8_t* key, const uint8_t* payload,
    const int32_t* chunk_offsets, int64_t chunk_tokens, int slots, int num_heads,
    int num_payload_heads, int qk_bits, int payload_bits, int64_t max_suffix_length,
    uint32_t* key_masks, uint8_t* query_history, uint8_t* payload_history, int32_t* lengths,
    int64_t capacity, int64_t max_length_after, uint8_t* output, int64_t* matched_key_end,
    void* workspace, size_t workspace_bytes, void* stream);

/* Per-kernel timing for benchmarks (no counterpart in the reference, which times whole
 * steps with CUDA events in benchmarks/rosa_soft.py:151-173).  While enabled, every kernel
 * launch made by this library is bracketed by a CUDA event pair on the launching stream.
 * rosa_b200_profile_collect waits for the recorded events, returns the number of distinct
 * kernel names and fills, per name, the summed device time in milliseconds and the launch
 * count; it then forgets the records.  Off by default; do not enable around stream capture. */
ROSA_B200_API void rosa_b200_profile_enable(int on);
ROSA_B200_API int rosa_b200_profile_collect(const char** names, float* total_ms, int* launches,
                                            int capacity);

/* Copies the status of the last call that used `workspace` to the host: the offsets check
 * (1..3), the capacity check of the streaming update (4), or ROSA_B200_STATUS_MMA_TIMEOUT when
 * a CTA of the backward gave up its bounded wait for the tensor core (it then skips its
 * remaining accumulator read-backs, so the gradients are incomplete, but the context stays
 * usable).  `workspace == NULL` reads the status of the last rosa_b200_hard_forward_static
 * call on the current device (its scratch is inside the library, so the caller has no pointer
 * to pass).  This is the one entry point that synchronises `stream`. */
ROSA_B200_API int rosa_b200_read_status(const void* workspace, void* stream, int* status);

/* The decoding rosa_b200_read_status applies to the two device status words (plan word, tensor-core
 * word), as a pure host function: the plan's code when it is non-zero, else
 * ROSA_B200_STATUS_MMA_TIMEOUT when the second word is set, else ROSA_B200_STATUS_OK.  No
 * counterpart in the reference (its kernels assert on the device instead of reporting). */
ROSA_B200_API int rosa_b200_decode_status(int plan_word, int mma_word);

#ifdef __cplusplus
}
#endif
#endif /* ROSA_SOFT_B200_H_ */
