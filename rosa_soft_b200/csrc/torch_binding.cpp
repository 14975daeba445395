// Thin torch binding of librosa_soft_b200.so.
//
// Registers the operator schemas of the reference extension verbatim
// (reference rosa_soft/csrc/export.cpp:25-30), implements them for the CUDA dispatch key only
// (no CPU kernels exist) and forwards every call to the C ABI declared in
// include/rosa_soft_b200.h.  The error texts are the reference wrapper's
// (rosa_soft/csrc/rosa_soft.cpp:62-376) because callers and tests match on them; the checks
// themselves are organised here as one description of the call (`Call`) that is built in three
// stages -- placement and dtype, rank, extents -- from small rule lists.  Inputs of any stride
// are made contiguous, max_suffix_length is clipped to the sequence bound, scalars are narrowed
// to float32.  Outputs and the workspace come from the caching allocator on the input's device;
// work is enqueued on the current stream under a device guard; nothing synchronises unless
// ROSA_SOFT_B200_CHECK_STATUS=1 asks for the device status word after every call.
//
// Also registered: rosa_soft::hard_inference (batched hard inference), the backward operator
// rosa_soft::surrogate_vjp_sharded (dense or packed) that takes the dropout coordinate offsets
// of a shard, and the custom class
// torch.classes.rosa_soft.RosaRuntime (constructor and methods of the reference's class,
// rosa_soft/csrc/rosa_runtime.cpp:570-582) over the streaming entry point of the C ABI.
//
// One deliberate difference: the reference flags its backward as non-deterministic
// (global float atomics).  This backward reduces in a fixed order and is bitwise
// reproducible, so it does not raise under torch.use_deterministic_algorithms(True).
#include <Python.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/custom_class.h>
#include <torch/extension.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <initializer_list>
#include <limits>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "rosa_soft_b200.h"

extern "C" {
PyObject* PyInit__C(void) {
  static struct PyModuleDef module_def = {
      PyModuleDef_HEAD_INIT, "_C", "rosa_soft_b200 operator registration", -1, nullptr,
  };
  return PyModule_Create(&module_def);
}
}

namespace {

using torch::Tensor;
using Triple = std::tuple<Tensor, Tensor, Tensor>;

constexpr int64_t kInt32Max = std::numeric_limits<int32_t>::max();

struct Rule {
  bool holds;
  std::string message;
};

void enforce(std::initializer_list<Rule> rules) {
  for (const Rule& rule : rules) TORCH_CHECK(rule.holds, rule.message);
}

bool status_check_requested() {
  static const bool on = [] {
    const char* v = std::getenv("ROSA_SOFT_B200_CHECK_STATUS");
    return v != nullptr && v[0] == '1';
  }();
  return on;
}

void check_rc(int rc, const char* op) {
  TORCH_CHECK(rc == 0, "rosa_soft::", op, ": ", rosa_b200_last_error());
}

// Opt-in (it synchronises the stream): turn the device status word into an exception.
void maybe_check_status(const Tensor& workspace, const char* op) {
  if (!status_check_requested()) return;
  int status = 0;
  check_rc(rosa_b200_read_status(workspace.data_ptr(), at::cuda::getCurrentCUDAStream().stream(),
                                 &status),
           op);
  TORCH_CHECK(status == ROSA_B200_STATUS_OK, "rosa_soft::", op, ": device status ", status,
              status == ROSA_B200_STATUS_MMA_TIMEOUT
                  ? " (a tensor-core wait gave up; gradients are incomplete)"
                  : " (cu_seqlens must start at zero, be nondecreasing and end at the packed "
                    "token count)");
}

// The geometry of one operator call, filled while the inputs are checked.
struct Call {
  bool dense = true;
  int64_t tokens = 0, heads = 0, bits = 0, value_heads = 0, value_dim = 0;
  int64_t sequences = 0, uniform_len = 0, horizon = 0;
  Tensor q, k, v, cu;   // contiguous
  int dtype = ROSA_B200_F32;

  const int32_t* offsets() const { return dense ? nullptr : cu.data_ptr<int32_t>(); }
};

Call describe_call(const Tensor& query, const Tensor& key, const Tensor& value, const Tensor& cu,
                   int64_t max_suffix_length) {
  Call c;
  c.dense = !cu.defined();
  // stage 1: placement and element types
  enforce({{query.is_cuda(), "query must be a CUDA tensor"},
           {key.is_cuda(), "key must be a CUDA tensor"},
           {value.is_cuda(), "value must be a CUDA tensor"}});
  if (c.dense) {
    enforce({{query.device() == key.device(), "query and key must be on the same CUDA device"},
             {query.device() == value.device(),
              "query and value must be on the same CUDA device"}});
  } else {
    enforce({{cu.is_cuda(), "cu_seqlens must be a CUDA tensor"},
             {query.device() == key.device() && query.device() == value.device() &&
                  query.device() == cu.device(),
              "all inputs and cu_seqlens must be on the same CUDA device"}});
  }
  const auto st = query.scalar_type();
  enforce({{st == torch::kFloat32 || st == torch::kFloat16 || st == torch::kBFloat16,
            "query must be float32, float16, or bfloat16"},
           {st == key.scalar_type(), "query/key dtype mismatch"},
           {st == value.scalar_type(), "query/value dtype mismatch"}});
  c.dtype = st == torch::kFloat32 ? ROSA_B200_F32 : st == torch::kFloat16 ? ROSA_B200_F16
                                                                          : ROSA_B200_BF16;
  // stage 2: ranks
  if (c.dense)
    enforce({{query.dim() == 4, "query must have shape (B, T, H, D)"},
             {key.dim() == 4, "key must have shape (B, T, H, D)"},
             {value.dim() == 4, "value must have shape (B, T, H_p, D_p)"}});
  else
    enforce({{query.dim() == 3, "query must have shape (N, H, D)"},
             {key.dim() == 3, "key must have shape (N, H, D)"},
             {value.dim() == 3, "value must have shape (N, H_p, D_p)"}});
  // stage 3: extents
  const int hd = c.dense ? 2 : 1;   // index of the head dimension
  c.heads = query.size(hd);
  c.bits = query.size(hd + 1);
  c.value_heads = value.size(hd);
  c.value_dim = value.size(hd + 1);
  if (c.dense) {
    c.sequences = query.size(0);
    c.uniform_len = query.size(1);
    c.tokens = c.sequences * c.uniform_len;
    enforce({{c.sequences > 0, "batch size must be positive"},
             {c.uniform_len > 0, "sequence length must be positive"},
             {c.heads > 0, "query head count must be positive"},
             {c.value_heads > 0, "value head count must be positive"},
             {c.value_dim > 0, "value dimension must be positive"},
             {c.sequences == key.size(0), "query/key batch mismatch"},
             {c.uniform_len == key.size(1), "query/key sequence mismatch"},
             {c.heads == key.size(2), "query/key head mismatch"},
             {c.bits == key.size(3), "query/key bit dimension mismatch"},
             {c.sequences == value.size(0), "query/value batch mismatch"},
             {c.uniform_len == value.size(1), "query/value sequence mismatch"}});
  } else {
    c.tokens = query.size(0);
    enforce({{c.tokens > 0, "packed token count must be positive"},
             {c.heads > 0, "query head count must be positive"},
             {c.value_heads > 0, "value head count must be positive"},
             {c.value_dim > 0, "value dimension must be positive"},
             {c.tokens == key.size(0), "query/key token mismatch"},
             {c.tokens == value.size(0), "query/value token mismatch"},
             {c.heads == key.size(1), "query/key head mismatch"},
             {c.bits == key.size(2), "query/key bit dimension mismatch"}});
  }
  enforce({{c.heads % c.value_heads == 0, "query heads must be divisible by value heads"},
           {c.bits > 0 && c.bits <= 32, "query/key bit dimension must be in [1, 32]"},
           {c.tokens * c.heads <= kInt32Max,
            c.dense ? "B * T * H must fit in int32" : "N * H must fit in int32"},
           {c.value_dim < kInt32Max, "value dimension is too large for the CUDA kernel index stride"}});
  if (!c.dense) {
    enforce({{cu.scalar_type() == torch::kInt32, "cu_seqlens must be int32"},
             {cu.dim() == 1 && cu.numel() >= 2,
              "cu_seqlens must be one-dimensional with at least two entries"},
             {cu.numel() - 1 < kInt32Max,
              "number of packed sequences is too large for CUDA indexing"}});
    c.sequences = cu.numel() - 1;
    c.cu = cu.contiguous();
  }
  enforce({{max_suffix_length >= 1, "max_suffix_length must be >= 1"}});
  c.horizon = std::min<int64_t>(max_suffix_length, c.dense ? c.uniform_len : c.tokens);
  c.q = query.contiguous();
  c.k = key.contiguous();
  c.v = value.contiguous();
  return c;
}

struct Controls {
  float scale, dropout_p, mismatch_scale;
};

// Narrowing of the three float controls with the range rules of the operator contract.
Controls narrow_controls(int64_t horizon, double scale, double dropout_p, double mismatch_scale) {
  const double float_max = static_cast<double>(std::numeric_limits<float>::max());
  const auto positive_normal = [](double x) {
    const float f = static_cast<float>(x);
    return f > 0.0f && std::isnormal(f);
  };
  enforce({{std::isfinite(scale) && scale > 0.0, "scale must be finite and > 0"},
           {std::isfinite(dropout_p) && dropout_p >= 0.0 && dropout_p <= 1.0 - std::ldexp(1.0, -24),
            "dropout_p must be finite and in [0, 1 - 2^-24]"},
           {std::isfinite(mismatch_scale) && mismatch_scale > 0.0,
            "mismatch_scale must be finite and > 0"},
           {positive_normal(scale),
            "scale must be representable as a positive normal float32 value"},
           {scale <= float_max / static_cast<double>(horizon),
            "max_suffix_length * scale must fit in float32"},
           {positive_normal(mismatch_scale),
            "mismatch_scale must be representable as a positive normal float32 value"},
           {mismatch_scale <= float_max / (static_cast<double>(horizon) * scale),
            "mismatch_scale * max_suffix_length * scale must fit in float32"}});
  return {static_cast<float>(scale), static_cast<float>(dropout_p),
          static_cast<float>(mismatch_scale)};
}

void check_backward_extras(const Call& c, const Tensor& query, const Tensor& grad_output,
                           const Tensor& packed_q, const Tensor& packed_k, const Tensor& seed,
                           double dropout_p, int64_t gradient_mask) {
  std::vector<int64_t> go_shape = query.sizes().vec();
  go_shape.back() = c.value_dim;
  enforce({{grad_output.is_cuda(), "grad_output must be a CUDA tensor"},
           {grad_output.device() == query.device(),
            "grad_output must be on the same CUDA device as query"},
           {grad_output.scalar_type() == query.scalar_type(), "grad_output dtype mismatch"},
           {grad_output.sizes() == torch::IntArrayRef(go_shape), "grad_output shape mismatch"}});
  const std::pair<const Tensor*, const char*> symbols[2] = {{&packed_q, "packed_query_symbols"},
                                                            {&packed_k, "packed_key_symbols"}};
  for (const auto& [t, name] : symbols) {
    const std::string n = name;
    enforce({{t->is_cuda(), n + " must be a CUDA tensor"},
             {t->device() == query.device(), n + " must be on the same CUDA device as query"},
             {t->scalar_type() == torch::kInt32, n + " must be int32"}});
    if (c.dense)
      enforce({{t->dim() == 3, n + " must have shape (B, H, T)"},
               {t->dim() == 3 && t->size(0) == c.sequences, n + " batch mismatch"},
               {t->dim() == 3 && t->size(1) == c.heads, n + " head mismatch"},
               {t->dim() == 3 && t->size(2) == c.uniform_len, n + " sequence mismatch"}});
    else
      enforce({{t->dim() == 2, n + " must have shape (H, N)"},
               {t->dim() == 2 && t->size(0) == c.heads && t->size(1) == c.tokens,
                n + " shape mismatch"}});
  }
  enforce({{seed.is_cuda(), "dropout_seed must be a CUDA tensor"},
           {seed.device() == query.device(),
            "dropout_seed must be on the same CUDA device as query"},
           {seed.scalar_type() == torch::kInt64, "dropout_seed must have dtype int64"},
           {seed.numel() == (dropout_p > 0.0 ? 1 : 0),
            "dropout_seed must be scalar exactly when dropout_p > 0"},
           {gradient_mask >= 1 && gradient_mask <= 7,
            "gradient_mask must be an integer bit mask in [1, 7]"}});
}

Tensor make_workspace(const Tensor& like, size_t bytes) {
  return torch::empty({static_cast<int64_t>(bytes)}, like.options().dtype(torch::kUInt8));
}

Triple run_hard_forward(const Tensor& query, const Tensor& key, const Tensor& value,
                        const Tensor& cu, int64_t max_suffix_length) {
  const Call c = describe_call(query, key, value, cu, max_suffix_length);
  const c10::cuda::CUDAGuard guard(query.device());
  std::vector<int64_t> out_shape = c.q.sizes().vec();
  out_shape.back() = c.value_dim;
  const auto i32 = c.q.options().dtype(torch::kInt32);
  Tensor out = torch::empty(out_shape, c.q.options());
  Tensor pq = c.dense ? torch::empty({c.sequences, c.heads, c.uniform_len}, i32)
                      : torch::empty({c.heads, c.tokens}, i32);
  Tensor pk = torch::empty_like(pq);
  const size_t bytes = rosa_b200_hard_forward_workspace_bytes(c.tokens, (int)c.heads, c.sequences);
  Tensor ws = make_workspace(c.q, bytes);
  check_rc(rosa_b200_hard_forward(c.q.data_ptr(), c.k.data_ptr(), c.v.data_ptr(), c.dtype, c.tokens,
                                  (int)c.heads, (int)c.bits, (int)c.value_heads, (int)c.value_dim,
                                  c.offsets(), c.sequences, c.uniform_len, c.horizon,
                                  out.data_ptr(), pq.data_ptr<int32_t>(), pk.data_ptr<int32_t>(),
                                  nullptr, ws.data_ptr(), bytes,
                                  at::cuda::getCurrentCUDAStream().stream()),
           "hard_forward");
  maybe_check_status(ws, "hard_forward");
  return {out, pq, pk};
}

Triple run_surrogate_vjp(const Tensor& query, const Tensor& key, const Tensor& value,
                         const Tensor& cu, const Tensor& grad_output, const Tensor& packed_q,
                         const Tensor& packed_k, const Tensor& seed, int64_t max_suffix_length,
                         double scale, double dropout_p, double mismatch_scale, int64_t mask,
                         int64_t batch_offset, int64_t head_offset) {
  const Call c = describe_call(query, key, value, cu, max_suffix_length);
  check_backward_extras(c, query, grad_output, packed_q, packed_k, seed, dropout_p, mask);
  const Controls sc = narrow_controls(c.horizon, scale, dropout_p, mismatch_scale);
  const c10::cuda::CUDAGuard guard(query.device());
  const Tensor go = grad_output.contiguous();
  const Tensor pq = packed_q.contiguous(), pk = packed_k.contiguous(), sd = seed.contiguous();
  const auto f32 = c.q.options().dtype(torch::kFloat32);
  Tensor dq = (mask & 1) ? torch::empty(c.q.sizes(), f32) : torch::empty({0}, f32);
  Tensor dk = (mask & 2) ? torch::empty(c.k.sizes(), f32) : torch::empty({0}, f32);
  Tensor dv = (mask & 4) ? torch::empty(c.v.sizes(), f32) : torch::empty({0}, f32);
  const size_t bytes = rosa_b200_surrogate_vjp_workspace_bytes(
      c.tokens, (int)c.heads, (int)c.bits, (int)c.value_heads, (int)c.value_dim, c.sequences,
      c.uniform_len, c.horizon, (int)mask);
  Tensor ws = make_workspace(c.q, bytes);
  check_rc(rosa_b200_surrogate_vjp(
               c.q.data_ptr(), c.k.data_ptr(), c.v.data_ptr(), go.data_ptr(), c.dtype, c.tokens,
               (int)c.heads, (int)c.bits, (int)c.value_heads, (int)c.value_dim, c.offsets(),
               c.sequences, c.uniform_len, c.horizon, pq.data_ptr<int32_t>(),
               pk.data_ptr<int32_t>(), sc.dropout_p > 0.0f ? sd.data_ptr<int64_t>() : nullptr,
               sc.scale, sc.dropout_p, sc.mismatch_scale, (int)mask, batch_offset, head_offset,
               (mask & 1) ? dq.data_ptr<float>() : nullptr,
               (mask & 2) ? dk.data_ptr<float>() : nullptr,
               (mask & 4) ? dv.data_ptr<float>() : nullptr, ws.data_ptr(), bytes,
               at::cuda::getCurrentCUDAStream().stream()),
           "surrogate_vjp");
  maybe_check_status(ws, "surrogate_vjp");
  return {dq, dk, dv};
}

Triple hard_forward_op(Tensor query, Tensor key, Tensor value, int64_t max_suffix_length) {
  return run_hard_forward(query, key, value, Tensor(), max_suffix_length);
}

Triple hard_forward_varlen_op(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens,
                              int64_t max_suffix_length) {
  return run_hard_forward(query, key, value, cu_seqlens, max_suffix_length);
}

Triple surrogate_vjp_masked_op(Tensor query, Tensor key, Tensor value, Tensor grad_output,
                               Tensor packed_query_symbols, Tensor packed_key_symbols,
                               Tensor dropout_seed, int64_t max_suffix_length, double scale,
                               double dropout_p, double mismatch_scale, int64_t gradient_mask) {
  return run_surrogate_vjp(query, key, value, Tensor(), grad_output, packed_query_symbols,
                           packed_key_symbols, dropout_seed, max_suffix_length, scale, dropout_p,
                           mismatch_scale, gradient_mask, 0, 0);
}

Triple surrogate_vjp_varlen_masked_op(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens,
                                      Tensor grad_output, Tensor packed_query_symbols,
                                      Tensor packed_key_symbols, Tensor dropout_seed,
                                      int64_t max_suffix_length, double scale, double dropout_p,
                                      double mismatch_scale, int64_t gradient_mask) {
  return run_surrogate_vjp(query, key, value, cu_seqlens, grad_output, packed_query_symbols,
                           packed_key_symbols, dropout_seed, max_suffix_length, scale, dropout_p,
                           mismatch_scale, gradient_mask, 0, 0);
}

// A shard of a larger problem: same as the masked operators plus the global coordinates of
// the shard's first sequence and first head inside the dropout counter.
Triple surrogate_vjp_sharded_op(Tensor query, Tensor key, Tensor value,
                                std::optional<Tensor> cu_seqlens, Tensor grad_output,
                                Tensor packed_query_symbols, Tensor packed_key_symbols,
                                Tensor dropout_seed, int64_t max_suffix_length, double scale,
                                double dropout_p, double mismatch_scale, int64_t gradient_mask,
                                int64_t batch_offset, int64_t head_offset) {
  TORCH_CHECK(batch_offset >= 0 && head_offset >= 0 && batch_offset <= kInt32Max &&
                  head_offset <= kInt32Max,
              "shard offsets must be non-negative 32-bit values");
  return run_surrogate_vjp(query, key, value, cu_seqlens.has_value() ? *cu_seqlens : Tensor(),
                           grad_output, packed_query_symbols, packed_key_symbols, dropout_seed,
                           max_suffix_length, scale, dropout_p, mismatch_scale, gradient_mask,
                           batch_offset, head_offset);
}

// Batched hard inference: query/key symbols int32 [streams, T, H] (or packed [N, H] with
// cu_seqlens), payload float32 [streams, T, Hp, Dp] / [N, Hp, Dp].
std::tuple<Tensor, Tensor> hard_inference_op(Tensor query_symbols, Tensor key_symbols,
                                             Tensor payload, std::optional<Tensor> cu_seqlens,
                                             int64_t max_suffix_length) {
  const bool dense = !cu_seqlens.has_value();
  TORCH_CHECK(query_symbols.is_cuda() && key_symbols.is_cuda() && payload.is_cuda(),
              "hard_inference requires CUDA tensors");
  TORCH_CHECK(query_symbols.scalar_type() == torch::kInt32 &&
                  key_symbols.scalar_type() == torch::kInt32,
              "symbols must be int32 words");
  TORCH_CHECK(payload.scalar_type() == torch::kFloat32, "payload must be float32");
  TORCH_CHECK(query_symbols.sizes() == key_symbols.sizes(), "query/key symbol shape mismatch");
  TORCH_CHECK(query_symbols.dim() == (dense ? 3 : 2) && payload.dim() == (dense ? 4 : 3),
              "symbols must be (streams, T, H) with payload (streams, T, Hp, Dp), or (N, H) with "
              "payload (N, Hp, Dp) and cu_seqlens");
  TORCH_CHECK(max_suffix_length >= 1, "max_suffix_length must be >= 1");
  const c10::cuda::CUDAGuard guard(query_symbols.device());
  const Tensor q = query_symbols.contiguous(), k = key_symbols.contiguous(),
               p = payload.contiguous();
  const int64_t N = dense ? q.size(0) * q.size(1) : q.size(0);
  const int64_t H = q.size(dense ? 2 : 1);
  const int64_t Hp = p.size(dense ? 2 : 1), Dp = p.size(dense ? 3 : 2);
  TORCH_CHECK(p.numel() == N * Hp * Dp, "payload token count mismatch");
  TORCH_CHECK(H % Hp == 0, "heads must be divisible by payload heads");
  Tensor cuc;
  if (!dense) {
    cuc = cu_seqlens->contiguous();
    TORCH_CHECK(cuc.is_cuda() && cuc.scalar_type() == torch::kInt32 && cuc.dim() == 1 &&
                    cuc.numel() >= 2,
                "cu_seqlens must be a one-dimensional CUDA int32 tensor");
  }
  const int64_t S = dense ? q.size(0) : cuc.numel() - 1;
  const int64_t T = dense ? q.size(1) : 0;
  std::vector<int64_t> out_shape = q.sizes().vec();
  Tensor matched = torch::empty(out_shape, q.options().dtype(torch::kInt64));
  out_shape.push_back(Dp);
  Tensor out = torch::empty(out_shape, p.options());
  const size_t bytes = rosa_b200_hard_inference_workspace_bytes(N, (int)H, S);
  Tensor ws = make_workspace(q, bytes);
  check_rc(rosa_b200_hard_inference(
               reinterpret_cast<const uint32_t*>(q.data_ptr<int32_t>()),
               reinterpret_cast<const uint32_t*>(k.data_ptr<int32_t>()), p.data_ptr<float>(), N,
               (int)H, (int)Hp, (int)Dp, dense ? nullptr : cuc.data_ptr<int32_t>(), S, T,
               max_suffix_length, out.data_ptr<float>(), matched.data_ptr<int64_t>(), ws.data_ptr(),
               bytes, at::cuda::getCurrentCUDAStream().stream()),
           "hard_inference");
  maybe_check_status(ws, "hard_inference");
  return {out, matched};
}

// ------------------------------------------------------------------ RosaRuntime class
// torch.classes.rosa_soft.RosaRuntime with the reference's constructor and methods
// (rosa_soft/csrc/rosa_runtime.cpp:300-331, 333-482, 484-582): update_packed(cu_seqlens, query,
// key, payload) -> (output uint8 [total, H], matched_key_end int64 [total, H]), reset, close,
// stats.  The state (query / payload histories and one occurrence bitmap per key symbol) lives
// on the GPU of the first update and every update is one rosa_b200_stream_update call on the
// current stream; cu_seqlens is read on the host (int32 or int64, CPU or CUDA) like the
// reference reads it, because the chunk lengths size the state.
class RosaRuntimeClass : public torch::CustomClassHolder {
 public:
  RosaRuntimeClass(int64_t num_heads, int64_t num_payload_heads, int64_t qk_bits,
                   int64_t payload_bits, int64_t max_suffix_length)
      : heads_(num_heads), payload_heads_(num_payload_heads), qk_bits_(qk_bits),
        payload_bits_(payload_bits), horizon_(max_suffix_length) {
    enforce({{heads_ > 0, "num_heads must be positive"},
             {payload_heads_ > 0, "num_payload_heads must be positive"},
             {payload_heads_ > 0 && heads_ % payload_heads_ == 0,
              "num_heads must be divisible by num_payload_heads"},
             {qk_bits_ > 0 && qk_bits_ <= 8, "qk_bits must be in [1, 8]"},
             {payload_bits_ > 0 && payload_bits_ <= 8, "payload_bits must be in [1, 8]"},
             {horizon_ > 0 && horizon_ <= kInt32Max, "max_suffix_length must be in [1, int32_max]"}});
  }

  std::tuple<Tensor, Tensor> update_packed(const Tensor& cu_seqlens, const Tensor& query,
                                           const Tensor& key, const Tensor& payload) {
    std::lock_guard<std::mutex> lock(mutex_);
    TORCH_CHECK(!closed_, "RosaRuntime is closed");
    enforce({{query.is_cuda() && key.is_cuda() && payload.is_cuda(),
              "RosaRuntime keeps its state on the GPU: query, key and payload must be CUDA tensors"},
             {query.scalar_type() == torch::kUInt8 && key.scalar_type() == torch::kUInt8 &&
                  payload.scalar_type() == torch::kUInt8,
              "query, key and payload must have dtype uint8"},
             {query.dim() == 2 && key.dim() == 2 && payload.dim() == 2,
              "query, key and payload must be two-dimensional (total_tokens, heads)"},
             {cu_seqlens.dim() == 1 && cu_seqlens.numel() >= 2,
              "cu_seqlens must be one-dimensional with at least two entries"},
             {cu_seqlens.scalar_type() == torch::kInt32 || cu_seqlens.scalar_type() == torch::kInt64,
              "cu_seqlens must be int32 or int64"}});
    enforce({{query.sizes() == key.sizes(), "query/key shape mismatch"},
             {query.size(1) == heads_, "query head count must equal num_heads"},
             {payload.size(1) == payload_heads_, "payload head count must equal num_payload_heads"},
             {payload.size(0) == query.size(0), "query/payload token mismatch"},
             {query.device() == key.device() && query.device() == payload.device(),
              "query, key and payload must be on the same CUDA device"}});
    const Tensor host_cu = cu_seqlens.to(torch::kCPU, torch::kInt64).contiguous();
    const int64_t* cu = host_cu.data_ptr<int64_t>();
    const int64_t slots = host_cu.numel() - 1;
    const int64_t total = query.size(0);
    TORCH_CHECK(cu[0] == 0, "cu_seqlens must start at 0");
    for (int64_t s = 0; s < slots; ++s)
      TORCH_CHECK(cu[s + 1] >= cu[s], "cu_seqlens must be non-decreasing");
    TORCH_CHECK(cu[slots] == total, "cu_seqlens[-1] must equal the total token count");
    if (slots_ < 0) {
      slots_ = slots;
      device_ = query.device();
      lengths_host_.assign(static_cast<size_t>(slots), 0);
    } else {
      TORCH_CHECK(slots == slots_, "RosaRuntime slot count is fixed after the first update");
      TORCH_CHECK(query.device() == device_, "RosaRuntime state lives on another device");
    }
    std::vector<int64_t> after(lengths_host_);
    int64_t needed = 0;
    for (int64_t s = 0; s < slots; ++s) {
      after[s] += cu[s + 1] - cu[s];
      needed = std::max(needed, after[s]);
    }
    TORCH_CHECK(needed <= kInt32Max - 31, "ROSA sequence length exceeded int32 range");
    const c10::cuda::CUDAGuard guard(device_);
    grow(needed);
    const auto u8 = query.options();
    Tensor output = torch::empty({total, heads_}, u8);
    Tensor matched = torch::empty({total, heads_}, u8.dtype(torch::kInt64));
    const Tensor q = query.contiguous(), k = key.contiguous(), p = payload.contiguous();
    const Tensor offsets = host_cu.to(torch::kInt32).to(device_);
    const size_t bytes = rosa_b200_stream_workspace_bytes(total, (int)heads_);
    Tensor ws = make_workspace(q, bytes);
    check_rc(rosa_b200_stream_update(
                 q.data_ptr<uint8_t>(), k.data_ptr<uint8_t>(), p.data_ptr<uint8_t>(),
                 offsets.data_ptr<int32_t>(), total, (int)slots, (int)heads_, (int)payload_heads_,
                 (int)qk_bits_, (int)payload_bits_, horizon_,
                 reinterpret_cast<uint32_t*>(key_masks_.data_ptr<int32_t>()),
                 query_history_.data_ptr<uint8_t>(), payload_history_.data_ptr<uint8_t>(),
                 lengths_.data_ptr<int32_t>(), capacity_, needed, output.data_ptr<uint8_t>(),
                 matched.data_ptr<int64_t>(), ws.data_ptr(), bytes,
                 at::cuda::getCurrentCUDAStream().stream()),
             "RosaRuntime.update_packed");
    lengths_host_ = after;   // committed only once the update has been enqueued
    return {output, matched};
  }

  void reset() {
    std::lock_guard<std::mutex> lock(mutex_);
    TORCH_CHECK(!closed_, "RosaRuntime is closed");
    clear();
  }

  void close() {
    std::lock_guard<std::mutex> lock(mutex_);
    clear();
    closed_ = true;
  }

  // (states, edges, payload_symbols, automata, sequences, logical_bytes): there is no
  // automaton, so the first two are zero; the bytes are those of the histories and bitmaps.
  std::tuple<int64_t, int64_t, int64_t, int64_t, int64_t, int64_t> stats() const {
    std::lock_guard<std::mutex> lock(mutex_);
    int64_t tokens = 0;
    for (int64_t n : lengths_host_) tokens += n;
    const int64_t slots = slots_ < 0 ? 0 : slots_;
    const int64_t bytes =
        tokens * (heads_ * (1 + ((int64_t)1 << qk_bits_) / 8) + payload_heads_);
    return {0, 0, tokens * payload_heads_, slots * heads_, slots, bytes};
  }

 private:
  void clear() {
    key_masks_ = Tensor();
    query_history_ = Tensor();
    payload_history_ = Tensor();
    lengths_ = Tensor();
    lengths_host_.clear();
    slots_ = -1;
    capacity_ = 0;
  }

  // Room for `needed` tokens per slot: the capacity doubles, old contents are kept.  All
  // copies are enqueued on the current stream, which also orders them after earlier updates.
  void grow(int64_t needed) {
    if (needed <= capacity_ && capacity_ > 0) return;
    int64_t capacity = std::max<int64_t>(256, capacity_);
    while (capacity < needed) capacity *= 2;
    const auto u8 = torch::TensorOptions().device(device_).dtype(torch::kUInt8);
    Tensor masks = torch::zeros({slots_, heads_, (int64_t)1 << qk_bits_, capacity / 32},
                                u8.dtype(torch::kInt32));
    Tensor qh = torch::empty({slots_, heads_, capacity}, u8);
    Tensor ph = torch::empty({slots_, payload_heads_, capacity}, u8);
    if (capacity_ > 0) {
      masks.narrow(3, 0, capacity_ / 32).copy_(key_masks_);
      qh.narrow(2, 0, capacity_).copy_(query_history_);
      ph.narrow(2, 0, capacity_).copy_(payload_history_);
    } else {
      lengths_ = torch::zeros({slots_}, u8.dtype(torch::kInt32));
    }
    key_masks_ = masks;
    query_history_ = qh;
    payload_history_ = ph;
    capacity_ = capacity;
  }

  const int64_t heads_, payload_heads_, qk_bits_, payload_bits_, horizon_;
  int64_t slots_ = -1, capacity_ = 0;
  bool closed_ = false;
  c10::Device device_{c10::kCPU};
  std::vector<int64_t> lengths_host_;
  Tensor key_masks_, query_history_, payload_history_, lengths_;
  mutable std::mutex mutex_;
};

}  // namespace

#ifdef ROSA_WITH_CUDA
TORCH_LIBRARY(rosa_soft, m) {
  m.def("hard_forward(Tensor query, Tensor key, Tensor value, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)");
  m.def("hard_forward_varlen(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)");
  m.def("surrogate_vjp_masked(Tensor query, Tensor key, Tensor value, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("surrogate_vjp_varlen_masked(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("surrogate_vjp_sharded(Tensor query, Tensor key, Tensor value, Tensor? cu_seqlens, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask, int batch_offset, int head_offset) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("hard_inference(Tensor query_symbols, Tensor key_symbols, Tensor payload, Tensor? cu_seqlens, int max_suffix_length) -> (Tensor output, Tensor matched_key_end_positions)");
  m.class_<RosaRuntimeClass>("RosaRuntime")
      .def(torch::init<int64_t, int64_t, int64_t, int64_t, int64_t>())
      .def("update_packed", &RosaRuntimeClass::update_packed)
      .def("reset", &RosaRuntimeClass::reset)
      .def("close", &RosaRuntimeClass::close)
      .def("stats", &RosaRuntimeClass::stats);
}

TORCH_LIBRARY_IMPL(rosa_soft, CUDA, m) {
  m.impl("hard_forward", &hard_forward_op);
  m.impl("hard_forward_varlen", &hard_forward_varlen_op);
  m.impl("surrogate_vjp_masked", &surrogate_vjp_masked_op);
  m.impl("surrogate_vjp_varlen_masked", &surrogate_vjp_varlen_masked_op);
  m.impl("surrogate_vjp_sharded", &surrogate_vjp_sharded_op);
  m.impl("hard_inference", &hard_inference_op);
}
#endif
