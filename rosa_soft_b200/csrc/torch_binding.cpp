// Thin torch binding of librosa_soft_b200.so.
//
// Registers the operator schemas of the reference extension verbatim
// (reference rosa_soft/csrc/export.cpp:25-30) plus one extra operator for batched hard
// inference, implements them for the CUDA dispatch key only (no CPU kernels exist), and
// forwards every call to the C ABI declared in include/rosa_soft_b200.h.  Validation and
// error texts follow the reference wrapper (rosa_soft/csrc/rosa_soft.cpp:62-549): inputs of
// any stride are made contiguous, max_suffix_length is clipped to the sequence bound,
// scalars are narrowed to float32 with the same range checks.  Outputs and the workspace
// come from the caching allocator on the input's device; work is enqueued on the current
// stream under a device guard; nothing synchronises.
//
// One deliberate difference: the reference flags its backward as non-deterministic
// (global float atomics).  This backward reduces in a fixed order and is bitwise
// reproducible, so it does not raise under torch.use_deterministic_algorithms(True).
#include <Python.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <tuple>

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

constexpr int64_t kKernelIndexSafetyMargin = 128;

int dtype_code(c10::ScalarType t) {
  if (t == torch::kFloat32) return ROSA_B200_F32;
  if (t == torch::kFloat16) return ROSA_B200_F16;
  return ROSA_B200_BF16;
}

bool is_supported_logit_dtype(c10::ScalarType dtype) {
  return dtype == torch::kFloat32 || dtype == torch::kFloat16 || dtype == torch::kBFloat16;
}

void check_rc(int rc, const char* op) {
  TORCH_CHECK(rc == 0, "rosa_soft::", op, ": ", rosa_b200_last_error());
}

float to_positive_normal_float(double value, const char* name) {
  const float converted = static_cast<float>(value);
  TORCH_CHECK(converted > 0.0f && std::isnormal(converted), name,
              " must be representable as a positive normal float32 value");
  return converted;
}

struct SurrogateScalars {
  float scale, dropout_p, mismatch_scale;
};

SurrogateScalars check_surrogate_scalars(int64_t effective_w, double scale, double dropout_p,
                                         double mismatch_scale) {
  TORCH_CHECK(std::isfinite(scale) && scale > 0.0, "scale must be finite and > 0");
  TORCH_CHECK(std::isfinite(dropout_p) && dropout_p >= 0.0 &&
                  dropout_p <= 1.0 - std::ldexp(1.0, -24),
              "dropout_p must be finite and in [0, 1 - 2^-24]");
  TORCH_CHECK(std::isfinite(mismatch_scale) && mismatch_scale > 0.0,
              "mismatch_scale must be finite and > 0");
  const float scale_f = to_positive_normal_float(scale, "scale");
  const double float_max = static_cast<double>(std::numeric_limits<float>::max());
  TORCH_CHECK(scale <= float_max / static_cast<double>(effective_w),
              "max_suffix_length * scale must fit in float32");
  const float mismatch_f = to_positive_normal_float(mismatch_scale, "mismatch_scale");
  TORCH_CHECK(mismatch_scale <= float_max / (static_cast<double>(effective_w) * scale),
              "mismatch_scale * max_suffix_length * scale must fit in float32");
  return {scale_f, static_cast<float>(dropout_p), mismatch_f};
}

void check_common_inputs(const Tensor& query, const Tensor& key, const Tensor& value,
                         int64_t max_suffix_length) {
  TORCH_CHECK(query.is_cuda(), "query must be a CUDA tensor");
  TORCH_CHECK(key.is_cuda(), "key must be a CUDA tensor");
  TORCH_CHECK(value.is_cuda(), "value must be a CUDA tensor");
  TORCH_CHECK(query.device() == key.device(), "query and key must be on the same CUDA device");
  TORCH_CHECK(query.device() == value.device(),
              "query and value must be on the same CUDA device");
  TORCH_CHECK(is_supported_logit_dtype(query.scalar_type()),
              "query must be float32, float16, or bfloat16");
  TORCH_CHECK(query.scalar_type() == key.scalar_type(), "query/key dtype mismatch");
  TORCH_CHECK(query.scalar_type() == value.scalar_type(), "query/value dtype mismatch");
  TORCH_CHECK(query.dim() == 4, "query must have shape (B, T, H, D)");
  TORCH_CHECK(key.dim() == 4, "key must have shape (B, T, H, D)");
  TORCH_CHECK(value.dim() == 4, "value must have shape (B, T, H_p, D_p)");
  TORCH_CHECK(query.size(0) > 0, "batch size must be positive");
  TORCH_CHECK(query.size(1) > 0, "sequence length must be positive");
  TORCH_CHECK(query.size(2) > 0, "query head count must be positive");
  TORCH_CHECK(value.size(2) > 0, "value head count must be positive");
  TORCH_CHECK(value.size(3) > 0, "value dimension must be positive");
  TORCH_CHECK(query.size(0) == key.size(0), "query/key batch mismatch");
  TORCH_CHECK(query.size(1) == key.size(1), "query/key sequence mismatch");
  TORCH_CHECK(query.size(2) == key.size(2), "query/key head mismatch");
  TORCH_CHECK(query.size(3) == key.size(3), "query/key bit dimension mismatch");
  TORCH_CHECK(query.size(0) == value.size(0), "query/value batch mismatch");
  TORCH_CHECK(query.size(1) == value.size(1), "query/value sequence mismatch");
  TORCH_CHECK(query.size(2) % value.size(2) == 0, "query heads must be divisible by value heads");
  TORCH_CHECK(query.size(3) > 0 && query.size(3) <= 32,
              "query/key bit dimension must be in [1, 32]");
  TORCH_CHECK(query.numel() / query.size(3) <= std::numeric_limits<int>::max(),
              "B * T * H must fit in int32");
  TORCH_CHECK(query.size(1) <= std::numeric_limits<int>::max() - kKernelIndexSafetyMargin,
              "sequence length is too large for the CUDA kernel index stride");
  TORCH_CHECK(value.size(3) <= std::numeric_limits<int>::max() - kKernelIndexSafetyMargin,
              "value dimension is too large for the CUDA kernel index stride");
  TORCH_CHECK(max_suffix_length >= 1, "max_suffix_length must be >= 1");
}

void check_varlen_inputs(const Tensor& query, const Tensor& key, const Tensor& value,
                         const Tensor& cu_seqlens, int64_t max_suffix_length) {
  TORCH_CHECK(query.is_cuda(), "query must be a CUDA tensor");
  TORCH_CHECK(key.is_cuda(), "key must be a CUDA tensor");
  TORCH_CHECK(value.is_cuda(), "value must be a CUDA tensor");
  TORCH_CHECK(cu_seqlens.is_cuda(), "cu_seqlens must be a CUDA tensor");
  TORCH_CHECK(query.device() == key.device() && query.device() == value.device() &&
                  query.device() == cu_seqlens.device(),
              "all inputs and cu_seqlens must be on the same CUDA device");
  TORCH_CHECK(is_supported_logit_dtype(query.scalar_type()),
              "query must be float32, float16, or bfloat16");
  TORCH_CHECK(query.scalar_type() == key.scalar_type(), "query/key dtype mismatch");
  TORCH_CHECK(query.scalar_type() == value.scalar_type(), "query/value dtype mismatch");
  TORCH_CHECK(query.dim() == 3, "query must have shape (N, H, D)");
  TORCH_CHECK(key.dim() == 3, "key must have shape (N, H, D)");
  TORCH_CHECK(value.dim() == 3, "value must have shape (N, H_p, D_p)");
  TORCH_CHECK(query.size(0) > 0, "packed token count must be positive");
  TORCH_CHECK(query.size(1) > 0, "query head count must be positive");
  TORCH_CHECK(value.size(1) > 0, "value head count must be positive");
  TORCH_CHECK(value.size(2) > 0, "value dimension must be positive");
  TORCH_CHECK(query.size(0) == key.size(0), "query/key token mismatch");
  TORCH_CHECK(query.size(0) == value.size(0), "query/value token mismatch");
  TORCH_CHECK(query.size(1) == key.size(1), "query/key head mismatch");
  TORCH_CHECK(query.size(2) == key.size(2), "query/key bit dimension mismatch");
  TORCH_CHECK(query.size(1) % value.size(1) == 0, "query heads must be divisible by value heads");
  TORCH_CHECK(query.size(2) > 0 && query.size(2) <= 32,
              "query/key bit dimension must be in [1, 32]");
  TORCH_CHECK(query.size(0) * query.size(1) <= std::numeric_limits<int>::max(),
              "N * H must fit in int32");
  TORCH_CHECK(query.size(0) <= std::numeric_limits<int>::max() - kKernelIndexSafetyMargin,
              "packed token count is too large for CUDA kernel indexing");
  TORCH_CHECK(value.size(2) <= std::numeric_limits<int>::max() - kKernelIndexSafetyMargin,
              "value dimension is too large for the CUDA kernel index stride");
  TORCH_CHECK(cu_seqlens.scalar_type() == torch::kInt32, "cu_seqlens must be int32");
  TORCH_CHECK(cu_seqlens.dim() == 1 && cu_seqlens.numel() >= 2,
              "cu_seqlens must be one-dimensional with at least two entries");
  TORCH_CHECK(cu_seqlens.numel() - 1 <= std::numeric_limits<int>::max() - kKernelIndexSafetyMargin,
              "number of packed sequences is too large for CUDA indexing");
  TORCH_CHECK(max_suffix_length >= 1, "max_suffix_length must be >= 1");
}

void check_packed_symbols(const Tensor& packed, const Tensor& query, const char* name) {
  TORCH_CHECK(packed.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(packed.device() == query.device(), name,
              " must be on the same CUDA device as query");
  TORCH_CHECK(packed.scalar_type() == torch::kInt32, name, " must be int32");
  if (query.dim() == 4) {
    TORCH_CHECK(packed.dim() == 3, name, " must have shape (B, H, T)");
    TORCH_CHECK(packed.size(0) == query.size(0), name, " batch mismatch");
    TORCH_CHECK(packed.size(1) == query.size(2), name, " head mismatch");
    TORCH_CHECK(packed.size(2) == query.size(1), name, " sequence mismatch");
  } else {
    TORCH_CHECK(packed.dim() == 2, name, " must have shape (H, N)");
    TORCH_CHECK(packed.size(0) == query.size(1) && packed.size(1) == query.size(0), name,
                " shape mismatch");
  }
}

void check_dropout_seed(const Tensor& seed, const Tensor& query, double dropout_p) {
  TORCH_CHECK(seed.is_cuda(), "dropout_seed must be a CUDA tensor");
  TORCH_CHECK(seed.device() == query.device(),
              "dropout_seed must be on the same CUDA device as query");
  TORCH_CHECK(seed.scalar_type() == torch::kInt64, "dropout_seed must have dtype int64");
  TORCH_CHECK(seed.numel() == (dropout_p > 0.0 ? 1 : 0),
              "dropout_seed must be scalar exactly when dropout_p > 0");
}

void check_gradient_mask(int64_t gradient_mask) {
  TORCH_CHECK(gradient_mask >= 1 && gradient_mask <= 7,
              "gradient_mask must be an integer bit mask in [1, 7]");
}

Tensor make_workspace(const Tensor& like, size_t bytes) {
  return torch::empty({static_cast<int64_t>(bytes)}, like.options().dtype(torch::kUInt8));
}

// shared forward driver: `cu` undefined means dense
Triple run_hard_forward(const Tensor& query, const Tensor& key, const Tensor& value,
                        const Tensor& cu, int64_t max_suffix_length) {
  const bool dense = !cu.defined();
  const c10::cuda::CUDAGuard guard(query.device());
  const Tensor q = query.contiguous(), k = key.contiguous(), v = value.contiguous();
  const Tensor cuc = dense ? cu : cu.contiguous();
  const int64_t N = dense ? q.size(0) * q.size(1) : q.size(0);
  const int hd = dense ? 2 : 1;
  const int64_t H = q.size(hd), D = q.size(hd + 1), Hv = v.size(hd), Dv = v.size(hd + 1);
  const int64_t S = dense ? q.size(0) : cuc.numel() - 1;
  const int64_t T = dense ? q.size(1) : 0;
  std::vector<int64_t> out_shape = q.sizes().vec();
  out_shape.back() = Dv;
  Tensor out = torch::empty(out_shape, q.options());
  Tensor pq = dense ? torch::empty({q.size(0), H, T}, q.options().dtype(torch::kInt32))
                    : torch::empty({H, N}, q.options().dtype(torch::kInt32));
  Tensor pk = torch::empty_like(pq);
  const size_t bytes = rosa_b200_hard_forward_workspace_bytes(N, (int)H, S);
  Tensor ws = make_workspace(q, bytes);
  check_rc(rosa_b200_hard_forward(
               q.data_ptr(), k.data_ptr(), v.data_ptr(), dtype_code(q.scalar_type()), N, (int)H,
               (int)D, (int)Hv, (int)Dv, dense ? nullptr : cuc.data_ptr<int32_t>(), S, T,
               max_suffix_length, out.data_ptr(), pq.data_ptr<int32_t>(), pk.data_ptr<int32_t>(),
               nullptr, ws.data_ptr(), bytes, at::cuda::getCurrentCUDAStream().stream()),
           "hard_forward");
  return {out, pq, pk};
}

Triple run_surrogate_vjp(const Tensor& query, const Tensor& key, const Tensor& value,
                         const Tensor& cu, const Tensor& grad_output, const Tensor& packed_q,
                         const Tensor& packed_k, const Tensor& seed, int64_t effective_w,
                         const SurrogateScalars& sc, int64_t mask) {
  const bool dense = !cu.defined();
  const c10::cuda::CUDAGuard guard(query.device());
  const Tensor q = query.contiguous(), k = key.contiguous(), v = value.contiguous();
  const Tensor go = grad_output.contiguous();
  const Tensor pq = packed_q.contiguous(), pk = packed_k.contiguous();
  const Tensor sd = seed.contiguous();
  const Tensor cuc = dense ? cu : cu.contiguous();
  const int64_t N = dense ? q.size(0) * q.size(1) : q.size(0);
  const int hd = dense ? 2 : 1;
  const int64_t H = q.size(hd), D = q.size(hd + 1), Hv = v.size(hd), Dv = v.size(hd + 1);
  const int64_t S = dense ? q.size(0) : cuc.numel() - 1;
  const int64_t T = dense ? q.size(1) : 0;
  const auto f32 = q.options().dtype(torch::kFloat32);
  Tensor dq = (mask & 1) ? torch::empty(q.sizes(), f32) : torch::empty({0}, f32);
  Tensor dk = (mask & 2) ? torch::empty(k.sizes(), f32) : torch::empty({0}, f32);
  Tensor dv = (mask & 4) ? torch::empty(v.sizes(), f32) : torch::empty({0}, f32);
  const size_t bytes = rosa_b200_surrogate_vjp_workspace_bytes(N, (int)H, (int)D, (int)Hv, (int)Dv,
                                                               S, T, effective_w, (int)mask);
  Tensor ws = make_workspace(q, bytes);
  check_rc(rosa_b200_surrogate_vjp(
               q.data_ptr(), k.data_ptr(), v.data_ptr(), go.data_ptr(), dtype_code(q.scalar_type()),
               N, (int)H, (int)D, (int)Hv, (int)Dv, dense ? nullptr : cuc.data_ptr<int32_t>(), S, T,
               effective_w, pq.data_ptr<int32_t>(), pk.data_ptr<int32_t>(),
               sc.dropout_p > 0.0f ? sd.data_ptr<int64_t>() : nullptr, sc.scale, sc.dropout_p,
               sc.mismatch_scale, (int)mask, 0, 0, (mask & 1) ? dq.data_ptr<float>() : nullptr,
               (mask & 2) ? dk.data_ptr<float>() : nullptr,
               (mask & 4) ? dv.data_ptr<float>() : nullptr, ws.data_ptr(), bytes,
               at::cuda::getCurrentCUDAStream().stream()),
           "surrogate_vjp");
  return {dq, dk, dv};
}

Triple hard_forward_op(Tensor query, Tensor key, Tensor value, int64_t max_suffix_length) {
  check_common_inputs(query, key, value, max_suffix_length);
  const int64_t w = std::min<int64_t>(max_suffix_length, query.size(1));
  return run_hard_forward(query, key, value, Tensor(), w);
}

Triple hard_forward_varlen_op(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens,
                              int64_t max_suffix_length) {
  check_varlen_inputs(query, key, value, cu_seqlens, max_suffix_length);
  const int64_t w = std::min<int64_t>(max_suffix_length, query.size(0));
  return run_hard_forward(query, key, value, cu_seqlens, w);
}

Triple surrogate_vjp_masked_op(Tensor query, Tensor key, Tensor value, Tensor grad_output,
                               Tensor packed_query_symbols, Tensor packed_key_symbols,
                               Tensor dropout_seed, int64_t max_suffix_length, double scale,
                               double dropout_p, double mismatch_scale, int64_t gradient_mask) {
  check_common_inputs(query, key, value, max_suffix_length);
  TORCH_CHECK(grad_output.is_cuda(), "grad_output must be a CUDA tensor");
  TORCH_CHECK(grad_output.device() == query.device(),
              "grad_output must be on the same CUDA device as query");
  TORCH_CHECK(grad_output.scalar_type() == query.scalar_type(), "grad_output dtype mismatch");
  TORCH_CHECK(grad_output.sizes() == torch::IntArrayRef({query.size(0), query.size(1),
                                                         query.size(2), value.size(3)}),
              "grad_output shape mismatch");
  check_packed_symbols(packed_query_symbols, query, "packed_query_symbols");
  check_packed_symbols(packed_key_symbols, query, "packed_key_symbols");
  const int64_t w = std::min<int64_t>(max_suffix_length, query.size(1));
  const auto sc = check_surrogate_scalars(w, scale, dropout_p, mismatch_scale);
  check_dropout_seed(dropout_seed, query, dropout_p);
  check_gradient_mask(gradient_mask);
  return run_surrogate_vjp(query, key, value, Tensor(), grad_output, packed_query_symbols,
                           packed_key_symbols, dropout_seed, w, sc, gradient_mask);
}

Triple surrogate_vjp_varlen_masked_op(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens,
                                      Tensor grad_output, Tensor packed_query_symbols,
                                      Tensor packed_key_symbols, Tensor dropout_seed,
                                      int64_t max_suffix_length, double scale, double dropout_p,
                                      double mismatch_scale, int64_t gradient_mask) {
  check_varlen_inputs(query, key, value, cu_seqlens, max_suffix_length);
  TORCH_CHECK(grad_output.is_cuda(), "grad_output must be a CUDA tensor");
  TORCH_CHECK(grad_output.device() == query.device(),
              "grad_output must be on the same CUDA device as query");
  TORCH_CHECK(grad_output.scalar_type() == query.scalar_type(), "grad_output dtype mismatch");
  TORCH_CHECK(grad_output.sizes() ==
                  torch::IntArrayRef({query.size(0), query.size(1), value.size(2)}),
              "grad_output shape mismatch");
  check_packed_symbols(packed_query_symbols, query, "packed_query_symbols");
  check_packed_symbols(packed_key_symbols, query, "packed_key_symbols");
  const int64_t w = std::min<int64_t>(max_suffix_length, query.size(0));
  const auto sc = check_surrogate_scalars(w, scale, dropout_p, mismatch_scale);
  check_dropout_seed(dropout_seed, query, dropout_p);
  check_gradient_mask(gradient_mask);
  return run_surrogate_vjp(query, key, value, cu_seqlens, grad_output, packed_query_symbols,
                           packed_key_symbols, dropout_seed, w, sc, gradient_mask);
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
  return {out, matched};
}

}  // namespace

#ifdef ROSA_WITH_CUDA
TORCH_LIBRARY(rosa_soft, m) {
  m.def("hard_forward(Tensor query, Tensor key, Tensor value, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)");
  m.def("hard_forward_varlen(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, int max_suffix_length) -> (Tensor output, Tensor packed_query_symbols, Tensor packed_key_symbols)");
  m.def("surrogate_vjp_masked(Tensor query, Tensor key, Tensor value, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("surrogate_vjp_varlen_masked(Tensor query, Tensor key, Tensor value, Tensor cu_seqlens, Tensor grad_output, Tensor packed_query_symbols, Tensor packed_key_symbols, Tensor dropout_seed, int max_suffix_length, float scale, float dropout_p, float mismatch_scale, int gradient_mask) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("hard_inference(Tensor query_symbols, Tensor key_symbols, Tensor payload, Tensor? cu_seqlens, int max_suffix_length) -> (Tensor output, Tensor matched_key_end_positions)");
}

TORCH_LIBRARY_IMPL(rosa_soft, CUDA, m) {
  m.impl("hard_forward", &hard_forward_op);
  m.impl("hard_forward_varlen", &hard_forward_varlen_op);
  m.impl("surrogate_vjp_masked", &surrogate_vjp_masked_op);
  m.impl("surrogate_vjp_varlen_masked", &surrogate_vjp_varlen_masked_op);
  m.impl("hard_inference", &hard_inference_op);
}
#endif
