// Hard forward for hosts that cannot provide a workspace.
//
// rosa_b200_hard_forward needs a scratch buffer that the caller allocates.  Some callers
// have no way to do that: a serving process that handed all device memory to its own arena
// at start-up and must not touch the CUDA allocator from its request loop (cudaMalloc
// synchronises the device and can fail under fragmentation), or a small embedding host
// that links this library without any device-memory manager of its own.  For them this
// file offers the same operation with the scratch placed in a fixed array that lives in
// the library's device image.  Inputs and outputs are still the caller's buffers.
//
// The array is one per GPU and shared by every call on that GPU.  It keeps whatever the
// previous call left in it, so each call re-initialises the parts that must start at zero
// (the per-row winner table) on the caller's stream before use.  Two calls that overlap
// on the same GPU (different streams or threads without ordering between them) would write
// the same scratch and race; callers must order them.
#include <mutex>

#include "common.cuh"

namespace {

// Limits of the static variant.  8 MiB of winners + 128 KiB of plan tables per GPU.
constexpr int64_t kStaticMaxTokenHeads = 1 << 20;  // N * H
constexpr int64_t kStaticMaxSequences = 4096;
constexpr size_t kStaticPlanBytes = 128 << 10;
constexpr size_t kStaticScratchBytes =
    kStaticPlanBytes + (size_t)kStaticMaxTokenHeads * sizeof(unsigned long long);

// In host code this name is only a handle for the runtime; the device address is obtained
// with cudaGetSymbolAddress below and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};

}  // namespace

namespace rosa {
// Once per device, with that device current: resolve the device address of the array.
// (Also used by rosa_b200_read_status to find the status words of the last static call.)
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  ROSA_CUDA_OK(cudaGetDevice(&dev));
  ROSA_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d is not supported", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    ROSA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_scratch));
    ROSA_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}
}  // namespace rosa

extern "C" ROSA_B200_API int rosa_b200_hard_forward_static(
    const void* query, const void* key, const void* value, int dtype, int64_t N, int H, int D,
    int Hv, int Dv, const int32_t* cu_seqlens, int64_t num_seq, int64_t uniform_len,
    int64_t max_suffix_length, void* output, int32_t* packed_query, int32_t* packed_key,
    int32_t* route_token, void* stream) {
  using namespace rosa;
  ROSA_REQUIRE(dtype >= ROSA_B200_F32 && dtype <= ROSA_B200_BF16,
               "dtype must be float32, float16 or bfloat16");
  ROSA_REQUIRE(N > 0 && H > 0 && Hv > 0 && Dv > 0, "N, H, Hv and Dv must be positive");
  ROSA_REQUIRE(D >= 1 && D <= 32, "query/key bit dimension must be in [1, 32]");
  ROSA_REQUIRE(H % Hv == 0, "query heads must be divisible by value heads");
  ROSA_REQUIRE(H <= 65535, "head count exceeds the CUDA grid limit");
  ROSA_REQUIRE(num_seq >= 1, "at least one sequence is required");
  ROSA_REQUIRE(max_suffix_length >= 1, "max_suffix_length must be >= 1");
  ROSA_REQUIRE(query && key && value && output && packed_query && packed_key,
               "null pointer argument");
  const bool dense = cu_seqlens == nullptr;
  if (dense)
    ROSA_REQUIRE(uniform_len >= 1 && num_seq * uniform_len == N,
                 "dense description needs num_seq * uniform_len == N");
  ROSA_REQUIRE(N * (int64_t)H <= kStaticMaxTokenHeads,
               "the static-scratch variant handles at most %lld token-heads (N * H), got %lld; "
               "use rosa_b200_hard_forward with a caller-provided workspace",
               (long long)kStaticMaxTokenHeads, (long long)(N * (int64_t)H));
  ROSA_REQUIRE(num_seq <= kStaticMaxSequences,
               "the static-scratch variant handles at most %lld sequences, got %lld; "
               "use rosa_b200_hard_forward with a caller-provided workspace",
               (long long)kStaticMaxSequences, (long long)num_seq);
  const PlanLayout pl = plan_layout(0, num_seq);
  ROSA_REQUIRE(pl.bytes <= kStaticPlanBytes, "internal: plan tables exceed the static area");

  void* scratch = nullptr;
  if (int rc = static_scratch_for_current_device(&scratch)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(scratch);

  FwdArgs a{};
  a.plan = make_plan(scratch, pl, cu_seqlens, N, num_seq, uniform_len, kFwdBand);
  a.q = query; a.k = key; a.v = value; a.dtype = dtype;
  a.N = N; a.H = H; a.D = D; a.Hv = Hv; a.Dv = Dv;
  const int64_t bound = dense ? uniform_len : N;
  a.W = (int)(max_suffix_length < bound ? max_suffix_length : bound);
  a.out = output; a.packed_q = packed_query; a.packed_k = packed_key;
  a.route_token = route_token;
  a.best = reinterpret_cast<unsigned long long*>(base + kStaticPlanBytes);
  a.sym_seq_stride = dense ? (int64_t)H * uniform_len : 0;
  a.sym_head_stride = dense ? uniform_len : N;
  const int64_t items =
      dense ? num_seq * (uniform_len >= 2 ? (uniform_len - 1 + kFwdBand - 1) / kFwdBand : 0)
            : N / kFwdBand + num_seq;

  launch_build_plan(a.plan, st);
  ROSA_CUDA_OK(cudaGetLastError());
  // the winner table still holds the previous call's results: start every row from "no match"
  ROSA_CUDA_OK(cudaMemsetAsync(a.best, 0, (size_t)N * H * sizeof(unsigned long long), st));
  if (int rc = launch_pack_symbols(query, key, dtype, N, H, D, dense, uniform_len, packed_query,
                                   packed_key, st))
    return rc;
  if (int rc = launch_hard_match(a, (int)items, st)) return rc;
  return launch_gather_output(a, st);
}
