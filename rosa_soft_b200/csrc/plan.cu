// Device-side segment plan: turns cu_seqlens (or a dense batch description) into the
// work-item tables the compute kernels consume, and validates the offsets without
// trapping.  Replaces validate_varlen_offsets_kernel and the per-thread binary search
// over cu_seqlens of the reference (rosa_soft/csrc/cuda/rosa_soft_kernels.cu:269-308).
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace rosa {

namespace {

thread_local char g_error[512] = "";

constexpr int kPlanThreads = 1024;

__global__ void __launch_bounds__(kPlanThreads) build_plan_kernel(Plan plan) {
  __shared__ int s_status;
  __shared__ long long s_scan[3][kPlanThreads];
  const int tid = threadIdx.x;
  const int S = plan.S;
  if (tid == 0) s_status = ROSA_B200_STATUS_OK;
  __syncthreads();

  if (plan.cu_seqlens != nullptr) {
    for (int s = tid; s <= S; s += kPlanThreads) {
      const int cur = plan.cu_seqlens[s];
      if (s == 0 && cur != 0) atomicMax(&s_status, (int)ROSA_B200_STATUS_BAD_FIRST_OFFSET);
      if (s > 0 && cur < plan.cu_seqlens[s - 1])
        atomicMax(&s_status, (int)ROSA_B200_STATUS_NOT_MONOTONE);
      if (s == S && (int64_t)cur != plan.N)
        atomicMax(&s_status, (int)ROSA_B200_STATUS_BAD_LAST_OFFSET);
    }
  }
  __syncthreads();
  const int status = s_status;
  if (tid == 0) {
    plan.status[0] = status;
    if (!plan.keep_mma_status) plan.status[1] = 0;
    plan.status[2] = 0;
    plan.status[3] = 0;
  }

  // each thread owns a contiguous chunk of sequences
  const int chunk = (S + kPlanThreads - 1) / kPlanThreads;
  const int s0 = min(S, tid * chunk), s1 = min(S, s0 + chunk);
  long long items = 0, rows = 0, cks = 0;
  for (int s = s0; s < s1; ++s) {
    int start, len;
    if (status != 0) {
      start = 0;
      len = 0;
    } else if (plan.cu_seqlens != nullptr) {
      start = plan.cu_seqlens[s];
      len = plan.cu_seqlens[s + 1] - start;
    } else {
      start = s * plan.uniform_len;
      len = plan.uniform_len;
    }
    plan.seg_start[s] = start;
    plan.seg_len[s] = len;
    const long long it =
        len >= 2 ? (len - 1 + plan.item_diagonals - 1) / plan.item_diagonals : 0;
    items += it;
    rows += it * len;
    cks += vjp_ck_count(len);
  }
  s_scan[0][tid] = items;
  s_scan[1][tid] = rows;
  s_scan[2][tid] = cks;
  __syncthreads();
  // inclusive Hillis-Steele scan over the per-thread totals
  for (int off = 1; off < kPlanThreads; off <<= 1) {
    long long a = 0, b = 0, c = 0;
    if (tid >= off) {
      a = s_scan[0][tid - off];
      b = s_scan[1][tid - off];
      c = s_scan[2][tid - off];
    }
    __syncthreads();
    s_scan[0][tid] += a;
    s_scan[1][tid] += b;
    s_scan[2][tid] += c;
    __syncthreads();
  }
  long long pi = s_scan[0][tid] - items, pr = s_scan[1][tid] - rows, pc = s_scan[2][tid] - cks;
  for (int s = s0; s < s1; ++s) {
    plan.item_prefix[s] = (int32_t)pi;
    plan.row_prefix[s] = pr;
    plan.ck_prefix[s] = pc;
    const int len = plan.seg_len[s];
    const long long it =
        len >= 2 ? (len - 1 + plan.item_diagonals - 1) / plan.item_diagonals : 0;
    pi += it;
    pr += it * len;
    pc += vjp_ck_count(len);
  }
  if (tid == kPlanThreads - 1) {
    plan.item_prefix[S] = (int32_t)s_scan[0][tid];
    plan.row_prefix[S] = s_scan[1][tid];
    plan.ck_prefix[S] = s_scan[2][tid];
  }
}

}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

const char* get_error() { return g_error; }

void launch_build_plan(const Plan& plan, cudaStream_t stream) {
  ProfileScope prof("build_plan", stream);
  build_plan_kernel<<<1, kPlanThreads, 0, stream>>>(plan);
}

// ---------------------------------------------------------------- profiler state
namespace {
struct ProfileRecord {
  const char* name;
  cudaEvent_t start, stop;
};
std::mutex g_prof_mutex;
bool g_prof_enabled = false;
std::vector<ProfileRecord> g_prof_records;
}  // namespace

ProfileScope::ProfileScope(const char* name, cudaStream_t stream) : slot_(-1), stream_(stream) {
  if (!g_prof_enabled) return;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  ProfileRecord r;
  r.name = name;
  if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) return;
  cudaEventRecord(r.start, stream);
  slot_ = (int)g_prof_records.size();
  g_prof_records.push_back(r);
}

ProfileScope::~ProfileScope() {
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  cudaEventRecord(g_prof_records[slot_].stop, stream_);
}

void profile_enable(bool on) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_prof_enabled = on;
}

// Waits for the recorded events, sums the durations per kernel name, clears the records.
int profile_collect(const char** names, float* total_ms, int* launches, int capacity) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  int n = 0;
  for (auto& r : g_prof_records) {
    float ms = 0.0f;
    cudaEventSynchronize(r.stop);
    cudaEventElapsedTime(&ms, r.start, r.stop);
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
    int i = 0;
    for (; i < n; ++i)
      if (names[i] == r.name) break;
    if (i == n) {
      if (n == capacity) continue;
      names[n] = r.name;
      total_ms[n] = 0.0f;
      launches[n] = 0;
      ++n;
    }
    total_ms[i] += ms;
    launches[i] += 1;
  }
  g_prof_records.clear();
  return n;
}

}  // namespace rosa
