// Pieces shared by the surrogate-VJP kernels: work-item geometry, the online-softmax merge,
// the transposing warp reduction and the flush-to-zero cutoff of the window product.
#pragma once

#include <math_constants.h>

#include "common.cuh"

namespace rosa {
namespace {

constexpr float kSqrtScale = 2.41421356237309504880f;  // sqrt(2) + 1

// ------------------------------------------------------------- item geometry
struct Item {
  int seq, it, h, start, len;
  int nitems;            // items of this sequence (per head)
  int w_begin, w_end;    // bands walked by this CTA
  int64_t rowslot;       // first partial-row slot of this (item, head)
  int64_t ck_base;       // first checkpoint block of this (sequence, head)
  int64_t item_linear;   // dense index over (sequence, head, item)
};

__device__ __forceinline__ void merge_stats(float& m, float& z, float& e, float m2, float z2,
                                            float e2) {
  if (m2 == -CUDART_INF_F) return;
  if (m == -CUDART_INF_F) {
    m = m2; z = z2; e = e2;
    return;
  }
  const float mm = fmaxf(m, m2);
  const float s1 = __expf(m - mm), s2 = __expf(m2 - mm);
  z = z * s1 + z2 * s2;
  e = e * s1 + e2 * s2;
  m = mm;
}

// Sum of eight per-lane values across a warp in 9 shuffles instead of 40: each step
// exchanges half of the remaining values with the partner lane.  On return every lane
// holds the warp total of value index ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 +
// ((lane >> 2) & 1).
__device__ __forceinline__ float warp_reduce8(const float (&v)[8], int lane) {
  const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
  float a[4], b[2];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = h16 ? v[i] : v[i + 4];
    const float keep = h16 ? v[i + 4] : v[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = h8 ? a[i] : a[i + 2];
    const float keep = h8 ? a[i + 2] : a[i];
    b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
  float c = (h4 ? b[1] : b[0]) + __shfl_xor_sync(0xffffffffu, h4 ? b[0] : b[1], 4);
  c += __shfl_xor_sync(0xffffffffu, c, 2);
  c += __shfl_xor_sync(0xffffffffu, c, 1);
  return c;
}

// Largest mismatch-count sum whose window product exp(-m * hs / D) is not flushed to zero
// (the kernels are compiled with flush-to-zero: exp(x) == 0 for x <= -88).
__device__ __forceinline__ int window_sum_cutoff(float neg_md) {
  if (!(neg_md < 0.0f)) return 1000000000;
  const float lim = -88.0f / neg_md;
  return lim < 1.0e9f ? (int)lim : 1000000000;
}

// Work item of a 1-D grid.  Heads vary fastest; for a dense batch the sequences vary next and
// the item index slowest, so that the longest items (the bands next to the main diagonal) of ALL
// sequences and heads are scheduled first and the tail of the launch consists of the shortest
// ones (with the sequence slowest, the long items of the last sequences would start late and
// finish alone).  Packed batches keep sequence-major order.
__device__ __forceinline__ bool load_item_1d(const VjpArgs& a, Item* o) {
  const int slot = blockIdx.x / a.H;
  if (a.plan.cu_seqlens == nullptr) {
    if (a.plan.status[0] != 0) return false;
    const int per = a.plan.item_prefix[1];          // items of every sequence
    if (per <= 0 || slot >= per * a.plan.S) return false;
    o->it = slot / a.plan.S;
    o->seq = slot - o->it * a.plan.S;
  } else if (!find_item(a.plan, slot, &o->seq, &o->it)) {
    return false;
  }
  o->h = blockIdx.x - slot * a.H;
  o->start = a.plan.seg_start[o->seq];
  o->len = a.plan.seg_len[o->seq];
  o->nitems = a.plan.item_prefix[o->seq + 1] - a.plan.item_prefix[o->seq];
  const int nbands = (int)vjp_bands(o->len);
  o->w_begin = o->it * a.bands_per_item;
  o->w_end = min(nbands, o->w_begin + a.bands_per_item);
  o->rowslot = a.plan.row_prefix[o->seq] * a.H +
               ((int64_t)o->h * o->nitems + o->it) * (int64_t)o->len;
  o->ck_base = a.plan.ck_prefix[o->seq] * a.H + (int64_t)o->h * vjp_ck_count(o->len);
  o->item_linear = (int64_t)a.plan.item_prefix[o->seq] * a.H + (int64_t)o->h * o->nitems + o->it;
  return true;
}

}  // namespace

// Adds four accumulator values to a partial gradient row that this CTA alone writes: the first
// touch stores, later ones go out as one vector reduction to L2 instead of a load, four adds and
// a store, so no thread waits for the old value.  The touches of one address come from different
// threads of the CTA in different row blocks, always with a CTA barrier in between, which orders
// them; the sum is therefore still formed in a fixed order.  (The reduction unit flushes
// subnormal float32 values to zero.)
__device__ __forceinline__ void accumulate_row4(float4* p, bool first, float a, float b, float c,
                                                float d) {
  if (first) {
    *p = make_float4(a, b, c, d);
  } else {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
                 "f"(d)
                 : "memory");
  }
}

// One component of such a row (rows whose width is not a multiple of four).
__device__ __forceinline__ void accumulate_row1(float* p, bool first, float a) {
  if (first) {
    *p = a;
  } else {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory");
  }
}

}  // namespace rosa
