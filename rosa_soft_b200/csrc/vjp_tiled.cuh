// Helpers shared by the register-tiled sweeps of the surrogate VJP: the byte-spread form of the
// value sign bits and the nibble-table lookup of the route utility.
#pragma once

#include "common.cuh"

namespace rosa {
namespace {

// Value sign bits of one route, one nibble per byte and pre-multiplied by four: byte g of the
// result is the shared-memory word offset (times 4 bytes) of the utility-table entry of value
// group g, so a lookup is one byte extraction and one load.
__device__ __forceinline__ uint32_t spread_nibbles(uint32_t bits16) {
  uint32_t out = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) out |= ((bits16 >> (4 * g)) & 15u) << (8 * g + 2);
  return out;
}

template <int kByte>
__device__ __forceinline__ uint32_t byte_of(uint32_t w) {
  uint32_t r;
  asm("prmt.b32 %0, %1, 0, %2;" : "=r"(r) : "r"(w), "n"(0x4440 | kByte));
  return r;
}

// u = gO(i) . sign(V[a]) from the nibble tables of block row r (table base `lut`)
template <int NG>
__device__ __forceinline__ float tiled_utility(const float* lut, uint32_t v0, uint32_t v1) {
  const char* base = reinterpret_cast<const char*>(lut);
  float u = *reinterpret_cast<const float*>(base + byte_of<0>(v0));
  u += *reinterpret_cast<const float*>(base + 64 + byte_of<1>(v0));
  if (NG > 2) {
    u += *reinterpret_cast<const float*>(base + 128 + byte_of<2>(v0));
    u += *reinterpret_cast<const float*>(base + 192 + byte_of<3>(v0));
  }
  if (NG > 4) {
    u += *reinterpret_cast<const float*>(base + 256 + byte_of<0>(v1));
    u += *reinterpret_cast<const float*>(base + 320 + byte_of<1>(v1));
    u += *reinterpret_cast<const float*>(base + 384 + byte_of<2>(v1));
    u += *reinterpret_cast<const float*>(base + 448 + byte_of<3>(v1));
  }
  return u;
}

}  // namespace
}  // namespace rosa
