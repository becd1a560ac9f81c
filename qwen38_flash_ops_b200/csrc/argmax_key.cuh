// The (value, index) order of ArgmaxRows as one 64-bit word: NaN beats every number, then the larger value
// (-0 == +0), then the lower index.  The unsigned maximum of such words is the winner, so a reduction needs
// no comparison function: redux.sync.max on the halves inside a warp, atomicMax across warps and CTAs.
// 0 means "no candidate"; every real candidate maps above it.
#pragma once

#include <cstdint>

namespace qfg {

__device__ __forceinline__ unsigned long long PackKey(float v, long long idx) {
  uint32_t ord;
  if (v != v) {
    ord = 0xFFFFFFFFu;
  } else {
    const uint32_t b = (v == 0.f) ? 0u : __float_as_uint(v);
    ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
  return (static_cast<unsigned long long>(ord) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(idx));
}
__device__ __forceinline__ long long KeyIndex(unsigned long long key) {
  return static_cast<long long>(0xFFFFFFFFu - static_cast<uint32_t>(key));
}
// the winning value; a NaN comes back as the canonical quiet NaN
__device__ __forceinline__ float KeyValue(unsigned long long key) {
  const uint32_t ord = static_cast<uint32_t>(key >> 32);
  const uint32_t bits = (ord == 0xFFFFFFFFu) ? 0x7FC00000u : ((ord & 0x80000000u) ? (ord & 0x7FFFFFFFu) : ~ord);
  return __uint_as_float(bits);
}
// maximum of a key over the warp: the maximum of the upper halves, then of the lower halves among the lanes
// that hold that upper half
__device__ __forceinline__ unsigned long long WarpMaxKey(unsigned long long key) {
  const uint32_t hi = static_cast<uint32_t>(key >> 32);
  const uint32_t top = __reduce_max_sync(0xffffffffu, hi);
  const uint32_t low = __reduce_max_sync(0xffffffffu, hi == top ? static_cast<uint32_t>(key) : 0u);
  return (static_cast<unsigned long long>(top) << 32) | low;
}

}  // namespace qfg
