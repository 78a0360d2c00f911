// Nearest entry of a sorted 256-entry code book (the blockwise 8-bit optimizer-state codec).
//
// A binary search costs eight dependent shared-memory reads per value, at addresses that differ
// from thread to thread (bank conflicts); in the 8-bit AdamW update it was most of the kernel.
// Here the value's own bit pattern picks a bracket: sign, exponent and the top four mantissa bits
// select one of 386 bins per sign, a table gives the last code at or below the bin's smallest
// value, and a short forward scan (the codes inside one bin: three or four at most where the
// book is densest) finishes.  The result, including ties, is the one the binary search gives.
// The table is derived from the code book by each CTA when it starts (a few searches per
// thread), so callers pass nothing new.
#pragma once
#include <stdint.h>

namespace cbk {

constexpr int kBins = 386;          // per sign: |x| < 2^-24, then 24 exponents x 16, then |x| >= 1
constexpr int kTable = 2 * kBins;   // positive bins first, then negative

// Bin of x (|x| <= 1 expected; anything else, NaN included, lands in a valid bin).
__device__ __forceinline__ int bin_index(float x) {
  const uint32_t b = __float_as_uint(x);
  int k = static_cast<int>((b & 0x7fffffffu) >> 19) - (103 << 4);
  k = k < -1 ? -1 : (k > 384 ? 384 : k);
  return static_cast<int>(b >> 31) * kBins + k + 1;
}

// A lower bound of every value that falls into bin `e`.
__device__ __forceinline__ float bin_floor(int e) {
  const int sign = e >= kBins;
  const int kk = sign ? e - kBins : e;
  if (kk == 0) return sign ? -5.9604645e-08f /* -2^-24 */ : 0.f;
  const int k = kk - 1;
  if (k == 384) return sign ? -INFINITY : 1.f;
  const float lower = __uint_as_float(static_cast<uint32_t>(k + (103 << 4)) << 19);
  const float upper = __uint_as_float(static_cast<uint32_t>(k + 1 + (103 << 4)) << 19);
  return sign ? -upper : lower;
}

// Fills table[kTable] (shared memory) from cb[256] (shared memory, sorted ascending).  All threads
// of the CTA call it; the caller synchronises before and after.
__device__ __forceinline__ void build_table(const float* cb, uint8_t* table) {
  for (int e = threadIdx.x; e < kTable; e += blockDim.x) {
    const float L = bin_floor(e);
    int lo = 0, hi = 255;                    // last index with cb[index] <= L, or 0
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cb[mid] <= L) lo = mid; else hi = mid;
    }
    table[e] = static_cast<uint8_t>(lo);
  }
}

__device__ __forceinline__ int nearest_code(const float* cb, const uint8_t* table, float x) {
  int lo = table[bin_index(x)];
  while (lo < 254 && cb[lo + 1] <= x) ++lo;
  return (x - cb[lo] <= cb[lo + 1] - x) ? lo : lo + 1;
}

}  // namespace cbk
