// Compare-exchange networks over 32 values held in registers (every index is a compile-time
// constant after unrolling): the W largest of 32 unsigned keys, in descending order.
//
//   1. bitonic sort inside groups of W values, even groups descending, odd groups ascending;
//   2. halving rounds: a descending group and its ascending neighbour are combined by taking
//      the element-wise maximum (a bitonic sequence that holds the W largest of the 2 W values)
//      which is then merged into a sorted group again, descending or ascending so that the next
//      round finds the same arrangement.
// Cost in compare-exchanges: W = 8: 156, W = 16: 208, W = 32: 240 (a full sort).
#pragma once

#include <stdint.h>

namespace moba {
namespace topk {

#if defined(__CUDACC__)
#define MOBA_TOPK_FN __host__ __device__ __forceinline__
#else
#define MOBA_TOPK_FN inline
#endif

// after the call: hi = max, lo = min
MOBA_TOPK_FN void ce(uint32_t& hi, uint32_t& lo) {
#if defined(__CUDA_ARCH__)
  const uint32_t a = max(hi, lo), b = min(hi, lo);       // two integer min/max instructions
#else
  const uint32_t a = hi > lo ? hi : lo, b = hi > lo ? lo : hi;
#endif
  hi = a;
  lo = b;
}

// Bitonic merge of the bitonic sequence v[base, base + W) into descending (kDesc) or ascending order.
template <int W, bool kDesc>
MOBA_TOPK_FN void bitonic_merge(uint32_t (&v)[32], int base) {
#pragma unroll
  for (int j = W / 2; j > 0; j >>= 1)
#pragma unroll
    for (int i = 0; i < W; ++i)
      if ((i & j) == 0) {
        if (kDesc) ce(v[base + i], v[base + i + j]);
        else ce(v[base + i + j], v[base + i]);
      }
}

// Sorts v[base, base + W) (any order) descending or ascending.
template <int W, bool kDesc>
MOBA_TOPK_FN void bitonic_sort(uint32_t (&v)[32], int base) {
  if constexpr (W > 1) {
    bitonic_sort<W / 2, true>(v, base);
    bitonic_sort<W / 2, false>(v, base + W / 2);
    bitonic_merge<W, kDesc>(v, base);
  }
}

// The W largest of the 32 keys end up in v[0, W), largest first; the rest of v is unspecified.
template <int W>
MOBA_TOPK_FN void top_of_32(uint32_t (&v)[32]) {
  static_assert(W == 8 || W == 16 || W == 32, "W is 8, 16 or 32");
  if constexpr (W == 32) {
    bitonic_sort<32, true>(v, 0);
  } else {
    // groups g = 0, 1, ...: even ones descending, odd ones ascending
#pragma unroll
    for (int g = 0; g < 32 / W; ++g) {
      if (g % 2 == 0) bitonic_sort<W, true>(v, g * W);
      else bitonic_sort<W, false>(v, g * W);
    }
    // halving rounds over the group pairs (0,1), (2,3), ...: the result of pair k goes to group k
#pragma unroll
    for (int groups = 32 / W; groups > 1; groups /= 2) {
#pragma unroll
      for (int k = 0; k < groups / 2; ++k) {
        const int a = 2 * k * W, b = (2 * k + 1) * W, dst = k * W;
#pragma unroll
        for (int i = 0; i < W; ++i) {
          const uint32_t x = v[a + i], y = v[b + i];
#if defined(__CUDA_ARCH__)
          v[dst + i] = max(x, y);
#else
          v[dst + i] = x > y ? x : y;
#endif
        }
        if (k % 2 == 0) bitonic_merge<W, true>(v, dst);
        else bitonic_merge<W, false>(v, dst);
      }
    }
  }
}

}  // namespace topk
}  // namespace moba
