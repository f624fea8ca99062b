// Addressing of the pooled-window cache [pages, bs + PS, Wc]: rows 0..bs-1 of a page hold its tokens, rows bs.. the
// pooled rows of the blocks of P tokens whose first token lies in the page (PS = ceil(bs / P)).  Shared by the kernels in
// pooled_window_attention.cu (append, pooling, FMA attention) and pooled_window_attention_mma.cu (tensor-core attention).
#pragma once
#include <limits.h>

#include "../common/util.cuh"

namespace llmctl {

// Row of the pooled entry of block b in the cache (in rows of Wc numbers).
__device__ __forceinline__ long long pooled_row(const int* __restrict__ table, int b, int P, int bs, int PS) {
  const long long first = static_cast<long long>(b) * P;
  const int page = static_cast<int>(first / bs);
  const int first_b = static_cast<int>((static_cast<long long>(page) * bs + P - 1) / P);   // first block starting in the page
  return static_cast<long long>(table[page]) * (bs + PS) + bs + (b - first_b);
}
__device__ __forceinline__ long long token_row(const int* __restrict__ table, int j, int bs, int PS) {
  return static_cast<long long>(table[j / bs]) * (bs + PS) + j % bs;
}


// Key u of a query tile's unified key list: pooled blocks 0..nb-1 first, then the tokens j0.. .  A key is seen by the
// query at position i iff lo <= i <= hi.
struct WindowKey {
  int lo, hi, row;
};
__device__ __forceinline__ WindowKey window_key(const int* __restrict__ table, int u, int nb, int j0, int NU, int S, int P, int bs, int PS) {
  WindowKey k{INT_MAX, INT_MIN, 0};                 // an empty range: padding keys are seen by nobody
  if (u < nb) {
    k.lo = u * P + P - 1 + S;
    k.hi = INT_MAX;
    k.row = static_cast<int>(pooled_row(table, u, P, bs, PS));
  } else if (u < NU) {
    const int j = j0 + (u - nb);
    k.lo = j;
    k.hi = S > 0 ? j + S - 1 : INT_MAX;
    k.row = static_cast<int>(token_row(table, j, bs, PS));
  }
  return k;
}

}  // namespace llmctl
