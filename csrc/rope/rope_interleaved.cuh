// Rotary embedding on interleaved pairs: coordinates (2i, 2i+1) of a vector form pair i, which is turned by the
// angle position * freq[i]; cos and sin are multiplied by `mult` (1 without frequency scaling; the YaRN
// attention factor otherwise).  The per-pair frequencies come from the host (ops/functional.py `rope_frequencies`),
// so plain, linear-interpolated and YaRN-blended spectra all use the same device code.  Angles are formed and
// evaluated in fp32 with the accurate sincosf.
#pragma once
#include "../common/dtype.cuh"

namespace llmctl {

// Rotated value of coordinate `d` (d < 2 * pairs) of the vector whose raw coordinates are read through `at(k)`.
template <typename Load>
__device__ __forceinline__ float rope_interleaved_coord(Load at, int d, int position, const float* __restrict__ freq, float mult) {
  const int i = d >> 1;
  float s, c;
  sincosf(static_cast<float>(position) * freq[i], &s, &c);
  s *= mult;
  c *= mult;
  const float u = at(2 * i), v = at(2 * i + 1);
  return (d & 1) ? (v * c + u * s) : (u * c - v * s);
}

}  // namespace llmctl
