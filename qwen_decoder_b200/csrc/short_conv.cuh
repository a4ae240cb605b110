// A short causal convolution over time on each channel, for a flat batch of portions of several requests:
//   y[t, c] = sum_j w[c, j] * in(t - taps + 1 + j, c),  j = 0 .. taps - 1
// in(s, c) is the step's own input row s while s lies inside the request's portion, else the request's kept input
// (the last taps - 1 inputs before the portion, oldest first, float32 [taps - 1, C]); a fresh state is zero, which
// stands for the zeros before a sequence's start.  float32 arithmetic, a fixed order of additions per element.
#pragma once
#include "common.cuh"

template <typename TI>
__device__ __forceinline__ float short_conv_at(const TI* __restrict__ u, long long ldu, int C, int taps,
                                               const float* __restrict__ w, const float* __restrict__ kept,
                                               int first_row, int t, int c) {
  float y = 0.f;
  const int li = t - first_row;                       // the token's place in its request's portion
  for (int j = 0; j < taps; j++) {
    const int s = li - (taps - 1) + j;
    const float v = s >= 0 ? to_float(u[(size_t)(first_row + s) * ldu + c])
                           : kept[(size_t)(taps - 1 + s) * C + c];
    y = fmaf(w[(size_t)c * taps + j], v, y);
  }
  return y;
}

// Moves channel c of a request's kept inputs on by the portion [first_row, end_row): afterwards they are the last
// taps - 1 inputs of the sequence again.  In place: entry k takes the old entry k + n, which has not been
// overwritten yet, or an input of the portion.
template <typename TI>
__device__ __forceinline__ void short_conv_advance(const TI* __restrict__ u, long long ldu, int C, int taps,
                                                   float* __restrict__ kept, int first_row, int end_row, int c) {
  const int n = end_row - first_row;
  for (int k = 0; k < taps - 1; k++) {
    const int s = n - (taps - 1) + k;                 // place in the portion of what entry k holds afterwards
    kept[(size_t)k * C + c] = s >= 0 ? to_float(u[(size_t)(first_row + s) * ldu + c]) : kept[(size_t)(k + n) * C + c];
  }
}
