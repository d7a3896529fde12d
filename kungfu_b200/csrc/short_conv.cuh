// A short causal convolution over time, per channel:  y_t[c] = sum_j w[c][j] * u_{t - taps + 1 + j}[c],  j = 0..taps-1,
// with zeros before the first token of a sequence.  The last column of w multiplies the current token.
//
// A step brings only some tokens of a request, so the last taps-1 inputs of every live request are kept as state,
// in order of time: state[slot][s][c] is the input at sequence index (length - (taps-1) + s).  Freshly admitted
// requests have an all-zero state, which is exactly "zeros before the start".
//
// The inputs of a step are columns col0..col0+C of a 32-bit matrix with `ld` columns (the result of a projection),
// to which an optional per-channel bias is added: the state holds the biased values.
#pragma once
#include "common.cuh"

constexpr int KF_MAX_TAPS = 8;

struct KfConvIn {
  const float* in;          // [rows, ld], 32-bit
  int ld, col0;             // the convolution's channels are columns col0 .. col0 + C - 1
  const void* in_bias;      // [C] or null; element type TW
  const float* state;       // [max_requests, taps - 1, C]
  int C, taps;
};

// The input of channel c at local index i among the request's rows of this step (rows row0, row0 + 1, ...);
// a negative index reaches into the state of the request's slot.
template <typename TW>
__device__ __forceinline__ float kf_conv_input(const KfConvIn& p, int row0, int slot, int i, int c) {
  if (i >= 0) {
    float v = p.in[(size_t)(row0 + i) * p.ld + p.col0 + c];
    if (p.in_bias) v += kf_load((const TW*)p.in_bias, c);
    return v;
  }
  return p.state[((size_t)slot * (p.taps - 1) + (p.taps - 1 + i)) * p.C + c];
}

// y of channel c at local index i; the sum runs from the oldest tap to the newest.
template <typename TW>
__device__ __forceinline__ float kf_conv_value(const KfConvIn& p, const TW* __restrict__ w, int row0, int slot, int i, int c) {
  float acc = 0.f;
  for (int j = 0; j < p.taps; ++j)
    acc = fmaf(kf_load(w, (size_t)c * p.taps + j), kf_conv_input<TW>(p, row0, slot, i - (p.taps - 1 - j), c), acc);
  return acc;
}
