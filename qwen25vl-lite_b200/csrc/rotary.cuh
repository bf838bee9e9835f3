// Rotary position encoding of part of a head: the first 2 * half channels are turned by the token's
// angles, the channels after them pass.  Two ways of pairing channels: ROTARY_INTERLEAVED pairs
// channel 2i with 2i + 1, ROTARY_HALVES pairs i with i + half.  The pair (u, v) becomes
// (u cos - v sin, v cos + u sin).  The angles come as a table [token][half][2] of (cos, sin), each
// already multiplied by the encoding's magnitude, float in both dtypes.
#pragma once
#include "common.cuh"

#define ROTARY_INTERLEAVED 0
#define ROTARY_HALVES 1

// Channel c of the head at x after rotation; ang: the token's (cos, sin) pairs, or nullptr for no rotation.
template <typename T>
__device__ __forceinline__ float rotary_channel(const T* __restrict__ x, int c, int half, int layout, const float* __restrict__ ang) {
  if (!ang || c >= 2 * half) return to_f32(x[c]);
  int i, iu, iv;
  bool second;
  if (layout == ROTARY_INTERLEAVED) { i = c >> 1; iu = 2 * i; iv = iu + 1; second = c & 1; }
  else { second = c >= half; i = second ? c - half : c; iu = i; iv = i + half; }
  const float u = to_f32(x[iu]), v = to_f32(x[iv]), cs = ang[2 * i], sn = ang[2 * i + 1];
  return second ? fmaf(v, cs, u * sn) : fmaf(u, cs, -v * sn);
}
