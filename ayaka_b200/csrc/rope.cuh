// Rotary position encoding, shared by the stand-alone kernel (rope.cu) and by kernels that
// rotate on the way (latent_attention.cu).
//
// A pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a) with
// a = p * f_i. The frequencies f_i come from the host as doubles, and the angle and its
// sine and cosine are formed in double precision: at position 100,000 a float product
// p * f_0 is already 0.004 off. One thread per pair fills the table of a row once; every
// head of the row then uses it.
#pragma once

#include "common.cuh"

namespace ayk {

constexpr int ROPE_MAX_PAIRS = 256;
enum RopeLayout : int { ROPE_NEIGHBOURS = 0, ROPE_HALVES = 1 };

// cos_s, sin_s: ROPE_MAX_PAIRS floats each in shared memory; a barrier must follow.
__device__ __forceinline__ void rope_fill_table(float* cos_s, float* sin_s, int position,
                                                const double* __restrict__ freq, int pairs) {
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    double s, c;
    sincos((double)position * freq[i], &s, &c);
    cos_s[i] = (float)c;
    sin_s[i] = (float)s;
  }
}

// indices of pair i's two members inside the rotated stretch of `dims` entries
__device__ __forceinline__ void rope_members(int i, int dims, int layout, int& a, int& b) {
  if (layout == ROPE_NEIGHBOURS) {
    a = 2 * i;
    b = 2 * i + 1;
  } else {
    a = i;
    b = i + dims / 2;
  }
}

}  // namespace ayk
