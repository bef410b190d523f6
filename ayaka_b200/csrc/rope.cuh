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

// The same table with fewer double-precision operations: the angle position * f is formed
// in double precision and brought into [-pi, pi] there (two multiplications and a rounding),
// its sine and cosine are then taken in single precision, whose error on so small an argument
// is about 1e-7. For kernels on a decode step's chain, where the double-precision sincos
// of the function above is most of the kernel's time.
__device__ __forceinline__ void rope_fill_table_reduced(float* cos_s, float* sin_s, int position,
                                                        const double* __restrict__ freq,
                                                        int pairs) {
  const double two_pi = 6.283185307179586476925287, inv_two_pi = 0.159154943091895335768884;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const double angle = (double)position * freq[i];
    const float reduced = (float)(angle - two_pi * rint(angle * inv_two_pi));
    float s, c;
    sincosf(reduced, &s, &c);
    cos_s[i] = c;
    sin_s[i] = s;
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
