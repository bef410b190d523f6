// Rotary position encoding in place on rows of [heads x head_stride] values: in every head
// the `dims` entries from `offset` on are rotated (pairs of neighbours, or entry i with
// entry i + dims/2), the rest passes. One CTA per row; see rope.cuh for the arithmetic.
#include "rope.cuh"

namespace ayk {

template <typename T>
__global__ void rope_kernel(T* __restrict__ x, int ld, const int* __restrict__ positions,
                            const double* __restrict__ freq, int heads, int head_stride,
                            int offset, int dims, int layout) {
  __shared__ float cos_s[ROPE_MAX_PAIRS], sin_s[ROPE_MAX_PAIRS];
  pdl_launch_dependents();
  const int row = blockIdx.x, pairs = dims / 2;
  rope_fill_table(cos_s, sin_s, positions[row], freq, pairs);
  pdl_wait_for(x);
  __syncthreads();
  T* base = x + (size_t)row * ld + offset;
  for (int idx = threadIdx.x; idx < heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs, i = idx % pairs;
    int a, b;
    rope_members(i, dims, layout, a, b);
    T* p = base + (size_t)h * head_stride;
    const float u = ldf(p + a), v = ldf(p + b);
    stf(p + a, u * cos_s[i] - v * sin_s[i]);
    stf(p + b, v * cos_s[i] + u * sin_s[i]);
  }
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16. freq: dims / 2 doubles on the device.
AYK_API int ayk_rope(void* x, int ld, const int* positions, const double* freq, int rows,
                     int heads, int head_stride, int offset, int dims, int layout, int type,
                     void* stream) {
  using namespace ayk;
  if (rows == 0 || heads == 0 || dims == 0) return AYK_OK;
  if (rows < 0 || heads < 0 || dims < 0 || dims % 2 || offset < 0 || offset + dims > head_stride ||
      (long long)heads * head_stride > ld || positions == nullptr || freq == nullptr ||
      (layout != ROPE_NEIGHBOURS && layout != ROPE_HALVES)) {
    return AYK_BAD_ARGUMENT;
  }
  if (dims / 2 > ROPE_MAX_PAIRS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return launch_kernel(rope_kernel<float>, dim3(rows), dim3(128), 0, s, 1, (float*)x, ld,
                         positions, freq, heads, head_stride, offset, dims, layout);
  }
  if (type == 1) {
    return launch_kernel(rope_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, s, 1,
                         (__nv_bfloat16*)x, ld, positions, freq, heads, head_stride, offset, dims,
                         layout);
  }
  return AYK_BAD_ARGUMENT;
}
