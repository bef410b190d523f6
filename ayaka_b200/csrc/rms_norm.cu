// Root-mean-square norms over fp32 rows: y = x * rsqrt(mean(x^2) + eps) * (offset + w), the
// mean taken over each of `groups` equal parts of the row on its own. `offset` is 0 for a
// plain weight and 1 for a weight stored as its deviation from one. `rows` may gather (output
// row i normalises input row rows[i]: the final norm runs on the wanted rows only).
//
// A gate may ride along (fp32, same row and column as x):
//   GATE_SILU_BEFORE: x is first multiplied by silu(gate), then normalised (the gated norm of a
//     state-space layer: the gate comes before the norm);
//   GATE_SIGMOID_AFTER: the normalised, weighted value is multiplied by sigmoid(gate) (the
//     output gate of a matrix-memory layer).
// Everything in fp32, rounded once to the output type. Any width.
#include "common.cuh"

namespace ayk {

enum GateMode : int { GATE_NONE = 0, GATE_SILU_BEFORE = 1, GATE_SIGMOID_AFTER = 2 };

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

template <typename TOut>
__global__ void rms_norm_kernel(const float* __restrict__ x, int ld_x,
                                const int* __restrict__ rows, const float* __restrict__ weight,
                                float weight_offset, float eps, int group_width,
                                const float* __restrict__ gate, int ld_gate, int gate_mode,
                                TOut* __restrict__ out, int ld_out) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int r = blockIdx.x, g = blockIdx.y;
  const int row = rows != nullptr ? rows[r] : r;
  pdl_wait_for(x, gate);
  const float* src = x + (size_t)row * ld_x + (size_t)g * group_width;
  const float* gt = gate != nullptr ? gate + (size_t)row * ld_gate + (size_t)g * group_width
                                    : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < group_width; c += blockDim.x) {
    float v = src[c];
    if (gate_mode == GATE_SILU_BEFORE) {
      const float z = gt[c];
      v *= z * sigmoid_f(z);
    }
    s += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(s, scratch) / (float)group_width + eps);
  const float* w = weight + (size_t)g * group_width;
  TOut* dst = out + (size_t)r * ld_out + (size_t)g * group_width;
  for (int c = threadIdx.x; c < group_width; c += blockDim.x) {
    float v = src[c];
    if (gate_mode == GATE_SILU_BEFORE) {
      const float z = gt[c];
      v *= z * sigmoid_f(z);
    }
    v = v * inv * (weight_offset + w[c]);
    if (gate_mode == GATE_SIGMOID_AFTER) v *= sigmoid_f(gt[c]);
    stf(dst + c, v);
  }
}

template <typename TOut>
int rms_norm(const float* x, int ld_x, const int* rows, const float* weight, float weight_offset,
             float eps, int groups, const float* gate, int ld_gate, int gate_mode, void* out,
             int ld_out, int n, int width, cudaStream_t stream) {
  if (n == 0) return AYK_OK;
  if (n < 0 || width < 1 || groups < 1 || width % groups || ld_x < width || ld_out < width ||
      !(eps > 0.f) || weight == nullptr || gate_mode < GATE_NONE ||
      gate_mode > GATE_SIGMOID_AFTER || ((gate_mode != GATE_NONE) != (gate != nullptr)) ||
      (gate != nullptr && ld_gate < width)) {
    return AYK_BAD_ARGUMENT;
  }
  const int group_width = width / groups;
  const int threads = group_width >= 2048 ? 512 : (group_width >= 512 ? 256 : 128);
  return launch_kernel(rms_norm_kernel<TOut>, dim3(n, groups), dim3(threads), 0, stream, 1, x,
                       ld_x, rows, weight, weight_offset, eps, group_width, gate, ld_gate,
                       gate_mode, (TOut*)out, ld_out);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// out_type: 0 = float32, 1 = bfloat16.
AYK_API int ayk_rms_norm(const float* x, int ld_x, const int* rows, const float* weight,
                         float weight_offset, float eps, int groups, const float* gate,
                         int ld_gate, int gate_mode, void* out, int ld_out, int n, int width,
                         int out_type, void* stream) {
  if (out_type == 0) {
    return ayk::rms_norm<float>(x, ld_x, rows, weight, weight_offset, eps, groups, gate, ld_gate,
                                gate_mode, out, ld_out, n, width, (cudaStream_t)stream);
  }
  if (out_type == 1) {
    return ayk::rms_norm<__nv_bfloat16>(x, ld_x, rows, weight, weight_offset, eps, groups, gate,
                                        ld_gate, gate_mode, out, ld_out, n, width,
                                        (cudaStream_t)stream);
  }
  return AYK_BAD_ARGUMENT;
}
