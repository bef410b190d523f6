// Softmax attention whose heads' scores are mixed before the softmax ("talking heads"), over
// paged keys and values, with keys visible only inside the query's own block of positions.
//
// With per-head factors temp[a], a mixing matrix talk[h][a] and the factor `scale`,
//   score_h(t, s) = sum_a talk[h][a] temp[a] scale (q_a(t) . k_kv(a)(s)),
// where kv(a) = a / (H / G) is head a's key/value head. The sum over a is linear in the
// queries, so it is taken on the query's side once per row: with
//   m_(h,g)(t) = sum_(a in group g) talk[h][a] temp[a] scale q_a(t)        (dim entries)
// the score is sum_g m_(h,g)(t) . k_g(s): attention of H heads over ONE key of G * dim
// entries per token (the token's key heads side by side), and nothing is mixed per (t, s)
// pair. The values stay per key/value head: head h sums v_kv(h).
//
// prepare (one launch per layer): from a row of the fused projection (fp32): the norm of the
// whole query projection and of the whole key projection by their root mean square (one
// mean over all heads' entries, a weight per entry; a bias of the projection is added first:
// `bias` follows the projection's columns, queries, keys, values), the rotation of the first `rot_dims`
// entries of every head, the mixed queries m (compute type), and the row's key and value
// into its cache slot.
// attention: one CTA per (row, head); fp32 scores, softmax and sums; the result times
// sigmoid(gate[h]) when a gate is given.
#include "rope.cuh"

namespace ayk {

constexpr int TALK_THREADS = 256;
constexpr int ATT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(TALK_THREADS)
talking_prepare_kernel(const float* __restrict__ proj, int ld_proj, int k_off, int v_off,
                       const float* __restrict__ bias, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                       float eps, const int* __restrict__ positions,
                       const double* __restrict__ freq, int rot_dims, int layout,
                       const float* __restrict__ talk, const float* __restrict__ temp,
                       float scale, const int* __restrict__ slot_mapping,
                       T* __restrict__ k_pages, T* __restrict__ v_pages, int page_size,
                       T* __restrict__ qmix, int ld_qmix, int H, int G, int dim, int vdim) {
  extern __shared__ __align__(16) float prep_smem[];
  __shared__ float scratch[33];
  float* qs = prep_smem;            // H * dim
  float* ks = qs + H * dim;         // G * dim
  float* cos_s = ks + G * dim;      // ROPE_MAX_PAIRS
  float* sin_s = cos_s + ROPE_MAX_PAIRS;
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x;
  const int qn = H * dim, kn = G * dim, pairs = rot_dims / 2;
  const int position = positions[row];
  rope_fill_table(cos_s, sin_s, position, freq, pairs);
  pdl_wait_for(proj);
  const float* src = proj + (size_t)row * ld_proj;
  float sq = 0.f, sk = 0.f;
  for (int i = tid; i < qn; i += TALK_THREADS) {
    const float v = src[i] + (bias != nullptr ? bias[i] : 0.f);
    qs[i] = v;
    sq += v * v;
  }
  for (int i = tid; i < kn; i += TALK_THREADS) {
    const float v = src[k_off + i] + (bias != nullptr ? bias[k_off + i] : 0.f);
    ks[i] = v;
    sk += v * v;
  }
  if (q_weight != nullptr) {
    const float inv = 1.f / sqrtf(block_sum(sq, scratch) / (float)qn + eps);
    for (int i = tid; i < qn; i += TALK_THREADS) qs[i] = qs[i] * inv * q_weight[i];
  }
  if (k_weight != nullptr) {
    const float inv = 1.f / sqrtf(block_sum(sk, scratch) / (float)kn + eps);
    for (int i = tid; i < kn; i += TALK_THREADS) ks[i] = ks[i] * inv * k_weight[i];
  }
  __syncthreads();
  // every pair of every head by one thread
  for (int idx = tid; idx < (H + G) * pairs; idx += TALK_THREADS) {
    const int head = idx / pairs, i = idx % pairs;
    float* v = head < H ? qs + head * dim : ks + (head - H) * dim;
    int a, b;
    rope_members(i, rot_dims, layout, a, b);
    const float x = v[a], y = v[b], c = cos_s[i], s = sin_s[i];
    v[a] = x * c - y * s;
    v[b] = y * c + x * s;
  }
  __syncthreads();
  const int per = H / G;
  T* mixed = qmix + (size_t)row * ld_qmix;
  for (int idx = tid; idx < H * kn; idx += TALK_THREADS) {
    const int h = idx / kn, g = (idx % kn) / dim, d = idx % dim;
    float sum = 0.f;
    for (int a = g * per; a < (g + 1) * per; ++a) {
      const float t = talk != nullptr ? talk[h * H + a] : (a == h ? 1.f : 0.f);
      const float factor = t * (temp != nullptr ? temp[a] : 1.f) * scale;
      sum = fmaf(factor, qs[a * dim + d], sum);
    }
    stf(mixed + idx, sum);
  }
  const int slot = slot_mapping != nullptr ? slot_mapping[row] : -1;
  if (slot >= 0 && k_pages != nullptr) {
    const int page = slot / page_size, s = slot % page_size;
    for (int i = tid; i < kn; i += TALK_THREADS) {
      const int g = i / dim, d = i % dim;
      stf(k_pages + (((size_t)page * G + g) * page_size + s) * dim + d, ks[i]);
    }
    for (int i = tid; i < G * vdim; i += TALK_THREADS) {
      const int g = i / vdim, d = i % vdim;
      stf(v_pages + (((size_t)page * G + g) * page_size + s) * vdim + d,
          src[v_off + i] + (bias != nullptr ? bias[v_off + i] : 0.f));
    }
  }
}

// One CTA per (row, head). Keys lo .. position with lo the start of the position's block of
// `chunk` positions (chunk 0: position 0), and not before position - window + 1 (window 0:
// no such limit). qmix rows: [H][G * dim].
template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
talking_attention_kernel(const T* __restrict__ qmix, int ld_qmix, const T* __restrict__ k_pages,
                         const T* __restrict__ v_pages, const int* __restrict__ block_table,
                         int ld_table, const int* __restrict__ request_of_row,
                         const int* __restrict__ positions, const float* __restrict__ gate,
                         int ld_gate, T* __restrict__ out, int ld_out, int H, int G, int dim,
                         int vdim, int page_size, int chunk, int window) {
  extern __shared__ __align__(16) float att_smem[];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int row = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int kn = G * dim;
  float* qv = att_smem;   // kn
  float* p = qv + kn;     // the keys' scores, then weights
  const int b = request_of_row[row];
  T* dst = out + (size_t)row * ld_out + (size_t)h * vdim;
  if (b < 0) {  // a row of padding
    for (int c = tid; c < vdim; c += ATT_THREADS) stf(dst + c, 0.f);
    return;
  }
  const int position = positions[row];
  int lo = chunk > 0 ? position - position % chunk : 0;
  if (window > 0) lo = max(lo, position - window + 1);
  const int keys = position - lo + 1;
  const int* table = block_table + (size_t)b * ld_table;
  pdl_wait_for(qmix, k_pages, v_pages, gate);
  const T* q = qmix + (size_t)row * ld_qmix + (size_t)h * kn;
  for (int i = tid; i < kn; i += ATT_THREADS) qv[i] = ldf(q + i);
  __syncthreads();
  float best = -INFINITY;
  for (int j = tid; j < keys; j += ATT_THREADS) {
    const int at = lo + j, page = table[at / page_size], s = at % page_size;
    float sum = 0.f;
    for (int g = 0; g < G; ++g) {
      const T* k = k_pages + (((size_t)page * G + g) * page_size + s) * dim;
      const float* qg = qv + g * dim;
      for (int d = 0; d < dim; ++d) sum = fmaf(qg[d], ldf(k + d), sum);
    }
    p[j] = sum;
    best = fmaxf(best, sum);
  }
  // the block's maximum, then the weights and their sum
  best = warp_max(best);
  __syncthreads();
  if ((tid & 31) == 0) scratch[tid >> 5] = best;
  __syncthreads();
  best = scratch[0];
  for (int w = 1; w < ATT_THREADS / 32; ++w) best = fmaxf(best, scratch[w]);
  float total = 0.f;
  for (int j = tid; j < keys; j += ATT_THREADS) {
    const float e = expf(p[j] - best);
    p[j] = e;
    total += e;
  }
  total = block_sum(total, scratch);  // (its barriers also publish p)
  const int kv = h / (H / G);
  float factor = 1.f / total;
  if (gate != nullptr) factor /= 1.f + expf(-gate[(size_t)row * ld_gate + h]);
  for (int c = tid; c < vdim; c += ATT_THREADS) {
    float sum = 0.f;
    for (int j = 0; j < keys; ++j) {
      const int at = lo + j, page = table[at / page_size], s = at % page_size;
      sum = fmaf(p[j], ldf(v_pages + (((size_t)page * G + kv) * page_size + s) * vdim + c), sum);
    }
    stf(dst + c, sum * factor);
  }
}

template <typename K> inline void allow_large_smem(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
}

template <typename T>
int talking_prepare(const float* proj, int ld_proj, int k_off, int v_off, const float* bias,
                    const float* q_weight, const float* k_weight, float eps, const int* positions, const double* freq,
                    int rot_dims, int layout, const float* talk, const float* temp, float scale,
                    const int* slot_mapping, void* k_pages, void* v_pages, int page_size,
                    void* qmix, int ld_qmix, int rows, int H, int G, int dim, int vdim,
                    cudaStream_t stream) {
  const size_t smem = ((size_t)(H + G) * dim + 2 * ROPE_MAX_PAIRS) * sizeof(float);
  if (smem > 160 * 1024) return AYK_TOO_LARGE;
  static const bool allowed = (allow_large_smem(talking_prepare_kernel<T>), true);
  (void)allowed;
  return launch_kernel(talking_prepare_kernel<T>, dim3(rows), dim3(TALK_THREADS), smem, stream,
                       1, proj, ld_proj, k_off, v_off, bias, q_weight, k_weight, eps, positions, freq,
                       rot_dims, layout, talk, temp, scale, slot_mapping, (T*)k_pages,
                       (T*)v_pages, page_size, (T*)qmix, ld_qmix, H, G, dim, vdim);
}

template <typename T>
int talking_attention(const void* qmix, int ld_qmix, const void* k_pages, const void* v_pages,
                      const int* block_table, int ld_table, const int* request_of_row,
                      const int* positions, const float* gate, int ld_gate, void* out,
                      int ld_out, int rows, int H, int G, int dim, int vdim, int page_size,
                      int chunk, int window, int reach, cudaStream_t stream) {
  const size_t smem = ((size_t)G * dim + reach) * sizeof(float);
  if (smem > 160 * 1024) return AYK_TOO_LARGE;
  static const bool allowed = (allow_large_smem(talking_attention_kernel<T>), true);
  (void)allowed;
  return launch_kernel(talking_attention_kernel<T>, dim3(rows, H), dim3(ATT_THREADS), smem,
                       stream, 1, (const T*)qmix, ld_qmix, (const T*)k_pages,
                       (const T*)v_pages, block_table, ld_table, request_of_row, positions, gate,
                       ld_gate, (T*)out, ld_out, H, G, dim, vdim, page_size, chunk, window);
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16 (mixed queries and pages). bias, q_weight / k_weight, talk,
// temp may be null (no bias, no norm, no mixing, no per-head factor); pages and slot_mapping may be null
// (nothing is stored).
AYK_API int ayk_talking_prepare(const float* proj, int ld_proj, int k_off, int v_off,
                                const float* bias, const float* q_weight, const float* k_weight, float eps,
                                const int* positions, const double* freq, int rot_dims,
                                int layout, const float* talk, const float* temp, float scale,
                                const int* slot_mapping, void* k_pages, void* v_pages,
                                int page_size, void* qmix, int ld_qmix, int rows, int H, int G,
                                int dim, int vdim, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || H < 1 || G < 1 || H % G || dim < 1 || vdim < 1 || proj == nullptr ||
      positions == nullptr || qmix == nullptr || rot_dims < 0 || rot_dims % 2 ||
      rot_dims > dim || (rot_dims > 0 && freq == nullptr) || !(eps > 0.f) ||
      ld_qmix < H * G * dim || k_off < H * dim || v_off < k_off + G * dim ||
      ld_proj < v_off + G * vdim || (k_pages != nullptr && (v_pages == nullptr ||
      slot_mapping == nullptr || page_size < 1)) ||
      (layout != ROPE_NEIGHBOURS && layout != ROPE_HALVES)) {
    return AYK_BAD_ARGUMENT;
  }
  if (rot_dims / 2 > ROPE_MAX_PAIRS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return talking_prepare<float>(proj, ld_proj, k_off, v_off, bias, q_weight, k_weight, eps,
                                  positions, freq, rot_dims, layout, talk, temp, scale,
                                  slot_mapping, k_pages, v_pages, page_size, qmix, ld_qmix, rows,
                                  H, G, dim, vdim, s);
  }
  if (type == 1) {
    return talking_prepare<__nv_bfloat16>(proj, ld_proj, k_off, v_off, bias, q_weight, k_weight, eps,
                                          positions, freq, rot_dims, layout, talk, temp, scale,
                                          slot_mapping, k_pages, v_pages, page_size, qmix,
                                          ld_qmix, rows, H, G, dim, vdim, s);
  }
  return AYK_BAD_ARGUMENT;
}

// `reach`: the most keys any row of the launch sees (bounds the shared memory).
AYK_API int ayk_talking_attention(const void* qmix, int ld_qmix, const void* k_pages,
                                  const void* v_pages, const int* block_table, int ld_table,
                                  const int* request_of_row, const int* positions,
                                  const float* gate, int ld_gate, void* out, int ld_out, int rows,
                                  int H, int G, int dim, int vdim, int page_size, int chunk,
                                  int window, int reach, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || H < 1 || G < 1 || H % G || dim < 1 || vdim < 1 || qmix == nullptr ||
      k_pages == nullptr || v_pages == nullptr || block_table == nullptr ||
      request_of_row == nullptr || positions == nullptr || out == nullptr || page_size < 1 ||
      chunk < 0 || window < 0 || reach < 1 || ld_qmix < H * G * dim || ld_out < H * vdim ||
      (gate != nullptr && ld_gate < H) || H > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return talking_attention<float>(qmix, ld_qmix, k_pages, v_pages, block_table, ld_table,
                                    request_of_row, positions, gate, ld_gate, out, ld_out, rows,
                                    H, G, dim, vdim, page_size, chunk, window, reach, s);
  }
  if (type == 1) {
    return talking_attention<__nv_bfloat16>(qmix, ld_qmix, k_pages, v_pages, block_table,
                                            ld_table, request_of_row, positions, gate, ld_gate,
                                            out, ld_out, rows, H, G, dim, vdim, page_size, chunk,
                                            window, reach, s);
  }
  return AYK_BAD_ARGUMENT;
}
