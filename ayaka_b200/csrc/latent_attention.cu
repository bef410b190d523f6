// Latent attention: attention whose keys and values are up-projections W_uk c, W_uv c of one
// small latent row c per token, beside one rotated key piece kr that all heads share. The
// cache keeps only [c | kr] per token ("latent pages": [page][slot][rank + rot], one pool row
// per token whatever the number of heads).
//
// The up-projections are never applied to cached rows. With q_h = [q_plain | q_rot]:
//   q_plain . (W_uk,h c) = (W_uk,h^T q_plain) . c        (the query is taken to latent space)
//   sum_s w_s W_uv,h c_s = W_uv,h (sum_s w_s c_s)        (the weighted sum stays latent)
// so a step is: prepare (norm of c, rotation of kr and q_rot, store of [c | kr]), one small
// product per head that forms qa_h = [W_uk,h^T q_plain | q_rot], attention of all heads over
// the same latent rows (scores qa_h . [c | kr], values = the first `rank` entries of the key
// row), one small product per head W_uv,h (.) with the output gate in its epilogue. The three
// kernels of this file; the projections before and after are the engine's matrix products.
//
// All arithmetic in fp32; T is the type of the cache, of the queries and of the outputs.
#include "rope.cuh"

namespace ayk {

// ---------------------------------------------------------------------------------------------
// prepare: one CTA per row of the step.
//   proj row (fp32): [ q: heads x (dim + rot) | c_raw: rank | kr_raw: rot | ... ]
//   latent page row <- [ c_raw * rsqrt(mean(c_raw^2) + eps) * w_c | rotate(kr_raw) ]
//   q_plain[row]    <- the heads' unrotated parts            [heads x dim]
//   qa[row]         <- rotate(q_rot) at [h][rank ..]          [heads x (rank + rot)]
// Only the first rot_dims entries of a rotated piece are turned; the rest passes.
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ proj, int ld_proj, int kv_offset,
                                      const float* __restrict__ latent_weight, float eps,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ slots,
                                      const double* __restrict__ freq, int rot_dims, int layout,
                                      T* __restrict__ pages, T* __restrict__ q_plain,
                                      int ld_plain, T* __restrict__ qa, int ld_qa, int heads,
                                      int dim, int rot, int rank) {
  __shared__ float cos_s[ROPE_MAX_PAIRS], sin_s[ROPE_MAX_PAIRS];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  const int row = blockIdx.x, pairs = rot_dims / 2;
  rope_fill_table(cos_s, sin_s, positions[row], freq, pairs);
  const int slot = slots != nullptr ? slots[row] : -1;
  pdl_wait_for(proj);
  const float* src = proj + (size_t)row * ld_proj;
  const float* c_raw = src + kv_offset;
  float s = 0.f;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) s += c_raw[j] * c_raw[j];
  const float inv = 1.f / sqrtf(block_sum(s, scratch) / (float)rank + eps);  // (also a barrier)
  if (pages != nullptr && slot >= 0) {
    T* dst = pages + (size_t)slot * (rank + rot);
    for (int j = threadIdx.x; j < rank; j += blockDim.x) {
      stf(dst + j, c_raw[j] * inv * latent_weight[j]);
    }
    const float* kr = c_raw + rank;
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
      int a, b;
      rope_members(i, rot_dims, layout, a, b);
      const float u = kr[a], v = kr[b];
      stf(dst + rank + a, u * cos_s[i] - v * sin_s[i]);
      stf(dst + rank + b, v * cos_s[i] + u * sin_s[i]);
    }
    for (int j = rot_dims + threadIdx.x; j < rot; j += blockDim.x) stf(dst + rank + j, kr[j]);
  }
  T* plain = q_plain + (size_t)row * ld_plain;
  for (int idx = threadIdx.x; idx < heads * dim; idx += blockDim.x) {
    const int h = idx / dim, j = idx % dim;
    stf(plain + idx, src[(size_t)h * (dim + rot) + j]);
  }
  T* turned = qa + (size_t)row * ld_qa;
  for (int idx = threadIdx.x; idx < heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs, i = idx % pairs;
    int a, b;
    rope_members(i, rot_dims, layout, a, b);
    const float* q_rot = src + (size_t)h * (dim + rot) + dim;
    T* dst = turned + (size_t)h * (rank + rot) + rank;
    const float u = q_rot[a], v = q_rot[b];
    stf(dst + a, u * cos_s[i] - v * sin_s[i]);
    stf(dst + b, v * cos_s[i] + u * sin_s[i]);
  }
  const int rest = rot - rot_dims;
  for (int idx = threadIdx.x; idx < heads * rest; idx += blockDim.x) {
    const int h = idx / rest, j = rot_dims + idx % rest;
    stf(turned + (size_t)h * (rank + rot) + rank + j, src[(size_t)h * (dim + rot) + dim + j]);
  }
}

// ---------------------------------------------------------------------------------------------
// One small product per head: out[n][h][j] = sum_i a[n][h][i] * W_h(i, j), fp32 sums in the
// order of i whatever the batch. W_h(i, j) sits at w + h * w_head + i * w_in + j * w_out, so a
// head's matrix is used as stored ([in, out] rows: w_in = cols, w_out = 1) or transposed
// ([out, in] rows: w_in = 1, w_out = cols). With `gate` (fp32 [n][h * J + j]) the result is
// multiplied by sigmoid(gate). Tiles of 32 rows x 64 columns, 16 of the inner dimension at a
// time through shared memory; a thread owns 2 x 4 results.
constexpr int HL_BM = 32, HL_BN = 64, HL_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ a, int ld_a, int a_head, const T* __restrict__ w,
                   long long w_head, int w_in, int w_out, const float* __restrict__ gate,
                   int ld_gate, T* __restrict__ out, int ld_out, int out_head, int rows, int I,
                   int J) {
  __shared__ float a_s[HL_BK][HL_BM + 1];
  __shared__ float w_s[HL_BK][HL_BN + 1];
  pdl_launch_dependents();
  const int h = blockIdx.z, m0 = blockIdx.x * HL_BM, n0 = blockIdx.y * HL_BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const T* wh = w + (size_t)h * w_head;
  pdl_wait_for(a, gate);
  const T* ah = a + (size_t)h * a_head;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < I; k0 += HL_BK) {
    for (int idx = threadIdx.x; idx < HL_BK * HL_BM; idx += 256) {
      const int kk = idx % HL_BK, mm = idx / HL_BK;
      const int m = m0 + mm, k = k0 + kk;
      a_s[kk][mm] = (m < rows && k < I) ? ldf(ah + (size_t)m * ld_a + k) : 0.f;
    }
    for (int idx = threadIdx.x; idx < HL_BK * HL_BN; idx += 256) {
      int kk, nn;
      if (w_out == 1) {  // consecutive threads along the unit stride
        nn = idx % HL_BN;
        kk = idx / HL_BN;
      } else {
        kk = idx % HL_BK;
        nn = idx / HL_BK;
      }
      const int n = n0 + nn, k = k0 + kk;
      w_s[kk][nn] = (n < J && k < I) ? ldf(wh + (size_t)k * w_in + (size_t)n * w_out) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_BK; ++kk) {
      const float a0 = a_s[kk][ty * 2], a1 = a_s[kk][ty * 2 + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float wv = w_s[kk][tx * 4 + c];
        acc[0][c] = fmaf(a0, wv, acc[0][c]);
        acc[1][c] = fmaf(a1, wv, acc[1][c]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int m = m0 + ty * 2 + r;
    if (m >= rows) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx * 4 + c;
      if (n >= J) continue;
      float v = acc[r][c];
      if (gate != nullptr) {
        const float z = gate[(size_t)m * ld_gate + (size_t)h * J + n];
        v *= 1.f / (1.f + expf(-z));
      }
      stf(out + (size_t)m * ld_out + (size_t)h * out_head + n, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// attention over latent pages: one warp per (row, head); the warps of a CTA take neighbouring
// heads of one row, so the key rows they share are fetched from memory once. The row at
// position p of request b sees keys max(0, p - window + 1) .. p (window 0: all), read through
// the block table in tiles of 32 keys counted from a multiple of 32: lane j scores key t0 + j
// over all rank + rot entries, the warp keeps a running maximum and sum (fp32, expf), then the
// lanes split the first `rank` entries of the key rows and add w_j * row_j. The tiling depends
// only on the position: a row's result is the same alone, in a portion or in a mixed batch.
constexpr int LA_WARPS = 4;

template <typename T> struct Chunk8;
template <> struct Chunk8<float> {
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};
template <> struct Chunk8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T, int R>  // a lane holds R of the rank output entries: rank <= 32 * R
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(const T* __restrict__ qa, int ld_qa, const T* __restrict__ pages,
                        const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ request_of_row,
                        const int* __restrict__ positions, T* __restrict__ out, int ld_out,
                        int num_heads, int rank, int key_dim, int key_pad, int page_size,
                        float scale, int window, int vector_ok) {
  extern __shared__ __align__(16) float la_smem[];
  float* q_s = la_smem + (size_t)(threadIdx.x >> 5) * key_pad;
  __shared__ float w_s[LA_WARPS][32];
  __shared__ long long off_s[LA_WARPS][32];
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x, head = blockIdx.y * LA_WARPS + warp;
  if (head >= num_heads) return;  // (no block barrier below)
  const int b = request_of_row[row], p = positions[row];
  pdl_wait_for(qa, pages);
  T* dst = out + (size_t)row * ld_out + (size_t)head * rank;
  if (b < 0) {
    for (int d = lane; d < rank; d += 32) stf(dst + d, 0.f);
    return;
  }
  const T* q = qa + (size_t)row * ld_qa + (size_t)head * key_dim;
  for (int d = lane; d < key_dim; d += 32) q_s[d] = ldf(q + d) * scale;
  __syncwarp();
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* table = block_table + (size_t)b * table_stride;
  float m = -INFINITY, l = 0.f;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  for (int t0 = (lo / 32) * 32; t0 <= p; t0 += 32) {
    const int t = t0 + lane;
    const bool valid = t >= lo && t <= p;
    long long off = -1;
    float score = -INFINITY;
    if (valid) {
      off = ((long long)table[t / page_size] * page_size + t % page_size) * key_dim;
      const T* key = pages + off;
      float dot = 0.f;
      if (vector_ok) {
        for (int d = 0; d < key_dim; d += 8) {
          float kv[8];
          Chunk8<T>::load(key + d, kv);
#pragma unroll
          for (int e = 0; e < 8; ++e) dot = fmaf(q_s[d + e], kv[e], dot);
        }
      } else {
        for (int d = 0; d < key_dim; ++d) dot = fmaf(q_s[d], ldf(key + d), dot);
      }
      score = dot;
    }
    const float m_new = fmaxf(m, warp_max(score));  // every tile holds at least one key
    const float wgt = valid ? expf(score - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(wgt);
    m = m_new;
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] *= corr;
    w_s[warp][lane] = wgt;
    off_s[warp][lane] = off;
    __syncwarp();
    const int count = min(32, p - t0 + 1);
    for (int j = 0; j < count; ++j) {
      const long long oj = off_s[warp][j];
      if (oj < 0) continue;
      const float wj = w_s[warp][j];
      const T* value = pages + oj;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int d = lane + 32 * r;
        if (d < rank) acc[r] = fmaf(wj, ldf(value + d), acc[r]);
      }
    }
    __syncwarp();
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = lane + 32 * r;
    if (d < rank) stf(dst + d, acc[r] * inv);
  }
}

template <typename T>
int latent_attention(const void* qa, int ld_qa, const void* pages, const int* block_table,
                     int table_stride, const int* request_of_row, const int* positions, void* out,
                     int ld_out, int rows, int num_heads, int rank, int rot, int page_size,
                     float scale, int window, cudaStream_t stream) {
  const int key_dim = rank + rot;
  const int key_pad = (key_dim + 7) / 8 * 8;
  const int vector_ok =
      (key_dim % 8 == 0 && ((uintptr_t)pages % 16) == 0) ? 1 : 0;
  const size_t smem = (size_t)LA_WARPS * key_pad * sizeof(float);
  const dim3 grid(rows, (num_heads + LA_WARPS - 1) / LA_WARPS), block(LA_WARPS * 32);
#define AYK_LA(R)                                                                              \
  return launch_kernel(latent_attention_kernel<T, R>, grid, block, smem, stream, 1,            \
                       (const T*)qa, ld_qa, (const T*)pages, block_table, table_stride,        \
                       request_of_row, positions, (T*)out, ld_out, num_heads, rank, key_dim,   \
                       key_pad, page_size, scale, window, vector_ok)
  if (rank <= 64) AYK_LA(2);
  if (rank <= 128) AYK_LA(4);
  if (rank <= 256) AYK_LA(8);
  if (rank <= 512) AYK_LA(16);
  AYK_LA(32);
#undef AYK_LA
}

}  // namespace ayk

AYK_API void ayk_set_pdl(int on) { ayk::pdl_enabled() = on; }

// type: 0 = float32, 1 = bfloat16 (cache, queries). pages may be null (a run that reads a
// cache another run wrote) or a row's slot negative: nothing is stored then.
AYK_API int ayk_latent_prepare(const float* proj, int ld_proj, int kv_offset,
                               const float* latent_weight, float eps, const int* positions,
                               const int* slots, const double* freq, int rot_dims, int layout,
                               void* pages, void* q_plain, int ld_plain, void* qa, int ld_qa,
                               int rows, int heads, int dim, int rot, int rank, int type,
                               void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || heads < 1 || dim < 0 || rot < 0 || rank < 1 || rot_dims < 0 || rot_dims % 2 ||
      rot_dims > rot || kv_offset < heads * (dim + rot) || ld_proj < kv_offset + rank + rot ||
      ld_plain < heads * dim || ld_qa < heads * (rank + rot) || proj == nullptr ||
      latent_weight == nullptr || positions == nullptr || (rot_dims > 0 && freq == nullptr) ||
      q_plain == nullptr || qa == nullptr || !(eps > 0.f) ||
      (layout != ROPE_NEIGHBOURS && layout != ROPE_HALVES)) {
    return AYK_BAD_ARGUMENT;
  }
  if (rot_dims / 2 > ROPE_MAX_PAIRS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return launch_kernel(latent_prepare_kernel<float>, dim3(rows), dim3(256), 0, s, 1, proj,
                         ld_proj, kv_offset, latent_weight, eps, positions, slots, freq, rot_dims,
                         layout, (float*)pages, (float*)q_plain, ld_plain, (float*)qa, ld_qa,
                         heads, dim, rot, rank);
  }
  if (type == 1) {
    return launch_kernel(latent_prepare_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, 1,
                         proj, ld_proj, kv_offset, latent_weight, eps, positions, slots, freq,
                         rot_dims, layout, (__nv_bfloat16*)pages, (__nv_bfloat16*)q_plain,
                         ld_plain, (__nv_bfloat16*)qa, ld_qa, heads, dim, rot, rank);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_head_linear(const void* a, int ld_a, int a_head, const void* w, long long w_head,
                            int w_in, int w_out, const float* gate, int ld_gate, void* out,
                            int ld_out, int out_head, int rows, int heads, int I, int J, int type,
                            void* stream) {
  using namespace ayk;
  if (rows == 0 || heads == 0 || J == 0) return AYK_OK;
  if (rows < 0 || heads < 0 || I < 1 || J < 0 || a == nullptr || w == nullptr || out == nullptr ||
      w_in < 1 || w_out < 1 || (w_in != 1 && w_out != 1) || heads > 65535) {
    return AYK_BAD_ARGUMENT;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const dim3 grid((rows + HL_BM - 1) / HL_BM, (J + HL_BN - 1) / HL_BN, heads);
  if (grid.y > 65535) return AYK_TOO_LARGE;
  if (type == 0) {
    return launch_kernel(head_linear_kernel<float>, grid, dim3(256), 0, s, 1, (const float*)a,
                         ld_a, a_head, (const float*)w, w_head, w_in, w_out, gate, ld_gate,
                         (float*)out, ld_out, out_head, rows, I, J);
  }
  if (type == 1) {
    return launch_kernel(head_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, 1,
                         (const __nv_bfloat16*)a, ld_a, a_head, (const __nv_bfloat16*)w, w_head,
                         w_in, w_out, gate, ld_gate, (__nv_bfloat16*)out, ld_out, out_head, rows,
                         I, J);
  }
  return AYK_BAD_ARGUMENT;
}

AYK_API int ayk_latent_attention(const void* qa, int ld_qa, const void* pages,
                                 const int* block_table, int table_stride,
                                 const int* request_of_row, const int* positions, void* out,
                                 int ld_out, int rows, int num_heads, int rank, int rot,
                                 int page_size, float scale, int window, int type, void* stream) {
  using namespace ayk;
  if (rows == 0) return AYK_OK;
  if (rows < 0 || num_heads < 1 || rank < 1 || rot < 0 || page_size < 1 || window < 0 ||
      qa == nullptr || pages == nullptr || block_table == nullptr || request_of_row == nullptr ||
      positions == nullptr || out == nullptr || ld_qa < num_heads * (rank + rot) ||
      ld_out < num_heads * rank) {
    return AYK_BAD_ARGUMENT;
  }
  if (rank > 1024 || rank + rot > 2048 || num_heads > 65535 * ayk::LA_WARPS) return AYK_TOO_LARGE;
  cudaStream_t s = (cudaStream_t)stream;
  if (type == 0) {
    return latent_attention<float>(qa, ld_qa, pages, block_table, table_stride, request_of_row,
                                   positions, out, ld_out, rows, num_heads, rank, rot, page_size,
                                   scale, window, s);
  }
  if (type == 1) {
    return latent_attention<__nv_bfloat16>(qa, ld_qa, pages, block_table, table_stride,
                                           request_of_row, positions, out, ld_out, rows, num_heads,
                                           rank, rot, page_size, scale, window, s);
  }
  return AYK_BAD_ARGUMENT;
}
