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
// `bias` follows the projection's columns, queries, keys, values), the rotation of the first
// `rot_dims` entries of every head, the mixed queries m (compute type), and the row's key and
// value into its cache slot.
// attention: fp32 scores, softmax and sums; the result times sigmoid(gate[h]) when a gate is
// given. float32: one CTA per (row, head) on the CUDA cores; bfloat16: the tensor-core kernel
// further down where the sizes allow.
#include "rope.cuh"

namespace ayk {

constexpr int TALK_THREADS = 256;
constexpr int ATT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(TALK_THREADS)
talking_prepare_kernel(const float* __restrict__ proj, int ld_proj, int k_off, int v_off,
                       const float* __restrict__ bias, const float* __restrict__ q_weight,
                       const float* __restrict__ k_weight, float eps, const int* __restrict__ positions,
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
  float* mix_s = sin_s + ROPE_MAX_PAIRS;  // H * H: talk[h][a] * temp[a] * scale
  pdl_launch_dependents();
  const int row = blockIdx.x, tid = threadIdx.x;
  const int qn = H * dim, kn = G * dim, pairs = rot_dims / 2;
  const int position = positions[row];
  // (weights and positions are not the kernel ahead's: all this runs under its tail)
  rope_fill_table_reduced(cos_s, sin_s, position, freq, pairs);
  for (int i = tid; i < H * H; i += TALK_THREADS) {
    const int a = i % H;
    const float t = talk != nullptr ? talk[i] : (a == i / H ? 1.f : 0.f);
    mix_s[i] = t * (temp != nullptr ? temp[a] : 1.f) * scale;
  }
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
  {
    // both sums of squares through one exchange
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((tid & 31) == 0) {
      scratch[tid >> 5] = sq;
      scratch[8 + (tid >> 5)] = sk;
    }
    __syncthreads();
    sq = sk = 0.f;
#pragma unroll
    for (int w = 0; w < TALK_THREADS / 32; ++w) {
      sq += scratch[w];
      sk += scratch[8 + w];
    }
  }
  if (q_weight != nullptr) {
    const float inv = 1.f / sqrtf(sq / (float)qn + eps);
    for (int i = tid; i < qn; i += TALK_THREADS) qs[i] = qs[i] * inv * q_weight[i];
  }
  if (k_weight != nullptr) {
    const float inv = 1.f / sqrtf(sk / (float)kn + eps);
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
  for (int j = tid; j < kn; j += TALK_THREADS) {  // entry j of the token-wide key: (g, d)
    const int g = j / dim, d = j - g * dim;
    const float* group = qs + (size_t)g * per * dim + d;  // the group's heads, dim apart
    for (int h = 0; h < H; ++h) {
      const float* factors = mix_s + h * H + g * per;
      float sum = 0.f;
      for (int a = 0; a < per; ++a) sum = fmaf(factors[a], group[a * dim], sum);
      stf(mixed + (size_t)h * kn + j, sum);
    }
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

// ---------------------------------------------------------------------------------------------
// The same attention on the warp-level tensor cores (bfloat16). A CTA takes `window_rows`
// consecutive rows of the step (16 for steps with prompt portions, 1 for steps of single
// rows, where a row's keys are its own) and eight heads, a warp per head. The rows of a
// window that belong to one request and one block of positions form a *segment*: they see
// the same keys, up to each row's own position. Per segment the keys come in tiles of 32:
// the CTA copies a tile's keys (all key heads side by side, as the mixed queries want them)
// and values into shared memory once, and every warp computes its head's scores
// (mma.sync m16n8k16, fp32 accumulators, the mixed queries held in registers), an online
// softmax in fp32, and the weighted sum of its key/value head's values. The weights enter
// that product as two bfloat16 terms, w = hi + lo, so that they carry 16 bits of mantissa
// instead of 8. Keys past the segment's last position are zero in shared memory. A tile's
// copies are asynchronous and fill one of two stages while the other is multiplied.
constexpr int MMA_HEADS = 8;
constexpr int MMA_KEYS = 32;

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int KSTEPS, int VT>  // G * dim <= 16 KSTEPS, vdim <= 8 VT
__global__ void __launch_bounds__(MMA_HEADS * 32)
talking_attention_mma_kernel(const __nv_bfloat16* __restrict__ qmix, int ld_qmix,
                             const __nv_bfloat16* __restrict__ k_pages,
                             const __nv_bfloat16* __restrict__ v_pages,
                             const int* __restrict__ block_table, int ld_table,
                             const int* __restrict__ request_of_row,
                             const int* __restrict__ positions, const float* __restrict__ gate,
                             int ld_gate, __nv_bfloat16* __restrict__ out, int ld_out, int rows,
                             int H, int G, int dim, int vdim, int page_size, int chunk,
                             int window_rows) {
  extern __shared__ __align__(16) unsigned char mma_smem[];
  __shared__ int req_s[16], pos_s[16];
  using bf16 = __nv_bfloat16;
  const int kn = G * dim, vn = G * vdim;
  const int ldk = kn + 8, ldv = vn + 8;  // rows padded: a fragment's rows in different banks
  const int stage_elems = MMA_KEYS * (ldk + ldv);
  bf16* stages = reinterpret_cast<bf16*>(mma_smem);           // two stages of keys, values
  int* pages_s = reinterpret_cast<int*>(stages + 2 * stage_elems);  // a segment's pages
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int row0 = blockIdx.x * window_rows, nrows = min(window_rows, rows - row0);
  const int h = blockIdx.y * MMA_HEADS + warp;
  const bool active = h < H;
  if (tid < 16) {
    req_s[tid] = tid < nrows ? request_of_row[row0 + tid] : -1;
    pos_s[tid] = tid < nrows ? positions[row0 + tid] : 0;
  }
  pdl_wait_for(qmix, k_pages, v_pages, gate);
  __syncthreads();
  // the head's mixed queries as A fragments: rows g and g + 8, k-step by k-step
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = g + (i & 1) * 8, c = ks * 16 + 2 * t + (i >> 1) * 8;
      qa[ks][i] = (active && r < nrows && c < kn)
                      ? *reinterpret_cast<const uint32_t*>(
                            qmix + (size_t)(row0 + r) * ld_qmix + (size_t)h * kn + c)
                      : 0u;
    }
  }
  float o[VT][4];
#pragma unroll
  for (int v = 0; v < VT; ++v)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[v][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int kvh = active ? h / (H / G) : 0;
  const bool wide = (dim % 8 == 0) && (vdim % 8 == 0);  // 16-byte copies
  // A token's keys and values are kc + vc pieces of 16 bytes. A warp copies the keys
  // warp, warp + 8, ... of a tile, a lane the pieces lane, lane + 32, ...: where a piece
  // lies in a page and in a stage does not depend on the tile, so it is worked out once.
  constexpr int MAX_PIECES = 6;  // (512 + 1024) / 8 / 32
  const int kc = kn / 8, vc = vn / 8;
  int piece_src[MAX_PIECES], piece_dst[MAX_PIECES];  // elements; src < 0: no such piece
#pragma unroll
  for (int i = 0; i < MAX_PIECES; ++i) {
    const int c = lane + 32 * i;
    const bool key = c < kc;
    const int e = (key ? c : c - kc) * 8;
    const int width = key ? dim : vdim, head = e / width, d = e % width;
    // bit 30 of the source marks a value piece; the row of the page's slot is added later
    piece_src[i] = c < kc + vc ? ((head * page_size) * width + d) | (key ? 0 : 1 << 30) : -1;
    piece_dst[i] = key ? e : MMA_KEYS * ldk + e;
  }
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

  int first = 0;
  while (first < nrows) {
    const int b = req_s[first];
    int last = first;
    if (b >= 0) {
      const int block = chunk > 0 ? pos_s[first] / chunk : 0;
      while (last + 1 < nrows && req_s[last + 1] == b &&
             (chunk > 0 ? pos_s[last + 1] / chunk : 0) == block &&
             pos_s[last + 1] == pos_s[last] + 1) {
        ++last;
      }
    }
    if (b >= 0) {
      const int c0 = chunk > 0 ? pos_s[first] - pos_s[first] % chunk : 0;
      const int p_last = pos_s[last];
      const int* table = block_table + (size_t)b * ld_table;
      // the segment's pages, fetched side by side; then the tiles of 32 keys travel into
      // two stages in turn (asynchronous 16-byte copies, zeros past the last position),
      // the next tile while this one is multiplied
      const int page0 = c0 / page_size, npages = p_last / page_size - page0 + 1;
      for (int i = tid; i < npages; i += MMA_HEADS * 32) pages_s[i] = table[page0 + i];
      __syncthreads();
      const int tiles = (p_last - c0) / MMA_KEYS + 1;
      auto issue = [&](int tile) {
        bf16* Kd = stages + (tile & 1) * stage_elems;
        bf16* Vd = Kd + MMA_KEYS * ldk;
        const int k0 = c0 + tile * MMA_KEYS;
        if (wide) {
#pragma unroll
          for (int jj = 0; jj < MMA_KEYS / MMA_HEADS; ++jj) {
            const int j = warp + MMA_HEADS * jj, at = k0 + j;
            const bool in = at <= p_last;
            const int index = page_shift >= 0 ? at >> page_shift : at / page_size;
            const int sl = at - index * page_size;
            const size_t page = in ? pages_s[index - page0] : 0;
            const bf16* k_row = k_pages + page * G * page_size * dim + (size_t)sl * dim;
            const bf16* v_row = v_pages + page * G * page_size * vdim + (size_t)sl * vdim;
            const int bytes = in ? 16 : 0;  // 0: the 16 bytes are filled with zeros
#pragma unroll
            for (int i = 0; i < MAX_PIECES; ++i) {
              if (piece_src[i] >= 0) {
                const bool value = (piece_src[i] >> 30) & 1;
                const bf16* src = (value ? v_row : k_row) + (piece_src[i] & ((1 << 30) - 1));
                const uint32_t dst = (uint32_t)__cvta_generic_to_shared(
                    Kd + (value ? j * ldv : j * ldk) + piece_dst[i]);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst),
                             "l"(src), "r"(bytes)
                             : "memory");
              }
            }
          }
        } else {
          for (int idx = tid; idx < MMA_KEYS * (kn + vn); idx += MMA_HEADS * 32) {
            const int j = idx / (kn + vn), c = idx % (kn + vn);
            const int at = k0 + j;
            const bool key = c < kn;
            const int e = key ? c : c - kn;
            bf16 value = __float2bfloat16_rn(0.f);
            if (at <= p_last) {
              const int page = pages_s[at / page_size - page0], sl = at % page_size;
              const int width = key ? dim : vdim, head = e / width, d = e % width;
              value = (key ? k_pages : v_pages)[(((size_t)page * G + head) * page_size + sl) *
                                                    width + d];
            }
            (key ? Kd + j * ldk : Vd + j * ldv)[e] = value;
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
      issue(0);
      for (int tile = 0; tile < tiles; ++tile) {
        const int k0 = c0 + tile * MMA_KEYS;
        if (tile + 1 < tiles) {
          issue(tile + 1);
          asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
          asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const bf16* Ks = stages + (tile & 1) * stage_elems;
        const bf16* Vs = Ks + MMA_KEYS * ldk;
        if (active) {
          float sc[MMA_KEYS / 8][4];
#pragma unroll
          for (int n = 0; n < MMA_KEYS / 8; ++n) {
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[n][i] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
              if (ks * 16 < kn) {
                const bf16* kb = Ks + (n * 8 + g) * ldk + ks * 16 + 2 * t;
                mma_bf16(sc[n], qa[ks], *reinterpret_cast<const uint32_t*>(kb),
                         *reinterpret_cast<const uint32_t*>(kb + 8));
              }
            }
          }
          // rows g (i = 0, 1) and g + 8 (i = 2, 3); key of column n * 8 + 2 t + (i & 1)
          float alpha[2];
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int r = g + 8 * half;
            const bool mine = r >= first && r <= last;
            const int reach = mine ? pos_s[r] : -1;
            float best = -INFINITY;
#pragma unroll
            for (int n = 0; n < MMA_KEYS / 8; ++n) {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int at = k0 + n * 8 + 2 * t + i;
                float& v = sc[n][2 * half + i];
                v = at <= reach ? v * 1.4426950408889634f : -INFINITY;  // (base 2 from here)
                best = fmaxf(best, v);
              }
            }
            best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 1));
            best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 2));
            const float m_new = fmaxf(m_run[half], best);
            alpha[half] = m_new == -INFINITY ? 1.f : exp2f(m_run[half] - m_new);
            float sum = 0.f;
#pragma unroll
            for (int n = 0; n < MMA_KEYS / 8; ++n) {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                float& v = sc[n][2 * half + i];
                v = m_new == -INFINITY ? 0.f : exp2f(v - m_new);
                sum += v;
              }
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[half] = l_run[half] * alpha[half] + sum;
            m_run[half] = m_new;
          }
#pragma unroll
          for (int v = 0; v < VT; ++v) {
            o[v][0] *= alpha[0];
            o[v][1] *= alpha[0];
            o[v][2] *= alpha[1];
            o[v][3] *= alpha[1];
          }
#pragma unroll
          for (int kk = 0; kk < MMA_KEYS / 16; ++kk) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // a0: row g, keys 2t..; a1: row g + 8; a2, a3: the same rows, keys + 8
              const float w0 = sc[2 * kk + (i >> 1)][2 * (i & 1)];
              const float w1 = sc[2 * kk + (i >> 1)][2 * (i & 1) + 1];
              const float h0 = __bfloat162float(__float2bfloat16_rn(w0));
              const float h1 = __bfloat162float(__float2bfloat16_rn(w1));
              hi[i] = pack_bf16(h0, h1);
              lo[i] = pack_bf16(w0 - h0, w1 - h1);
            }
#pragma unroll
            for (int v = 0; v < VT; ++v) {
              if (v * 8 < vdim) {
                const int col = kvh * vdim + v * 8 + g;
                const unsigned short* vb =
                    reinterpret_cast<const unsigned short*>(Vs) + (kk * 16 + 2 * t) * ldv + col;
                const uint32_t b0 = (uint32_t)vb[0] | ((uint32_t)vb[ldv] << 16);
                const uint32_t b1 = (uint32_t)vb[8 * ldv] | ((uint32_t)vb[9 * ldv] << 16);
                mma_bf16(o[v], hi, b0, b1);
                mma_bf16(o[v], lo, b0, b1);
              }
            }
          }
        }
        __syncthreads();  // the stage is filled again at the next turn
      }
    }
    first = last + 1;
  }
  if (!active) return;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    if (r >= nrows) continue;
    float factor = l_run[half] > 0.f ? 1.f / l_run[half] : 0.f;
    if (gate != nullptr) factor /= 1.f + expf(-gate[(size_t)(row0 + r) * ld_gate + h]);
    bf16* dst = out + (size_t)(row0 + r) * ld_out + (size_t)h * vdim;
#pragma unroll
    for (int v = 0; v < VT; ++v) {
      const int c = v * 8 + 2 * t;
      if (c < vdim) {  // (vdim is a multiple of 8 here: both columns are inside)
        *reinterpret_cast<uint32_t*>(dst + c) =
            pack_bf16(o[v][2 * half] * factor, o[v][2 * half + 1] * factor);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Steps of single rows on the tensor cores. With one query row per request, the rows of an
// m16n8k16 tile are sixteen *heads* of that row: one warp scores a tile of 16 keys for all of
// them at once, and the warps of a CTA share out the row's tiles (warp w takes tiles w,
// w + W, ...), each with a running maximum and sum of its own; the shares are merged through
// shared memory in warp order. Heads of different key/value heads want different values:
// per key/value head the weights of the other heads' rows are zeroed and the product added
// into the same accumulators. A CTA per (row, sixteen heads).
constexpr int DEC_KEYS = 16;

template <int KSTEPS, int VT>
__global__ void __launch_bounds__(256)
talking_decode_mma_kernel(const __nv_bfloat16* __restrict__ qmix, int ld_qmix,
                          const __nv_bfloat16* __restrict__ k_pages,
                          const __nv_bfloat16* __restrict__ v_pages,
                          const int* __restrict__ block_table, int ld_table,
                          const int* __restrict__ request_of_row,
                          const int* __restrict__ positions, const float* __restrict__ gate,
                          int ld_gate, __nv_bfloat16* __restrict__ out, int ld_out, int H, int G,
                          int dim, int vdim, int page_size, int chunk, int max_pages) {
  extern __shared__ __align__(16) unsigned char dec_smem[];
  using bf16 = __nv_bfloat16;
  const int kn = G * dim, vn = G * vdim;
  const int ldk = kn + 8, ldv = vn + 8;
  const int warps = blockDim.x >> 5;
  const int tile_elems = DEC_KEYS * (ldk + ldv);
  const int merge_floats = 16 * (8 * VT + 2);  // per warp: o [16][8 VT], maximum, sum
  bf16* tiles = reinterpret_cast<bf16*>(dec_smem);
  float* merge = reinterpret_cast<float*>(tiles + (size_t)warps * tile_elems);
  int* pages_s = reinterpret_cast<int*>(merge + (size_t)warps * merge_floats);
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int row = blockIdx.x, h0 = blockIdx.y * 16, heads = min(16, H - h0);
  const int b = request_of_row[row];
  if (b < 0) {  // a row of padding
    for (int i = tid; i < heads * vdim; i += blockDim.x) {
      out[(size_t)row * ld_out + (size_t)h0 * vdim + i] = __float2bfloat16_rn(0.f);
    }
    return;
  }
  const int position = positions[row];
  const int c0 = chunk > 0 ? position - position % chunk : 0;
  const int page0 = c0 / page_size, npages = min(position / page_size - page0 + 1, max_pages);
  const int* table = block_table + (size_t)b * ld_table;
  pdl_wait_for(qmix, k_pages, v_pages, gate);
  for (int i = tid; i < npages; i += blockDim.x) pages_s[i] = table[page0 + i];
  // the sixteen heads' mixed queries as A fragments: rows g and g + 8 are heads
  uint32_t qa[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = g + (i & 1) * 8, c = ks * 16 + 2 * t + (i >> 1) * 8;
      qa[ks][i] = (r < heads && c < kn)
                      ? *reinterpret_cast<const uint32_t*>(
                            qmix + (size_t)row * ld_qmix + (size_t)(h0 + r) * kn + c)
                      : 0u;
    }
  }
  float o[VT][4];
#pragma unroll
  for (int v = 0; v < VT; ++v)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[v][i] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int per = H / G;
  const int kv_of[2] = {(h0 + g) / per, (h0 + g + 8) / per};  // the rows' key/value heads
  const int kv_first = h0 / per, kv_last = (h0 + heads - 1) / per;
  const int kc = kn / 8, vc = vn / 8;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  // where a lane's 16-byte pieces of a token lie in a page and in the tile: worked out once
  constexpr int DEC_PIECES = 6;  // (512 + 1024) / 8 / 32
  int piece_src[DEC_PIECES], piece_dst[DEC_PIECES];  // elements; src < 0: no such piece
#pragma unroll
  for (int i = 0; i < DEC_PIECES; ++i) {
    const int c = lane + 32 * i;
    const bool key = c < kc;
    const int e = (key ? c : c - kc) * 8;
    const int width = key ? dim : vdim, head = e / width, d = e % width;
    piece_src[i] = c < kc + vc ? ((head * page_size) * width + d) | (key ? 0 : 1 << 30) : -1;
    piece_dst[i] = key ? e : DEC_KEYS * ldk + e;
  }
  bf16* Ks = tiles + (size_t)warp * tile_elems;
  bf16* Vs = Ks + DEC_KEYS * ldk;
  __syncthreads();
  const int ntiles = (position - c0) / DEC_KEYS + 1;
  for (int tile = warp; tile < ntiles; tile += warps) {
    const int k0 = c0 + tile * DEC_KEYS;
    __syncwarp();  // the warp has finished with the tile before
#pragma unroll 4
    for (int j = 0; j < DEC_KEYS; ++j) {
      const int at = k0 + j;
      const bool in = at <= position;
      const int index = page_shift >= 0 ? at >> page_shift : at / page_size;
      const int sl = at - index * page_size;
      const size_t page = in ? pages_s[min(index - page0, npages - 1)] : 0;
      const bf16* k_row = k_pages + page * G * page_size * dim + (size_t)sl * dim;
      const bf16* v_row = v_pages + page * G * page_size * vdim + (size_t)sl * vdim;
      const int bytes = in ? 16 : 0;  // 0: the 16 bytes are filled with zeros
#pragma unroll
      for (int i = 0; i < DEC_PIECES; ++i) {
        if (piece_src[i] >= 0) {
          const bool value = (piece_src[i] >> 30) & 1;
          const bf16* src = (value ? v_row : k_row) + (piece_src[i] & ((1 << 30) - 1));
          const uint32_t dst = (uint32_t)__cvta_generic_to_shared(
              Ks + (value ? j * ldv : j * ldk) + piece_dst[i]);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                       "r"(bytes)
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    float sc[DEC_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < DEC_KEYS / 8; ++n) {
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[n][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        if (ks * 16 < kn) {
          const bf16* kb = Ks + (n * 8 + g) * ldk + ks * 16 + 2 * t;
          mma_bf16(sc[n], qa[ks], *reinterpret_cast<const uint32_t*>(kb),
                   *reinterpret_cast<const uint32_t*>(kb + 8));
        }
      }
    }
    float alpha[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float best = -INFINITY;
#pragma unroll
      for (int n = 0; n < DEC_KEYS / 8; ++n) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int at = k0 + n * 8 + 2 * t + i;
          float& v = sc[n][2 * half + i];
          v = at <= position ? v * 1.4426950408889634f : -INFINITY;  // (base 2 from here)
          best = fmaxf(best, v);
        }
      }
      best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 1));
      best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, 2));
      const float m_new = fmaxf(m_run[half], best);  // (a tile holds a visible key: finite)
      alpha[half] = exp2f(m_run[half] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int n = 0; n < DEC_KEYS / 8; ++n) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          float& v = sc[n][2 * half + i];
          v = exp2f(v - m_new);
          sum += v;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[half] = l_run[half] * alpha[half] + sum;
      m_run[half] = m_new;
    }
#pragma unroll
    for (int v = 0; v < VT; ++v) {
      o[v][0] *= alpha[0];
      o[v][1] *= alpha[0];
      o[v][2] *= alpha[1];
      o[v][3] *= alpha[1];
    }
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float w0 = sc[i >> 1][2 * (i & 1)], w1 = sc[i >> 1][2 * (i & 1) + 1];
      const float x0 = __bfloat162float(__float2bfloat16_rn(w0));
      const float x1 = __bfloat162float(__float2bfloat16_rn(w1));
      hi[i] = pack_bf16(x0, x1);
      lo[i] = pack_bf16(w0 - x0, w1 - x1);
    }
    for (int kv = kv_first; kv <= kv_last; ++kv) {
      // rows (heads) of other key/value heads add nothing: their weights are zeroed
      uint32_t a_hi[4], a_lo[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool mine = kv_of[i & 1] == kv;
        a_hi[i] = mine ? hi[i] : 0u;
        a_lo[i] = mine ? lo[i] : 0u;
      }
#pragma unroll
      for (int v = 0; v < VT; ++v) {
        if (v * 8 < vdim) {
          const int col = kv * vdim + v * 8 + g;
          const unsigned short* vb =
              reinterpret_cast<const unsigned short*>(Vs) + (2 * t) * ldv + col;
          const uint32_t b0 = (uint32_t)vb[0] | ((uint32_t)vb[ldv] << 16);
          const uint32_t b1 = (uint32_t)vb[8 * ldv] | ((uint32_t)vb[9 * ldv] << 16);
          mma_bf16(o[v], a_hi, b0, b1);
          mma_bf16(o[v], a_lo, b0, b1);
        }
      }
    }
  }
  // every warp's share into its own rows of the merge area, then all threads merge
  float* mine = merge + (size_t)warp * merge_floats;
#pragma unroll
  for (int v = 0; v < VT; ++v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      mine[(g + (i >> 1) * 8) * (8 * VT + 2) + v * 8 + 2 * t + (i & 1)] = o[v][i];
    }
  }
  if (t == 0) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      mine[(g + 8 * half) * (8 * VT + 2) + 8 * VT] = m_run[half];
      mine[(g + 8 * half) * (8 * VT + 2) + 8 * VT + 1] = l_run[half];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < heads * vdim; idx += blockDim.x) {
    const int r = idx / vdim, c = idx - r * vdim;
    float best = -INFINITY;
    for (int w = 0; w < warps; ++w) {
      best = fmaxf(best, merge[(size_t)w * merge_floats + r * (8 * VT + 2) + 8 * VT]);
    }
    float total = 0.f, value = 0.f;
    for (int w = 0; w < warps; ++w) {  // in warp order, whatever the batch
      const float* part = merge + (size_t)w * merge_floats + r * (8 * VT + 2);
      const float m = part[8 * VT];
      const float weight = m == -INFINITY ? 0.f : exp2f(m - best);
      total = fmaf(part[8 * VT + 1], weight, total);
      value = fmaf(part[c], weight, value);
    }
    float factor = total > 0.f ? 1.f / total : 0.f;
    if (gate != nullptr) factor /= 1.f + expf(-gate[(size_t)row * ld_gate + h0 + r]);
    out[(size_t)row * ld_out + (size_t)(h0 + r) * vdim + c] = __float2bfloat16_rn(value * factor);
  }
}

template <typename K> inline void allow_large_smem(K kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

template <typename T>
int talking_prepare(const float* proj, int ld_proj, int k_off, int v_off, const float* bias,
                    const float* q_weight, const float* k_weight, float eps, const int* positions, const double* freq,
                    int rot_dims, int layout, const float* talk, const float* temp, float scale,
                    const int* slot_mapping, void* k_pages, void* v_pages, int page_size,
                    void* qmix, int ld_qmix, int rows, int H, int G, int dim, int vdim,
                    cudaStream_t stream) {
  const size_t smem = ((size_t)(H + G) * dim + 2 * ROPE_MAX_PAIRS + (size_t)H * H) * sizeof(float);
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

// `reach`: the most keys any row of the launch sees (bounds the shared memory of the CUDA-core
// kernel). `window_rows`: rows of the step per CTA of the tensor-core kernel, which serves
// bfloat16 when the sizes allow (1: a step of single rows; 16: prompt portions; 0: never).
AYK_API int ayk_talking_attention(const void* qmix, int ld_qmix, const void* k_pages,
                                  const void* v_pages, const int* block_table, int ld_table,
                                  const int* request_of_row, const int* positions,
                                  const float* gate, int ld_gate, void* out, int ld_out, int rows,
                                  int H, int G, int dim, int vdim, int page_size, int chunk,
                                  int window, int reach, int window_rows, int type,
                                  void* stream) {
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
  const int kn = G * dim;
  const size_t mma_smem = 2 * (size_t)MMA_KEYS * (kn + 8 + G * vdim + 8) * sizeof(__nv_bfloat16) +
                          ((size_t)reach / page_size + 2) * sizeof(int);
  if (type == 1 && window == 0 && window_rows >= 1 && window_rows <= 16 && kn % 16 == 0 &&
      kn <= 512 && vdim % 8 == 0 && vdim <= 128 && G * vdim <= 1024 &&
      mma_smem <= 200 * 1024 &&
      ld_qmix % 2 == 0 && ld_out % 2 == 0 && ((uintptr_t)qmix | (uintptr_t)out) % 4 == 0 &&
      ((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0) {
    if (window_rows == 1) {
      // steps of single rows: sixteen heads as a tile's rows, the warps share out the keys
      const size_t per_warp = (size_t)DEC_KEYS * (kn + 8 + G * vdim + 8) * sizeof(__nv_bfloat16);
      const int vt = vdim <= 64 ? 8 : 16;
      const size_t merge_bytes = (size_t)16 * (8 * vt + 2) * sizeof(float);
      const int max_pages = reach / page_size + 2;
      const int tiles = (reach + DEC_KEYS - 1) / DEC_KEYS + 1;
      int warps = 8;
      while (warps > 1 && (warps * (per_warp + merge_bytes) > 180 * 1024 || warps >= 2 * tiles)) {
        warps /= 2;
      }
      const size_t smem = warps * (per_warp + merge_bytes) + (size_t)max_pages * sizeof(int);
      const dim3 dec_grid(rows, (H + 15) / 16);
#define AYK_TALK_DEC(KS, VT)                                                                   \
  {                                                                                            \
    static const bool allowed = (allow_large_smem(talking_decode_mma_kernel<KS, VT>), true);   \
    (void)allowed;                                                                             \
    return launch_kernel(talking_decode_mma_kernel<KS, VT>, dec_grid, dim3(warps * 32), smem,  \
                         s, 1, (const __nv_bfloat16*)qmix, ld_qmix,                            \
                         (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,         \
                         block_table, ld_table, request_of_row, positions, gate, ld_gate,      \
                         (__nv_bfloat16*)out, ld_out, H, G, dim, vdim, page_size, chunk,       \
                         max_pages);                                                           \
  }
      if (smem <= 200 * 1024 && dim % 8 == 0) {
        if (kn <= 256 && vdim <= 64) AYK_TALK_DEC(16, 8);
        if (kn <= 256) AYK_TALK_DEC(16, 16);
        if (vdim <= 64) AYK_TALK_DEC(32, 8);
        AYK_TALK_DEC(32, 16);
      }
#undef AYK_TALK_DEC
    }
    const dim3 grid((rows + window_rows - 1) / window_rows, (H + MMA_HEADS - 1) / MMA_HEADS);
#define AYK_TALK_MMA(KS, VT)                                                                   \
  {                                                                                            \
    static const bool allowed = (allow_large_smem(talking_attention_mma_kernel<KS, VT>), true); \
    (void)allowed;                                                                             \
    return launch_kernel(talking_attention_mma_kernel<KS, VT>, grid, dim3(MMA_HEADS * 32),     \
                         mma_smem, s, 1, (const __nv_bfloat16*)qmix, ld_qmix,                  \
                         (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,         \
                         block_table, ld_table, request_of_row, positions, gate, ld_gate,      \
                         (__nv_bfloat16*)out, ld_out, rows, H, G, dim, vdim, page_size, chunk, \
                         window_rows);                                                         \
  }
    if (kn <= 128 && vdim <= 64) AYK_TALK_MMA(8, 8);
    if (kn <= 128) AYK_TALK_MMA(8, 16);
    if (kn <= 256 && vdim <= 64) AYK_TALK_MMA(16, 8);
    if (kn <= 256) AYK_TALK_MMA(16, 16);
    if (vdim <= 64) AYK_TALK_MMA(32, 8);
    AYK_TALK_MMA(32, 16);
#undef AYK_TALK_MMA
  }
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
