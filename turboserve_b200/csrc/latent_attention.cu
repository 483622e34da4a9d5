// Latent attention: every position keeps one row [latent c: rank | shared rotated key part: rot]
// in the paged cache, and all query heads attend over those rows.
//
// A head's key is W_uk c and its value W_uv c.  Neither is ever formed: with
// q~ = W_uk^T q_plain (rank numbers per head and token) the score of key j is
// (q~ . c_j + q_rot . r_j) * scale, and the head's output is W_uv (sum_j p_j c_j).  So the step is
//
//   latent_prepare    RMS norm of the new tokens' latent (fp32, with its weight), rotation of the shared key
//                     part and of every head's rotated query part (fp32 angles, cos and sin times a
//                     constant), append of [c | r] to the request's pages
//   head_linear       out[t, h, :] = W[h] in[t, h, :] for all heads in one launch (q_plain -> q~, and
//                     sum p c -> the head's value), fp32 accumulation; optionally times sigmoid(gate[t, h])
//   latent_attention  softmax attention of every (token, head) over the cached rows of its window; the
//                     value of a key is the first `rank` elements of its row
//   latent_gather     the rows of a range of positions of one request, from its pages into one matrix
//   latent_softmax    the softmax of a matrix of scores under the causal mask and the window (fp32 in,
//                     the weights rounded to the type of the value product out)
//
// The last two serve long portions of prompts in bfloat16: there the scores of a stretch of queries (all heads)
// against the rows they can see, and the weighted sums of the latents, are two matrix products of the library
// (bfloat16 operands, fp32 accumulation, the scores kept in fp32), with latent_softmax between them.
//
// latent_attention scores G heads of a token in one block so that a key row is read once for all of
// them.  Keys are taken in tiles of 32 counted from the window's first key and dealt to 16 streams
// whose partial results are merged in stream order (as attention_generic.cu does): the order of every
// sum depends on (first key, position) alone, never on how a request was cut into steps or batched.
// Scores, softmax and the sums are fp32; outputs are rounded once.
#include "common.cuh"

#define LA_STREAMS 16

// ---------------------------------------------------------------------------------------
// latent_prepare: one block per token.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_prepare_kernel(T* __restrict__ q, long long q_stride, const T* __restrict__ down,
                                      long long down_stride, const float* __restrict__ norm_weight,
                                      const float* __restrict__ inv_freq, float amplitude,
                                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                      const int* __restrict__ block_table, int table_stride, T* __restrict__ pages,
                                      int page_size, int heads, int dim, int rot, int rank, float eps,
                                      T* __restrict__ packed, long long packed_stride, int* __restrict__ status) {
  extern __shared__ __align__(16) float la_smem[];  // cos[rot / 2], sin[rot / 2]
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int half = rot / 2;
  float* cos_s = la_smem;
  float* sin_s = la_smem + half;
  pdl_wait();
  pdl_trigger<64>();
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cos_s[i] = c * amplitude;
    sin_s[i] = s * amplitude;
  }
  __syncthreads();
  T* q_row = q + (size_t)t * q_stride;
  for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    T* part = q_row + (size_t)h * (dim + rot) + dim;
    const float u = to_float(part[i]), v = to_float(part[i + half]);
    const T a = from_float<T>(u * cos_s[i] - v * sin_s[i]), b = from_float<T>(v * cos_s[i] + u * sin_s[i]);
    part[i] = a;
    part[i + half] = b;
    if (packed) {  // the query rows attention reads: per head [rank carried | rot rotated]
      T* to = packed + (size_t)t * packed_stride + (size_t)h * (rank + rot) + rank;
      to[i] = a;
      to[i + half] = b;
    }
  }
  if (!down) return;
  const T* d_row = down + (size_t)t * down_stride;
  float sum_sq = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float x = to_float(d_row[i]);
    sum_sq = fmaf(x, x, sum_sq);
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)rank + eps);
  const int page = block_table[(size_t)seq * table_stride + pos / page_size];
  if (page < 0) {
    if (threadIdx.x == 0 && status) atomicOr(status, 2);
    return;
  }
  T* row = pages + ((size_t)page * page_size + pos % page_size) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) row[i] = from_float<T>(to_float(d_row[i]) * inv * norm_weight[i]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = to_float(d_row[rank + i]), v = to_float(d_row[rank + i + half]);
    row[rank + i] = from_float<T>(u * cos_s[i] - v * sin_s[i]);
    row[rank + i + half] = from_float<T>(v * cos_s[i] + u * sin_s[i]);
  }
}

TS_EXPORT int ts_latent_prepare(int dtype, void* q, long long q_stride, const void* down, long long down_stride,
                                const float* norm_weight, const float* inv_freq, float amplitude,
                                const int* positions, const int* seq_of_token, const int* block_table,
                                int table_stride, void* pages, int page_size, int num_tokens, int heads, int dim,
                                int rot, int rank, float eps, void* packed, long long packed_stride, int* status,
                                cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rot < 0 || rot % 2 || heads < 1 || dim < 0 || rank < 1 || page_size < 1) return TS_ERR_SIZE;
  if (down && (!norm_weight || !pages)) return TS_ERR_ARGUMENT;
  const size_t smem = (size_t)rot * sizeof(float);
  if (dtype == TS_F32)
    ts_launch(latent_prepare_kernel<float>, dim3(num_tokens), dim3(128), smem, stream, (float*)q, q_stride,
              (const float*)down, down_stride, norm_weight, inv_freq, amplitude, positions, seq_of_token, block_table,
              table_stride, (float*)pages, page_size, heads, dim, rot, rank, eps, (float*)packed, packed_stride, status);
  else if (dtype == TS_BF16)
    ts_launch(latent_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), smem, stream, (__nv_bfloat16*)q,
              q_stride, (const __nv_bfloat16*)down, down_stride, norm_weight, inv_freq, amplitude, positions,
              seq_of_token, block_table, table_stride, (__nv_bfloat16*)pages, page_size, heads, dim, rot, rank, eps,
              (__nv_bfloat16*)packed, packed_stride, status);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// head_linear: out[t, h * out_head + n] = sum_k in[t, h * in_head + k] * w[h][n][k], n < N, k < K.
// A 64 x 64 tile of one head per block, 16-wide K steps through shared memory, a 4 x 4 micro-tile a
// thread; every output adds its products in increasing k, so a row does not depend on the others.
// ---------------------------------------------------------------------------------------
#define HL_M 64
#define HL_N 64
#define HL_K 16

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ in, long long in_stride, int in_head, const T* __restrict__ w,
                   T* __restrict__ out, long long out_stride, int out_head, int m, int n, int k,
                   const T* __restrict__ gate, long long gate_stride) {
  pdl_wait();
  pdl_trigger();
  __shared__ float a_s[HL_K][HL_M + 4];
  __shared__ float w_s[HL_K][HL_N + 4];
  const int tid = threadIdx.x, head = blockIdx.z;
  const int tile_m = blockIdx.y * HL_M, tile_n = blockIdx.x * HL_N;
  const int tx = tid % 16, ty = tid / 16;
  const T* a = in + (size_t)head * in_head;
  const T* wh = w + (size_t)head * n * k;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  const int load_row = tid / 4, load_col = (tid % 4) * 4;
  for (int k0 = 0; k0 < k; k0 += HL_K) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + load_col + e;
      const int am = tile_m + load_row, wn = tile_n + load_row;
      a_s[load_col + e][load_row] = (am < m && kk < k) ? to_float(a[(size_t)am * in_stride + kk]) : 0.0f;
      w_s[load_col + e][load_row] = (wn < n && kk < k) ? to_float(wh[(size_t)wn * k + kk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_K; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_s[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_s[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = tile_m + ty * 4 + i;
    if (row >= m) continue;
    // a gate per (row, head): the head's outputs times the sigmoid of one number, in fp32 before the rounding
    const float open = gate ? 1.0f / (1.0f + expf(-to_float(gate[(size_t)row * gate_stride + head]))) : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tile_n + tx * 4 + j;
      if (col < n) out[(size_t)row * out_stride + (size_t)head * out_head + col] = from_float<T>(acc[i][j] * open);
    }
  }
}

TS_EXPORT int ts_head_linear(int dtype, const void* in, long long in_stride, int in_head, const void* w, void* out,
                             long long out_stride, int out_head, int m, int heads, int n, int k,
                             const void* gate, long long gate_stride, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || heads <= 0) return 0;
  if (k < 0 || heads > 65535 || (m + HL_M - 1) / HL_M > 65535) return TS_ERR_SIZE;
  dim3 grid((n + HL_N - 1) / HL_N, (m + HL_M - 1) / HL_M, heads);
  if (dtype == TS_F32)
    ts_launch(head_linear_kernel<float>, grid, dim3(256), 0, stream, (const float*)in, in_stride, in_head,
              (const float*)w, (float*)out, out_stride, out_head, m, n, k, (const float*)gate, gate_stride);
  else if (dtype == TS_BF16)
    ts_launch(head_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)in, in_stride,
              in_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, out_head, m, n, k,
              (const __nv_bfloat16*)gate, gate_stride);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// latent_attention: one block per (token, group of G heads).
// q rows are [heads][rank + rot] (the query carried into the latent space, then its rotated part); out rows [heads][rank].
// NR = ceil(rank / 32) value elements a lane, an even number.
// ---------------------------------------------------------------------------------------
template <typename T> struct LaVec;
template <> struct LaVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct LaVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ void la_load2(const float* p, float& a, float& b) {
  const float2 v = *reinterpret_cast<const float2*>(p);
  a = v.x;
  b = v.y;
}
__device__ __forceinline__ void la_load2(const __nv_bfloat16* p, float& a, float& b) {
  const unsigned v = *reinterpret_cast<const unsigned*>(p);
  a = __uint_as_float(v << 16);
  b = __uint_as_float(v & 0xffff0000u);
}

template <typename T, int G, int NR>
__global__ void __launch_bounds__(LA_STREAMS * 32)
latent_attention_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                        const T* __restrict__ pages, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions, int page_size,
                        int rank, int rot, int window, float scale, int vector_ok, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger<8>();
  extern __shared__ __align__(16) float la_smem[];
  const int width = rank + rot;
  float* q_s = la_smem;                                   // [G][width]
  float* part_acc = q_s + G * width;                      // [LA_STREAMS][G][rank]
  float* part_ml = part_acc + LA_STREAMS * G * rank;      // [LA_STREAMS][G][2]

  const int t = blockIdx.x, head0 = blockIdx.y * G;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head0 * width;
  for (int i = threadIdx.x; i < G * width; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_tiles = (pos - lo + 1 + 31) / 32;
  const bool pair_ok = rank % 2 == 0 && width % 2 == 0 && !((uintptr_t)pages & 7);  // two value elements a load
  for (int stream = warp; stream < LA_STREAMS; stream += num_warps) {
    float m[G], l[G], acc[G][NR];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.0f;
#pragma unroll
      for (int i = 0; i < NR; ++i) acc[g][i] = 0.0f;
    }
    for (int tile = stream; tile < num_tiles; tile += LA_STREAMS) {
      const int key = lo + tile * 32 + lane;
      bool valid = key <= pos;
      size_t row = 0;
      float s[G];
#pragma unroll
      for (int g = 0; g < G; ++g) s[g] = 0.0f;
      if (valid) {
        const int page = table[key / page_size];
        if (page < 0) {
          if (status) atomicOr(status, 4);
          valid = false;
        } else {
          row = ((size_t)page * page_size + key % page_size) * width;
          const T* k_row = pages + row;
          if (vector_ok) {
            constexpr int V = LaVec<T>::N;
#pragma unroll 4
            for (int i = 0; i < width; i += V) {  // a lane walks its own row: neighbouring loads share a 32-byte sector
              float kv[V];
              LaVec<T>::load(k_row + i, kv);
#pragma unroll
              for (int g = 0; g < G; ++g) {
                const float4* q4 = reinterpret_cast<const float4*>(q_s + g * width + i);  // one 16-byte broadcast for four products
#pragma unroll
                for (int j = 0; j < V / 4; ++j) {
                  const float4 qv = q4[j];
                  s[g] = fmaf(qv.x, kv[4 * j], s[g]);
                  s[g] = fmaf(qv.y, kv[4 * j + 1], s[g]);
                  s[g] = fmaf(qv.z, kv[4 * j + 2], s[g]);
                  s[g] = fmaf(qv.w, kv[4 * j + 3], s[g]);
                }
              }
            }
          } else {
            for (int i = 0; i < width; ++i) {
              const float kv = to_float(k_row[i]);
#pragma unroll
              for (int g = 0; g < G; ++g) s[g] = fmaf(q_s[g * width + i], kv, s[g]);
            }
          }
        }
      }
      float p[G];
      bool any = false;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float sg = valid ? s[g] * scale : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(sg));
        if (m_new == -INFINITY) {
          p[g] = 0.0f;
          continue;
        }
        any = true;
        const float corr = expf(m[g] - m_new);
        p[g] = valid ? expf(sg - m_new) : 0.0f;
        l[g] = l[g] * corr + warp_sum(p[g]);
#pragma unroll
        for (int i = 0; i < NR; ++i) acc[g][i] *= corr;
        m[g] = m_new;
      }
      if (!any) continue;
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
      for (int j = 0; j < in_tile; ++j) {
        const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, j);
        const int ok = __shfl_sync(0xffffffffu, (int)valid, j);
        float pj[G];
#pragma unroll
        for (int g = 0; g < G; ++g) pj[g] = __shfl_sync(0xffffffffu, p[g], j);
        if (!ok) continue;
        const T* v_row = pages + rj;
#pragma unroll
        for (int i = 0; i < NR; i += 2) {  // a lane owns the value elements 2 * lane + 64 * (i / 2) and the one after
          const int d = 2 * lane + 32 * i;
          if (d >= rank) continue;
          float v0, v1 = 0.0f;
          if (pair_ok) {
            la_load2(v_row + d, v0, v1);
          } else {
            v0 = to_float(v_row[d]);
            if (d + 1 < rank) v1 = to_float(v_row[d + 1]);
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            acc[g][i] = fmaf(pj[g], v0, acc[g][i]);
            acc[g][i + 1] = fmaf(pj[g], v1, acc[g][i + 1]);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int i = 0; i < NR; i += 2) {
        const int d = 2 * lane + 32 * i;
        if (d < rank) part_acc[((size_t)stream * G + g) * rank + d] = acc[g][i];
        if (d + 1 < rank) part_acc[((size_t)stream * G + g) * rank + d + 1] = acc[g][i + 1];
      }
      if (lane == 0) {
        part_ml[(stream * G + g) * 2] = m[g];
        part_ml[(stream * G + g) * 2 + 1] = l[g];
      }
    }
  }
  __syncthreads();
  // merge the streams in stream order: warp w takes heads w, w + num_warps, ...
  for (int g = warp; g < G; g += num_warps) {
    float m_all = -INFINITY;
    for (int w = 0; w < LA_STREAMS; ++w) m_all = fmaxf(m_all, part_ml[(w * G + g) * 2]);
    float weight[LA_STREAMS];
    float l_all = 0.0f;
    for (int w = 0; w < LA_STREAMS; ++w) {
      const float mw = part_ml[(w * G + g) * 2];
      weight[w] = mw == -INFINITY ? 0.0f : expf(mw - m_all);
      l_all += part_ml[(w * G + g) * 2 + 1] * weight[w];
    }
    const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
    T* o_row = out + (size_t)t * out_stride + (size_t)(head0 + g) * rank;
    for (int d = lane; d < rank; d += 32) {
      float v = 0.0f;
      for (int w = 0; w < LA_STREAMS; ++w) v += part_acc[((size_t)w * G + g) * rank + d] * weight[w];
      o_row[d] = from_float<T>(v * inv);
    }
  }
}

template <typename T, int G, int NR>
static int launch_latent_attention(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* pages, const int* block_table, int table_stride,
                                   const int* seq_of_token, const int* positions, int num_tokens, int page_size,
                                   int heads, int rank, int rot, int window, float scale, int* status,
                                   cudaStream_t stream) {
  const int width = rank + rot;
  const size_t smem = ((size_t)G * width + (size_t)LA_STREAMS * G * rank + 2 * LA_STREAMS * G) * sizeof(float);
  if (smem > 200 * 1024) return TS_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attention_kernel<T, G, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int vector_ok = width % LaVec<T>::N == 0 && !((uintptr_t)pages & 15);
  const int threads = (long long)num_tokens * (heads / G) <= 2048 ? LA_STREAMS * 32 : 4 * 32;
  ts_launch(latent_attention_kernel<T, G, NR>, dim3(num_tokens, heads / G), dim3(threads), smem, stream, (const T*)q,
            q_stride, (T*)out, out_stride, (const T*)pages, block_table, table_stride, seq_of_token, positions,
            page_size, rank, rot, window, scale, vector_ok, status);
  return ts_launch_status();
}

template <typename T, int NR>
static int latent_attention_by_group(int group, const void* q, long long q_stride, void* out, long long out_stride,
                                     const void* pages, const int* block_table, int table_stride,
                                     const int* seq_of_token, const int* positions, int num_tokens, int page_size,
                                     int heads, int rank, int rot, int window, float scale, int* status,
                                     cudaStream_t stream) {
#define LA_CASE(GV)                                                                                               \
  if constexpr (GV * NR <= 64)                                                                                    \
    if (group == GV)                                                                                              \
      return launch_latent_attention<T, GV, NR>(q, q_stride, out, out_stride, pages, block_table, table_stride,  \
                                                seq_of_token, positions, num_tokens, page_size, heads, rank, rot, \
                                                window, scale, status, stream);
  LA_CASE(8)
  LA_CASE(4)
  LA_CASE(2)
  LA_CASE(1)
#undef LA_CASE
  return TS_ERR_SIZE;
}

// The most heads a block takes together for this rank (accumulators: G * ceil(rank / 32) <= 64 a lane).
TS_EXPORT int ts_latent_attention_group(int heads, int rank) {
  const int nr = rank <= 64 ? 2 : rank <= 128 ? 4 : rank <= 256 ? 8 : rank <= 512 ? 16 : 32;
  for (int g = 8; g > 1; g >>= 1)
    if (heads % g == 0 && g * nr <= 64) return g;
  return 1;
}

TS_EXPORT int ts_latent_attention(int dtype, const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* pages, const int* block_table, int table_stride,
                                  const int* seq_of_token, const int* positions, int num_tokens, int page_size,
                                  int heads, int rank, int rot, int window, float scale, int* status,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rank < 1 || rank > 1024 || rot < 0 || heads < 1 || page_size < 1 || window < 0) return TS_ERR_SIZE;
  if (heads > 65535) return TS_ERR_SIZE;
  if (dtype != TS_F32 && dtype != TS_BF16) return TS_ERR_DTYPE;
  const int group = ts_latent_attention_group(heads, rank);
#define LA_RANK(NRV)                                                                                                  \
  return dtype == TS_F32                                                                                              \
             ? latent_attention_by_group<float, NRV>(group, q, q_stride, out, out_stride, pages, block_table,         \
                                                     table_stride, seq_of_token, positions, num_tokens, page_size,    \
                                                     heads, rank, rot, window, scale, status, stream)                 \
             : latent_attention_by_group<__nv_bfloat16, NRV>(group, q, q_stride, out, out_stride, pages, block_table, \
                                                             table_stride, seq_of_token, positions, num_tokens,       \
                                                             page_size, heads, rank, rot, window, scale, status,      \
                                                             stream);
  if (rank <= 64) { LA_RANK(2) }
  if (rank <= 128) { LA_RANK(4) }
  if (rank <= 256) { LA_RANK(8) }
  if (rank <= 512) { LA_RANK(16) }
  LA_RANK(32)
#undef LA_RANK
}

// ---------------------------------------------------------------------------------------
// latent_gather: rows[j] = the cached row of position first + j of request seq, j < count; rows count .. padded - 1
// are zeroed (the matrix products that follow take a multiple of eight rows).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pages, const int* __restrict__ table, int page_size, int width,
                                     int first, int count, T* __restrict__ rows, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger<1>();
  const int j = blockIdx.x;
  T* to = rows + (size_t)j * width;
  int page = -1;
  if (j < count) {
    page = table[(first + j) / page_size];
    if (page < 0 && threadIdx.x == 0 && status) atomicOr(status, 4);
  }
  if (page < 0) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from_float<T>(0.0f);
    return;
  }
  const T* from = pages + ((size_t)page * page_size + (first + j) % page_size) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from[i];
}

TS_EXPORT int ts_latent_gather(int dtype, const void* pages, const int* table, int page_size, int width, int first,
                               int count, int padded, void* rows, int* status, cudaStream_t stream) {
  if (padded <= 0) return 0;
  if (count > padded || first < 0 || page_size < 1 || width < 1) return TS_ERR_ARGUMENT;
  if (dtype == TS_F32)
    ts_launch(latent_gather_kernel<float>, dim3(padded), dim3(128), 0, stream, (const float*)pages, table, page_size, width,
              first, count, (float*)rows, status);
  else if (dtype == TS_BF16)
    ts_launch(latent_gather_kernel<__nv_bfloat16>, dim3(padded), dim3(128), 0, stream, (const __nv_bfloat16*)pages, table,
              page_size, width, first, count, (__nv_bfloat16*)rows, status);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// latent_softmax: scores [rows][ld] fp32, row r belongs to the query at position first_query + r / heads; column j is
// the key at position first_key + j.  A query at p sees the keys p - window < key <= p (window 0: every key <= p).
// weights[r][j] = exp(scale * s - max) / sum over the seen keys, 0 elsewhere (all ld columns are written).
// One block per row; the sums are fp32 in a fixed order.
// ---------------------------------------------------------------------------------------
#define LS_HELD 16  // a row of up to 2,048 scores is held in registers

template <typename T>
__global__ void __launch_bounds__(128)
latent_softmax_kernel(const float* __restrict__ scores, T* __restrict__ weights, int ld, int heads, int num_keys,
                      int first_query, int first_key, int window, float scale) {
  __shared__ float scratch[33];
  __shared__ float red_max[4];
  pdl_wait();
  pdl_trigger<1>();
  const int r = blockIdx.x;
  const int pos = first_query + r / heads;
  int lo = (window > 0 ? max(0, pos - window + 1) : 0) - first_key;
  int hi = pos - first_key;  // inclusive
  lo = max(lo, 0);
  hi = min(hi, num_keys - 1);
  const float* s = scores + (size_t)r * ld;
  T* w = weights + (size_t)r * ld;
  if (ld <= 128 * LS_HELD) {
    // the row is read once and held: element j of a thread is column threadIdx.x + 128 * j
    float held[LS_HELD];
    float biggest = -INFINITY;
#pragma unroll
    for (int j = 0; j < LS_HELD; ++j) {
      const int c = threadIdx.x + 128 * j;
      held[j] = (c >= lo && c <= hi) ? s[c] * scale : -INFINITY;
      biggest = fmaxf(biggest, held[j]);
    }
    biggest = warp_max(biggest);
    if ((threadIdx.x & 31) == 0) red_max[threadIdx.x >> 5] = biggest;
    __syncthreads();
    biggest = fmaxf(fmaxf(red_max[0], red_max[1]), fmaxf(red_max[2], red_max[3]));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < LS_HELD; ++j) {
      held[j] = held[j] == -INFINITY ? 0.0f : expf(held[j] - biggest);
      sum += held[j];
    }
    const float total = block_sum(sum, scratch);
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
#pragma unroll
    for (int j = 0; j < LS_HELD; ++j) {
      const int c = threadIdx.x + 128 * j;
      if (c < ld) w[c] = from_float<T>(held[j] * inv);
    }
    return;
  }
  float biggest = -INFINITY;
  for (int j = lo + threadIdx.x; j <= hi; j += blockDim.x) biggest = fmaxf(biggest, s[j] * scale);
  biggest = warp_max(biggest);
  if ((threadIdx.x & 31) == 0) red_max[threadIdx.x >> 5] = biggest;
  __syncthreads();
  biggest = fmaxf(fmaxf(red_max[0], red_max[1]), fmaxf(red_max[2], red_max[3]));
  float sum = 0.0f;
  for (int j = lo + threadIdx.x; j <= hi; j += blockDim.x) sum += expf(s[j] * scale - biggest);
  const float total = block_sum(sum, scratch);
  const float inv = total > 0.0f ? 1.0f / total : 0.0f;
  for (int j = threadIdx.x; j < ld; j += blockDim.x)
    w[j] = from_float<T>(j >= lo && j <= hi ? expf(s[j] * scale - biggest) * inv : 0.0f);
}

TS_EXPORT int ts_latent_softmax(int dtype, const float* scores, void* weights, int rows, int ld, int heads, int num_keys,
                                int first_query, int first_key, int window, float scale, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (ld < num_keys || heads < 1 || window < 0) return TS_ERR_ARGUMENT;
  if (dtype == TS_F32)
    ts_launch(latent_softmax_kernel<float>, dim3(rows), dim3(128), 0, stream, scores, (float*)weights, ld, heads, num_keys,
              first_query, first_key, window, scale);
  else if (dtype == TS_BF16)
    ts_launch(latent_softmax_kernel<__nv_bfloat16>, dim3(rows), dim3(128), 0, stream, scores, (__nv_bfloat16*)weights, ld, heads,
              num_keys, first_query, first_key, window, scale);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
