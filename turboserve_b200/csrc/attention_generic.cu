// Paged attention for any dtype, head size and head grouping: the 32-bit path of the model
// and the fallback for sizes the tensor-core kernels refuse.
//
// One block per (query token, query head).  The query at absolute position p sees keys lo..p
// of its own sequence, lo = max(0, p - window + 1) (window == 0: lo = 0), read from the paged
// cache through the sequence's block table; the keys of this step have been appended before
// the kernel runs, so a token sees itself.  Keys are taken in tiles of 32 counted from lo and
// dealt to GENERIC_STREAMS = 16 streams: stream s takes tiles s, s + 16, ...; one lane scores
// one key, then the tile's values are accumulated with every lane owning head dims lane,
// lane + 32, ...  The sixteen partial results are merged in stream order.  The order of every
// sum is therefore a function of (lo, p) alone: the output of a token does not depend on how
// the sequence was cut into steps or on what else is in the batch.  How many warps work the
// streams does not change a bit either: a step of many tokens runs four warps a block, each
// four streams one after the other; a step of few tokens (decoding) sixteen warps, one each.
//
// Scores, softmax (natural exp, running maximum) and the value sum are fp32; the output is
// rounded once.  What it replaces in the reference: gather + mask + SDPA per sequence
// (src/turboserve/engine/model/attention.py:139-148,184-209) with scale = head_dim^-0.5
// (src/turboserve/engine/model/model_config.py:224-227).
#include "common.cuh"

#define GENERIC_STREAMS 16
#define MAX_DIMS_PER_LANE 8  // head_dim <= 256

// blockDim.x / 32 warps, a divisor of GENERIC_STREAMS
template <typename T>
__global__ void __launch_bounds__(GENERIC_STREAMS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                               long long out_stride, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int table_stride, const int* __restrict__ seq_of_token,
                               const int* __restrict__ positions, int page_size, int num_heads,
                               int num_kv_heads, int head_dim, int v_dim, int window, float scale,
                               float softcap, int sink, const float* __restrict__ sink_values,
                               int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  float* q_s = smem;                               // [head_dim]
  float* part_acc = smem + head_dim;               // [GENERIC_STREAMS][v_dim]
  float* part_ml = part_acc + GENERIC_STREAMS * v_dim;  // [GENERIC_STREAMS][2]

  const int t = blockIdx.x, head = blockIdx.y;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kv_head = head / (num_heads / num_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head * head_dim;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_keys = pos - lo + 1;
  const int num_tiles = (num_keys + 31) / 32;
  const bool wide = sizeof(T) == 4 && head_dim % 4 == 0 && !((uintptr_t)k_pages & 15);  // key rows are 16-byte aligned
  for (int stream = warp; stream < GENERIC_STREAMS; stream += num_warps) {
    float m = -INFINITY, l = 0.0f;
    float acc[MAX_DIMS_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] = 0.0f;
    for (int tile = stream; tile < num_tiles; tile += GENERIC_STREAMS) {
      const int key = lo + tile * 32 + lane;
      const bool valid = key <= pos;
      float s = -INFINITY;
      size_t row = 0;  // of the key's value
      if (valid) {
        const int page = table[key / page_size];
        if (page < 0) {
          if (status) atomicOr(status, 4);
        } else {
          const size_t place = ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head;
          row = place * v_dim;
          const T* k_row = k_pages + place * head_dim;
          float dot = 0.0f;
          if (wide) {  // the same products in the same order, four to a load
            const float4* k4 = reinterpret_cast<const float4*>(k_row);
            for (int i = 0; i < head_dim / 4; ++i) {
              const float4 kv = k4[i];
              dot = fmaf(q_s[4 * i], kv.x, dot);
              dot = fmaf(q_s[4 * i + 1], kv.y, dot);
              dot = fmaf(q_s[4 * i + 2], kv.z, dot);
              dot = fmaf(q_s[4 * i + 3], kv.w, dot);
            }
          } else {
            for (int i = 0; i < head_dim; ++i) dot = fmaf(q_s[i], to_float(k_row[i]), dot);
          }
          s = dot * scale;
          if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
        }
      }
      const float tile_max = warp_max(s);
      const float m_new = fmaxf(m, tile_max);
      if (m_new == -INFINITY) continue;  // only unreadable keys so far
      const float corr = expf(m - m_new);
      const float p = s == -INFINITY ? 0.0f : expf(s - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] *= corr;
      m = m_new;
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
      for (int j = 0; j < in_tile; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, j);
        if (pj == 0.0f) continue;
        const T* v_row = v_pages + rj;
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
          const int dim = lane + 32 * i;
          if (dim < v_dim) acc[i] = fmaf(pj, to_float(v_row[dim]), acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
      const int dim = lane + 32 * i;
      if (dim < v_dim) part_acc[stream * v_dim + dim] = acc[i];
    }
    if (lane == 0) {
      part_ml[stream * 2] = m;
      part_ml[stream * 2 + 1] = l;
    }
  }
  __syncthreads();
  if (warp == 0) {
    float m_all = -INFINITY;
    for (int w = 0; w < GENERIC_STREAMS; ++w) m_all = fmaxf(m_all, part_ml[w * 2]);
    float weight[GENERIC_STREAMS];
    float l_all = 0.0f;
    if (sink) {  // a key whose value is nothing: it only adds to the denominator; its score is 0 or the head's own
      const float s0 = sink_values ? sink_values[head] : 0.0f;
      m_all = fmaxf(m_all, s0);
      l_all = expf(s0 - m_all);
    }
    for (int w = 0; w < GENERIC_STREAMS; ++w) {
      const float mw = part_ml[w * 2];
      weight[w] = mw == -INFINITY ? 0.0f : expf(mw - m_all);
      l_all += part_ml[w * 2 + 1] * weight[w];
    }
    const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
    T* o_row = out + (size_t)t * out_stride + (size_t)head * v_dim;
    for (int dim = lane; dim < v_dim; dim += 32) {
      float v = 0.0f;
      for (int w = 0; w < GENERIC_STREAMS; ++w) v += part_acc[w * v_dim + dim] * weight[w];
      o_row[dim] = from_float<T>(v * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same, one block per (query token, key head): the QH query heads that share a key head are
// scored against every key row and accumulate every value row together, so a step that decodes
// reads its keys and values once, 16 bytes at a time where the rows are 16-byte aligned.  Sixteen
// warps, one per stream; a tile's weights go through a small buffer in shared memory from the lanes
// that scored the keys to all lanes for the value sum.  Streams are merged by one warp per head.
// Every sum has the order of the kernel above, so both give the same bits.
// ---------------------------------------------------------------------------------------------
#define GROUP_MAX_PER_LANE 4  // v_dim <= 128

template <typename T> struct RowVec;
template <> struct RowVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct RowVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

template <typename T, int QH>
__global__ void __launch_bounds__(GENERIC_STREAMS * 32)
paged_attention_group_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
                             const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                             const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_of_token,
                             const int* __restrict__ positions, int page_size, int num_kv_heads, int head_dim, int v_dim,
                             int window, float scale, float softcap, int sink, const float* __restrict__ sink_values,
                             int vector_rows, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float smem[];
  float* q_s = smem;                                               // [QH][head_dim]
  float* part_acc = q_s + QH * head_dim;                           // [GENERIC_STREAMS][QH][v_dim]
  float* part_ml = part_acc + GENERIC_STREAMS * QH * v_dim;        // [GENERIC_STREAMS][QH][2]
  float* weights = part_ml + GENERIC_STREAMS * QH * 2;             // [GENERIC_STREAMS][32][QH]
  unsigned long long* rows_s = reinterpret_cast<unsigned long long*>(weights + GENERIC_STREAMS * 32 * QH);  // [GENERIC_STREAMS][32]

  const int t = blockIdx.x, kv_head = blockIdx.y;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;
  const T* q_row = q + (size_t)t * q_stride + (size_t)kv_head * QH * head_dim;
  for (int i = threadIdx.x; i < QH * head_dim; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_tiles = (pos - lo + 32) / 32;
  const int stream = warp;
  float* my_weights = weights + stream * 32 * QH;
  unsigned long long* my_rows = rows_s + stream * 32;
  float top[QH], sum[QH];
  float acc[QH][GROUP_MAX_PER_LANE];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    top[h] = -INFINITY;
    sum[h] = 0.0f;
#pragma unroll
    for (int i = 0; i < GROUP_MAX_PER_LANE; ++i) acc[h][i] = 0.0f;
  }
  for (int tile = stream; tile < num_tiles; tile += GENERIC_STREAMS) {
    const int key = lo + tile * 32 + lane;
    float d[QH];
#pragma unroll
    for (int h = 0; h < QH; ++h) d[h] = 0.0f;
    bool readable = false;
    size_t v_row = 0;
    if (key <= pos) {
      const int page = table[key / page_size];
      if (page < 0) {
        if (status) atomicOr(status, 4);
      } else {
        readable = true;
        const size_t place = ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head;
        v_row = place * v_dim;
        const T* k_row = k_pages + place * head_dim;
        if (vector_rows) {
          constexpr int W = RowVec<T>::N;
#pragma unroll 4
          for (int i = 0; i < head_dim; i += W) {
            float kv[W];
            RowVec<T>::load(k_row + i, kv);
#pragma unroll
            for (int h = 0; h < QH; ++h) {
              const float* qh = q_s + h * head_dim + i;
              float total = d[h];
#pragma unroll
              for (int e = 0; e < W; ++e) total = fmaf(qh[e], kv[e], total);
              d[h] = total;
            }
          }
        } else {
          for (int i = 0; i < head_dim; ++i) {
            const float kv = to_float(k_row[i]);
#pragma unroll
            for (int h = 0; h < QH; ++h) d[h] = fmaf(q_s[h * head_dim + i], kv, d[h]);
          }
        }
      }
    }
    bool any = false;
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      float sc = -INFINITY;
      if (readable) {
        sc = d[h] * scale;
        if (softcap > 0.0f) sc = softcap * tanhf(sc / softcap);
      }
      const float next = fmaxf(top[h], warp_max(sc));
      float p = 0.0f, corr = 1.0f;
      if (next != -INFINITY) {
        any = true;
        corr = expf(top[h] - next);
        p = sc == -INFINITY ? 0.0f : expf(sc - next);
        sum[h] = sum[h] * corr + warp_sum(p);
        top[h] = next;
      }
#pragma unroll
      for (int i = 0; i < GROUP_MAX_PER_LANE; ++i) acc[h][i] *= corr;
      my_weights[lane * QH + h] = p;
    }
    my_rows[lane] = (unsigned long long)v_row;
    __syncwarp();
    if (any) {
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
#pragma unroll 4
      for (int j = 0; j < in_tile; ++j) {
        const T* v = v_pages + my_rows[j];
        float x[GROUP_MAX_PER_LANE];
#pragma unroll
        for (int i = 0; i < GROUP_MAX_PER_LANE; ++i) {
          const int e = lane + 32 * i;
          x[i] = e < v_dim ? to_float(v[e]) : 0.0f;
        }
        const float* w = my_weights + j * QH;
#pragma unroll
        for (int h = 0; h < QH; ++h) {
          const float wh = w[h];
#pragma unroll
          for (int i = 0; i < GROUP_MAX_PER_LANE; ++i) acc[h][i] = fmaf(wh, x[i], acc[h][i]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int h = 0; h < QH; ++h) {
#pragma unroll
    for (int i = 0; i < GROUP_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < v_dim) part_acc[(stream * QH + h) * v_dim + e] = acc[h][i];
    }
    if (lane == 0) {
      part_ml[(stream * QH + h) * 2] = top[h];
      part_ml[(stream * QH + h) * 2 + 1] = sum[h];
    }
  }
  __syncthreads();
  if (warp < QH) {
    const int h = warp;
    float m_all = -INFINITY;
    for (int w = 0; w < GENERIC_STREAMS; ++w) m_all = fmaxf(m_all, part_ml[(w * QH + h) * 2]);
    float weight[GENERIC_STREAMS];
    float l_all = 0.0f;
    if (sink) {
      const float s0 = sink_values ? sink_values[kv_head * QH + h] : 0.0f;
      m_all = fmaxf(m_all, s0);
      l_all = expf(s0 - m_all);
    }
    for (int w = 0; w < GENERIC_STREAMS; ++w) {
      const float mw = part_ml[(w * QH + h) * 2];
      weight[w] = mw == -INFINITY ? 0.0f : expf(mw - m_all);
      l_all += part_ml[(w * QH + h) * 2 + 1] * weight[w];
    }
    const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
    T* o_row = out + (size_t)t * out_stride + (size_t)(kv_head * QH + h) * v_dim;
    for (int dim = lane; dim < v_dim; dim += 32) {
      float v = 0.0f;
      for (int w = 0; w < GENERIC_STREAMS; ++w) v += part_acc[(w * QH + h) * v_dim + dim] * weight[w];
      o_row[dim] = from_float<T>(v * inv);
    }
  }
}

template <typename T, int QH>
static int paged_attention_group_launch(const void* q, long long q_stride, void* out, long long out_stride,
                                        const void* k_pages, const void* v_pages, const int* block_table,
                                        int table_stride, const int* seq_of_token, const int* positions, int num_tokens,
                                        int page_size, int num_kv_heads, int head_dim, int v_dim, int window, float scale,
                                        float softcap, int sink, const float* sink_values, int* status, cudaStream_t stream) {
  const size_t floats = (size_t)QH * head_dim + (size_t)GENERIC_STREAMS * QH * v_dim + (size_t)GENERIC_STREAMS * QH * 2 +
                        (size_t)GENERIC_STREAMS * 32 * QH;
  const size_t smem = floats * sizeof(float) + (size_t)GENERIC_STREAMS * 32 * sizeof(unsigned long long);
  if (smem > 200 * 1024) return TS_ERR_SIZE;
  auto kernel = paged_attention_group_kernel<T, QH>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int vector_rows = (head_dim * sizeof(T)) % 16 == 0 && !((uintptr_t)k_pages & 15);
  ts_launch(kernel, dim3(num_tokens, num_kv_heads), dim3(GENERIC_STREAMS * 32), smem, stream, (const T*)q, q_stride, (T*)out,
            out_stride, (const T*)k_pages, (const T*)v_pages, block_table, table_stride, seq_of_token, positions, page_size,
            num_kv_heads, head_dim, v_dim, window, scale, softcap, sink, sink_values, vector_rows, status);
  return ts_launch_status();
}

// The kernel with every option: value rows of their own width (v_dim), scores capped as
// softcap * tanh(score / softcap) (softcap 0: as they are), and a sink (sink != 0: the softmax's
// denominator holds one more term, as if one more key had no value; it scores 0, or, with sink_values,
// the number its query head has learned: exp(sink_values[head]), neither scaled nor capped).
TS_EXPORT int ts_paged_attention_capped(int dtype, const void* q, long long q_stride, void* out,
                                        long long out_stride, const void* k_pages,
                                        const void* v_pages, const int* block_table,
                                        int table_stride, const int* seq_of_token,
                                        const int* positions, int num_tokens, int page_size,
                                        int num_heads, int num_kv_heads, int head_dim, int v_dim, int window,
                                        float scale, float softcap, int sink, const float* sink_values, int* status,
                                        cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (head_dim < 1 || head_dim > 32 * MAX_DIMS_PER_LANE || v_dim < 1 || v_dim > 32 * MAX_DIMS_PER_LANE) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TS_ERR_SIZE;
  if (num_heads > 65535 || page_size < 1 || window < 0 || softcap < 0.0f) return TS_ERR_ARGUMENT;
  const int per_group = num_heads / num_kv_heads;
  // a step of few tokens (decoding): the heads of a key head together, keys and values read once
  if ((long long)num_tokens * num_heads <= 2048 && per_group <= 8 && v_dim <= 32 * GROUP_MAX_PER_LANE && num_kv_heads <= 65535 &&
      (dtype == TS_F32 || dtype == TS_BF16)) {
#define GROUP_CASE(HEADS)                                                                                               \
  case HEADS:                                                                                                           \
    return dtype == TS_F32                                                                                              \
               ? paged_attention_group_launch<float, HEADS>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, \
                                                            table_stride, seq_of_token, positions, num_tokens, page_size, \
                                                            num_kv_heads, head_dim, v_dim, window, scale, softcap, sink, \
                                                            sink_values, status, stream)                                              \
               : paged_attention_group_launch<__nv_bfloat16, HEADS>(q, q_stride, out, out_stride, k_pages, v_pages,     \
                                                                    block_table, table_stride, seq_of_token, positions, \
                                                                    num_tokens, page_size, num_kv_heads, head_dim, v_dim, \
                                                                    window, scale, softcap, sink, sink_values, status, stream)
    switch (per_group) {
      GROUP_CASE(1); GROUP_CASE(2); GROUP_CASE(3); GROUP_CASE(4); GROUP_CASE(5); GROUP_CASE(6); GROUP_CASE(7); GROUP_CASE(8);
    }
#undef GROUP_CASE
  }
  dim3 grid(num_tokens, num_heads);
  const size_t smem = ((size_t)head_dim + (size_t)v_dim * GENERIC_STREAMS + 2 * GENERIC_STREAMS) * sizeof(float);
  // few blocks (a decode step): a warp per stream; many: four warps, four streams each
  const int threads = (long long)num_tokens * num_heads <= 2048 ? GENERIC_STREAMS * 32 : 4 * 32;
  if (dtype == TS_F32)
    ts_launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(threads), smem, stream, 
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pages,
        (const float*)v_pages, block_table, table_stride, seq_of_token, positions, page_size,
        num_heads, num_kv_heads, head_dim, v_dim, window, scale, softcap, sink, sink_values, status);
  else if (dtype == TS_BF16)
    ts_launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, table_stride,
        seq_of_token, positions, page_size, num_heads, num_kv_heads, head_dim, v_dim, window, scale,
        softcap, sink, sink_values, status);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

TS_EXPORT int ts_paged_attention_generic(int dtype, const void* q, long long q_stride, void* out,
                                         long long out_stride, const void* k_pages,
                                         const void* v_pages, const int* block_table,
                                         int table_stride, const int* seq_of_token,
                                         const int* positions, int num_tokens, int page_size,
                                         int num_heads, int num_kv_heads, int head_dim, int window,
                                         float scale, int* status, cudaStream_t stream) {
  return ts_paged_attention_capped(dtype, q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                                   seq_of_token, positions, num_tokens, page_size, num_heads, num_kv_heads, head_dim,
                                   head_dim, window, scale, 0.0f, 0, nullptr, status, stream);
}
