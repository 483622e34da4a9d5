// Softmax attention with capped scores and a sink for steps that bring portions of prompts: bfloat16, tensor cores.
//
// The same function as the capped kernel of attention_generic.cu (key rows of `dim`, value rows of `vdim` elements,
// score = cap * tanh(scale * <q, k> / cap) when cap > 0, a sink that adds one to the softmax's denominator, a window),
// tiled: a block takes 64 consecutive query positions of one request and one query head (four warps of 16 rows), and
// walks the keys its rows can see in tiles of 64, fetched from the paged cache by cp.async into a ring of two stages.
// Per tile: S = Q K^T by mma.sync m16n8k16 (bf16 in, fp32 out); scale, cap and mask in fp32 (scores are kept in units
// of log 2, so that every exponential is a power of two); running maximum and sum in fp32; P rounded to bfloat16 as
// the A operand of O += P V (the value fragments come transposed out of shared memory by ldmatrix).  The sink enters
// at the end as exp(s - maximum) in the denominator, s = 0 or the number the query head has learned (sink_values).
//
// Tiles of keys are counted from key 0 (or from the first key the block's rows can see under a window, rounded down
// to a multiple of 64), and a row's sums run over them in order, so without a window what a position gets does not
// depend on how its request was cut into steps.
//
// Which rows a block takes is found on the device: tile b of the grid is the b-th tile of 64 rows in request order (a
// request of n positions has ceil(n / 64) tiles); the grid holds an upper bound of tiles and the blocks beyond the
// last one return.
//
// Sizes: dim a multiple of 16 up to 256, vdim a multiple of 16 up to 128; any page size; any grouping of heads.
#include "common.cuh"

#define CA_ROWS 64
#define CA_KEYS 64
#define CA_THREADS 128
#define CA_PAD 8  // elements between rows of a tile in shared memory: row starts fall on different banks

__device__ __forceinline__ void ca_cp16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // zero bytes read: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ca_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void ca_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ca_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware unit (two units in the last place of fp32; -inf gives 0)
__device__ __forceinline__ float ca_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ unsigned ca_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// cap * tanh(x / cap) through tanh(y) = 1 - 2 / (2^(2 y log2 e) + 1): an absolute error of a few 1e-7 of the cap
__device__ __forceinline__ float ca_cap(float x, float cap, float two_log2e_over_cap) {
  const float e = ca_exp2(x * two_log2e_over_cap);
  return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}

template <int KMAX, int VMAX>
__global__ void __launch_bounds__(CA_THREADS)
capped_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, long long q_stride, __nv_bfloat16* __restrict__ out,
                            long long out_stride, const __nv_bfloat16* __restrict__ k_pages,
                            const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_table,
                            int table_stride, const int* __restrict__ query_start, const int* __restrict__ context_lens,
                            int num_seqs, int page_size, int num_heads, int num_kv_heads, int dim, int vdim, int window,
                            float scale, float softcap, int sink, const float* __restrict__ sink_values,
                            int* __restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int tile_info[2];
  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int head = blockIdx.y;
  const int kv_head = head / (num_heads / num_kv_heads);
  if (tid == 0) {
    int left = blockIdx.x, found = -1, first_row = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = query_start[s + 1] - query_start[s];
      const int tiles = (n + CA_ROWS - 1) / CA_ROWS;
      if (left < tiles) {
        found = s;
        first_row = left * CA_ROWS;
        break;
      }
      left -= tiles;
    }
    tile_info[0] = found;
    tile_info[1] = first_row;
  }
  __syncthreads();
  const int seq = tile_info[0];
  if (seq < 0) return;
  const int seq_begin = query_start[seq], seq_rows = query_start[seq + 1] - seq_begin;
  const int row0 = tile_info[1];
  const int rows = min(CA_ROWS, seq_rows - row0);
  const int token0 = seq_begin + row0;
  const int pos0 = context_lens[seq] - seq_rows + row0;  // position of the tile's first row
  const int pos_last = pos0 + rows - 1;
  const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int key_begin = (lo / CA_KEYS) * CA_KEYS;
  const int num_tiles = (pos_last - key_begin) / CA_KEYS + 1;
  const int* table = block_table + (size_t)seq * table_stride;

  const int k_ld = dim + CA_PAD, v_ld = vdim + CA_PAD;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [64][k_ld]
  __nv_bfloat16* k_s = q_s + CA_ROWS * k_ld;                          // [2][64][k_ld]
  __nv_bfloat16* v_s = k_s + 2 * CA_KEYS * k_ld;                      // [2][64][v_ld]

  // the queries of the tile, once
  {
    const int chunks = dim / 8;
    for (int i = tid; i < CA_ROWS * chunks; i += CA_THREADS) {
      const int r = i / chunks, c = i % chunks;
      const bool valid = r < rows;
      const __nv_bfloat16* src = q + (size_t)(token0 + (valid ? r : 0)) * q_stride + (size_t)head * dim + c * 8;
      ca_cp16(q_s + r * k_ld + c * 8, src, valid);
    }
  }
  // two threads bring a key's row and its value row: one page lookup and one address a thread and tile
  auto fetch = [&](int tile, int stage) {
    const int key0 = key_begin + tile * CA_KEYS;
    const int k_chunks = dim / 8, v_chunks = vdim / 8;
    const int r = tid >> 1, half = tid & 1;
    const int key = key0 + r;
    int page = -1;
    if (key <= pos_last) {
      page = table[key / page_size];
      if (page < 0 && key >= lo && status) atomicOr(status, 4);
    }
    const bool valid = page >= 0;
    const size_t slot = valid ? ((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head : 0;
    __nv_bfloat16* ks = k_s + (stage * CA_KEYS + r) * k_ld;
    __nv_bfloat16* vs = v_s + (stage * CA_KEYS + r) * v_ld;
    const __nv_bfloat16* k_src = k_pages + slot * dim;
    const __nv_bfloat16* v_src = v_pages + slot * vdim;
    for (int c = half; c < k_chunks; c += 2) ca_cp16(ks + c * 8, k_src + c * 8, valid);
    for (int c = half; c < v_chunks; c += 2) ca_cp16(vs + c * 8, v_src + c * 8, valid);
  };
  fetch(0, 0);
  ca_commit();

  float acc[VMAX][4];
  float top[2] = {-INFINITY, -INFINITY}, sum[2] = {0.0f, 0.0f};  // the maxima in units of log 2
#pragma unroll
  for (int i = 0; i < VMAX; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  const int k16 = dim / 16, v16 = vdim / 16;
  const float log2e = 1.44269504088896340736f;
  const float scale_log2 = scale * log2e;
  const float cap_log2 = softcap * log2e, cap_factor = softcap > 0.0f ? 2.0f * log2e / softcap : 0.0f;
  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  const int my_pos[2] = {pos0 + my_row[0], pos0 + my_row[1]};

  for (int tile = 0; tile < num_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < num_tiles) fetch(tile + 1, stage ^ 1);
    ca_commit();
    ca_wait<1>();
    __syncthreads();
    const __nv_bfloat16* ks = k_s + stage * CA_KEYS * k_ld;
    const __nv_bfloat16* vs = v_s + stage * CA_KEYS * v_ld;
    const int key0 = key_begin + tile * CA_KEYS;
    float s[CA_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < CA_KEYS / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < KMAX; ++kk) {
      if (kk < k16) {
        unsigned a[4];
        const __nv_bfloat16* qa = q_s + my_row[0] * k_ld + kk * 16 + 2 * t4;
        a[0] = *reinterpret_cast<const unsigned*>(qa);
        a[1] = *reinterpret_cast<const unsigned*>(qa + 8 * k_ld);
        a[2] = *reinterpret_cast<const unsigned*>(qa + 8);
        a[3] = *reinterpret_cast<const unsigned*>(qa + 8 * k_ld + 8);
#pragma unroll
        for (int n = 0; n < CA_KEYS / 8; n += 2) {
          // four 8 x 8 pieces of the key tile: keys n * 8 .. + 15, this step's 16 elements
          const int piece = lane >> 3;
          const __nv_bfloat16* src = ks + (n * 8 + (piece >> 1) * 8 + (lane & 7)) * k_ld + kk * 16 + (piece & 1) * 8;
          unsigned b0, b1, b2, b3;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(src);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "r"(addr));
          ca_mma(s[n], a, b0, b1);
          ca_mma(s[n + 1], a, b2, b3);
        }
      }
    }
    // scale and cap (in units of log 2), mask, running maximum and sum (rows g and g + 8 of the warp's 16); a tile
    // that every row of the block sees whole needs no mask
    float tile_top[2] = {-INFINITY, -INFINITY};
    const bool whole = key0 + CA_KEYS - 1 <= pos0 && (window <= 0 || pos0 + CA_ROWS - 1 - key0 < window);
#pragma unroll
    for (int n = 0; n < CA_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        float x = softcap > 0.0f ? ca_cap(s[n][e] * scale, cap_log2, cap_factor) : s[n][e] * scale_log2;
        if (!whole) {
          const int key = key0 + n * 8 + 2 * t4 + (e & 1);
          const bool seen = my_row[r] < rows && key <= my_pos[r] && (window <= 0 || my_pos[r] - key < window);
          if (!seen) x = -INFINITY;
        }
        s[n][e] = x;
        tile_top[r] = fmaxf(tile_top[r], x);
      }
    }
    float corr[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 1));
      tile_top[r] = fmaxf(tile_top[r], __shfl_xor_sync(0xffffffffu, tile_top[r], 2));
      const float next = fmaxf(top[r], tile_top[r]);
      base[r] = next == -INFINITY ? 0.0f : next;
      corr[r] = ca_exp2(top[r] == -INFINITY ? -INFINITY : top[r] - base[r]);
      top[r] = next;
    }
    float part[2] = {0.0f, 0.0f};
#pragma unroll
    for (int n = 0; n < CA_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = ca_exp2(s[n][e] - base[e >> 1]);
        s[n][e] = p;
        part[e >> 1] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) sum[r] = sum[r] * corr[r] + part[r];
    // the maxima seldom move after a row's first tiles: nothing to rescale then
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < VMAX; ++i) {
        acc[i][0] *= corr[0];
        acc[i][1] *= corr[0];
        acc[i][2] *= corr[1];
        acc[i][3] *= corr[1];
      }
    }
    // O += P V
#pragma unroll
    for (int kt = 0; kt < CA_KEYS / 16; ++kt) {
      unsigned a[4];
      a[0] = ca_pack(s[2 * kt][0], s[2 * kt][1]);
      a[1] = ca_pack(s[2 * kt][2], s[2 * kt][3]);
      a[2] = ca_pack(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      a[3] = ca_pack(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
      for (int vt = 0; vt < VMAX / 2; ++vt) {
        if (vt < v16) {
          const int matrix = lane >> 3;
          const __nv_bfloat16* src = vs + (kt * 16 + (matrix & 1) * 8 + (lane & 7)) * v_ld + vt * 16 + (matrix >> 1) * 8;
          unsigned b0, b1, b2, b3;
          const unsigned addr = (unsigned)__cvta_generic_to_shared(src);
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                       : "r"(addr));
          ca_mma(acc[2 * vt], a, b0, b1);
          ca_mma(acc[2 * vt + 1], a, b2, b3);
        }
      }
    }
    __syncthreads();  // the stage is free for the tile after next
  }
  ca_wait<0>();

  // the denominator (with the sink: one more key that scores 0, or what its head has learned, so exp(that - maximum)
  // more), and the rows
  const float sink_log2 = sink && sink_values ? sink_values[head] * 1.4426950408889634f : 0.0f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float total = sum[r];
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    if (sink) total = top[r] == -INFINITY ? 1.0f : total + ca_exp2(sink_log2 - top[r]);
    const float inv = total > 0.0f ? 1.0f / total : 0.0f;
    if (my_row[r] < rows) {
      __nv_bfloat16* dst = out + (size_t)(token0 + my_row[r]) * out_stride + (size_t)head * vdim + 2 * t4;
#pragma unroll
      for (int i = 0; i < VMAX; ++i) {
        if (i < 2 * v16) *reinterpret_cast<unsigned*>(dst + i * 8) = ca_pack(acc[i][2 * r] * inv, acc[i][2 * r + 1] * inv);
      }
    }
  }
}

template <int KMAX, int VMAX>
static int capped_attention_mma_launch(const void* q, long long q_stride, void* out, long long out_stride,
                                       const void* k_pages, const void* v_pages, const int* block_table, int table_stride,
                                       const int* query_start, const int* context_lens, int num_tokens, int num_seqs,
                                       int page_size, int num_heads, int num_kv_heads, int dim, int vdim, int window,
                                       float scale, float softcap, int sink, const float* sink_values, int* status,
                                       cudaStream_t stream) {
  const size_t smem = ((size_t)3 * CA_ROWS * (dim + CA_PAD) + (size_t)2 * CA_KEYS * (vdim + CA_PAD)) * sizeof(__nv_bfloat16);
  auto kernel = capped_attention_mma_kernel<KMAX, VMAX>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured = true;
  }
  const int tiles = (num_tokens + CA_ROWS - 1) / CA_ROWS + num_seqs;  // no request has more tiles than n / 64 + 1
  ts_launch(kernel, dim3(tiles, num_heads), dim3(CA_THREADS), smem, stream, (const __nv_bfloat16*)q, q_stride,
            (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table,
            table_stride, query_start, context_lens, num_seqs, page_size, num_heads, num_kv_heads, dim, vdim, window, scale,
            softcap, sink, sink_values, status);
  return ts_launch_status();
}

TS_EXPORT int ts_paged_attention_capped_mma(const void* q, long long q_stride, void* out, long long out_stride,
                                            const void* k_pages, const void* v_pages, const int* block_table,
                                            int table_stride, const int* query_start, const int* context_lens,
                                            int num_tokens, int num_seqs, int page_size, int num_heads, int num_kv_heads,
                                            int dim, int vdim, int window, float scale, float softcap, int sink,
                                            const float* sink_values, int* status, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (dim < 16 || dim % 16 || vdim < 16 || vdim % 16 || dim > 256 || vdim > 128) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads || num_heads > 65535) return TS_ERR_SIZE;
  if (page_size < 1 || window < 0 || !(scale > 0.0f) || softcap < 0.0f) return TS_ERR_ARGUMENT;
  if (q_stride % 8 || out_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
      ((uintptr_t)out & 3))
    return TS_ERR_ALIGN;
#define CA_CASE(K, V)                                                                                                  \
  return capped_attention_mma_launch<K, V>(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride, \
                                           query_start, context_lens, num_tokens, num_seqs, page_size, num_heads,     \
                                           num_kv_heads, dim, vdim, window, scale, softcap, sink, sink_values, status, stream)
  if (dim <= 64 && vdim <= 64) CA_CASE(4, 8);
  if (dim <= 128) CA_CASE(8, 16);
  CA_CASE(16, 16);
#undef CA_CASE
}
