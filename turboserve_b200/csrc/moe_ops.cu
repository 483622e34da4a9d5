// Mixture of experts: the router, and the experts' products for steps of few tokens and of many.
//
//   moe_route      per token: logits z = W_r h in fp32 (W_r is kept in fp32), s = softmax(z) over all experts
//                  (or, mode bit 0, s = sigmoid(z), every expert on its own),
//                  experts in `groups` equal groups of neighbours of which only the `keep` groups with the
//                  largest maximum may be chosen from, the `top` largest allowed scores, and their weights
//                  s / (sum of the chosen s + 1e-20) (or, mode bit 1, the chosen s as they are).  Ties go to
//                  the lower index.
//   A weight may stand on the expert's OUTPUT (the kernels that add the experts' rows up take `weights`) or on its
//   INPUT, expert(w h) (the kernels that make gate and up take `in_weights`: gate (w h) = w (gate h), so the factor
//   enters in fp32 on the sums, before the rounding and the activation; the adding kernels then get no weights).
//   Few tokens (every request brings one): no sorting, every (token, chosen expert) pair streams its expert's rows
//     moe_pair_gate_up   hidden[pair, f] = act(gate_e[f] . h) * (up_e[f] . h), a warp per feature
//     moe_pair_down      out[t] = sum_k weight_k * (down_{e_k} hidden[t, k]) (+ addend[t]), a warp per output,
//                        the k-th expert's term added k-th, fp32, rounded once
//   Some tokens (a decode step of a batch): the pairs are put in expert order by one block, and a block per
//   (expert, tile of features) streams that expert's rows once for up to eight of its tokens at a time
//     moe_expert_rows    rows[first_e + i] = f(W_e a_i): gated (act(gate) * up, from the tokens' inputs gathered
//                        through the order) or plain (the down projection of the rows before), fp32 sums
//   Many tokens: the pairs are put in expert order so that every expert's rows are one matrix product
//     moe_count / moe_offsets / moe_place   how many pairs each expert has, where its rows start, and the
//                                           row of every pair (atomic counters: which row a pair gets within its
//                                           expert varies, what is computed for it does not)
//     moe_gather     rows of the input in that order
//     moe_combine    out[t] = sum_k weight_k * rows[place[t, k]] (+ addend[t]) in fp32, k-th term k-th
#include "common.cuh"

#define MOE_MAX_TOP 32

template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ router, int width, int experts,
                 int top, int groups, int keep, int mode, int* __restrict__ chosen, float* __restrict__ weights) {
  extern __shared__ float mr_smem[];
  float* h = mr_smem;            // [width]
  float* score = h + width;      // [experts]
  float* group_best = score + experts;  // [groups]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  const T* row = x + (size_t)t * x_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) h[i] = to_float(row[i]);
  __syncthreads();
  for (int e = warp; e < experts; e += warps) {
    const float* w = router + (size_t)e * width;
    float dot = 0.0f;
    for (int i = lane; i < width; i += 32) dot = fmaf(w[i], h[i], dot);
    dot = warp_sum(dot);
    if (lane == 0) score[e] = dot;
  }
  __syncthreads();
  if (warp != 0) return;
  if (mode & 1) {  // every expert's score on its own
    for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
  } else {  // softmax over all experts
    float biggest = -INFINITY;
    for (int e = lane; e < experts; e += 32) biggest = fmaxf(biggest, score[e]);
    biggest = warp_max(biggest);
    float total = 0.0f;
    for (int e = lane; e < experts; e += 32) total += expf(score[e] - biggest);
    total = warp_sum(total);
    for (int e = lane; e < experts; e += 32) score[e] = expf(score[e] - biggest) / total;
  }
  __syncwarp();
  const int per_group = experts / groups;
  if (groups > 1 && keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per_group; e < (g + 1) * per_group; ++e) best = fmaxf(best, score[e]);
      group_best[g] = best;
    }
    __syncwarp();
    if (lane == 0) {
      // `keep` times: the best group not yet kept is marked by the value 2 (scores never exceed 1)
      for (int round = 0; round < keep; ++round) {
        int arg = -1;
        float best = -INFINITY;
        for (int g = 0; g < groups; ++g)
          if (group_best[g] <= 1.5f && group_best[g] > best) {
            best = group_best[g];
            arg = g;
          }
        if (arg < 0) break;
        group_best[arg] = 2.0f;  // scores are probabilities (<= 1): 2 marks "kept"
      }
    }
    __syncwarp();
  } else {
    for (int g = lane; g < groups; g += 32) group_best[g] = 2.0f;
    __syncwarp();
  }
  if (lane == 0) {
    int picked[MOE_MAX_TOP];
    float picked_score[MOE_MAX_TOP];
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      int arg = -1;
      float best = -INFINITY;
      for (int e = 0; e < experts; ++e) {
        if (group_best[e / per_group] != 2.0f) continue;
        bool taken = false;
        for (int j = 0; j < k; ++j) taken |= picked[j] == e;
        if (!taken && score[e] > best) {
          best = score[e];
          arg = e;
        }
      }
      if (arg < 0) {  // fewer allowed experts than top: the remaining places carry no weight
        arg = k ? picked[0] : 0;
        best = 0.0f;
      }
      picked[k] = arg;
      picked_score[k] = best;
      sum += best;
    }
    for (int k = 0; k < top; ++k) {
      chosen[(size_t)t * top + k] = picked[k];
      weights[(size_t)t * top + k] = (mode & 2) ? picked_score[k] : picked_score[k] / (sum + 1e-20f);
    }
  }
}

TS_EXPORT int ts_moe_route(int dtype, const void* x, long long x_stride, const float* router, int num_tokens,
                           int width, int experts, int top, int groups, int keep, int mode, int* chosen, float* weights,
                           cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (experts < 1 || top < 1 || top > MOE_MAX_TOP || top > experts || groups < 1 || experts % groups || keep < 1 ||
      keep > groups)
    return TS_ERR_SIZE;
  const size_t smem = ((size_t)width + experts + groups) * sizeof(float);
  if (smem > 200 * 1024) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_route_kernel<float>, dim3(num_tokens), dim3(128), smem, stream, (const float*)x, x_stride, router, width,
              experts, top, groups, keep, mode, chosen, weights);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_route_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), smem, stream, (const __nv_bfloat16*)x, x_stride,
              router, width, experts, top, groups, keep, mode, chosen, weights);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// Steps of few tokens.
// ---------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float row_dot(const T* __restrict__ w, const float* __restrict__ h, int n, int lane);
template <> __device__ __forceinline__ float row_dot<float>(const float* __restrict__ w, const float* __restrict__ h, int n, int lane) {
  float dot = 0.0f;
  if (n % 4 == 0 && !((uintptr_t)w & 15)) {
    for (int i = lane * 4; i < n; i += 128) {
      const float4 a = *reinterpret_cast<const float4*>(w + i);
      dot = fmaf(a.x, h[i], dot); dot = fmaf(a.y, h[i + 1], dot); dot = fmaf(a.z, h[i + 2], dot); dot = fmaf(a.w, h[i + 3], dot);
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(w[i], h[i], dot);
  }
  return warp_sum(dot);
}
template <> __device__ __forceinline__ float row_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ h, int n, int lane) {
  float dot = 0.0f;
  if (n % 8 == 0 && !((uintptr_t)w & 15)) {
#pragma unroll 8
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 a = *reinterpret_cast<const uint4*>(w + i);
      const unsigned p[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        dot = fmaf(__uint_as_float(p[j] << 16), h[i + 2 * j], dot);
        dot = fmaf(__uint_as_float(p[j] & 0xffff0000u), h[i + 2 * j + 1], dot);
      }
    }
  } else {
    for (int i = lane; i < n; i += 32) dot = fmaf(__bfloat162float(w[i]), h[i], dot);
  }
  return warp_sum(dot);
}

#define MOE_FEATURES_PER_BLOCK 32

// gate_up: [experts][2 * ff][width], an expert's gate rows first, then its up rows.
template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_gate_up_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ gate_up,
                        const int* __restrict__ chosen, const float* __restrict__ in_weights, T* __restrict__ hidden,
                        int width, int ff, int top, int act) {
  extern __shared__ float mp_smem[];  // [width]
  const int pair = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  const T* row = x + (size_t)(pair / top) * x_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) mp_smem[i] = to_float(row[i]);
  __syncthreads();
  const int expert = chosen[pair];
  const float scale_in = in_weights ? in_weights[pair] : 1.0f;
  const T* base = gate_up + (size_t)expert * 2 * ff * width;
  const int f_end = min(ff, (int)(blockIdx.y + 1) * MOE_FEATURES_PER_BLOCK);
  for (int f = blockIdx.y * MOE_FEATURES_PER_BLOCK + warp; f < f_end; f += warps) {
    // gate and up are rounded to the activation type first, as a product that writes them would
    const float g = to_float(from_float<T>(scale_in * row_dot<T>(base + (size_t)f * width, mp_smem, width, lane)));
    const float u = to_float(from_float<T>(scale_in * row_dot<T>(base + (size_t)(ff + f) * width, mp_smem, width, lane)));
    if (lane == 0) hidden[(size_t)pair * ff + f] = from_float<T>(activation(g, act) * u);
  }
}

TS_EXPORT int ts_moe_pair_gate_up(int dtype, const void* x, long long x_stride, const void* gate_up, const int* chosen,
                                  const float* in_weights, void* hidden, int num_tokens, int width, int ff, int top, int act,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024 || ff < 1 || top < 1) return TS_ERR_SIZE;
  dim3 grid(num_tokens * top, (ff + MOE_FEATURES_PER_BLOCK - 1) / MOE_FEATURES_PER_BLOCK);
  if (grid.y > 65535) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_pair_gate_up_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_gate_up_kernel<float>, grid, dim3(256), smem, stream, (const float*)x, x_stride, (const float*)gate_up,
              chosen, in_weights, (float*)hidden, width, ff, top, act);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_pair_gate_up_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)x, x_stride,
              (const __nv_bfloat16*)gate_up, chosen, in_weights, (__nv_bfloat16*)hidden, width, ff, top, act);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// down: [experts][width][ff].
template <typename T>
__global__ void __launch_bounds__(256)
moe_pair_down_kernel(const T* __restrict__ hidden, const T* __restrict__ down, const int* __restrict__ chosen,
                     const float* __restrict__ weights, const T* __restrict__ addend, T* __restrict__ out, int width,
                     int ff, int top) {
  extern __shared__ float mp_smem[];  // [top][ff]
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  for (int i = threadIdx.x; i < top * ff; i += blockDim.x) mp_smem[i] = to_float(hidden[(size_t)t * top * ff + i]);
  __syncthreads();
  const int o_end = min(width, (int)(blockIdx.y + 1) * MOE_FEATURES_PER_BLOCK);
  for (int o = blockIdx.y * MOE_FEATURES_PER_BLOCK + warp; o < o_end; o += warps) {
    float sum = 0.0f;
    for (int k = 0; k < top; ++k) {
      const int expert = chosen[(size_t)t * top + k];
      const float part = row_dot<T>(down + ((size_t)expert * width + o) * ff, mp_smem + (size_t)k * ff, ff, lane);
      sum = fmaf(weights ? weights[(size_t)t * top + k] : 1.0f, to_float(from_float<T>(part)), sum);
    }
    if (lane == 0) {
      if (addend) sum += to_float(addend[(size_t)t * width + o]);
      out[(size_t)t * width + o] = from_float<T>(sum);
    }
  }
}

TS_EXPORT int ts_moe_pair_down(int dtype, const void* hidden, const void* down, const int* chosen, const float* weights,
                               const void* addend, void* out, int num_tokens, int width, int ff, int top,
                               cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const size_t smem = (size_t)top * ff * sizeof(float);
  if (smem > 200 * 1024 || ff < 1 || top < 1) return TS_ERR_SIZE;
  dim3 grid(num_tokens, (width + MOE_FEATURES_PER_BLOCK - 1) / MOE_FEATURES_PER_BLOCK);
  if (grid.y > 65535) return TS_ERR_SIZE;
  if (dtype == TS_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_pair_down_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_down_kernel<float>, grid, dim3(256), smem, stream, (const float*)hidden, (const float*)down, chosen,
              weights, (const float*)addend, (float*)out, width, ff, top);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_pair_down_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(moe_pair_down_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, (const __nv_bfloat16*)hidden,
              (const __nv_bfloat16*)down, chosen, weights, (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, width, ff, top);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// Steps of many tokens: pairs in expert order.
// counters: [experts] counts, then [experts + 1] offsets, then [experts] cursors (int32).
// ---------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counters) {
  pdl_wait();
  pdl_trigger<1>();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < pairs) atomicAdd(counters + chosen[i], 1);
}

__global__ void moe_offsets_kernel(int experts, int* __restrict__ counters) {
  pdl_wait();
  pdl_trigger<1>();
  if (threadIdx.x != 0) return;
  int* offsets = counters + experts;
  int* cursors = offsets + experts + 1;
  int total = 0;
  for (int e = 0; e < experts; ++e) {
    offsets[e] = total;
    cursors[e] = 0;
    total += counters[e];
  }
  offsets[experts] = total;
}

__global__ void moe_place_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counters,
                                 int* __restrict__ place, int* __restrict__ pair_of_row) {
  pdl_wait();
  pdl_trigger<1>();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = chosen[i];
  const int row = counters[experts + e] + atomicAdd(counters + 2 * experts + 1 + e, 1);
  place[i] = row;
  pair_of_row[row] = i;
}

// One block puts up to MOE_SORT_SMALL pairs in expert order (counts, first rows and cursors in shared memory).
#define MOE_SORT_SMALL 4096
__global__ void __launch_bounds__(256)
moe_sort_small_kernel(const int* __restrict__ chosen, int pairs, int experts, int* __restrict__ counters,
                      int* __restrict__ place, int* __restrict__ pair_of_row) {
  extern __shared__ int ms_smem[];  // counts[experts], first[experts + 1], cursor[experts]
  int* counts = ms_smem;
  int* first = counts + experts;
  int* cursor = first + experts + 1;
  pdl_wait();
  pdl_trigger<1>();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = cursor[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(counts + chosen[i], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int total = 0;
    for (int e = 0; e < experts; ++e) {
      first[e] = total;
      total += counts[e];
    }
    first[experts] = total;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counters[e] = counts[e];
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) counters[experts + e] = first[e];
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = chosen[i];
    const int row = first[e] + atomicAdd(cursor + e, 1);
    place[i] = row;
    pair_of_row[row] = i;
  }
}

// ---------------------------------------------------------------------------------------
// moe_expert_rows: block (expert e, tile of output features).  The expert's rows (first_e .. first_e + count_e - 1 in
// expert order) are taken eight at a time into shared memory; a warp per output feature reads that feature's weights
// once and forms its sum with each of the eight rows.  GATED: weights [experts][2 * n_out][k] (gate rows, then up
// rows), out = act(gate . a) * (up . a), the inputs gathered from x through pair_of_row / top.  Else: weights
// [experts][n_out][k], inputs are the rows of `in` in expert order.
// ---------------------------------------------------------------------------------------
#define ME_ROWS 8

template <typename T> struct MeVec;
template <> struct MeVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct MeVec<__nv_bfloat16> {
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

// The sums of one weight row (TWO: of two, a gate row and its up row) with the eight rows in shared memory.
template <typename T, bool TWO>
__device__ __forceinline__ void me_dots(const T* __restrict__ w, const T* __restrict__ w2, const T* __restrict__ rows_s, int k,
                                        int lane, bool vector_ok, float* acc, float* acc2) {
#pragma unroll
  for (int r = 0; r < ME_ROWS; ++r) acc[r] = acc2[r] = 0.0f;
  if (vector_ok) {
    constexpr int V = MeVec<T>::N;
#pragma unroll 2
    for (int i = lane * V; i < k; i += 32 * V) {
      float wv[V], wv2[V];
      MeVec<T>::load(w + i, wv);
      if (TWO) MeVec<T>::load(w2 + i, wv2);
#pragma unroll
      for (int r = 0; r < ME_ROWS; ++r) {
        float av[V];
        MeVec<T>::load(rows_s + (size_t)r * k + i, av);
#pragma unroll
        for (int j = 0; j < V; ++j) {
          acc[r] = fmaf(wv[j], av[j], acc[r]);
          if (TWO) acc2[r] = fmaf(wv2[j], av[j], acc2[r]);
        }
      }
    }
  } else {
    for (int i = lane; i < k; i += 32) {
      const float wv = to_float(w[i]);
      const float wv2 = TWO ? to_float(w2[i]) : 0.0f;
#pragma unroll
      for (int r = 0; r < ME_ROWS; ++r) {
        const float av = to_float(rows_s[(size_t)r * k + i]);
        acc[r] = fmaf(wv, av, acc[r]);
        if (TWO) acc2[r] = fmaf(wv2, av, acc2[r]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < ME_ROWS; ++r) {
    acc[r] = warp_sum(acc[r]);
    if (TWO) acc2[r] = warp_sum(acc2[r]);
  }
}

#define ME_FEATURES_PER_BLOCK 16

template <typename T, bool GATED>
__global__ void __launch_bounds__(256)
moe_expert_rows_kernel(const T* __restrict__ in, long long in_stride, const T* __restrict__ weights,
                       const int* __restrict__ counters, const int* __restrict__ pair_of_row, T* __restrict__ out, int k,
                       int n_out, int top, int experts, int act, const float* __restrict__ in_weights) {
  extern __shared__ __align__(16) unsigned char me_smem[];
  T* rows_s = reinterpret_cast<T*>(me_smem);  // [ME_ROWS][k]
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger<1>();
  const int count = counters[e], first = counters[experts + e];
  if (count == 0) return;
  const T* w = weights + (size_t)e * (GATED ? 2 : 1) * n_out * k;
  const bool vector_ok = k % MeVec<T>::N == 0 && !((uintptr_t)weights & 15);
  const int f_end = min(n_out, (int)(blockIdx.y + 1) * ME_FEATURES_PER_BLOCK);
  for (int chunk = 0; chunk < count; chunk += ME_ROWS) {
    const int rows = min(ME_ROWS, count - chunk);
    __syncthreads();
    if (vector_ok && in_stride % MeVec<T>::N == 0 && !((uintptr_t)in & 15)) {  // 16 bytes a copy
      constexpr int V = MeVec<T>::N;
      const int per_row = k / V;
      for (int idx = threadIdx.x; idx < ME_ROWS * per_row; idx += blockDim.x) {
        const int r = idx / per_row, i = (idx % per_row) * V;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < rows) {
          const int row = first + chunk + r;
          const T* src = GATED ? in + (size_t)(pair_of_row[row] / top) * in_stride : in + (size_t)row * in_stride;
          v = *reinterpret_cast<const uint4*>(src + i);
        }
        *reinterpret_cast<uint4*>(rows_s + (size_t)r * k + i) = v;
      }
    } else {
      for (int idx = threadIdx.x; idx < ME_ROWS * k; idx += blockDim.x) {
        const int r = idx / k, i = idx % k;
        T v = from_float<T>(0.0f);
        if (r < rows) {
          const int row = first + chunk + r;
          const T* src = GATED ? in + (size_t)(pair_of_row[row] / top) * in_stride : in + (size_t)row * in_stride;
          v = src[i];
        }
        rows_s[idx] = v;
      }
    }
    __syncthreads();
    for (int f = blockIdx.y * ME_FEATURES_PER_BLOCK + warp; f < f_end; f += warps) {
      float a[ME_ROWS], b[ME_ROWS];
      me_dots<T, GATED>(w + (size_t)f * k, w + (size_t)(n_out + f) * k, rows_s, k, lane, vector_ok, a, b);
      if (lane < rows) {
        float mine = 0.0f, other = 0.0f;
#pragma unroll
        for (int r = 0; r < ME_ROWS; ++r)
          if (r == lane) {
            mine = a[r];
            if (GATED) other = b[r];
          }
        float result = mine;
        if (GATED) {  // gate and up are rounded to the activation type first, as a product that writes them would
          const float scale_in = in_weights ? in_weights[pair_of_row[first + chunk + lane]] : 1.0f;
          result = activation(to_float(from_float<T>(scale_in * mine)), act) * to_float(from_float<T>(scale_in * other));
        }
        out[(size_t)(first + chunk + lane) * n_out + f] = from_float<T>(result);
      }
    }
  }
}

// The same on tensor cores for bfloat16 and an inner size that is a multiple of 32: a warp owns 16 output features (the
// M side of mma.sync.m16n8k16, their weight rows read straight from global memory into the A fragments) and the eight
// rows in shared memory are the N side; gated, a second set of accumulators takes the up rows of the same features.
// Four warps share a group of features, each with a quarter of the inner size, so that sixteen warps a block have loads
// in flight; their partial sums meet in shared memory and are added in a fixed order.
#define MT_GROUPS 4   // groups of 16 features a block
#define MT_SLICES 4   // warps that share a group, each with a quarter of the inner size (their sums meet in shared memory)

__device__ __forceinline__ void mt_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// NT: tiles of eight rows a pass (1, or 2 when the experts have more than eight rows each on average: an expert's weights
// are then read once for sixteen of its rows).
template <bool GATED, int NT>
__global__ void __launch_bounds__(32 * MT_GROUPS * MT_SLICES, NT == 1 ? 2 : 1)
moe_expert_rows_mma_kernel(const __nv_bfloat16* __restrict__ in, long long in_stride,
                           const __nv_bfloat16* __restrict__ weights, const int* __restrict__ counters,
                           const int* __restrict__ pair_of_row, __nv_bfloat16* __restrict__ out, int k, int n_out, int top,
                           int experts, int act, const float* __restrict__ in_weights) {
  constexpr int ROWS = 8 * NT;
  extern __shared__ __align__(16) unsigned char me_smem[];
  __nv_bfloat16* rows_s = reinterpret_cast<__nv_bfloat16*>(me_smem);  // [ROWS][k + 32]: rows 64 bytes apart in banks
  const int ld = k + 32;
  float* parts = reinterpret_cast<float*>(rows_s + (size_t)ROWS * ld);  // [MT_SLICES][MT_GROUPS][32 lanes][8 * NT]
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp % MT_GROUPS, slice = warp / MT_GROUPS;
  const int g = lane >> 2, t = lane & 3;
  pdl_wait();
  pdl_trigger<1>();
  const int count = counters[e], first = counters[experts + e];
  if (count == 0) return;
  const __nv_bfloat16* w = weights + (size_t)e * (GATED ? 2 : 1) * n_out * k;
  const int f0 = (blockIdx.y * MT_GROUPS + group) * 16;
  // the two weight rows this lane reads (features f0 + g and f0 + g + 8), clamped; results beyond n_out are not stored
  const __nv_bfloat16* row_lo = w + (size_t)min(f0 + g, n_out - 1) * k;
  const __nv_bfloat16* row_hi = w + (size_t)min(f0 + g + 8, n_out - 1) * k;
  const size_t up = (size_t)n_out * k;
  // this warp's stretch of the inner size: whole steps of 32, the slices as equal as they come
  const int steps = k / 32;
  const int k_first = (steps * slice / MT_SLICES) * 32, k_last = (steps * (slice + 1) / MT_SLICES) * 32;
  for (int chunk = 0; chunk < count; chunk += ROWS) {
    const int rows = min(ROWS, count - chunk);
    __syncthreads();
    const int per_row = k / 8;
    for (int idx = threadIdx.x; idx < ROWS * per_row; idx += blockDim.x) {
      const int r = idx / per_row, i = (idx % per_row) * 8;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) {
        const int row = first + chunk + r;
        const __nv_bfloat16* src = GATED ? in + (size_t)(pair_of_row[row] / top) * in_stride : in + (size_t)row * in_stride;
        v = *reinterpret_cast<const uint4*>(src + i);
      }
      *reinterpret_cast<uint4*>(rows_s + (size_t)r * ld + i) = v;
    }
    __syncthreads();
    float c[NT][4], c2[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) c[nt][i] = c2[nt][i] = 0.0f;
    // 32 inner elements a step, as two products of 16.  A sum over k does not care which k meets which lane, as long as
    // A and B agree: lane t takes the eight elements k0 + 8t .. + 7 of its rows with one 16-byte load each, and uses the
    // pairs (0,1), (2,3) for the first product's two k halves and (4,5), (6,7) for the second's; B is read the same way.
    const __nv_bfloat16* b_row = rows_s + (size_t)g * ld + 8 * t;
    if (f0 < n_out) {
#pragma unroll 4
      for (int k0 = k_first; k0 < k_last; k0 += 32) {
        const uint4 lo = *reinterpret_cast<const uint4*>(row_lo + k0 + 8 * t);
        const uint4 hi = *reinterpret_cast<const uint4*>(row_hi + k0 + 8 * t);
        uint4 lo2 = make_uint4(0u, 0u, 0u, 0u), hi2 = lo2;
        if (GATED) {
          lo2 = *reinterpret_cast<const uint4*>(row_lo + up + k0 + 8 * t);
          hi2 = *reinterpret_cast<const uint4*>(row_hi + up + k0 + 8 * t);
        }
        const unsigned a_first[4] = {lo.x, hi.x, lo.y, hi.y}, a_second[4] = {lo.z, hi.z, lo.w, hi.w};
        const unsigned u_first[4] = {lo2.x, hi2.x, lo2.y, hi2.y}, u_second[4] = {lo2.z, hi2.z, lo2.w, hi2.w};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 b = *reinterpret_cast<const uint4*>(b_row + (size_t)nt * 8 * ld + k0);
          mt_mma(c[nt], a_first, b.x, b.y);
          mt_mma(c[nt], a_second, b.z, b.w);
          if (GATED) {
            mt_mma(c2[nt], u_first, b.x, b.y);
            mt_mma(c2[nt], u_second, b.z, b.w);
          }
        }
      }
    }
    float* mine = parts + (((size_t)slice * MT_GROUPS + group) * 32 + lane) * 8 * NT;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        mine[nt * 8 + i] = c[nt][i];
        mine[nt * 8 + 4 + i] = c2[nt][i];
      }
    __syncthreads();
    if (slice != 0 || f0 >= n_out) continue;
    // the slices' sums are added in slice order; element 0, 1 of a tile: feature f0 + g for its rows 2t and 2t + 1; 2, 3: f0 + g + 8
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float sum = 0.0f, sum2 = 0.0f;
#pragma unroll
        for (int sl = 0; sl < MT_SLICES; ++sl) {
          const float* theirs = parts + (((size_t)sl * MT_GROUPS + group) * 32 + lane) * 8 * NT + nt * 8;
          sum += theirs[i];
          sum2 += theirs[4 + i];
        }
        const int feature = f0 + g + (i >= 2 ? 8 : 0), r = nt * 8 + 2 * t + (i & 1);
        if (feature >= n_out || r >= rows) continue;
        float result = sum;
        if (GATED) {
          const float scale_in = in_weights ? in_weights[pair_of_row[first + chunk + r]] : 1.0f;
          const float gate = __bfloat162float(__float2bfloat16_rn(scale_in * sum)), upv = __bfloat162float(__float2bfloat16_rn(scale_in * sum2));
          result = activation(gate, act) * upv;
        }
        out[(size_t)(first + chunk + r) * n_out + feature] = __float2bfloat16_rn(result);
      }
  }
}

template <bool GATED, int NT>
static int launch_expert_rows_mma(const void* in, long long in_stride, const void* weights, const int* counters,
                                  const int* pair_of_row, void* out, int k, int n_out, int top, int experts, int act,
                                  const float* in_weights, cudaStream_t stream) {
  const size_t smem = (size_t)8 * NT * (k + 32) * 2 + (size_t)MT_SLICES * MT_GROUPS * 32 * 8 * NT * sizeof(float);
  dim3 tiles(experts, (n_out + 16 * MT_GROUPS - 1) / (16 * MT_GROUPS));
  if (tiles.y > 65535 || smem > 200 * 1024) return TS_ERR_SIZE;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(moe_expert_rows_mma_kernel<GATED, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ts_launch(moe_expert_rows_mma_kernel<GATED, NT>, tiles, dim3(32 * MT_GROUPS * MT_SLICES), smem, stream,
            (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)weights, counters, pair_of_row, (__nv_bfloat16*)out, k,
            n_out, top, experts, act, in_weights);
  return ts_launch_status();
}

// in: the step's inputs [tokens][in_stride] (gated) or the rows of the gated call [pairs][k] (plain).
TS_EXPORT int ts_moe_expert_rows(int dtype, int gated, const void* in, long long in_stride, const void* weights,
                                 const int* counters, const int* pair_of_row, void* out, int k, int n_out, int top,
                                 int experts, int num_pairs, int act, const float* in_weights, cudaStream_t stream) {
  if (!gated) in_weights = nullptr;
  if (experts <= 0 || n_out <= 0) return 0;
  const size_t item = dtype == TS_F32 ? 4 : 2;
  const size_t smem = (size_t)ME_ROWS * k * item;
  if (smem > 200 * 1024 || k < 1 || top < 1) return TS_ERR_SIZE;
  if (dtype == TS_BF16 && k % 32 == 0 && in_stride % 8 == 0 && !(((uintptr_t)in | (uintptr_t)weights) & 15)) {
    // experts with more than eight rows each on average take sixteen rows a pass, where shared memory has the room
    int code = TS_ERR_SIZE;
    if (num_pairs > 8 * experts)
      code = gated ? launch_expert_rows_mma<true, 2>(in, in_stride, weights, counters, pair_of_row, out, k, n_out, top, experts, act, in_weights, stream)
                   : launch_expert_rows_mma<false, 2>(in, in_stride, weights, counters, pair_of_row, out, k, n_out, top, experts, act, in_weights, stream);
    if (code == TS_ERR_SIZE)
      code = gated ? launch_expert_rows_mma<true, 1>(in, in_stride, weights, counters, pair_of_row, out, k, n_out, top, experts, act, in_weights, stream)
                   : launch_expert_rows_mma<false, 1>(in, in_stride, weights, counters, pair_of_row, out, k, n_out, top, experts, act, in_weights, stream);
    if (code != TS_ERR_SIZE) return code;
  }
  dim3 grid(experts, (n_out + ME_FEATURES_PER_BLOCK - 1) / ME_FEATURES_PER_BLOCK);
  if (grid.y > 65535) return TS_ERR_SIZE;
#define ME_LAUNCH(TYPE, G)                                                                                             \
  do {                                                                                                                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(moe_expert_rows_kernel<TYPE, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    ts_launch(moe_expert_rows_kernel<TYPE, G>, grid, dim3(256), smem, stream, (const TYPE*)in, in_stride,              \
              (const TYPE*)weights, counters, pair_of_row, (TYPE*)out, k, n_out, top, experts, act, in_weights);       \
  } while (0)
  if (dtype == TS_F32) {
    if (gated) ME_LAUNCH(float, true); else ME_LAUNCH(float, false);
  } else if (dtype == TS_BF16) {
    if (gated) ME_LAUNCH(__nv_bfloat16, true); else ME_LAUNCH(__nv_bfloat16, false);
  } else {
    return TS_ERR_DTYPE;
  }
#undef ME_LAUNCH
  return ts_launch_status();
}

TS_EXPORT int ts_moe_sort(const int* chosen, int pairs, int experts, int* counters, int* place, int* pair_of_row,
                          cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (pairs <= MOE_SORT_SMALL && experts <= 2048) {
    ts_launch(moe_sort_small_kernel, dim3(1), dim3(256), (size_t)(3 * experts + 1) * sizeof(int), stream, chosen, pairs,
              experts, counters, place, pair_of_row);
    return ts_launch_status();
  }
  cudaMemsetAsync(counters, 0, (size_t)experts * sizeof(int), stream);
  const unsigned blocks = (unsigned)((pairs + 255) / 256);
  ts_launch(moe_count_kernel, dim3(blocks), dim3(256), 0, stream, chosen, pairs, experts, counters);
  ts_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, stream, experts, counters);
  ts_launch(moe_place_kernel, dim3(blocks), dim3(256), 0, stream, chosen, pairs, experts, counters, place, pair_of_row);
  return ts_launch_status();
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, long long x_stride, const int* __restrict__ pair_of_row,
                                  T* __restrict__ rows, int width, int top, const float* __restrict__ in_weights) {
  pdl_wait();
  pdl_trigger<1>();
  const int r = blockIdx.x;
  const int pair = pair_of_row[r];
  const T* src = x + (size_t)(pair / top) * x_stride;
  T* dst = rows + (size_t)r * width;
  if (in_weights) {  // the expert reads its token's row times the pair's weight
    const float w = in_weights[pair];
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_float<T>(w * to_float(src[i]));
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

TS_EXPORT int ts_moe_gather(int dtype, const void* x, long long x_stride, const int* pair_of_row, void* rows, int pairs,
                            int width, int top, const float* in_weights, cudaStream_t stream) {
  if (pairs <= 0) return 0;
  if (dtype == TS_F32)
    ts_launch(moe_gather_kernel<float>, dim3(pairs), dim3(128), 0, stream, (const float*)x, x_stride, pair_of_row,
              (float*)rows, width, top, in_weights);
  else if (dtype == TS_BF16)
    ts_launch(moe_gather_kernel<__nv_bfloat16>, dim3(pairs), dim3(128), 0, stream, (const __nv_bfloat16*)x, x_stride,
              pair_of_row, (__nv_bfloat16*)rows, width, top, in_weights);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place,
                                   const float* __restrict__ weights, const T* __restrict__ addend, T* __restrict__ out,
                                   int width, int top) {
  pdl_wait();
  pdl_trigger<1>();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float sum = 0.0f;
    for (int k = 0; k < top; ++k)
      sum = fmaf(weights ? weights[(size_t)t * top + k] : 1.0f, to_float(rows[(size_t)place[(size_t)t * top + k] * width + i]), sum);
    if (addend) sum += to_float(addend[(size_t)t * width + i]);
    out[(size_t)t * width + i] = from_float<T>(sum);
  }
}

TS_EXPORT int ts_moe_combine(int dtype, const void* rows, const int* place, const float* weights, const void* addend,
                             void* out, int num_tokens, int width, int top, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dtype == TS_F32)
    ts_launch(moe_combine_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, (const float*)rows, place, weights,
              (const float*)addend, (float*)out, width, top);
  else if (dtype == TS_BF16)
    ts_launch(moe_combine_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, (const __nv_bfloat16*)rows, place,
              weights, (const __nv_bfloat16*)addend, (__nv_bfloat16*)out, width, top);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
