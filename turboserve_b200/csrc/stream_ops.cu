// Kernels on the residual stream for blocks whose branches run side by side, and two small
// element-wise ones: a plain (ungated) activation and a scaling of rows.
//
//   stream_norm   x = residual + delta_a + delta_b + shift (each optional), summed in fp32 in that
//                 order (with a factor other than 1: residual + mult * (delta_a + delta_b) + shift);
//                 written back to the residual (unless rows are selected); then
//                 out1 = x * rsqrt(mean(x^2) + eps) * gain1 and, if asked, out2 = the same * gain2.
//                 One launch does what a layer with two parallel branches needs between the branches
//                 of the layer before and its own: both pending updates, the vector that a repeated
//                 stretch of layers adds before each pass, and both norms of the same input.
//   stream_add    the sum alone (a block that cannot take two updates, or a shift before one).
//   norm_add      residual += mult * (update * rsqrt(mean(update^2) + eps) * gain), the norm taken on a
//                 sublayer's OUTPUT, all in fp32; the new residual is also written in the activation
//                 type as the next sublayer's input.  Without an update it only writes that copy.
//   norm_add_norm norm_add for the sublayer that ran, an optional matrix of fp32 rows added, and the norm before the
//                 sublayer that runs next, in one pass over the row (a block with norms on both sides of its sublayers).
//   activation    out = act(in), act one of relu^2, gelu(tanh), silu, tanh, in fp32, rounded once.
//   scale_rows    fp32 rows times a constant, in place (a head whose logits are scaled).
//   softcap_rows  fp32 rows through cap * tanh(x / cap), in place (a head whose logits are capped).
#include "common.cuh"

template <typename T>
__global__ void stream_norm_kernel(float* __restrict__ residual, const T* __restrict__ delta_a,
                                   const T* __restrict__ delta_b, const float* __restrict__ shift,
                                   const float* __restrict__ gain1, T* __restrict__ out1,
                                   const float* __restrict__ gain2, T* __restrict__ out2,
                                   const int* __restrict__ rows, int hidden, float eps, float mult) {
  extern __shared__ __align__(16) float row_cache[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_wait();
  pdl_trigger<32>();
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  const T* da = delta_a ? delta_a + (size_t)src * hidden : nullptr;
  const T* db = delta_b ? delta_b + (size_t)src * hidden : nullptr;
  float sum_sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x = res[i];
    if (mult == 1.0f) {
      if (da) x += to_float(da[i]);
      if (db) x += to_float(db[i]);
    } else {
      float u = da ? to_float(da[i]) : 0.0f;
      if (db) u += to_float(db[i]);
      x = fmaf(mult, u, x);
    }
    if (shift) x += shift[i];
    row_cache[i] = x;
    if (!rows) res[i] = x;
    sum_sq = fmaf(x, x, sum_sq);
  }
  if (!out1) return;
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  T* o1 = out1 + (size_t)r * hidden;
  T* o2 = out2 ? out2 + (size_t)r * hidden : nullptr;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = row_cache[i] * inv;
    o1[i] = from_float<T>(x * gain1[i]);
    if (o2) o2[i] = from_float<T>(x * gain2[i]);
  }
}

TS_EXPORT int ts_stream_norm(int dtype, float* residual, const void* delta_a, const void* delta_b,
                             const float* shift, const float* gain1, void* out1, const float* gain2,
                             void* out2, const int* rows, int num_rows, int hidden, float eps, float mult,
                             cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden < 1 || (size_t)hidden * sizeof(float) > 200 * 1024) return TS_ERR_SIZE;
  if ((out1 && !gain1) || (out2 && (!gain2 || !out1))) return TS_ERR_ARGUMENT;
  int threads = (hidden + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (dtype == TS_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(stream_norm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, residual, (const float*)delta_a,
              (const float*)delta_b, shift, gain1, (float*)out1, gain2, (float*)out2, rows, hidden, eps, mult);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(stream_norm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), smem, stream, residual,
              (const __nv_bfloat16*)delta_a, (const __nv_bfloat16*)delta_b, shift, gain1, (__nv_bfloat16*)out1, gain2,
              (__nv_bfloat16*)out2, rows, hidden, eps, mult);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// A block whose norms stand behind its sublayers: the sublayer read the stream itself, its output is
// normed (statistics over the update alone), scaled and added.  One block per row.
template <typename T>
__global__ void norm_add_kernel(float* __restrict__ residual, const T* __restrict__ update,
                                const float* __restrict__ gain, T* __restrict__ copy, int hidden, float eps,
                                float mult) {
  extern __shared__ __align__(16) float row_cache[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_wait();
  pdl_trigger<32>();
  float* res = residual + (size_t)r * hidden;
  T* out = copy ? copy + (size_t)r * hidden : nullptr;
  if (!update) {
    if (out)
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = from_float<T>(res[i]);
    return;
  }
  const T* up = update + (size_t)r * hidden;
  float sum_sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float u = to_float(up[i]);
    row_cache[i] = u;
    sum_sq = fmaf(u, u, sum_sq);
  }
  const float total = block_sum(sum_sq, scratch);
  const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = fmaf(mult, row_cache[i] * inv * gain[i], res[i]);
    res[i] = x;
    if (out) out[i] = from_float<T>(x);
  }
}

TS_EXPORT int ts_norm_add(int dtype, float* residual, const void* update, const float* gain, void* copy,
                          int num_rows, int hidden, float eps, float mult, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden < 1 || (size_t)hidden * sizeof(float) > 200 * 1024) return TS_ERR_SIZE;
  if (update && !gain) return TS_ERR_ARGUMENT;
  int threads = (hidden + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (dtype == TS_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_add_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_add_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, residual, (const float*)update, gain,
              (float*)copy, hidden, eps, mult);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_add_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_add_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), smem, stream, residual,
              (const __nv_bfloat16*)update, gain, (__nv_bfloat16*)copy, hidden, eps, mult);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// A block with norms before AND behind its sublayers: what stands between two sublayers is one kernel,
//     residual += update * rsqrt(mean(update^2) + eps_post) * gain_post      (the norm behind the sublayer that ran)
//     residual += extra                                                      (fp32 rows, e.g. the embedding's output
//                                                                             that a repeated stretch adds before a pass)
//     out = residual * rsqrt(mean(residual^2) + eps_pre) * gain_pre          (the norm before the sublayer that runs next)
// each part optional, everything in fp32, `out` rounded once.  With `rows` the listed rows alone are worked and the
// residual is left as it is (the final norm, at the rows whose logits are wanted).  One block per row; a thread meets
// the same elements in every pass, so the row lives in shared memory without a barrier of its own.
template <typename T>
__global__ void norm_add_norm_kernel(float* __restrict__ residual, const T* __restrict__ update,
                                     const float* __restrict__ gain_post, float eps_post, const float* __restrict__ extra,
                                     const float* __restrict__ gain_pre, float eps_pre, T* __restrict__ out,
                                     const int* __restrict__ rows, int hidden) {
  extern __shared__ __align__(16) float row_cache[];
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_wait();
  pdl_trigger<32>();
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  float inv_post = 0.0f;
  if (update) {
    const T* up = update + (size_t)src * hidden;
    float sum_sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float u = to_float(up[i]);
      row_cache[i] = u;
      sum_sq = fmaf(u, u, sum_sq);
    }
    inv_post = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps_post);
  }
  const float* ex = extra ? extra + (size_t)src * hidden : nullptr;
  float sum_sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float x = res[i];
    if (update) x += row_cache[i] * inv_post * gain_post[i];
    if (ex) x += ex[i];
    if (!rows && (update || ex)) res[i] = x;
    row_cache[i] = x;
    sum_sq = fmaf(x, x, sum_sq);
  }
  if (!out) return;
  const float inv_pre = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)hidden + eps_pre);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_float<T>(row_cache[i] * inv_pre * gain_pre[i]);
}

// The same with 16-byte loads and stores, for rows whose width is a multiple of four and whose tensors are aligned:
// a thread takes four neighbours a pass; the update and the residual are both fetched before the first sum is awaited
// (two rows of shared memory), so the row's loads are all in flight together.  Every sum is taken as in the kernel
// above: first the update's norm, then the residual, then the added rows.
template <typename T> struct Four;
template <> struct Four<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Four<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
    v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 x;
    x.x = *reinterpret_cast<unsigned*>(&a);
    x.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
};

template <typename T>
__global__ void norm_add_norm_vec_kernel(float* __restrict__ residual, const T* __restrict__ update,
                                         const float* __restrict__ gain_post, float eps_post,
                                         const float* __restrict__ extra, const float* __restrict__ gain_pre, float eps_pre,
                                         T* __restrict__ out, const int* __restrict__ rows, int hidden) {
  extern __shared__ __align__(16) float row_cache[];  // [2][hidden]: the update, the residual
  __shared__ float scratch[33];
  float* u_cache = row_cache;
  float* x_cache = row_cache + hidden;
  const int r = blockIdx.x;
  pdl_wait();
  pdl_trigger<32>();
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  const T* up = update ? update + (size_t)src * hidden : nullptr;
  const float* ex = extra ? extra + (size_t)src * hidden : nullptr;
  float sum_u = 0.0f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float x[4];
    Four<float>::load(res + i, x);
    if (up) {
      float u[4];
      Four<T>::load(up + i, u);
      Four<float>::store(u_cache + i, u);
#pragma unroll
      for (int e = 0; e < 4; ++e) sum_u = fmaf(u[e], u[e], sum_u);
    }
    Four<float>::store(x_cache + i, x);
  }
  const float inv_post = up ? 1.0f / sqrtf(block_sum(sum_u, scratch) / (float)hidden + eps_post) : 0.0f;
  float sum_x = 0.0f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float x[4];
    Four<float>::load(x_cache + i, x);
    if (up) {
      float u[4], g[4];
      Four<float>::load(u_cache + i, u);
      Four<float>::load(gain_post + i, g);
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] += u[e] * inv_post * g[e];
    }
    if (ex) {
      float a[4];
      Four<float>::load(ex + i, a);
#pragma unroll
      for (int e = 0; e < 4; ++e) x[e] += a[e];
    }
    if (!rows && (up || ex)) Four<float>::store(res + i, x);
    if (out) Four<float>::store(x_cache + i, x);
#pragma unroll
    for (int e = 0; e < 4; ++e) sum_x = fmaf(x[e], x[e], sum_x);
  }
  if (!out) return;
  const float inv_pre = 1.0f / sqrtf(block_sum(sum_x, scratch) / (float)hidden + eps_pre);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    float x[4], g[4];
    Four<float>::load(x_cache + i, x);
    Four<float>::load(gain_pre + i, g);
#pragma unroll
    for (int e = 0; e < 4; ++e) x[e] = x[e] * inv_pre * g[e];
    Four<T>::store(o + i, x);
  }
}

template <typename T>
static bool norm_add_norm_vec(float* residual, const void* update, const float* gain_post, float eps_post, const float* extra,
                              const float* gain_pre, float eps_pre, void* out, const int* rows, int num_rows, int hidden,
                              cudaStream_t stream) {
  const size_t smem = (size_t)2 * hidden * sizeof(float);
  const uintptr_t wide = (uintptr_t)residual | (uintptr_t)gain_post | (uintptr_t)extra | (uintptr_t)gain_pre;
  const uintptr_t narrow = (uintptr_t)update | (uintptr_t)out;
  if (hidden % 4 || smem > 200 * 1024 || (wide & 15) || (narrow & (sizeof(T) * 4 - 1))) return false;
  int threads = (hidden / 4 + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(norm_add_norm_vec_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ts_launch(norm_add_norm_vec_kernel<T>, dim3(num_rows), dim3(threads), smem, stream, residual, (const T*)update, gain_post,
            eps_post, extra, gain_pre, eps_pre, (T*)out, rows, hidden);
  return true;
}

TS_EXPORT int ts_norm_add_norm(int dtype, float* residual, const void* update, const float* gain_post, float eps_post,
                               const float* extra, const float* gain_pre, float eps_pre, void* out, const int* rows,
                               int num_rows, int hidden, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden < 1 || (size_t)hidden * sizeof(float) > 200 * 1024) return TS_ERR_SIZE;
  if ((update && !gain_post) || (out && !gain_pre)) return TS_ERR_ARGUMENT;
  if (dtype == TS_F32 && norm_add_norm_vec<float>(residual, update, gain_post, eps_post, extra, gain_pre, eps_pre, out, rows,
                                                   num_rows, hidden, stream))
    return ts_launch_status();
  if (dtype == TS_BF16 && norm_add_norm_vec<__nv_bfloat16>(residual, update, gain_post, eps_post, extra, gain_pre, eps_pre, out,
                                                            rows, num_rows, hidden, stream))
    return ts_launch_status();
  int threads = (hidden + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (dtype == TS_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_add_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_add_norm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, residual, (const float*)update,
              gain_post, eps_post, extra, gain_pre, eps_pre, (float*)out, rows, hidden);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_add_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_add_norm_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), smem, stream, residual,
              (const __nv_bfloat16*)update, gain_post, eps_post, extra, gain_pre, eps_pre, (__nv_bfloat16*)out, rows, hidden);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// out = act(in): 0 relu^2, 1 gelu (tanh form), 2 silu, 3 tanh.
__device__ __forceinline__ float plain_activation(float x, int act) {
  if (act == 0) {
    const float r = fmaxf(x, 0.0f);
    return r * r;
  }
  if (act == 1) {
    const float inner = 0.79788456080286535588f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
  }
  if (act == 3) return tanhf(x);
  return x / (1.0f + expf(-x));
}

template <typename T>
__global__ void activation_kernel(const T* __restrict__ in, T* __restrict__ out, long long count, int act) {
  pdl_wait();
  pdl_trigger<1>();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
    out[i] = from_float<T>(plain_activation(to_float(in[i]), act));
}

TS_EXPORT int ts_activation(int dtype, const void* in, void* out, long long count, int act, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (act < 0 || act > 3) return TS_ERR_ARGUMENT;
  long long blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == TS_F32)
    ts_launch(activation_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, stream, (const float*)in, (float*)out, count, act);
  else if (dtype == TS_BF16)
    ts_launch(activation_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in,
              (__nv_bfloat16*)out, count, act);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

__global__ void scale_rows_kernel(float* __restrict__ data, long long count, float factor) {
  pdl_wait();
  pdl_trigger<1>();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) data[i] *= factor;
}

TS_EXPORT int ts_scale_rows(float* data, long long count, float factor, cudaStream_t stream) {
  if (count <= 0) return 0;
  long long blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ts_launch(scale_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, data, count, factor);
  return ts_launch_status();
}

// fp32 rows bent into (-cap, cap): x <- cap * tanh(x / cap), in place (a head whose logits are capped).
__global__ void softcap_rows_kernel(float* __restrict__ data, long long count, float cap) {
  pdl_wait();
  pdl_trigger<1>();
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float inv = 1.0f / cap;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) data[i] = cap * tanhf(data[i] * inv);
}

TS_EXPORT int ts_softcap_rows(float* data, long long count, float cap, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (!(cap > 0.0f)) return TS_ERR_ARGUMENT;
  long long blocks = (count + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  ts_launch(softcap_rows_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, data, count, cap);
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// norm_pair_mix: out = wa * (a / rms(a) * gain_a) + wb * (b / rms(b) * gain_b), each input normed over the whole
// row on its own (eps inside the root), in fp32, rounded once.  Two mixers that read the same input side by
// side leave their outputs this way as one update of the stream.  One block per row.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void norm_pair_mix_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ gain_a,
                                     const float* __restrict__ gain_b, T* __restrict__ out, int hidden, float eps,
                                     float wa, float wb) {
  extern __shared__ __align__(16) float row_cache[];  // [2][hidden]
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  pdl_wait();
  pdl_trigger<1>();
  const T* ra = a + (size_t)r * hidden;
  const T* rb = b + (size_t)r * hidden;
  float sa = 0.0f, sb = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float x = to_float(ra[i]), y = to_float(rb[i]);
    row_cache[i] = x;
    row_cache[hidden + i] = y;
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  const float ta = block_sum(sa, scratch);
  const float tb = block_sum(sb, scratch);
  const float ia = wa / sqrtf(ta / (float)hidden + eps), ib = wb / sqrtf(tb / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_float<T>(fmaf(row_cache[i] * ia, gain_a[i], row_cache[hidden + i] * ib * gain_b[i]));
}

TS_EXPORT int ts_norm_pair_mix(int dtype, const void* a, const void* b, const float* gain_a, const float* gain_b, void* out,
                               int num_rows, int hidden, float eps, float wa, float wb, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (hidden < 1 || (size_t)hidden * 2 * sizeof(float) > 200 * 1024) return TS_ERR_SIZE;
  int threads = (hidden + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  const size_t smem = (size_t)hidden * 2 * sizeof(float);
  if (dtype == TS_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_pair_mix_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_pair_mix_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, (const float*)a, (const float*)b,
              gain_a, gain_b, (float*)out, hidden, eps, wa, wb);
  } else if (dtype == TS_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_pair_mix_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(norm_pair_mix_kernel<__nv_bfloat16>, dim3(num_rows), dim3(threads), smem, stream, (const __nv_bfloat16*)a,
              (const __nv_bfloat16*)b, gain_a, gain_b, (__nv_bfloat16*)out, hidden, eps, wa, wb);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// shift_mix: blends of every token's row with the row of the token before it in its request,
//     out[t][s] = x[t] + (x[t - 1] - x[t]) * mu[s]          (s = 0 .. mixes - 1, mu[s] a row of floats)
// written side by side as [tokens][mixes * hidden].  The row before a step's first token of a request is the one
// the request kept in its state slot (`last`, [slots][hidden], in the activation type); before position 0 it is
// zeros.  A second kernel then keeps each request's last row of this step.  fp32 arithmetic, rounded once.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu, const T* __restrict__ last,
                                 T* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ query_start, const int* __restrict__ slots, int hidden, int mixes) {
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  pdl_wait();
  pdl_trigger<1>();
  if (seq < 0) return;
  const T* before = nullptr;
  if (positions[t] > 0) before = t > query_start[seq] ? x + (size_t)(t - 1) * hidden : last + (size_t)slots[seq] * hidden;
  const T* row = x + (size_t)t * hidden;
  T* o = out + (size_t)t * mixes * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float now = to_float(row[i]);
    const float step = (before ? to_float(before[i]) : 0.0f) - now;
    for (int s = 0; s < mixes; ++s) o[(size_t)s * hidden + i] = from_float<T>(fmaf(step, mu[(size_t)s * hidden + i], now));
  }
}

template <typename T>
__global__ void shift_keep_kernel(const T* __restrict__ x, T* __restrict__ last, const int* __restrict__ query_start,
                                  const int* __restrict__ slots, int hidden) {
  const int seq = blockIdx.x;
  pdl_wait();
  const int first = query_start[seq], end = query_start[seq + 1];
  if (end <= first) return;
  const T* row = x + (size_t)(end - 1) * hidden;
  T* to = last + (size_t)slots[seq] * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) to[i] = row[i];
}

TS_EXPORT int ts_shift_mix(int dtype, const void* x, const float* mu, void* last, void* out, const int* positions,
                           const int* seq_of_token, const int* query_start, const int* slots, int num_tokens, int num_seqs,
                           int hidden, int mixes, cudaStream_t stream) {
  if (num_tokens <= 0 || num_seqs <= 0) return 0;
  if (hidden < 1 || mixes < 1) return TS_ERR_SIZE;
  const int threads = hidden >= 256 ? 256 : 64;
  if (dtype == TS_F32) {
    ts_launch(shift_mix_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)x, mu, (const float*)last,
              (float*)out, positions, seq_of_token, query_start, slots, hidden, mixes);
    ts_launch(shift_keep_kernel<float>, dim3(num_seqs), dim3(threads), 0, stream, (const float*)x, (float*)last, query_start,
              slots, hidden);
  } else if (dtype == TS_BF16) {
    ts_launch(shift_mix_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)x, mu,
              (const __nv_bfloat16*)last, (__nv_bfloat16*)out, positions, seq_of_token, query_start, slots, hidden, mixes);
    ts_launch(shift_keep_kernel<__nv_bfloat16>, dim3(num_seqs), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
              (__nv_bfloat16*)last, query_start, slots, hidden);
  } else {
    return TS_ERR_DTYPE;
  }
  return ts_launch_status();
}
