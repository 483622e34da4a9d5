// The state-space recurrence with a scalar decay per head (the "state space duality" layer), on a
// packed batch of requests with the state kept per request between steps, and the gated, grouped
// RMS norm that follows it.
//
// Per head h (value size P, state size N, group g = h / (heads / groups)) and position t:
//
//   dt_t = softplus(raw_t[h] + dt_bias[h])                   (fp32, no clamp)
//   S_t  = exp(-exp(A_log[h]) * dt_t) * S_{t-1} + dt_t * B_t[g] x_t[h]^T      (S is N x P, fp32)
//   y_t[h] = S_t^T C_t[g] + D[h] * x_t[h]
//
// ssd_scan: one block per (head, request, tile of P).  A step's positions of a request are taken in
// order, eight at a time through shared memory (two buffers: the next eight are on their way from
// global memory into registers while the current eight are worked); a thread owns CPT (1 or 2) value columns
// and sixteen state rows of them (NS lanes share its columns and add their parts of y
// by shuffles), so the state stays in registers over the whole portion and is read and written once.
// Two columns a thread mean fewer loads from shared memory per multiply-add and half the blocks; the
// launch takes two when that still fills the device.  The products and multiply-adds on the state are the
// packed fp32x2 instructions of sm_100 (two rows of a column a register pair).  The state of a request
// lives in its slot of `state` ([slots, heads, P, N], fp32); a request that starts has a zeroed
// slot.  One token per request (decoding) and long portions of prompts run the same code, and the
// sums of an output are added in one order whatever the number of columns a thread, so an output is
// the same bits however a request is cut into steps and whatever else the batch holds.
//
// gated_group_norm: v = y * silu(z); every one of `parts` equal parts of a row is divided by its
// own root mean square (eps inside the root) and multiplied by the weight; fp32, rounded once.
#include "common.cuh"

#define SSD_THREADS 128
#define SSD_WARPS 4
#define SSD_ROWS_PER_THREAD 16
#define SSD_BATCH 8
#define SSD_PF_ROWS 4  // inputs are fetched a batch ahead into registers when N <= 128 ...
#define SSD_PF_COLS 2  // ... and a block's tile of P is at most 64 columns wide

// Two fp32 values in one 64-bit register and the packed multiply and multiply-add of sm_100 (each half is
// the IEEE operation of the scalar instruction, so packing changes no bit).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// Row r (0 .. 15) of lane s of NS: four consecutive rows, then on by 4 * NS, so that the NS lanes of a
// column read consecutive 16-byte pieces of B and C from shared memory.
__device__ __forceinline__ int ssd_row(int r, int s, int NS) { return (r >> 2) * (NS * 4) + s * 4 + (r & 3); }

template <typename T, int CPT>
__global__ void __launch_bounds__(SSD_THREADS)
ssd_scan_kernel(const T* __restrict__ xbc, long long xbc_stride, const T* __restrict__ dt_raw, long long dt_stride,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, const int* __restrict__ query_start,
                const int* __restrict__ slots, int heads, int groups, int P, int N, int NS) {
  extern __shared__ __align__(16) float smem[];
  const int head = blockIdx.x, seq = blockIdx.y;
  const int p_tile = SSD_THREADS / NS * CPT;
  const int p0 = blockIdx.z * p_tile;
  const int n_pad = SSD_ROWS_PER_THREAD * NS;  // rows of B and C in shared memory; those from N on are zero
  const int per_batch = SSD_BATCH * (2 * n_pad + p_tile);
  const int per_buffer = per_batch + 2 * SSD_BATCH;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = tid % NS, pl = tid / NS;
  const int group = head / (heads / groups);
  const int inner = heads * P;
  const float rate = expf(a_log[head]);
  const float bias = dt_bias[head], skip = d_skip[head];
  pdl_wait();
  pdl_trigger();
  const int begin = query_start[seq], n = query_start[seq + 1] - begin;
  if (n <= 0) return;
  float* slot_state = state + (((size_t)slots[seq] * heads + head) * P) * N;
  f32x2 S[CPT][SSD_ROWS_PER_THREAD / 2];  // rows 2 i and 2 i + 1 of the thread's sixteen share a register pair
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int p = p0 + pl * CPT + c;
#pragma unroll
    for (int i = 0; i < SSD_ROWS_PER_THREAD / 2; ++i) {
      const int row = ssd_row(2 * i, s, NS);
      const float lo = (p < P && row < N) ? slot_state[(size_t)p * N + row] : 0.0f;
      const float hi = (p < P && row + 1 < N) ? slot_state[(size_t)p * N + row + 1] : 0.0f;
      S[c][i] = pack2(lo, hi);
    }
  }
  for (int i = tid; i < 2 * per_buffer; i += SSD_THREADS) smem[i] = 0.0f;
  __syncthreads();
  // one batch in shared memory: B [8][n_pad], C [8][n_pad], x [8][p_tile], then step sizes and decays [8] each.
  // Warp w brings positions w and w + 4 of a batch.
  const bool ahead = N <= 32 * SSD_PF_ROWS && p_tile <= 32 * SSD_PF_COLS;
  float pb[2][SSD_PF_ROWS], pc[2][SSD_PF_ROWS], px[2][SSD_PF_COLS];
  float pre_dt = 0.0f;
  auto load = [&](int base) {
    const int count = min(SSD_BATCH, n - base);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int tt = warp + SSD_WARPS * k;
      const T* src = xbc + (size_t)(begin + base + min(tt, count - 1)) * xbc_stride;
      const T* b_src = src + inner + group * N;
      const T* c_src = b_src + (size_t)groups * N;
#pragma unroll
      for (int j = 0; j < SSD_PF_ROWS; ++j) {
        const int row = lane + 32 * j;
        pb[k][j] = row < N ? to_float(b_src[row]) : 0.0f;
        pc[k][j] = row < N ? to_float(c_src[row]) : 0.0f;
      }
#pragma unroll
      for (int j = 0; j < SSD_PF_COLS; ++j) {
        const int col = lane + 32 * j;
        px[k][j] = (col < p_tile && p0 + col < P) ? to_float(src[head * P + p0 + col]) : 0.0f;
      }
    }
    if (tid < count) pre_dt = to_float(dt_raw[(size_t)(begin + base + tid) * dt_stride + head]);
  };
  auto store = [&](int base, float* buffer) {
    const int count = min(SSD_BATCH, n - base);
    float* sB = buffer;
    float* sC = buffer + SSD_BATCH * n_pad;
    float* sx = buffer + 2 * SSD_BATCH * n_pad;
    if (ahead) {
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int tt = warp + SSD_WARPS * k;
#pragma unroll
        for (int j = 0; j < SSD_PF_ROWS; ++j) {
          const int row = lane + 32 * j;
          if (row < N) {
            sB[tt * n_pad + row] = pb[k][j];
            sC[tt * n_pad + row] = pc[k][j];
          }
        }
#pragma unroll
        for (int j = 0; j < SSD_PF_COLS; ++j) {
          const int col = lane + 32 * j;
          if (col < p_tile) sx[tt * p_tile + col] = px[k][j];
        }
      }
    } else {
      for (int tt = warp; tt < count; tt += SSD_WARPS) {
        const T* src = xbc + (size_t)(begin + base + tt) * xbc_stride;
        const T* b_src = src + inner + group * N;
        const T* c_src = b_src + (size_t)groups * N;
        for (int row = lane; row < N; row += 32) {
          sB[tt * n_pad + row] = to_float(b_src[row]);
          sC[tt * n_pad + row] = to_float(c_src[row]);
        }
        for (int col = lane; col < p_tile; col += 32)
          sx[tt * p_tile + col] = p0 + col < P ? to_float(src[head * P + p0 + col]) : 0.0f;
      }
      if (tid < count) pre_dt = to_float(dt_raw[(size_t)(begin + base + tid) * dt_stride + head]);
    }
    if (tid < count) {
      const float v = pre_dt + bias;
      const float step = v > 20.0f ? v : log1pf(expf(v));
      buffer[per_batch + tid] = step;
      buffer[per_batch + SSD_BATCH + tid] = expf(-rate * step);
    }
  };
  if (ahead) load(0);
  store(0, smem);
  __syncthreads();
  for (int base = 0, turn = 0; base < n; base += SSD_BATCH, turn ^= 1) {
    const int count = min(SSD_BATCH, n - base);
    const bool more = base + SSD_BATCH < n;
    if (more && ahead) load(base + SSD_BATCH);
    const float* buffer = smem + turn * per_buffer;
    const float* sB = buffer;
    const float* sC = buffer + SSD_BATCH * n_pad;
    const float* sx = buffer + 2 * SSD_BATCH * n_pad;
    const float* sdt = buffer + per_batch;
    const float* sdecay = sdt + SSD_BATCH;
    // several positions in flight: the next position's state update does not wait for this one's sum over the lanes
#pragma unroll 4
    for (int tt = 0; tt < count; ++tt) {
      const float decay = sdecay[tt];
      const float4* Bt = reinterpret_cast<const float4*>(sB + tt * n_pad + s * 4);
      const float4* Ct = reinterpret_cast<const float4*>(sC + tt * n_pad + s * 4);
      const f32x2 decay2 = pack2(decay, decay);
      float x[CPT];
      f32x2 dx2[CPT], part[CPT][2];
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        x[c] = sx[tt * p_tile + pl * CPT + c];
        const float dx = sdt[tt] * x[c];
        dx2[c] = pack2(dx, dx);
      }
#pragma unroll
      for (int k = 0; k < SSD_ROWS_PER_THREAD / 4; ++k) {
        const float4 b4 = Bt[k * NS], c4 = Ct[k * NS];
        const f32x2 b[2] = {pack2(b4.x, b4.y), pack2(b4.z, b4.w)}, cv[2] = {pack2(c4.x, c4.y), pack2(c4.z, c4.w)};
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            S[c][2 * k + e] = fma2(decay2, S[c][2 * k + e], mul2(dx2[c], b[e]));
            part[c][e] = k == 0 ? mul2(S[c][e], cv[e]) : fma2(S[c][2 * k + e], cv[e], part[c][e]);
          }
        }
      }
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        float p0v, p1v, p2v, p3v;
        unpack2(part[c][0], p0v, p1v);
        unpack2(part[c][1], p2v, p3v);
        float total = (p0v + p1v) + (p2v + p3v);
        for (int offset = NS >> 1; offset > 0; offset >>= 1) total += __shfl_xor_sync(0xffffffffu, total, offset);
        const int p = p0 + pl * CPT + c;
        if (s == 0 && p < P) y[(size_t)(begin + base + tt) * inner + head * P + p] = total + skip * x[c];
      }
    }
    if (more) store(base + SSD_BATCH, smem + (turn ^ 1) * per_buffer);
    __syncthreads();
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c) {
    const int p = p0 + pl * CPT + c;
#pragma unroll
    for (int i = 0; i < SSD_ROWS_PER_THREAD / 2; ++i) {
      const int row = ssd_row(2 * i, s, NS);
      float lo, hi;
      unpack2(S[c][i], lo, hi);
      if (p < P && row < N) slot_state[(size_t)p * N + row] = lo;
      if (p < P && row + 1 < N) slot_state[(size_t)p * N + row + 1] = hi;
    }
  }
}

template <typename T, int CPT>
static void ssd_scan_launch(dim3 grid, size_t smem, cudaStream_t stream, const void* xbc, long long xbc_stride,
                            const void* dt_raw, long long dt_stride, const float* dt_bias, const float* a_log,
                            const float* d_skip, float* state, float* y, const int* query_start, const int* slots,
                            int heads, int groups, int P, int N, int NS) {
  auto kernel = ssd_scan_kernel<T, CPT>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ts_launch(kernel, grid, dim3(SSD_THREADS), smem, stream, (const T*)xbc, xbc_stride, (const T*)dt_raw, dt_stride, dt_bias,
            a_log, d_skip, state, y, query_start, slots, heads, groups, P, N, NS);
}

TS_EXPORT int ts_ssd_scan(int dtype, const void* xbc, long long xbc_stride, const void* dt_raw, long long dt_stride,
                          const float* dt_bias, const float* a_log, const float* d_skip, float* state, float* y,
                          const int* query_start, const int* slots, int num_seqs, int heads, int groups, int P, int N,
                          int num_tokens, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1) return TS_ERR_SIZE;
  if (dtype != TS_F32 && dtype != TS_BF16) return TS_ERR_DTYPE;
  int NS = 1;
  while (N > SSD_ROWS_PER_THREAD * NS) NS *= 2;
  if (NS > 32) return TS_ERR_SIZE;  // state sizes above 512 are not taken
  if (num_seqs > 65535) return TS_ERR_SIZE;
  // the most columns a thread that still leave two blocks for every multiprocessor; a step's requests
  // that bring nothing (padding) end at once, so the requests are counted by the step's tokens
  static int sms = 0;
  if (!sms) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  }
  const int live = num_tokens > 0 && num_tokens < num_seqs ? num_tokens : num_seqs;
  int cpt = 2;  // four columns a thread were measured too: slower than two on every shape (registers)
  while (cpt > 1) {
    const int tile = SSD_THREADS / NS * cpt;
    if (tile <= 2 * P && (long long)heads * live * ((P + tile - 1) / tile) >= 2LL * sms) break;
    cpt >>= 1;
  }
  static int forced = -1;  // TURBOSERVE_B200_SCAN_COLUMNS=1|2 overrides the choice (for measurements)
  if (forced < 0) {
    const char* env = getenv("TURBOSERVE_B200_SCAN_COLUMNS");
    forced = env ? atoi(env) : 0;
  }
  if (forced == 1 || forced == 2) cpt = forced;
  const int p_tile = SSD_THREADS / NS * cpt;
  const int tiles = (P + p_tile - 1) / p_tile;
  if (tiles > 65535) return TS_ERR_SIZE;
  const size_t smem = (size_t)2 * SSD_BATCH * (2 * SSD_ROWS_PER_THREAD * NS + p_tile + 2) * sizeof(float);
  dim3 grid(heads, num_seqs, tiles);
#define SSD_CASE(TYPE, COLS)                                                                                          \
  ssd_scan_launch<TYPE, COLS>(grid, smem, stream, xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, d_skip, state, y, \
                              query_start, slots, heads, groups, P, N, NS)
  if (dtype == TS_F32) {
    if (cpt == 2) SSD_CASE(float, 2); else SSD_CASE(float, 1);
  } else {
    if (cpt == 2) SSD_CASE(__nv_bfloat16, 2); else SSD_CASE(__nv_bfloat16, 1);
  }
#undef SSD_CASE
  return ts_launch_status();
}

template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ z, long long z_stride,
                                        const float* __restrict__ weight, T* __restrict__ out, int inner, int parts,
                                        float eps, int cached) {
  extern __shared__ float gated[];  // the part's gated values, when they fit
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger<1>();
  const int t = blockIdx.x, part = blockIdx.y;
  const int width = inner / parts;
  const float* y_row = y + (size_t)t * inner + (size_t)part * width;
  const T* z_row = z + (size_t)t * z_stride + (size_t)part * width;
  float squares = 0.0f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float gate = to_float(z_row[i]);
    const float v = y_row[i] * (gate / (1.0f + expf(-gate)));
    if (cached) gated[i] = v;
    squares = fmaf(v, v, squares);
  }
  const float total = block_sum(squares, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  T* o_row = out + (size_t)t * inner + (size_t)part * width;
  const float* w = weight + (size_t)part * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v;
    if (cached) {
      v = gated[i];
    } else {
      const float gate = to_float(z_row[i]);
      v = y_row[i] * (gate / (1.0f + expf(-gate)));
    }
    o_row[i] = from_float<T>(v * inv * w[i]);
  }
}

TS_EXPORT int ts_gated_group_norm(int dtype, const float* y, const void* z, long long z_stride, const float* weight,
                                  void* out, int num_tokens, int inner, int parts, float eps, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (inner < 1 || parts < 1 || inner % parts || parts > 65535) return TS_ERR_SIZE;
  const int width = inner / parts;
  int threads = (width + 31) / 32 * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  dim3 grid(num_tokens, parts);
  const int cached = (size_t)width * sizeof(float) <= 40 * 1024;
  const size_t smem = cached ? (size_t)width * sizeof(float) : 0;
  if (dtype == TS_F32)
    ts_launch(gated_group_norm_kernel<float>, grid, dim3(threads), smem, stream, y, (const float*)z, z_stride, weight,
              (float*)out, inner, parts, eps, cached);
  else if (dtype == TS_BF16)
    ts_launch(gated_group_norm_kernel<__nv_bfloat16>, grid, dim3(threads), smem, stream, y, (const __nv_bfloat16*)z, z_stride,
              weight, (__nv_bfloat16*)out, inner, parts, eps, cached);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

// ---------------------------------------------------------------------------------------
// selective_scan: the state-space recurrence with a state per channel and a decay per channel and state index.
//
// Per channel c (of `inner`), state index n (of N) and position t, all in fp32:
//
//   dt_t[c]  = softplus(dt_raw_t[c] + dt_bias[c])
//   S_t[c,n] = exp(dt_t[c] * A[c,n]) * S_{t-1}[c,n] + dt_t[c] * x_t[c] * B_t[n],        A = -exp(A_log)
//   y_t[c]   = sum_n S_t[c,n] * C_t[n] + D[c] * x_t[c]
//   out_t[c] = y_t[c] * silu(z_t[c])                                  (rounded once)
//
// x is the convolved and activated input, B_t and C_t columns of the low-rank projection of x, dt_raw the fp32
// product of its first columns with the step-size matrix, z the gate half of the input projection.  The state of a
// request lives in its slot ([slots][inner][N], fp32), is read once before the step's first position of the
// request and written once after its last.  A block owns one request and SEL_THREADS / L channels; L lanes share a
// channel, lane l holding states l, l + L, ... in registers (at most SEL_PER_LANE of them), and add their parts of
// y by shuffles in a fixed order.  Positions come `batch` at a time through shared memory (as many as fit, up to
// SEL_BATCH).  L follows from `inner` and N alone: the fewest lanes that leave a lane SEL_PER_LANE states, then doubled
// while the grid of one request has fewer than SEL_BLOCKS blocks, so that one long portion fills the SMs; a block is a
// warp group with little shared memory, so several are resident per SM and one's loads hide behind another's
// arithmetic.  One token per request and long portions run the same code, so an output is the same bits however a
// request is cut into steps.
// ---------------------------------------------------------------------------------------
#define SEL_THREADS 128
#define SEL_BATCH 32
#define SEL_BLOCKS 296  // two blocks for each of 148 SMs
#define SEL_SMEM (40 * 1024)
#define SEL_PER_LANE 16

template <typename T, int NPL>  // NPL: states a lane (1, 2, 4, 8 or 16)
__global__ void __launch_bounds__(SEL_THREADS)
selective_scan_kernel(const T* __restrict__ x, long long x_stride, const float* __restrict__ dt_raw,
                      const float* __restrict__ dt_bias, const T* __restrict__ bc, long long bc_stride, int b_first,
                      int c_first, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      const T* __restrict__ z, long long z_stride, float* __restrict__ state, T* __restrict__ out,
                      long long out_stride, const int* __restrict__ query_start, const int* __restrict__ slots, int inner,
                      int n_state, int lanes, int batch) {
  extern __shared__ __align__(16) float sel_smem[];
  const int channels = SEL_THREADS / lanes;              // channels a block
  const int npad = lanes * NPL;                          // states, padded
  float* x_s = sel_smem;                                 // [batch][channels]
  float* dt_s = x_s + batch * channels;                  // [batch][channels]
  float* z_s = dt_s + batch * channels;                  // [batch][channels]
  float* y_s = z_s + batch * channels;                   // [batch][channels]
  float* b_s = y_s + batch * channels;                   // [batch][npad]
  float* c_s = b_s + batch * npad;                       // [batch][npad]
  const int seq = blockIdx.x, tid = threadIdx.x;
  const int dl = tid % lanes, cl = tid / lanes, ch = blockIdx.y * channels + cl;
  const bool live = ch < inner;
  float a[NPL], s[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = dl + i * lanes;
    a[i] = (live && n < n_state) ? -expf(a_log[(size_t)ch * n_state + n]) : 0.0f;
  }
  pdl_wait();
  pdl_trigger();
  const int first = query_start[seq], last = query_start[seq + 1];
  if (last <= first) return;
  float* s_ptr = state + ((size_t)slots[seq] * inner + (live ? ch : 0)) * n_state;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = dl + i * lanes;
    s[i] = (live && n < n_state) ? s_ptr[n] : 0.0f;
  }
  for (int t0 = first; t0 < last; t0 += batch) {
    const int count = min(batch, last - t0);
    __syncthreads();  // everyone is done with the batch before
#pragma unroll 4
    for (int idx = tid; idx < count * channels; idx += SEL_THREADS) {
      const int p = idx / channels, c = blockIdx.y * channels + idx % channels;
      float xv = 0.0f, dv = 0.0f, zv = 0.0f;
      if (c < inner) {
        xv = to_float(x[(size_t)(t0 + p) * x_stride + c]);
        const float raw = dt_raw[(size_t)(t0 + p) * inner + c] + dt_bias[c];
        dv = raw > 20.0f ? raw : log1pf(expf(raw));
        zv = to_float(z[(size_t)(t0 + p) * z_stride + c]);
      }
      x_s[idx] = xv;
      dt_s[idx] = dv;
      z_s[idx] = zv;
    }
#pragma unroll 4
    for (int idx = tid; idx < count * npad; idx += SEL_THREADS) {
      const int p = idx / npad, n = idx % npad;
      const T* row = bc + (size_t)(t0 + p) * bc_stride;
      b_s[idx] = n < n_state ? to_float(row[b_first + n]) : 0.0f;
      c_s[idx] = n < n_state ? to_float(row[c_first + n]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 4
    for (int p = 0; p < count; ++p) {
      const float dt = dt_s[p * channels + cl];
      const float dx = dt * x_s[p * channels + cl];
      const float* bp = b_s + p * npad + dl;
      const float* cp = c_s + p * npad + dl;
      float y = 0.0f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        s[i] = fmaf(expf(dt * a[i]), s[i], dx * bp[i * lanes]);
        y = fmaf(s[i], cp[i * lanes], y);
      }
      for (int offset = lanes >> 1; offset > 0; offset >>= 1) y += __shfl_xor_sync(0xffffffffu, y, offset);
      if (dl == 0) y_s[p * channels + cl] = y;
    }
    __syncthreads();
    // the skip, the gate and the store, once per output and along the channels
    for (int idx = tid; idx < count * channels; idx += SEL_THREADS) {
      const int p = idx / channels, c = blockIdx.y * channels + idx % channels;
      if (c < inner) {
        const float zv = z_s[idx];
        out[(size_t)(t0 + p) * out_stride + c] = from_float<T>(fmaf(d_skip[c], x_s[idx], y_s[idx]) * (zv / (1.0f + expf(-zv))));
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = dl + i * lanes;
      if (n < n_state) s_ptr[n] = s[i];
    }
  }
}

template <typename T>
static int launch_selective_scan(const T* x, long long x_stride, const float* dt_raw, const float* dt_bias, const T* bc,
                                 long long bc_stride, int b_first, int c_first, const float* a_log, const float* d_skip,
                                 const T* z, long long z_stride, float* state, T* out, long long out_stride,
                                 const int* query_start, const int* slots, int num_seqs, int inner, int n_state,
                                 cudaStream_t stream) {
  // lanes a channel: the fewest (a power of two up to 32) that leave a lane at most SEL_PER_LANE states; a lane's
  // count is rounded up to a power of two
  int lanes = 1;
  while (lanes < 32 && (n_state + lanes - 1) / lanes > SEL_PER_LANE) lanes <<= 1;
  // ... then more lanes (down to one state a lane) while one request's blocks would not fill the SMs
  while (lanes < 32 && lanes < n_state && (long long)inner * lanes < (long long)SEL_BLOCKS * SEL_THREADS) lanes <<= 1;
  int npl = 1;
  while (npl * lanes < n_state) npl <<= 1;
  if (npl > SEL_PER_LANE) return TS_ERR_SIZE;
  const int channels = SEL_THREADS / lanes;
  int batch = SEL_BATCH;
  while (batch > 4 && (size_t)batch * (4 * channels + 2 * lanes * npl) * sizeof(float) > SEL_SMEM) batch >>= 1;
  dim3 grid(num_seqs, (inner + channels - 1) / channels);
  if (grid.y > 65535) return TS_ERR_SIZE;
  const size_t smem = (size_t)batch * (4 * channels + 2 * lanes * npl) * sizeof(float);
#define SEL_LAUNCH(N)                                                                                                    \
  ts_launch(selective_scan_kernel<T, N>, grid, dim3(SEL_THREADS), smem, stream, x, x_stride, dt_raw, dt_bias, bc, bc_stride, \
            b_first, c_first, a_log, d_skip, z, z_stride, state, out, out_stride, query_start, slots, inner, n_state, lanes, batch)
  switch (npl) {
    case 1: SEL_LAUNCH(1); break;
    case 2: SEL_LAUNCH(2); break;
    case 4: SEL_LAUNCH(4); break;
    case 8: SEL_LAUNCH(8); break;
    default: SEL_LAUNCH(16); break;
  }
#undef SEL_LAUNCH
  return ts_launch_status();
}

TS_EXPORT int ts_selective_scan(int dtype, const void* x, long long x_stride, const float* dt_raw, const float* dt_bias,
                                const void* bc, long long bc_stride, int b_first, int c_first, const float* a_log,
                                const float* d_skip, const void* z, long long z_stride, float* state, void* out,
                                long long out_stride, const int* query_start, const int* slots, int num_seqs, int inner,
                                int n_state, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (inner < 1 || n_state < 1 || n_state > 32 * SEL_PER_LANE) return TS_ERR_SIZE;
  if (dtype == TS_F32)
    return launch_selective_scan<float>((const float*)x, x_stride, dt_raw, dt_bias, (const float*)bc, bc_stride, b_first,
                                        c_first, a_log, d_skip, (const float*)z, z_stride, state, (float*)out, out_stride,
                                        query_start, slots, num_seqs, inner, n_state, stream);
  if (dtype == TS_BF16)
    return launch_selective_scan<__nv_bfloat16>((const __nv_bfloat16*)x, x_stride, dt_raw, dt_bias, (const __nv_bfloat16*)bc,
                                                bc_stride, b_first, c_first, a_log, d_skip, (const __nv_bfloat16*)z, z_stride,
                                                state, (__nv_bfloat16*)out, out_stride, query_start, slots, num_seqs, inner,
                                                n_state, stream);
  return TS_ERR_DTYPE;
}
