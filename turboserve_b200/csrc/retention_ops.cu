// Retention: linear attention with a fixed decay per head, no softmax and no denominator.
//
//   retention_prepare  per token: q_t, k_t = rotate(q_t), rotate(k_t) * key_scale in fp32 (angles p * f_i, cos and
//                      sin times a constant), written as fp32 in the order the scan's threads read them, and v_t
//                      as fp32; once per token and head, whatever the number of blocks that scan the head
//   retention_scan     per request and head, over the step's positions in order:
//                          S_t = decay_h S_{t-1} + k_t v_t^T                       (S: dim x vdim, fp32)
//                          y_t = S_t^T q_t
//                      The state of a request lives in its slot as [heads][vdim][dim] fp32; it is read once
//                      before the step's first position and written once after its last.
//   head_norm_gate     out = y / rms_head(y) * silu(g): every head's y divided by its root mean square (eps
//                      inside the root, no weight), times the gate, rounded once.
//
// Two more forms share these kernels.  With `in_act` = 1 the prepare kernel applies silu to q, k and v as it reads
// them (linear attention whose projections pass an activation).  With rows of decays (`decay_raw`, fp32, one per
// token, head and key channel, from which w = exp(-exp(decay_raw + decay_bias)) is made in fp32) and a bonus u per
// head and key channel, the scan is the time-mixing recurrence with a decay the input chooses:
//     y_t = (S_{t-1} + diag(u) k_t v_t^T)^T q_t,        S_t = diag(w_t) S_{t-1} + k_t v_t^T
// the current token entering its own output through the bonus alone.
//
// A block of the scan owns one (request, head, slice of value columns).  DS lanes share a value column, each
// holding RPT rows of the state in registers (rows dl * RPT .. + RPT - 1, padded with zeros beyond dim); the
// column's output is their partial sums added by shuffles in a fixed order.  Positions come eight at a time
// through two buffers of shared memory filled by cp.async a batch ahead.  Every sum of a position has one
// order whatever the cut of the request into steps, so a position's output is the same bits decoded alone or
// inside a prompt.
#include "common.cuh"

#define RS_THREADS 128
#define RS_BATCH 8

// Rows a thread and lanes a column for a head size: 8 rows up to 128, 16 up to 256; DS a power of two <= 16.
static inline void retention_tiling(int dim, int* rpt, int* ds) {
  *rpt = dim <= 128 ? 8 : 16;
  int d = 1;
  while (d * *rpt < dim) d <<= 1;
  *ds = d;
}

// qk: [tokens][heads][planes][padded] fp32 (planes: q, k and, with decays, w), row r of a head at
// (r % RPT) * DS + r / RPT; vf: [tokens][heads][vpad] fp32.
template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ qkv, long long stride, int q_first, int k_first,
                                         int v_first, const float* __restrict__ inv_freq, int rot, float amplitude,
                                         float key_scale, const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token, float* __restrict__ qk,
                                         float* __restrict__ vf, int heads, int dim, int vdim, int rpt, int ds, int vpad,
                                         int in_act, const float* __restrict__ decay_raw,
                                         const float* __restrict__ decay_bias) {
  extern __shared__ float rp_smem[];  // cos[rot / 2], sin[rot / 2]
  const int t = blockIdx.x, half = rot / 2, padded = rpt * ds;
  float* cos_s = rp_smem;
  float* sin_s = rp_smem + half;
  pdl_wait();
  pdl_trigger<64>();
  if (seq_of_token[t] < 0) return;
  const int pos = positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    cos_s[i] = cs * amplitude;
    sin_s[i] = sn * amplitude;
  }
  __syncthreads();
  const T* row = qkv + (size_t)t * stride;
  const int planes = decay_raw ? 3 : 2;
  auto silu_of = [](float z) { return z / (1.0f + expf(-z)); };
  for (int idx = threadIdx.x; idx < heads * padded; idx += blockDim.x) {
    const int h = idx / padded, at = idx % padded;
    const int r = (at % ds) * rpt + at / ds;
    float qv = 0.0f, kv = 0.0f, wv = 0.0f;
    if (r < dim) {
      const T* qh = row + q_first + (size_t)h * dim;
      const T* kh = row + k_first + (size_t)h * dim;
      qv = to_float(qh[r]);
      kv = to_float(kh[r]);
      if (in_act) {
        qv = silu_of(qv);
        kv = silu_of(kv);
      }
      if (decay_raw) wv = expf(-expf(decay_raw[((size_t)t * heads + h) * dim + r] + decay_bias[(size_t)h * dim + r]));
      if (r < rot) {  // the pair (u, v) becomes (u cos - v sin, v cos + u sin)
        const int i = r < half ? r : r - half;
        const float qm = to_float(qh[r < half ? r + half : r - half]), km = to_float(kh[r < half ? r + half : r - half]);
        qv = r < half ? qv * cos_s[i] - qm * sin_s[i] : qv * cos_s[i] + qm * sin_s[i];
        kv = r < half ? kv * cos_s[i] - km * sin_s[i] : kv * cos_s[i] + km * sin_s[i];
      }
      kv *= key_scale;
    }
    float* to = qk + (((size_t)t * heads + h) * planes) * padded + at;
    to[0] = qv;
    to[padded] = kv;
    if (decay_raw) to[2 * padded] = wv;
  }
  for (int idx = threadIdx.x; idx < heads * vpad; idx += blockDim.x) {
    const int h = idx / vpad, c = idx % vpad;
    float v = c < vdim ? to_float(row[v_first + (size_t)h * vdim + c]) : 0.0f;
    if (in_act) v = silu_of(v);
    vf[(size_t)t * heads * vpad + idx] = v;
  }
}

__device__ __forceinline__ void rs_copy16(float* to, const float* from) {
  const unsigned addr = (unsigned)__cvta_generic_to_shared(to);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(from) : "memory");
}

template <int RPT, bool CHOSEN>  // CHOSEN: a decay per position and key channel, and a bonus (`decay` then holds the bonus)
__global__ void __launch_bounds__(RS_THREADS)
retention_scan_kernel(const float* __restrict__ qk, const float* __restrict__ vf, const float* __restrict__ decay,
                      const int* __restrict__ query_start, const int* __restrict__ slots, float* __restrict__ state,
                      float* __restrict__ y, int heads, int dim, int vdim, int ds, int vpad) {
  extern __shared__ __align__(16) float rs_smem[];
  const int padded = ds * RPT;
  const int cols = RS_THREADS / ds;
  constexpr int PLANES = CHOSEN ? 3 : 2;
  const int per_position = PLANES * padded + cols;       // floats of one position: q, k, (w,) the block's value columns
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x, dl = tid % ds, col = col0 + tid / ds;
  pdl_wait();
  pdl_trigger();
  const int first = query_start[seq], last = query_start[seq + 1];
  if (last <= first) return;
  const int slot = slots[seq];
  const float gamma = CHOSEN ? 0.0f : decay[head];
  const bool live = col < vdim;
  float bonus[CHOSEN ? RPT : 1];
  if constexpr (CHOSEN) {
#pragma unroll
    for (int i = 0; i < RPT; ++i) bonus[i] = dl * RPT + i < dim ? decay[(size_t)head * dim + dl * RPT + i] : 0.0f;
  }

  auto fetch = [&](int t0, float* to) {
    const int count = min(RS_BATCH, last - t0);
    const int q_chunks = PLANES * padded / 4, v_chunks = cols / 4;
    for (int idx = tid; idx < count * (q_chunks + v_chunks); idx += RS_THREADS) {
      const int p = idx / (q_chunks + v_chunks), c = idx % (q_chunks + v_chunks);
      if (c < q_chunks)
        rs_copy16(to + p * per_position + 4 * c, qk + (((size_t)(t0 + p) * heads + head) * PLANES) * padded + 4 * c);
      else
        rs_copy16(to + p * per_position + PLANES * padded + 4 * (c - q_chunks),
                  vf + ((size_t)(t0 + p) * heads + head) * vpad + col0 + 4 * (c - q_chunks));
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(first, rs_smem);

  float* s_ptr = state + (((size_t)slot * heads + head) * vdim + (live ? col : 0)) * dim + dl * RPT;
  float s[RPT];
  if (dim % 4 == 0) {
#pragma unroll
    for (int i = 0; i < RPT; i += 4) {
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (live && dl * RPT + i < dim) v = *reinterpret_cast<const float4*>(s_ptr + i);
      s[i] = v.x; s[i + 1] = v.y; s[i + 2] = v.z; s[i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < RPT; ++i) s[i] = (live && dl * RPT + i < dim) ? s_ptr[i] : 0.0f;
  }

  int buffer = 0;
  for (int t0 = first; t0 < last; t0 += RS_BATCH, buffer ^= 1) {
    const int count = min(RS_BATCH, last - t0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // this batch has landed for everyone, and everyone is done with the other buffer
    if (t0 + RS_BATCH < last) fetch(t0 + RS_BATCH, rs_smem + (buffer ^ 1) * RS_BATCH * per_position);
    const float* base = rs_smem + buffer * RS_BATCH * per_position;
    if constexpr (CHOSEN) {
      // the rows of the state sit at dl * RPT + i; element i of a plane for this lane at i * ds + dl
      for (int p = 0; p < count; ++p) {
        const float* qp = base + p * per_position + dl;
        const float* kp = qp + padded;
        const float* wp = qp + 2 * padded;
        const float v = base[p * per_position + 3 * padded + tid / ds];
        float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
        for (int i = 0; i < RPT; i += 2) {
          const float kv0 = kp[i * ds] * v, kv1 = kp[(i + 1) * ds] * v;
          o0 = fmaf(fmaf(bonus[i], kv0, s[i]), qp[i * ds], o0);
          o1 = fmaf(fmaf(bonus[i + 1], kv1, s[i + 1]), qp[(i + 1) * ds], o1);
          s[i] = fmaf(wp[i * ds], s[i], kv0);
          s[i + 1] = fmaf(wp[(i + 1) * ds], s[i + 1], kv1);
        }
        float o = o0 + o1;
        for (int offset = ds >> 1; offset > 0; offset >>= 1) o += __shfl_xor_sync(0xffffffffu, o, offset);
        if (dl == 0 && live) y[(size_t)(t0 + p) * heads * vdim + (size_t)head * vdim + col] = o;
      }
      continue;
    }
    if (count == RS_BATCH) {
      // a full batch, unrolled: the positions depend on one another through the state alone (one multiply-add
      // deep), so their loads, partial sums and shuffles overlap
      float o[RS_BATCH];
#pragma unroll
      for (int half = 0; half < RS_BATCH; half += 4) {
        // four positions' inputs into registers first, then their multiply-adds: the loads do not wait on one another
        float kr[4][RPT], qr[4][RPT], vr[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float* qp = base + (half + p) * per_position + dl;
          vr[p] = base[(half + p) * per_position + 2 * padded + tid / ds];
#pragma unroll
          for (int i = 0; i < RPT; ++i) {
            qr[p][i] = qp[i * ds];
            kr[p][i] = qp[padded + i * ds];
          }
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
          for (int i = 0; i < RPT; i += 2) {
            s[i] = fmaf(gamma, s[i], kr[p][i] * vr[p]);
            s[i + 1] = fmaf(gamma, s[i + 1], kr[p][i + 1] * vr[p]);
            o0 = fmaf(s[i], qr[p][i], o0);
            o1 = fmaf(s[i + 1], qr[p][i + 1], o1);
          }
          o[half + p] = o0 + o1;
        }
      }
      for (int offset = ds >> 1; offset > 0; offset >>= 1) {
#pragma unroll
        for (int p = 0; p < RS_BATCH; ++p) o[p] += __shfl_xor_sync(0xffffffffu, o[p], offset);
      }
      if (dl == 0 && live) {
#pragma unroll
        for (int p = 0; p < RS_BATCH; ++p) y[(size_t)(t0 + p) * heads * vdim + (size_t)head * vdim + col] = o[p];
      }
      continue;
    }
    for (int p = 0; p < count; ++p) {
      const float* qp = base + p * per_position + dl;
      const float* kp = qp + padded;
      const float v = base[p * per_position + 2 * padded + tid / ds];
      float o0 = 0.0f, o1 = 0.0f;
#pragma unroll
      for (int i = 0; i < RPT; i += 2) {
        s[i] = fmaf(gamma, s[i], kp[i * ds] * v);
        s[i + 1] = fmaf(gamma, s[i + 1], kp[(i + 1) * ds] * v);
        o0 = fmaf(s[i], qp[i * ds], o0);
        o1 = fmaf(s[i + 1], qp[(i + 1) * ds], o1);
      }
      float o = o0 + o1;
      for (int offset = ds >> 1; offset > 0; offset >>= 1) o += __shfl_xor_sync(0xffffffffu, o, offset);
      if (dl == 0 && live) y[(size_t)(t0 + p) * heads * vdim + (size_t)head * vdim + col] = o;
    }
  }
  if (live) {
    if (dim % 4 == 0) {
#pragma unroll
      for (int i = 0; i < RPT; i += 4)
        if (dl * RPT + i < dim) *reinterpret_cast<float4*>(s_ptr + i) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < RPT; ++i)
        if (dl * RPT + i < dim) s_ptr[i] = s[i];
    }
  }
}

// Floats of scratch the scan needs per token: the rotated q and k and the values in fp32, in the scan's order.
TS_EXPORT int ts_retention_scratch_per_token(int heads, int dim, int vdim) {
  int rpt, ds;
  retention_tiling(dim, &rpt, &ds);
  const int cols = RS_THREADS / ds;
  return heads * (2 * rpt * ds + (vdim + cols - 1) / cols * cols);
}

// The same for the form with a decay per position and key channel (one more plane).
TS_EXPORT int ts_chosen_decay_scratch_per_token(int heads, int dim, int vdim) {
  int rpt, ds;
  retention_tiling(dim, &rpt, &ds);
  const int cols = RS_THREADS / ds;
  return heads * (3 * rpt * ds + (vdim + cols - 1) / cols * cols);
}

// decay: one value per head (decay_raw null), or the bonus [heads][dim] (with decay_raw [tokens][heads * dim] and
// decay_bias [heads * dim]).  in_act 1: silu on q, k and v as they are read (not together with a rotation).
static int retention_scan_any(int dtype, const void* qkv, long long stride, int q_first, int k_first, int v_first,
                              const float* decay, const float* inv_freq, int rot, float amplitude, float key_scale,
                              int in_act, const float* decay_raw, const float* decay_bias, const int* positions,
                              const int* seq_of_token, const int* query_start, const int* slots, float* state, float* y,
                              float* scratch, int num_tokens, int num_seqs, int heads, int dim, int vdim,
                              cudaStream_t stream) {
  if (num_seqs <= 0 || num_tokens <= 0) return 0;
  if (dim < 1 || dim > 256 || vdim < 1 || heads < 1 || heads > 65535 || rot < 0 || rot % 2 || rot > dim) return TS_ERR_SIZE;
  if ((uintptr_t)scratch & 15) return TS_ERR_ALIGN;
  if ((in_act && rot) || in_act < 0 || in_act > 1 || (decay_raw && !decay_bias)) return TS_ERR_ARGUMENT;
  int rpt, ds;
  retention_tiling(dim, &rpt, &ds);
  const int cols = RS_THREADS / ds, padded = rpt * ds;
  const int vpad = (vdim + cols - 1) / cols * cols;
  const int planes = decay_raw ? 3 : 2;
  float* qk = scratch;
  float* vf = scratch + (size_t)num_tokens * heads * planes * padded;
  const size_t prepare_smem = (size_t)rot * sizeof(float);
  if (dtype == TS_F32)
    ts_launch(retention_prepare_kernel<float>, dim3(num_tokens), dim3(128), prepare_smem, stream, (const float*)qkv, stride,
              q_first, k_first, v_first, inv_freq, rot, amplitude, key_scale, positions, seq_of_token, qk, vf, heads, dim,
              vdim, rpt, ds, vpad, in_act, decay_raw, decay_bias);
  else if (dtype == TS_BF16)
    ts_launch(retention_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), prepare_smem, stream,
              (const __nv_bfloat16*)qkv, stride, q_first, k_first, v_first, inv_freq, rot, amplitude, key_scale, positions,
              seq_of_token, qk, vf, heads, dim, vdim, rpt, ds, vpad, in_act, decay_raw, decay_bias);
  else
    return TS_ERR_DTYPE;
  dim3 grid(num_seqs, heads, vpad / cols);
  const size_t smem = (size_t)2 * RS_BATCH * (planes * padded + cols) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaFuncSetAttribute(retention_scan_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(retention_scan_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  const float* cf_qk = qk;
  const float* cf_vf = vf;
  if (decay_raw) {
    if (rpt == 8)
      ts_launch(retention_scan_kernel<8, true>, grid, dim3(RS_THREADS), smem, stream, cf_qk, cf_vf, decay, query_start, slots,
                state, y, heads, dim, vdim, ds, vpad);
    else
      ts_launch(retention_scan_kernel<16, true>, grid, dim3(RS_THREADS), smem, stream, cf_qk, cf_vf, decay, query_start, slots,
                state, y, heads, dim, vdim, ds, vpad);
  } else if (rpt == 8) {
    ts_launch(retention_scan_kernel<8, false>, grid, dim3(RS_THREADS), smem, stream, cf_qk, cf_vf, decay, query_start, slots,
              state, y, heads, dim, vdim, ds, vpad);
  } else {
    ts_launch(retention_scan_kernel<16, false>, grid, dim3(RS_THREADS), smem, stream, cf_qk, cf_vf, decay, query_start, slots,
              state, y, heads, dim, vdim, ds, vpad);
  }
  return ts_launch_status();
}

TS_EXPORT int ts_retention_scan(int dtype, const void* qkv, long long stride, int q_first, int k_first, int v_first,
                                const float* decay, const float* inv_freq, int rot, float amplitude,
                                float key_scale, const int* positions, const int* seq_of_token, const int* query_start,
                                const int* slots, float* state, float* y, float* scratch, int num_tokens, int num_seqs,
                                int heads, int dim, int vdim, cudaStream_t stream) {
  return retention_scan_any(dtype, qkv, stride, q_first, k_first, v_first, decay, inv_freq, rot, amplitude, key_scale, 0,
                            nullptr, nullptr, positions, seq_of_token, query_start, slots, state, y, scratch, num_tokens,
                            num_seqs, heads, dim, vdim, stream);
}

// Retention whose q, k and v pass an activation first (in_act 1: silu).
TS_EXPORT int ts_retention_scan_act(int dtype, const void* qkv, long long stride, int q_first, int k_first, int v_first,
                                    const float* decay, float key_scale, int in_act, const int* positions,
                                    const int* seq_of_token, const int* query_start, const int* slots, float* state,
                                    float* y, float* scratch, int num_tokens, int num_seqs, int heads, int dim, int vdim,
                                    cudaStream_t stream) {
  return retention_scan_any(dtype, qkv, stride, q_first, k_first, v_first, decay, nullptr, 0, 1.0f, key_scale, in_act,
                            nullptr, nullptr, positions, seq_of_token, query_start, slots, state, y, scratch, num_tokens,
                            num_seqs, heads, dim, vdim, stream);
}

// The recurrence with a decay per position and key channel and a bonus for the current token.  q, k and v are read
// from three matrices' columns of one row stride (they may lie in one buffer); decay_raw is fp32 [tokens][heads * dim].
TS_EXPORT int ts_chosen_decay_scan(int dtype, const void* qkv, long long stride, int q_first, int k_first, int v_first,
                                   const float* bonus, const float* decay_raw, const float* decay_bias,
                                   const int* positions, const int* seq_of_token, const int* query_start, const int* slots,
                                   float* state, float* y, float* scratch, int num_tokens, int num_seqs, int heads, int dim,
                                   int vdim, cudaStream_t stream) {
  if (!decay_raw || !decay_bias || !bonus) return TS_ERR_ARGUMENT;
  return retention_scan_any(dtype, qkv, stride, q_first, k_first, v_first, bonus, nullptr, 0, 1.0f, 1.0f, 0, decay_raw,
                            decay_bias, positions, seq_of_token, query_start, slots, state, y, scratch, num_tokens, num_seqs,
                            heads, dim, vdim, stream);
}

// One warp per (token, part): a row of y is cut into `parts` equal parts of `width` elements, each divided by its
// own root mean square (the heads of a row one by one, or the whole row at once), times `weight` (a row's worth
// of floats, or none), times act(gate): silu (0) or the logistic sigmoid (1).
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ y, const T* __restrict__ gate, long long gate_stride,
                                      T* __restrict__ out, long long pairs, int heads, int vdim, float eps,
                                      const float* __restrict__ weight, int gate_act) {
  pdl_wait();
  pdl_trigger<1>();
  const long long pair = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = pair / heads;
  const int head = (int)(pair % heads);
  const float* row = y + (size_t)pair * vdim;
  float sum_sq = 0.0f;
  for (int i = lane; i < vdim; i += 32) sum_sq = fmaf(row[i], row[i], sum_sq);
  sum_sq = warp_sum(sum_sq);
  const float inv = 1.0f / sqrtf(sum_sq / (float)vdim + eps);
  const T* g = gate + (size_t)t * gate_stride + (size_t)head * vdim;
  const float* w = weight ? weight + (size_t)head * vdim : nullptr;
  T* o = out + (size_t)pair * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float z = to_float(g[i]);
    const float sigmoid = 1.0f / (1.0f + expf(-z));
    float v = row[i] * inv;
    if (w) v *= w[i];
    o[i] = from_float<T>(v * (gate_act == 1 ? sigmoid : z * sigmoid));
  }
}

static int head_norm_gate_any(int dtype, const float* y, const void* gate, long long gate_stride, void* out,
                              int num_tokens, int heads, int vdim, float eps, const float* weight, int gate_act,
                              cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (heads < 1 || vdim < 1) return TS_ERR_SIZE;
  if (gate_act < 0 || gate_act > 1) return TS_ERR_ARGUMENT;
  const long long pairs = (long long)num_tokens * heads;
  const int warps = 8;
  const unsigned blocks = (unsigned)((pairs + warps - 1) / warps);
  if (dtype == TS_F32)
    ts_launch(head_norm_gate_kernel<float>, dim3(blocks), dim3(32 * warps), 0, stream, y, (const float*)gate, gate_stride,
              (float*)out, pairs, heads, vdim, eps, weight, gate_act);
  else if (dtype == TS_BF16)
    ts_launch(head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(32 * warps), 0, stream, y,
              (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, pairs, heads, vdim, eps, weight, gate_act);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}

TS_EXPORT int ts_head_norm_gate(int dtype, const float* y, const void* gate, long long gate_stride, void* out,
                                int num_tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  return head_norm_gate_any(dtype, y, gate, gate_stride, out, num_tokens, heads, vdim, eps, nullptr, 0, stream);
}

// parts * width is a row of y; weight may be null.
TS_EXPORT int ts_part_norm_gate(int dtype, const float* y, const void* gate, long long gate_stride, void* out,
                                int num_tokens, int parts, int width, float eps, const float* weight, int gate_act,
                                cudaStream_t stream) {
  return head_norm_gate_any(dtype, y, gate, gate_stride, out, num_tokens, parts, width, eps, weight, gate_act, stream);
}
