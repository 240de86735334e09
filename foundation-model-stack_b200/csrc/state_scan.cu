// Mixers that carry a matrix of state per head from token to token, and the short causal convolutions in front of
// them.  Everything that enters a recurrence is float32: step sizes, decays, gates, unit norms, the state itself;
// the state of every sequence lies in float32 between steps and a step starts from what its slot holds.
//
//   causal_conv         y[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1) + j, c]) over the rows of one sequence;
//                       the rows before a step's first come from the slot's tail (the last taps - 1 inputs, zeros for
//                       a new sequence); a second kernel leaves the tail for the next step
//   selective_scan      per head, S [state, vdim]:  S = exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
//                       with dt = softplus(dt_raw + dt_bias); B and C are shared by the heads of a group
//   delta_rule_scan     per head, S [dim, vdim]:  S = diag(g) S;  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q
//                       with q, k unit vectors (q also times dim^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias))
//   gated_group_rmsnorm rows cut into groups, each divided by its own root mean square, times a weight; a gate
//                       multiplies either before the norm (silu) or after it (sigmoid)
//
// The scans walk a sequence's tokens in order: one thread block per (sequence, head, run of value columns), a thread
// per (value column, every fourth state row) with its part of the state in registers; the tokens' vectors come
// through shared memory sixteen tokens at a time, and the four threads of a column add their sums by shuffles.  The
// order of the sums does not depend on how a prompt was cut into steps or on what else is in the batch.
// State layout: [slots, heads, vdim, rows] (the state's rows contiguous), so that a thread's part is one run.
#include "common.cuh"

// Kernels of a step may start while the kernel before them still runs (programmatic dependent launch); no pointer
// is declared __restrict__, and what the kernel right before wrote is read after griddepcontrol.wait.
namespace {
constexpr int CH = 16;      // tokens brought into shared memory at a time
constexpr int PARTS = 4;    // threads that share a value column
constexpr int VB = 32;      // value columns of a block (VB * PARTS = 128 threads)
constexpr int MAX_TAPS = 16;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

// ---- causal convolution ------------------------------------------------------------------------------
// x: rows of `stride` values (the convolved channels are its first `channels` from the pointer on); one thread per
// (row, channel)
template <typename T>
__global__ void causal_conv_kernel(const T* x, int stride, const float* w, const float* bias, const float* tail,
                                   const int* token_seq, const int* first_row, const int* slots, float* out,
                                   int n_tokens, int channels, int taps, int act, int n_seqs, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n_tokens * channels) return;
  const int t = (int)(i / channels), c = (int)(i - (size_t)t * channels);
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int local = t - first_row[seq];  // the row's place among its sequence's rows of this step
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const float* tl = tail + (size_t)slot * (taps - 1) * channels;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int back = taps - 1 - j;  // how many rows before this one
    const float v = back <= local ? to_f32(x[(size_t)(t - back) * stride + c])
                                  : tl[(size_t)(taps - 1 + local - back) * channels + c];
    acc = fmaf(w[(size_t)c * taps + j], v, acc);
  }
  out[i] = act ? acc * sigmoid_f(acc) : acc;
}

// the tail after the step: the last taps - 1 inputs of (old tail, the step's rows); one thread per (sequence, channel)
template <typename T>
__global__ void conv_tail_kernel(const T* x, int stride, float* tail, const int* first_row, const int* slots,
                                 int channels, int taps, int n_seqs, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, seq = blockIdx.y;
  if (c >= channels) return;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], n = first_row[seq + 1] - lo;
  float* tl = tail + (size_t)slot * (taps - 1) * channels;
  float keep[MAX_TAPS];
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps - 1) break;
    const int local = n - (taps - 1) + j;
    keep[j] = local >= 0 ? to_f32(x[(size_t)(lo + local) * stride + c]) : tl[(size_t)(j + n) * channels + c];
  }
#pragma unroll
  for (int j = 0; j < MAX_TAPS; ++j) {
    if (j >= taps - 1) break;
    tl[(size_t)j * channels + c] = keep[j];
  }
}

// ---- selective state-space scan ----------------------------------------------------------------------
// xbc [tokens, inner + 2 groups * N] float32 (after the convolution): x | B | C;  dt_raw: column `head` of rows of
// `dt_stride` values;  y [tokens, inner] float32.  NP: state rows a thread holds (N <= PARTS * NP).
template <typename T, int NP>
__global__ void selective_scan_kernel(const float* xbc, const T* dt_raw, int dt_stride, const float* dt_bias,
                                      const float* a_log, const float* d_skip, float* state, float* y,
                                      const int* first_row, const int* slots, int heads, int vdim, int n_state,
                                      int groups, int write_state, int n_slots) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, part = tid % PARTS, vl = tid / PARTS, v = v0 + vl;
  const bool v_ok = v < vdim;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  const int inner = heads * vdim, row_w = inner + 2 * groups * n_state;
  const int group = head / (heads / groups);
  float* sB = smem;                      // [CH][n_state]
  float* sC = sB + CH * n_state;         // [CH][n_state]
  float* sx = sC + CH * n_state;         // [CH][VB]
  float* sdt = sx + CH * VB;             // [CH]
  float* sdec = sdt + CH;                // [CH]
  const float A = expf(a_log[head]), D = d_skip[head], bias = dt_bias[head];
  float s[NP];
  float* st = state + (((size_t)slot * heads + head) * vdim + (v_ok ? v : 0)) * n_state;
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int n = j * PARTS + part;
    s[j] = (v_ok && n < n_state) ? st[n] : 0.f;
  }
  for (int c0 = lo; c0 < hi; c0 += CH) {
    const int cn = min(CH, hi - c0);
    __syncthreads();
    for (int i = tid; i < cn * n_state; i += blockDim.x) {
      const int t = i / n_state, n = i - t * n_state;
      const float* r = xbc + (size_t)(c0 + t) * row_w + inner + (size_t)group * n_state + n;
      sB[i] = r[0];
      sC[i] = r[(size_t)groups * n_state];
    }
    for (int i = tid; i < cn * VB; i += blockDim.x) {
      const int t = i / VB, e = i - t * VB;
      sx[i] = v0 + e < vdim ? xbc[(size_t)(c0 + t) * row_w + (size_t)head * vdim + v0 + e] : 0.f;
    }
    if (tid < cn) {
      const float dt = softplus_f(to_f32(dt_raw[(size_t)(c0 + tid) * dt_stride + head]) + bias);
      sdt[tid] = dt;
      sdec[tid] = expf(-A * dt);
    }
    __syncthreads();
    for (int t = 0; t < cn; ++t) {
      const float xv = sx[t * VB + vl], dtx = sdt[t] * xv, dec = sdec[t];
      const float* b = sB + t * n_state + part;
      const float* c = sC + t * n_state + part;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        if (j * PARTS + part < n_state) {
          s[j] = fmaf(dec, s[j], dtx * b[j * PARTS]);
          acc = fmaf(s[j], c[j * PARTS], acc);
        }
      }
      acc = quad_sum(acc);
      if (part == 0 && v_ok) y[(size_t)(c0 + t) * inner + (size_t)head * vdim + v] = fmaf(D, xv, acc);
    }
  }
  if (write_state && v_ok) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      const int n = j * PARTS + part;
      if (n < n_state) st[n] = s[j];
    }
  }
}

// ---- gated delta rule --------------------------------------------------------------------------------
// qkv [tokens, 2 kvheads * dim + heads * vdim] float32 (after the convolution): q | k | v;  beta_raw: column `head`
// of rows of `beta_stride` values;  a_raw [tokens, heads * dim] (the decay's projection);  o [tokens, heads * vdim]
template <typename T, int NP>
__global__ void delta_rule_scan_kernel(const float* qkv, const T* beta_raw, int beta_stride, const T* a_raw,
                                       const float* dt_bias, const float* a_log, float* state, float* o,
                                       const int* first_row, const int* slots, int heads, int kvheads, int dim, int vdim,
                                       int write_state, int n_slots) {
  extern __shared__ float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, part = tid % PARTS, vl = tid / PARTS, v = v0 + vl;
  const int lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const bool v_ok = v < vdim;
  const int slot = __ldcg(slots + seq);
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  const int kvh = head / (heads / kvheads);
  const int row_w = 2 * kvheads * dim + heads * vdim;
  float* sq = smem;               // [CH][dim]
  float* sk = sq + CH * dim;      // [CH][dim]
  float* sg = sk + CH * dim;      // [CH][dim]
  float* sv = sg + CH * dim;      // [CH][VB]
  float* sbeta = sv + CH * VB;    // [CH]
  const float A = expf(a_log[head]);
  const float q_scale = 1.f / sqrtf((float)dim);
  float s[NP];
  float* st = state + (((size_t)slot * heads + head) * vdim + (v_ok ? v : 0)) * dim;
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int n = j * PARTS + part;
    s[j] = (v_ok && n < dim) ? st[n] : 0.f;
  }
  for (int c0 = lo; c0 < hi; c0 += CH) {
    const int cn = min(CH, hi - c0);
    __syncthreads();
    for (int i = tid; i < cn * dim; i += blockDim.x) {
      const int t = i / dim, n = i - t * dim;
      const float* r = qkv + (size_t)(c0 + t) * row_w + (size_t)kvh * dim + n;
      sq[i] = r[0];
      sk[i] = r[(size_t)kvheads * dim];
      const float a = to_f32(a_raw[(size_t)(c0 + t) * heads * dim + (size_t)head * dim + n]) + dt_bias[(size_t)head * dim + n];
      sg[i] = expf(-A * softplus_f(a));
    }
    for (int i = tid; i < cn * VB; i += blockDim.x) {
      const int t = i / VB, e = i - t * VB;
      sv[i] = v0 + e < vdim ? qkv[(size_t)(c0 + t) * row_w + 2 * (size_t)kvheads * dim + (size_t)head * vdim + v0 + e] : 0.f;
    }
    if (tid < cn) sbeta[tid] = sigmoid_f(to_f32(beta_raw[(size_t)(c0 + tid) * beta_stride + head]));
    __syncthreads();
    for (int t = warp; t < cn; t += nwarps) {  // unit vectors: a warp per token
      float qq = 0.f, kk = 0.f;
      for (int n = lane; n < dim; n += 32) {
        qq = fmaf(sq[t * dim + n], sq[t * dim + n], qq);
        kk = fmaf(sk[t * dim + n], sk[t * dim + n], kk);
      }
      const float qi = q_scale / sqrtf(warp_sum(qq) + 1e-6f), ki = 1.f / sqrtf(warp_sum(kk) + 1e-6f);
      for (int n = lane; n < dim; n += 32) {
        sq[t * dim + n] *= qi;
        sk[t * dim + n] *= ki;
      }
    }
    __syncthreads();
    for (int t = 0; t < cn; ++t) {
      const float* q = sq + t * dim + part;
      const float* k = sk + t * dim + part;
      const float* g = sg + t * dim + part;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        if (j * PARTS + part < dim) {
          s[j] *= g[j * PARTS];
          acc = fmaf(s[j], k[j * PARTS], acc);
        }
      }
      const float u = sbeta[t] * (sv[t * VB + vl] - quad_sum(acc));
      float out = 0.f;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        if (j * PARTS + part < dim) {
          s[j] = fmaf(k[j * PARTS], u, s[j]);
          out = fmaf(s[j], q[j * PARTS], out);
        }
      }
      out = quad_sum(out);
      if (part == 0 && v_ok) o[(size_t)(c0 + t) * heads * vdim + (size_t)head * vdim + v] = out;
    }
  }
  if (write_state && v_ok) {
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      const int n = j * PARTS + part;
      if (n < dim) st[n] = s[j];
    }
  }
}

// ---- norm over groups of a row, with a gate ----------------------------------------------------------
// x [tokens, width] float32; groups of `gs` values; weight[c % weight_period]; gate: columns of rows of gate_stride
// values.  gate_mode 1: x * silu(gate) before the norm;  2: sigmoid(gate) after the norm and the weight;  0: none.
// One warp per (token, group).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(const float* x, const T* gate, int gate_stride, int gate_mode,
                                           const float* weight, int weight_period, float eps, float factor, T* out,
                                           int n_tokens, int width, int gs) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const size_t unit = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int per_row = width / gs;
  if (unit >= (size_t)n_tokens * per_row) return;
  const size_t t = unit / per_row;
  const int c0 = (int)(unit - t * per_row) * gs;
  const float* xr = x + t * width + c0;
  const T* gr = gate ? gate + t * gate_stride + c0 : nullptr;
  float ss = 0.f;
  for (int e = lane; e < gs; e += 32) {
    float v = xr[e];
    if (gate_mode == 1) {
      const float z = to_f32(gr[e]);
      v *= z * sigmoid_f(z);
    }
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float)gs + eps);
  for (int e = lane; e < gs; e += 32) {
    float v = xr[e];
    if (gate_mode == 1) {
      const float z = to_f32(gr[e]);
      v *= z * sigmoid_f(z);
    }
    v = v * inv * weight[(c0 + e) % weight_period];
    if (gate_mode == 2) v *= sigmoid_f(to_f32(gr[e]));
    out[t * width + c0 + e] = from_f32<T>(v * factor);
  }
}
}  // namespace

FMS_API int fms_scan_chunk_tokens() { return CH; }

FMS_API int fms_causal_conv(const void* x, int dtype, int stride, const float* w, const float* bias, float* tail,
                            const int* token_seq, const int* first_row, const int* slots, float* out, int n_tokens,
                            int n_seqs, int channels, int taps, int act, int write_state, int n_slots,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || taps > MAX_TAPS) return fms_fail("causal_conv: %d taps (1..%d)", taps, MAX_TAPS);
  const size_t total = (size_t)n_tokens * channels;
  FMS_DISPATCH_DTYPE(dtype, T, {
    fms_launch(causal_conv_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, (const T*)x, stride, w,
               bias, (const float*)tail, token_seq, first_row, slots, out, n_tokens, channels, taps, act, n_seqs, n_slots);
    if (write_state && taps > 1)
      fms_launch(conv_tail_kernel<T>, dim3((channels + 127) / 128, n_seqs), dim3(128), 0, stream, (const T*)x, stride, tail,
                 first_row, slots, channels, taps, n_seqs, n_slots);
  });
  return fms_launch_status("causal_conv");
}

FMS_API int fms_selective_scan(const float* xbc, const void* dt_raw, int dtype, int dt_stride, const float* dt_bias,
                               const float* a_log, const float* d_skip, float* state, float* y, const int* first_row,
                               const int* slots, int n_seqs, int heads, int vdim, int n_state, int groups,
                               int write_state, int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || n_state <= 0 || n_state > PARTS * 64 || vdim <= 0)
    return fms_fail("selective_scan: %d heads, %d groups, state %d (up to %d), vdim %d", heads, groups, n_state, PARTS * 64, vdim);
  const dim3 grid(n_seqs, heads, (vdim + VB - 1) / VB), block(VB * PARTS);
  const size_t smem = ((size_t)2 * CH * n_state + CH * VB + 2 * CH) * sizeof(float);
  const int np = (n_state + PARTS - 1) / PARTS;
#define FMS_SCAN(NP)                                                                                                    \
  do {                                                                                                                  \
    cudaFuncSetAttribute(selective_scan_kernel<T, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    fms_launch(selective_scan_kernel<T, NP>, grid, block, smem, stream, xbc, (const T*)dt_raw, dt_stride, dt_bias, a_log, \
               d_skip, state, y, first_row, slots, heads, vdim, n_state, groups, write_state, n_slots);                  \
  } while (0)
  FMS_DISPATCH_DTYPE(dtype, T, {
    if (np <= 8) FMS_SCAN(8);
    else if (np <= 16) FMS_SCAN(16);
    else if (np <= 32) FMS_SCAN(32);
    else FMS_SCAN(64);
  });
#undef FMS_SCAN
  return fms_launch_status("selective_scan");
}

FMS_API int fms_delta_rule_scan(const float* qkv, const void* beta_raw, int dtype, int beta_stride, const void* a_raw,
                                const float* dt_bias, const float* a_log, float* state, float* o, const int* first_row,
                                const int* slots, int n_seqs, int heads, int kvheads, int dim, int vdim, int write_state,
                                int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (heads <= 0 || kvheads <= 0 || heads % kvheads || dim <= 0 || dim > PARTS * 64 || vdim <= 0)
    return fms_fail("delta_rule_scan: %d heads over %d, dim %d (up to %d), vdim %d", heads, kvheads, dim, PARTS * 64, vdim);
  const dim3 grid(n_seqs, heads, (vdim + VB - 1) / VB), block(VB * PARTS);
  const size_t smem = ((size_t)3 * CH * dim + CH * VB + CH) * sizeof(float);
  const int np = (dim + PARTS - 1) / PARTS;
#define FMS_SCAN(NP)                                                                                                    \
  do {                                                                                                                  \
    cudaFuncSetAttribute(delta_rule_scan_kernel<T, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    fms_launch(delta_rule_scan_kernel<T, NP>, grid, block, smem, stream, qkv, (const T*)beta_raw, beta_stride,           \
               (const T*)a_raw, dt_bias, a_log, state, o, first_row, slots, heads, kvheads, dim, vdim, write_state,      \
               n_slots);                                                                                                 \
  } while (0)
  FMS_DISPATCH_DTYPE(dtype, T, {
    if (np <= 8) FMS_SCAN(8);
    else if (np <= 16) FMS_SCAN(16);
    else if (np <= 32) FMS_SCAN(32);
    else FMS_SCAN(64);
  });
#undef FMS_SCAN
  return fms_launch_status("delta_rule_scan");
}

FMS_API int fms_gated_group_rmsnorm(const float* x, const void* gate, int dtype, int gate_stride, int gate_mode,
                                    const float* weight, int weight_period, float eps, float factor, void* out,
                                    int n_tokens, int width, int group_size, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (group_size <= 0 || width % group_size || weight_period <= 0)
    return fms_fail("gated_group_rmsnorm: rows of %d in groups of %d", width, group_size);
  if (gate_mode != 0 && gate == nullptr) return fms_fail("gated_group_rmsnorm: a gate mode without a gate");
  const size_t units = (size_t)n_tokens * (width / group_size);
  FMS_DISPATCH_DTYPE(dtype, T, fms_launch(gated_group_rmsnorm_kernel<T>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream,
                                          x, (const T*)gate, gate_stride, gate_mode, weight, weight_period, eps, factor,
                                          (T*)out, n_tokens, width, group_size));
  return fms_launch_status("gated_group_rmsnorm");
}
