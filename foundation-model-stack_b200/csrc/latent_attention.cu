// Attention over a cache of latent rows: every cached position holds ONE row [c | kr] for all heads — c (`rank`
// values) is the normed down-projection from which a head's keys and values would be made by two matrices, kr (`rot`
// values) the rotated key part that all heads share.  The head's up-projections are folded into the query and taken
// out of the result, so nothing but the latent rows is ever read:
//   score_h(i, j) = (ql_h(i) . c(j) + qr_h(i) . kr(j)) * scale        ql_h = W_uk,h^T q_h (made before this kernel)
//   p = softmax over j <= i, with one more term exp(sink_h) in the denominator that has no key and no value
//   ol_h(i) = sum_j p(i, j) c(j), times sigmoid(gate_h(i))             the head's value is W_uv,h ol_h (made after)
// Scores, softmax and sums are float32.  The cache is the block cache of the other attention kernels with one
// key head of rank + rot values and no value plane.
//
// latent_prepare: from the fused projection [q heads (dim + rot each) | c (rank) | kr (rot) | gates (heads)] of a
// step's rows it norms c (RMS, a gain per value), rotates kr and every head's rot part by the row's position
// (adjacent pairs (2i, 2i+1), the first rot_dims values, angle = position * inv_freq[i], float32), writes [c | kr]
// into the cache at the row's slot and place and the rotated query parts into q_full[:, h, rank:].
#include "common.cuh"


// Kernels of a step may start while the kernel before them is still running (programmatic dependent launch) and
// read what that kernel wrote right after griddepcontrol.wait.  No pointer here is declared __restrict__: the
// compiler must not turn such a read into a non-coherent load or move it ahead of the wait, and the few words of
// bookkeeping that the kernel before wrote (positions, offsets, groups) are read with ld_fresh (from L2).
#define __restrict__
__device__ __forceinline__ int ld_fresh(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcg(p); }

namespace {
constexpr int SPLIT = 256;  // keys of one split of a decode step: fixed, so a sequence's sums depend on its length only
constexpr int KT = 32;      // keys brought into shared memory at a time
constexpr int HG = 8;       // heads a block takes
constexpr int THREADS = 256;

template <typename T, typename TG>
__global__ void __launch_bounds__(128) latent_prepare_kernel(
    const T* __restrict__ proj, int proj_width, T* __restrict__ q_full, const TG* __restrict__ c_gain, float eps,
    const float* __restrict__ inv_freq, int rot_dims, const int* __restrict__ positions,
    const int* __restrict__ position_ids, const int* __restrict__ token_seq, const int* __restrict__ slots,
    T* __restrict__ cache, const int* __restrict__ table, int table_stride, int block_tokens, int heads, int dim, int rot,
    int rank, int write_cache, int n_seqs, int n_slots, int n_blocks, int* __restrict__ error_flag) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * proj_width;
  const int q_cols = heads * (dim + rot);
  const float position = (float)(position_ids ? ld_fresh(position_ids + t) : ld_fresh(positions + t));
  const int width = rank + rot;
  // the rotated part of every head's query
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < heads * rot; i += blockDim.x) {
    const int h = i / rot, j = i - h * rot;
    const T* src = row + (size_t)h * (dim + rot) + dim;
    float v;
    if (j < 2 * half) {
      const int pair = j >> 1;
      float sn, cs;
      sincosf(position * inv_freq[pair], &sn, &cs);
      const float a = to_f32(src[2 * pair]), b = to_f32(src[2 * pair + 1]);
      v = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
    } else {
      v = to_f32(src[j]);
    }
    q_full[((size_t)t * heads + h) * width + rank + j] = from_f32<T>(v);
  }
  if (!write_cache) return;
  const int seq = token_seq[t];
  if (!FMS_IN(seq, n_seqs)) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, n_slots)) return;
  const int pos = ld_fresh(positions + t);
  const int blk = table[(size_t)slot * table_stride + pos / block_tokens];
  if (blk < 0 || blk >= n_blocks) {
    if (threadIdx.x == 0 && error_flag) atomicExch(error_flag, 2);
    return;
  }
  T* dst = cache + ((size_t)blk * block_tokens + pos % block_tokens) * width;
  const T* c = row + q_cols;
  float ss = 0.f;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    const float v = to_f32(c[d]);
    ss += v * v;
  }
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
  for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = from_f32<T>(to_f32(c[d]) * inv * to_f32(c_gain[d]));
  const T* kr = c + rank;
  for (int j = threadIdx.x; j < rot; j += blockDim.x) {
    float v;
    if (j < 2 * half) {
      const int pair = j >> 1;
      float sn, cs;
      sincosf(position * inv_freq[pair], &sn, &cs);
      const float a = to_f32(kr[2 * pair]), b = to_f32(kr[2 * pair + 1]);
      v = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
    } else {
      v = to_f32(kr[j]);
    }
    dst[rank + j] = from_f32<T>(v);
  }
}

struct LatentArgs {
  const void* q;      // [tokens, heads, rank + rot]
  void* out;          // [tokens, heads, rank]
  const void* cache;  // [blocks, block_tokens, rank + rot]
  const void* gate;   // first gate logit of row 0: gate[t * gate_stride + h]; null: no gate
  const void* sink;   // [heads] or null
  const int* table;
  const int* slots;
  const int* token_seq;
  const int* positions;
  float* part_o;   // [tokens, heads, splits, rank]
  float* part_ml;  // [tokens, heads, splits, 2]
  long gate_stride;
  int table_stride, block_tokens, heads, rank, rot, n_splits, n_seqs, n_slots, n_blocks;
  float scale;
};

// One block per (row, split of keys, group of HG heads).  Keys come KT at a time into shared memory as float32; a warp
// takes the scores of one head (a lane a key), then 32 threads a head take the sums over the keys for rank / 32
// values each (NACC of them in registers).
template <typename T, typename TS, int NACC>
__global__ void __launch_bounds__(THREADS) latent_attention_kernel(LatentArgs a) {
  extern __shared__ float sm[];
  const int width = a.rank + a.rot;
  const int kstride = width | 1;  // odd: lanes that read the same value of different keys meet different banks
  float* qs = sm;                      // [HG][width]
  float* ks = qs + HG * width;         // [KT][kstride]
  float* ps = ks + KT * kstride;       // [HG][KT]
  float* alpha = ps + HG * KT;         // [HG]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * HG;
  const int nh = min(HG, a.heads - h0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = ld_fresh(a.positions + t);
  const int seq = a.token_seq[t];
  if (!FMS_IN(seq, a.n_seqs)) return;
  const int slot = a.slots[seq];
  if (!FMS_IN(slot, a.n_slots)) return;
  const bool whole = a.n_splits == 1;  // one split takes all keys and writes the result itself
  const int lo = whole ? 0 : split * SPLIT;
  const int hi = whole ? pos + 1 : min(pos + 1, lo + SPLIT);
  const T* q = (const T*)a.q + ((size_t)t * a.heads + h0) * width;
  for (int i = threadIdx.x; i < nh * width; i += THREADS) qs[i] = to_f32(q[i]);
  float acc[NACC];
#pragma unroll
  for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;  // of head `warp`, kept alike by all lanes of the warp
  const T* cache = (const T*)a.cache;
  for (int k0 = lo; k0 < hi; k0 += KT) {
    __syncthreads();  // the last tile's sums are taken (and, the first time, q is in place)
    const int nk = min(KT, hi - k0);
    for (int i = threadIdx.x; i < nk * width; i += THREADS) {
      const int j = i / width, d = i - j * width;
      const int p = k0 + j;
      const int blk = a.table[(size_t)slot * a.table_stride + p / a.block_tokens];
      float v = 0.f;
      if (blk >= 0 && blk < a.n_blocks) v = to_f32(cache[((size_t)blk * a.block_tokens + p % a.block_tokens) * width + d]);
      ks[j * kstride + d] = v;
    }
    __syncthreads();
    if (warp < nh) {
      float s = -INFINITY;
      if (lane < nk) {
        const float* qh = qs + warp * width;
        const float* kj = ks + lane * kstride;
        float dot = 0.f;
        for (int d = 0; d < width; ++d) dot = fmaf(qh[d], kj[d], dot);
        s = dot * a.scale;
      }
      const float m_new = fmaxf(m_run, warp_max(s));
      const float p = lane < nk ? expf(s - m_new) : 0.f;
      const float al = expf(m_run - m_new);  // 0 the first time
      l_run = l_run * al + warp_sum(p);
      m_run = m_new;
      ps[warp * KT + lane] = p;
      if (lane == 0) alpha[warp] = al;
    }
    __syncthreads();
    {
      const int h = threadIdx.x >> 5;  // 32 threads a head
      if (h < nh) {
        const float al = alpha[h];
        const float* ph = ps + h * KT;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
          const int d = lane + 32 * i;
          if (d < a.rank) {
            float v = acc[i] * al;
            for (int j = 0; j < nk; ++j) v = fmaf(ph[j], ks[j * kstride + d], v);
            acc[i] = v;
          }
        }
      }
    }
  }
  if (warp >= nh) return;
  const int h = h0 + warp;
  if (whole) {
    float m = m_run, denom = l_run;
    if (a.sink) {
      const float sk = to_f32(((const TS*)a.sink)[h]);
      m = fmaxf(m_run, sk);
      denom = l_run * expf(m_run - m) + expf(sk - m);
    }
    float f = expf(m_run - m) / denom;
    if (a.gate) f *= 1.f / (1.f + expf(-to_f32(((const T*)a.gate)[(size_t)t * a.gate_stride + h])));
    T* o = (T*)a.out + ((size_t)t * a.heads + h) * a.rank;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < a.rank) o[d] = from_f32<T>(acc[i] * f);
    }
  } else {
    const size_t at = ((size_t)t * a.heads + h) * a.n_splits + split;
    if (lane == 0) {
      a.part_ml[2 * at] = m_run;
      a.part_ml[2 * at + 1] = l_run;
    }
    float* o = a.part_o + at * a.rank;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < a.rank) o[d] = acc[i];
    }
  }
}

// Merges a row's splits: a block per (row, head).
template <typename T, typename TS>
__global__ void __launch_bounds__(128) latent_combine_kernel(LatentArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y;
  const int pos = ld_fresh(a.positions + t);
  const int used = min(a.n_splits, pos / SPLIT + 1);
  const size_t at = ((size_t)t * a.heads + h) * a.n_splits;
  float m = a.sink ? to_f32(((const TS*)a.sink)[h]) : -INFINITY;
  for (int s = 0; s < used; ++s) m = fmaxf(m, a.part_ml[2 * (at + s)]);
  float denom = a.sink ? expf(to_f32(((const TS*)a.sink)[h]) - m) : 0.f;
  for (int s = 0; s < used; ++s) denom += a.part_ml[2 * (at + s) + 1] * expf(a.part_ml[2 * (at + s)] - m);
  float f = 1.f / denom;
  if (a.gate) f *= 1.f / (1.f + expf(-to_f32(((const T*)a.gate)[(size_t)t * a.gate_stride + h])));
  T* o = (T*)a.out + ((size_t)t * a.heads + h) * a.rank;
  for (int d = threadIdx.x; d < a.rank; d += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < used; ++s) v = fmaf(a.part_o[(at + s) * a.rank + d], expf(a.part_ml[2 * (at + s)] - m), v);
    o[d] = from_f32<T>(v * f);
  }
}

template <typename T, typename TS>
int launch_attention(const LatentArgs& a, int n_tokens, cudaStream_t stream) {
  const int width = a.rank + a.rot;
  const size_t smem = ((size_t)HG * width + (size_t)KT * (width | 1) + HG * KT + HG) * sizeof(float);
  if (smem > 220 * 1024) return fms_fail("latent_attention: rows of %d values do not fit shared memory", width);
  dim3 grid(n_tokens, a.n_splits, (a.heads + HG - 1) / HG);
  if (grid.y > 65535 || grid.z > 65535) return fms_fail("latent_attention: %d splits, %d heads", a.n_splits, a.heads);
#define FMS_LATENT_LAUNCH(NACC)                                                                                         \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(latent_attention_kernel<T, TS, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    fms_launch(latent_attention_kernel<T, TS, NACC>, grid, dim3(THREADS), smem, stream, a);                             \
  } while (0)
  if (a.rank <= 128) FMS_LATENT_LAUNCH(4);
  else if (a.rank <= 256) FMS_LATENT_LAUNCH(8);
  else if (a.rank <= 512) FMS_LATENT_LAUNCH(16);
  else return fms_fail("latent_attention: a latent of %d values is more than the kernel keeps (512)", a.rank);
#undef FMS_LATENT_LAUNCH
  if (fms_launch_status("latent_attention")) return 1;
  if (a.n_splits > 1) {
    fms_launch(latent_combine_kernel<T, TS>, dim3(n_tokens, a.heads), dim3(128), 0, stream, a);
    return fms_launch_status("latent_attention (combine)");
  }
  return 0;
}
}  // namespace

FMS_API int fms_latent_split_tokens() { return SPLIT; }

FMS_API int fms_latent_prepare(const void* proj, int dtype, int proj_width, void* q_full, const void* c_gain, int gain_dtype,
                               float eps, const float* inv_freq, int rot_dims, const int* positions,
                               const int* position_ids, const int* token_seq, const int* slots, void* cache,
                               const int* table, int table_stride, int block_tokens, int n_tokens, int heads, int dim,
                               int rot, int rank, int write_cache, int n_seqs, int n_slots, int n_blocks, int* error_flag,
                               cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || dim < 0 || rot < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1))
    return fms_fail("latent_prepare: heads %d, dim %d, rot %d (%d rotated), rank %d", heads, dim, rot, rot_dims, rank);
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(gain_dtype, TG,
                     fms_launch(latent_prepare_kernel<T, TG>, dim3(n_tokens), dim3(128), 0, stream, (const T*)proj,
                                proj_width, (T*)q_full, (const TG*)c_gain, eps, inv_freq, rot_dims, positions,
                                position_ids, token_seq, slots, (T*)cache, table, table_stride, block_tokens, heads, dim,
                                rot, rank, write_cache, n_seqs, n_slots, n_blocks, error_flag)));
  return fms_launch_status("latent_prepare");
}

// n_splits == 1: every row takes all its keys in one block (a prompt's rows); else splits of fms_latent_split_tokens()
// keys and a merge, with part_o [tokens, heads, splits, rank] and part_ml [tokens, heads, splits, 2] as scratch.
FMS_API int fms_latent_attention(const void* q, void* out, int dtype, const void* cache, const void* gate, long gate_stride,
                                 const void* sink, int sink_dtype, const int* table, int table_stride, int block_tokens,
                                 const int* slots, const int* token_seq, const int* positions, int n_tokens, int n_splits,
                                 float* part_o, float* part_ml, int heads, int rank, int rot, float scale, int n_seqs,
                                 int n_slots, int n_blocks, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (n_splits < 1 || (n_splits > 1 && (part_o == nullptr || part_ml == nullptr)))
    return fms_fail("latent_attention: %d splits without scratch", n_splits);
  LatentArgs a;
  a.q = q; a.out = out; a.cache = cache; a.gate = gate; a.sink = sink; a.table = table; a.slots = slots;
  a.token_seq = token_seq; a.positions = positions; a.part_o = part_o; a.part_ml = part_ml; a.gate_stride = gate_stride;
  a.table_stride = table_stride; a.block_tokens = block_tokens; a.heads = heads; a.rank = rank; a.rot = rot;
  a.n_splits = n_splits; a.n_seqs = n_seqs; a.n_slots = n_slots; a.n_blocks = n_blocks; a.scale = scale;
  FMS_DISPATCH_DTYPE(dtype, T, FMS_DISPATCH_DTYPE(sink ? sink_dtype : dtype, TS, return launch_attention<T, TS>(a, n_tokens, stream)));
  return 0;
}
