// Gated element-wise recurrences over a step's tokens, with the state of every sequence kept in float32 between steps.
//
// minGRU: the gates read the current token only, so all of a step's gate values are known before the scan starts:
//   proj[t] = [ zl | u | g ]  (three runs of `width` values, what the fused projection with its biases gave)
//   z = sigmoid(zl)            candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z) S_(t-1) + z candidate          y[t] = S_t * silu(g)
// Everything after the projection is float32; y is stored in the compute dtype.  S starts at what state[slot]
// holds (zero for a new sequence) and is written back after the step's last token.
//
// Two ways through a step.  Few tokens a sequence (decode, short continuations): one thread per (sequence, channel)
// walks the tokens in order.  Many tokens: the tokens are cut into chunks of CHUNK (32); S_t = a_t S_(t-1) + b_t is a
// composition of affine maps, so (1) every (chunk, channel) composes its own maps into one (A, B) from a zero
// start, (2) one thread per (sequence, channel) walks the chunks in order and leaves every chunk's start state,
// (3) every (chunk, channel) walks its tokens again from that start state and writes y.  The chunk boundaries
// depend on the row's place in its step, so a prompt cut into steps differs from the whole prompt by rounding only.
#include "common.cuh"


// Kernels of a step may start while the kernel before them is still running (programmatic dependent launch) and
// read what that kernel wrote right after griddepcontrol.wait.  No pointer here is declared __restrict__: the
// compiler must not turn such a read into a non-coherent load or move it ahead of the wait, and the few words of
// bookkeeping that the kernel before wrote (positions, offsets, groups) are read with ld_fresh (from L2).
#define __restrict__
__device__ __forceinline__ int ld_fresh(const int* p) { return __ldcg(p); }
__device__ __forceinline__ float ld_fresh(const float* p) { return __ldcg(p); }

namespace {
constexpr int CHUNK = 32;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float mingru_candidate(float u) { return u >= 0.f ? u + 0.5f : sigmoid_f(u); }

template <typename T>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, float* __restrict__ state, T* __restrict__ y,
                                   const int* __restrict__ first_row, const int* __restrict__ slots, int width,
                                   int n_slots, int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= width) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, n_slots)) return;
  const int lo = first_row[seq], hi = first_row[seq + 1];
  float s = state[(size_t)slot * width + c];
  const size_t stride = 3 * (size_t)width;
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const T* p = proj + (size_t)t * stride + c;
    const float z = sigmoid_f(to_f32(p[0]));
    const float u = to_f32(p[width]);
    const float g = to_f32(p[2 * (size_t)width]);
    s = (1.f - z) * s + z * mingru_candidate(u);
    y[(size_t)t * width + c] = from_f32<T>(s * (g * sigmoid_f(g)));
  }
  if (write_state) state[(size_t)slot * width + c] = s;
}

// (1) chunk i of the step's chunk list: rows chunk_rows[2i] .. chunk_rows[2i + 1] - 1 of one sequence
template <typename T>
__global__ void mingru_chunk_compose_kernel(const T* __restrict__ proj, const int* __restrict__ chunk_rows,
                                            float* __restrict__ ab, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int chunk = blockIdx.y;
  if (c >= width) return;
  const int lo = chunk_rows[2 * chunk], hi = chunk_rows[2 * chunk + 1];
  float a = 1.f, b = 0.f;
  const size_t stride = 3 * (size_t)width;
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const T* p = proj + (size_t)t * stride + c;
    const float z = sigmoid_f(to_f32(p[0]));
    const float u = to_f32(p[width]);
    a = (1.f - z) * a;
    b = (1.f - z) * b + z * mingru_candidate(u);
  }
  ab[(size_t)chunk * 2 * width + c] = a;
  ab[(size_t)chunk * 2 * width + width + c] = b;
}

// (2) per sequence: walks its chunks (first_chunk[seq] .. first_chunk[seq + 1] - 1), turns each chunk's A into the
// state the chunk starts from, and leaves the sequence's state after the step
__global__ void mingru_chunk_carry_kernel(float* __restrict__ ab, const int* __restrict__ first_chunk,
                                          float* __restrict__ state, const int* __restrict__ slots, int width, int n_slots,
                                          int write_state) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int seq = blockIdx.y;
  if (c >= width) return;
  const int slot = slots[seq];
  if (!FMS_IN(slot, n_slots)) return;
  float s = state[(size_t)slot * width + c];
  for (int k = first_chunk[seq]; k < first_chunk[seq + 1]; ++k) {
    float* e = ab + (size_t)k * 2 * width;
    const float a = e[c], b = e[width + c];
    e[c] = s;  // where the chunk starts
    s = a * s + b;
  }
  if (write_state) state[(size_t)slot * width + c] = s;
}

// (3) the chunk's tokens again, from its start state
template <typename T>
__global__ void mingru_chunk_apply_kernel(const T* __restrict__ proj, const int* __restrict__ chunk_rows,
                                          const float* __restrict__ ab, T* __restrict__ y, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int chunk = blockIdx.y;
  if (c >= width) return;
  const int lo = chunk_rows[2 * chunk], hi = chunk_rows[2 * chunk + 1];
  float s = ab[(size_t)chunk * 2 * width + c];
  const size_t stride = 3 * (size_t)width;
#pragma unroll 4
  for (int t = lo; t < hi; ++t) {
    const T* p = proj + (size_t)t * stride + c;
    const float z = sigmoid_f(to_f32(p[0]));
    const float u = to_f32(p[width]);
    const float g = to_f32(p[2 * (size_t)width]);
    s = (1.f - z) * s + z * mingru_candidate(u);
    y[(size_t)t * width + c] = from_f32<T>(s * (g * sigmoid_f(g)));
  }
}
}  // namespace

FMS_API int fms_recurrent_chunk_tokens() { return CHUNK; }

// proj [n_tokens, 3 width], y [n_tokens, width] in `dtype`; state [n_slots, width] float32; first_row [n_seqs + 1];
// slots [n_seqs].  With chunk_rows (int [n_chunks, 2]), first_chunk (int [n_seqs + 1]) and ab (float [n_chunks, 2,
// width]) the step runs chunk by chunk, else token by token.
FMS_API int fms_mingru_scan(const void* proj, int dtype, float* state, void* y, const int* first_row, const int* slots,
                            int n_seqs, int width, int n_slots, int write_state, const int* chunk_rows,
                            const int* first_chunk, int n_chunks, float* ab, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (width <= 0) return fms_fail("mingru_scan: width %d", width);
  if (n_seqs > 65535 || n_chunks > 65535) return fms_fail("mingru_scan: %d sequences, %d chunks in one launch", n_seqs, n_chunks);
  const int threads = 128;
  const int bx = (width + threads - 1) / threads;
  if (chunk_rows == nullptr || n_chunks <= 0) {
    FMS_DISPATCH_DTYPE(dtype, T,
                       fms_launch(mingru_scan_kernel<T>, dim3(bx, n_seqs), dim3(threads), 0, stream, (const T*)proj, state,
                                  (T*)y, first_row, slots, width, n_slots, write_state));
    return fms_launch_status("mingru_scan");
  }
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(mingru_chunk_compose_kernel<T>, dim3(bx, n_chunks), dim3(threads), 0, stream,
                                (const T*)proj, chunk_rows, ab, width));
  if (fms_launch_status("mingru_scan (compose)")) return 1;
  fms_launch(mingru_chunk_carry_kernel, dim3(bx, n_seqs), dim3(threads), 0, stream, ab, first_chunk, state, slots, width,
             n_slots, write_state);
  if (fms_launch_status("mingru_scan (carry)")) return 1;
  FMS_DISPATCH_DTYPE(dtype, T,
                     fms_launch(mingru_chunk_apply_kernel<T>, dim3(bx, n_chunks), dim3(threads), 0, stream, (const T*)proj,
                                chunk_rows, (const float*)ab, (T*)y, width));
  return fms_launch_status("mingru_scan (apply)");
}
