// minGRU: a gated recurrence whose gates read only the current token.
//
//   z_t = sigmoid(pz_t + bz);  u_t = px_t + bx;  c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) elsewhere
//   S_t = (1 - z_t) S_(t-1) + z_t c_t              (element by element; S float32, carried in the request's state slot)
//   out_t = S_t * silu(pg_t)
//
// p = pz | px | pg are the columns of one projection [n, 3 W] (activation dtype).  Gates, candidate and state are
// float32.  Any mix of prompt portions and single tokens: a sequence's rows are q_start[s] .. q_start[s + 1] - 1.
//
// A recurrence S_t = a_t S_(t-1) + b_t is walked in two levels for long portions: the rows of a sequence are cut into
// chunks; every chunk is walked from zero (its own b's) while the product of its a's is kept; a second, short walk
// over the chunks' ends hands each chunk the state at its start; the third pass adds a_(start..t) * S_start.  Short
// portions and single tokens take the plain walk.
#include "common.cuh"

using namespace dli;

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T>
__device__ __forceinline__ void gates(const T* __restrict__ p, int W, int c, float bz, float bx, float& a, float& b) {
  const float z = sigmoidf_(to_float(p[c]) + bz);
  const float u = to_float(p[W + c]) + bx;
  const float cand = u >= 0.f ? u + 0.5f : sigmoidf_(u);
  a = 1.f - z;
  b = z * cand;
}

// plain walk: one thread per (sequence, channel)
template <typename T>
__global__ void mingru_walk_kernel(T* __restrict__ out, const T* __restrict__ p, const float* __restrict__ bz, const float* __restrict__ bx,
                                   float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ state_slot, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = q_start[s], r1 = q_start[s + 1];
  if (c >= W || r0 >= r1) return;
  float* st = state + (size_t)state_slot[s] * W + c;
  float S = *st;
  const float zb = bz[c], xb = bx[c];
#pragma unroll 4
  for (int r = r0; r < r1; ++r) {
    const T* pr = p + (size_t)r * 3 * W;
    float a, b;
    gates(pr, W, c, zb, xb, a, b);
    S = fmaf(a, S, b);
    const float g = to_float(pr[2 * W + c]);
    out[(size_t)r * W + c] = from_float<T>(S * (g * sigmoidf_(g)));
  }
  *st = S;
}

// level one: every chunk from zero; local[r] = state contribution of the chunk's own rows, carry_a / carry_b per chunk
template <typename T>
__global__ void mingru_chunk_kernel(float* __restrict__ local, float* __restrict__ carry_a, float* __restrict__ carry_b, float* __restrict__ decay,
                                    float* __restrict__ state_in, const float* __restrict__ state, const int* __restrict__ state_slot,
                                    const T* __restrict__ p, const float* __restrict__ bz, const float* __restrict__ bx,
                                    const int* __restrict__ q_start, int W, int chunk, int chunks_per_seq) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.z, k = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = q_start[s] + k * chunk;
  const int r1 = min(q_start[s + 1], r0 + chunk);
  if (c >= W || r0 >= r1) return;
  // the state the sequence brings is set aside here: the next kernel's chunks read the copy, its last chunk writes the slot
  if (k == 0) state_in[(size_t)s * W + c] = state[(size_t)state_slot[s] * W + c];
  const float zb = bz[c], xb = bx[c];
  float S = 0.f, A = 1.f;
#pragma unroll 4
  for (int r = r0; r < r1; ++r) {
    float a, b;
    gates(p + (size_t)r * 3 * W, W, c, zb, xb, a, b);
    S = fmaf(a, S, b);
    A *= a;
    local[(size_t)r * W + c] = S;
    decay[(size_t)r * W + c] = A;  // product of the a's from the chunk's first row through r
  }
  const size_t at = ((size_t)s * chunks_per_seq + k) * W + c;
  carry_a[at] = A;
  carry_b[at] = S;
}

// level two and three: the state at each chunk's start, then out = (local + decay * S_start) * silu(g)
template <typename T>
__global__ void mingru_finish_kernel(T* __restrict__ out, const float* __restrict__ local, const float* __restrict__ carry_a,
                                     const float* __restrict__ carry_b, const float* __restrict__ decay, const float* __restrict__ state_in,
                                     const T* __restrict__ p, float* __restrict__ state, const int* __restrict__ q_start,
                                     const int* __restrict__ state_slot, int W, int chunk, int chunks_per_seq) {
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.z, k = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int first = q_start[s], last = q_start[s + 1];
  const int r0 = first + k * chunk;
  const int r1 = min(last, r0 + chunk);
  if (c >= W || r0 >= r1) return;
  float S0 = state_in[(size_t)s * W + c];
  for (int j = 0; j < k; ++j) {  // the chunks in front of this one, in order
    const size_t at = ((size_t)s * chunks_per_seq + j) * W + c;
    S0 = fmaf(carry_a[at], S0, carry_b[at]);
  }
  float S = S0;
#pragma unroll 4
  for (int r = r0; r < r1; ++r) {
    const size_t i = (size_t)r * W + c;
    S = fmaf(decay[i], S0, local[i]);
    const float g = to_float(p[(size_t)r * 3 * W + 2 * W + c]);
    out[i] = from_float<T>(S * (g * sigmoidf_(g)));
  }
  if (r1 == last) state[(size_t)state_slot[s] * W + c] = S;  // the chunk that holds the sequence's last row leaves the state
}

}  // namespace

// scratch (needed only when max_len > chunk): (2 n + (2 chunks_per_seq + 1) seqs) * W floats, chunks_per_seq = ceil(max_len / chunk)
DLI_EXPORT int dli_mingru_scan(void* out, const void* p, const float* bz, const float* bx, float* state, const int* q_start,
                               const int* state_slot, int n, int seqs, int W, int max_len, int chunk, float* scratch, int dtype,
                               cudaStream_t stream) {
  if (n == 0 || seqs == 0) return 0;
  if (W < 1) return DLI_ERR_UNSUPPORTED;
  const int threads = W >= 128 ? 128 : 32 * ((W + 31) / 32);
  const int bx_ = (W + threads - 1) / threads;
  if (scratch == nullptr || chunk < 1 || max_len <= chunk) {
    dim3 grid(bx_, seqs);
    if (dtype == DLI_F32)
      launch_pdl((mingru_walk_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)out, (const float*)p, bz, bx, state, q_start, state_slot, W);
    else
      launch_pdl((mingru_walk_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)p, bz, bx,
                 state, q_start, state_slot, W);
    return (int)cudaGetLastError();
  }
  const int cps = (max_len + chunk - 1) / chunk;
  float* local = scratch;
  float* decay = local + (size_t)n * W;
  float* carry_a = decay + (size_t)n * W;
  float* carry_b = carry_a + (size_t)seqs * cps * W;
  float* state_in = carry_b + (size_t)seqs * cps * W;
  dim3 grid(bx_, cps, seqs);
  if (dtype == DLI_F32) {
    launch_pdl((mingru_chunk_kernel<float>), grid, dim3(threads), 0, stream, 1, local, carry_a, carry_b, decay, state_in, (const float*)state,
               state_slot, (const float*)p, bz, bx, q_start, W, chunk, cps);
    launch_pdl((mingru_finish_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)out, (const float*)local, (const float*)carry_a,
               (const float*)carry_b, (const float*)decay, (const float*)state_in, (const float*)p, state, q_start, state_slot, W, chunk, cps);
  } else {
    launch_pdl((mingru_chunk_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, local, carry_a, carry_b, decay, state_in,
               (const float*)state, state_slot, (const __nv_bfloat16*)p, bz, bx, q_start, W, chunk, cps);
    launch_pdl((mingru_finish_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, (const float*)local,
               (const float*)carry_a, (const float*)carry_b, (const float*)decay, (const float*)state_in, (const __nv_bfloat16*)p, state, q_start,
               state_slot, W, chunk, cps);
  }
  return (int)cudaGetLastError();
}
