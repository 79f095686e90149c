// Kernels around a float32 residual stream whose sublayers are normed on their OUTPUT (x += m * norm(f(x))):
//
//   * token embedding times a factor, plus a row of a second table chosen by a hash of (previous token, token);
//     the previous token of a sequence's first row in this step comes from the request's state slot;
//   * RMS norm in equal consecutive groups of a sublayer's output, times a weight and a factor, added to the
//     stream, which is also written out in the activation dtype for the next sublayer's product;
//   * the same norm of rows of the stream itself (the model's last norm), with an optional row gather;
//   * act(gate) * table[token] for a per-layer token input;
//   * a weighted sum of the embedding output and the streams that the layers so far have left (depth average).
//
// All arithmetic is float32; a row's sums are added in an order fixed by the sizes.
#include "common.cuh"

using namespace dli;

namespace {

constexpr int THREADS = 256;
constexpr int MAX_GROUPS = 64;

__device__ __forceinline__ float gelu_tanh(float z) { return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))); }

// ---------------------------------------------------------------- embedding with a hashed pair table
template <typename T>
__global__ void pair_embedding_kernel(float* __restrict__ h, const T* __restrict__ table, float scale, const T* __restrict__ pair_table,
                                      int buckets, int mul_prev, int mul_cur, const int* __restrict__ ids, const int* __restrict__ positions,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ q_start, const int* __restrict__ state_slot,
                                      int* __restrict__ prev_state, T* __restrict__ y, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_row;
  const int r = blockIdx.x;
  const int id = ids[r];
  if (threadIdx.x == 0) {
    int row = -1;
    if (pair_table != nullptr) {
      const int s = seq_of_token[r];
      const int first = q_start[s];
      const int slot = state_slot[s];
      if (positions[r] == 0) {
        row = buckets;  // a sequence's first token has no pair: the table's last row
      } else {
        const int prev = r > first ? ids[r - 1] : prev_state[slot];
        row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % buckets);
      }
      // the block of the sequence's first row in this step (the only reader of the slot) leaves the step's last token there
      if (r == first) prev_state[slot] = ids[q_start[s + 1] - 1];
    }
    s_row = row;
  }
  __syncthreads();
  const int row = s_row;
  const T* e = table + (size_t)id * H;
  const T* b = row >= 0 ? pair_table + (size_t)row * H : nullptr;
  float* o = h + (size_t)r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = to_float(e[c]) * scale;
    if (b != nullptr) v += to_float(b[c]);
    o[c] = v;
    if (y != nullptr) y[(size_t)r * H + c] = from_float<T>(v);
  }
}

// ---------------------------------------------------------------- RMS norm in groups
// 1 / sqrt(mean(v^2) + eps) of each of `groups` equal consecutive parts of a row, left in rstd[] (shared).
template <typename Load>
__device__ __forceinline__ void group_rstd(Load load, int H, int groups, float eps, float* rstd, float* red) {
  const int gs = H / groups;
  for (int g = 0; g < groups; ++g) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < gs; c += blockDim.x) {
      const float v = load(g * gs + c);
      ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) rstd[g] = rsqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
}

// h += mult * norm(a) * w; y = h in the activation dtype (if y).  TA: dtype of a and y.
template <typename TA>
__global__ void group_norm_add_kernel(float* __restrict__ h, const TA* __restrict__ a, const float* __restrict__ w, int groups, float eps,
                                      float mult, TA* __restrict__ y, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  __shared__ float rstd[MAX_GROUPS];
  const size_t row = (size_t)blockIdx.x * H;
  const TA* ar = a + row;
  group_rstd([&](int c) { return to_float(ar[c]); }, H, groups, eps, rstd, red);
  const int gs = H / groups;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = h[row + c] + mult * (to_float(ar[c]) * rstd[c / gs] * w[c]);
    h[row + c] = v;
    if (y != nullptr) y[row + c] = from_float<TA>(v);
  }
}

// y[i] = norm(h[rows[i]]) * w  (rows == nullptr: row i)
template <typename TY>
__global__ void group_norm_rows_kernel(TY* __restrict__ y, const float* __restrict__ h, const float* __restrict__ w, const int* __restrict__ rows,
                                       int groups, float eps, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  __shared__ float rstd[MAX_GROUPS];
  const float* hr = h + (size_t)(rows != nullptr ? rows[blockIdx.x] : blockIdx.x) * H;
  group_rstd([&](int c) { return hr[c]; }, H, groups, eps, rstd, red);
  const int gs = H / groups;
  for (int c = threadIdx.x; c < H; c += blockDim.x) y[(size_t)blockIdx.x * H + c] = from_float<TY>(hr[c] * rstd[c / gs] * w[c]);
}

// ---------------------------------------------------------------- g[r, j] = gelu_tanh(g[r, j]) * table[ids[r], col0 + j]
template <typename T>
__global__ void gelu_mul_rows_kernel(T* __restrict__ g, const T* __restrict__ table, int table_cols, int col0, const int* __restrict__ ids,
                                     int n, int dim) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n * dim;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / dim;
    const int j = (int)(idx - r * dim);
    const float e = to_float(table[(size_t)ids[r] * table_cols + col0 + j]);
    g[idx] = from_float<T>(gelu_tanh(to_float(g[idx])) * e);
  }
}

// ---------------------------------------------------------------- out = w[0] * x0 + sum_{j >= 1} w[j] * hist[j - 1]; y = out in the activation dtype
template <typename TY>
__global__ void depth_average_kernel(float* __restrict__ out, const float* __restrict__ x0, const float* __restrict__ hist, long long stride,
                                     const float* __restrict__ w, int count, TY* __restrict__ y, long long total) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    float acc = w[0] * x0[idx];
    for (int j = 1; j < count; ++j) acc = fmaf(w[j], hist[(j - 1) * stride + idx], acc);
    out[idx] = acc;
    if (y != nullptr) y[idx] = from_float<TY>(acc);
  }
}

inline int grid_for(long long total) {
  const long long want = (total + THREADS - 1) / THREADS, most = (long long)sm_count() * 16;
  return (int)(want < most ? (want > 0 ? want : 1) : most);
}

}  // namespace

DLI_EXPORT int dli_pair_embedding(float* h, const void* table, float scale, const void* pair_table, int buckets, int mul_prev, int mul_cur,
                                  const int* ids, const int* positions, const int* seq_of_token, const int* q_start, const int* state_slot,
                                  int* prev_state, void* y, int n, int H, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (pair_table != nullptr && (buckets < 1 || prev_state == nullptr)) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    launch_pdl((pair_embedding_kernel<float>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const float*)table, scale, (const float*)pair_table,
               buckets, mul_prev, mul_cur, ids, positions, seq_of_token, q_start, state_slot, prev_state, (float*)y, H);
  else
    launch_pdl((pair_embedding_kernel<__nv_bfloat16>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const __nv_bfloat16*)table, scale,
               (const __nv_bfloat16*)pair_table, buckets, mul_prev, mul_cur, ids, positions, seq_of_token, q_start, state_slot, prev_state,
               (__nv_bfloat16*)y, H);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_group_norm_add(float* h, const void* a, const float* w, int groups, float eps, float mult, void* y, int n, int H, int dtype,
                                  cudaStream_t stream) {
  if (n == 0) return 0;
  if (groups < 1 || groups > MAX_GROUPS || H % groups) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    launch_pdl((group_norm_add_kernel<float>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const float*)a, w, groups, eps, mult, (float*)y, H);
  else
    launch_pdl((group_norm_add_kernel<__nv_bfloat16>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const __nv_bfloat16*)a, w, groups, eps, mult,
               (__nv_bfloat16*)y, H);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_group_norm_rows(void* y, const float* h, const float* w, const int* rows, int groups, float eps, int n, int H, int dtype,
                                   cudaStream_t stream) {
  if (n == 0) return 0;
  if (groups < 1 || groups > MAX_GROUPS || H % groups) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    launch_pdl((group_norm_rows_kernel<float>), dim3(n), dim3(THREADS), 0, stream, 1, (float*)y, h, w, rows, groups, eps, H);
  else
    launch_pdl((group_norm_rows_kernel<__nv_bfloat16>), dim3(n), dim3(THREADS), 0, stream, 1, (__nv_bfloat16*)y, h, w, rows, groups, eps, H);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_gelu_mul_rows(void* g, const void* table, int table_cols, int col0, const int* ids, int n, int dim, int dtype,
                                 cudaStream_t stream) {
  if (n == 0 || dim == 0) return 0;
  if (col0 < 0 || col0 + dim > table_cols) return DLI_ERR_UNSUPPORTED;
  const int grid = grid_for((long long)n * dim);
  if (dtype == DLI_F32)
    launch_pdl((gelu_mul_rows_kernel<float>), dim3(grid), dim3(THREADS), 0, stream, 1, (float*)g, (const float*)table, table_cols, col0, ids, n, dim);
  else
    launch_pdl((gelu_mul_rows_kernel<__nv_bfloat16>), dim3(grid), dim3(THREADS), 0, stream, 1, (__nv_bfloat16*)g, (const __nv_bfloat16*)table,
               table_cols, col0, ids, n, dim);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_depth_average(float* out, const float* x0, const float* hist, long long stride, const float* w, int count, void* y, long long total, int dtype,
                                 cudaStream_t stream) {
  if (total == 0) return 0;
  if (count < 1) return DLI_ERR_UNSUPPORTED;
  const int grid = grid_for(total);
  if (dtype == DLI_F32)
    launch_pdl((depth_average_kernel<float>), dim3(grid), dim3(THREADS), 0, stream, 1, out, x0, hist, stride, w, count, (float*)y, total);
  else
    launch_pdl((depth_average_kernel<__nv_bfloat16>), dim3(grid), dim3(THREADS), 0, stream, 1, out, x0, hist, stride, w, count, (__nv_bfloat16*)y, total);
  return (int)cudaGetLastError();
}
