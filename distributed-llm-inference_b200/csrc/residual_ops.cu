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
// Four consecutive numbers of a row at once (the callers take this path when the row and a group are multiples of four
// long, so a vector starts on its own size's boundary and lies in one group).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// 1 / sqrt(mean(v^2) + eps) of each of `groups` equal consecutive parts of a row, left in rstd[] (shared).  The warps
// divide the groups between them, several warps to a group where there are fewer groups than warps; which numbers a lane
// adds, and in which order the lanes' and warps' sums meet, is fixed by the sizes alone.
template <typename T>
__device__ __forceinline__ void group_rstd(const T* row, int H, int groups, float eps, bool vec, float* rstd, float* partial /* >= groups * warps */) {
  const int gs = H / groups;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int per = warps / groups > 1 ? warps / groups : 1;  // warps to a group
  int len = (gs + per - 1) / per;  // numbers of a group that one warp adds
  if (vec) len = (len + 3) & ~3;
  for (int ch = warp; ch < groups * per; ch += warps) {
    const int g = ch / per, part = ch - g * per;
    const int first = part * len, last = min(gs, first + len);
    const T* src = row + (size_t)g * gs;
    float ss = 0.f;
    if (vec) {
      for (int c = first + lane * 4; c < last; c += 128) {
        const float4 v = load4(src + c);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      }
    } else {
      for (int c = first + lane; c < last; c += 32) {
        const float v = to_float(src[c]);
        ss = fmaf(v, v, ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) partial[ch] = ss;
  }
  __syncthreads();
  for (int g = threadIdx.x; g < groups; g += blockDim.x) {
    float ss = 0.f;
    for (int i = 0; i < per; ++i) ss += partial[g * per + i];
    rstd[g] = rsqrtf(ss / (float)gs + eps);
  }
  __syncthreads();
}

// h += mult * norm(a) * w; y = h in the activation dtype (if y).  TA: dtype of a and y.
template <typename TA>
__global__ void group_norm_add_kernel(float* __restrict__ h, const TA* __restrict__ a, const float* __restrict__ w, int groups, float eps,
                                      float mult, TA* __restrict__ y, int H, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float partial[MAX_GROUPS * (THREADS / 32)];
  __shared__ float rstd[MAX_GROUPS];
  const size_t row = (size_t)blockIdx.x * H;
  const TA* ar = a + row;
  group_rstd(ar, H, groups, eps, vec != 0, rstd, partial);
  const int gs = H / groups;
  if (vec) {
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4) {
      const float4 av = load4(ar + c), wv = load4(w + c);
      float4 hv = load4(h + row + c);
      const float f = mult * rstd[c / gs];
      hv.x += f * (av.x * wv.x);
      hv.y += f * (av.y * wv.y);
      hv.z += f * (av.z * wv.z);
      hv.w += f * (av.w * wv.w);
      store4(h + row + c, hv);
      if (y != nullptr) store4(y + row + c, hv);
    }
    return;
  }
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = h[row + c] + mult * rstd[c / gs] * (to_float(ar[c]) * w[c]);
    h[row + c] = v;
    if (y != nullptr) y[row + c] = from_float<TA>(v);
  }
}

// y[i] = norm(h[rows[i]]) * w  (rows == nullptr: row i)
template <typename TY>
__global__ void group_norm_rows_kernel(TY* __restrict__ y, const float* __restrict__ h, const float* __restrict__ w, const int* __restrict__ rows,
                                       int groups, float eps, int H, int vec) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float partial[MAX_GROUPS * (THREADS / 32)];
  __shared__ float rstd[MAX_GROUPS];
  const float* hr = h + (size_t)(rows != nullptr ? rows[blockIdx.x] : blockIdx.x) * H;
  group_rstd(hr, H, groups, eps, vec != 0, rstd, partial);
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

// Rows and groups that are multiples of four numbers long, on pointers that let four numbers be read at once.
inline int vector_rows(int H, int groups, const void* h, const void* w, const void* a, const void* y) {
  const uintptr_t all = (uintptr_t)h | (uintptr_t)w | (uintptr_t)a | (uintptr_t)y;
  return H % 4 == 0 && (H / groups) % 4 == 0 && all % 16 == 0;
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
  const int vec = vector_rows(H, groups, h, w, a, y);
  if (dtype == DLI_F32)
    launch_pdl((group_norm_add_kernel<float>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const float*)a, w, groups, eps, mult, (float*)y, H, vec);
  else
    launch_pdl((group_norm_add_kernel<__nv_bfloat16>), dim3(n), dim3(THREADS), 0, stream, 1, h, (const __nv_bfloat16*)a, w, groups, eps, mult,
               (__nv_bfloat16*)y, H, vec);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_group_norm_rows(void* y, const float* h, const float* w, const int* rows, int groups, float eps, int n, int H, int dtype,
                                   cudaStream_t stream) {
  if (n == 0) return 0;
  if (groups < 1 || groups > MAX_GROUPS || H % groups) return DLI_ERR_UNSUPPORTED;
  const int vec = vector_rows(H, groups, h, w, nullptr, nullptr);
  if (dtype == DLI_F32)
    launch_pdl((group_norm_rows_kernel<float>), dim3(n), dim3(THREADS), 0, stream, 1, (float*)y, h, w, rows, groups, eps, H, vec);
  else
    launch_pdl((group_norm_rows_kernel<__nv_bfloat16>), dim3(n), dim3(THREADS), 0, stream, 1, (__nv_bfloat16*)y, h, w, rows, groups, eps, H, vec);
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
