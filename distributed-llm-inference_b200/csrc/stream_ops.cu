// Kernels around a residual stream whose sublayer outputs carry a learned scale per feature, the re-entry of a looped
// span through a product over [stream | embedding], and the blends of a token with the one before it (token shift).
#include <math_constants.h>

#include "common.cuh"

using namespace dli;

namespace {

// v = h[s] + ls * (fa * a[s] + fb * b[s])   (b may be null; a may be null: nothing is added), s = rows ? rows[r] : r
// without rows the sum is written back to h;  y[r] = v / sqrt(mean(v^2) + eps) * w   (y may be null: the addition alone)
// One block per row; float32 arithmetic, one rounding.  The second pass reads the sums back (from h, or recomputes them
// when h is left alone), so nothing depends on the row's length.
template <typename T>
__global__ void add_rmsnorm_scaled_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ a, float fa, const T* __restrict__ b,
                                          float fb, const float* __restrict__ ls, const float* __restrict__ w, float eps,
                                          const int* __restrict__ rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float* hrow = h + s * H;
  const T* arow = a ? a + s * H : nullptr;
  const T* brow = b ? b + s * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hrow[i];
    if (arow) {
      float d = fa * to_float(arow[i]);
      if (brow) d = fmaf(fb, to_float(brow[i]), d);
      v = fmaf(ls[i], d, v);
    }
    if (!rows && arow) hrow[i] = v;
    ss = fmaf(v, v, ss);
  }
  if (!y) return;
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
  T* yrow = y + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = hrow[i];  // written by this thread above, if it was written
    if (rows && arow) {
      float d = fa * to_float(arow[i]);
      if (brow) d = fmaf(fb, to_float(brow[i]), d);
      v = fmaf(ls[i], d, v);
    }
    yrow[i] = from_float<T>(v * inv * w[i]);
  }
}

// The same, eight features a thread at a time with 16- and 32-byte accesses (H % 8 == 0, aligned rows).
template <typename T>
__global__ void add_rmsnorm_scaled_vec_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ a, float fa, const T* __restrict__ b,
                                              float fb, const float* __restrict__ ls, const float* __restrict__ w, float eps,
                                              const int* __restrict__ rows, int H) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float* hrow = h + s * H;
  const T* arow = a ? a + s * H : nullptr;
  const T* brow = b ? b + s * H : nullptr;
  auto value = [&](int i, float (&v)[8]) {
    load8(hrow + i, v);
    if (arow) {
      float av[8], sv[8];
      load8(arow + i, av);
      load8(ls + i, sv);
      if (brow) {
        float bv[8];
        load8(brow + i, bv);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = fmaf(sv[k], fmaf(fb, bv[k], fa * av[k]), v[k]);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = fmaf(sv[k], fa * av[k], v[k]);
      }
    }
  };
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8];
    value(i, v);
    if (!rows && arow) store8(hrow + i, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
  }
  if (!y) return;
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)H + eps);
  T* yrow = y + (size_t)r * H;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float v[8], wv[8];
    if (rows && arow) value(i, v);
    else load8(hrow + i, v);  // written by this thread above, if it was written
    load8(w + i, wv);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = v[k] * inv * wv[k];
    store8(yrow + i, v);
  }
}

// out[t] = [ T(h[t]) | table[ids[t]] ]: the stream and the embedding of the step's tokens side by side.
template <typename T>
__global__ void concat_stream_rows_kernel(T* __restrict__ out, const float* __restrict__ h, const T* __restrict__ table,
                                          const int* __restrict__ ids, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const T* row = table + (size_t)ids[t] * W;
  T* dst = out + t * 2 * W;
  const float* src = h + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    dst[i] = from_float<T>(src[i]);
    dst[W + i] = row[i];
  }
}

// out[j][t] = x[t] + (before(t) - x[t]) * mu[j], j < blends; before(t) is the row of the token in front of t in its
// sequence: x[t - 1] inside the step, the sequence's carried row state[slot] at the step's first token (zeros when the
// sequence begins).  float32 arithmetic, one rounding.
template <typename T>
__global__ void token_shift_blend_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ mu, const T* __restrict__ state,
                                         const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                         const int* __restrict__ state_slot, int n, int W, int blends) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const T* cur = x + (size_t)t * W;
  const T* prev = t > q_start[seq] ? cur - W : state + (size_t)state_slot[seq] * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float c = to_float(cur[i]);
    const float d = to_float(prev[i]) - c;
    for (int j = 0; j < blends; ++j) out[((size_t)j * n + t) * W + i] = from_float<T>(fmaf(d, mu[(size_t)j * W + i], c));
  }
}

// The same, eight features a thread at a time (W % 8 == 0, aligned rows).
template <typename T>
__global__ void token_shift_blend_vec_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ mu, const T* __restrict__ state,
                                             const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                             const int* __restrict__ state_slot, int n, int W, int blends) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = seq_of_token[t];
  const T* cur = x + (size_t)t * W;
  const T* prev = t > q_start[seq] ? cur - W : state + (size_t)state_slot[seq] * W;
  for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {
    float c[8], d[8];
    load8(cur + i, c);
    load8(prev + i, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) d[k] -= c[k];
    for (int j = 0; j < blends; ++j) {
      float m[8], o[8];
      load8(mu + (size_t)j * W + i, m);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = fmaf(d[k], m[k], c[k]);
      store8(out + ((size_t)j * n + t) * W + i, o);
    }
  }
}

inline int row_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

}  // namespace

DLI_EXPORT int dli_add_rmsnorm_scaled(void* y, float* h, const void* a, float fa, const void* b, float fb, const float* ls, const float* w,
                                      float eps, const int* rows, int n_rows, int H, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (H < 1 || (a && !ls) || (y && !w) || (b && !a)) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if ((H % 8) == 0 && ((((uintptr_t)y) | ((uintptr_t)h) | ((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)ls) | ((uintptr_t)w)) & 15) == 0) {
    const int threads = H >= 4096 ? 256 : (H >= 1024 ? 128 : 64);
    if (dtype == DLI_F32)
      e = launch_pdl((add_rmsnorm_scaled_vec_kernel<float>), dim3(n_rows), dim3(threads), 0, stream, 1, (float*)y, h, (const float*)a, fa, (const float*)b, fb,
                     ls, w, eps, rows, H);
    else
      e = launch_pdl((add_rmsnorm_scaled_vec_kernel<__nv_bfloat16>), dim3(n_rows), dim3(threads), 0, stream, 1, (__nv_bfloat16*)y, h,
                     (const __nv_bfloat16*)a, fa, (const __nv_bfloat16*)b, fb, ls, w, eps, rows, H);
    return (int)e;
  }
  if (dtype == DLI_F32)
    e = launch_pdl((add_rmsnorm_scaled_kernel<float>), dim3(n_rows), dim3(row_threads(H)), 0, stream, 1, (float*)y, h, (const float*)a, fa,
                   (const float*)b, fb, ls, w, eps, rows, H);
  else
    e = launch_pdl((add_rmsnorm_scaled_kernel<__nv_bfloat16>), dim3(n_rows), dim3(row_threads(H)), 0, stream, 1, (__nv_bfloat16*)y, h,
                   (const __nv_bfloat16*)a, fa, (const __nv_bfloat16*)b, fb, ls, w, eps, rows, H);
  return (int)e;
}

DLI_EXPORT int dli_concat_stream_rows(void* out, const float* h, const void* table, const int* ids, int n, int W, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (W < 1) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((concat_stream_rows_kernel<float>), dim3(n), dim3(row_threads(W)), 0, stream, 1, (float*)out, h, (const float*)table, ids, W);
  else
    e = launch_pdl((concat_stream_rows_kernel<__nv_bfloat16>), dim3(n), dim3(row_threads(W)), 0, stream, 1, (__nv_bfloat16*)out, h,
                   (const __nv_bfloat16*)table, ids, W);
  return (int)e;
}

DLI_EXPORT int dli_token_shift_blend(void* out, const void* x, const float* mu, const void* state, const int* seq_of_token, const int* q_start,
                                     const int* state_slot, int n, int W, int blends, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (W < 1 || blends < 1) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if ((W % 8) == 0 && ((((uintptr_t)out) | ((uintptr_t)x) | ((uintptr_t)mu) | ((uintptr_t)state)) & 15) == 0) {
    const int threads = W >= 4096 ? 256 : (W >= 1024 ? 128 : 64);
    if (dtype == DLI_F32)
      e = launch_pdl((token_shift_blend_vec_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, (float*)out, (const float*)x, mu, (const float*)state,
                     seq_of_token, q_start, state_slot, n, W, blends);
    else
      e = launch_pdl((token_shift_blend_vec_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)x, mu,
                     (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, n, W, blends);
    return (int)e;
  }
  if (dtype == DLI_F32)
    e = launch_pdl((token_shift_blend_kernel<float>), dim3(n), dim3(row_threads(W)), 0, stream, 1, (float*)out, (const float*)x, mu,
                   (const float*)state, seq_of_token, q_start, state_slot, n, W, blends);
  else
    e = launch_pdl((token_shift_blend_kernel<__nv_bfloat16>), dim3(n), dim3(row_threads(W)), 0, stream, 1, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)x, mu, (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, n, W, blends);
  return (int)e;
}
