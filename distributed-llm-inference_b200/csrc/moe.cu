// A routed mixture of gated feed-forwards: the router (float32 throughout), and the experts' products for steps of few
// tokens, one (token, chosen expert) pair at a time on the CUDA cores.  (Steps of many tokens in bfloat16 take the
// grouped tensor-core products of moe_grouped.cu.)
#include <math_constants.h>

#include "common.cuh"

using namespace dli;

namespace {

constexpr int ROUTE_THREADS = 512;  // at most: sixteen warps, an expert's row each, for a step of few tokens (a handful of blocks); four warps a token for many
constexpr int MAX_TOP = 32;

// sum_i w[i] * xs[i] over a warp (xs: the token's row as floats in shared memory); 16-byte loads when `vec`
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ xs, int len, int lane, bool vec) {
  float acc = 0.f;
  if (vec) {
    for (int i = lane * 8; i < len; i += 256) {
      float v[8];
      load8(w + i, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc = fmaf(v[k], xs[i + k], acc);
    }
  } else {
    for (int i = lane; i < len; i += 32) acc = fmaf(to_float(w[i]), xs[i], acc);
  }
  return warp_sum(acc);
}

// One block per token.  z = W_r x (float32 sums of float32 products); s = sigmoid(z); choice = s + correction.
// Groups: `groups` equal runs of neighbouring experts; a group's mark is the sum of its two largest choice scores (its
// one score if it has one expert); only the `keep` groups with the largest marks stay eligible.  The `top` eligible experts
// with the largest choice scores are chosen (ties: the lower index), in that order; weights = s[chosen] / (sum + 1e-20) * scale.
template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS) moe_route_kernel(int* __restrict__ ids, float* __restrict__ weights, const T* __restrict__ x,
                                                                  const float* __restrict__ router, const float* __restrict__ correction,
                                                                  int W, int E, int top, int groups, int keep, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];  // x [W] | score [E] | choice [E] | mark [groups]
  float* xs = sm;
  float* score = xs + W;
  float* choice = score + E;
  float* mark = choice + E;
  __shared__ int picked[MAX_TOP];
  const size_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < W; i += blockDim.x) xs[i] = to_float(x[t * W + i]);
  __syncthreads();
  const bool vec = (W % 8) == 0 && (((uintptr_t)router) & 15) == 0;
  for (int e = warp; e < E; e += blockDim.x >> 5) {
    const float z = warp_dot<float>(router + (size_t)e * W, xs, W, lane, vec);
    if (lane == 0) {
      const float s = 1.f / (1.f + expf(-z));
      score[e] = s;
      choice[e] = s + correction[e];
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (groups > 1) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -CUDART_INF_F, b = -CUDART_INF_F;  // the two largest
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; }
        else if (c > b) b = c;
      }
      mark[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // the `keep` best groups: the others' experts cannot be chosen
    for (int round = 0; round < groups - keep; ++round) {  // drop the worst remaining group (ties: the higher index goes first)
      float worst = CUDART_INF_F;
      int at = -1;
      for (int g = lane; g < groups; g += 32) {
        const float m = mark[g];
        if (m != CUDART_INF_F && (m < worst || (m == worst && g > at))) { worst = m; at = g; }
      }
      for (int off = 16; off > 0; off >>= 1) {
        const float ow = __shfl_xor_sync(0xffffffffu, worst, off);
        const int oa = __shfl_xor_sync(0xffffffffu, at, off);
        if (oa >= 0 && (at < 0 || ow < worst || (ow == worst && oa > at))) { worst = ow; at = oa; }
      }
      if (lane == 0) mark[at] = CUDART_INF_F;  // +inf marks a dropped group
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (mark[e / per] == CUDART_INF_F) choice[e] = -CUDART_INF_F;
    __syncwarp();
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -CUDART_INF_F;
    int at = -1;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (at < 0 || c > best) {
        if (c > best || at < 0) { best = c; at = e; }
      }
    }
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oa = __shfl_xor_sync(0xffffffffu, at, off);
      if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    if (lane == 0) {
      picked[k] = at;
      choice[at] = -CUDART_INF_F;
    }
    total += score[at];
    __syncwarp();
  }
  const float f = scale / (total + 1e-20f);
  for (int k = lane; k < top; k += 32) {
    ids[t * top + k] = picked[k];
    weights[t * top + k] = score[picked[k]] * f;
  }
}

constexpr int PAIR_THREADS = 128;
constexpr int PAIR_ROWS = 16;  // rows of the intermediate size a block computes

__device__ __forceinline__ float glu_act(float g, int act) {
  if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  if (act == 2) return g / (1.f + expf(-1.702f * g));
  return g / (1.f + expf(-g));
}

// hidden[pair][j] = act(gate_e[j] . x) * (up_e[j] . x), e = ids[pair], x the pair's token; w [E][2 ff][W]: gate rows, then up rows.
// The two sums are rounded to the activation dtype before the activation, as a product that stored them would have.
template <typename T>
__global__ void __launch_bounds__(PAIR_THREADS) moe_pair_gate_up_kernel(T* __restrict__ hidden, const T* __restrict__ x, const int* __restrict__ ids,
                                                                        const T* __restrict__ w, int W, int ff, int top, int act) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float xs[];
  const size_t pair = blockIdx.y;
  const size_t t = pair / top;
  const int e = ids[pair];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < W; i += PAIR_THREADS) xs[i] = to_float(x[t * W + i]);
  __syncthreads();
  const T* we = w + (size_t)e * 2 * ff * W;
  const bool vec = (W % 8) == 0 && (((uintptr_t)w) & 15) == 0;
  const int j0 = blockIdx.x * PAIR_ROWS;
  for (int j = j0 + warp; j < min(j0 + PAIR_ROWS, ff); j += PAIR_THREADS / 32) {
    const float g = warp_dot<T>(we + (size_t)j * W, xs, W, lane, vec);
    const float u = warp_dot<T>(we + (size_t)(ff + j) * W, xs, W, lane, vec);
    if (lane == 0) hidden[pair * ff + j] = from_float<T>(glu_act(to_float(from_float<T>(g)), act) * to_float(from_float<T>(u)));
  }
}

// out[t][c] = sum_k weights[t][k] * (down_e(k)[c] . hidden[t top + k]), added in the order of the choice, float32, one rounding.
// w [E][W][ff].
template <typename T>
__global__ void __launch_bounds__(PAIR_THREADS) moe_pair_down_kernel(T* __restrict__ out, const T* __restrict__ hidden, const int* __restrict__ ids,
                                                                     const float* __restrict__ weights, const T* __restrict__ w, int W, int ff,
                                                                     int top) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float hs[];  // the token's `top` hidden rows
  const size_t t = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < top * ff; i += PAIR_THREADS) hs[i] = to_float(hidden[t * top * ff + i]);
  __syncthreads();
  const bool vec = (ff % 8) == 0 && (((uintptr_t)w) & 15) == 0;
  const int c0 = blockIdx.x * PAIR_ROWS;
  for (int c = c0 + warp; c < min(c0 + PAIR_ROWS, W); c += PAIR_THREADS / 32) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int e = ids[t * top + k];
      const float d = warp_dot<T>(w + ((size_t)e * W + c) * ff, hs + (size_t)k * ff, ff, lane, vec);
      acc = fmaf(weights[t * top + k], d, acc);
    }
    if (lane == 0) out[t * W + c] = from_float<T>(acc);
  }
}

template <typename K>
inline cudaError_t allow_smem(K kernel, size_t smem, MaxPerDevice& set) {
  if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    set.here() = (int)smem;
  }
  return cudaSuccess;
}

}  // namespace

DLI_EXPORT int dli_moe_route(int* ids, float* weights, const void* x, const float* router, const float* correction, int n, int W, int E, int top,
                             int groups, int keep, float scale, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (W < 1 || E < 1 || top < 1 || top > MAX_TOP || groups < 1 || E % groups || keep < 1 || keep > groups || top > keep * (E / groups))
    return DLI_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)W + 2 * E + groups) * sizeof(float);
  if (smem > 200 * 1024) return DLI_ERR_UNSUPPORTED;
  const int threads = n <= 256 ? ROUTE_THREADS : 128;
  cudaError_t e;
  if (dtype == DLI_F32) {
    static MaxPerDevice set;
    if ((e = allow_smem(moe_route_kernel<float>, smem, set)) != cudaSuccess) return (int)e;
    e = launch_pdl((moe_route_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, ids, weights, (const float*)x, router, correction, W, E,
                   top, groups, keep, scale);
  } else {
    static MaxPerDevice set;
    if ((e = allow_smem(moe_route_kernel<__nv_bfloat16>, smem, set)) != cudaSuccess) return (int)e;
    e = launch_pdl((moe_route_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, ids, weights, (const __nv_bfloat16*)x, router,
                   correction, W, E, top, groups, keep, scale);
  }
  return (int)e;
}

// hidden: scratch [n top][ff] in the activation dtype.
DLI_EXPORT int dli_moe_pairs(void* out, void* hidden, const void* x, const int* ids, const float* weights, const void* w_gate_up, const void* w_down,
                             int n, int W, int ff, int top, int act, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const size_t smem_up = (size_t)W * sizeof(float), smem_down = (size_t)top * ff * sizeof(float);
  if (W < 1 || ff < 1 || top < 1 || (long long)n * top > 65535 || smem_up > 200 * 1024 || smem_down > 200 * 1024) return DLI_ERR_UNSUPPORTED;
  const dim3 grid_up((ff + PAIR_ROWS - 1) / PAIR_ROWS, n * top), grid_down((W + PAIR_ROWS - 1) / PAIR_ROWS, n);
  cudaError_t e;
  if (dtype == DLI_F32) {
    static MaxPerDevice set_up, set_down;
    if ((e = allow_smem(moe_pair_gate_up_kernel<float>, smem_up, set_up)) != cudaSuccess) return (int)e;
    if ((e = allow_smem(moe_pair_down_kernel<float>, smem_down, set_down)) != cudaSuccess) return (int)e;
    e = launch_pdl((moe_pair_gate_up_kernel<float>), grid_up, dim3(PAIR_THREADS), smem_up, stream, 1, (float*)hidden, (const float*)x, ids,
                   (const float*)w_gate_up, W, ff, top, act);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_pair_down_kernel<float>), grid_down, dim3(PAIR_THREADS), smem_down, stream, 1, (float*)out, (const float*)hidden, ids, weights,
                   (const float*)w_down, W, ff, top);
  } else {
    static MaxPerDevice set_up, set_down;
    if ((e = allow_smem(moe_pair_gate_up_kernel<__nv_bfloat16>, smem_up, set_up)) != cudaSuccess) return (int)e;
    if ((e = allow_smem(moe_pair_down_kernel<__nv_bfloat16>, smem_down, set_down)) != cudaSuccess) return (int)e;
    e = launch_pdl((moe_pair_gate_up_kernel<__nv_bfloat16>), grid_up, dim3(PAIR_THREADS), smem_up, stream, 1, (__nv_bfloat16*)hidden,
                   (const __nv_bfloat16*)x, ids, (const __nv_bfloat16*)w_gate_up, W, ff, top, act);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_pair_down_kernel<__nv_bfloat16>), grid_down, dim3(PAIR_THREADS), smem_down, stream, 1, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)hidden, ids, weights, (const __nv_bfloat16*)w_down, W, ff, top);
  }
  return (int)e;
}
