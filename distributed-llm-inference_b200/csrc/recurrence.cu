// Linear recurrences whose matrix state decays per head AND key channel: the token-shift recurrence with a bonus for the
// current token, and the delta rule with channel-wise decay.  Everything that enters the recurrence is float32: a
// preparation kernel per mixer leaves float32 rows, and one scan kernel walks every sequence's tokens in order.
//
// A token's row (floats): A [kq_heads][d] what the state is read with | K [kq_heads][d] keys | G [heads][d] decays |
// V [heads][dv] values | B [heads] betas; head h reads A and K of head h / (heads / kq_heads).
#include <math_constants.h>

#include "common.cuh"

using namespace dli;

namespace {

struct RowLayout {
  int a, k, g, v, b, stride;
};

__host__ __device__ inline RowLayout row_layout(int kq_heads, int heads, int d, int dv) {
  RowLayout L;
  L.a = 0;
  L.k = kq_heads * d;
  L.g = 2 * kq_heads * d;
  L.v = L.g + heads * d;
  L.b = L.v + heads * dv;
  L.stride = (L.b + heads + 3) & ~3;
  return L;
}

__device__ __forceinline__ float softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// Token-shift recurrence: r, k, v are slabs 0, 1, 2 of rkvg [4][n][heads d]; the decay is exp(-exp(wz + w0)).
template <typename T>
__global__ void shift_decay_prep_kernel(float* __restrict__ rows, const T* __restrict__ rkvg, const T* __restrict__ wz,
                                        const float* __restrict__ w0, int n, int heads, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const int I = heads * d;
  const RowLayout L = row_layout(heads, heads, d, d);
  float* row = rows + t * L.stride;
  const size_t slab = (size_t)n * I;
  for (int i = threadIdx.x; i < I; i += blockDim.x) {
    row[L.a + i] = to_float(rkvg[t * I + i]);
    row[L.k + i] = to_float(rkvg[slab + t * I + i]);
    row[L.v + i] = to_float(rkvg[2 * slab + t * I + i]);
    row[L.g + i] = expf(-expf(to_float(wz[t * I + i]) + w0[i]));
  }
}

// Delta rule with a decay per channel: qkv [n][2 kq d + heads dv] after convolution and activation; q and k become unit
// vectors per head (unit_eps inside the root), q also times d^-1/2; beta = sigmoid(u[t][b_col + h]);
// decay = exp(-exp(a_log[h]) softplus(a[t][h d + i] + dt_bias[h d + i])).  A warp per head.
template <typename T>
__global__ void channel_delta_prep_kernel(float* __restrict__ rows, const T* __restrict__ qkv, const T* __restrict__ u, long long u_stride,
                                          int b_col, const T* __restrict__ a, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                          int heads, int kq, int d, int dv, float unit_eps) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  const RowLayout L = row_layout(kq, heads, d, dv);
  float* row = rows + t * L.stride;
  const T* src = qkv + t * (size_t)(2 * kq * d + heads * dv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int head = warp; head < 2 * kq; head += warps) {  // q heads, then k heads
    const T* part = src + (size_t)head * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float x = to_float(part[i]);
      ss = fmaf(x, x, ss);
    }
    ss = warp_sum(ss);
    float f = 1.f / sqrtf(ss + unit_eps);
    if (head < kq) f *= 1.f / sqrtf((float)d);
    float* dst = row + (size_t)head * d;  // A then K lie back to back
    for (int i = lane; i < d; i += 32) dst[i] = to_float(part[i]) * f;
  }
  for (int i = threadIdx.x; i < heads * d; i += blockDim.x) {
    const int h = i / d;
    row[L.g + i] = expf(-expf(a_log[h]) * softplus(to_float(a[t * (size_t)(heads * d) + i]) + dt_bias[i]));
  }
  for (int i = threadIdx.x; i < heads * dv; i += blockDim.x) row[L.v + i] = to_float(src[2 * kq * d + i]);
  for (int i = threadIdx.x; i < heads; i += blockDim.x) row[L.b + i] = 1.f / (1.f + expf(-to_float(u[t * u_stride + b_col + i])));
}

constexpr int REC_R_MAX = 32;   // key rows of a state column that one thread keeps in registers: 32, 16 or 8 (the fewer, the more threads share a column)
constexpr int REC_THREADS = 128;  // at most; a CTA has as many threads as its columns need
constexpr int REC_TOKENS = 16;  // tokens staged in shared memory at a time, the next sixteen on their way meanwhile

// Staged vectors are laid out in slices of R floats, each followed by 4 floats of padding, so that the threads of a
// warp that hold different slices read different banks.
__host__ __device__ inline int slice_at(int i, int R) { return i + ((i / R) << 2); }
__host__ __device__ inline int staged_floats(int ks, int R) { return ks * (R + 4); }
__host__ __device__ inline int token_floats(int ks, int cols, int R) { return (3 * staged_floats(ks, R) + cols + 1 + 3) & ~3; }

__device__ __forceinline__ void copy_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One CTA: some value columns of one head of one sequence.  KS threads (consecutive lanes) share a column, each with
// R key rows of it in registers (rows beyond d are zeros).  MODE 0 (bonus): o = sum_i a_i (S_i + u_i k_i v);
// S_i <- g_i S_i + k_i v.  MODE 1 (delta): S_i <- g_i S_i; w = beta (v - sum_i k_i S_i); S_i <- S_i + k_i w; o = sum_i a_i S_i.
// state [slots][heads][dv][d] (a value column's key rows are contiguous).  Sums over the key rows are added in an
// order fixed by d alone, token after token, so a result does not depend on how a sequence was cut into steps.
// Tokens arrive by asynchronous copies, sixteen at a time, the next sixteen under way while these are walked.
template <int MODE, int REC_R>
__global__ void __launch_bounds__(REC_THREADS) decay_recurrence_kernel(float* __restrict__ o, const float* __restrict__ rows,
                                                                       float* __restrict__ state, const int* __restrict__ q_start,
                                                                       const int* __restrict__ state_slot, const float* __restrict__ bonus,
                                                                       int heads, int kq, int d, int dv, int ks, int cols_per_cta) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  const int seq = blockIdx.z, head = blockIdx.y;
  const int t0 = q_start[seq], t1 = q_start[seq + 1];
  if (t1 <= t0) return;
  const RowLayout L = row_layout(kq, heads, d, dv);
  const int kqh = head / (heads / kq);
  const int dpad = staged_floats(ks, REC_R);
  const int tok_floats = token_floats(ks, cols_per_cta, REC_R);  // per staged token: A | K | G | V of this CTA's columns | beta
  const int buf_floats = REC_TOKENS * tok_floats;
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int col_local = tid / ks, slice = tid - col_local * ks;
  const int col0 = blockIdx.x * cols_per_cta;
  const int col = col0 + col_local;
  const bool active = col_local < cols_per_cta && col < dv;
  const int i0 = slice * REC_R;
  const bool vec = (d & 3) == 0;  // rows of whole 16-byte chunks (the row's parts then start on 16-byte boundaries too)

  // the places behind the head size stay zero in both buffers: no copy writes them
  for (int e = tid; e < 2 * buf_floats; e += nthreads) sm[e] = 0.f;
  __syncthreads();

  // A thread copies the same places of every token of a tile: where they lie is worked out once per place, not once per token.
  auto stage = [&](int buf, int base) {
    const int cnt = min(REC_TOKENS, t1 - base);
    float* dst0 = sm + buf * buf_floats;
    const float* row0 = rows + (size_t)base * L.stride;
    if (vec) {
      const int chunks = d >> 2;
      for (int c = tid; c < 3 * chunks; c += nthreads) {
        const int which = c / chunks, i = (c - which * chunks) << 2;
        const float* src = row0 + (which == 0 ? L.a + kqh * d : (which == 1 ? L.k + kqh * d : L.g + head * d)) + i;
        float* dst = dst0 + which * dpad + slice_at(i, REC_R);
        for (int tok = 0; tok < cnt; ++tok) copy_async16(dst + tok * tok_floats, src + (size_t)tok * L.stride);
      }
    } else {
      for (int c = tid; c < 3 * d; c += nthreads) {
        const int which = c / d, i = c - which * d;
        const float* src = row0 + (which == 0 ? L.a + kqh * d : (which == 1 ? L.k + kqh * d : L.g + head * d)) + i;
        float* dst = dst0 + which * dpad + slice_at(i, REC_R);
        for (int tok = 0; tok < cnt; ++tok) copy_async4(dst + tok * tok_floats, src + (size_t)tok * L.stride);
      }
    }
    const int extra = cols_per_cta + (MODE == 1 ? 1 : 0);
    for (int c = tid; c < extra; c += nthreads) {
      const float* src;
      if (c == cols_per_cta) src = row0 + L.b + head;
      else if (col0 + c < dv) src = row0 + L.v + head * dv + col0 + c;
      else continue;
      float* dst = dst0 + 3 * dpad + c;
      for (int tok = 0; tok < cnt; ++tok) copy_async4(dst + tok * tok_floats, src + (size_t)tok * L.stride);
    }
  };

  stage(0, t0);
  copy_commit();

  float S[REC_R], U[REC_R];
  float* srow = state + (((size_t)state_slot[seq] * heads + head) * dv + (active ? col : 0)) * d;
  if (vec) {
#pragma unroll
    for (int r = 0; r < REC_R; r += 4) {
      const int i = i0 + r;
      float4 sv = make_float4(0.f, 0.f, 0.f, 0.f), uv = sv;
      if (i < d) {
        if (active) sv = *reinterpret_cast<const float4*>(srow + i);
        if (MODE == 0) uv = *reinterpret_cast<const float4*>(bonus + (size_t)head * d + i);
      }
      S[r] = sv.x; S[r + 1] = sv.y; S[r + 2] = sv.z; S[r + 3] = sv.w;
      U[r] = uv.x; U[r + 1] = uv.y; U[r + 2] = uv.z; U[r + 3] = uv.w;
    }
  } else {
#pragma unroll
    for (int r = 0; r < REC_R; ++r) {
      const int i = i0 + r;
      S[r] = (active && i < d) ? srow[i] : 0.f;
      U[r] = (MODE == 0 && i < d) ? bonus[(size_t)head * d + i] : 0.f;
    }
  }

  int buf = 0;
  for (int base = t0; base < t1; base += REC_TOKENS, buf ^= 1) {
    const int cnt = min(REC_TOKENS, t1 - base);
    if (base + REC_TOKENS < t1) stage(buf ^ 1, base + REC_TOKENS);  // (its readers finished before the barrier that ended the last round)
    copy_commit();
    copy_wait<1>();
    __syncthreads();
    const float* tile = sm + buf * buf_floats;
#pragma unroll 2
    for (int tok = 0; tok < cnt; ++tok) {
      const float4* A = reinterpret_cast<const float4*>(tile + tok * tok_floats + slice_at(i0, REC_R));
      const float4* K = reinterpret_cast<const float4*>(tile + tok * tok_floats + dpad + slice_at(i0, REC_R));
      const float4* G = reinterpret_cast<const float4*>(tile + tok * tok_floats + 2 * dpad + slice_at(i0, REC_R));
      const float v = tile[tok * tok_floats + 3 * dpad + (col_local < cols_per_cta ? col_local : 0)];
      float acc4[4] = {0.f, 0.f, 0.f, 0.f};  // four running sums: the chain of dependent multiply-adds is a quarter as long
      if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < REC_R; r += 4) {
          const float4 a = A[r >> 2], k = K[r >> 2], g = G[r >> 2];
          const float av[4] = {a.x, a.y, a.z, a.w}, kvv[4] = {k.x, k.y, k.z, k.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float kv = kvv[q] * v;
            acc4[q] = fmaf(av[q], fmaf(U[r + q], kv, S[r + q]), acc4[q]);
            S[r + q] = fmaf(gv[q], S[r + q], kv);
          }
        }
      } else {
        const float beta = tile[tok * tok_floats + 3 * dpad + cols_per_cta];
        float ks4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < REC_R; r += 4) {
          const float4 k = K[r >> 2], g = G[r >> 2];
          const float kvv[4] = {k.x, k.y, k.z, k.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            S[r + q] *= gv[q];
            ks4[q] = fmaf(kvv[q], S[r + q], ks4[q]);
          }
        }
        float ks_sum = (ks4[0] + ks4[1]) + (ks4[2] + ks4[3]);
        for (int off = 1; off < ks; off <<= 1) ks_sum += __shfl_xor_sync(0xffffffffu, ks_sum, off);
        const float w = beta * (v - ks_sum);
#pragma unroll
        for (int r = 0; r < REC_R; r += 4) {
          const float4 a = A[r >> 2], k = K[r >> 2];
          const float av[4] = {a.x, a.y, a.z, a.w}, kvv[4] = {k.x, k.y, k.z, k.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            S[r + q] = fmaf(kvv[q], w, S[r + q]);
            acc4[q] = fmaf(av[q], S[r + q], acc4[q]);
          }
        }
      }
      float acc = (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]);
      for (int off = 1; off < ks; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (active && slice == 0) o[(size_t)(base + tok) * heads * dv + (size_t)head * dv + col] = acc;
    }
    __syncthreads();  // this buffer is copied into again in the round after next
  }
  copy_wait<0>();
  if (active) {
    if (vec) {
#pragma unroll
      for (int r = 0; r < REC_R; r += 4) {
        const int i = i0 + r;
        if (i < d) *reinterpret_cast<float4*>(srow + i) = make_float4(S[r], S[r + 1], S[r + 2], S[r + 3]);
      }
    } else {
#pragma unroll
      for (int r = 0; r < REC_R; ++r) {
        const int i = i0 + r;
        if (i < d) srow[i] = S[r];
      }
    }
  }
}

}  // namespace

DLI_EXPORT int dli_decay_recurrence_row(int kq_heads, int heads, int d, int dv) { return row_layout(kq_heads, heads, d, dv).stride; }

DLI_EXPORT int dli_shift_decay_prep(float* rows, const void* rkvg, const void* wz, const float* w0, int n, int heads, int d, int dtype,
                                    cudaStream_t stream) {
  if (n == 0) return 0;
  if (heads < 1 || d < 1) return DLI_ERR_UNSUPPORTED;
  const int threads = heads * d >= 1024 ? 256 : 128;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((shift_decay_prep_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, rows, (const float*)rkvg, (const float*)wz, w0, n, heads, d);
  else
    e = launch_pdl((shift_decay_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, rows, (const __nv_bfloat16*)rkvg,
                   (const __nv_bfloat16*)wz, w0, n, heads, d);
  return (int)e;
}

DLI_EXPORT int dli_channel_delta_prep(float* rows, const void* qkv, const void* u, long long u_stride, int b_col, const void* a,
                                      const float* dt_bias, const float* a_log, int n, int heads, int kq, int d, int dv, float unit_eps, int dtype,
                                      cudaStream_t stream) {
  if (n == 0) return 0;
  if (heads < 1 || kq < 1 || heads % kq || d < 1 || dv < 1) return DLI_ERR_UNSUPPORTED;
  const int threads = heads * d >= 1024 ? 256 : 128;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((channel_delta_prep_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, rows, (const float*)qkv, (const float*)u, u_stride,
                   b_col, (const float*)a, dt_bias, a_log, heads, kq, d, dv, unit_eps);
  else
    e = launch_pdl((channel_delta_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, rows, (const __nv_bfloat16*)qkv,
                   (const __nv_bfloat16*)u, u_stride, b_col, (const __nv_bfloat16*)a, dt_bias, a_log, heads, kq, d, dv, unit_eps);
  return (int)e;
}

// mode 0: bonus (needs `bonus` [heads][d]); mode 1: delta.  d up to 512.  rows_per_lane: 32, 16 or 8 key rows a lane, or 0: chosen here.
DLI_EXPORT int dli_decay_recurrence(float* o, const float* rows, float* state, const int* q_start, const int* state_slot, const float* bonus,
                                    int num_seqs, int heads, int kq, int d, int dv, int mode, int rows_per_lane, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (heads < 1 || kq < 1 || heads % kq || d < 1 || dv < 1 || d > 512 || (mode == 0 && !bonus) || mode < 0 || mode > 1 || heads > 65535 ||
      num_seqs > 65535)
    return DLI_ERR_UNSUPPORTED;
  // Key rows a thread: 32 where there are warps enough (a decode step of many sequences); for the bonus recurrence 16 or 8 where
  // a few long sequences would leave the GPU idle, so that more threads share a column and a token's chain of multiply-adds
  // gets shorter (one prompt of 4,096 tokens, 16 heads of 64 x 64: 1,512 us at 32, 1,238 at 16, 1,152 at 8).
  int R = REC_R_MAX;
  auto lanes = [&](int r) { int k = 1; while (k * r < d) k <<= 1; return k; };
  if (rows_per_lane == 32 || rows_per_lane == 16 || rows_per_lane == 8) R = rows_per_lane;
  else if (rows_per_lane != 0) return DLI_ERR_UNSUPPORTED;
  else if (mode == 0)  // (the delta rule adds two rounds of shuffles a token for every halving: measured, it is fastest at 32 everywhere)
    while (R > 8 && lanes(R / 2) <= 32 && (long long)num_seqs * heads * dv * lanes(R) / 32 < 4LL * sm_count()) R >>= 1;
  const int ks = lanes(R);
  if (ks > 32) return DLI_ERR_UNSUPPORTED;
  // columns a CTA: all that 128 threads hold, fewer while the grid would leave SMs idle (never under a warp's worth of threads)
  int cols = REC_THREADS / ks;
  if (cols < 1) cols = 1;
  if (cols > dv) cols = dv;
  while (cols * ks > 32 && (long long)((dv + cols - 1) / cols) * heads * num_seqs < 2LL * sm_count()) cols = (cols + 1) / 2;
  const int threads = ((cols * ks + 31) / 32) * 32;
  const size_t smem = (size_t)2 * REC_TOKENS * token_floats(ks, cols, R) * sizeof(float);
  if (smem > 227 * 1024) return DLI_ERR_UNSUPPORTED;
  const dim3 grid((dv + cols - 1) / cols, heads, num_seqs);
  cudaError_t e = cudaSuccess;
#define DLI_REC(MODE, RR)                                                                                                              \
  {                                                                                                                                    \
    static MaxPerDevice set;                                                                                                           \
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {                                                                             \
      e = cudaFuncSetAttribute(decay_recurrence_kernel<MODE, RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
      if (e != cudaSuccess) return (int)e;                                                                                             \
      set.here() = (int)smem;                                                                                                          \
    }                                                                                                                                  \
    e = launch_pdl((decay_recurrence_kernel<MODE, RR>), grid, dim3(threads), smem, stream, 1, o, rows, state, q_start, state_slot, bonus, heads, \
                   kq, d, dv, ks, cols);                                                                                               \
  }
  if (mode == 0) {
    if (R == 32) DLI_REC(0, 32) else if (R == 16) DLI_REC(0, 16) else DLI_REC(0, 8)
  } else {
    if (R == 32) DLI_REC(1, 32) else if (R == 16) DLI_REC(1, 16) else DLI_REC(1, 8)
  }
#undef DLI_REC
  return (int)e;
}
