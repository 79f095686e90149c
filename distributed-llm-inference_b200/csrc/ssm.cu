// A state-space mixer's steps between its two projections: the short causal convolution with its carried
// inputs, the selective scan with its carried state, and the gated norm in groups.  A step's tokens are any
// mix of prompt portions and single decoded tokens; each sequence continues from its own state slot.
// Everything that enters the recurrence is float32: step sizes, decays, the state and the sums.
#include "common.cuh"

using namespace dli;

namespace {

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
// for outputs that are rounded to bfloat16 anyway: the fast exponential and division (a few ulp of float32)
template <typename T> __device__ __forceinline__ float silu_out(float x) { return silu(x); }
template <> __device__ __forceinline__ float silu_out<__nv_bfloat16>(float x) { return __fdividef(x, 1.f + __expf(-x)); }
// what follows the convolution: SiLU (act != 0) or nothing
template <typename T> __device__ __forceinline__ float conv_out(int act, float x) { return act ? silu_out<T>(x) : x; }
// the gate of the group norm: SiLU, or (mode 2) the logistic function
__device__ __forceinline__ float norm_gate(float z, int mode) { return mode == 2 ? 1.f / (1.f + expf(-z)) : silu(z); }
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// out[t, c] = silu(bias[c] + sum_j w[j, c] * in(t - (taps - 1) + j, c)) (w [taps, C]: a tap's weights are contiguous);
// in() of a place before the step's
// first token of the sequence is the sequence's carried input (state [slots, taps - 1, C], oldest first;
// zeros when the sequence begins).  The input's channel c is column col0 + c of u.
template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ u, long long u_stride, int col0,
                                        const float* __restrict__ w, const float* __restrict__ bias, const T* __restrict__ state,
                                        const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                        const int* __restrict__ state_slot, int C, int taps, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const int first = q_start[s];
  const int r0 = t - first;
  const T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int r = r0 - (taps - 1) + j;
    const float x = r >= 0 ? to_float(u[(size_t)(first + r) * u_stride + col0 + c]) : to_float(carried[(size_t)(taps - 1 + r) * C + c]);
    acc = fmaf(w[(size_t)j * C + c], x, acc);
  }
  out[(size_t)t * C + c] = from_float<T>(conv_out<T>(act, acc));
}

// The same, eight channels a thread with 16-byte accesses (C, col0 and the row strides multiples of 8).  A block takes
// eight consecutive tokens of a slab of channels (threadIdx.y), so the rows that neighbouring tokens share are read
// from L1, not again from L2.
template <typename T>
__global__ void causal_conv_silu_vec_kernel(T* __restrict__ out, const T* __restrict__ u, long long u_stride, int col0,
                                            const float* __restrict__ w, const float* __restrict__ bias, const T* __restrict__ state,
                                            const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                            const int* __restrict__ state_slot, int n, int C, int taps, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int t = blockIdx.x * blockDim.y + threadIdx.y;
  if (c >= C || t >= n) return;
  const int s = seq_of_token[t];
  const int first = q_start[s];
  const int r0 = t - first;
  const T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  float acc[8];
  if (bias) load8(bias + c, acc);
  else {
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  }
  for (int j = 0; j < taps; ++j) {
    const int r = r0 - (taps - 1) + j;
    float x[8];
    if (r >= 0) load8(u + (size_t)(first + r) * u_stride + col0 + c, x);
    else load8(carried + (size_t)(taps - 1 + r) * C + c, x);
    float wv[8];
    load8(w + (size_t)j * C + c, wv);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = fmaf(wv[k], x[k], acc[k]);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = conv_out<T>(act, acc[k]);
  store8(out + (size_t)t * C + c, acc);
}

// For 2 to 4 taps: a thread takes eight channels of CONV_TOKS consecutive tokens, keeps the taps' weights and the last
// TAPS - 1 inputs in registers and reads one new row per token (the window is read anew where a sequence begins).
constexpr int CONV_TOKS = 8;

template <typename T, int TAPS>
__global__ void causal_conv_silu_window_kernel(T* __restrict__ out, const T* __restrict__ u, long long u_stride, int col0,
                                               const float* __restrict__ w, const float* __restrict__ bias, const T* __restrict__ state,
                                               const int* __restrict__ seq_of_token, const int* __restrict__ q_start,
                                               const int* __restrict__ state_slot, int n, int C, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int t0 = blockIdx.x * CONV_TOKS;
  float wv[TAPS][8], bv[8], win[TAPS - 1][8];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) load8(w + (size_t)j * C + c, wv[j]);
  if (bias) load8(bias + c, bv);
  else {
#pragma unroll
    for (int k = 0; k < 8; ++k) bv[k] = 0.f;
  }
  // the thread's rows and their sequences are requested together, before any arithmetic (rows behind the last token
  // repeat it and are not stored)
  float cur[CONV_TOKS][8];
  int seq[CONV_TOKS];
#pragma unroll
  for (int i = 0; i < CONV_TOKS; ++i) {
    const int t = min(t0 + i, n - 1);
    seq[i] = seq_of_token[t];
    load8(u + (size_t)t * u_stride + col0 + c, cur[i]);
  }
  int prev = -1;
#pragma unroll
  for (int i = 0; i < CONV_TOKS; ++i) {
    const int t = t0 + i;
    if (t >= n) break;
    const int s = seq[i];
    if (s != prev) {  // the first token of this thread, or of a sequence: the window comes from memory
      const int first = q_start[s];
      const int r0 = t - first;
      const T* carried = state + (size_t)state_slot[s] * (TAPS - 1) * C;
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) {
        const int r = r0 - (TAPS - 1) + j;
        if (r >= 0) load8(u + (size_t)(first + r) * u_stride + col0 + c, win[j]);
        else load8(carried + (size_t)(TAPS - 1 + r) * C + c, win[j]);
      }
      prev = s;
    }
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float a = bv[k];
#pragma unroll
      for (int j = 0; j < TAPS - 1; ++j) a = fmaf(wv[j][k], win[j][k], a);
      acc[k] = conv_out<T>(act, fmaf(wv[TAPS - 1][k], cur[i][k], a));
    }
    store8(out + (size_t)t * C + c, acc);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
#pragma unroll
      for (int j = 0; j + 1 < TAPS - 1; ++j) win[j][k] = win[j + 1][k];
      win[TAPS - 2][k] = cur[i][k];
    }
  }
}

// After the convolution: each sequence's carried inputs become its last taps - 1 inputs (older carried
// inputs move up when the step brought fewer).  In place: slot i is written from slot i + q_len or from u.
template <typename T>
__global__ void conv_state_update_kernel(T* __restrict__ state, const T* __restrict__ u, long long u_stride, int col0,
                                         const int* __restrict__ q_start, const int* __restrict__ state_slot, int C, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = blockIdx.y;
  const int first = q_start[s], len = q_start[s + 1] - first;
  T* carried = state + (size_t)state_slot[s] * (taps - 1) * C;
  for (int i = 0; i < taps - 1; ++i) {
    const int r = len - (taps - 1) + i;
    carried[(size_t)i * C + c] = r >= 0 ? u[(size_t)(first + r) * u_stride + col0 + c] : carried[(size_t)(i + len) * C + c];
  }
}

// The scan.  Per (sequence, head): S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x P), y = S^T C + D x, with
// dt = softplus(dt_raw + dt_bias), over the sequence's tokens of this step in order; S starts from and returns
// to the sequence's slot of state [slots, heads, P, N] (N fastest: a thread's share of a column is contiguous).
// A CTA owns PB columns p of one head; NS threads (8, or 16 where the launch would otherwise leave the
// GPU short of warps) share a pair of columns (p, p + 1), thread nl holding n = (k * NS + nl) * 4 + j
// (k < NPT / 4, j < 4) of both, so that a B or C value read from shared memory serves
// two multiply-adds; the eight add their shares of y by shuffles, always in the same order.  The step's tokens
// come through shared memory in tiles of TB tokens (x of the CTA's columns, B and C of the head's group, the
// step sizes and decays, which one thread per token computes), so the walk over a tile touches no global memory;
// the tile's y leaves through shared memory too.
//   xbc [n, inner + 2 G N]: x | B | C after convolution and activation; dt_raw: column dt_col + head of u.
constexpr int SCAN_TB = 32;
constexpr int SCAN_MAXV = 17;  // 16-byte loads of the next tile a thread may hold in registers

// eight consecutive staged values as floats
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(q[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
}

// PREFETCH (bfloat16 inputs whose runs of eight are 16-byte aligned): the next tile's x, B, C and step sizes are
// requested into registers before the walk over the current tile and stored to shared memory after it, so the
// walk hides their latency.  Otherwise a tile is staged element by element before its walk.
template <typename T, int NPT, int NS, bool PREFETCH>
__global__ void __launch_bounds__(256) ssm_scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ u,
                                                       long long u_stride, int dt_col, const float* __restrict__ dt_bias,
                                                       const float* __restrict__ A_log, const float* __restrict__ D,
                                                       float* __restrict__ state, const int* __restrict__ q_start,
                                                       const int* __restrict__ state_slot, int heads, int P, int N, int groups, int PB) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NP = NPT * NS;  // N rounded up: rows beyond N hold zeros and stay zero
  extern __shared__ __align__(16) float smem[];
  float* Bs = smem;                     // [TB][NP]
  float* Cs = Bs + SCAN_TB * NP;        // [TB][NP]
  float* xs = Cs + SCAN_TB * NP;        // [TB][PB]
  float* ys = xs + SCAN_TB * PB;        // [TB][PB]
  float* dts = ys + SCAN_TB * PB;       // [TB]
  float* decs = dts + SCAN_TB;          // [TB]
  const int head = blockIdx.x, s = blockIdx.y;
  const int tid = threadIdx.x, nl = tid & (NS - 1), pl = 2 * (tid / NS);
  const int p0 = blockIdx.z * PB, p = p0 + pl;
  const bool live = p < P, live1 = p + 1 < P;
  const int inner = heads * P, C = inner + 2 * groups * N;
  const int g = head / (heads / groups);
  const int first = q_start[s], last = q_start[s + 1];
  float* S0 = state + (((size_t)state_slot[s] * heads + head) * P + (live ? p : 0)) * N;
  const bool vec = (N & 3) == 0;
  float S[NPT], S1[NPT];  // columns p and p + 1
#pragma unroll
  for (int k = 0; k < NPT / 4; ++k) {
    const int n0 = (k * NS + nl) * 4;
    if (live && vec && n0 < N) {
      const float4 v = *reinterpret_cast<const float4*>(S0 + n0);
      S[4 * k] = v.x; S[4 * k + 1] = v.y; S[4 * k + 2] = v.z; S[4 * k + 3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) S[4 * k + j] = (live && n0 + j < N) ? S0[n0 + j] : 0.f;
    }
    if (live1 && vec && n0 < N) {
      const float4 v = *reinterpret_cast<const float4*>(S0 + N + n0);
      S1[4 * k] = v.x; S1[4 * k + 1] = v.y; S1[4 * k + 2] = v.z; S1[4 * k + 3] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) S1[4 * k + j] = (live1 && n0 + j < N) ? S0[N + n0 + j] : 0.f;
    }
  }
  const float A = expf(A_log[head]), bias = dt_bias[head], Dh = D[head];
  const int xcol = head * P + p0, bcol = inner + g * N, ccol = inner + groups * N + g * N;
  if (first >= last) goto store_state;
  {
    // ---- staging of a tile: element by element, or (PREFETCH) in two halves around the walk over the tile before
    const int width = PB + 2 * NP;
    const int xi = PB >> 3, ni = N >> 3, per_tok = xi + 2 * ni;  // runs of eight per token: x, B, C
    uint4 buf[PREFETCH ? SCAN_MAXV : 1];
    float dt_next = 0.f;
    auto request = [&](int tile) {
      if constexpr (PREFETCH) {
        const int cnt = min(SCAN_TB, last - tile);
#pragma unroll
        for (int i = 0; i < SCAN_MAXV; ++i) {
          const int item = tid + i * blockDim.x;
          if (item < cnt * per_tok) {
            const int tok = item / per_tok, o = item - tok * per_tok;
            const T* row = xbc + (size_t)(tile + tok) * C;
            const T* src = o < xi ? row + xcol + o * 8 : (o < xi + ni ? row + bcol + (o - xi) * 8 : row + ccol + (o - xi - ni) * 8);
            buf[i] = *reinterpret_cast<const uint4*>(src);
          }
        }
        if (tid < cnt) dt_next = to_float(u[(size_t)(tile + tid) * u_stride + dt_col + head]);
      }
    };
    auto stage = [&](int tile) {
      const int cnt = min(SCAN_TB, last - tile);
      if constexpr (PREFETCH) {
#pragma unroll
        for (int i = 0; i < SCAN_MAXV; ++i) {
          const int item = tid + i * blockDim.x;
          if (item < cnt * per_tok) {
            const int tok = item / per_tok, o = item - tok * per_tok;
            float v[8];
            unpack8(buf[i], v);
            float* dst;
            if (o < xi) {
              dst = xs + tok * PB + o * 8;
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (p0 + o * 8 + k >= P) v[k] = 0.f;
            } else if (o < xi + ni) {
              dst = Bs + tok * NP + (o - xi) * 8;
            } else {
              dst = Cs + tok * NP + (o - xi - ni) * 8;
            }
            reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
          }
        }
      } else {
        for (int e = tid; e < cnt * width; e += blockDim.x) {
          const int tok = e / width, off = e - tok * width;
          const T* row = xbc + (size_t)(tile + tok) * C;
          if (off < PB) {
            xs[tok * PB + off] = (p0 + off < P) ? to_float(row[xcol + off]) : 0.f;
          } else if (off < PB + NP) {
            const int n = off - PB;
            Bs[tok * NP + n] = n < N ? to_float(row[bcol + n]) : 0.f;
          } else {
            const int n = off - PB - NP;
            Cs[tok * NP + n] = n < N ? to_float(row[ccol + n]) : 0.f;
          }
        }
        if (tid < cnt) dt_next = to_float(u[(size_t)(tile + tid) * u_stride + dt_col + head]);
      }
      if (tid < cnt) {
        const float dt = softplus(dt_next + bias);
        dts[tid] = dt;
        decs[tid] = expf(-A * dt);
      }
    };
    if constexpr (PREFETCH) {  // columns of B and C beyond N are never staged: zero once
      if (N < NP) {
        for (int e = tid; e < 2 * SCAN_TB * NP; e += blockDim.x) Bs[e] = 0.f;
        __syncthreads();
      }
    }
    request(first);
    stage(first);
    __syncthreads();
    for (int tile = first; tile < last; tile += SCAN_TB) {
      const int cnt = min(SCAN_TB, last - tile);
      const bool more = tile + SCAN_TB < last;
      if (more) request(tile + SCAN_TB);
#pragma unroll 2
      for (int t = 0; t < cnt; ++t) {
        const float2 x = *reinterpret_cast<const float2*>(xs + t * PB + pl);
        const float dt = dts[t], decay = decs[t];
        const float dtx0 = dt * x.x, dtx1 = dt * x.y;
        const float4* b4 = reinterpret_cast<const float4*>(Bs + t * NP);
        const float4* c4 = reinterpret_cast<const float4*>(Cs + t * NP);
        float a0 = 0.f, a1 = 0.f, e0 = 0.f, e1 = 0.f;  // two partial sums a column: shorter chains, a fixed order
#pragma unroll
        for (int k = 0; k < NPT / 4; ++k) {
          const float4 b = b4[k * NS + nl], c = c4[k * NS + nl];
          S[4 * k] = fmaf(decay, S[4 * k], b.x * dtx0);
          S[4 * k + 1] = fmaf(decay, S[4 * k + 1], b.y * dtx0);
          S[4 * k + 2] = fmaf(decay, S[4 * k + 2], b.z * dtx0);
          S[4 * k + 3] = fmaf(decay, S[4 * k + 3], b.w * dtx0);
          S1[4 * k] = fmaf(decay, S1[4 * k], b.x * dtx1);
          S1[4 * k + 1] = fmaf(decay, S1[4 * k + 1], b.y * dtx1);
          S1[4 * k + 2] = fmaf(decay, S1[4 * k + 2], b.z * dtx1);
          S1[4 * k + 3] = fmaf(decay, S1[4 * k + 3], b.w * dtx1);
          a0 = fmaf(S[4 * k], c.x, a0);
          a1 = fmaf(S[4 * k + 1], c.y, a1);
          a0 = fmaf(S[4 * k + 2], c.z, a0);
          a1 = fmaf(S[4 * k + 3], c.w, a1);
          e0 = fmaf(S1[4 * k], c.x, e0);
          e1 = fmaf(S1[4 * k + 1], c.y, e1);
          e0 = fmaf(S1[4 * k + 2], c.z, e0);
          e1 = fmaf(S1[4 * k + 3], c.w, e1);
        }
        float acc0 = a0 + a1, acc1 = e0 + e1;
#pragma unroll
        for (int o = 1; o < NS; o <<= 1) {
          acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
          acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
        }
        if (nl == 0) *reinterpret_cast<float2*>(ys + t * PB + pl) = make_float2(fmaf(Dh, x.x, acc0), fmaf(Dh, x.y, acc1));
      }
      __syncthreads();  // the tile has been walked: its inputs may be overwritten, its y is complete
      for (int e = tid; e < cnt * PB; e += blockDim.x) {
        const int tok = e / PB, off = e - tok * PB;
        if (p0 + off < P) y[(size_t)(tile + tok) * inner + xcol + off] = ys[e];
      }
      if (more) stage(tile + SCAN_TB);
      __syncthreads();  // the next tile is staged, and ys has been read
    }
  }
store_state:
  if (!live) return;
#pragma unroll
  for (int k = 0; k < NPT / 4; ++k) {
    const int n0 = (k * NS + nl) * 4;
    if (vec && n0 < N) {
      *reinterpret_cast<float4*>(S0 + n0) = make_float4(S[4 * k], S[4 * k + 1], S[4 * k + 2], S[4 * k + 3]);
      if (live1) *reinterpret_cast<float4*>(S0 + N + n0) = make_float4(S1[4 * k], S1[4 * k + 1], S1[4 * k + 2], S1[4 * k + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + j < N) {
          S0[n0 + j] = S[4 * k + j];
          if (live1) S0[N + n0 + j] = S1[4 * k + j];
        }
    }
  }
}

// out[t, part] = g / sqrt(mean(g^2 over the part) + eps) * w, g = y * silu(z); the row is cut into `parts`
// equal runs.  z is column z_col + c of u.  One block per (token, part).  gate_after: the gate stays out of the
// norm, out = y / sqrt(mean(y^2) + eps) * w * silu(z).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ u, long long u_stride,
                                           int z_col, const float* __restrict__ w, int inner, int parts, float eps, int gate_after) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int part = blockIdx.y, t = blockIdx.x;
  const int size = inner / parts, c0 = part * size;
  const float* yrow = y + (size_t)t * inner + c0;
  const T* zrow = u + (size_t)t * u_stride + z_col + c0;
  float q = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float gv = gate_after ? yrow[i] : yrow[i] * norm_gate(to_float(zrow[i]), gate_after);
    q = fmaf(gv, gv, q);
  }
  const float r = 1.f / sqrtf(block_sum(q, red) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float gate = norm_gate(to_float(zrow[i]), gate_after);
    out[(size_t)t * inner + c0 + i] = from_float<T>(gate_after ? yrow[i] * r * w[c0 + i] * gate : yrow[i] * gate * r * w[c0 + i]);
  }
}

// The same with the part's values in registers between the two passes and 16- and 32-byte accesses: a thread owns
// CHUNKS runs of eight columns (size % 8 == 0, size <= 8 * THREADS * CHUNKS, aligned rows).
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS) gated_group_rmsnorm_vec_kernel(T* __restrict__ out, const float* __restrict__ y,
                                                                          const T* __restrict__ u, long long u_stride, int z_col,
                                                                          const float* __restrict__ w, int inner, int parts, float eps,
                                                                          int gate_after) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int part = blockIdx.y, t = blockIdx.x;
  const int size = inner / parts, c0 = part * size;
  const float* yrow = y + (size_t)t * inner + c0;
  const T* zrow = u + (size_t)t * u_stride + z_col + c0;
  float gv[CHUNKS][8];
  float q = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < size) {
      float z[8];
      load8(yrow + col, gv[c]);
      load8(zrow + col, z);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float gate = norm_gate(z[k], gate_after);
        q = gate_after ? fmaf(gv[c][k], gv[c][k], q) : fmaf(gv[c][k] * gate, gv[c][k] * gate, q);
        gv[c][k] *= gate;  // the gate is a factor of the output either way
      }
    }
  }
  const float r = 1.f / sqrtf(block_sum(q, red) / (float)size + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < size) {
      float wv[8], o[8];
      load8(w + c0 + col, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = gv[c][k] * r * wv[k];
      store8(out + (size_t)t * inner + c0 + col, o);
    }
  }
}

template <typename T, int NPT, int NS>
int launch_scan_shape(float* y, const T* xbc, const T* u, long long u_stride, int dt_col, const float* dt_bias, const float* A_log,
                      const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int P, int N, int groups,
                      int max_len, cudaStream_t stream) {
  // columns per CTA (a pair of them per NS threads, 256 threads at most), fewer for narrow heads and where it takes
  // smaller CTAs to give every SM one
  const int most = 512 / NS;
  int PB = P >= most ? most : ((P + 7) / 8) * 8;
  while (PB > 16 && (long long)heads * num_seqs * ((P + PB - 1) / PB) < sm_count()) PB /= 2;
  PB = ((PB + 7) / 8) * 8;
  const int threads = PB / 2 * NS;
  const dim3 grid(heads, num_seqs, (P + PB - 1) / PB), block(threads);
  const size_t smem = (size_t)(2 * SCAN_TB * NPT * NS + 2 * SCAN_TB * PB + 2 * SCAN_TB) * sizeof(float);
  // runs of eight inputs by 16-byte loads into registers, a tile ahead: bfloat16, every run aligned, few enough a thread
  // (only where some sequence brings more than one tile: a decode step has nothing to fetch ahead)
  const int per_thread = (SCAN_TB * (PB / 8 + 2 * (N / 8)) + threads - 1) / threads;
  const bool prefetch = sizeof(T) == 2 && max_len > SCAN_TB && (P % 8) == 0 && (N % 8) == 0 && ((uintptr_t)xbc & 15) == 0 && per_thread <= SCAN_MAXV;
  if (prefetch && sizeof(T) == 2) {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      cudaError_t e = cudaFuncSetAttribute(ssm_scan_kernel<T, NPT, NS, sizeof(T) == 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    return (int)launch_pdl((ssm_scan_kernel<T, NPT, NS, sizeof(T) == 2>), grid, block, smem, stream, 1, y, xbc, u, u_stride, dt_col, dt_bias, A_log,
                           D, state, q_start, state_slot, heads, P, N, groups, PB);
  }
  static MaxPerDevice set;
  if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
    cudaError_t e = cudaFuncSetAttribute(ssm_scan_kernel<T, NPT, NS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    set.here() = (int)smem;
  }
  return (int)launch_pdl((ssm_scan_kernel<T, NPT, NS, false>), grid, block, smem, stream, 1, y, xbc, u, u_stride, dt_col, dt_bias, A_log, D, state,
                         q_start, state_slot, heads, P, N, groups, PB);
}

template <typename T>
int launch_scan(float* y, const T* xbc, const T* u, long long u_stride, int dt_col, const float* dt_bias, const float* A_log,
                const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs, int heads, int P, int N, int groups,
                int max_len, cudaStream_t stream) {
  // Threads per pair of columns: 8 hold the most state each (the fewest shared-memory reads per multiply-add); 16 where 8
  // would leave an SM with fewer than four warps, as one long prompt on a few heads does.  (Measured on a B200, 4,096
  // tokens, state 128 x 64: 64 heads 1.70 ms with 8 and 1.42 with 16; 128 heads 1.74 and 2.46; 32 made everything slower.)
  const long long pairs = (long long)heads * num_seqs * ((P + 1) / 2);
  const int ns = ((pairs * 8 < 4LL * 32 * sm_count() && N > 32) || N > 256) ? 16 : 8;  // (a state above 256 takes 16 threads a pair to hold it)
  const int quads = (N + 4 * ns - 1) / (4 * ns);  // float4 runs of n per thread
#define DLI_SCAN(NPT, NS) \
  return launch_scan_shape<T, NPT, NS>(y, xbc, u, u_stride, dt_col, dt_bias, A_log, D, state, q_start, state_slot, num_seqs, heads, P, N, groups, max_len, stream)
  if (ns == 8) {
    if (quads <= 1) DLI_SCAN(4, 8);
    if (quads <= 2) DLI_SCAN(8, 8);
    if (quads <= 4) DLI_SCAN(16, 8);
    if (quads <= 8) DLI_SCAN(32, 8);
  } else {
    if (quads <= 1) DLI_SCAN(4, 16);
    if (quads <= 2) DLI_SCAN(8, 16);
    if (quads <= 4) DLI_SCAN(16, 16);
    if (quads <= 8) DLI_SCAN(32, 16);
  }
#undef DLI_SCAN
  return DLI_ERR_UNSUPPORTED;
}

}  // namespace

DLI_EXPORT int dli_causal_conv_silu(void* out, const void* u, long long u_stride, int col0, const float* w, const float* bias,
                                    const void* state, const int* seq_of_token, const int* q_start, const int* state_slot, int n, int C,
                                    int taps, int act, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (C < 1 || taps < 1 || (C + 127) / 128 > 65535) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if ((C % 8) == 0 && (col0 % 8) == 0 && (u_stride % 8) == 0 && (((uintptr_t)out | (uintptr_t)u | (uintptr_t)state | (uintptr_t)bias | (uintptr_t)w) & 15) == 0) {
    const int items = C / 8;
    if (taps >= 2 && taps <= 4 && n > 64) {  // portions: a sliding window in registers
      const int wt = items >= 128 ? 128 : 64;
      const dim3 wgrid((n + CONV_TOKS - 1) / CONV_TOKS, (items + wt - 1) / wt);
#define DLI_CONV_WIN(T, TAPS)                                                                                                      \
  return (int)launch_pdl((causal_conv_silu_window_kernel<T, TAPS>), wgrid, dim3(wt), 0, stream, 1, (T*)out, (const T*)u, u_stride, col0, w, \
                         bias, (const T*)state, seq_of_token, q_start, state_slot, n, C, act)
      if (dtype == DLI_F32) {
        if (taps == 2) DLI_CONV_WIN(float, 2);
        if (taps == 3) DLI_CONV_WIN(float, 3);
        DLI_CONV_WIN(float, 4);
      } else {
        if (taps == 2) DLI_CONV_WIN(__nv_bfloat16, 2);
        if (taps == 3) DLI_CONV_WIN(__nv_bfloat16, 3);
        DLI_CONV_WIN(__nv_bfloat16, 4);
      }
#undef DLI_CONV_WIN
    }
    const dim3 vblock(32, 8), vgrid((n + 7) / 8, (items + 31) / 32);
    if (dtype == DLI_F32)
      e = launch_pdl((causal_conv_silu_vec_kernel<float>), vgrid, vblock, 0, stream, 1, (float*)out, (const float*)u, u_stride, col0, w, bias,
                     (const float*)state, seq_of_token, q_start, state_slot, n, C, taps, act);
    else
      e = launch_pdl((causal_conv_silu_vec_kernel<__nv_bfloat16>), vgrid, vblock, 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)u,
                     u_stride, col0, w, bias, (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, n, C, taps, act);
    return (int)e;
  }
  const dim3 grid(n, (C + 127) / 128), block(128);
  if (dtype == DLI_F32)
    e = launch_pdl((causal_conv_silu_kernel<float>), grid, block, 0, stream, 1, (float*)out, (const float*)u, u_stride, col0, w, bias,
                   (const float*)state, seq_of_token, q_start, state_slot, C, taps, act);
  else
    e = launch_pdl((causal_conv_silu_kernel<__nv_bfloat16>), grid, block, 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)u, u_stride,
                   col0, w, bias, (const __nv_bfloat16*)state, seq_of_token, q_start, state_slot, C, taps, act);
  return (int)e;
}

DLI_EXPORT int dli_conv_state_update(void* state, const void* u, long long u_stride, int col0, const int* q_start, const int* state_slot,
                                     int num_seqs, int C, int taps, int dtype, cudaStream_t stream) {
  if (num_seqs == 0 || taps <= 1) return 0;
  if (num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
  const dim3 grid((C + 127) / 128, num_seqs), block(128);
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((conv_state_update_kernel<float>), grid, block, 0, stream, 1, (float*)state, (const float*)u, u_stride, col0, q_start,
                   state_slot, C, taps);
  else
    e = launch_pdl((conv_state_update_kernel<__nv_bfloat16>), grid, block, 0, stream, 1, (__nv_bfloat16*)state, (const __nv_bfloat16*)u,
                   u_stride, col0, q_start, state_slot, C, taps);
  return (int)e;
}

DLI_EXPORT int dli_ssm_scan(float* y, const void* xbc, const void* u, long long u_stride, int dt_col, const float* dt_bias,
                            const float* A_log, const float* D, float* state, const int* q_start, const int* state_slot, int num_seqs,
                            int heads, int P, int N, int groups, int max_len, int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (heads < 1 || groups < 1 || heads % groups || P < 1 || N < 1 || num_seqs > 65535) return DLI_ERR_UNSUPPORTED;
  if (dtype == DLI_F32)
    return launch_scan<float>(y, (const float*)xbc, (const float*)u, u_stride, dt_col, dt_bias, A_log, D, state, q_start, state_slot,
                              num_seqs, heads, P, N, groups, max_len, stream);
  return launch_scan<__nv_bfloat16>(y, (const __nv_bfloat16*)xbc, (const __nv_bfloat16*)u, u_stride, dt_col, dt_bias, A_log, D, state,
                                    q_start, state_slot, num_seqs, heads, P, N, groups, max_len, stream);
}

DLI_EXPORT int dli_gated_group_rmsnorm(void* out, const float* y, const void* u, long long u_stride, int z_col, const float* w, int n,
                                       int inner, int parts, float eps, int gate_after, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (parts < 1 || parts > 65535 || inner % parts) return DLI_ERR_UNSUPPORTED;
  const int size = inner / parts;
  const dim3 grid(n, parts);
  cudaError_t e;
  if ((size % 8) == 0 && size <= 8192 && (z_col % 8) == 0 && (u_stride % 8) == 0 &&
      (((uintptr_t)out | (uintptr_t)y | (uintptr_t)u | (uintptr_t)w) & 15) == 0) {
#define DLI_GN_VEC(T, THREADS, CHUNKS)                                                                                               \
  return (int)launch_pdl((gated_group_rmsnorm_vec_kernel<T, THREADS, CHUNKS>), grid, dim3(THREADS), 0, stream, 1, (T*)out, y, (const T*)u, \
                         u_stride, z_col, w, inner, parts, eps, gate_after)
#define DLI_GN_SIZES(T)                       \
  if (size <= 256) DLI_GN_VEC(T, 32, 1);      \
  if (size <= 512) DLI_GN_VEC(T, 64, 1);      \
  if (size <= 1024) DLI_GN_VEC(T, 128, 1);    \
  if (size <= 2048) DLI_GN_VEC(T, 256, 1);    \
  if (size <= 4096) DLI_GN_VEC(T, 256, 2);    \
  DLI_GN_VEC(T, 256, 4)
    if (dtype == DLI_F32) {
      DLI_GN_SIZES(float);
    } else {
      DLI_GN_SIZES(__nv_bfloat16);
    }
#undef DLI_GN_SIZES
#undef DLI_GN_VEC
  }
  const int threads = size >= 1024 ? 256 : 128;
  if (dtype == DLI_F32)
    e = launch_pdl((gated_group_rmsnorm_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)out, y, (const float*)u, u_stride, z_col, w,
                   inner, parts, eps, gate_after);
  else
    e = launch_pdl((gated_group_rmsnorm_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, y,
                   (const __nv_bfloat16*)u, u_stride, z_col, w, inner, parts, eps, gate_after);
  return (int)e;
}
