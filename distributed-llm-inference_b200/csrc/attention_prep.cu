// What lies between an attention mixer's projections and its attention kernel when queries and keys are
// normed over their whole projection, or when the keys and values are one cached latent; and what lies behind the
// attention kernel when its output is gated.
// float32 and bfloat16 instantiations; all arithmetic is float32.
#include "common.cuh"

using namespace dli;

namespace {

// One block per token.  proj row: q (nh * d columns) | k (nkv * d columns), then whatever else the product made.
//   q <- q / rms(q over all nh * d) * wq,  k <- k / rms(k over all nkv * d) * wk      (normed != 0)
//   rotary (rotate-half pairing, first `rot` dimensions of each head, angle float32(position) * inv_freq[i])
//   q -> q_out [n, nh * d];  k -> k_pool at the token's slot;
//   v_pool gets the keys as projected (values_from_keys != 0) or the nkv * d columns behind k.
template <typename T>
__global__ void qk_norm_rotary_store_kernel(T* __restrict__ q_out, const T* __restrict__ proj, long long proj_stride,
                                            const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                            const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                            const int* __restrict__ slots, T* __restrict__ k_pool, T* __restrict__ v_pool, int nh,
                                            int nkv, int d, int rot, int page_size, int write_kv, int normed, int values_from_keys) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];  // (nh + nkv) * d
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nq = nh * d, nk = nkv * d;
  const T* src = proj + (size_t)t * proj_stride;
  float sq = 0.f, sk = 0.f;
  for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) {
    const float x = to_float(src[e]);
    row[e] = x;
    if (e < nq) sq = fmaf(x, x, sq); else sk = fmaf(x, x, sk);
  }
  float rq = 1.f, rk = 1.f;
  if (normed) {
    rq = 1.f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    rk = 1.f / sqrtf(block_sum(sk, red) / (float)nk + eps);
  } else {
    __syncthreads();
  }
  const float pos = (float)positions[t];
  const int half = rot >> 1;
  long long kv_base = 0;
  if (write_kv) {
    const int slot = slots[t];
    kv_base = ((long long)(slot / page_size) * nkv * page_size + slot % page_size) * d;  // + kvh * page_size * d + i
  }
  for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) {
    const bool is_q = e < nq;
    if (!is_q && !write_kv) continue;
    const int c = is_q ? e : e - nq;          // column inside q or k
    const int head = c / d, i = c - head * d;
    const float r = is_q ? rq : rk;
    const float* w = is_q ? wq : wk;
    float x = row[e] * r * (normed ? w[c] : 1.f);
    if (i < rot) {
      const int j = i < half ? i : i - half;
      const int pe = i < half ? e + half : e - half, pc = i < half ? c + half : c - half;
      const float xp = row[pe] * r * (normed ? w[pc] : 1.f);
      float sn, cs;
      sincosf(pos * inv_freq[j], &sn, &cs);
      x = i < half ? x * cs - xp * sn : x * cs + xp * sn;
    }
    if (is_q) {
      q_out[(size_t)t * nq + c] = from_float<T>(x);
    } else {
      const long long at = kv_base + (long long)head * page_size * d + i;
      k_pool[at] = from_float<T>(x);
      v_pool[at] = values_from_keys ? src[e] : src[e + nk];
    }
  }
}

// The same with 16-byte accesses, for d % 8 == 0, rot % 16 == 0 and 16-byte aligned rows.  A work item is a run of
// eight columns — together with its partner run, half the rotated span further, where it is rotated.  The token's
// cosines and sines are computed once, in shared memory, not once per head.
template <typename T>
__global__ void qk_norm_rotary_store_vec_kernel(T* __restrict__ q_out, const T* __restrict__ proj, long long proj_stride,
                                                const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                                const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                                const int* __restrict__ slots, T* __restrict__ k_pool, T* __restrict__ v_pool, int nh,
                                                int nkv, int d, int rot, int page_size, int write_kv, int normed, int values_from_keys) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float cs[];  // cos [rot / 2] | sin [rot / 2]
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int nq = nh * d, nk = nkv * d, half = rot >> 1;
  const T* src = proj + (size_t)t * proj_stride;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &cs[half + j], &cs[j]);
  float rq = 1.f, rk = 1.f;
  if (normed) {
    float sq = 0.f, sk = 0.f;
    for (int e = threadIdx.x * 8; e < nq + nk; e += blockDim.x * 8) {
      float x[8];
      load8(src + e, x);
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) ss = fmaf(x[k], x[k], ss);
      if (e < nq) sq += ss; else sk += ss;
    }
    rq = 1.f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    rk = 1.f / sqrtf(block_sum(sk, red) / (float)nk + eps);
  } else {
    __syncthreads();
  }
  long long kv_base = 0;
  if (write_kv) {
    const int slot = slots[t];
    kv_base = ((long long)(slot / page_size) * nkv * page_size + slot % page_size) * d;
  }
  // items per head: half / 8 rotated pairs, then (d - rot) / 8 runs that pass unrotated
  const int pair_items = half >> 3, per_head = pair_items + ((d - rot) >> 3);
  const int heads = nh + (write_kv ? nkv : 0);
  for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
    const int head = item / per_head, it = item - head * per_head;
    const bool is_q = head < nh;
    const int hh = is_q ? head : head - nh;
    const float r = is_q ? rq : rk;
    const float* w = (is_q ? wq : wk) + hh * d;
    const T* hsrc = src + head * d;  // q heads, then k heads, lie back to back
    T* dst = is_q ? q_out + (size_t)t * nq + hh * d : k_pool + kv_base + (long long)hh * page_size * d;
    T* vdst = is_q ? nullptr : v_pool + kv_base + (long long)hh * page_size * d;
    const T* vsrc = values_from_keys ? hsrc : hsrc + nk;
    if (it < pair_items) {
      const int i = it * 8;
      float lo[8], hi[8], wl[8], wh[8], ol[8], oh[8];
      load8(hsrc + i, lo);
      load8(hsrc + i + half, hi);
      if (vdst) {
        *reinterpret_cast<uint4*>(vdst + i) = *reinterpret_cast<const uint4*>(vsrc + i);
        *reinterpret_cast<uint4*>(vdst + i + half) = *reinterpret_cast<const uint4*>(vsrc + i + half);
        if (sizeof(T) == 4) {
          *reinterpret_cast<uint4*>(vdst + i + 4) = *reinterpret_cast<const uint4*>(vsrc + i + 4);
          *reinterpret_cast<uint4*>(vdst + i + half + 4) = *reinterpret_cast<const uint4*>(vsrc + i + half + 4);
        }
      }
      if (normed) {
        load8(w + i, wl);
        load8(w + i + half, wh);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float a = lo[k] * r * (normed ? wl[k] : 1.f), b = hi[k] * r * (normed ? wh[k] : 1.f);
        const float c = cs[i + k], sn = cs[half + i + k];
        ol[k] = a * c - b * sn;
        oh[k] = b * c + a * sn;
      }
      store8(dst + i, ol);
      store8(dst + i + half, oh);
    } else {
      const int i = rot + (it - pair_items) * 8;
      float x[8], wv[8];
      load8(hsrc + i, x);
      if (vdst) {
        *reinterpret_cast<uint4*>(vdst + i) = *reinterpret_cast<const uint4*>(vsrc + i);
        if (sizeof(T) == 4) *reinterpret_cast<uint4*>(vdst + i + 4) = *reinterpret_cast<const uint4*>(vsrc + i + 4);
      }
      if (normed) {
        load8(w + i, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) x[k] = x[k] * r * wv[k];
      }
      store8(dst + i, x);
    }
  }
}

// out[t, c] *= sigmoid(gate[t, c]), eight columns a thread (cols % 8 == 0, aligned rows)
template <typename T>
__global__ void sigmoid_gate_vec_kernel(T* __restrict__ out, const T* __restrict__ gate, long long gate_stride, int n, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = cols >> 3;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * per_row) return;
  const int t = (int)(idx / per_row), c = (int)(idx - (long long)t * per_row) * 8;
  float o[8], g[8];
  load8(out + (size_t)t * cols + c, o);
  load8(gate + (size_t)t * gate_stride + c, g);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = o[k] / (1.f + expf(-g[k]));
  store8(out + (size_t)t * cols + c, o);
}

// out[t, c] *= sigmoid(gate[t * gate_stride + c])
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, const T* __restrict__ gate, long long gate_stride, int n, int cols) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)n * cols) return;
  const int t = (int)(idx / cols), c = (int)(idx - (long long)t * cols);
  const float g = to_float(gate[(size_t)t * gate_stride + c]);
  out[idx] = from_float<T>(to_float(out[idx]) / (1.f + expf(-g)));
}

}  // namespace

DLI_EXPORT int dli_qk_norm_rotary_store(void* q_out, const void* proj, long long proj_stride, const float* wq, const float* wk,
                                        float eps, const int* positions, const float* inv_freq, const int* slots, void* k_pool,
                                        void* v_pool, int n, int nh, int nkv, int d, int rot, int page_size, int write_kv,
                                        int normed, int values_from_keys, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  const size_t smem = (size_t)(nh + nkv) * d * sizeof(float);
  if (nh < 1 || nkv < 1 || d < 1 || rot < 0 || rot > d || (rot & 1) || smem > 200 * 1024 || (rot && !inv_freq) ||
      (normed && (!wq || !wk)) || (write_kv && (!slots || !k_pool || !v_pool)))
    return DLI_ERR_UNSUPPORTED;
  const int threads = (nh + nkv) * d >= 2048 ? 512 : 256;
  cudaError_t e;
  const size_t esize = dtype == DLI_F32 ? 4 : 2;
  const bool aligned = (d % 8) == 0 && (rot % 16) == 0 && (proj_stride % 8) == 0 && rot * sizeof(float) <= 48 * 1024 &&
                       (((uintptr_t)q_out | (uintptr_t)proj | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)wq | (uintptr_t)wk) & 15) == 0 &&
                       ((size_t)d * esize) % 16 == 0;
  if (aligned) {
    const int items = (nh + nkv) * (d / 8);
    const int vt = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
    const size_t vsmem = (size_t)rot * sizeof(float);
    if (dtype == DLI_F32)
      e = launch_pdl((qk_norm_rotary_store_vec_kernel<float>), dim3(n), dim3(vt), vsmem, stream, 1, (float*)q_out, (const float*)proj,
                     proj_stride, wq, wk, eps, positions, inv_freq, slots, (float*)k_pool, (float*)v_pool, nh, nkv, d, rot, page_size,
                     write_kv, normed, values_from_keys);
    else
      e = launch_pdl((qk_norm_rotary_store_vec_kernel<__nv_bfloat16>), dim3(n), dim3(vt), vsmem, stream, 1, (__nv_bfloat16*)q_out,
                     (const __nv_bfloat16*)proj, proj_stride, wq, wk, eps, positions, inv_freq, slots, (__nv_bfloat16*)k_pool,
                     (__nv_bfloat16*)v_pool, nh, nkv, d, rot, page_size, write_kv, normed, values_from_keys);
    return (int)e;
  }
  if (dtype == DLI_F32) {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(qk_norm_rotary_store_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((qk_norm_rotary_store_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)q_out, (const float*)proj,
                   proj_stride, wq, wk, eps, positions, inv_freq, slots, (float*)k_pool, (float*)v_pool, nh, nkv, d, rot, page_size,
                   write_kv, normed, values_from_keys);
  } else {
    static MaxPerDevice set;
    if ((int)smem > 48 * 1024 && set.here() < (int)smem) {
      e = cudaFuncSetAttribute(qk_norm_rotary_store_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
      set.here() = (int)smem;
    }
    e = launch_pdl((qk_norm_rotary_store_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)q_out,
                   (const __nv_bfloat16*)proj, proj_stride, wq, wk, eps, positions, inv_freq, slots, (__nv_bfloat16*)k_pool,
                   (__nv_bfloat16*)v_pool, nh, nkv, d, rot, page_size, write_kv, normed, values_from_keys);
  }
  return (int)e;
}

// ---------------------------------------------------------------- attention over a cached latent
// One block per token.  proj row: per head d plain and dr rotated query numbers (nh heads), then the down projection:
// r latent numbers and dr numbers of a key part that all heads share.
//   latent <- latent / rms(latent) * w_norm                      (float32; eps inside the root)
//   the first `rot` of the dr numbers of the key part and of every head's query part are rotated by the position
//   (rotate-half pairing, angle float32(position) * inv_freq[i]); the rest pass through
//   cache row  latent | key part      -> k_pool [pages][1][page_size][r + dr] at the token's slot (if slots)
//   query parts                       -> q_out [n][nh][r + dr], columns r .. r + dr of every head
template <typename T>
__global__ void latent_prep_kernel(T* __restrict__ q_out, const T* __restrict__ proj, long long proj_stride,
                                   const float* __restrict__ w_norm, float eps, const int* __restrict__ positions,
                                   const float* __restrict__ inv_freq, const int* __restrict__ slots, T* __restrict__ k_pool, int nh,
                                   int d, int dr, int r, int rot, int page_size, float amp) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float trig[];  // cos[half] | sin[half]
  __shared__ float red[33];
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const T* src = proj + (size_t)t * proj_stride;
  const T* down = src + (size_t)nh * (d + dr);
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    trig[i] = cs * amp;  // amp: one factor on every cosine and sine (1: none)
    trig[half + i] = sn * amp;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < r; i += blockDim.x) {
    const float x = to_float(down[i]);
    ss = fmaf(x, x, ss);
  }
  const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)r + eps);  // (the barriers inside also publish trig)
  const int slot = slots ? slots[t] : -1;
  const int row = r + dr;
  T* krow = slot >= 0 ? k_pool + (size_t)slot * row : nullptr;  // one KV head: a page is page_size rows back to back
  if (krow)
    for (int i = threadIdx.x; i < r; i += blockDim.x) krow[i] = from_float<T>(to_float(down[i]) * inv * w_norm[i]);
  // rotated parts, a pair of partners (i, i + half) a thread: head nh is the shared key part
  const int pairs = half + (dr - rot);  // per head: the rotated pairs, then the numbers that pass through
  for (int e = threadIdx.x; e < (nh + 1) * pairs; e += blockDim.x) {
    const int head = e / pairs, j = e - head * pairs;
    const T* part = head < nh ? src + (size_t)head * (d + dr) + d : down + r;
    T* dst = head < nh ? q_out + ((size_t)t * nh + head) * row + r : (krow ? krow + r : nullptr);
    if (!dst) continue;
    if (j < half) {
      const float lo = to_float(part[j]), hi = to_float(part[j + half]);
      const float cs = trig[j], sn = trig[half + j];
      dst[j] = from_float<T>(lo * cs - hi * sn);
      dst[j + half] = from_float<T>(hi * cs + lo * sn);
    } else {
      dst[rot + j - half] = part[rot + j - half];
    }
  }
}

DLI_EXPORT int dli_latent_prep(void* q_out, const void* proj, long long proj_stride, const float* w_norm, float eps, const int* positions,
                               const float* inv_freq, const int* slots, void* k_pool, int n, int nh, int d, int dr, int r, int rot,
                               int page_size, float amp, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (nh < 1 || d < 1 || dr < 0 || r < 1 || rot < 0 || rot > dr || (rot & 1) || (rot && !inv_freq) || (slots && !k_pool) || page_size < 1 ||
      rot * sizeof(float) > 48 * 1024)
    return DLI_ERR_UNSUPPORTED;
  const int work = r > (nh + 1) * dr ? r : (nh + 1) * dr;
  const int threads = work >= 4096 ? 256 : 128;  // small blocks: a token's work is short, and more blocks fit an SM
  const size_t smem = (size_t)(rot > 0 ? rot : 1) * sizeof(float);
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((latent_prep_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)q_out, (const float*)proj, proj_stride,
                   w_norm, eps, positions, inv_freq, slots, (float*)k_pool, nh, d, dr, r, rot, page_size, amp);
  else
    e = launch_pdl((latent_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)q_out,
                   (const __nv_bfloat16*)proj, proj_stride, w_norm, eps, positions, inv_freq, slots, (__nv_bfloat16*)k_pool, nh, d, dr, r,
                   rot, page_size, amp);
  return (int)e;
}

// ---------------------------------------------------------------- rotation, then a unit root mean square per head, then the pages
// One block per token, a warp per head.  x row: q (nh heads of d) | k (nkv heads of d) | v (nkv heads of dv), as the
// convolution left them.  Every q and k head is rotated on its first `rot` dimensions (rotate-half pairing, angle
// float32(position) * inv_freq[i]) and then, if unit_eps >= 0, divided by sqrt(mean(head^2) + unit_eps), all in float32.
// Rows of D = max(d, dv) numbers leave, the shorter of keys and values padded with zeros:
//   q -> q_out [n][nh][D];   k -> k_pool, v -> v_pool [pages][nkv][page_size][D] at the token's slot (if slots)
template <typename T>
__global__ void rotary_unit_store_kernel(T* __restrict__ q_out, const T* __restrict__ x, long long x_stride, const int* __restrict__ positions,
                                         const float* __restrict__ inv_freq, const int* __restrict__ slots, T* __restrict__ k_pool,
                                         T* __restrict__ v_pool, int nh, int nkv, int d, int dv, int D, int rot, float unit_eps, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];  // cos[half] | sin[half] | a head of d floats per warp
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  float* trig = sm;
  float* buf = sm + rot + (size_t)warp * d;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &trig[half + i], &trig[i]);
  __syncthreads();
  const T* src = x + (size_t)t * x_stride;
  const int slot = slots ? slots[t] : -1;
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? slot % page_size : 0;
  for (int head = warp; head < nh + 2 * nkv; head += warps) {
    if (head >= nh + nkv) {  // a value head: copied, padded
      if (slot < 0) continue;
      const int g = head - nh - nkv;
      const T* part = src + (size_t)(nh + nkv) * d + (size_t)g * dv;
      T* dst = v_pool + ((page * nkv + g) * page_size + off) * D;
      for (int i = lane; i < D; i += 32) dst[i] = i < dv ? part[i] : from_float<T>(0.f);
      continue;
    }
    const T* part = src + (size_t)head * d;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      float v;
      if (i < half) {
        v = to_float(part[i]) * trig[i] - to_float(part[i + half]) * trig[half + i];
      } else if (i < rot) {
        v = to_float(part[i]) * trig[i - half] + to_float(part[i - half]) * trig[i];
      } else {
        v = to_float(part[i]);
      }
      buf[i] = v;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv = unit_eps >= 0.f ? 1.f / sqrtf(ss / (float)d + unit_eps) : 1.f;
    T* dst;
    if (head < nh) {
      dst = q_out + ((size_t)t * nh + head) * D;
    } else {
      if (slot < 0) { __syncwarp(); continue; }
      dst = k_pool + ((page * nkv + (head - nh)) * page_size + off) * D;
    }
    __syncwarp();
    for (int i = lane; i < D; i += 32) dst[i] = from_float<T>(i < d ? buf[i] * inv : 0.f);
    __syncwarp();
  }
}

DLI_EXPORT int dli_rotary_unit_store(void* q_out, const void* x, long long x_stride, const int* positions, const float* inv_freq,
                                     const int* slots, void* k_pool, void* v_pool, int n, int nh, int nkv, int d, int dv, int rot,
                                     float unit_eps, int page_size, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (nh < 1 || nkv < 1 || d < 1 || dv < 1 || rot < 0 || rot > d || (rot & 1) || (rot && !inv_freq) || (slots && (!k_pool || !v_pool)) || page_size < 1)
    return DLI_ERR_UNSUPPORTED;
  const int D = d > dv ? d : dv;
  const int heads = nh + 2 * nkv;
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 64);
  const size_t smem = ((size_t)rot + (size_t)(threads / 32) * d) * sizeof(float);
  if (smem > 48 * 1024) return DLI_ERR_UNSUPPORTED;
  cudaError_t e;
  if (dtype == DLI_F32)
    e = launch_pdl((rotary_unit_store_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)q_out, (const float*)x, x_stride, positions,
                   inv_freq, slots, (float*)k_pool, (float*)v_pool, nh, nkv, d, dv, D, rot, unit_eps, page_size);
  else
    e = launch_pdl((rotary_unit_store_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)q_out,
                   (const __nv_bfloat16*)x, x_stride, positions, inv_freq, slots, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh, nkv, d, dv, D,
                   rot, unit_eps, page_size);
  return (int)e;
}

// ---------------------------------------------------------------- a product per head, for a decode step's few tokens
// out[t, h, f] = sum_i x[t, h, i] * w[h, i, f]  (float32 sums), times sigmoid(gate[t, h, f]) if a gate is given.
// x, out and gate are column slices of wider rows (row and head strides in elements); w [heads][in][features] is
// contiguous.  One block per (token, head): the token's `in` numbers wait in shared memory; a thread takes a run of
// VEC features (8 with 16-byte loads of w, else 1) and every `slices`-th row of w, so that a thread's loads are few
// and independent of one another; the slices' partial sums meet in shared memory and are added in slice order.
template <typename T, int VEC>
__global__ void heads_matvec_kernel(T* __restrict__ out, long long out_row, int out_head, const T* __restrict__ x, long long x_row, int x_head,
                                    const T* __restrict__ w, const T* __restrict__ gate, long long gate_row, int in, int features, int slices) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float hm_smem[];
  float* xs = hm_smem;        // [in]
  float* part = xs + in;      // [slices][features]
  const int t = blockIdx.x, h = blockIdx.y;
  const T* xp = x + (size_t)t * x_row + (size_t)h * x_head;
  for (int i = threadIdx.x; i < in; i += blockDim.x) xs[i] = to_float(xp[i]);
  __syncthreads();
  const T* wp = w + (size_t)h * in * features;
  const int runs = features / VEC;
  const int run = threadIdx.x % runs, slice = threadIdx.x / runs;
  if (slice < slices) {
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
#pragma unroll 4
    for (int i = slice; i < in; i += slices) {
      const float xi = xs[i];
      if (VEC == 8) {
        float wv[8];
        load8(wp + (size_t)i * features + run * 8, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = fmaf(xi, wv[k], acc[k]);
      } else {
        acc[0] = fmaf(xi, to_float(wp[(size_t)i * features + run]), acc[0]);
      }
    }
#pragma unroll
    for (int k = 0; k < VEC; ++k) part[slice * features + run * VEC + k] = acc[k];
  }
  __syncthreads();
  for (int f = threadIdx.x; f < features; f += blockDim.x) {
    float v = 0.f;
    for (int sl = 0; sl < slices; ++sl) v += part[sl * features + f];
    if (gate) v *= 1.f / (1.f + expf(-to_float(gate[(size_t)t * gate_row + (size_t)h * features + f])));
    out[(size_t)t * out_row + (size_t)h * out_head + f] = from_float<T>(v);
  }
}

template <typename T>
static int launch_heads_matvec(void* out, long long out_row, int out_head, const void* x, long long x_row, int x_head, const void* w,
                               const void* gate, long long gate_row, int n, int heads, int in, int features, cudaStream_t stream) {
  const int threads = 256;
  const bool vec = (features % 8) == 0 && features / 8 <= threads && (((uintptr_t)w) & 15) == 0;
  const int runs = vec ? features / 8 : features;
  if (!vec && runs > threads) return DLI_ERR_UNSUPPORTED;
  int slices = threads / runs;
  if (slices > in) slices = in;
  const size_t smem = (size_t)(in + slices * features) * sizeof(float);
  if (smem > 48 * 1024) return DLI_ERR_UNSUPPORTED;
  if (vec)
    return (int)launch_pdl((heads_matvec_kernel<T, 8>), dim3(n, heads), dim3(threads), smem, stream, 1, (T*)out, out_row, out_head, (const T*)x, x_row,
                           x_head, (const T*)w, (const T*)gate, gate_row, in, features, slices);
  return (int)launch_pdl((heads_matvec_kernel<T, 1>), dim3(n, heads), dim3(threads), smem, stream, 1, (T*)out, out_row, out_head, (const T*)x, x_row,
                         x_head, (const T*)w, (const T*)gate, gate_row, in, features, slices);
}

DLI_EXPORT int dli_heads_matvec(void* out, long long out_row, int out_head, const void* x, long long x_row, int x_head, const void* w,
                                const void* gate, long long gate_row, int n, int heads, int in, int features, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (heads < 1 || heads > 65535 || in < 1 || features < 1) return DLI_ERR_UNSUPPORTED;
  return dtype == DLI_F32 ? launch_heads_matvec<float>(out, out_row, out_head, x, x_row, x_head, w, gate, gate_row, n, heads, in, features, stream)
                          : launch_heads_matvec<__nv_bfloat16>(out, out_row, out_head, x, x_row, x_head, w, gate, gate_row, n, heads, in, features,
                                                               stream);
}

DLI_EXPORT int dli_sigmoid_gate(void* out, const void* gate, long long gate_stride, int n, int cols, int dtype, cudaStream_t stream) {
  if (n == 0 || cols == 0) return 0;
  const long long total = (long long)n * cols;
  cudaError_t e;
  if ((cols % 8) == 0 && (gate_stride % 8) == 0 && (((uintptr_t)out | (uintptr_t)gate) & 15) == 0) {
    const int vblocks = (int)((total / 8 + 255) / 256);
    if (dtype == DLI_F32)
      e = launch_pdl((sigmoid_gate_vec_kernel<float>), dim3(vblocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate, gate_stride, n, cols);
    else
      e = launch_pdl((sigmoid_gate_vec_kernel<__nv_bfloat16>), dim3(vblocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)gate, gate_stride, n, cols);
    return (int)e;
  }
  const int blocks = (int)((total + 255) / 256);
  if (dtype == DLI_F32)
    e = launch_pdl((sigmoid_gate_kernel<float>), dim3(blocks), dim3(256), 0, stream, 1, (float*)out, (const float*)gate, gate_stride, n, cols);
  else
    e = launch_pdl((sigmoid_gate_kernel<__nv_bfloat16>), dim3(blocks), dim3(256), 0, stream, 1, (__nv_bfloat16*)out,
                   (const __nv_bfloat16*)gate, gate_stride, n, cols);
  return (int)e;
}
