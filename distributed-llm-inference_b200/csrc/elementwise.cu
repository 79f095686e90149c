// Embedding gather, fused residual-add + RMSNorm, rotary embedding fused with
// the write of keys and values into cache pages, and SiLU(gate) * up.
// Each kernel has a float32 and a bfloat16 instantiation; all arithmetic is float32.
#include "common.cuh"

using namespace dli;

// ---------------------------------------------------------------- embedding
// h[t, :] = float(table[ids[t], :]); h is the float32 residual stream.
template <typename T>
__global__ void embedding_kernel(float* __restrict__ h, const T* __restrict__ table, const int* __restrict__ ids, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* src = table + (size_t)ids[t] * H;
  float* dst = h + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_float(src[i]);
}

// bfloat16 rows of H % 8 == 0: 16-byte loads, two float4 stores per thread
__global__ void embedding_bf16_vec_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ table,
                                          const int* __restrict__ ids, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)ids[t] * H);
  float4* dst = reinterpret_cast<float4*>(h + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = src[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
    const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
    dst[2 * i] = make_float4(a.x, a.y, b.x, b.y);
    dst[2 * i + 1] = make_float4(c.x, c.y, d.x, d.y);
  }
}

DLI_EXPORT int dli_embedding(float* h, const void* table, const int* ids, int n, int H, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dtype == DLI_BF16 && H % 8 == 0) {
    launch_pdl((embedding_bf16_vec_kernel), dim3(n), dim3(H >= 2048 ? 256 : 64), 0, stream, 1, h, (const __nv_bfloat16*)table, ids, H);
    return (int)cudaGetLastError();
  }
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == DLI_F32)
    launch_pdl((embedding_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, h, (const float*)table, ids, H);
  else
    launch_pdl((embedding_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, h, (const __nv_bfloat16*)table, ids, H);
  return (int)cudaGetLastError();
}

// Token ids that were sampled on the device one step earlier and never travelled to the host:
// ids[i] = source[src[i]] wherever src[i] >= 0.
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ source, const int* __restrict__ src, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && src[i] >= 0) ids[i] = source[src[i]];
}

DLI_EXPORT int dli_patch_tokens(int* ids, const int* source, const int* src, int n, cudaStream_t stream) {
  if (n == 0) return 0;
  launch_pdl(patch_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, ids, source, src, n);
  return (int)cudaGetLastError();
}

// One page copied to another in every layer of a cache group (a forked request gets its own last
// page before it appends): pool [layers, pages, page_bytes]; 16-byte units.
__global__ void copy_page_kernel(uint4* __restrict__ pool, long long layer_units, long long page_units, int src, int dst) {
  pdl_launch_dependents();
  pdl_wait();
  uint4* base = pool + (size_t)blockIdx.y * layer_units;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < page_units; i += (long long)gridDim.x * blockDim.x)
    base[(size_t)dst * page_units + i] = base[(size_t)src * page_units + i];
}

DLI_EXPORT int dli_copy_page(void* pool, long long layer_bytes, long long page_bytes, int layers, int src, int dst, cudaStream_t stream) {
  if (layers == 0 || src == dst) return 0;
  if ((page_bytes % 16) || (layer_bytes % 16) || ((uintptr_t)pool % 16)) return DLI_ERR_UNSUPPORTED;
  const long long units = page_bytes / 16;
  const int blocks = (int)((units + 255) / 256 < 64 ? (units + 255) / 256 : 64);
  launch_pdl(copy_page_kernel, dim3(blocks, layers), dim3(256), 0, stream, 1, (uint4*)pool, layer_bytes / 16, units, src, dst);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- add + rmsnorm
// For output row r (source row s = rows ? rows[r] : r):
//   v = h[s] + delta[s]            (float32; written back to h[s] when rows == nullptr)
//   y[r] = v * rsqrt(mean(v^2) + eps) * w
// One block per row; the row is kept in registers between the two passes when it fits.
template <typename T, int THREADS, int PER_THREAD>
__global__ void add_rmsnorm_kernel(T* __restrict__ y, float* __restrict__ h, const T* __restrict__ delta,
                                   const float* __restrict__ w, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  const T* drow = delta ? delta + (size_t)s * H : nullptr;
  float v[PER_THREAD];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) {
    const int i = threadIdx.x + k * THREADS;
    float x = 0.f;
    if (i < H) {
      x = hrow[i];
      if (drow) x += to_float(drow[i]);
      if (!rows && drow) hrow[i] = x;
    }
    v[k] = x;
    ss += x * x;
  }
  // columns beyond THREADS * PER_THREAD (very wide models): streamed, re-read in pass two
  for (int i = threadIdx.x + PER_THREAD * THREADS; i < H; i += THREADS) {
    float x = hrow[i];
    if (drow) x += to_float(drow[i]);
    if (!rows && drow) hrow[i] = x;
    ss += x * x;
  }
  const float total = block_sum(ss, red);
  const float inv = rsqrtf(total / (float)H + eps);
  T* yrow = y + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i < H) yrow[i] = from_float<T>(v[k] * inv * w[i]);
  }
  for (int i = threadIdx.x + PER_THREAD * THREADS; i < H; i += THREADS) {
    float x = hrow[i];
    if (rows && drow) x += to_float(drow[i]);
    yrow[i] = from_float<T>(x * inv * w[i]);
  }
}

// The same for H % 8 == 0 and H <= 8 * THREADS * CHUNKS: each thread owns CHUNKS runs of 8
// columns, read and written 16 or 32 bytes at a time, and keeps them in registers between the
// sum of squares and the scaling.  The order of the additions is fixed by H and THREADS.
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_vec_kernel(T* __restrict__ y, float* __restrict__ h,
                                                                  const T* __restrict__ delta, const float* __restrict__ w,
                                                                  const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  const T* drow = delta ? delta + (size_t)s * H : nullptr;
  float v[CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < H) {
      load8(hrow + col, v[c]);
      if (drow) {
        float d[8];
        load8(drow + col, d);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] += d[k];
        if (!rows) store8(hrow + col, v[c]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[c][k] * v[c][k];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  T* yrow = y + (size_t)r * H;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < H) {
      float wv[8], o[8];
      load8(w + col, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = v[c][k] * inv * wv[k];
      store8(yrow + col, o);
    }
  }
}

template <typename T>
static int launch_add_rmsnorm_vec(void* y, float* h, const void* delta, const float* w, const int* rows, int n_rows, int H,
                                  float eps, cudaStream_t stream) {
  if (H <= 8 * 128 * 1)
    launch_pdl((add_rmsnorm_vec_kernel<T, 128, 1>), dim3(n_rows), dim3(128), 0, stream, 1, (T*)y, h, (const T*)delta, w, rows, H, eps);
  else if (H <= 8 * 256 * 1)
    launch_pdl((add_rmsnorm_vec_kernel<T, 256, 1>), dim3(n_rows), dim3(256), 0, stream, 1, (T*)y, h, (const T*)delta, w, rows, H, eps);
  else if (H <= 8 * 256 * 2)
    launch_pdl((add_rmsnorm_vec_kernel<T, 256, 2>), dim3(n_rows), dim3(256), 0, stream, 1, (T*)y, h, (const T*)delta, w, rows, H, eps);
  else
    launch_pdl((add_rmsnorm_vec_kernel<T, 512, 4>), dim3(n_rows), dim3(512), 0, stream, 1, (T*)y, h, (const T*)delta, w, rows, H, eps);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_add_rmsnorm(void* y, float* h, const void* delta, const float* w, const int* rows, int n_rows, int H,
                               float eps, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (H % 8 == 0 && H <= 8 * 512 * 4) {
    return dtype == DLI_F32 ? launch_add_rmsnorm_vec<float>(y, h, delta, w, rows, n_rows, H, eps, stream)
                            : launch_add_rmsnorm_vec<__nv_bfloat16>(y, h, delta, w, rows, n_rows, H, eps, stream);
  }
  constexpr int THREADS = 256, PER = 16;  // 4096 columns in registers, more are streamed
  if (dtype == DLI_F32)
    launch_pdl((add_rmsnorm_kernel<float, THREADS, PER>), dim3(n_rows), dim3(THREADS), 0, stream, 1, (float*)y, h, (const float*)delta, w, rows, H, eps);
  else
    launch_pdl((add_rmsnorm_kernel<__nv_bfloat16, THREADS, PER>), dim3(n_rows), dim3(THREADS), 0, stream, 1, (__nv_bfloat16*)y, h, (const __nv_bfloat16*)delta, w, rows, H, eps);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- two deltas, two norms of one stream
// v = h[s] + (a[s] + b[s]) (either delta may be absent), y1[r] = v * rsqrt(mean(v^2) + eps) * w1 and, if y2, the same
// with w2: the inputs of two branches that read one stream through norms of their own.  Without `rows` v goes back
// to h.  One block a row; float32 arithmetic, one rounding per output.
template <typename T, int THREADS, int PER_THREAD>
__global__ void add_rmsnorm_pair_kernel(T* __restrict__ y1, T* __restrict__ y2, float* __restrict__ h, const T* __restrict__ a,
                                        const T* __restrict__ b, const float* __restrict__ w1, const float* __restrict__ w2,
                                        const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  const T* arow = a ? a + (size_t)s * H : nullptr;
  const T* brow = b ? b + (size_t)s * H : nullptr;
  const bool any = arow || brow;
  auto value = [&](int i) {
    float x = hrow[i];
    if (any) x += (arow ? to_float(arow[i]) : 0.f) + (brow ? to_float(brow[i]) : 0.f);
    return x;
  };
  float v[PER_THREAD];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) {
    const int i = threadIdx.x + k * THREADS;
    v[k] = i < H ? value(i) : 0.f;
    ss += v[k] * v[k];
  }
  // columns beyond THREADS * PER_THREAD (very wide models): streamed, computed again in pass two
  for (int i = threadIdx.x + PER_THREAD * THREADS; i < H; i += THREADS) {
    const float x = value(i);
    ss += x * x;
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
  T* y1row = y1 + (size_t)r * H;
  T* y2row = y2 ? y2 + (size_t)r * H : nullptr;
#pragma unroll
  for (int k = 0; k < PER_THREAD; ++k) {
    const int i = threadIdx.x + k * THREADS;
    if (i < H) {
      if (!rows && any) hrow[i] = v[k];
      y1row[i] = from_float<T>(v[k] * inv * w1[i]);
      if (y2row) y2row[i] = from_float<T>(v[k] * inv * w2[i]);
    }
  }
  for (int i = threadIdx.x + PER_THREAD * THREADS; i < H; i += THREADS) {
    const float x = value(i);
    if (!rows && any) hrow[i] = x;
    y1row[i] = from_float<T>(x * inv * w1[i]);
    if (y2row) y2row[i] = from_float<T>(x * inv * w2[i]);
  }
}

// The same for H % 8 == 0 and H <= 8 * THREADS * CHUNKS, 16 and 32 bytes at a time, the row in registers.
template <typename T, int THREADS, int CHUNKS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_pair_vec_kernel(T* __restrict__ y1, T* __restrict__ y2, float* __restrict__ h,
                                                                       const T* __restrict__ a, const T* __restrict__ b,
                                                                       const float* __restrict__ w1, const float* __restrict__ w2,
                                                                       const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int s = rows ? rows[r] : r;
  float* hrow = h + (size_t)s * H;
  const T* arow = a ? a + (size_t)s * H : nullptr;
  const T* brow = b ? b + (size_t)s * H : nullptr;
  float v[CHUNKS][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < H) {
      load8(hrow + col, v[c]);
      if (arow || brow) {
        float d[8], e[8];
        if (arow) load8(arow + col, d);
        if (brow) load8(brow + col, e);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[c][k] += (arow ? d[k] : 0.f) + (brow ? e[k] : 0.f);
        if (!rows) store8(hrow + col, v[c]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[c][k] * v[c][k];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int col = (threadIdx.x + c * THREADS) * 8;
    if (col < H) {
      float wv[8], o[8];
      load8(w1 + col, wv);
#pragma unroll
      for (int k = 0; k < 8; ++k) o[k] = v[c][k] * inv * wv[k];
      store8(y1 + (size_t)r * H + col, o);
      if (y2) {
        load8(w2 + col, wv);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = v[c][k] * inv * wv[k];
        store8(y2 + (size_t)r * H + col, o);
      }
    }
  }
}

template <typename T>
static int launch_add_rmsnorm_pair(void* y1, void* y2, float* h, const void* a, const void* b, const float* w1, const float* w2,
                                   const int* rows, int n_rows, int H, float eps, cudaStream_t stream) {
#define DLI_PAIR_VEC(THREADS, CHUNKS)                                                                                              \
  return (int)launch_pdl((add_rmsnorm_pair_vec_kernel<T, THREADS, CHUNKS>), dim3(n_rows), dim3(THREADS), 0, stream, 1, (T*)y1, (T*)y2, h, \
                         (const T*)a, (const T*)b, w1, w2, rows, H, eps)
  const bool aligned = (((uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)h | (uintptr_t)a | (uintptr_t)b | (uintptr_t)w1 | (uintptr_t)w2) & 15) == 0;
  if (H % 8 == 0 && H <= 8 * 512 * 4 && aligned) {
    if (H <= 8 * 128) DLI_PAIR_VEC(128, 1);
    if (H <= 8 * 256) DLI_PAIR_VEC(256, 1);
    if (H <= 8 * 256 * 2) DLI_PAIR_VEC(256, 2);
    DLI_PAIR_VEC(512, 4);
  }
#undef DLI_PAIR_VEC
  return (int)launch_pdl((add_rmsnorm_pair_kernel<T, 256, 16>), dim3(n_rows), dim3(256), 0, stream, 1, (T*)y1, (T*)y2, h, (const T*)a,
                         (const T*)b, w1, w2, rows, H, eps);
}

DLI_EXPORT int dli_add_rmsnorm_pair(void* y1, void* y2, float* h, const void* a, const void* b, const float* w1, const float* w2,
                                    const int* rows, int n_rows, int H, float eps, int dtype, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  if (!y1 || !w1 || (y2 && !w2) || H < 1) return DLI_ERR_UNSUPPORTED;
  return dtype == DLI_F32 ? launch_add_rmsnorm_pair<float>(y1, y2, h, a, b, w1, w2, rows, n_rows, H, eps, stream)
                          : launch_add_rmsnorm_pair<__nv_bfloat16>(y1, y2, h, a, b, w1, w2, rows, n_rows, H, eps, stream);
}

// ---------------------------------------------------------------- logits: a factor, then a soft cap
// x <- x * scale; if cap > 0, x <- cap * tanh(x / cap).  float32, in place.
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t total, float scale, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const float v = x[i] * scale;
    x[i] = cap > 0.f ? cap * tanhf(v * inv_cap) : v;
  }
}

DLI_EXPORT int dli_scale_softcap(float* x, long long total, float scale, float cap, cudaStream_t stream) {
  if (total <= 0) return 0;
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  const long long most = (long long)sm_count() * 16;
  return (int)launch_pdl(scale_softcap_kernel, dim3((unsigned)(blocks < most ? blocks : most)), dim3(threads), 0, stream, 1, x, (size_t)total,
                         scale, cap);
}

// ---------------------------------------------------------------- rotary + cache write
// qkv: [n, (nh + 2 nkv) * d], rows = tokens.  Query heads are rotated in place; key heads are
// rotated and written to the key pool, value heads are copied to the value pool, at the token's
// slot (page * page_size + offset; a negative slot writes nothing).  Pool layout of one layer:
// [page][kv_head][page_size][d].  Rotation pairs element i with i + rot/2 for i < rot/2
// (rotate-half); elements >= rot pass through.  Angle = float(position) * inv_freq[i], float32.
template <typename T>
__global__ void rotary_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                    const int* __restrict__ slots, T* __restrict__ k_pool, T* __restrict__ v_pool, int nh,
                                    int nkv, int d, int rot, int page_size, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float trig[];  // cos[half], sin[half] of this token's angles
  const int t = blockIdx.x;
  const int half = rot >> 1;
  const int row = (nh + 2 * nkv) * d;
  T* base = qkv + (size_t)t * row;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &trig[half + i], &trig[i]);
  __syncthreads();
  const int slot = slots ? slots[t] : -1;
  const bool store = write_kv && slot >= 0;
  const int page = store ? slot / page_size : 0, off = store ? slot % page_size : 0;

  // rotated halves of q and k heads: one thread per (head, i < half)
  const int rot_items = (nh + nkv) * half;
  for (int idx = threadIdx.x; idx < rot_items; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    const float cs = trig[i], sn = trig[half + i];
    T* x = base + (size_t)head * d;
    const float a = to_float(x[i]), b = to_float(x[i + half]);
    const T ra = from_float<T>(a * cs - b * sn);
    const T rb = from_float<T>(b * cs + a * sn);
    if (head < nh) {
      x[i] = ra;
      x[i + half] = rb;
    } else if (store) {
      T* dst = k_pool + (((size_t)page * nkv + (head - nh)) * page_size + off) * d;
      dst[i] = ra;
      dst[i + half] = rb;
    }
  }
  if (!store) return;
  // pass-through part of keys (elements >= rot) and all of the values
  const int tail = d - rot;
  for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
    const int head = idx / tail, i = rot + idx - head * tail;
    k_pool[(((size_t)page * nkv + head) * page_size + off) * d + i] = base[(size_t)(nh + head) * d + i];
  }
  for (int idx = threadIdx.x; idx < nkv * d; idx += blockDim.x) {
    const int head = idx / d, i = idx - head * d;
    v_pool[(((size_t)page * nkv + head) * page_size + off) * d + i] = base[(size_t)(nh + nkv + head) * d + i];
  }
}

// cos | sin of every token's angles, [n, rot] float32 (cos in the first rot / 2 columns): computed once
// per step and read by every layer's rotary kernel, instead of once per layer.
__global__ void rotary_table_kernel(float* __restrict__ table, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                    int n, int half) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n * half) return;
  const int t = idx / half, i = idx - t * half;
  float sn, cs;
  sincosf((float)positions[t] * inv_freq[i], &sn, &cs);
  table[(size_t)t * 2 * half + i] = cs;
  table[(size_t)t * 2 * half + half + i] = sn;
}

DLI_EXPORT int dli_rotary_table(float* table, const int* positions, const float* inv_freq, int n, int rot, cudaStream_t stream) {
  if (n == 0 || rot == 0) return 0;
  if (rot & 1) return DLI_ERR_UNSUPPORTED;
  const int total = n * (rot >> 1);
  launch_pdl((rotary_table_kernel), dim3((total + 255) / 256), dim3(256), 0, stream, 1, table, positions, inv_freq, n, rot >> 1);
  return (int)cudaGetLastError();
}

// bfloat16 with rot % 16 == 0 and d % 8 == 0: every access is 16 bytes.  Work items of a token:
// (head of q or k, run of eight rotated pairs), (kv head, run of eight pass-through elements),
// (kv head, run of eight value elements).
__global__ void rotary_store_bf16_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                             const float* __restrict__ inv_freq, const float* __restrict__ table,
                                             const int* __restrict__ slots,
                                             __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool, int nh, int nkv,
                                             int d, int rot, int page_size, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float trig[];
  const int t = blockIdx.x;
  const int half = rot >> 1;
  __nv_bfloat16* base = qkv + (size_t)t * (nh + 2 * nkv) * d;
  // with a table of the step's cosines and sines every thread reads its eight of each straight from it (one
  // round of loads, no barrier); without one the block computes the token's into shared memory first
  const float* trig_row = table ? table + (size_t)t * rot : trig;
  if (!table) {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &trig[half + i], &trig[i]);
    __syncthreads();
  }
  const int slot = slots ? slots[t] : -1;
  const bool store = write_kv && slot >= 0;
  const int page = store ? slot / page_size : 0, off = store ? slot % page_size : 0;
  const int hc = half >> 3;                 // runs of eight pairs per head
  const int rot_items = (nh + nkv) * hc;
  const int tail_items = store ? nkv * ((d - rot) >> 3) : 0;
  const int v_items = store ? nkv * (d >> 3) : 0;
  for (int idx = threadIdx.x; idx < rot_items + tail_items + v_items; idx += blockDim.x) {
    if (idx < rot_items) {
      const int head = idx / hc, i = (idx - head * hc) << 3;
      __nv_bfloat16* x = base + (size_t)head * d;
      float a[8], b[8], cs8[8], sn8[8];
      load8(x + i, a);
      load8(x + i + half, b);
      *reinterpret_cast<float4*>(cs8) = *reinterpret_cast<const float4*>(trig_row + i);
      *reinterpret_cast<float4*>(cs8 + 4) = *reinterpret_cast<const float4*>(trig_row + i + 4);
      *reinterpret_cast<float4*>(sn8) = *reinterpret_cast<const float4*>(trig_row + half + i);
      *reinterpret_cast<float4*>(sn8 + 4) = *reinterpret_cast<const float4*>(trig_row + half + i + 4);
      float ra[8], rb[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float cs = cs8[k], sn = sn8[k];
        ra[k] = a[k] * cs - b[k] * sn;
        rb[k] = b[k] * cs + a[k] * sn;
      }
      if (head < nh) {
        store8(x + i, ra);
        store8(x + i + half, rb);
      } else if (store) {
        __nv_bfloat16* dst = k_pool + (((size_t)page * nkv + (head - nh)) * page_size + off) * d;
        store8(dst + i, ra);
        store8(dst + i + half, rb);
      }
    } else if (idx < rot_items + tail_items) {
      const int per = (d - rot) >> 3;
      const int j = idx - rot_items, head = j / per, i = rot + ((j - head * per) << 3);
      *reinterpret_cast<uint4*>(k_pool + (((size_t)page * nkv + head) * page_size + off) * d + i) =
          *reinterpret_cast<const uint4*>(base + (size_t)(nh + head) * d + i);
    } else {
      const int per = d >> 3;
      const int j = idx - rot_items - tail_items, head = j / per, i = (j - head * per) << 3;
      *reinterpret_cast<uint4*>(v_pool + (((size_t)page * nkv + head) * page_size + off) * d + i) =
          *reinterpret_cast<const uint4*>(base + (size_t)(nh + nkv + head) * d + i);
    }
  }
}

DLI_EXPORT int dli_rotary_store(void* qkv, const int* positions, const float* inv_freq, const float* table, const int* slots,
                                void* k_pool, void* v_pool, int n, int nh, int nkv, int d, int rot, int page_size, int write_kv,
                                int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (rot < 0 || rot > d || (rot & 1)) return DLI_ERR_UNSUPPORTED;
  if (rot > 0 && inv_freq == nullptr) return DLI_ERR_UNSUPPORTED;
  const int threads = 256;
  const size_t smem = (size_t)rot * sizeof(float);
  if (dtype == DLI_BF16 && rot % 16 == 0 && d % 8 == 0) {
    launch_pdl((rotary_store_bf16_vec_kernel), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)qkv, positions, inv_freq, table, slots,
               (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh, nkv, d, rot, page_size, write_kv);
    return (int)cudaGetLastError();
  }
  if (dtype == DLI_F32)
    launch_pdl((rotary_store_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)qkv, positions, inv_freq, slots, (float*)k_pool,
                                                          (float*)v_pool, nh, nkv, d, rot, page_size, write_kv);
  else
    launch_pdl((rotary_store_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)qkv, positions, inv_freq, slots,
                                                                  (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh, nkv, d,
                                                                  rot, page_size, write_kv);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- silu(gate) * up
// gu: [n, 2 I]; out: [n, I].  Plain layout: gate in columns [0, I), up in [I, 2 I).  Tiled layout
// (the one the decode matrix product's fused epilogue wants of the weights): blocks of 128 columns,
// gate features 64 j .. 64 j + 63 in columns 128 j .., their up features in columns 128 j + 64 ...
__device__ __forceinline__ void gate_up_columns(int i, int I, int tiled, int& g, int& u) {
  if (tiled) {
    g = (i >> 6) * 128 + (i & 63);
    u = g + 64;
  } else {
    g = i;
    u = I + i;
  }
}

// what a gated feed-forward applies to its gate: 0 silu, 1 gelu with the tanh approximation, 2 g * sigmoid(1.702 g)
__device__ __forceinline__ float glu_activation(float g, int act) {
  if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  if (act == 2) return g / (1.f + expf(-1.702f * g));
  return g / (1.f + expf(-g));
}
// act(min(g, limit)) * (clamp(u, -limit, limit) + shift); limit <= 0: no bounds
__device__ __forceinline__ float glu_value(float g, float u, int act, float limit, float shift) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  return glu_activation(g, act) * (u + shift);
}

template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int n, int I, int tiled, int act, float limit, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n * I;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    int gc, uc;
    gate_up_columns(i, I, tiled, gc, uc);
    const float g = to_float(gu[t * 2 * I + gc]);
    const float u = to_float(gu[t * 2 * I + uc]);
    out[idx] = from_float<T>(glu_value(g, u, act, limit, shift));
  }
}

// bfloat16, I % 8 == 0: one 16-byte load of gate and of up, one 16-byte store, per thread
__global__ void silu_mul_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu, int I, int tiled, int act,
                                         float limit, float shift) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= I / 8) return;
  int gc, uc;
  gate_up_columns(i * 8, I, tiled, gc, uc);  // eight columns never cross a block of 64
  const uint4 g = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + gc);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * I + uc);
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 r;
  __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 a = __bfloat1622float2(gp[k]), b = __bfloat1622float2(up[k]);
    rp[k] = __floats2bfloat162_rn(glu_value(a.x, b.x, act, limit, shift), glu_value(a.y, b.y, act, limit, shift));
  }
  reinterpret_cast<uint4*>(out + (size_t)t * I)[i] = r;
}

DLI_EXPORT int dli_silu_mul(void* out, const void* gu, int n, int I, int tiled, int act, float limit, float shift, int dtype,
                            cudaStream_t stream) {
  if ((tiled && (I % 64)) || act < 0 || act > 2) return DLI_ERR_UNSUPPORTED;
  if (n == 0) return 0;
  if (dtype == DLI_BF16 && I % 8 == 0 && n <= 65535) {
    dim3 grid((I / 8 + 255) / 256, n);
    launch_pdl((silu_mul_bf16_vec_kernel), dim3(grid), dim3(256), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, I, tiled, act, limit, shift);
    return (int)cudaGetLastError();
  }
  const size_t total = (size_t)n * I;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < (size_t)sm_count() * 16 ? (total + threads - 1) / threads : (size_t)sm_count() * 16);
  if (dtype == DLI_F32)
    launch_pdl((silu_mul_kernel<float>), dim3(blocks), dim3(threads), 0, stream, 1, (float*)out, (const float*)gu, n, I, tiled, act, limit, shift);
  else
    launch_pdl((silu_mul_kernel<__nv_bfloat16>), dim3(blocks), dim3(threads), 0, stream, 1, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, n, I, tiled, act, limit, shift);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- activation of a plain (ungated) feed-forward
// x <- act(x) in place; kinds: 0 relu(x)^2, 1 gelu with the tanh approximation, 2 silu, 3 tanh.
#define DLI_ACT_RELU2 0
#define DLI_ACT_GELU_TANH 1
#define DLI_ACT_SILU 2
#define DLI_ACT_TANH 3

__device__ __forceinline__ float apply_activation(float z, int kind) {
  if (kind == DLI_ACT_RELU2) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  if (kind == DLI_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (kind == DLI_ACT_TANH) return tanhf(z);
  return z / (1.f + expf(-z));
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ x, size_t total, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    x[i] = from_float<T>(apply_activation(to_float(x[i]), kind));
}

// bfloat16, total % 8 == 0: 16 bytes a thread
__global__ void activation_bf16_vec_kernel(__nv_bfloat16* __restrict__ x, size_t units, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < units; i += (size_t)gridDim.x * blockDim.x) {
    float v[8];
    load8(x + i * 8, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = apply_activation(v[k], kind);
    store8(x + i * 8, v);
  }
}

DLI_EXPORT int dli_activation(void* x, long long total, int kind, int dtype, cudaStream_t stream) {
  if (total == 0) return 0;
  if (kind < 0 || kind > 3) return DLI_ERR_UNSUPPORTED;
  const int threads = 256;
  const size_t cap = (size_t)sm_count() * 16;
  if (dtype == DLI_BF16 && total % 8 == 0 && ((uintptr_t)x % 16) == 0) {
    const size_t units = (size_t)total / 8;
    const size_t blocks = (units + threads - 1) / threads;
    launch_pdl((activation_bf16_vec_kernel), dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(threads), 0, stream, 1, (__nv_bfloat16*)x, units, kind);
    return (int)cudaGetLastError();
  }
  const size_t blocks = ((size_t)total + threads - 1) / threads;
  const dim3 grid((unsigned)(blocks < cap ? blocks : cap));
  if (dtype == DLI_F32)
    launch_pdl((activation_kernel<float>), grid, dim3(threads), 0, stream, 1, (float*)x, (size_t)total, kind);
  else
    launch_pdl((activation_kernel<__nv_bfloat16>), grid, dim3(threads), 0, stream, 1, (__nv_bfloat16*)x, (size_t)total, kind);
  return (int)cudaGetLastError();
}
