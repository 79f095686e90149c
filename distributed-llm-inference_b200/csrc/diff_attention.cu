// Differential attention over the paged cache: every query head carries two attention maps over the same values,
//
//   o = softmax(q1 K1^T s) V - lambda * softmax(q2 K2^T s) V,   o <- o / rms(o) * post,   o <- o * sigmoid(gate),
//
// with q and k normed per head and map (RMS over the map's `dim` numbers, one weight shared by all heads and maps) and
// rotated by position on their first `rot` dimensions (dimension 2i paired with 2i + 1; frequencies from a table, so any
// scaling of them is the caller's; cosine and sine times `amp`).  Causal, with a sliding window that always keeps a
// sequence's first `keep_first` tokens: position i sees j <= i when i - j < window or j < keep_first (window 0: all).
//
// Cache rows: a token's key row of one KV head is [map 1 | map 2] (2 dim numbers), its value row `vdim` numbers:
//   k_pool [pages, nkv, page_size, 2 dim],  v_pool [pages, nkv, page_size, vdim].
//
// Two kernels here, both for float32 and bfloat16 storage with float32 arithmetic:
//   * prep: norm + rotation of q (written to q_out) and of k (written to the pages with v), one block a token;
//   * attention on CUDA cores: one warp per (token, query head) walks the kept first keys and then the window in chunks
//     of 32 keys, both maps side by side with one pass over the values, and finishes with the difference, the head's
//     norm and the gate.  The order of every sum depends only on the token's own position.
#include "common.cuh"
#include <math_constants.h>

using namespace dli;

namespace {

// ---------------------------------------------------------------- prep
// proj row: q heads [nh][2][dim] from column 0; k heads [nkv][2][dim] from k_col; v [nkv][vdim] from v_col (k_col < 0: the
// layer reads another layer's keys and values and writes none).
template <typename T>
__global__ void diff_prep_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int proj_stride, int k_col, int v_col,
                                 const float* __restrict__ wq, const float* __restrict__ wk, float eps, const int* __restrict__ positions,
                                 const float* __restrict__ freq, float amp, const int* __restrict__ slots, T* __restrict__ k_pool,
                                 T* __restrict__ v_pool, int nh, int nkv, int dim, int vdim, int rot, int page_size) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const float pos = (float)positions[t];
  const T* row = proj + (size_t)t * proj_stride;
  const bool writes = k_col >= 0;
  long long kbase = 0, vbase = 0;
  if (writes) {
    const int slot = slots[t];
    const int page = slot / page_size, off = slot - page * page_size;
    kbase = ((long long)page * nkv * page_size + off) * 2 * dim;  // + g * page_size * 2 dim
    vbase = ((long long)page * nkv * page_size + off) * vdim;
  }
  const int q_units = nh * 2, k_units = writes ? nkv * 2 : 0;
  for (int u = warp; u < q_units + k_units; u += warps) {
    const bool is_q = u < q_units;
    const int unit = is_q ? u : u - q_units;
    const T* src = row + (is_q ? 0 : k_col) + (size_t)unit * dim;
    const float* w = is_q ? wq : wk;
    T* dst;
    if (is_q) {
      dst = q_out + (size_t)t * q_units * dim + (size_t)unit * dim;
    } else {
      const int g = unit >> 1, m = unit & 1;
      dst = k_pool + kbase + (long long)g * page_size * 2 * dim + m * dim;
    }
    float ss = 0.f;
    for (int e = lane; e < dim; e += 32) {
      const float v = to_float(src[e]);
      ss = fmaf(v, v, ss);
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)dim + eps);
    for (int j = lane; 2 * j < dim; j += 32) {
      const int e0 = 2 * j, e1 = e0 + 1;
      float a = to_float(src[e0]) * rstd * w[e0];
      float b = e1 < dim ? to_float(src[e1]) * rstd * w[e1] : 0.f;
      if (e1 < rot) {
        float sn, cs;
        sincosf(pos * freq[j], &sn, &cs);
        sn *= amp;
        cs *= amp;
        const float ra = a * cs - b * sn, rb = b * cs + a * sn;
        a = ra;
        b = rb;
      }
      dst[e0] = from_float<T>(a);
      if (e1 < dim) dst[e1] = from_float<T>(b);
    }
  }
  if (writes) {
    for (int i = threadIdx.x; i < nkv * vdim; i += blockDim.x) {
      const int g = i / vdim, e = i - g * vdim;
      v_pool[vbase + (long long)g * page_size * vdim + e] = row[v_col + i];
    }
  }
}

// ---------------------------------------------------------------- attention on CUDA cores
template <typename T, int R>
__global__ void diff_attention_simt_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                           const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ positions, const T* __restrict__ gate, int gate_stride, int n, int nh, int nkv,
                                           int dim, int vdim, int page_size, int window, int keep_first, float scale, float lambda, float post,
                                           float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int lane = threadIdx.x & 31;
  const int warp_in_block = threadIdx.x >> 5;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
  if (warp >= (long long)n * nh) return;
  const int t = (int)(warp / nh), h = (int)(warp % nh);
  const int kvh = h / (nh / nkv);
  const int p = positions[t];
  const int* table = block_tables + (size_t)seq_of_token[t] * max_blocks;
  float* qs = smem + warp_in_block * 2 * dim;
  for (int i = lane; i < 2 * dim; i += 32) qs[i] = to_float(q[((size_t)t * nh + h) * 2 * dim + i]);
  __syncwarp();

  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int kept = min(keep_first, lo);  // keys 0 .. kept - 1 lie in front of the window and are seen all the same
  float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, l1 = 0.f, l2 = 0.f;
  float acc1[R], acc2[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc1[r] = acc2[r] = 0.f;

  for (int seg = 0; seg < 2; ++seg) {
    const int first = seg == 0 ? 0 : lo, end = seg == 0 ? kept : p + 1;
    for (int base = first; base < end; base += 32) {
      const int key = base + lane;
      const bool valid = key < end;
      float s1 = -CUDART_INF_F, s2 = -CUDART_INF_F;
      long long vrow = 0;
      if (valid) {
        const int page = table[key / page_size];
        const long long at = ((long long)page * nkv + kvh) * page_size + key % page_size;
        const T* kr = k_pool + at * 2 * dim;
        vrow = at * vdim;
        float d1 = 0.f, d2 = 0.f;
        for (int i = 0; i < dim; ++i) {
          d1 = fmaf(qs[i], to_float(kr[i]), d1);
          d2 = fmaf(qs[dim + i], to_float(kr[dim + i]), d2);
        }
        s1 = d1 * scale;
        s2 = d2 * scale;
      }
      const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
      const float p1 = valid ? expf(s1 - n1) : 0.f, p2 = valid ? expf(s2 - n2) : 0.f;
      const float c1 = expf(m1 - n1), c2 = expf(m2 - n2);  // 0 on the first chunk
      l1 = l1 * c1 + warp_sum(p1);
      l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acc1[r] *= c1;
        acc2[r] *= c2;
      }
      const int count = min(32, end - base);
      for (int j = 0; j < count; ++j) {
        const float b1 = __shfl_sync(0xffffffffu, p1, j), b2 = __shfl_sync(0xffffffffu, p2, j);
        const T* vr = v_pool + __shfl_sync(0xffffffffu, vrow, j);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = lane + 32 * r;
          if (i < vdim) {
            const float v = to_float(vr[i]);
            acc1[r] = fmaf(b1, v, acc1[r]);
            acc2[r] = fmaf(b2, v, acc2[r]);
          }
        }
      }
      m1 = n1;
      m2 = n2;
    }
  }
  const float i1 = 1.f / l1, i2 = lambda / l2;
  float o[R];
  float ss = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    o[r] = i < vdim ? acc1[r] * i1 - acc2[r] * i2 : 0.f;
    ss = fmaf(o[r], o[r], ss);
  }
  const float g = gate != nullptr ? 1.f / (1.f + expf(-to_float(gate[(size_t)t * gate_stride + h]))) : 1.f;
  const float f = rsqrtf(warp_sum(ss) / (float)vdim + eps) * post * g;
  T* dst = out + ((size_t)t * nh + h) * vdim;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = lane + 32 * r;
    if (i < vdim) dst[i] = from_float<T>(o[r] * f);
  }
}

}  // namespace

DLI_EXPORT int dli_diff_prep(void* q_out, const void* proj, int proj_stride, int k_col, int v_col, const float* wq, const float* wk, float eps,
                             const int* positions, const float* freq, float amp, const int* slots, void* k_pool, void* v_pool, int n, int nh,
                             int nkv, int dim, int vdim, int rot, int page_size, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (rot % 2 || rot < 0 || rot > dim || nkv < 1 || nh % nkv) return DLI_ERR_UNSUPPORTED;
  const int units = 2 * nh + (k_col >= 0 ? 2 * nkv : 0);
  const int threads = 32 * (units < 8 ? units : 8);
  if (dtype == DLI_F32)
    launch_pdl((diff_prep_kernel<float>), dim3(n), dim3(threads), 0, stream, 1, (float*)q_out, (const float*)proj, proj_stride, k_col, v_col, wq,
               wk, eps, positions, freq, amp, slots, (float*)k_pool, (float*)v_pool, nh, nkv, dim, vdim, rot, page_size);
  else
    launch_pdl((diff_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), 0, stream, 1, (__nv_bfloat16*)q_out, (const __nv_bfloat16*)proj,
               proj_stride, k_col, v_col, wq, wk, eps, positions, freq, amp, slots, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh, nkv, dim,
               vdim, rot, page_size);
  return (int)cudaGetLastError();
}

DLI_EXPORT int dli_diff_attention_simt(void* out, const void* q, const void* k_pool, const void* v_pool, const int* block_tables, int max_blocks,
                                       const int* seq_of_token, const int* positions, const void* gate, int gate_stride, int n, int nh, int nkv,
                                       int dim, int vdim, int page_size, int window, int keep_first, float scale, float lambda, float post,
                                       float eps, int dtype, cudaStream_t stream) {
  if (n == 0) return 0;
  if (dim < 1 || vdim < 1 || vdim > 512 || nkv < 1 || nh % nkv) return DLI_ERR_UNSUPPORTED;
  const int warps = 4;
  const long long total = (long long)n * nh;
  const int blocks = (int)((total + warps - 1) / warps);
  const size_t smem = (size_t)warps * 2 * dim * sizeof(float);
  if (smem > 48 * 1024) return DLI_ERR_UNSUPPORTED;
#define DLI_DIFF(T, R)                                                                                                                      \
  launch_pdl((diff_attention_simt_kernel<T, R>), dim3(blocks), dim3(warps * 32), smem, stream, 1, (T*)out, (const T*)q, (const T*)k_pool,    \
             (const T*)v_pool, block_tables, max_blocks, seq_of_token, positions, (const T*)gate, gate_stride, n, nh, nkv, dim, vdim,        \
             page_size, window, keep_first, scale, lambda, post, eps)
  if (dtype == DLI_F32) {
    if (vdim <= 128) DLI_DIFF(float, 4);
    else DLI_DIFF(float, 16);
  } else {
    if (vdim <= 128) DLI_DIFF(__nv_bfloat16, 4);
    else DLI_DIFF(__nv_bfloat16, 16);
  }
#undef DLI_DIFF
  return (int)cudaGetLastError();
}
