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
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const __nv_bfloat16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store2(__nv_bfloat16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

// pairs != 0: every size and column is even, dim <= 256 and the pointers allow it, so a lane reads the two numbers that
// rotate together at once and keeps them from the norm's sum to the rotation.
template <typename T>
__global__ void diff_prep_kernel(T* __restrict__ q_out, const T* __restrict__ proj, int proj_stride, int k_col, int v_col,
                                 const float* __restrict__ wq, const float* __restrict__ wk, float eps, const int* __restrict__ positions,
                                 const float* __restrict__ freq, float amp, const int* __restrict__ slots, T* __restrict__ k_pool,
                                 T* __restrict__ v_pool, int nh, int nkv, int dim, int vdim, int rot, int page_size, int pairs) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float trig[];  // the token's cosines [rot / 2] and sines [rot / 2] times amp, shared by all heads and maps
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; 2 * j < rot; j += blockDim.x) {
    float sn, cs;
    sincosf(pos * freq[j], &sn, &cs);
    trig[j] = cs * amp;
    trig[rot / 2 + j] = sn * amp;
  }
  bool trig_ready = false;  // every warp has at least one unit: it meets the others behind its first unit's loads
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
    if (pairs) {
      float2 x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = lane + 32 * i;
        if (2 * j < dim) {
          x[i] = load2(src + 2 * j);
          ss = fmaf(x[i].x, x[i].x, fmaf(x[i].y, x[i].y, ss));
        }
      }
      const float rstd = rsqrtf(warp_sum(ss) / (float)dim + eps);
      if (!trig_ready) {
        __syncthreads();
        trig_ready = true;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = lane + 32 * i;
        if (2 * j < dim) {
          const float2 w2 = load2(w + 2 * j);
          float a = x[i].x * rstd * w2.x, b = x[i].y * rstd * w2.y;
          if (2 * j + 1 < rot) {
            const float cs = trig[j], sn = trig[rot / 2 + j];
            const float ra = a * cs - b * sn, rb = b * cs + a * sn;
            a = ra;
            b = rb;
          }
          store2(dst + 2 * j, make_float2(a, b));
        }
      }
      continue;
    }
    for (int e = lane; e < dim; e += 32) {
      const float v = to_float(src[e]);
      ss = fmaf(v, v, ss);
    }
    const float rstd = rsqrtf(warp_sum(ss) / (float)dim + eps);
    if (!trig_ready) {
      __syncthreads();
      trig_ready = true;
    }
    for (int j = lane; 2 * j < dim; j += 32) {
      const int e0 = 2 * j, e1 = e0 + 1;
      float a = to_float(src[e0]) * rstd * w[e0];
      float b = e1 < dim ? to_float(src[e1]) * rstd * w[e1] : 0.f;
      if (e1 < rot) {
        const float cs = trig[j], sn = trig[rot / 2 + j];
        const float ra = a * cs - b * sn, rb = b * cs + a * sn;
        a = ra;
        b = rb;
      }
      dst[e0] = from_float<T>(a);
      if (e1 < dim) dst[e1] = from_float<T>(b);
    }
  }
  if (writes && pairs) {
    for (int i = 2 * threadIdx.x; i < nkv * vdim; i += 2 * blockDim.x) {
      const int g = i / vdim, e = i - g * vdim;
      store2(v_pool + vbase + (long long)g * page_size * vdim + e, load2(row + v_col + i));  // float32 both ways, or bfloat16 unchanged
    }
  } else if (writes) {
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
  const size_t smem = (size_t)rot * sizeof(float);
  if (smem > 48 * 1024) return DLI_ERR_UNSUPPORTED;
  const uintptr_t ptrs = (uintptr_t)q_out | (uintptr_t)proj | (uintptr_t)wq | (uintptr_t)wk | (uintptr_t)k_pool | (uintptr_t)v_pool;
  const int pairs = dim % 2 == 0 && dim <= 256 && vdim % 2 == 0 && proj_stride % 2 == 0 && (k_col < 0 || (k_col % 2 == 0 && v_col % 2 == 0)) && ptrs % 8 == 0;
  if (dtype == DLI_F32)
    launch_pdl((diff_prep_kernel<float>), dim3(n), dim3(threads), smem, stream, 1, (float*)q_out, (const float*)proj, proj_stride, k_col, v_col, wq,
               wk, eps, positions, freq, amp, slots, (float*)k_pool, (float*)v_pool, nh, nkv, dim, vdim, rot, page_size, pairs);
  else
    launch_pdl((diff_prep_kernel<__nv_bfloat16>), dim3(n), dim3(threads), smem, stream, 1, (__nv_bfloat16*)q_out, (const __nv_bfloat16*)proj,
               proj_stride, k_col, v_col, wq, wk, eps, positions, freq, amp, slots, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh, nkv, dim,
               vdim, rot, page_size, pairs);
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

// ---------------------------------------------------------------- attention on tensor cores (bfloat16)
// Compiled only with -DDIFF_DK=<dim> -DDIFF_DV=<vdim> (multiples of 16): one library per pair of sizes.
//
//   * a CTA owns a tile of up to 64 rows, a row being one (token, query head) pair, all of one KV head; warps 0-3 run
//     map 1 of these rows, warps 4-7 map 2, on the SAME key and value tiles in shared memory: a key row of the cache holds
//     both maps side by side, and the values are shared, so each is fetched once;
//   * the four warps of a map divide the tile between them by rows and keys: 4 x 16 rows with all 64 keys of a key tile
//     each, or, when the CTA has no more than 32 (16) rows — a short portion, a single decoded token with its KV group's
//     heads —, 2 (1) x 16 rows with 32 (16) keys each, so that no warp idles while a single token walks a long window;
//   * 64 keys a tile, copied in place from the pages by cp.async through the block table, double buffered; first the tiles of
//     the kept first tokens that lie in front of the window, then the window's;
//   * scores, running maximum, sums and outputs in float32 (online softmax), probabilities rounded to bfloat16 only as the
//     operand of the P V product (mma.sync m16n8k16); a key tile that every row of the warp sees whole skips the mask, and
//     the running output is rescaled only when some row's maximum has grown;
//   * at the end every warp leaves its unnormalised output, maximum and sum in shared memory; a warp per row then merges the
//     key ranges of each map, takes the difference, norms the head, applies the gate and stores whole rows.
//   A sequence that brings one token is a tile of its KV group's heads; prompt portions and single tokens share the launch.
#if defined(DIFF_DK) && defined(DIFF_DV)

namespace tc {

typedef __nv_bfloat16 bf16;
constexpr int DK = DIFF_DK, DV = DIFF_DV;
static_assert(DK % 16 == 0 && DV % 16 == 0 && DK >= 16 && DV >= 16 && DK <= 256 && DV <= 256, "sizes must be multiples of 16 up to 256");
constexpr int BLOCK_M = 64, BLOCK_N = 64, THREADS = 256, WARPS = THREADS / 32;
constexpr int KROW = 2 * DK * 2 + 16;  // bytes of a padded shared-memory row of queries or keys (both maps)
constexpr int VROW = DV * 2 + 16;
constexpr int KTILE = BLOCK_N * KROW, VTILE = BLOCK_N * VROW;
constexpr int KCHUNKS = 2 * DK / 8, VCHUNKS = DV / 8;  // 16-byte chunks of a row
constexpr int STAGE_BYTES = 2 * (KTILE + VTILE);
constexpr int PROW = DV + (DV % 32 == 0 ? 8 : 24);  // floats of a row of partial results: DV outputs, maximum, sum; 8 mod 32 keeps the float2 stores apart
constexpr int COMBINE_BYTES = WARPS * 16 * PROW * 4;
constexpr int SMEM_BYTES = BLOCK_M * KROW + (STAGE_BYTES > COMBINE_BYTES ? STAGE_BYTES : COMBINE_BYTES);
constexpr int MIN_CTAS = (DK <= 128 && DV <= 128 && 2 * SMEM_BYTES + 2048 <= 227 * 1024) ? 2 : 1;  // two CTAs an SM where 128 registers a thread suffice

struct Params {
  bf16* out;           // [n, nh * DV]
  const bf16* q;       // [n, nh * 2 * DK]
  const bf16* k_pool;  // [pages, nkv, page_size, 2 DK]
  const bf16* v_pool;  // [pages, nkv, page_size, DV]
  const int* block_tables;
  int max_blocks;
  const int* q_start;
  const int* kv_len;
  const bf16* gate;
  int gate_stride;
  int nh, nkv, page_size, window, keep_first;
  int tokens_per_tile, heads_per_chunk, head_chunks;
  float scale_log2, lambda, post, eps;
  int splits;      // > 1: single tokens only, the key tiles of each divided between `splits` CTAs, partial results in scratch
  float* scratch;  // [rows of (sequence, head)][splits][2 maps][DV + 2]
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// What a CTA knows of its tile.
struct Tile {
  int pos0, rows_used, Gc, nheads, hi, lo, kept, kept_tiles, first_tile, num_tiles, kvh;
  int it0, it1;  // the CTA's share of the key tiles (all of them unless single tokens' keys are split between CTAs)
  const int* table;
};

// The walk over the key tiles with the map's four warps arranged as (4 / KS) row tiles x KS key ranges.  Leaves every active
// warp's unnormalised output, maximum and sum in `part` (which overlays the key and value stages).
template <int KS>
__device__ __forceinline__ void walk(const Params& p, const Tile& T, unsigned char* sQ, unsigned char* sK, unsigned char* sV, float* part) {
  constexpr int NKEYS = BLOCK_N / KS;  // keys of a tile that one warp takes
  constexpr int NJ = NKEYS / 8, NKK = NKEYS / 16;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int map = warp >> 2, w4 = warp & 3;
  const int wrow = (w4 / KS) * 16, koff = (w4 % KS) * NKEYS;
  const bool warp_active = wrow < T.rows_used;
  const int Gc = T.Gc;

  auto tile_index = [&](int it) { return it < T.kept_tiles ? it : T.first_tile + (it - T.kept_tiles); };
  // Four threads a key row.  The row's page is looked up one tile ahead of its copies (locate), so that the block table's
  // answer has arrived when the copies are issued: page < 0 is a row that no query of the tile sees (zeros, nothing read).
  const int lrow = tid >> 2;
  auto locate = [&](int it) -> int {
    if (it >= T.it1) return -1;
    const int key = tile_index(it) * BLOCK_N + lrow;
    const bool ok = key < T.hi && (key >= T.lo || key < T.kept);
    return ok ? T.table[key / p.page_size] : -1;
  };
  auto load_tile = [&](int stage, int it, int page) {
    const int key = tile_index(it) * BLOCK_N + lrow;
    const bool ok = page >= 0;
    const size_t at = ok ? ((size_t)page * p.nkv + T.kvh) * p.page_size + key % p.page_size : 0;
    const bf16* gK = p.k_pool + at * 2 * DK;
    const bf16* gV = p.v_pool + at * DV;
    const uint32_t dK = smem_u32(sK + stage * KTILE + lrow * KROW), dV = smem_u32(sV + stage * VTILE + lrow * VROW);
    const int bytes = ok ? 16 : 0;
#pragma unroll
    for (int i = 0; i < (KCHUNKS + VCHUNKS + 3) / 4; ++i) {
      const int c = (tid & 3) + 4 * i;
      if (c < KCHUNKS) cp_async16(dK + c * 16, gK + c * 8, bytes);
      else if (c < KCHUNKS + VCHUNKS) cp_async16(dV + (c - KCHUNKS) * 16, gV + (c - KCHUNKS) * 8, bytes);
    }
  };

  const int r0 = wrow + (lane >> 2), r1 = r0 + 8;
  int rpos[2];
  bool rvalid[2];
  {
    const int t0 = r0 / Gc, t1 = r1 / Gc;
    rvalid[0] = r0 < T.rows_used && (r0 - t0 * Gc) < T.nheads;
    rvalid[1] = r1 < T.rows_used && (r1 - t1 * Gc) < T.nheads;
    rpos[0] = T.pos0 + t0;
    rpos[1] = T.pos0 + t1;
  }
  // positions of the warp's first and last token: a key range at or below the first and inside the last one's window is seen whole
  const int pos_min = T.pos0 + wrow / Gc, pos_max = T.pos0 + min(wrow + 15, T.rows_used - 1) / Gc;
  float m[2] = {-CUDART_INF_F, -CUDART_INF_F}, l[2] = {0.f, 0.f};
  float o[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  if (T.it0 < T.it1) load_tile(0, T.it0, locate(T.it0));
  cp_async_commit();
  int page_next = locate(T.it0 + 1);
  for (int it = T.it0; it < T.it1; ++it) {
    const int stage = (it - T.it0) & 1;
    if (it + 1 < T.it1) load_tile(stage ^ 1, it + 1, page_next);
    cp_async_commit();
    page_next = locate(it + 2);
    cp_async_wait<1>();
    __syncthreads();
    if (warp_active) {
      const unsigned char* wQ = sQ + wrow * KROW + map * DK * 2;
      const unsigned char* tK = sK + stage * KTILE + koff * KROW + map * DK * 2;
      const unsigned char* tV = sV + stage * VTILE + koff * VROW;
      const int base = tile_index(it) * BLOCK_N + koff;
      float sc[NJ][4];
#pragma unroll
      for (int j = 0; j < NJ; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK / 16; ++kk) {
        uint32_t a[4];
        ldsm4(a, smem_u32(wQ + (lane & 15) * KROW + (kk * 16 + (lane >> 4) * 8) * 2));
#pragma unroll
        for (int jp = 0; jp < NKK; ++jp) {
          uint32_t b[4];
          const int key = jp * 16 + (lane & 7) + (lane >> 4) * 8;
          const int dim = kk * 16 + ((lane >> 3) & 1) * 8;
          ldsm4(b, smem_u32(tK + key * KROW + dim * 2));
          mma16816(sc[2 * jp], a, b[0], b[1]);
          mma16816(sc[2 * jp + 1], a, b[2], b[3]);
        }
      }
      float tmax[2] = {-CUDART_INF_F, -CUDART_INF_F};
      const bool whole = base + NKEYS - 1 <= pos_min && (p.window <= 0 || base > pos_max - p.window || base + NKEYS <= p.keep_first);
      if (whole) {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            sc[j][e] *= p.scale_log2;
            tmax[e >> 1] = fmaxf(tmax[e >> 1], sc[j][e]);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int rr = e >> 1;
            const int key = base + j * 8 + (lane & 3) * 2 + (e & 1);
            bool ok = rvalid[rr] && key <= rpos[rr];
            if (p.window > 0) ok = ok && (key > rpos[rr] - p.window || key < p.keep_first);
            const float t = ok ? sc[j][e] * p.scale_log2 : -CUDART_INF_F;
            sc[j][e] = t;
            tmax[rr] = fmaxf(tmax[rr], t);
          }
        }
      }
      float corr[2], msafe[2];
      bool grew = false;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 1));
        tmax[rr] = fmaxf(tmax[rr], __shfl_xor_sync(0xffffffffu, tmax[rr], 2));
        const float mnew = fmaxf(m[rr], tmax[rr]);
        grew = grew || mnew > m[rr];
        msafe[rr] = (mnew == -CUDART_INF_F) ? 0.f : mnew;
        corr[rr] = exp2f(m[rr] - msafe[rr]);
        m[rr] = mnew;
      }
      if (__any_sync(0xffffffffu, grew)) {  // else both factors are 1 in every lane
        l[0] *= corr[0];
        l[1] *= corr[1];
#pragma unroll
        for (int j = 0; j < DV / 8; ++j) {
          o[j][0] *= corr[0]; o[j][1] *= corr[0];
          o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
      }
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(sc[j][e] - msafe[e >> 1]);
          sc[j][e] = pv;
          l[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int kk = 0; kk < NKK; ++kk) {
        uint32_t a[4];
        a[0] = pack2(sc[2 * kk][0], sc[2 * kk][1]);
        a[1] = pack2(sc[2 * kk][2], sc[2 * kk][3]);
        a[2] = pack2(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        a[3] = pack2(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int jp = 0; jp < DV / 16; ++jp) {
          uint32_t b[4];
          const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          const int dim = jp * 16 + (lane >> 4) * 8;
          ldsm4t(b, smem_u32(tV + key * VROW + dim * 2));
          mma16816(o[2 * jp], a, b[0], b[1]);
          mma16816(o[2 * jp + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();  // the stage is overwritten by the copies issued next iteration
  }
  cp_async_wait<0>();
  __syncthreads();  // the stages are free: the partial results go where they were

  if (warp_active) {
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
      l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
      float* dst = part + ((size_t)warp * 16 + (lane >> 2) + 8 * rr) * PROW;
#pragma unroll
      for (int j = 0; j < DV / 8; ++j) *reinterpret_cast<float2*>(dst + j * 8 + (lane & 3) * 2) = make_float2(o[j][2 * rr], o[j][2 * rr + 1]);
      if ((lane & 3) == 0) {
        dst[DV] = m[rr];
        dst[DV + 1] = l[rr];
      }
    }
  }
}

constexpr int NC = (DV + 63) / 64;  // pairs of outputs a lane holds when a warp holds a row
constexpr int SROW = DV + 2;         // floats of one map's partial result in the scratch of split keys: outputs, maximum, sum

// A warp merges `count` partial results of one row and map, `stride` floats apart, each DV unnormalised outputs followed by
// its maximum (in units of log2) and its sum: the merged outputs (still unnormalised), their maximum and sum.
// MANY: the partial results are many and far (the scratch of split keys): maxima and sums are read a partial result a
// lane, so that their loads are in flight together; else (a CTA's own few, in shared memory) every lane reads them all.
template <bool MANY>
__device__ __forceinline__ void merge_partials(const float* src, size_t stride, int count, int lane, float (&val)[NC][2], float& mx, float& sum) {
  if (MANY) {
    float m_lane = -CUDART_INF_F;
    for (int i = lane; i < count; i += 32) m_lane = fmaxf(m_lane, src[i * stride + DV]);
    mx = warp_max(m_lane);
    float s_lane = 0.f;
    for (int i = lane; i < count; i += 32) {
      const float mi = src[i * stride + DV];
      s_lane = fmaf(mi == -CUDART_INF_F ? 0.f : exp2f(mi - mx), src[i * stride + DV + 1], s_lane);
    }
    sum = warp_sum(s_lane);
  } else {
    mx = -CUDART_INF_F;
    for (int i = 0; i < count; ++i) mx = fmaxf(mx, src[i * stride + DV]);
    sum = 0.f;
    for (int i = 0; i < count; ++i) {
      const float mi = src[i * stride + DV];
      sum = fmaf(mi == -CUDART_INF_F ? 0.f : exp2f(mi - mx), src[i * stride + DV + 1], sum);
    }
  }
#pragma unroll
  for (int c = 0; c < NC; ++c) val[c][0] = val[c][1] = 0.f;
#pragma unroll 4
  for (int i = 0; i < count; ++i) {
    const float* pr = src + i * stride;
    const float mi = pr[DV];
    const float f = mi == -CUDART_INF_F ? 0.f : exp2f(mi - mx);  // a key range in which the row saw nothing
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int d = c * 64 + lane * 2;
      if (d < DV) {
        const float2 v = *reinterpret_cast<const float2*>(pr + d);
        val[c][0] = fmaf(f, v.x, val[c][0]);
        val[c][1] = fmaf(f, v.y, val[c][1]);
      }
    }
  }
}

// The end of a row: a1 / l1 - lambda a2 / l2, the head's norm, the gate, and the store.
__device__ __forceinline__ void finish_row(const Params& p, float (&v1)[NC][2], const float (&v2)[NC][2], float l1, float l2, size_t t, int head,
                                           int lane) {
  const float i1 = l1 > 0.f ? 1.f / l1 : 0.f, i2 = l2 > 0.f ? p.lambda / l2 : 0.f;
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const float a = v1[c][0] * i1 - v2[c][0] * i2, b = v1[c][1] * i1 - v2[c][1] * i2;
    v1[c][0] = a;
    v1[c][1] = b;
    ss = fmaf(a, a, fmaf(b, b, ss));  // lanes beyond DV hold zeros
  }
  ss = warp_sum(ss);
  const float g = p.gate != nullptr ? 1.f / (1.f + expf(-__bfloat162float(p.gate[t * p.gate_stride + head]))) : 1.f;
  const float f = rsqrtf(ss / (float)DV + p.eps) * p.post * g;
  bf16* dst = p.out + (t * p.nh + head) * DV;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const int d = c * 64 + lane * 2;
    if (d < DV) *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(v1[c][0] * f, v1[c][1] * f);
  }
}

__global__ void __launch_bounds__(THREADS, MIN_CTAS) diff_attention_tc_kernel(const Params p) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* sQ = smem;
  unsigned char* sK = smem + BLOCK_M * KROW;
  unsigned char* sV = sK + 2 * KTILE;
  float* part = reinterpret_cast<float*>(sK);  // after the walk: [WARPS][16][PROW]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int s = blockIdx.y;
  const int tile = p.splits > 1 ? 0 : blockIdx.x, split = p.splits > 1 ? blockIdx.x : 0;
  const int kvh = blockIdx.z / p.head_chunks, hc = blockIdx.z - kvh * p.head_chunks;
  const int q0 = p.q_start[s];
  const int qlen = p.q_start[s + 1] - q0;
  const int tok0 = tile * p.tokens_per_tile;
  if (tok0 >= qlen) return;
  const int kvlen = p.kv_len[s];
  const int ntok = min(p.tokens_per_tile, qlen - tok0);
  const int G = p.nh / p.nkv, Gc = p.heads_per_chunk;
  const int head0 = kvh * G + hc * Gc;
  Tile T;
  T.Gc = Gc;
  T.kvh = kvh;
  T.nheads = min(Gc, G - hc * Gc);
  T.pos0 = kvlen - qlen + tok0;
  T.rows_used = ntok * Gc;
  T.table = p.block_tables + (size_t)s * p.max_blocks;
  // keys of the tile: the kept first tokens in front of the window, [0, kept), and the window's, [lo, hi)
  T.hi = T.pos0 + ntok;
  T.lo = (p.window > 0 && T.pos0 - p.window + 1 > 0) ? T.pos0 - p.window + 1 : 0;
  T.kept = min(p.keep_first, T.lo);
  T.kept_tiles = (T.kept + BLOCK_N - 1) / BLOCK_N;
  T.first_tile = max(T.lo / BLOCK_N, T.kept_tiles);
  T.num_tiles = T.kept_tiles + max(0, (T.hi + BLOCK_N - 1) / BLOCK_N - T.first_tile);
  T.it0 = 0;
  T.it1 = T.num_tiles;
  if (p.splits > 1) {  // single tokens only: CTA `split` walks its share of the key tiles, possibly none
    const int per = (T.num_tiles + p.splits - 1) / p.splits;
    T.it0 = min(T.num_tiles, split * per);
    T.it1 = min(T.num_tiles, T.it0 + per);
  }

  for (int idx = tid; idx < BLOCK_M * KCHUNKS; idx += THREADS) {
    const int r = idx / KCHUNKS, c = idx - r * KCHUNKS;
    const int tok = r / Gc, hd = r - tok * Gc;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < T.rows_used && hd < T.nheads) v = *reinterpret_cast<const uint4*>(p.q + ((size_t)(q0 + tok0 + tok) * p.nh + head0 + hd) * 2 * DK + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * KROW + c * 16) = v;
  }

  int KS;
  if (T.rows_used <= 16) {
    KS = 4;
    walk<4>(p, T, sQ, sK, sV, part);
  } else if (T.rows_used <= 32) {
    KS = 2;
    walk<2>(p, T, sQ, sK, sV, part);
  } else {
    KS = 1;
    walk<1>(p, T, sQ, sK, sV, part);
  }
  __syncthreads();

  // a warp per row: merge the key ranges of each map; then the row's end, or, with keys split between CTAs, the scratch
  for (int r = warp; r < T.rows_used; r += WARPS) {
    const int tok = r / Gc, hd = r - tok * Gc;
    if (hd >= T.nheads) continue;
    float val[2][NC][2], mx[2], sum[2];
#pragma unroll
    for (int mp = 0; mp < 2; ++mp)
      merge_partials<false>(part + ((size_t)(mp * 4 + (r >> 4) * KS) * 16 + (r & 15)) * PROW, (size_t)16 * PROW, KS, lane, val[mp], mx[mp], sum[mp]);
    const size_t t = (size_t)(q0 + tok0 + tok);
    if (p.splits <= 1) {
      finish_row(p, val[0], val[1], sum[0], sum[1], t, head0 + hd, lane);
    } else {
#pragma unroll
      for (int mp = 0; mp < 2; ++mp) {
        float* dst = p.scratch + (((size_t)s * p.nh + head0 + hd) * p.splits + split) * 2 * SROW + mp * SROW;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int d = c * 64 + lane * 2;
          if (d < DV) *reinterpret_cast<float2*>(dst + d) = make_float2(val[mp][c][0], val[mp][c][1]);
        }
        if (lane == 0) {
          dst[DV] = mx[mp];
          dst[DV + 1] = sum[mp];
        }
      }
    }
  }
}

// Keys split between CTAs: a warp per (sequence, head) merges the splits of each map and ends the row.
__global__ void diff_merge_splits_kernel(const Params p, int num_seqs) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= num_seqs * p.nh) return;
  const int s = row / p.nh, head = row - s * p.nh;
  float val[2][NC][2], mx[2], sum[2];
#pragma unroll
  for (int mp = 0; mp < 2; ++mp) merge_partials<true>(p.scratch + (size_t)row * p.splits * 2 * SROW + mp * SROW, (size_t)2 * SROW, p.splits, lane, val[mp], mx[mp], sum[mp]);
  finish_row(p, val[0], val[1], sum[0], sum[1], (size_t)p.q_start[s], head, lane);
}

}  // namespace tc

DLI_EXPORT int dli_diff_attention_tc(void* out, const void* q, const void* k_pool, const void* v_pool, const int* block_tables, int max_blocks,
                                     const int* q_start, const int* kv_len, int num_seqs, int max_q_len, const void* gate, int gate_stride,
                                     int nh, int nkv, int page_size, int window, int keep_first, float scale, float lambda, float post, float eps,
                                     int splits, float* scratch, cudaStream_t stream) {
  using namespace tc;
  if (num_seqs == 0 || max_q_len == 0) return 0;
  if (nkv < 1 || nh % nkv) return DLI_ERR_UNSUPPORTED;
  if (splits > 1 && (max_q_len != 1 || scratch == nullptr || splits > 65535)) return DLI_ERR_UNSUPPORTED;
  static OncePerDevice attr;
  if (!attr.here()) {
    cudaError_t e = cudaFuncSetAttribute(diff_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(diff_attention_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    attr.here() = true;
  }
  Params p;
  p.out = (bf16*)out; p.q = (const bf16*)q; p.k_pool = (const bf16*)k_pool; p.v_pool = (const bf16*)v_pool;
  p.block_tables = block_tables; p.max_blocks = max_blocks; p.q_start = q_start; p.kv_len = kv_len;
  p.gate = (const bf16*)gate; p.gate_stride = gate_stride;
  p.nh = nh; p.nkv = nkv; p.page_size = page_size; p.window = window; p.keep_first = keep_first;
  const int G = nh / nkv;
  p.heads_per_chunk = G < BLOCK_M ? G : BLOCK_M;
  p.head_chunks = (G + p.heads_per_chunk - 1) / p.heads_per_chunk;
  p.tokens_per_tile = BLOCK_M / p.heads_per_chunk;
  p.scale_log2 = scale * 1.4426950408889634f; p.lambda = lambda; p.post = post; p.eps = eps;
  p.splits = splits > 1 ? splits : 1; p.scratch = scratch;
  const int tiles = p.splits > 1 ? p.splits : (max_q_len + p.tokens_per_tile - 1) / p.tokens_per_tile;
  if (num_seqs > 65535 || nkv * p.head_chunks > 65535) return DLI_ERR_UNSUPPORTED;
  launch_pdl(diff_attention_tc_kernel, dim3(tiles, num_seqs, nkv * p.head_chunks), dim3(THREADS), SMEM_BYTES, stream, 1, p);
  if (p.splits > 1) {
    const int warps = 4;
    launch_pdl(diff_merge_splits_kernel, dim3((num_seqs * nh + warps - 1) / warps), dim3(warps * 32), 0, stream, 1, p, num_seqs);
  }
  return (int)cudaGetLastError();
}
#endif
