// The experts' products of a routed feed-forward for steps of many tokens (bfloat16): the (token, expert) pairs are
// sorted by expert on the device (a counting sort; no shape depends on the data), and two grouped products run over the
// sorted rows on the tensor cores (mma.sync m16n8k16 fed by ldmatrix, float32 sums), a tile of 64 rows belonging to one expert:
//   hidden[row] = act(gate_e x) * (up_e x)        (both sums rounded to bfloat16 first, as a stored product would be)
//   partial[row] = down_e hidden[row]             (float32)
//   out[t] = sum_k weights[t][k] * partial[row of pair (t, k)], in the order of k, float32, one rounding.
#include <math_constants.h>

#include "common.cuh"

using namespace dli;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int BM = 64, BN = 64, BK = 64, PAD = 8, THREADS = 128;
constexpr int LDS = BK + PAD;  // elements of a staged row: 144 bytes, so the eight rows of an 8 x 8 fragment lie in different banks
constexpr int TILE_ELEMS = BM * LDS;  // one staged tile of 64 rows (A, or one of B's)
constexpr int SORT_SMALL_MAX_PAIRS = 2048;  // up to here one block sorts the pairs in one launch

// counts <- 0, and -1 into the tile and row maps (what no expert claims stays -1)
__global__ void moe_init_kernel(int* __restrict__ counts, int n_counts, int* __restrict__ maps, int n_maps) {
  pdl_launch_dependents();
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_counts + n_maps; i += gridDim.x * blockDim.x) {
    if (i < n_counts) counts[i] = 0;
    else maps[i - n_counts] = -1;
  }
}

__global__ void moe_count_kernel(const int* __restrict__ ids, int pairs, int* __restrict__ counts, int* __restrict__ rank) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p < pairs) rank[p] = atomicAdd(&counts[ids[p]], 1);
}

// offsets[e]: first sorted row of expert e, every expert's run padded to whole tiles; tile_expert[tile]: the tile's expert
// (-1 behind the last one: set by the caller beforehand).
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets, int* __restrict__ tile_expert) {
  pdl_launch_dependents();
  pdl_wait();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      at += (counts[e] + BM - 1) / BM * BM;
    }
    offsets[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int tile = offsets[e] / BM; tile < offsets[e + 1] / BM; ++tile) tile_expert[tile] = e;
}

// pos[p]: the sorted row of pair p; row_pair[row]: the pair of a sorted row (-1 for padding: set by the caller beforehand)
__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ rank, const int* __restrict__ offsets, int pairs,
                                   int* __restrict__ pos, int* __restrict__ row_pair) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pairs) return;
  const int row = offsets[ids[p]] + rank[p];
  pos[p] = row;
  row_pair[row] = p;
}

// The whole sort in one block, for steps of few pairs (a decode step): maps to -1, counts and ranks in shared memory, offsets,
// tile map, scatter.  One launch instead of four.
__global__ void moe_sort_small_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ offsets, int* __restrict__ pos,
                                      int* __restrict__ tile_expert, int tiles, int* __restrict__ row_pair) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int sh[];  // counts [E] | offsets [E + 1]
  int* cnt = sh;
  int* off = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  for (int i = threadIdx.x; i < tiles; i += blockDim.x) tile_expert[i] = -1;
  for (int i = threadIdx.x; i < tiles * BM; i += blockDim.x) row_pair[i] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) pos[p] = atomicAdd(&cnt[ids[p]], 1);  // the pair's rank for now
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = at;
      at += (cnt[e] + BM - 1) / BM * BM;
    }
    off[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < E)
      for (int tile = off[e] / BM; tile < off[e + 1] / BM; ++tile) tile_expert[tile] = e;
  }
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int row = off[ids[p]] + pos[p];
    pos[p] = row;
    row_pair[row] = p;
  }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src, int bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ float glu_act(float g, int act) {
  if (act == 1) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  if (act == 2) return g / (1.f + expf(-1.702f * g));
  return g / (1.f + expf(-g));
}

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// C[row][n] = sum_k A[src(row)][k] * B_e[n][k] over one tile of 64 sorted rows of expert e = tile_expert[tile] and 64 columns.
// GLU: two B tiles (rows n and half + n of the expert's matrix) and C = act(first) * second, bfloat16; else C float32.
// row_pair (GLU): the sorted row's pair, whose token pair / top is the row of A (-1: zeros); without it the row of A is the sorted row.
// k-tiles of 64 arrive by asynchronous copies STAGES deep: three for a step of few tokens, which only streams the experts' matrices
// and is bound by the bytes in flight; two for many tokens, where more CTAs an SM hide more latency.  Fragments are read with ldmatrix.
template <bool GLU, int STAGES>
__global__ void __launch_bounds__(THREADS) moe_grouped_gemm_kernel(const bf16* __restrict__ A, long long a_stride, const int* __restrict__ row_pair,
                                                                   int top, const bf16* __restrict__ B, long long b_expert_stride, int half,
                                                                   void* __restrict__ C, long long c_stride, int N, int K,
                                                                   const int* __restrict__ tile_expert, int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int tile_m = blockIdx.y;
  const int e = tile_expert[tile_m];
  if (e < 0) return;
  constexpr int NB = GLU ? 2 : 1;
  constexpr int STAGE_ELEMS = (1 + NB) * TILE_ELEMS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp >> 1, wn = warp & 1;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * BN;
  const bf16* Be = B + (size_t)e * b_expert_stride;

  // the four 16-byte chunks of A (and of each B tile) this thread copies per k-tile: rows r0 + 16 i, one column of chunks
  const int r0 = tid >> 3, cc = (tid & 7) * 8;
  const bf16* a_src[4];
  const bf16* b_src[NB][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 16 * i;
    const int row = tile_m * BM + r;
    if (row_pair) {
      const int p = row_pair[row];
      a_src[i] = p >= 0 ? A + (size_t)(p / top) * a_stride : nullptr;
    } else {
      a_src[i] = A + (size_t)row * a_stride;
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) b_src[j][i] = n0 + r < N ? Be + (size_t)(j * half + n0 + r) * K : nullptr;
  }

  auto load = [&](int stage, int k0) {
    bf16* As = smem + stage * STAGE_ELEMS;
    const bool in_k = k0 + cc < K;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + 16 * i;
      const bool a_ok = in_k && a_src[i] != nullptr;
      cp_async16(As + r * LDS + cc, a_ok ? (const void*)(a_src[i] + k0 + cc) : (const void*)A, a_ok ? 16 : 0);
#pragma unroll
      for (int j = 0; j < NB; ++j) {
        const bool b_ok = in_k && b_src[j][i] != nullptr;
        cp_async16(As + (1 + j) * TILE_ELEMS + r * LDS + cc, b_ok ? (const void*)(b_src[j][i] + k0 + cc) : (const void*)B, b_ok ? 16 : 0);
      }
    }
  };

  float acc[NB][2][4][4];
#pragma unroll
  for (int j = 0; j < NB; ++j)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int ni = 0; ni < 4; ++ni)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[j][mi][ni][q] = 0.f;

  const int k_tiles = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < k_tiles) load(s, s * BK);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // k-tile kt has landed, and everyone is done with the stage that is filled next
    const int next = kt + STAGES - 1;
    if (next < k_tiles) load(next % STAGES, next * BK);
    cp_async_commit();
    const bf16* As = smem + (kt % STAGES) * STAGE_ELEMS;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) ldmatrix_x4(a[mi], As + (wm * 32 + mi * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          uint32_t b4[4];
          ldmatrix_x4(b4, As + (1 + j) * TILE_ELEMS + (wn * 32 + p * 16 + (lane & 7) + ((lane >> 4) << 3)) * LDS + kk + ((lane >> 3) & 1) * 8);
          const uint32_t blo[2] = {b4[0], b4[1]}, bhi[2] = {b4[2], b4[3]};
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma_bf16(acc[j][mi][2 * p], a[mi], blo);
            mma_bf16(acc[j][mi][2 * p + 1], a[mi], bhi);
          }
        }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < 4; ++ni)
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const size_t row = (size_t)tile_m * BM + wm * 32 + mi * 16 + g + hrow * 8;
        const int col = n0 + wn * 32 + ni * 8 + 2 * t;
        if (col >= N) continue;
        const float v0 = acc[0][mi][ni][2 * hrow], v1 = acc[0][mi][ni][2 * hrow + 1];
        if (GLU) {
          const float u0 = acc[NB - 1][mi][ni][2 * hrow], u1 = acc[NB - 1][mi][ni][2 * hrow + 1];
          bf16* dst = reinterpret_cast<bf16*>(C) + row * c_stride + col;
          dst[0] = __float2bfloat16_rn(glu_act(round_bf16(v0), act) * round_bf16(u0));
          if (col + 1 < N) dst[1] = __float2bfloat16_rn(glu_act(round_bf16(v1), act) * round_bf16(u1));
        } else {
          float* dst = reinterpret_cast<float*>(C) + row * c_stride + col;
          dst[0] = v0;
          if (col + 1 < N) dst[1] = v1;
        }
      }
}

__global__ void moe_combine_kernel(bf16* __restrict__ out, const float* __restrict__ partial, const int* __restrict__ pos,
                                   const float* __restrict__ weights, int W, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t t = blockIdx.x;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weights[t * top + k], partial[(size_t)pos[t * top + k] * W + c], acc);
    out[t * W + c] = __float2bfloat16_rn(acc);
  }
}

}  // namespace

// Upper bound of the tiles the sorted rows take: every expert's run is padded to whole tiles.
DLI_EXPORT int dli_moe_grouped_tiles(int pairs, int E) { return (pairs < E ? pairs : E) + pairs / BM; }
DLI_EXPORT int dli_moe_grouped_tile_rows() { return BM; }

// ints: scratch of E + 1 (counts) + E + 1 (offsets) + 2 pairs (rank, pos) + tiles (tile_expert) + tiles * BM (row_pair) ints;
// hidden: [tiles * BM][ff] bfloat16; partial: [tiles * BM][W] float32.  stages: 2 or 3 deep copies, or 0: chosen here.
DLI_EXPORT int dli_moe_grouped(void* out, const void* x, const int* ids, const float* weights, const void* w_gate_up, const void* w_down, int* ints,
                               void* hidden, float* partial, int n, int W, int ff, int E, int top, int act, int stages, cudaStream_t stream) {
  if (n == 0) return 0;
  if (W < 8 || ff < 8 || (W % 8) || (ff % 8) || E < 1 || top < 1 || ((((uintptr_t)x) | ((uintptr_t)w_gate_up) | ((uintptr_t)w_down) | ((uintptr_t)hidden)) & 15))
    return DLI_ERR_UNSUPPORTED;
  const int pairs = n * top;
  const int tiles = dli_moe_grouped_tiles(pairs, E);
  if (tiles > 65535) return DLI_ERR_UNSUPPORTED;
  int* counts = ints;
  int* offsets = counts + E + 1;
  int* rank = offsets + E + 1;
  int* pos = rank + pairs;
  int* tile_expert = pos + pairs;
  int* row_pair = tile_expert + tiles;
  cudaError_t e;
  if (pairs <= SORT_SMALL_MAX_PAIRS && (2 * E + 1) * sizeof(int) <= 48 * 1024) {
    e = launch_pdl((moe_sort_small_kernel), dim3(1), dim3(256), (size_t)(2 * E + 1) * sizeof(int), stream, 1, ids, pairs, E, offsets, pos, tile_expert, tiles,
                   row_pair);
    if (e != cudaSuccess) return (int)e;
  } else {
    const int n_maps = tiles + tiles * BM;
    e = launch_pdl((moe_init_kernel), dim3((E + 1 + n_maps + 255) / 256 < 1024 ? (E + 1 + n_maps + 255) / 256 : 1024), dim3(256), 0, stream, 1, counts, E + 1,
                   tile_expert, n_maps);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_count_kernel), dim3((pairs + 255) / 256), dim3(256), 0, stream, 1, ids, pairs, counts, rank);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_plan_kernel), dim3(1), dim3(256), 0, stream, 1, (const int*)counts, E, offsets, tile_expert);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_scatter_kernel), dim3((pairs + 255) / 256), dim3(256), 0, stream, 1, ids, (const int*)rank, (const int*)offsets, pairs, pos, row_pair);
    if (e != cudaSuccess) return (int)e;
  }
  constexpr int TILE_BYTES = TILE_ELEMS * (int)sizeof(bf16);
  static OncePerDevice configured;
  if (!configured.here()) {
    e = cudaFuncSetAttribute(moe_grouped_gemm_kernel<true, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 3 * TILE_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(moe_grouped_gemm_kernel<false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 3 * 2 * TILE_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(moe_grouped_gemm_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 3 * TILE_BYTES);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(moe_grouped_gemm_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 2 * TILE_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured.here() = true;
  }
  const int deep = stages == 2 || stages == 3 ? stages : (pairs > 16 * E ? 2 : 3);  // many rows an expert: the products bound the time, not the stream
  const dim3 grid_up((ff + BN - 1) / BN, tiles), grid_down((W + BN - 1) / BN, tiles);
  if (deep == 3) {
    e = launch_pdl((moe_grouped_gemm_kernel<true, 3>), grid_up, dim3(THREADS), 3 * 3 * TILE_BYTES, stream, 1, (const bf16*)x, (long long)W, (const int*)row_pair, top,
                   (const bf16*)w_gate_up, (long long)2 * ff * W, ff, hidden, (long long)ff, ff, W, (const int*)tile_expert, act);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_grouped_gemm_kernel<false, 3>), grid_down, dim3(THREADS), 3 * 2 * TILE_BYTES, stream, 1, (const bf16*)hidden, (long long)ff,
                   (const int*)nullptr, top, (const bf16*)w_down, (long long)W * ff, 0, (void*)partial, (long long)W, W, ff, (const int*)tile_expert, 0);
  } else {
    e = launch_pdl((moe_grouped_gemm_kernel<true, 2>), grid_up, dim3(THREADS), 2 * 3 * TILE_BYTES, stream, 1, (const bf16*)x, (long long)W, (const int*)row_pair, top,
                   (const bf16*)w_gate_up, (long long)2 * ff * W, ff, hidden, (long long)ff, ff, W, (const int*)tile_expert, act);
    if (e != cudaSuccess) return (int)e;
    e = launch_pdl((moe_grouped_gemm_kernel<false, 2>), grid_down, dim3(THREADS), 2 * 2 * TILE_BYTES, stream, 1, (const bf16*)hidden, (long long)ff,
                   (const int*)nullptr, top, (const bf16*)w_down, (long long)W * ff, 0, (void*)partial, (long long)W, W, ff, (const int*)tile_expert, 0);
  }
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl((moe_combine_kernel), dim3(n), dim3(W >= 1024 ? 256 : 128), 0, stream, 1, (bf16*)out, (const float*)partial, (const int*)pos, weights, W, top);
  return (int)e;
}
