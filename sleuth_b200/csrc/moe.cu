// Routed experts: router, grouping of (token, choice) pairs by expert, the experts' two products, the weighted sum.
//
// Nothing here needs the host to know how many tokens an expert got: the router counts, a second kernel lays the
// pairs out expert by expert, and the product kernels are launched over the largest number of row tiles that the
// counts could need; a block finds its expert and tile from the counts and leaves when there is none. A step with
// routed experts can therefore be recorded once and replayed.
//
//   moe_route_kernel     logits = W_r h + b in float32, the `top` largest (lowest index first among equals), weights
//                        = softmax over the chosen logits; counts the pairs of each expert
//   moe_group_kernel     place[pair] = where the pair's row lies in the expert-ordered list, list[place] = pair
//   moe_gate_up_kernel   act[place, j] = f(gate_e[j] . h) * (up_e[j] . h), f = silu or relu
//   moe_down_kernel      y[pair, :] = weight[pair] * (down_e act[place])   (float32)
//   moe_combine_kernel   x[t, :] += sum over the token's choices of y, in the order of the choices
// In bfloat16 with inner sizes that are multiples of 8 the two products run on the tensor cores (moe_mma_kernel);
// the kernels above then serve float32 and odd sizes.
#include "mma_sync.cuh"

namespace slb {

constexpr int kMoeTile = 32;        // rows (pairs) of a product tile
constexpr int kMoeCols = 64;        // output columns of a product tile
constexpr int kMoeK = 32;           // inner-dimension slice staged in shared memory

// One warp per token.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ bias,
                                 int* __restrict__ choice, float* __restrict__ weight, int* __restrict__ rank,
                                 int* __restrict__ counts, int tokens, int dim, int E, int top) {
  pdl_enter();
  extern __shared__ float sm[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * warps + warp;
  if (t >= tokens) return;
  float* z = sm + (size_t)warp * E;
  const T* row = h + (size_t)t * dim;
  for (int e = 0; e < E; ++e) {
    const float* w = wr + (size_t)e * dim;
    float s = 0.f;
    for (int i = lane; i < dim; i += 32) s = fmaf(to_f32(row[i]), w[i], s);
    s = warp_sum(s);
    if (lane == 0) z[e] = s + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  float first = 0.f, mass = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
    }
    best_e = min(best_e, E - 1);                 // only logits that are not numbers get here
    if (k == 0) first = best;
    const float p = expf(best - first);
    mass += p;
    if (lane == 0) {
      choice[(size_t)t * top + k] = best_e;
      weight[(size_t)t * top + k] = p;
      z[best_e] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = lane; k < top; k += 32) {
    weight[(size_t)t * top + k] /= mass;
    rank[(size_t)t * top + k] = atomicAdd(&counts[choice[(size_t)t * top + k]], 1);
  }
}

// place[pair] = first row of the pair's expert + the pair's rank there; list[place] = pair.
__global__ void moe_group_kernel(const int* __restrict__ choice, const int* __restrict__ rank,
                                 const int* __restrict__ counts, int* __restrict__ place, int* __restrict__ list,
                                 int pairs, int E) {
  pdl_enter();
  extern __shared__ int first[];
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      first[e] = run;
      run += counts[e];
    }
  }
  __syncthreads();
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < pairs; p += gridDim.x * blockDim.x) {
    const int at = first[choice[p]] + rank[p];
    place[p] = at;
    list[at] = p;
  }
}

// Which expert and which of its row tiles (of `tile` rows) block `b` takes; false when the counts leave it nothing.
__device__ __forceinline__ bool moe_find_tile(const int* counts, int E, int b, int& expert, int& row0, int& rows,
                                              int tile = kMoeTile) {
  int first = 0;
  for (int e = 0; e < E; ++e) {
    const int c = counts[e];
    const int tiles = (c + tile - 1) / tile;
    if (b < tiles) {
      expert = e;
      row0 = first + b * tile;
      rows = min(tile, c - b * tile);
      return true;
    }
    b -= tiles;
    first += c;
  }
  return false;
}

// A 32 x 64 tile of  C = A B^T  on 256 threads (thread: 2 rows x 4 columns), float32 sums, k ascending.
// A rows come through `a_row(r)` (a pointer to the r-th row), B rows through `b_row(c)`.
template <typename T, typename ARow, typename BRow>
__device__ __forceinline__ void moe_tile_product(ARow a_row, BRow b_row, int rows, int cols, int K, float (&acc)[2][4],
                                                 float* As, float* Bs) {
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // ty: rows ty*2.., tx: columns tx*4..
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kMoeK) {
    const int nk = min(kMoeK, K - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < kMoeTile * kMoeK; i += blockDim.x) {
      const int r = i / kMoeK, k = i % kMoeK;
      As[k * (kMoeTile + 1) + r] = (r < rows && k < nk) ? to_f32(a_row(r)[k0 + k]) : 0.f;
    }
    for (int i = threadIdx.x; i < kMoeCols * kMoeK; i += blockDim.x) {
      const int c = i / kMoeK, k = i % kMoeK;
      Bs[k * (kMoeCols + 1) + c] = (c < cols && k < nk) ? to_f32(b_row(c)[k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kMoeK; ++k) {
      const float a0 = As[k * (kMoeTile + 1) + ty * 2], a1 = As[k * (kMoeTile + 1) + ty * 2 + 1];
      const float* bp = Bs + k * (kMoeCols + 1) + tx * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float bv = bp[j];
        acc[0][j] = fmaf(a0, bv, acc[0][j]);
        acc[1][j] = fmaf(a1, bv, acc[1][j]);
      }
    }
  }
}

// grid (row tiles, column tiles of 32 gate + 32 up columns). w_gu [E, 2 * ff, dim]: gate rows then up rows.
template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T* __restrict__ h, const T* __restrict__ w_gu,
                                                          const int* __restrict__ counts, const int* __restrict__ list,
                                                          T* __restrict__ act, int E, int top, int dim, int ff, int relu) {
  pdl_enter();
  __shared__ float As[kMoeK * (kMoeTile + 1)];
  __shared__ float Bs[kMoeK * (kMoeCols + 1)];
  __shared__ int toks[kMoeTile];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows)) return;
  if (threadIdx.x < kMoeTile) toks[threadIdx.x] = threadIdx.x < rows ? list[row0 + threadIdx.x] / top : 0;
  __syncthreads();
  const int j0 = blockIdx.y * 32;
  const int nj = min(32, ff - j0);
  const T* w = w_gu + (size_t)expert * 2 * ff * dim;
  float acc[2][4];
  // tile columns 0..31: gate rows j0.., columns 32..63: up rows j0..
  moe_tile_product<T>([&](int r) { return h + (size_t)toks[r] * dim; },
                      [&](int c) { return w + (size_t)((c < 32 ? 0 : ff) + j0 + min(c & 31, nj - 1)) * dim; }, rows, 64,
                      dim, acc, As, Bs);
  // a thread holds four gate columns or four up columns: pair them through shared memory
  __syncthreads();
  float* Cs = Bs;      // [32 rows][65]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) Cs[(ty * 2 + i) * 65 + tx * 4 + j] = acc[i][j];
  __syncthreads();
  for (int i = threadIdx.x; i < kMoeTile * 32; i += blockDim.x) {
    const int r = i / 32, j = i % 32;
    if (r >= rows || j >= nj) continue;
    const float g = Cs[r * 65 + j], u = Cs[r * 65 + 32 + j];
    const float f = relu ? fmaxf(g, 0.f) : g / (1.0f + expf(-g));
    act[(size_t)(row0 + r) * ff + j0 + j] = from_f32<T>(f * u);
  }
}

// grid (row tiles, column tiles of 64). w_down [E, dim, ff]. y[pair, :] float32.
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                       const int* __restrict__ counts, const int* __restrict__ list,
                                                       const float* __restrict__ weight, float* __restrict__ y, int E,
                                                       int dim, int ff) {
  pdl_enter();
  __shared__ float As[kMoeK * (kMoeTile + 1)];
  __shared__ float Bs[kMoeK * (kMoeCols + 1)];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows)) return;
  const int n0 = blockIdx.y * kMoeCols;
  const int nn = min(kMoeCols, dim - n0);
  const T* w = w_down + (size_t)expert * dim * ff;
  float acc[2][4];
  moe_tile_product<T>([&](int r) { return act + (size_t)(row0 + r) * ff; },
                      [&](int c) { return w + (size_t)(n0 + min(c, nn - 1)) * ff; }, rows, nn, ff, acc, As, Bs);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
    const int pair = list[row0 + r];
    const float wt = weight[pair];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = tx * 4 + j;
      if (c < nn) y[(size_t)pair * dim + n0 + c] = wt * acc[i][j];
    }
  }
}

// ---- the same two products on the warp-level tensor cores (bfloat16, inner sizes that are multiples of 8) ----
// A block of four warps takes 64 rows x 128 columns; a warp 16 rows x all columns (mma.sync m16n8k16, float32 sums).
// The inner dimension goes through shared memory 32 values at a time, two buffers filled by 16-byte asynchronous
// copies; rows are padded to 40 values, which keeps ldmatrix free of bank conflicts. GATED: the 128 columns are 64
// gate rows and the 64 up rows that belong to them, so that a thread holds both halves of each of its outputs.
constexpr int kMmaRows = 64, kMmaCols = 128, kMmaK = 32, kMmaPad = 40;

template <bool GATED>
__global__ void __launch_bounds__(128) moe_mma_kernel(const __nv_bfloat16* __restrict__ a_rows, const __nv_bfloat16* __restrict__ w,
                                                      const int* __restrict__ counts, const int* __restrict__ list,
                                                      const float* __restrict__ weight, __nv_bfloat16* __restrict__ act,
                                                      float* __restrict__ y, int E, int top, int K, int N, int relu) {
  pdl_enter();
  __shared__ __align__(16) __nv_bfloat16 As[2][kMmaRows * kMmaPad];
  __shared__ __align__(16) __nv_bfloat16 Bs[2][kMmaCols * kMmaPad];
  __shared__ int src_row[kMmaRows];
  int expert, row0, rows;
  if (!moe_find_tile(counts, E, blockIdx.x, expert, row0, rows, kMmaRows)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  // GATED: N = ff, the block's columns are gate rows n0 .. n0 + 63 and up rows N + n0 .. ; A rows are token rows of h.
  // else:  N = the output width, columns n0 .. n0 + 127; A rows are the expert-ordered rows of act.
  const int n0 = blockIdx.y * (GATED ? 64 : kMmaCols);
  const int ncols = min(GATED ? 64 : kMmaCols, N - n0);
  if (tid < kMmaRows) src_row[tid] = tid < rows ? (GATED ? list[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const __nv_bfloat16* wb = w + (size_t)expert * (GATED ? 2 : 1) * N * K;

  auto load = [&](int stage, int k0) {
    // 64 rows x 4 sixteen-byte pieces of A, 128 rows x 4 of B
    for (int i = tid; i < kMmaRows * 4; i += 128) {
      const int r = i >> 2, c = (i & 3) * 8;
      __nv_bfloat16* dst = &As[stage][r * kMmaPad + c];
      if (src_row[r] >= 0 && k0 + c < K) cp_async16(smem_u32(dst), a_rows + (size_t)src_row[r] * K + k0 + c);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    for (int i = tid; i < kMmaCols * 4; i += 128) {
      const int r = i >> 2, c = (i & 3) * 8;
      __nv_bfloat16* dst = &Bs[stage][r * kMmaPad + c];
      int col;      // the weight row behind tile column r
      if (GATED) col = (r & 63) < ncols ? (r < 64 ? 0 : N) + n0 + (r & 63) : -1;
      else col = r < ncols ? n0 + r : -1;
      if (col >= 0 && k0 + c < K) cp_async16(smem_u32(dst), wb + (size_t)col * K + k0 + c);
      else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };

  float acc[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int steps = (K + kMmaK - 1) / kMmaK;
  load(0, 0);
  for (int s = 0; s < steps; ++s) {
    const int stage = s & 1;
    if (s + 1 < steps) {
      load(stage ^ 1, (s + 1) * kMmaK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t a_base = smem_u32(&As[stage][0]), b_base = smem_u32(&Bs[stage][0]);
#pragma unroll
    for (int kb = 0; kb < kMmaK / 16; ++kb) {
      uint32_t af[4];
      ldmatrix_x4(af, a_base + 2 * ((warp * 16 + (lane & 15)) * kMmaPad + kb * 16 + ((lane >> 4) << 3)));
#pragma unroll
      for (int jp = 0; jp < 8; ++jp) {       // 16 columns at a time
        uint32_t bf[4];
        ldmatrix_x4(bf, b_base + 2 * ((jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kMmaPad + kb * 16 + (((lane >> 3) & 1) << 3)));
        mma_bf16(acc[2 * jp], af, bf[0], bf[1]);
        mma_bf16(acc[2 * jp + 1], af, bf[2], bf[3]);
      }
    }
    __syncthreads();
  }
  // a thread holds rows g and g + 8 of its warp, columns j * 8 + 2 * t4 (+1) of every column tile j
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = warp * 16 + g + 8 * half;
    if (r >= rows) continue;
    if (GATED) {
      __nv_bfloat16* dst = act + (size_t)(row0 + r) * N + n0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = j * 8 + 2 * t4 + e;
          if (c >= ncols) continue;
          const float gv = acc[j][2 * half + e], uv = acc[j + 8][2 * half + e];
          const float f = relu ? fmaxf(gv, 0.f) : gv / (1.0f + expf(-gv));
          dst[c] = __float2bfloat16_rn(f * uv);
        }
      }
    } else {
      const int pair = list[row0 + r];
      const float wt = weight[pair];
      float* dst = y + (size_t)pair * N + n0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int c = j * 8 + 2 * t4 + e;
          if (c < ncols) dst[c] = wt * acc[j][2 * half + e];
        }
      }
    }
  }
}

__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, int top, int dim, size_t total) {
  pdl_enter();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += step) {
    const size_t t = i / dim, d = i - t * dim;
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += y[(t * top + k) * dim + d];
    x[i] += s;
  }
}

}  // namespace slb

using namespace slb;

// choice, rank, place, list: int32 [tokens * top]; weight: float32 [tokens * top]; counts: int32 [E] (zeroed here).
extern "C" int slb_moe_route(const void* h, const float* w_router, const float* bias, int* choice, float* weight,
                             int* rank, int* counts, int* place, int* list, int tokens, int dim, int E, int top,
                             int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && E > 0 && top > 0 && top <= E, "moe_route: tokens=%d dim=%d experts=%d top=%d",
              tokens, dim, E, top);
  SLB_REQUIRE(E <= 4096, "moe_route: at most 4096 experts, got %d", E);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "moe_route: unknown dtype %d", dtype);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * E, s);
  SLB_REQUIRE(e == cudaSuccess, "moe_route: clearing the counts failed (%s)", cudaGetErrorString(e));
  const int warps = E <= 1024 ? 4 : 1;
  const size_t smem = (size_t)warps * E * sizeof(float);
  const dim3 grid((tokens + warps - 1) / warps), block(warps * 32);
  if (dtype == kF32)
    launch(moe_route_kernel<float>, grid, block, smem, s, (const float*)h, w_router, bias, choice, weight, rank, counts, tokens, dim, E, top);
  else
    launch(moe_route_kernel<__nv_bfloat16>, grid, block, smem, s, (const __nv_bfloat16*)h, w_router, bias, choice, weight, rank,
           counts, tokens, dim, E, top);
  int rc = check_launch("moe_route");
  if (rc) return rc;
  const int pairs = tokens * top;
  int blocks = (pairs + 255) / 256;
  if (blocks > sm_count() * 4) blocks = sm_count() * 4;
  launch(moe_group_kernel, dim3(blocks), dim3(256), sizeof(int) * E, s, (const int*)choice, (const int*)rank, (const int*)counts, place,
         list, pairs, E);
  return check_launch("moe_group");
}

// act: [tokens * top, ff] in the run dtype; y: float32 [tokens * top, dim]; x: the float32 stream [tokens, dim].
extern "C" int slb_moe_experts(const void* h, const void* w_gu, const void* w_down, const int* counts, const int* list,
                               const float* weight, void* act, float* y, float* x, int tokens, int dim, int ff, int E,
                               int top, int relu, int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && dim > 0 && ff > 0 && E > 0 && top > 0, "moe_experts: tokens=%d dim=%d ff=%d experts=%d top=%d",
              tokens, dim, ff, E, top);
  SLB_REQUIRE(dtype == kF32 || dtype == kBF16, "moe_experts: unknown dtype %d", dtype);
  if (tokens == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const long long pairs = (long long)tokens * top;
  // every expert with a pair has at most pairs/tile + 1 tiles more than full ones: an upper bound the host knows
  const long long tiles = pairs / kMoeTile + (pairs < E ? pairs : E);
  SLB_REQUIRE(tiles < (1LL << 31), "moe_experts: too many pairs (%lld)", pairs);
  const dim3 block(256);
  const dim3 g1((unsigned)tiles, (ff + 31) / 32), g2((unsigned)tiles, (dim + kMoeCols - 1) / kMoeCols);
  const bool aligned = ((uintptr_t)h | (uintptr_t)w_gu | (uintptr_t)w_down | (uintptr_t)act) % 16 == 0;
  if (dtype == kBF16 && dim % 8 == 0 && ff % 8 == 0 && aligned) {
    const long long tiles64 = pairs / kMmaRows + (pairs < E ? pairs : E);
    launch(moe_mma_kernel<true>, dim3((unsigned)tiles64, (ff + 63) / 64), dim3(128), 0, s, (const __nv_bfloat16*)h,
           (const __nv_bfloat16*)w_gu, counts, list, weight, (__nv_bfloat16*)act, (float*)nullptr, E, top, dim, ff, relu);
    launch(moe_mma_kernel<false>, dim3((unsigned)tiles64, (dim + kMmaCols - 1) / kMmaCols), dim3(128), 0, s,
           (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, counts, list, weight, (__nv_bfloat16*)nullptr, y, E, top, ff,
           dim, relu);
  } else if (dtype == kF32) {
    launch(moe_gate_up_kernel<float>, g1, block, 0, s, (const float*)h, (const float*)w_gu, counts, list, (float*)act, E, top, dim, ff, relu);
    launch(moe_down_kernel<float>, g2, block, 0, s, (const float*)act, (const float*)w_down, counts, list, weight, y, E, dim, ff);
  } else {
    launch(moe_gate_up_kernel<__nv_bfloat16>, g1, block, 0, s, (const __nv_bfloat16*)h, (const __nv_bfloat16*)w_gu, counts, list,
           (__nv_bfloat16*)act, E, top, dim, ff, relu);
    launch(moe_down_kernel<__nv_bfloat16>, g2, block, 0, s, (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, counts, list,
           weight, y, E, dim, ff);
  }
  int rc = check_launch("moe_experts");
  if (rc) return rc;
  const size_t total = (size_t)tokens * dim;
  size_t blocks = (total + 255) / 256;
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  launch(moe_combine_kernel, dim3((unsigned)blocks), block, 0, s, x, (const float*)y, top, dim, total);
  return check_launch("moe_combine");
}
