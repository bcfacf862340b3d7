// After the fused q/k/v projection: bias, per-head RMSNorm of q and k, rotation, and the cache write.
//
// One warp handles one (token, head) row of the projection output [tokens, (H + 2K) * head_dim]:
//   q heads: (+bias) -> RMSNorm over head_dim with the layer's q gain -> rotation -> q_out [tokens, H, head_dim]
//   k heads: (+bias) -> RMSNorm with the k gain -> rotation -> key page of the token's sequence
//   v heads: (+bias) -> value page, unchanged
// Norm before rotation, values never normalised (sleuth/forge/model/attention.py:121-126); rotation pairs
// channel i with i + rot/2: (a, b) -> (a*cos - b*sin, b*cos + a*sin) (sleuth/forge/model/rope.py:41-55); the
// reference's own fused form is sleuth/forge/model/fused_ops.py:53-85. Everything is float32 between the load and
// the single rounding at the store. cos/sin come from tables [positions, rot/2] that the position part built in
// float32, so the angles are those of the reference's tables (rope.py:30-38).
//
// A token's key and value go to page block_table[seq, pos / 64], row pos % 64 of the pool
// [pages, kv_heads, 64, head_dim].
#include "common.cuh"

namespace slb {

struct QkvPostArgs {
  const void* qkv;
  const float* bias;        // [(H + 2K) * hd] or null
  const float* q_gain;      // [hd] or null (no QK-norm)
  const float* k_gain;
  const float* cos_table;   // [positions, rot / 2] or null (no rotation)
  const float* sin_table;
  void* q_out;              // [tokens, H, hd]
  void* k_pool;             // [pages, K, 64, hd] or null (this application only reads a shared cache)
  void* v_pool;
  const int* tok_seq;       // [tokens]
  const int* tok_pos;       // [tokens]
  const int* block_table;   // [seqs, table_stride]
  int table_stride;
  int tokens, heads, kv_heads, head_dim, rot_dim;
  float eps;
};

template <typename T, int PER_LANE>
__global__ void qkv_post_kernel(QkvPostArgs a) {
  pdl_enter();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rows_per_token = a.heads + 2 * a.kv_heads;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)a.tokens * rows_per_token) return;
  const int t = (int)(item / rows_per_token);
  const int r = (int)(item - (long long)t * rows_per_token);
  const int hd = a.head_dim, half = a.rot_dim >> 1;

  const T* src = (const T*)a.qkv + ((size_t)t * rows_per_token + r) * hd;
  const float* bias = a.bias ? a.bias + (size_t)r * hd : nullptr;

  // lane l holds channels l, l + 32, ... (PER_LANE of them, guarded by head_dim)
  float v[PER_LANE];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int c = lane + 32 * i;
    float x = 0.0f;
    if (c < hd) {
      x = to_f32(src[c]);
      if (bias) x += bias[c];
    }
    v[i] = x;
    ss = fmaf(x, x, ss);
  }

  const bool is_q = r < a.heads;
  const bool is_k = !is_q && r < a.heads + a.kv_heads;
  const float* gain = is_q ? a.q_gain : (is_k ? a.k_gain : nullptr);

  if (is_q || is_k) {
    if (gain) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)hd + a.eps);
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) v[i] = (v[i] * inv) * gain[c];
      }
    }
    if (a.cos_table && half > 0) {
      // Channel c < half pairs with c + half. The partner lives in another lane or register, so the
      // row goes through shared memory once.
      __shared__ float stage_all[8][256];
      float* stage = stage_all[threadIdx.x >> 5];
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < hd) stage[c] = v[i];
      }
      __syncwarp();
      const int pos = a.tok_pos[t];
      const float* cs = a.cos_table + (size_t)pos * half;
      const float* sn = a.sin_table + (size_t)pos * half;
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < a.rot_dim) {
          const int j = c < half ? c : c - half;
          const float co = cs[j], si = sn[j];
          const float other = c < half ? -stage[c + half] : stage[c - half];
          v[i] = v[i] * co + other * si;
        }
      }
    }
  }

  T* dst;
  if (is_q) {
    dst = (T*)a.q_out + ((size_t)t * a.heads + r) * hd;
  } else {
    if (a.k_pool == nullptr) return;
    const int kh = is_k ? r - a.heads : r - a.heads - a.kv_heads;
    const int pos = a.tok_pos[t];
    const int page = a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens];
    T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
    dst = pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + (pos % kPageTokens)) * hd;
  }
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int c = lane + 32 * i;
    if (c < hd) dst[c] = from_f32<T>(v[i]);
  }
}

// Head sizes 64, 128 and 256 with the whole head rotated (or none of it): lane l holds the EPL = head_dim / 32
// contiguous channels l * EPL .., one vector load and store per lane, and a channel's rotation partner
// (head_dim / 2 away) sits at the same place in lane l ^ 16, so a shuffle replaces the shared-memory staging.
template <typename T, int EPL>
struct alignas(sizeof(T) * EPL) LaneVec {
  T v[EPL];
};

template <typename T, int EPL>
__global__ void qkv_post_vec_kernel(QkvPostArgs a) {
  pdl_enter();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int rows_per_token = a.heads + 2 * a.kv_heads;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)a.tokens * rows_per_token) return;
  const int t = (int)(item / rows_per_token);
  const int r = (int)(item - (long long)t * rows_per_token);
  constexpr int HD = 32 * EPL;
  const int c0 = lane * EPL;

  const LaneVec<T, EPL> in = *reinterpret_cast<const LaneVec<T, EPL>*>(
      (const T*)a.qkv + ((size_t)t * rows_per_token + r) * HD + c0);
  float v[EPL];
  float ss = 0.0f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    float x = to_f32(in.v[e]);
    if (a.bias) x += a.bias[(size_t)r * HD + c0 + e];
    v[e] = x;
    ss = fmaf(x, x, ss);
  }
  const bool is_q = r < a.heads;
  const bool is_k = !is_q && r < a.heads + a.kv_heads;
  const float* gain = is_q ? a.q_gain : (is_k ? a.k_gain : nullptr);
  const int pos = a.tok_pos[t];
  if (is_q || is_k) {
    if (gain) {
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
      for (int e = 0; e < EPL; ++e) v[e] = (v[e] * inv) * gain[c0 + e];
    }
    if (a.cos_table) {
      const float* cs = a.cos_table + (size_t)pos * (HD / 2) + (lane & 15) * EPL;
      const float* sn = a.sin_table + (size_t)pos * (HD / 2) + (lane & 15) * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float partner = __shfl_xor_sync(0xffffffffu, v[e], 16);
        const float other = lane < 16 ? -partner : partner;
        v[e] = v[e] * cs[e] + other * sn[e];
      }
    }
  }
  T* dst;
  if (is_q) {
    dst = (T*)a.q_out + ((size_t)t * a.heads + r) * HD;
  } else {
    if (a.k_pool == nullptr) return;
    const int kh = is_k ? r - a.heads : r - a.heads - a.kv_heads;
    const int page = a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens];
    T* pool = (T*)(is_k ? a.k_pool : a.v_pool);
    dst = pool + (((size_t)page * a.kv_heads + kh) * kPageTokens + (pos % kPageTokens)) * HD;
  }
  LaneVec<T, EPL> out;
#pragma unroll
  for (int e = 0; e < EPL; ++e) out.v[e] = from_f32<T>(v[e]);
  *reinterpret_cast<LaneVec<T, EPL>*>(dst + c0) = out;
}

template <typename T>
static int launch_qkv_post(const QkvPostArgs& a, cudaStream_t s) {
  const long long items = (long long)a.tokens * (a.heads + 2 * a.kv_heads);
  const int warps = 8;
  const long long blocks = (items + warps - 1) / warps;
  SLB_REQUIRE(blocks < (1ll << 31), "qkv_post: too many rows (%lld)", items);
  const bool whole = a.cos_table == nullptr || a.rot_dim == a.head_dim;
  if (whole && (a.head_dim == 64 || a.head_dim == 128 || a.head_dim == 256) && ((uintptr_t)a.qkv % 16 == 0)) {
    if (a.head_dim == 64) launch(qkv_post_vec_kernel<T, 2>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    else if (a.head_dim == 128) launch(qkv_post_vec_kernel<T, 4>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    else launch(qkv_post_vec_kernel<T, 8>, dim3((int)blocks), dim3(warps * 32), 0, s, a);
    return check_launch("qkv_post");
  }
  const int per_lane = (a.head_dim + 31) / 32;
  switch (per_lane) {
    case 1: launch(qkv_post_kernel<T, 1>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 2: launch(qkv_post_kernel<T, 2>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 3: launch(qkv_post_kernel<T, 3>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    case 4: launch(qkv_post_kernel<T, 4>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
    default: launch(qkv_post_kernel<T, 8>, dim3((int)blocks), dim3(warps * 32), 0, s, a); break;
  }
  return check_launch("qkv_post");
}


// The general form after separate q, k and v projections of any sizes: q [H * dk], k [G * dk], v [G * dv] side by side
// in one float32 row per token. RMS norm of q and k either per head (gains [dk]) or over the whole projection at once
// (all heads of q together, all heads of k together, before they are split; gains [H * dk] and [G * dk]), then the
// rotation of the first rot_dim channels of each head, pairing channel i with i + rot_dim/2 (halves) or channel 2i with
// 2i + 1 (neighbours): (a, b) -> (a cos - b sin, b cos + a sin) with the angle of pair i from the tables
// [positions, rot_dim / 2]. Values are stored as they are. Float32 between the load and the one rounding at the store;
// the sums of squares are formed in an order that the row's layout alone fixes, so a token's result depends on nothing
// but its own row.
struct QkvSpanArgs {
  const float* qkv;         // [tokens, H * dk + G * dk + G * dv]
  const float* q_gain;      // null: no norm
  const float* k_gain;
  const float* cos_table;   // [positions, rot / 2] or null
  const float* sin_table;
  void* q_out;              // [tokens, H, dk]
  void* k_pool;             // [pages, G, 64, dk] or null
  void* v_pool;             // [pages, G, 64, dv]
  const int* tok_seq;
  const int* tok_pos;
  const int* block_table;
  int table_stride;
  int tokens, heads, kv_heads, key_dim, value_dim, rot_dim;
  int norm_dim;             // channels of a head that count in the norms' means (key_dim, or fewer when the heads
                            // carry zero channels at their end that only pad them to a width the kernels take)
  int neighbours;           // 1: pairs (2i, 2i + 1); 0: pairs (i, i + rot / 2)
  int whole;                // 1: one norm over the whole projection; 0: one per head
  float eps;
};

constexpr int kSpanMaxHeads = 512;     // q heads + kv heads

// grid (tokens, slices): a slice takes a share of the token's heads, so that a step of few tokens still fills the SMs;
// every slice forms the sums of squares it needs itself, in the same order, from the same row.
template <typename T>
__global__ void __launch_bounds__(256) qkv_post_span_kernel(QkvSpanArgs a) {
  pdl_enter();
  __shared__ float head_ss[kSpanMaxHeads];
  __shared__ float scratch[33];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = a.heads, G = a.kv_heads, dk = a.key_dim, dv = a.value_dim;
  const size_t row_len = (size_t)(H + G) * dk + (size_t)G * dv;
  const float* row = a.qkv + (size_t)t * row_len;
  const bool normed = a.q_gain != nullptr;
  // the token's place in the cache is looked up first: these dependent loads then overlap the row's
  const int pos = a.tok_pos[t];
  const int page = a.k_pool != nullptr ? a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens] : 0;
  const int nthreads = blockDim.x, nwarps = blockDim.x >> 5;
  const int per_slice = (H + G + gridDim.y - 1) / gridDim.y;
  const int hh0 = blockIdx.y * per_slice, hh1 = min(H + G, hh0 + per_slice);
  float inv_q = 1.0f, inv_k = 1.0f;
  if (normed && a.whole) {
    const int nq = H * dk, nk = G * dk;
    float sq = 0.0f, sk = 0.0f;
    for (int i = threadIdx.x; i < nq; i += nthreads) sq = fmaf(row[i], row[i], sq);
    for (int i = threadIdx.x; i < nk; i += nthreads) sk = fmaf(row[nq + i], row[nq + i], sk);
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    inv_q = 1.0f / sqrtf(sq / (float)(H * a.norm_dim) + a.eps);
    inv_k = 1.0f / sqrtf(sk / (float)(G * a.norm_dim) + a.eps);
  } else if (normed) {
    for (int hh = hh0 + warp; hh < hh1; hh += nwarps) {
      const float* src = row + (size_t)hh * dk;
      float ss = 0.0f;
      for (int c = lane; c < dk; c += 32) ss = fmaf(src[c], src[c], ss);
      ss = warp_sum(ss);
      if (lane == 0) head_ss[hh] = ss;
    }
    __syncthreads();
  }
  const int half_rot = a.cos_table ? a.rot_dim >> 1 : 0;
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half_rot : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half_rot : nullptr;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (a.k_pool != nullptr) {
    const size_t slot = (size_t)page * G * kPageTokens + (pos % kPageTokens);      // + head * 64, in rows
    kdst = (T*)a.k_pool + slot * dk;
    vdst = (T*)a.v_pool + slot * dv;
  }
  const int pairs_per_head = dk >> 1;
  for (int item = threadIdx.x; item < (hh1 - hh0) * pairs_per_head; item += nthreads) {
    const int hh = hh0 + item / pairs_per_head, pi = item % pairs_per_head;
    const bool is_q = hh < H;
    if (!is_q && kdst == nullptr) continue;
    int c0, c1;
    const bool turns = pi < half_rot;
    if (turns) {
      c0 = a.neighbours ? 2 * pi : pi;
      c1 = a.neighbours ? 2 * pi + 1 : pi + half_rot;
    } else {
      c0 = 2 * half_rot + 2 * (pi - half_rot);
      c1 = c0 + 1;
    }
    const float* src = row + (size_t)hh * dk;
    float x0 = src[c0], x1 = src[c1];
    if (normed) {
      const float inv = a.whole ? (is_q ? inv_q : inv_k) : 1.0f / sqrtf(head_ss[hh] / (float)a.norm_dim + a.eps);
      const float* gain = is_q ? a.q_gain : a.k_gain;
      const int g0 = a.whole ? (is_q ? hh : hh - H) * dk : 0;
      x0 = (x0 * inv) * gain[g0 + c0];
      x1 = (x1 * inv) * gain[g0 + c1];
    }
    if (turns) {
      const float co = cs[pi], si = sn[pi];
      const float y0 = x0 * co - x1 * si, y1 = x1 * co + x0 * si;
      x0 = y0;
      x1 = y1;
    }
    T* dst = is_q ? (T*)a.q_out + ((size_t)t * H + hh) * dk : kdst + (size_t)(hh - H) * kPageTokens * dk;
    dst[c0] = from_f32<T>(x0);
    dst[c1] = from_f32<T>(x1);
  }
  if (vdst != nullptr) {      // the values of the kv heads among this slice's heads (kv head g rides with head H + g)
    const float* src = row + (size_t)(H + G) * dk;
    const int g0 = max(hh0, H) - H, g1 = hh1 - H;
    for (int i = g0 * dv + threadIdx.x; i < g1 * dv; i += nthreads) {
      const int g = i / dv, c = i - g * dv;
      vdst[(size_t)g * kPageTokens * dv + c] = from_f32<T>(src[i]);
    }
  }
}

template <typename T>
__device__ __forceinline__ void store4(T* dst, const float4& v) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(dst) = v;
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = pk;
  }
}

// The form for neighbour pairing with key, value and rotated widths that are multiples of 4 and 16-byte aligned
// tensors: a thread takes four channels (two pairs) per item and keeps its at most MAXI items of the slice, with their
// gains and angles, in registers from the first pass on; every load is asked for before the sums of squares are
// joined, so a block waits for memory about twice instead of once per pass and table. When one slice holds the whole
// row (steps of many tokens) the sums come from those registers too and the row is read once.
template <typename T, int MAXI>
__global__ void __launch_bounds__(256) qkv_post_span_quad_kernel(QkvSpanArgs a) {
  pdl_enter();
  __shared__ float head_ss[kSpanMaxHeads];
  __shared__ float scratch[33];
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = a.heads, G = a.kv_heads, dk = a.key_dim, dv = a.value_dim;
  const size_t row_len = (size_t)(H + G) * dk + (size_t)G * dv;
  const float* row = a.qkv + (size_t)t * row_len;
  const float4* row4 = reinterpret_cast<const float4*>(row);
  const bool normed = a.q_gain != nullptr;
  const int pos = a.tok_pos[t];
  const int page = a.k_pool != nullptr ? a.block_table[(size_t)a.tok_seq[t] * a.table_stride + pos / kPageTokens] : 0;
  const int nthreads = blockDim.x, nwarps = blockDim.x >> 5;
  const int per_slice = (H + G + gridDim.y - 1) / gridDim.y;
  const int hh0 = blockIdx.y * per_slice, hh1 = min(H + G, hh0 + per_slice);
  const int quads = dk >> 2, n_items = (hh1 - hh0) * quads;
  const int half_rot = a.cos_table ? a.rot_dim >> 1 : 0;
  const float* cs = a.cos_table ? a.cos_table + (size_t)pos * half_rot : nullptr;
  const float* sn = a.cos_table ? a.sin_table + (size_t)pos * half_rot : nullptr;

  float4 v[MAXI], g[MAXI];
  float2 co[MAXI], si[MAXI];
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    const int item = threadIdx.x + i * nthreads;
    v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    g[i] = make_float4(1.f, 1.f, 1.f, 1.f);
    co[i] = make_float2(1.f, 1.f);
    si[i] = make_float2(0.f, 0.f);
    if (item < n_items) {
      const int hh = hh0 + item / quads, c = (item % quads) * 4;
      v[i] = row4[hh0 * quads + item];
      if (normed) {
        const bool is_q = hh < H;
        const float* gain = (is_q ? a.q_gain : a.k_gain) + (a.whole ? (is_q ? hh : hh - H) * dk : 0);
        g[i] = *reinterpret_cast<const float4*>(gain + c);
      }
      if (c < 2 * half_rot) {
        co[i] = *reinterpret_cast<const float2*>(cs + (c >> 1));
        si[i] = *reinterpret_cast<const float2*>(sn + (c >> 1));
      }
    }
  }
  T* kdst = nullptr;
  if (a.k_pool != nullptr) {
    const size_t slot = (size_t)page * G * kPageTokens + (pos % kPageTokens);      // + head * 64, in rows
    kdst = (T*)a.k_pool + slot * dk;
    // the values of the kv heads among this slice's heads (kv head g rides with head H + g): nothing to wait for
    T* vdst = (T*)a.v_pool + slot * dv;
    const float4* src4 = reinterpret_cast<const float4*>(row + (size_t)(H + G) * dk);
    const int vq = dv >> 2, g0 = max(hh0, H) - H, g1 = hh1 - H;
    for (int i = g0 * vq + threadIdx.x; i < g1 * vq; i += nthreads) {
      const int gh = i / vq, c = (i - gh * vq) * 4;
      store4<T>(vdst + (size_t)gh * kPageTokens * dv + c, src4[i]);
    }
  }
  float inv_q = 1.0f, inv_k = 1.0f;
  if (normed && a.whole) {
    const int nq4 = H * quads, nk4 = G * quads;
    float sq = 0.0f, sk = 0.0f;
    if (gridDim.y == 1) {         // this block holds the whole row: item i is float4 i of the row
#pragma unroll
      for (int i = 0; i < MAXI; ++i) {
        const int item = threadIdx.x + i * nthreads;
        const float ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, v[i].w * v[i].w)));
        if (item < nq4) sq += ss; else sk += ss;      // items past the row hold zeros
      }
    } else {
      for (int i = threadIdx.x; i < nq4 + nk4; i += nthreads) {      // the same values to the same threads as above
        const float4 x = row4[i];
        const float ss = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
        if (i < nq4) sq += ss; else sk += ss;
      }
    }
    sq = block_sum(sq, scratch);
    sk = block_sum(sk, scratch);
    inv_q = 1.0f / sqrtf(sq / (float)(H * a.norm_dim) + a.eps);
    inv_k = 1.0f / sqrtf(sk / (float)(G * a.norm_dim) + a.eps);
  } else if (normed) {
    for (int hh = hh0 + warp; hh < hh1; hh += nwarps) {
      const float* src = row + (size_t)hh * dk;
      float ss = 0.0f;
      for (int c = lane; c < dk; c += 32) ss = fmaf(src[c], src[c], ss);
      ss = warp_sum(ss);
      if (lane == 0) head_ss[hh] = ss;
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < MAXI; ++i) {
    const int item = threadIdx.x + i * nthreads;
    if (item >= n_items) continue;
    const int hh = hh0 + item / quads, c = (item % quads) * 4;
    const bool is_q = hh < H;
    if (!is_q && kdst == nullptr) continue;
    float4 x = v[i];
    if (normed) {
      const float inv = a.whole ? (is_q ? inv_q : inv_k) : 1.0f / sqrtf(head_ss[hh] / (float)a.norm_dim + a.eps);
      x.x = (x.x * inv) * g[i].x; x.y = (x.y * inv) * g[i].y; x.z = (x.z * inv) * g[i].z; x.w = (x.w * inv) * g[i].w;
    }
    if (c < 2 * half_rot) {
      const float x0 = x.x * co[i].x - x.y * si[i].x, x1 = x.y * co[i].x + x.x * si[i].x;
      const float x2 = x.z * co[i].y - x.w * si[i].y, x3 = x.w * co[i].y + x.z * si[i].y;
      x = make_float4(x0, x1, x2, x3);
    }
    T* dst = (is_q ? (T*)a.q_out + ((size_t)t * H + hh) * dk : kdst + (size_t)(hh - H) * kPageTokens * dk) + c;
    store4<T>(dst, x);
  }
}

}  // namespace slb

using namespace slb;

extern "C" int slb_qkv_post(const void* qkv, const float* bias, const float* q_gain, const float* k_gain,
                            const float* cos_table, const float* sin_table, void* q_out, void* k_pool, void* v_pool,
                            const int* tok_seq, const int* tok_pos, const int* block_table, int table_stride,
                            int tokens, int heads, int kv_heads, int head_dim, int rot_dim, float eps, int dtype,
                            void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads >= 0, "qkv_post: tokens=%d heads=%d kv_heads=%d", tokens, heads,
              kv_heads);
  SLB_REQUIRE(head_dim > 0 && head_dim <= 256 && head_dim % 2 == 0,
              "qkv_post: head_dim %d is not supported (even, at most 256)", head_dim);
  SLB_REQUIRE(rot_dim >= 0 && rot_dim <= head_dim && rot_dim % 2 == 0, "qkv_post: rot_dim=%d for head_dim=%d",
              rot_dim, head_dim);
  SLB_REQUIRE((q_gain == nullptr) == (k_gain == nullptr) || kv_heads == 0, "qkv_post: q and k gains go together");
  SLB_REQUIRE(kv_heads == 0 || k_pool == nullptr || (v_pool && block_table && table_stride > 0),
              "qkv_post: a cache write needs both pools and a block table");
  if (tokens == 0) return 0;
  QkvPostArgs a;
  a.qkv = qkv; a.bias = bias; a.q_gain = q_gain; a.k_gain = k_gain;
  a.cos_table = rot_dim > 0 ? cos_table : nullptr; a.sin_table = sin_table;
  a.q_out = q_out; a.k_pool = k_pool; a.v_pool = v_pool;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.block_table = block_table; a.table_stride = table_stride;
  a.tokens = tokens; a.heads = heads; a.kv_heads = kv_heads; a.head_dim = head_dim; a.rot_dim = rot_dim;
  a.eps = eps;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == kF32) return launch_qkv_post<float>(a, s);
  if (dtype == kBF16) return launch_qkv_post<__nv_bfloat16>(a, s);
  return fail(1, "qkv_post: unknown dtype %d", dtype);
}

extern "C" int slb_qkv_post_span(const float* qkv, const float* q_gain, const float* k_gain, const float* cos_table,
                                 const float* sin_table, void* q_out, void* k_pool, void* v_pool, const int* tok_seq,
                                 const int* tok_pos, const int* block_table, int table_stride, int tokens, int heads,
                                 int kv_heads, int key_dim, int value_dim, int rot_dim, int neighbours, int whole, float eps,
                                 int norm_dim, int dtype, void* stream) {
  SLB_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads + kv_heads <= kSpanMaxHeads,
              "qkv_post_span: tokens=%d heads=%d kv_heads=%d (at most %d heads together)", tokens, heads, kv_heads, kSpanMaxHeads);
  SLB_REQUIRE(key_dim > 0 && key_dim % 2 == 0 && value_dim > 0, "qkv_post_span: key size %d must be even, value size %d positive",
              key_dim, value_dim);
  SLB_REQUIRE(rot_dim >= 0 && rot_dim <= key_dim && rot_dim % 2 == 0, "qkv_post_span: rot_dim=%d for key size %d", rot_dim, key_dim);
  SLB_REQUIRE((q_gain == nullptr) == (k_gain == nullptr), "qkv_post_span: q and k gains go together");
  SLB_REQUIRE(rot_dim == 0 || (cos_table && sin_table), "qkv_post_span: a rotation needs its tables");
  SLB_REQUIRE(k_pool == nullptr || (v_pool && block_table && table_stride > 0), "qkv_post_span: a cache write needs both pools and a block table");
  if (tokens == 0) return 0;
  QkvSpanArgs a;
  a.qkv = qkv; a.q_gain = q_gain; a.k_gain = k_gain;
  a.cos_table = rot_dim > 0 ? cos_table : nullptr; a.sin_table = sin_table;
  a.q_out = q_out; a.k_pool = k_pool; a.v_pool = v_pool;
  a.tok_seq = tok_seq; a.tok_pos = tok_pos; a.block_table = block_table; a.table_stride = table_stride;
  a.tokens = tokens; a.heads = heads; a.kv_heads = kv_heads; a.key_dim = key_dim; a.value_dim = value_dim; a.rot_dim = rot_dim;
  a.neighbours = neighbours ? 1 : 0; a.whole = whole ? 1 : 0; a.eps = eps;
  SLB_REQUIRE(norm_dim >= 0 && norm_dim <= key_dim, "qkv_post_span: %d of %d channels count in the norms", norm_dim, key_dim);
  a.norm_dim = norm_dim > 0 ? norm_dim : key_dim;
  cudaStream_t s = (cudaStream_t)stream;
  // slices of a token's heads: enough blocks for two per SM when the step brings few tokens (the number depends on the
  // step's size only; which slice handles a head changes nothing in its result)
  int slices = (2 * sm_count() + tokens - 1) / tokens;
  slices = slices < 1 ? 1 : (slices > 16 ? 16 : slices);
  if (slices > heads + kv_heads) slices = heads + kv_heads;
  const bool aligned = ((uintptr_t)qkv | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)q_out | (uintptr_t)k_pool |
                        (uintptr_t)v_pool) % 16 == 0 && ((uintptr_t)cos_table | (uintptr_t)sin_table) % 8 == 0;
  // many tokens: smaller blocks, so that all of them are resident at once (the float32 run keeps one block shape, so
  // that a row's sums are formed in the same order in every step)
  const int threads = dtype == kBF16 && tokens >= 1024 ? 128 : 256;
  const int per_slice = (heads + kv_heads + slices - 1) / slices;
  const int items = (per_slice * (key_dim / 4) + threads - 1) / threads;      // four-channel items a thread holds
  const bool quad = neighbours && key_dim % 4 == 0 && value_dim % 4 == 0 && rot_dim % 4 == 0 && aligned && items <= 8 &&
                    (dtype == kF32 || dtype == kBF16);
  const dim3 grid(tokens, slices), block(threads);
  if (quad && dtype == kF32) {
    if (items <= 4) launch(qkv_post_span_quad_kernel<float, 4>, grid, block, 0, s, a);
    else launch(qkv_post_span_quad_kernel<float, 8>, grid, block, 0, s, a);
  } else if (quad) {
    if (items <= 4) launch(qkv_post_span_quad_kernel<__nv_bfloat16, 4>, grid, block, 0, s, a);
    else launch(qkv_post_span_quad_kernel<__nv_bfloat16, 8>, grid, block, 0, s, a);
  } else if (dtype == kF32) {
    launch(qkv_post_span_kernel<float>, grid, block, 0, s, a);
  } else if (dtype == kBF16) {
    launch(qkv_post_span_kernel<__nv_bfloat16>, grid, block, 0, s, a);
  } else {
    return fail(1, "qkv_post_span: unknown dtype %d", dtype);
  }
  return check_launch("qkv_post_span");
}
