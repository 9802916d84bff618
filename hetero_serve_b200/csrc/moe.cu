// Routed feed-forward (mixture of experts).
//
// route    per token: z = W_r h in float32 (or handed in, formed as one product over the step),
//          s = sigmoid(z).  Experts form `n_groups` equal groups
//          of neighbours; a group's score is the sum of its two largest s; only experts of the
//          `keep` best groups are eligible; the `top` eligible experts with the largest s are
//          chosen (the lower index wins a tie) with weights s / (sum of the chosen s + 1e-20).
// expert   g = min(W_g h, limit), u = clamp(W_u h, -limit, limit), y = g * sigmoid(1.702 g) * (u + 1)
// layer    x += sum_k weight_k * (W_d[e_k] y_k), experts in the order they were chosen
//
// A second routing rule (route_top): z = W_r h + b in float32, the `top` largest logits are chosen
// (the lower index wins a tie) and weighted by the softmax over the chosen logits alone; and a
// second expert activation (act 1): y = silu(W_g h) * (W_u h), no limit.
//
// Expert matrices are stacked as they are stored: gate / up [E, ff, width], down [E, width, ff]
// (the summed index runs fastest).  Two paths:
//   * few (token, expert) pairs, and all of float32: every pair streams its expert's rows, one
//     warp per output row with 16-byte loads (a matrix-vector product per pair);
//   * many pairs in bfloat16: the pairs are sorted by expert on the device (no host round
//     trip), and tiles of 64 pairs x 64 outputs of one expert go through mma.sync m16n8k16 with
//     float32 accumulators (two stages of cp.async copies, fragments by ldmatrix); the down projection's rows are added into the stream per token in
//     the order the experts were chosen, so a token's result does not depend on its neighbours.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace hs {

// (value, index) argmax over a warp; larger value wins, then the lower index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// -- path 1: a matrix-vector product per pair ---------------------------------------------------
// dot of a weight row (n contiguous values) with a float32 vector in shared memory, over a warp
__device__ __forceinline__ float row_dot(const float* __restrict__ w, const float* v, int n,
                                         int lane) {
  float acc = 0.f;
  if ((n & 3) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int k = lane * 4; k < n; k += 128) {
      const float4 a = *(const float4*)(w + k);
      acc = fmaf(a.x, v[k], acc); acc = fmaf(a.y, v[k + 1], acc);
      acc = fmaf(a.z, v[k + 2], acc); acc = fmaf(a.w, v[k + 3], acc);
    }
  } else {
    for (int k = lane; k < n; k += 32) acc = fmaf(w[k], v[k], acc);
  }
  return warp_sum(acc);
}
__device__ __forceinline__ float row_dot(const __nv_bfloat16* __restrict__ w, const float* v,
                                         int n, int lane) {
  float acc = 0.f;
  if ((n & 7) == 0 && (((uintptr_t)w) & 15) == 0) {
    for (int k = lane * 8; k < n; k += 256) {
      const uint4 raw = *(const uint4*)(w + k);
      const __nv_bfloat162* p = (const __nv_bfloat162*)&raw;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        acc = fmaf(f.x, v[k + 2 * i], acc);
        acc = fmaf(f.y, v[k + 2 * i + 1], acc);
      }
    }
  } else {
    for (int k = lane; k < n; k += 32) acc = fmaf(__bfloat162float(w[k]), v[k], acc);
  }
  return warp_sum(acc);
}

constexpr int ROUTE_THREADS = 256;

// One block per token: the warps share the experts' dot products, warp 0 then chooses.
template <typename TH>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(int* __restrict__ sel_idx, float* __restrict__ sel_w, const TH* __restrict__ h,
                 const float* __restrict__ w_router, const int* __restrict__ tok_req, int width,
                 int E, int top, int n_groups, int keep, const float* __restrict__ z_in) {
  extern __shared__ float smem[];
  float* s_h = smem;                // [width]
  float* s_s = smem + width;        // [E] scores (-1 once taken)
  float* s_g = s_s + E;             // [n_groups] (-2 marks a kept group)
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (z_in) {                        // the logits were formed as one matrix product over the step
    for (int e = threadIdx.x; e < E; e += ROUTE_THREADS)
      s_s[e] = 1.0f / (1.0f + expf(-z_in[(size_t)t * E + e]));
  } else {
    for (int k = threadIdx.x; k < width; k += ROUTE_THREADS) s_h[k] = to_f(h[(size_t)t * width + k]);
    __syncthreads();
    for (int e = warp; e < E; e += ROUTE_THREADS / 32) {
      const float* wr = w_router + (size_t)e * width;
      const float z = row_dot(wr, s_h, width, lane);
      if (lane == 0) s_s[e] = 1.0f / (1.0f + expf(-z));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  const int per = E / n_groups;
  for (int g = lane; g < n_groups; g += 32) {
    float a = -1.f, b = -1.f;                          // the two largest of the group
    for (int j = 0; j < per; ++j) {
      const float v = s_s[g * per + j];
      if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
    }
    s_g[g] = per > 1 ? a + b : a;
  }
  __syncwarp();
  for (int round = 0; round < keep; ++round) {
    float bv = -1.f;
    int bi = 0x7fffffff;
    for (int g = lane; g < n_groups; g += 32)
      if (s_g[g] > bv) { bv = s_g[g]; bi = g; }
    warp_argmax(bv, bi);
    if (lane == 0) s_g[bi] = -2.f;
    __syncwarp();
  }
  float chosen_v = 0.f;                                // lane k keeps the k-th choice (top <= 32)
  int chosen_i = 0;
  float total = 0.f;
  for (int round = 0; round < top; ++round) {
    float bv = -1.f;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s_g[e / per] == -2.f ? s_s[e] : -1.f;
      if (v > bv) { bv = v; bi = e; }
    }
    warp_argmax(bv, bi);
    if (lane == round) { chosen_v = bv; chosen_i = bi; }
    total += bv;
    if (lane == 0) s_s[bi] = -1.f;                     // taken
    __syncwarp();
  }
  if (lane < top) {
    sel_idx[(size_t)t * top + lane] = chosen_i;
    sel_w[(size_t)t * top + lane] = chosen_v / (total + 1e-20f);
  }
}

// One block per token: z = W_r h + b (or handed in), the `top` largest, softmax over the chosen.
template <typename TH>
__global__ void __launch_bounds__(1024)
moe_route_top_kernel(int* __restrict__ sel_idx, float* __restrict__ sel_w,
                     const TH* __restrict__ h, const float* __restrict__ w_router,
                     const float* __restrict__ bias, const int* __restrict__ tok_req, int width,
                     int E, int top, const float* __restrict__ z_in) {
  extern __shared__ float smem[];
  float* s_h = smem;                // [width]
  float* s_z = smem + width;        // [E] logits (-inf once taken)
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (z_in) {
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      s_z[e] = z_in[(size_t)t * E + e] + (bias ? bias[e] : 0.f);
  } else {
    for (int k = threadIdx.x; k < width; k += blockDim.x) s_h[k] = to_f(h[(size_t)t * width + k]);
    __syncthreads();
    for (int e = warp; e < E; e += blockDim.x / 32) {
      const float z = row_dot(w_router + (size_t)e * width, s_h, width, lane);
      if (lane == 0) s_z[e] = z + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float chosen_v = -INFINITY;                          // lane k keeps the k-th choice (top <= 32)
  int chosen_i = 0;
  for (int round = 0; round < top; ++round) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s_z[e];
      if (v > bv || (bi == 0x7fffffff && v == v)) { bv = v; bi = e; }
    }
    warp_argmax(bv, bi);
    if (lane == round) { chosen_v = bv; chosen_i = bi; }
    if (lane == 0 && bi < E) s_z[bi] = -INFINITY;      // taken
    __syncwarp();
  }
  // softmax over the chosen logits: the first choice is the largest
  const float top_v = __shfl_sync(0xffffffffu, chosen_v, 0);
  const float ex = lane < top ? expf(chosen_v - top_v) : 0.f;
  float total = 0.f;
  for (int k = 0; k < top; ++k) total += __shfl_sync(0xffffffffu, ex, k);
  if (lane < top) {
    sel_idx[(size_t)t * top + lane] = chosen_i;
    sel_w[(size_t)t * top + lane] = ex / total;
  }
}

// act 0: the clamped form above; act 1: silu(g) * u; act 2: relu(u)^2 (an expert without a gate
// matrix)
__device__ __forceinline__ float expert_act(float g, float u, float limit, int act) {
  if (act == 1) return g / (1.0f + expf(-g)) * u;
  if (act == 2) { const float r = fmaxf(u, 0.f); return r * r; }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
}

// a matrix-vector product per pair: rows of the expert, one warp each
constexpr int GEMV_THREADS = 256;
constexpr int GEMV_ROWS = 32;       // output rows a block covers

// NS weight rows at once against one vector: the loads of all rows of a step over k are issued
// before any is used, so that a lane has NS 16-byte loads in flight.  Rows whose pointer is null
// give 0.  The per-row sum runs over k in the same order as row_dot's.
template <int NS>
__device__ __forceinline__ void rows_dot(float* res, const __nv_bfloat16* const* rows,
                                         const float* v, int n, int lane) {
  float acc[NS];
#pragma unroll
  for (int r = 0; r < NS; ++r) acc[r] = 0.f;
  bool vec = (n & 7) == 0;
#pragma unroll
  for (int r = 0; r < NS; ++r) vec = vec && (((uintptr_t)rows[r]) & 15) == 0;
  if (vec) {
    for (int k = lane * 8; k < n; k += 256) {
      uint4 raw[NS];
#pragma unroll
      for (int r = 0; r < NS; ++r)
        raw[r] = rows[r] ? *(const uint4*)(rows[r] + k) : make_uint4(0, 0, 0, 0);
      const float4 v0 = *(const float4*)(v + k), v1 = *(const float4*)(v + k + 4);
#pragma unroll
      for (int r = 0; r < NS; ++r) {
        const __nv_bfloat162* p = (const __nv_bfloat162*)&raw[r];
        float2 f = __bfloat1622float2(p[0]);
        acc[r] = fmaf(f.x, v0.x, acc[r]); acc[r] = fmaf(f.y, v0.y, acc[r]);
        f = __bfloat1622float2(p[1]);
        acc[r] = fmaf(f.x, v0.z, acc[r]); acc[r] = fmaf(f.y, v0.w, acc[r]);
        f = __bfloat1622float2(p[2]);
        acc[r] = fmaf(f.x, v1.x, acc[r]); acc[r] = fmaf(f.y, v1.y, acc[r]);
        f = __bfloat1622float2(p[3]);
        acc[r] = fmaf(f.x, v1.z, acc[r]); acc[r] = fmaf(f.y, v1.w, acc[r]);
      }
    }
  } else {
    for (int k = lane; k < n; k += 32)
#pragma unroll
      for (int r = 0; r < NS; ++r)
        if (rows[r]) acc[r] = fmaf(__bfloat162float(rows[r][k]), v[k], acc[r]);
  }
#pragma unroll
  for (int r = 0; r < NS; ++r) res[r] = warp_sum(acc[r]);
}
template <int NS>
__device__ __forceinline__ void rows_dot(float* res, const float* const* rows, const float* v,
                                         int n, int lane) {
#pragma unroll
  for (int r = 0; r < NS; ++r) res[r] = rows[r] ? row_dot(rows[r], v, n, lane) : 0.f;
}

template <typename TW>
__global__ void __launch_bounds__(GEMV_THREADS)
moe_gate_up_rows_kernel(float* __restrict__ y, const TW* __restrict__ h,
                        const TW* __restrict__ w_gate, const TW* __restrict__ w_up,
                        const int* __restrict__ sel_idx, const int* __restrict__ tok_req,
                        int width, int ff, int top, int E, float limit, int act) {
  extern __shared__ __align__(16) float s_h[];         // [width]
  const int pair = blockIdx.x;
  const int t = pair / top;
  if (tok_req[t] < 0) return;
  const int e = sel_idx[pair];
  if (e < 0 || e >= E) return;
  for (int k = threadIdx.x; k < width; k += GEMV_THREADS) s_h[k] = to_f(h[(size_t)t * width + k]);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int NW = GEMV_THREADS / 32, PER = GEMV_ROWS / NW;      // rows a warp: 4
  const int f0 = blockIdx.y * GEMV_ROWS + warp;
  const TW* rows[2 * PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int f = f0 + i * NW;
    const size_t row = ((size_t)e * ff + f) * width;
    rows[2 * i] = (f < ff && w_gate) ? w_gate + row : nullptr;
    rows[2 * i + 1] = f < ff ? w_up + row : nullptr;
  }
  float res[2 * PER];
  rows_dot<2 * PER>(res, rows, s_h, width, lane);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int f = f0 + i * NW;
    if (lane == 0 && f < ff) y[(size_t)pair * ff + f] = expert_act(res[2 * i], res[2 * i + 1], limit, act);
  }
}

constexpr int MAX_TOP_AT_ONCE = 8;

template <typename TW>
__global__ void __launch_bounds__(GEMV_THREADS)
moe_down_rows_kernel(float* __restrict__ x, const float* __restrict__ y,
                     const TW* __restrict__ w_down, const int* __restrict__ sel_idx,
                     const float* __restrict__ sel_w, const int* __restrict__ tok_req, int width,
                     int ff, int top, int E) {
  extern __shared__ __align__(16) float s_y[];         // [top][ff4]: rows padded to 16 bytes
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int ff4 = (ff + 3) & ~3;
  for (int i = threadIdx.x; i < top * ff4; i += GEMV_THREADS) {
    const int k = i / ff4, f = i - k * ff4;
    s_y[i] = f < ff ? y[((size_t)t * top + k) * ff + f] : 0.f;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_end = min(width, (int)(blockIdx.y + 1) * GEMV_ROWS);
  for (int n = blockIdx.y * GEMV_ROWS + warp; n < n_end; n += GEMV_THREADS / 32) {
    float sum = 0.f;
    for (int k0 = 0; k0 < top; k0 += MAX_TOP_AT_ONCE) {
      // the rows of up to eight chosen experts for this output, fetched together; each is
      // summed against its own activations, then weighted, in the order of the choice
      float acc[MAX_TOP_AT_ONCE];
      if (sizeof(TW) == 2 && (ff & 7) == 0) {
        const TW* rows[MAX_TOP_AT_ONCE];
#pragma unroll
        for (int i = 0; i < MAX_TOP_AT_ONCE; ++i) {
          const int e = k0 + i < top ? sel_idx[(size_t)t * top + k0 + i] : -1;
          rows[i] = (e >= 0 && e < E) ? w_down + ((size_t)e * width + n) * ff : nullptr;
          acc[i] = 0.f;
        }
        for (int k = lane * 8; k < ff; k += 256) {
          uint4 raw[MAX_TOP_AT_ONCE];
#pragma unroll
          for (int i = 0; i < MAX_TOP_AT_ONCE; ++i)
            raw[i] = rows[i] ? *(const uint4*)((const __nv_bfloat16*)rows[i] + k)
                             : make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int i = 0; i < MAX_TOP_AT_ONCE; ++i) {
            if (!rows[i]) continue;
            const float* v = s_y + (size_t)(k0 + i) * ff4 + k;
            const __nv_bfloat162* p = (const __nv_bfloat162*)&raw[i];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 f = __bfloat1622float2(p[q]);
              acc[i] = fmaf(f.x, v[2 * q], acc[i]);
              acc[i] = fmaf(f.y, v[2 * q + 1], acc[i]);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < MAX_TOP_AT_ONCE; ++i) acc[i] = warp_sum(acc[i]);
      } else {
#pragma unroll
        for (int i = 0; i < MAX_TOP_AT_ONCE; ++i) {
          const int e = k0 + i < top ? sel_idx[(size_t)t * top + k0 + i] : -1;
          acc[i] = (e >= 0 && e < E)
                       ? row_dot(w_down + ((size_t)e * width + n) * ff,
                                 s_y + (size_t)(k0 + i) * ff4, ff, lane)
                       : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < MAX_TOP_AT_ONCE; ++i)
        if (k0 + i < top) sum = fmaf(sel_w[(size_t)t * top + k0 + i], acc[i], sum);
    }
    if (lane == 0) x[(size_t)t * width + n] += sum;
  }
}

// -- path 2: pairs sorted by expert, tiles on the tensor cores --------------------------------
constexpr int SORT_THREADS = 1024;

// work: [0] number of tiles; then per expert E counts, E segment starts; then per tile its
// expert and its first row.  pair_pos[pair] = row of the pair in expert order (-1: not there),
// row_token[row] = the token of that row.
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(int* __restrict__ work, int* __restrict__ pair_pos, int* __restrict__ row_token,
                const int* __restrict__ sel_idx, const int* __restrict__ tok_req, int n_tokens,
                int top, int E, int max_tiles) {
  extern __shared__ int s_cnt[];             // [E] counts, then [E] cursors
  int* s_cur = s_cnt + E;
  for (int e = threadIdx.x; e < E; e += SORT_THREADS) s_cnt[e] = 0;
  __syncthreads();
  const int pairs = n_tokens * top;
  for (int p = threadIdx.x; p < pairs; p += SORT_THREADS) {
    const int e = sel_idx[p];
    if (tok_req[p / top] >= 0 && e >= 0 && e < E) atomicAdd(&s_cnt[e], 1);
  }
  __syncthreads();
  int* counts = work + 1;
  int* starts = work + 1 + E;
  int* tile_e = work + 1 + 2 * E;
  int* tile_r = tile_e + max_tiles;
  if (threadIdx.x == 0) {
    int at = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      counts[e] = s_cnt[e];
      starts[e] = at;
      s_cur[e] = at;
      for (int r = 0; r < s_cnt[e] && tiles < max_tiles; r += TM) {
        tile_e[tiles] = e;
        tile_r[tiles] = at + r;
        ++tiles;
      }
      at += s_cnt[e];
    }
    work[0] = tiles;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += SORT_THREADS) {
    const int e = sel_idx[p];
    int pos = -1;
    if (tok_req[p / top] >= 0 && e >= 0 && e < E) {
      pos = atomicAdd(&s_cur[e], 1);
      row_token[pos] = p / top;
    }
    pair_pos[p] = pos;
  }
}

// One block: 64 rows of one expert's segment x 64 outputs.  NB = 2: gate and up together with
// the activation as epilogue (out: bfloat16 rows); NB = 1: the down projection (out: float32).
// A rows: `a` indexed through row_token when GATHER (the normed rows of the tokens), else the
// sorted rows themselves.  4 warps, each 32 x 32 of the tile.  Two stages of tiles in shared
// memory (the next one is copied while this one is used); fragments come through ldmatrix.
// ACT (with NB = 1): the rows leave activated in bfloat16 as with NB = 2 (an expert without a gate).
template <int NB, bool GATHER, bool ACT = (NB == 2)>
__global__ void __launch_bounds__(128)
moe_tiles_kernel(void* __restrict__ out, const __nv_bfloat16* __restrict__ a,
                 const __nv_bfloat16* __restrict__ w0, const __nv_bfloat16* __restrict__ w1,
                 const int* __restrict__ work, const int* __restrict__ row_token, int E,
                 int max_tiles, int N, int K, float limit, int act) {
  __shared__ __align__(16) __nv_bfloat16 s_a[2][TM * TS];
  __shared__ __align__(16) __nv_bfloat16 s_b[NB][2][TN * TS];
  const int tile = blockIdx.x;
  if (tile >= work[0]) return;
  const int e = work[1 + 2 * E + tile];
  const int row0 = work[1 + 2 * E + max_tiles + tile];
  const int seg_end = work[1 + E + e] + work[1 + e];
  const int rows = min(TM, seg_end - row0);
  const int n0 = blockIdx.y * TN;
  const int ncols = min(TN, N - n0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int g = lane >> 2, tq = lane & 3;
  auto a_row = [&](int r) {
    const int src = GATHER ? row_token[row0 + r] : row0 + r;
    return a + (size_t)src * K;
  };
  const __nv_bfloat16* b0 = w0 + ((size_t)e * N + n0) * K;
  const __nv_bfloat16* b1 = NB == 2 ? w1 + ((size_t)e * N + n0) * K : nullptr;
  auto b0_row = [&](int r) { return b0 + (size_t)r * K; };
  auto b1_row = [&](int r) { return b1 + (size_t)r * K; };
  float acc[NB][2][4][4];
#pragma unroll
  for (int x = 0; x < NB; ++x)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[x][i][j][c] = 0.f;
  auto copy = [&](int buf, int k0) {
    tile_copy(s_a[buf], a_row, rows, k0, a);
    tile_copy(s_b[0][buf], b0_row, ncols, k0, w0);
    if (NB == 2) tile_copy(s_b[NB - 1][buf], b1_row, ncols, k0, w0);
    asm volatile("cp.async.commit_group;");
  };
  copy(0, 0);
  int buf = 0;
  // lane's row and column offsets inside a 16 x 16 (A) or two 8 x 16 (B) block for ldmatrix
  const int a_r = lane & 15, a_c = (lane >> 4) * 8;
  const int b_r = (lane & 7) + (lane >> 4) * 8, b_c = ((lane >> 3) & 1) * 8;
  for (int k0 = 0; k0 < K; k0 += TK, buf ^= 1) {
    if (k0 + TK < K) {
      copy(buf ^ 1, k0 + TK);
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t fa[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(fa[i], s_a[buf] + (wm + 16 * i + a_r) * TS + kk + a_c);
#pragma unroll
      for (int x = 0; x < NB; ++x)
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          uint32_t fb[4];                         // b0, b1 of column block j, then of j + 1
          ldmatrix_x4(fb, s_b[x][buf] + (wn + 8 * j + b_r) * TS + kk + b_c);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            mma_bf16(acc[x][i][j], fa[i], fb);
            mma_bf16(acc[x][i][j + 1], fa[i], fb + 2);
          }
        }
    }
    __syncthreads();                              // this stage is copied into again next turn
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = wm + 16 * i + g + 8 * half;
        const int c = wn + 8 * j + 2 * tq;
        if (r >= rows) continue;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (c + q >= ncols) continue;
          const size_t at = (size_t)(row0 + r) * N + n0 + c + q;
          if (ACT)
            ((__nv_bfloat16*)out)[at] = __float2bfloat16_rn(
                expert_act(acc[0][i][j][2 * half + q], acc[NB - 1][i][j][2 * half + q], limit, act));
          else
            ((float*)out)[at] = acc[0][i][j][2 * half + q];
        }
      }
}

// x[t] += sum_k weight_k * rows[pair_pos[t, k]], experts in the order they were chosen
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ rows,
                                   const int* __restrict__ pair_pos,
                                   const float* __restrict__ sel_w,
                                   const int* __restrict__ tok_req, int width, int top) {
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  for (int n = threadIdx.x; n < width; n += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) {
      const int pos = pair_pos[(size_t)t * top + k];
      if (pos >= 0) sum = fmaf(sel_w[(size_t)t * top + k], rows[(size_t)pos * width + n], sum);
    }
    x[(size_t)t * width + n] += sum;
  }
}

}  // namespace hs

HS_EXPORT int hs_moe_route(int* sel_idx, float* sel_w, const void* h, const float* w_router,
                           const int* tok_req, int n_tokens, int width, int E, int top,
                           int n_groups, int keep, int h_dtype, const float* z_in, void* stream) {
  if (!sel_idx || !sel_w || !h || !w_router || !tok_req) return HS_ERR_ARGUMENT;
  if (E <= 0 || top <= 0 || top > 32 || n_groups <= 0 || E % n_groups || keep <= 0 ||
      keep > n_groups || top > keep * (E / n_groups))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)(width + E + n_groups) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (h_dtype == HS_DT_F32)
    hs::moe_route_kernel<float><<<n_tokens, hs::ROUTE_THREADS, smem, st>>>(
        sel_idx, sel_w, (const float*)h, w_router, tok_req, width, E, top, n_groups, keep, z_in);
  else if (h_dtype == HS_DT_BF16)
    hs::moe_route_kernel<__nv_bfloat16><<<n_tokens, hs::ROUTE_THREADS, smem, st>>>(
        sel_idx, sel_w, (const __nv_bfloat16*)h, w_router, tok_req, width, E, top, n_groups,
        keep, z_in);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_moe_route_top(int* sel_idx, float* sel_w, const void* h, const float* w_router,
                               const float* bias, const int* tok_req, int n_tokens, int width,
                               int E, int top, int h_dtype, const float* z_in, void* stream) {
  if (!sel_idx || !sel_w || !h || !w_router || !tok_req) return HS_ERR_ARGUMENT;
  if (E <= 0 || top <= 0 || top > 32 || top > E) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)(width + E) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  int threads = 32 * E;
  threads = threads < 128 ? 128 : (threads > 1024 ? 1024 : threads);
  if (h_dtype == HS_DT_F32)
    e = hs_launch(hs::moe_route_top_kernel<float>, dim3(n_tokens), dim3(threads), smem,
                  st, hs_pdl_enabled(), sel_idx, sel_w, (const float*)h, w_router, bias, tok_req,
                  width, E, top, z_in);
  else if (h_dtype == HS_DT_BF16)
    e = hs_launch(hs::moe_route_top_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem, st, hs_pdl_enabled(), sel_idx, sel_w,
                  (const __nv_bfloat16*)h, w_router, bias, tok_req, width, E, top, z_in);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

// Scratch of the sorted path for n_tokens x top pairs: ints (work lists, pair positions, row
// tokens) and bytes of rows (bfloat16 activations, then float32 outputs of the down projection).
// Returns 0 and zeros when the sorted path does not take the shape.
namespace hs {
// the experts of a token id stand in a table [rows, top]; each weighs 1/top
__global__ void moe_route_table_kernel(int* __restrict__ sel_idx, float* __restrict__ sel_w,
                                       const int* __restrict__ table, int rows,
                                       const int* __restrict__ tok_ids,
                                       const int* __restrict__ tok_req,
                                       const int* __restrict__ feedback, int n_feedback,
                                       int n_tokens, int top, int E, int* __restrict__ status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * top) return;
  const int t = i / top, k = i - t * top;
  if (tok_req[t] < 0) return;
  int id = tok_ids[t];
  if (id < 0 && feedback != nullptr && -(id + 1) < n_feedback) id = feedback[-(id + 1)];
  int e = -1;
  if (id >= 0 && id < rows) e = table[(size_t)id * top + k];
  if (e < 0 || e >= E) {
    atomicOr(status, HS_STATUS_BAD_TOKEN);
    e = -1;                                   // the expert kernels skip such a pair
  }
  sel_idx[i] = e;
  sel_w[i] = 1.0f / (float)top;
}
}  // namespace hs

HS_EXPORT int hs_moe_route_table(int* sel_idx, float* sel_w, const int* table, int rows,
                                 const int* tok_ids, const int* tok_req, const int* feedback,
                                 int n_feedback, int n_tokens, int top, int E, int* status,
                                 void* stream) {
  if (!sel_idx || !sel_w || !table || !tok_ids || !tok_req || !status) return HS_ERR_ARGUMENT;
  if (rows <= 0 || top <= 0 || E <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const int n = n_tokens * top;
  hs::moe_route_table_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      sel_idx, sel_w, table, rows, tok_ids, tok_req, feedback, n_feedback, n_tokens, top, E,
      status);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_moe_sorted_scratch(int n_tokens, int width, int ff, int top, int E, int dtype,
                                    long long* ints, long long* bytes) {
  *ints = 0;
  *bytes = 0;
  const long long pairs = (long long)n_tokens * top;
  if (dtype != HS_DT_BF16 || width % hs::TK || ff % hs::TK || pairs < 256 || E > 4096)
    return HS_OK;
  const long long max_tiles = pairs / hs::TM + E;
  *ints = 1 + 2LL * E + 2 * max_tiles + 2 * pairs;
  *bytes = ((pairs * ff * 2 + 255) / 256) * 256 + pairs * width * 4;
  return HS_OK;
}

// `y`: float32 scratch [pairs, ff] of the row path.  `ints` / `rows`: scratch of the sorted path
// (sized by hs_moe_sorted_scratch; null to use the row path).
HS_EXPORT int hs_moe_experts(float* x, float* y, const void* h, const void* w_gate,
                             const void* w_up, const void* w_down, const int* sel_idx,
                             const float* sel_w, const int* tok_req, int n_tokens, int width,
                             int ff, int top, int E, float limit, int act_kind, int dtype, int* ints,
                             void* rows, void* stream) {
  if (!x || !h || !w_up || !w_down || !sel_idx || !sel_w || !tok_req || (!w_gate && act_kind != 2))
    return HS_ERR_ARGUMENT;
  if (width <= 0 || ff <= 0 || top <= 0 || E <= 0 || act_kind < 0 || act_kind > 2) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (ints && rows) {
    long long need_i = 0, need_b = 0;
    hs_moe_sorted_scratch(n_tokens, width, ff, top, E, dtype, &need_i, &need_b);
    if (need_i == 0) return HS_ERR_UNSUPPORTED;
    const int pairs = n_tokens * top;
    const int max_tiles = pairs / hs::TM + E;
    int* work = ints;
    int* pair_pos = ints + 1 + 2 * E + 2 * max_tiles;
    int* row_token = pair_pos + pairs;
    __nv_bfloat16* act = (__nv_bfloat16*)rows;
    float* down = (float*)((char*)rows + (((size_t)pairs * ff * 2 + 255) / 256) * 256);
    hs::moe_sort_kernel<<<1, hs::SORT_THREADS, 2 * E * sizeof(int), st>>>(
        work, pair_pos, row_token, sel_idx, tok_req, n_tokens, top, E, max_tiles);
    HS_LAUNCH_CHECK();
    const __nv_bfloat16* hb = (const __nv_bfloat16*)h;
    if (w_gate)
      hs::moe_tiles_kernel<2, true><<<dim3(max_tiles, (ff + hs::TN - 1) / hs::TN), 128, 0, st>>>(
          act, hb, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, work, row_token, E,
          max_tiles, ff, width, limit, act_kind);
    else
      hs::moe_tiles_kernel<1, true, true><<<dim3(max_tiles, (ff + hs::TN - 1) / hs::TN), 128, 0, st>>>(
          act, hb, (const __nv_bfloat16*)w_up, nullptr, work, row_token, E, max_tiles, ff, width,
          limit, act_kind);
    HS_LAUNCH_CHECK();
    hs::moe_tiles_kernel<1, false><<<dim3(max_tiles, (width + hs::TN - 1) / hs::TN), 128, 0, st>>>(
        down, act, (const __nv_bfloat16*)w_down, nullptr, work, row_token, E, max_tiles, width,
        ff, limit, act_kind);
    HS_LAUNCH_CHECK();
    hs::moe_combine_kernel<<<n_tokens, 256, 0, st>>>(x, down, pair_pos, sel_w, tok_req, width,
                                                     top);
    HS_LAUNCH_CHECK();
    return HS_OK;
  }
  if (!y) return HS_ERR_ARGUMENT;
  const size_t smem_h = (size_t)width * sizeof(float);
  const size_t smem_y = (size_t)top * ((ff + 3) & ~3) * sizeof(float);
  if (smem_h > 200 * 1024 || smem_y > 200 * 1024) return HS_ERR_UNSUPPORTED;
  dim3 g1(n_tokens * top, (ff + hs::GEMV_ROWS - 1) / hs::GEMV_ROWS);
  dim3 g2(n_tokens, (width + hs::GEMV_ROWS - 1) / hs::GEMV_ROWS);
#define HS_MOE(TW)                                                                             \
  do {                                                                                         \
    auto k1 = hs::moe_gate_up_rows_kernel<TW>;                                                 \
    auto k2 = hs::moe_down_rows_kernel<TW>;                                                    \
    if (smem_h > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_h);      \
    if (smem_y > 48 * 1024)                                                                    \
      cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_y);      \
    k1<<<g1, hs::GEMV_THREADS, smem_h, st>>>(y, (const TW*)h, (const TW*)w_gate,               \
                                             (const TW*)w_up, sel_idx, tok_req, width, ff,     \
                                             top, E, limit, act_kind);                         \
    HS_LAUNCH_CHECK();                                                                         \
    k2<<<g2, hs::GEMV_THREADS, smem_y, st>>>(x, y, (const TW*)w_down, sel_idx, sel_w, tok_req, \
                                             width, ff, top, E);                               \
  } while (0)
  if (dtype == HS_DT_F32) HS_MOE(float);
  else if (dtype == HS_DT_BF16) HS_MOE(__nv_bfloat16);
  else return HS_ERR_UNSUPPORTED;
#undef HS_MOE
  HS_LAUNCH_CHECK();
  return HS_OK;
}
