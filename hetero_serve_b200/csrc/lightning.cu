// Linear attention with a constant decay per head (lightning attention), as a recurrence on a
// float32 state S [dim, vdim] per head and request:
//
//     q, k, v = act(projection columns)        act = silu, applied here in float32
//     S <- decay_h * S + k v^T ;   o = S^T q    token after token
//
// The state lives in the request's state slot ([heads, dim, vdim] floats) and is carried from
// step to step.  One block per (request, head, group of value columns): a thread keeps 16 rows
// of one column of S in registers, the P = ceil(dim / 16) (rounded up to a power of two) parts
// of a column are neighbouring lanes of one warp and fold their shares of o by a butterfly.
// The tokens' rows are staged through shared memory 16 tokens at a time, two buffers in turn:
// for steps of many tokens the activations are applied by a pass of their own into compact rows
// and the recurrence fetches the next portion by cp.async while it walks the current one.  A
// token's arithmetic is the same chain whatever the batch or the cut of the prompt: results are
// bit-equal across both.
//
// Retention is the same recurrence with q and k turned by the token's position on their first
// rot_dims numbers (number i pairs with i + rot_dims/2) and k scaled: with a table of
// frequencies the rows are turned where they are activated (in the pass of its own, or while
// they are staged), by the same expression in both places.
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

constexpr int LA_THREADS = 128;
constexpr int LA_ROWS = 16;          // state rows a thread keeps
constexpr int LA_PART = LA_ROWS + 4; // floats between two parts' rows of a token in shared memory:
                                     // the parts of a column read 16-byte pieces from distinct banks
constexpr int LA_TOK = 16;           // tokens staged at a time (8 when dim is above 128)

__device__ __forceinline__ float la_act(float z, int act) {
  return act == HS_ACT_SILU ? z / (1.0f + expf(-z)) : z;
}
// entry d of a head's q or k vector `vec`: activated, turned by position `pos` when d lies in the
// first rot_dims numbers (rot_dims 0: never), times `mul`
__device__ __forceinline__ float la_entry(const float* __restrict__ vec, int d, int act,
                                          int rot_dims, const float* __restrict__ freq, int pos,
                                          float mul) {
  float own = la_act(vec[d], act);
  if (d < rot_dims) {
    const int half = rot_dims >> 1;
    const bool low = d < half;
    const float partner = la_act(vec[low ? d + half : d - half], act);
    float c, sn;
    pair_angle(pos, freq[low ? d : d - half], &c, &sn);
    const float cross = __fmul_rn(partner, sn);
    own = fmaf(own, c, low ? -cross : cross);
  }
  return __fmul_rn(own, mul);
}
__device__ __forceinline__ void la_cp16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
               : "memory");
}

// dst[t, :] = act(q | k | v columns of proj[t]) as one compact row of 2 H D + H V floats
__global__ void lightning_act_kernel(float* __restrict__ dst, const float* __restrict__ proj,
                                     int n_tokens, int stride, int q_off, int k_off, int v_off,
                                     int hd, int hv, int act, int D,
                                     const int* __restrict__ tok_pos,
                                     const float* __restrict__ freq, int rot_dims,
                                     float k_scale) {
  pdl_trigger();
  pdl_wait();
  const int row_len = 2 * hd + hv;
  for (int t = blockIdx.x; t < n_tokens; t += gridDim.x) {
    const float* row = proj + (size_t)t * stride;
    float* out = dst + (size_t)t * row_len;
    const int pos = rot_dims > 0 ? tok_pos[t] : 0;
    for (int c = threadIdx.x; c < row_len; c += blockDim.x) {
      if (c < 2 * hd) {
        const bool is_q = c < hd;
        const int e = is_q ? c : c - hd, d = e % D;
        out[c] = la_entry(row + (is_q ? q_off : k_off) + (e - d), d, act, rot_dims, freq, pos,
                          is_q ? 1.0f : k_scale);
      } else {
        out[c] = la_act(row[v_off + c - 2 * hd], act);
      }
    }
  }
}

// One token on a thread's 16 state rows: s <- decay s + k v, and the thread's share of o = S^T q
// as four partial sums folded pairwise (the same order wherever the token stands).
__device__ __forceinline__ float la_token(float (&s)[LA_ROWS], const float* kp, const float* qp,
                                          float vt, float dh) {
  float part_sum[LA_ROWS / 4];
#pragma unroll
  for (int i4 = 0; i4 < LA_ROWS / 4; ++i4) {
    const float4 k4 = *(const float4*)(kp + 4 * i4), q4 = *(const float4*)(qp + 4 * i4);
    s[4 * i4 + 0] = fmaf(k4.x, vt, dh * s[4 * i4 + 0]);
    s[4 * i4 + 1] = fmaf(k4.y, vt, dh * s[4 * i4 + 1]);
    s[4 * i4 + 2] = fmaf(k4.z, vt, dh * s[4 * i4 + 2]);
    s[4 * i4 + 3] = fmaf(k4.w, vt, dh * s[4 * i4 + 3]);
    float a = s[4 * i4 + 0] * q4.x;
    a = fmaf(s[4 * i4 + 1], q4.y, a);
    a = fmaf(s[4 * i4 + 2], q4.z, a);
    part_sum[i4] = fmaf(s[4 * i4 + 3], q4.w, a);
  }
  return (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
}

// A portion of up to ntok tokens of request rows (from token `tok` on) into one buffer (q [ntok][Dp],
// k [ntok][Dp], v [ntok][cols]).  `bulk`: the rows are activated already and 16-byte aligned,
// and go in by cp.async (the walk over the portion before runs meanwhile); otherwise plain loads
// with the activation applied on the way.
__device__ __forceinline__ void la_stage(float* s_q, const float* __restrict__ proj, int tok,
                                         int here, int stride, int q_off, int k_off, int v_off,
                                         int h, int D, int V, int Dp, int cols, int v0, int ntok,
                                         int act, int bulk, const int* __restrict__ tok_pos,
                                         const float* __restrict__ freq, int rot_dims,
                                         float k_scale) {
  float* s_k = s_q + ntok * Dp;
  float* s_v = s_k + ntok * Dp;
  if (bulk) {
    const int dq = D / 4, cq = cols / 4;
    for (int e = threadIdx.x; e < here * dq; e += LA_THREADS) {
      const int tt = e / dq, c = e - tt * dq;
      const float* row = proj + (size_t)(tok + tt) * stride + (size_t)h * D + 4 * c;
      const int at = tt * Dp + (4 * c) / LA_ROWS * LA_PART + (4 * c) % LA_ROWS;
      la_cp16(s_q + at, row + q_off);
      la_cp16(s_k + at, row + k_off);
    }
    for (int e = threadIdx.x; e < here * cq; e += LA_THREADS) {
      const int tt = e / cq, c = e - tt * cq;
      if (v0 + 4 * c < V)
        la_cp16(s_v + tt * cols + 4 * c,
                proj + (size_t)(tok + tt) * stride + v_off + (size_t)h * V + v0 + 4 * c);
    }
  } else {
#pragma unroll 4
    for (int e = threadIdx.x; e < here * D; e += LA_THREADS) {
      const int tt = e / D, d = e - tt * D;
      const float* row = proj + (size_t)(tok + tt) * stride + (size_t)h * D;
      const int at = tt * Dp + d / LA_ROWS * LA_PART + d % LA_ROWS;
      const int pos = rot_dims > 0 ? tok_pos[tok + tt] : 0;
      s_q[at] = la_entry(row + q_off, d, act, rot_dims, freq, pos, 1.0f);
      s_k[at] = la_entry(row + k_off, d, act, rot_dims, freq, pos, k_scale);
    }
    for (int e = threadIdx.x; e < here * cols; e += LA_THREADS) {
      const int tt = e / cols, c = e - tt * cols;
      if (v0 + c < V)
        s_v[e] = la_act(proj[(size_t)(tok + tt) * stride + v_off + (size_t)h * V + v0 + c], act);
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(LA_THREADS, 1)
lightning_kernel(float* __restrict__ o, float* __restrict__ state, const float* __restrict__ proj,
                 const float* __restrict__ decay, const int* __restrict__ req_start,
                 const int* __restrict__ req_len, const int* __restrict__ req_slot, int stride,
                 int q_off, int k_off, int v_off, int H, int D, int V, int P, int act, int ntok,
                 int bulk, const int* __restrict__ tok_pos, const float* __restrict__ freq,
                 int rot_dims, float k_scale) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int Dp = P * LA_PART;                       // a token's q (or k) row: P parts, padded
  const int cols = LA_THREADS / P;                  // value columns of this block
  const int per_buf = ntok * (2 * Dp + cols);       // a buffer: q [ntok][Dp], k [ntok][Dp], v [ntok][cols]
  const int r = blockIdx.z, h = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int t0 = req_start[r];
  const int slot = req_slot[r];
  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int v0 = blockIdx.x * cols;
  const int v = v0 + col;
  const bool col_ok = v < V;
  const float dh = decay[h];
  float* S = state + ((size_t)slot * H + h) * D * V;
  float s[LA_ROWS];
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    s[i] = (col_ok && d < D) ? S[(size_t)d * V + v] : 0.f;
  }
  if (D != P * LA_ROWS || V % cols) {               // rows or columns past the sizes read as zero
    for (int e = threadIdx.x; e < 2 * per_buf; e += LA_THREADS) smem[e] = 0.f;
    __syncthreads();
  }
  la_stage(smem, proj, t0, min(ntok, n), stride, q_off, k_off, v_off, h, D, V, Dp, cols, v0, ntok,
           act, bulk, tok_pos, freq, rot_dims, k_scale);
  int buf = 0;
  for (int base = 0; base < n; base += ntok, buf ^= 1) {
    const int here = min(ntok, n - base);
    if (base + ntok < n) {
      la_stage(smem + (buf ^ 1) * per_buf, proj, t0 + base + ntok, min(ntok, n - base - ntok), stride,
               q_off, k_off, v_off, h, D, V, Dp, cols, v0, ntok, act, bulk, tok_pos, freq, rot_dims,
               k_scale);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* s_q = smem + buf * per_buf;
    const float* s_k = s_q + ntok * Dp;
    const float* s_v = s_k + ntok * Dp;
    int tt = 0;
    for (; tt + 4 <= here; tt += 4) {               // four tokens: their sums and folds overlap
      float acc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        acc[u] = la_token(s, s_k + (tt + u) * Dp + part * LA_PART,
                          s_q + (tt + u) * Dp + part * LA_PART, s_v[(tt + u) * cols + col], dh);
      for (int off = 1; off < P; off <<= 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], off);
      }
      if (part == 0 && col_ok) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          o[(size_t)(t0 + base + tt + u) * H * V + (size_t)h * V + v] = acc[u];
      }
    }
    for (; tt < here; ++tt) {
      float acc = la_token(s, s_k + tt * Dp + part * LA_PART, s_q + tt * Dp + part * LA_PART,
                           s_v[tt * cols + col], dh);
      for (int off = 1; off < P; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col_ok) o[(size_t)(t0 + base + tt) * H * V + (size_t)h * V + v] = acc;
    }
    __syncthreads();                                // this buffer is staged into again next turn
  }
#pragma unroll
  for (int i = 0; i < LA_ROWS; ++i) {
    const int d = part * LA_ROWS + i;
    if (col_ok && d < D) S[(size_t)d * V + v] = s[i];
  }
}

}  // namespace hs

// proj: float32 rows of `stride` columns holding q (H*D at q_off), k (H*D at k_off) and v (H*V at
// v_off), head by head; o: float32 [tokens, H*V]; state: [slots, H*D*V] float32.  `scratch`
// (n_tokens * (2 H D + H V) floats, or null): with it the activations are applied in a pass of
// their own and the recurrence streams the activated rows; the results are the same bits.
HS_EXPORT int hs_lightning_recurrence(float* o, float* state, const float* proj,
                                      const float* decay, const int* req_start,
                                      const int* req_len, const int* req_slot, int n_requests,
                                      int n_tokens, int stride, int q_off, int k_off, int v_off,
                                      int H, int D, int V, int act, float* scratch,
                                      const int* tok_pos, const float* freq, int rot_dims,
                                      float k_scale, void* stream) {
  if (!o || !state || !proj || !decay || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > D || (rot_dims > 0 && (!freq || !tok_pos)))
    return HS_ERR_ARGUMENT;
  if (H <= 0 || D <= 0 || V <= 0 || D > 16 * hs::LA_ROWS || (act != HS_ACT_NONE && act != HS_ACT_SILU))
    return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0 || n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int P = 1;
  while (P * hs::LA_ROWS < D) P *= 2;
  const int cols = hs::LA_THREADS / P;
  const int ntok = P * hs::LA_ROWS > 128 ? hs::LA_TOK / 2 : hs::LA_TOK;   // at most 45 KB
  int bulk = 0;
  if (scratch && D % 4 == 0 && V % 4 == 0 && (((uintptr_t)scratch) & 15) == 0) {
    const int hd = H * D, hv = H * V;
    int blocks = n_tokens < 148 * 8 ? n_tokens : 148 * 8;
    cudaError_t e = hs_launch(hs::lightning_act_kernel, dim3(blocks), dim3(256), 0, st,
                              hs_pdl_enabled(), scratch, proj, n_tokens, stride, q_off, k_off,
                              v_off, hd, hv, act, D, tok_pos, freq, rot_dims, k_scale);
    if (e != cudaSuccess) return (int)e;
    proj = scratch;
    stride = 2 * hd + hv;
    q_off = 0; k_off = hd; v_off = 2 * hd;
    act = HS_ACT_NONE;
    rot_dims = 0;           // the rows are turned and scaled already
    k_scale = 1.0f;
    bulk = 1;
  }
  const size_t smem = (size_t)2 * ntok * (2 * P * hs::LA_PART + cols) * sizeof(float);
  dim3 grid((V + cols - 1) / cols, H, n_requests);
  cudaError_t e = hs_launch(hs::lightning_kernel, grid, dim3(hs::LA_THREADS), smem, st,
                            hs_pdl_enabled(), o, state, proj, decay, req_start, req_len, req_slot,
                            stride, q_off, k_off, v_off, H, D, V, P, act, ntok, bulk, tok_pos, freq,
                            rot_dims, k_scale);
  if (e != cudaSuccess) return (int)e;
  return HS_OK;
}
