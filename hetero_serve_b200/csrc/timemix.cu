// Time mixing with a decay per token, head and key channel, and the small launches around
// recurrent mixers that norm each head's output.
//
//   token_shift_mix    out[s][t] = x[t] + (x'[t] - x[t]) * mu[s] for every stream s, with x' the
//                      row before (the slot's kept row for a request's first row of the step);
//                      the block of a request's first row also keeps the step's last row
//   timemix_decay      w = exp(-exp(W2 tanh(low) + w0)), float32, W2 handed in transposed
//   timemix_recurrence per (request, head, group of value columns), token after token on the
//                      float32 state S [dim, dim] of the request's slot:
//                          o = (S + diag(u) k v^T)^T r ;   S <- diag(w) S + k v^T
//                      a thread keeps 16 rows of one column of S in registers, the parts of a
//                      column are neighbouring lanes of one warp and fold their shares of o by a
//                      butterfly; the tokens' rows come through two shared-memory buffers of 16
//                      tokens, the next one by cp.async while the current one is walked
//   head_norm_gate     out = o / rms(o) per head (* weight) * silu or sigmoid(gate) * scale,
//                      rounded once
//   gather_mul         out[t] = g[t] * table[token[t]][offset : offset + dim]
//
// A token's arithmetic is the same chain whatever the batch or the cut of the prompt: results
// are bit-equal across both.
#include "common.cuh"

namespace hs {

// the token of row t: a negative id -(s + 1) stands for feedback[s]
__device__ __forceinline__ int resolve_token(const int* __restrict__ ids, int t,
                                             const int* __restrict__ feedback, int n_feedback) {
  int id = ids[t];
  if (id < 0 && feedback != nullptr && -(id + 1) < n_feedback) id = feedback[-(id + 1)];
  return id;
}

// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
token_shift_mix_kernel(T* __restrict__ out, const T* __restrict__ x, const float* __restrict__ mu,
                       float* __restrict__ state, int state_stride, int state_offset,
                       const int* __restrict__ tok_req, const int* __restrict__ req_start,
                       const int* __restrict__ req_len, const int* __restrict__ req_slot,
                       int n_tokens, int width, int n_streams) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int t0 = req_start[r];
  const bool first = t == t0;
  float* kept = state + (size_t)req_slot[r] * state_stride + state_offset;
  const T* cur = x + (size_t)t * width;
  const T* before = x + (size_t)(t - 1) * width;
  const T* last = x + (size_t)(t0 + req_len[r] - 1) * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float a = to_f(cur[c]);
    const float p = first ? kept[c] : to_f(before[c]);
    const float d = p - a;
    for (int s = 0; s < n_streams; ++s)
      out[((size_t)s * n_tokens + t) * width + c] = from_f<T>(fmaf(d, mu[(size_t)s * width + c], a));
    // only this block reads the kept row, and it has read entry c: the step's last row goes in
    if (first) kept[c] = to_f(last[c]);
  }
}

// w2t is the second matrix transposed, [rank][channels]: the threads of a block read a row of it
// side by side, once for DK_TOK tokens.  Every (token, channel) sum runs over the inner index in
// order, whatever the batch.
constexpr int DK_TOK = 8;
__global__ void __launch_bounds__(256)
timemix_decay_kernel(float* __restrict__ out, const float* __restrict__ low,
                     const float* __restrict__ w2t, const float* __restrict__ w0, int n_tokens,
                     int channels, int rank) {
  extern __shared__ float s_low[];                  // [DK_TOK][rank]: tanh of the tokens' inner rows
  pdl_trigger();
  pdl_wait();
  const int t0 = blockIdx.x * DK_TOK;
  const int here = min(DK_TOK, n_tokens - t0);
  for (int e = threadIdx.x; e < here * rank; e += blockDim.x)
    s_low[e] = tanhf(low[(size_t)t0 * rank + e]);
  for (int e = here * rank + threadIdx.x; e < DK_TOK * rank; e += blockDim.x) s_low[e] = 0.f;
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float acc[DK_TOK];
#pragma unroll
  for (int u = 0; u < DK_TOK; ++u) acc[u] = 0.f;
  for (int j = 0; j < rank; ++j) {
    const float wv = w2t[(size_t)j * channels + c];
#pragma unroll
    for (int u = 0; u < DK_TOK; ++u) acc[u] = fmaf(wv, s_low[u * rank + j], acc[u]);
  }
  const float b = w0[c];
#pragma unroll
  for (int u = 0; u < DK_TOK; ++u)
    if (u < here) out[(size_t)(t0 + u) * channels + c] = expf(-expf(acc[u] + b));
}

// ---------------------------------------------------------------------------------------
constexpr int TM_THREADS = 128;
constexpr int TM_ROWS = 16;           // state rows a thread keeps
constexpr int TM_PART = TM_ROWS + 4;  // floats between two parts' rows in shared memory
constexpr int TM_TOK = 16;            // tokens staged at a time (8 or 4 when dim is above 64 or 128)

__device__ __forceinline__ void tm_cp16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
               : "memory");
}

// One token on a thread's 16 state rows.  With b = k v (one product per row):
//   share of o = sum_i (s_i + u_i b_i) r_i ;   s_i <- w_i s_i + b_i
__device__ __forceinline__ float tm_token(float (&s)[TM_ROWS], const float* rp, const float* kp,
                                          const float* wp, const float (&u)[TM_ROWS], float vt) {
  float part_sum[TM_ROWS / 4];
#pragma unroll
  for (int i4 = 0; i4 < TM_ROWS / 4; ++i4) {
    const float4 r4 = *(const float4*)(rp + 4 * i4), k4 = *(const float4*)(kp + 4 * i4);
    const float4 w4 = *(const float4*)(wp + 4 * i4);
    const float rr[4] = {r4.x, r4.y, r4.z, r4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
    const float ww[4] = {w4.x, w4.y, w4.z, w4.w};
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = 4 * i4 + j;
      const float b = __fmul_rn(kk[j], vt);
      a = fmaf(fmaf(u[i], b, s[i]), rr[j], a);
      s[i] = fmaf(ww[j], s[i], b);
    }
    part_sum[i4] = a;
  }
  return (part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]);
}

// A portion of up to ntok tokens (from token `tok` on) into one buffer: r, k, w [ntok][Dp] and
// v [ntok][cols].  `vec`: rows are 16-byte aligned and go in by cp.async, else by plain loads.
__device__ __forceinline__ void tm_stage(float* s_r, const float* __restrict__ r,
                                         const float* __restrict__ k, const float* __restrict__ w,
                                         const float* __restrict__ v, int tok, int here, int h,
                                         int H, int D, int Dp, int cols, int v0, int ntok, int vec) {
  float* s_k = s_r + ntok * Dp;
  float* s_w = s_k + ntok * Dp;
  float* s_v = s_w + ntok * Dp;
  const size_t stride = (size_t)H * D;
  if (vec) {
    const int dq = D / 4, cq = cols / 4;
    for (int e = threadIdx.x; e < here * dq; e += TM_THREADS) {
      const int tt = e / dq, c = e - tt * dq;
      const size_t src = (size_t)(tok + tt) * stride + (size_t)h * D + 4 * c;
      const int at = tt * Dp + (4 * c) / TM_ROWS * TM_PART + (4 * c) % TM_ROWS;
      tm_cp16(s_r + at, r + src);
      tm_cp16(s_k + at, k + src);
      tm_cp16(s_w + at, w + src);
    }
    for (int e = threadIdx.x; e < here * cq; e += TM_THREADS) {
      const int tt = e / cq, c = e - tt * cq;
      if (v0 + 4 * c < D)
        tm_cp16(s_v + tt * cols + 4 * c, v + (size_t)(tok + tt) * stride + (size_t)h * D + v0 + 4 * c);
    }
  } else {
    for (int e = threadIdx.x; e < here * D; e += TM_THREADS) {
      const int tt = e / D, d = e - tt * D;
      const size_t src = (size_t)(tok + tt) * stride + (size_t)h * D + d;
      const int at = tt * Dp + d / TM_ROWS * TM_PART + d % TM_ROWS;
      s_r[at] = r[src];
      s_k[at] = k[src];
      s_w[at] = w[src];
    }
    for (int e = threadIdx.x; e < here * cols; e += TM_THREADS) {
      const int tt = e / cols, c = e - tt * cols;
      if (v0 + c < D) s_v[e] = v[(size_t)(tok + tt) * stride + (size_t)h * D + v0 + c];
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(TM_THREADS, 1)
timemix_kernel(float* __restrict__ o, float* __restrict__ state, int state_stride,
               const float* __restrict__ r, const float* __restrict__ k,
               const float* __restrict__ v, const float* __restrict__ w,
               const float* __restrict__ u, const int* __restrict__ req_start,
               const int* __restrict__ req_len, const int* __restrict__ req_slot, int H, int D,
               int P, int ntok, int vec) {
  extern __shared__ __align__(16) float smem[];
  pdl_trigger();
  pdl_wait();
  const int Dp = P * TM_PART;
  const int cols = TM_THREADS / P;                  // value columns of this block
  const int per_buf = ntok * (3 * Dp + cols);
  const int rq = blockIdx.z, h = blockIdx.y;
  const int n = req_len[rq];
  if (n <= 0) return;
  const int t0 = req_start[rq];
  const int part = threadIdx.x % P, col = threadIdx.x / P;
  const int v0 = blockIdx.x * cols;
  const int vc = v0 + col;
  const bool col_ok = vc < D;
  float* S = state + (size_t)req_slot[rq] * state_stride + (size_t)h * D * D;
  float s[TM_ROWS], uu[TM_ROWS];
#pragma unroll
  for (int i = 0; i < TM_ROWS; ++i) {
    const int d = part * TM_ROWS + i;
    s[i] = (col_ok && d < D) ? S[(size_t)d * D + vc] : 0.f;
    uu[i] = d < D ? u[(size_t)h * D + d] : 0.f;
  }
  if (D != P * TM_ROWS || D % cols) {               // rows or columns past the sizes read as zero
    for (int e = threadIdx.x; e < 2 * per_buf; e += TM_THREADS) smem[e] = 0.f;
    __syncthreads();
  }
  tm_stage(smem, r, k, w, v, t0, min(ntok, n), h, H, D, Dp, cols, v0, ntok, vec);
  int buf = 0;
  for (int base = 0; base < n; base += ntok, buf ^= 1) {
    const int here = min(ntok, n - base);
    if (base + ntok < n) {
      tm_stage(smem + (buf ^ 1) * per_buf, r, k, w, v, t0 + base + ntok,
               min(ntok, n - base - ntok), h, H, D, Dp, cols, v0, ntok, vec);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* s_r = smem + buf * per_buf;
    const float* s_k = s_r + ntok * Dp;
    const float* s_w = s_k + ntok * Dp;
    const float* s_v = s_w + ntok * Dp;
    int tt = 0;
    for (; tt + 2 <= here; tt += 2) {               // two tokens: their folds overlap
      float acc[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int at = (tt + q) * Dp + part * TM_PART;
        acc[q] = tm_token(s, s_r + at, s_k + at, s_w + at, uu, s_v[(tt + q) * cols + col]);
      }
      for (int off = 1; off < P; off <<= 1) {
#pragma unroll
        for (int q = 0; q < 2; ++q) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], off);
      }
      if (part == 0 && col_ok) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
          o[(size_t)(t0 + base + tt + q) * H * D + (size_t)h * D + vc] = acc[q];
      }
    }
    for (; tt < here; ++tt) {
      const int at = tt * Dp + part * TM_PART;
      float acc = tm_token(s, s_r + at, s_k + at, s_w + at, uu, s_v[tt * cols + col]);
      for (int off = 1; off < P; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (part == 0 && col_ok) o[(size_t)(t0 + base + tt) * H * D + (size_t)h * D + vc] = acc;
    }
    __syncthreads();                                // this buffer is staged into again next turn
  }
#pragma unroll
  for (int i = 0; i < TM_ROWS; ++i) {
    const int d = part * TM_ROWS + i;
    if (col_ok && d < D) S[(size_t)d * D + vc] = s[i];
  }
}

// ---------------------------------------------------------------------------------------
// a warp per (token, head): the head's rows of o, its root mean square, weight, gate, scale
template <typename TO>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(TO* __restrict__ out, const float* __restrict__ o,
                      const float* __restrict__ weight, const float* __restrict__ gate,
                      int gate_stride, int gate_offset, int n_tokens, int H, int D, float eps,
                      int gate_silu, float out_scale) {
  pdl_trigger();
  pdl_wait();
  const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n_tokens * H) return;
  const int t = item / H, h = item - t * H;
  const float* row = o + (size_t)t * H * D + (size_t)h * D;
  float ss = 0.f;
  for (int e = lane; e < D; e += 32) ss = fmaf(row[e], row[e], ss);
  ss = warp_sum(ss);
  const float rn = 1.0f / sqrtf(ss / (float)D + eps);
  for (int e = lane; e < D; e += 32) {
    float val = row[e] * rn;
    if (weight) val *= weight[(size_t)h * D + e];
    if (gate) {
      const float z = gate[(size_t)t * gate_stride + gate_offset + (size_t)h * D + e];
      val *= gate_silu ? z / (1.0f + expf(-z)) : 1.0f / (1.0f + expf(-z));
    }
    out[(size_t)t * H * D + (size_t)h * D + e] = from_f<TO>(val * out_scale);
  }
}

template <typename TO, typename TT>
__global__ void __launch_bounds__(128)
gather_mul_kernel(TO* __restrict__ out, const float* __restrict__ g, const TT* __restrict__ table,
                  int table_rows, int table_cols, const int* __restrict__ tok_ids,
                  const int* __restrict__ tok_req, const int* __restrict__ feedback,
                  int n_feedback, int dim, int col_offset, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (tok_req[t] < 0) return;
  const int id = resolve_token(tok_ids, t, feedback, n_feedback);
  if (id < 0 || id >= table_rows) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_TOKEN);
    return;
  }
  const TT* row = table + (size_t)id * table_cols + col_offset;
  for (int c = threadIdx.x; c < dim; c += blockDim.x)
    out[(size_t)t * dim + c] = from_f<TO>(g[(size_t)t * dim + c] * to_f(row[c]));
}

}  // namespace hs

HS_EXPORT int hs_token_shift_mix(void* out, const void* x, const float* mu, float* state,
                                 int state_stride, int state_offset, const int* tok_req,
                                 const int* req_start, const int* req_len, const int* req_slot,
                                 int n_tokens, int width, int n_streams, int dtype, void* stream) {
  if (!out || !x || !mu || !state || !tok_req || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  if (width <= 0 || n_streams <= 0 || state_offset < 0 || state_offset + width > state_stride)
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (dtype == HS_DT_F32)
    e = hs_launch(hs::token_shift_mix_kernel<float>, dim3(n_tokens), dim3(256), 0, st,
                  hs_pdl_enabled(), (float*)out, (const float*)x, mu, state, state_stride,
                  state_offset, tok_req, req_start, req_len, req_slot, n_tokens, width, n_streams);
  else if (dtype == HS_DT_BF16)
    e = hs_launch(hs::token_shift_mix_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, st,
                  hs_pdl_enabled(), (__nv_bfloat16*)out, (const __nv_bfloat16*)x, mu, state,
                  state_stride, state_offset, tok_req, req_start, req_len, req_slot, n_tokens,
                  width, n_streams);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_timemix_decay(float* out, const float* low, const float* w2t, const float* w0,
                               int n_tokens, int channels, int rank, void* stream) {
  if (!out || !low || !w2t || !w0) return HS_ERR_ARGUMENT;
  if (channels <= 0 || rank <= 0 || rank > 1024) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const dim3 grid((n_tokens + hs::DK_TOK - 1) / hs::DK_TOK, (channels + 255) / 256);
  if (grid.y > 65535) return HS_ERR_TOO_LARGE;
  cudaError_t e = hs_launch(hs::timemix_decay_kernel, grid, dim3(256),
                            (size_t)hs::DK_TOK * rank * sizeof(float), (cudaStream_t)stream,
                            hs_pdl_enabled(), out, low, w2t, w0, n_tokens, channels, rank);
  return e == cudaSuccess ? HS_OK : (int)e;
}

// r, k, v, w: float32 [tokens, H * D], head by head; u: [H * D]; o: float32 [tokens, H * D];
// the state of slot s starts at state + s * state_stride ([H, D, D] floats).
HS_EXPORT int hs_timemix_recurrence(float* o, float* state, int state_stride, const float* r,
                                    const float* k, const float* v, const float* w,
                                    const float* u, const int* req_start, const int* req_len,
                                    const int* req_slot, int n_requests, int n_tokens, int H,
                                    int D, void* stream) {
  if (!o || !state || !r || !k || !v || !w || !u || !req_start || !req_len || !req_slot)
    return HS_ERR_ARGUMENT;
  if (H <= 0 || D <= 0 || D > 16 * hs::TM_ROWS || state_stride < H * D * D)
    return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0 || n_tokens <= 0) return HS_OK;
  int P = 1;
  while (P * hs::TM_ROWS < D) P *= 2;
  const int cols = hs::TM_THREADS / P;
  const int ntok = P <= 4 ? hs::TM_TOK : (P == 8 ? hs::TM_TOK / 2 : hs::TM_TOK / 4);   // at most 34 KB
  const bool aligned = ((((uintptr_t)r) | ((uintptr_t)k) | ((uintptr_t)v) | ((uintptr_t)w)) & 15) == 0;
  const int vec = (D % 4 == 0 && cols % 4 == 0 && aligned) ? 1 : 0;
  const size_t smem = (size_t)2 * ntok * (3 * P * hs::TM_PART + cols) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  if (n_requests > 65535 || H > 65535) return HS_ERR_TOO_LARGE;
  dim3 grid((D + cols - 1) / cols, H, n_requests);
  cudaError_t e = hs_launch(hs::timemix_kernel, grid, dim3(hs::TM_THREADS), smem,
                            (cudaStream_t)stream, hs_pdl_enabled(), o, state, state_stride, r, k,
                            v, w, u, req_start, req_len, req_slot, H, D, P, ntok, vec);
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_head_norm_gate(void* out, const float* o, const float* weight,
                                const float* gate, int gate_stride, int gate_offset,
                                int n_tokens, int H, int D, float eps, int gate_silu,
                                float out_scale, int out_dtype, void* stream) {
  if (!out || !o) return HS_ERR_ARGUMENT;
  if (H <= 0 || D <= 0 || (gate && (gate_offset < 0 || gate_offset + H * D > gate_stride)))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const long long items = (long long)n_tokens * H;
  const unsigned blocks = (unsigned)((items + 7) / 8);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (out_dtype == HS_DT_F32)
    e = hs_launch(hs::head_norm_gate_kernel<float>, dim3(blocks), dim3(256), 0, st,
                  hs_pdl_enabled(), (float*)out, o, weight, gate, gate_stride, gate_offset,
                  n_tokens, H, D, eps, gate_silu, out_scale);
  else if (out_dtype == HS_DT_BF16)
    e = hs_launch(hs::head_norm_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st,
                  hs_pdl_enabled(), (__nv_bfloat16*)out, o, weight, gate, gate_stride,
                  gate_offset, n_tokens, H, D, eps, gate_silu, out_scale);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_gather_mul(void* out, const float* g, const void* table, int table_rows,
                            int table_cols, const int* tok_ids, const int* tok_req,
                            const int* feedback, int n_feedback, int n_tokens, int dim,
                            int col_offset, int out_dtype, int table_dtype, int* status,
                            void* stream) {
  if (!out || !g || !table || !tok_ids || !tok_req || !status) return HS_ERR_ARGUMENT;
  if (dim <= 0 || col_offset < 0 || col_offset + dim > table_cols || out_dtype != table_dtype)
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (out_dtype == HS_DT_F32)
    e = hs_launch(hs::gather_mul_kernel<float, float>, dim3(n_tokens), dim3(128), 0, st,
                  hs_pdl_enabled(), (float*)out, g, (const float*)table, table_rows, table_cols,
                  tok_ids, tok_req, feedback, n_feedback, dim, col_offset, status);
  else if (out_dtype == HS_DT_BF16)
    e = hs_launch(hs::gather_mul_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(n_tokens), dim3(128),
                  0, st, hs_pdl_enabled(), (__nv_bfloat16*)out, g, (const __nv_bfloat16*)table,
                  table_rows, table_cols, tok_ids, tok_req, feedback, n_feedback, dim, col_offset,
                  status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}
