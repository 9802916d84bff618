// Softmax attention over a sliding window plus pooled blocks behind it, over the paged cache.
//
// The cache keeps one row [key (D) | value (V)] per token and key/value head (pool
// [pages][kv_heads][page_size][D + V]); a companion pool of the same layout keeps one row of
// means per block of `block` positions (its "position" is the block's index).
//
//   pooled_prepare    from the float32 projection [q | k | v]: q and k RMS-normed per head
//                     (weight of size D shared by the heads), turned by the token's position on
//                     their first rot_dims numbers (number d pairs with d + rot_dims/2), the
//                     values turned by the position over all of V; q to a float32 buffer, the
//                     row [k | v] straight into the token's page: norm, rotation and append fused
//   pooled_means      for every token that completes a block: the mean of the block's rows as
//                     the cache holds them, written to the companion pool
//   pooled_attention  a warp per (token, query head): the visible block rows, then the window's
//                     token rows, 32 keys a round (a key per lane for the scores, a column per
//                     lane for the values), one running softmax over both kinds; the head's
//                     output is turned back by the query's position and written in the compute
//                     type.  With a list of tokens (the single-query section of a step's work
//                     lists) only those are served; the prompt portions then run on the tensor
//                     cores (attention_pooled_mma.cu)
//
// Angles are formed in double and reduced there (rotary.cuh); scores, softmax state and
// accumulators are float32.  A row's result depends on its own request only: the keys are
// walked in an order fixed by the position.
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

constexpr int PA_WARPS = 8;

// ---------------------------------------------------------------------------------------
template <typename TC>
__global__ void __launch_bounds__(PA_WARPS * 32)
pooled_prepare_kernel(float* __restrict__ q_out, TC* __restrict__ pool,
                      const float* __restrict__ proj, int proj_stride,
                      const float* __restrict__ wq, const float* __restrict__ wk,
                      const float* __restrict__ freq_qk, const float* __restrict__ freq_v,
                      const int* __restrict__ table, int max_pages, int num_pages,
                      const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
                      int H, int G, int D, int V, int rot_dims, float eps, int page_size,
                      int writes, TC* __restrict__ coarse, const int* __restrict__ ctable,
                      int cmax_pages, int cnum_pages, int block, int* __restrict__ status) {
  extern __shared__ float s_vec[];                 // [PA_WARPS][max(D, V)]
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ext = max(D, V);
  float* sv = s_vec + (size_t)warp * ext;
  TC* row = nullptr;
  if (writes) {
    const int pi = pos / page_size;
    const int page = pi < max_pages ? table[(size_t)r * max_pages + pi] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    } else {
      row = pool + ((size_t)page * G * page_size + (pos % page_size)) * (size_t)(D + V);
    }
  }
  const float* pr = proj + (size_t)t * proj_stride;
  const int jobs = H + 2 * G;                      // query heads, key heads, value heads
  for (int job = warp; job < jobs; job += PA_WARPS) {
    const bool is_q = job < H, is_k = !is_q && job < H + G;
    const int n = (is_q || is_k) ? D : V;
    const float* src = is_q ? pr + (size_t)job * D
                     : is_k ? pr + (size_t)H * D + (size_t)(job - H) * D
                            : pr + (size_t)(H + G) * D + (size_t)(job - H - G) * V;
    const float* w = is_q ? wq : is_k ? wk : nullptr;
    float ss = 0.f;
    for (int e = lane; e < n; e += 32) {
      const float v = src[e];
      sv[e] = v;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    __syncwarp();
    const float rn = (w != nullptr) ? 1.0f / sqrtf(ss / (float)n + eps) : 1.0f;
    const int dims = (is_q || is_k) ? rot_dims : (freq_v ? V : 0);
    const float* freq = (is_q || is_k) ? freq_qk : freq_v;
    const int half = dims >> 1;
    float* qdst = is_q ? q_out + (size_t)t * H * D + (size_t)job * D : nullptr;
    TC* cdst = nullptr;
    if (!is_q && row != nullptr) {
      const int g = is_k ? job - H : job - H - G;
      cdst = row + (size_t)g * page_size * (D + V) + (is_k ? 0 : D);
    }
    for (int e = lane; e < n; e += 32) {
      float own = sv[e] * rn * (w ? w[e] : 1.0f);
      if (e < dims) {
        const int pe = e < half ? e + half : e - half;
        const float partner = sv[pe] * rn * (w ? w[pe] : 1.0f);
        float c, s;
        pair_angle(pos, freq[e < half ? e : e - half], &c, &s);
        own = e < half ? own * c - partner * s : own * c + partner * s;
      }
      if (qdst) qdst[e] = own;
      if (cdst) cdst[e] = from_f<TC>(own);
    }
    __syncwarp();
  }
  // With the companion pool (handed in only when every request brings ONE token, so that the
  // other rows of a block are of earlier steps): a token that completes a block forms the
  // block's mean row here, summed as pooled_means sums it.
  if (coarse == nullptr || row == nullptr || (pos + 1) % block) return;
  __syncthreads();                                 // this token's row is in its page
  const int b = pos / block;
  const int cpi = b / page_size;
  const int cpage = cpi < cmax_pages ? ctable[(size_t)r * cmax_pages + cpi] : -1;
  if (cpage < 0 || cpage >= cnum_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    return;
  }
  const int row_len = D + V;
  const float inv = 1.0f / (float)block;
  for (int idx = threadIdx.x; idx < G * row_len; idx += blockDim.x) {
    const int g = idx / row_len, e = idx - g * row_len;
    float acc = 0.f;
    bool ok = true;
    for (int j = b * block; j <= pos; ++j) {
      const int pi = j / page_size;
      const int page = pi < max_pages ? table[(size_t)r * max_pages + pi] : -1;
      if (page < 0 || page >= num_pages) { ok = false; break; }
      acc += to_f(pool[(((size_t)page * G + g) * page_size + (j % page_size)) * (size_t)row_len + e]);
    }
    if (!ok) {
      atomicOr(status, HS_STATUS_BAD_PAGE);
      continue;
    }
    coarse[(((size_t)cpage * G + g) * page_size + (b % page_size)) * (size_t)row_len + e] =
        from_f<TC>(acc * inv);
  }
}

// ---------------------------------------------------------------------------------------
template <typename TC>
__global__ void __launch_bounds__(128)
pooled_means_kernel(TC* __restrict__ coarse, const int* __restrict__ ctable, int cmax_pages,
                    int cnum_pages, const TC* __restrict__ pool, const int* __restrict__ table,
                    int max_pages, int num_pages, const int* __restrict__ tok_pos,
                    const int* __restrict__ tok_req, int G, int row_len, int block,
                    int page_size, int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, g = blockIdx.y;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  if ((pos + 1) % block) return;                    // this token completes no block
  const int b = pos / block;
  const int cpi = b / page_size;
  const int cpage = cpi < cmax_pages ? ctable[(size_t)r * cmax_pages + cpi] : -1;
  if (cpage < 0 || cpage >= cnum_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    return;
  }
  TC* dst = coarse + (((size_t)cpage * G + g) * page_size + (b % page_size)) * (size_t)row_len;
  const float inv = 1.0f / (float)block;
  for (int e = threadIdx.x; e < row_len; e += blockDim.x) {
    float acc = 0.f;
    bool ok = true;
    for (int j = b * block; j <= pos; ++j) {
      const int pi = j / page_size;
      const int page = pi < max_pages ? table[(size_t)r * max_pages + pi] : -1;
      if (page < 0 || page >= num_pages) { ok = false; break; }
      acc += to_f(pool[(((size_t)page * G + g) * page_size + (j % page_size)) * (size_t)row_len + e]);
    }
    if (!ok) {
      if (e == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
      return;
    }
    dst[e] = from_f<TC>(acc * inv);
  }
}

// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float dot_row(const float* __restrict__ k, const float* q, int D,
                                         bool vec) {
  float s = 0.f;
  if (vec) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int i = 0; i < D / 4; ++i) {
      const float4 a = k4[i];
      s = fmaf(a.x, q[4 * i], s); s = fmaf(a.y, q[4 * i + 1], s);
      s = fmaf(a.z, q[4 * i + 2], s); s = fmaf(a.w, q[4 * i + 3], s);
    }
  } else {
    for (int i = 0; i < D; ++i) s = fmaf(k[i], q[i], s);
  }
  return s;
}
__device__ __forceinline__ float dot_row(const __nv_bfloat16* __restrict__ k, const float* q,
                                         int D, bool vec) {
  float s = 0.f;
  if (vec) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int i = 0; i < D / 8; ++i) {
      const uint4 a = k8[i];
      const unsigned w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // a bfloat16 is the upper half of a float
        s = fmaf(__uint_as_float(w[j] << 16), q[8 * i + 2 * j], s);
        s = fmaf(__uint_as_float(w[j] & 0xffff0000u), q[8 * i + 2 * j + 1], s);
      }
    }
  } else {
    for (int i = 0; i < D; ++i) s = fmaf(__bfloat162float(k[i]), q[i], s);
  }
  return s;
}

// PA_MAXC: value columns a lane owns (V <= 32 * PA_MAXC); the launcher picks 2, 8 or 32.
// A block serves one (token, head).  Its warps take rounds of 32 keys in turn (warp w the rounds
// w, w + PA_WARPS, ...), each with a running maximum, sum and output of its own, and the block
// joins them at the end: a single token's keys are walked by eight warps side by side instead of
// one after the other.  How the keys are dealt depends on the token's own position only.
template <typename TC, typename TO, int PA_MAXC>
__global__ void __launch_bounds__(PA_WARPS * 32)
pooled_attention_kernel(TO* __restrict__ out, const float* __restrict__ q,
                        const TC* __restrict__ pool, const int* __restrict__ table,
                        int max_pages, int num_pages, const TC* __restrict__ coarse,
                        const int* __restrict__ ctable, int cmax_pages, int cnum_pages,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_req,
                        const float* __restrict__ freq_v, int n_tokens, int H, int G, int D,
                        int V, int window, int block, float scale, int page_size, int vec,
                        const int* __restrict__ listed, const int* __restrict__ plan_head,
                        int* __restrict__ status) {
  extern __shared__ float s_pa[];                  // q [D] | acc [PA_WARPS][V] | m, l [2 PA_WARPS]
  float* sq = s_pa;
  float* s_acc = s_pa + D;
  float* s_ml = s_acc + (size_t)PA_WARPS * V;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = blockIdx.x;
  // with a list only the listed tokens are served, as many as the list's head says
  const int n_here = listed ? min(n_tokens, plan_head[0]) : n_tokens;
  if (item >= (long long)n_here * H) return;
  // consecutive tokens of one head are neighbours in the grid: their windows overlap in the L2
  const int h = (int)(item / n_here), entry = (int)(item - (long long)h * n_here);
  const int t = listed ? listed[3 * entry] : entry;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  const int g = h / (H / G);
  const float* qr = q + (size_t)t * H * D + (size_t)h * D;
  for (int e = threadIdx.x; e < D; e += PA_WARPS * 32) sq[e] = qr[e] * scale;
  __syncthreads();
  const int row_len = D + V;
  const int first = max(0, pos - window + 1);
  const int seen = max(0, (pos - window + 1) / block);    // blocks wholly behind the window
  const int n_keys = seen + (pos - first + 1);
  const int* tab = table + (size_t)r * max_pages;
  const int* ctab = ctable + (size_t)r * cmax_pages;
  float m = -INFINITY, l = 0.f;
  float acc[PA_MAXC];
#pragma unroll
  for (int c = 0; c < PA_MAXC; ++c) acc[c] = 0.f;
  bool bad = false;
  for (int base = warp * 32; base < n_keys; base += PA_WARPS * 32) {
    const int kk = base + lane;
    const TC* krow = nullptr;
    if (kk < n_keys) {
      if (kk < seen) {
        const int pi = kk / page_size;
        const int page = pi < cmax_pages ? ctab[pi] : -1;
        if (page < 0 || page >= cnum_pages) bad = true;
        else krow = coarse + (((size_t)page * G + g) * page_size + (kk % page_size)) * (size_t)row_len;
      } else {
        const int j = first + (kk - seen);
        const int pi = j / page_size;
        const int page = pi < max_pages ? tab[pi] : -1;
        if (page < 0 || page >= num_pages) bad = true;
        else krow = pool + (((size_t)page * G + g) * page_size + (j % page_size)) * (size_t)row_len;
      }
    }
    const float s = krow ? dot_row(krow, sq, D, vec != 0) : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;               // no valid key in this round
    const float corr = expf(m - m_new);             // m = -inf: 0
    const float p = krow ? expf(s - m_new) : 0.f;
    l = fmaf(l, corr, warp_sum(p));
    m = m_new;
#pragma unroll
    for (int c = 0; c < PA_MAXC; ++c) acc[c] *= corr;
    const int n_round = min(32, n_keys - base);
    // four value rows in flight: their loads are issued before the first is used
    for (int jj = 0; jj < n_round; jj += 4) {
      float pj[4];
      const TC* vr[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int src = (jj + u) & 31;
        pj[u] = __shfl_sync(0xffffffffu, p, src);
        const unsigned long long ptr =
            __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)krow, src);
        vr[u] = jj + u < n_round && ptr != 0ull ? reinterpret_cast<const TC*>((uintptr_t)ptr) + D
                                                : nullptr;
      }
#pragma unroll
      for (int c = 0; c < PA_MAXC; ++c) {
        const int e = c * 32 + lane;
        if (e < V) {
          float v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = vr[u] ? to_f(vr[u][e]) : 0.f;
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (vr[u]) acc[c] = fmaf(pj[u], v[u], acc[c]);
        }
      }
    }
  }
  if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
  // the warps' shares joined under one maximum, in the order of the warps
  if (lane == 0) {
    s_ml[warp] = m;
    s_ml[PA_WARPS + warp] = l;
  }
#pragma unroll
  for (int c = 0; c < PA_MAXC; ++c) {
    const int e = c * 32 + lane;
    if (e < V) s_acc[(size_t)warp * V + e] = acc[c];
  }
  __syncthreads();
  float top = -INFINITY;
#pragma unroll
  for (int w = 0; w < PA_WARPS; ++w) top = fmaxf(top, s_ml[w]);
  float total = 0.f, share[PA_WARPS];
#pragma unroll
  for (int w = 0; w < PA_WARPS; ++w) {
    share[w] = s_ml[w] == -INFINITY ? 0.f : expf(s_ml[w] - top);
    total = fmaf(s_ml[PA_WARPS + w], share[w], total);
  }
  const float inv = total > 0.f ? 1.0f / total : 0.f;
  __syncthreads();
  for (int e = threadIdx.x; e < V; e += PA_WARPS * 32) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < PA_WARPS; ++w) o = fmaf(s_acc[(size_t)w * V + e], share[w], o);
    s_acc[e] = o * inv;                            // row 0 of the shares: each thread its own e
  }
  __syncthreads();
  // the head's output, turned back by the query's position (pairs e, e + V/2)
  TO* orow = out + (size_t)t * H * V + (size_t)h * V;
  const int half = V >> 1;
  for (int e = threadIdx.x; e < V; e += PA_WARPS * 32) {
    float own = s_acc[e];
    if (freq_v != nullptr) {
      const float partner = s_acc[e < half ? e + half : e - half];
      float c, s;
      pair_angle(pos, freq_v[e < half ? e : e - half], &c, &s);
      own = e < half ? own * c + partner * s : own * c - partner * s;      // the angle negated
    }
    orow[e] = from_f<TO>(own);
  }
}

}  // namespace hs

HS_EXPORT int hs_pooled_prepare(float* q_out, void* pool, const float* proj, int proj_stride,
                                const float* wq, const float* wk, const float* freq_qk,
                                const float* freq_v, const int* table, int max_pages,
                                int num_pages, const int* tok_pos, const int* tok_req,
                                int n_tokens, int H, int G, int D, int V, int rot_dims, float eps,
                                int page_size, int writes, int cache_dtype, void* coarse,
                                const int* ctable, int cmax_pages, int cnum_pages, int block,
                                int* status, void* stream) {
  if (!q_out || !pool || !proj || !table || !tok_pos || !tok_req || !status)
    return HS_ERR_ARGUMENT;
  if (coarse && (!ctable || block <= 0 || cmax_pages <= 0 || !writes)) return HS_ERR_ARGUMENT;
  if ((wq == nullptr) != (wk == nullptr) || (rot_dims > 0 && !freq_qk)) return HS_ERR_ARGUMENT;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || rot_dims < 0 || rot_dims % 2 ||
      rot_dims > D || (freq_v && V % 2) || page_size <= 0)
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)hs::PA_WARPS * (D > V ? D : V) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (cache_dtype == HS_DT_BF16)
    e = hs_launch(hs::pooled_prepare_kernel<__nv_bfloat16>, dim3(n_tokens),
                  dim3(hs::PA_WARPS * 32), smem, st, hs_pdl_enabled(), q_out,
                  (__nv_bfloat16*)pool, proj, proj_stride, wq, wk, freq_qk, freq_v, table,
                  max_pages, num_pages, tok_pos, tok_req, H, G, D, V, rot_dims, eps, page_size,
                  writes, (__nv_bfloat16*)coarse, ctable, cmax_pages, cnum_pages, block, status);
  else if (cache_dtype == HS_DT_F32)
    e = hs_launch(hs::pooled_prepare_kernel<float>, dim3(n_tokens), dim3(hs::PA_WARPS * 32), smem,
                  st, hs_pdl_enabled(), q_out, (float*)pool, proj, proj_stride, wq, wk, freq_qk,
                  freq_v, table, max_pages, num_pages, tok_pos, tok_req, H, G, D, V, rot_dims,
                  eps, page_size, writes, (float*)coarse, ctable, cmax_pages, cnum_pages, block,
                  status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_pooled_means(void* coarse, const int* ctable, int cmax_pages, int cnum_pages,
                              const void* pool, const int* table, int max_pages, int num_pages,
                              const int* tok_pos, const int* tok_req, int n_tokens, int G,
                              int row_len, int block, int page_size, int cache_dtype, int* status,
                              void* stream) {
  if (!coarse || !ctable || !pool || !table || !tok_pos || !tok_req || !status)
    return HS_ERR_ARGUMENT;
  if (G <= 0 || row_len <= 0 || block <= 0 || page_size <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  if (G > 65535) return HS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (cache_dtype == HS_DT_BF16)
    e = hs_launch(hs::pooled_means_kernel<__nv_bfloat16>, dim3(n_tokens, G), dim3(128), 0, st,
                  hs_pdl_enabled(), (__nv_bfloat16*)coarse, ctable, cmax_pages, cnum_pages,
                  (const __nv_bfloat16*)pool, table, max_pages, num_pages, tok_pos, tok_req, G,
                  row_len, block, page_size, status);
  else if (cache_dtype == HS_DT_F32)
    e = hs_launch(hs::pooled_means_kernel<float>, dim3(n_tokens, G), dim3(128), 0, st,
                  hs_pdl_enabled(), (float*)coarse, ctable, cmax_pages, cnum_pages,
                  (const float*)pool, table, max_pages, num_pages, tok_pos, tok_req, G, row_len,
                  block, page_size, status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_pooled_attention(void* out, const float* q, const void* pool, const int* table,
                                  int max_pages, int num_pages, const void* coarse,
                                  const int* ctable, int cmax_pages, int cnum_pages,
                                  const int* tok_pos, const int* tok_req, const float* freq_v,
                                  int n_tokens, int H, int G, int D, int V, int window, int block,
                                  float scale, int page_size, int cache_dtype, int out_dtype,
                                  const int* listed, const int* plan_head, int* status,
                                  void* stream) {
  if (!out || !q || !pool || !table || !coarse || !ctable || !tok_pos || !tok_req || !status ||
      (listed && !plan_head))
    return HS_ERR_ARGUMENT;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || V > 1024 || window <= 0 ||
      block <= 0 || page_size <= 0 || (freq_v && V % 2))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = ((size_t)D + (size_t)hs::PA_WARPS * (V + 2)) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  const long long items = (long long)n_tokens * H;
  if (items > 0x7fffffffLL) return HS_ERR_TOO_LARGE;
  const dim3 grid((unsigned)items), blk(hs::PA_WARPS * 32);
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = hs_pdl_enabled();
  // 16-byte reads of a key row need rows that start and end on 16 bytes
  const int per16 = cache_dtype == HS_DT_BF16 ? 8 : 4;
  const int vec = (D % per16 == 0 && V % per16 == 0) ? 1 : 0;
  cudaError_t e;
#define HS_PA_LAUNCH_C(TC, TO, C)                                                                \
  e = hs_launch(hs::pooled_attention_kernel<TC, TO, C>, grid, blk, smem, st, pdl, (TO*)out, q,   \
                (const TC*)pool, table, max_pages, num_pages, (const TC*)coarse, ctable,         \
                cmax_pages, cnum_pages, tok_pos, tok_req, freq_v, n_tokens, H, G, D, V, window,  \
                block, scale, page_size, vec, listed, plan_head, status)
#define HS_PA_LAUNCH(TC, TO)                                                                     \
  do {                                                                                           \
    if (V <= 64) HS_PA_LAUNCH_C(TC, TO, 2);                                                      \
    else if (V <= 256) HS_PA_LAUNCH_C(TC, TO, 8);                                                \
    else HS_PA_LAUNCH_C(TC, TO, 32);                                                             \
  } while (0)
  if (cache_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_PA_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (cache_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_PA_LAUNCH(float, float);
  else return HS_ERR_UNSUPPORTED;
#undef HS_PA_LAUNCH
#undef HS_PA_LAUNCH_C
  return e == cudaSuccess ? HS_OK : (int)e;
}
