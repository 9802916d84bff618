// Grouped softmax attention over the paged cache with a linear bias of the distance and a
// sliding window that keeps the first tokens, on the CUDA cores.
//
// The cache keeps one row [key (D) | value (V)] per token and key/value head (pool
// [pages][kv_heads][page_size][D + V]).
//
//   span_prepare    from the float32 projection: q (and k) divided by their root mean square per
//                   head when asked (no weight), q to a float32 buffer, the row [k | v] straight
//                   into the token's page; the values are columns of their own or the keys as
//                   projected.  A layer that only reads another's rows writes nothing and has
//                   no key or value columns.
//   span_attention  a block per (token, query head).  Query i sees j <= i with i - j < window
//                   (window 0: all) or j < keep_first; score = q . k * scale - slope_h * (i - j);
//                   its eight warps take rounds of 32 keys in turn (a key per lane for the
//                   scores, a column per lane for the values, four value rows in flight), each
//                   with a running softmax of its own, joined under one maximum at the end; the
//                   output may be multiplied element by element by the sigmoid of gate columns
//                   and by a scale before it is rounded.  With a list of tokens (the
//                   single-query section of a step's work lists) only those are served.
//
// Scores, softmax state and accumulators are float32.  A row's result depends on its own
// request only: the keys are dealt to the warps in an order fixed by the position.
#include "common.cuh"

namespace hs {

constexpr int SA_WARPS = 8;

template <typename TC>
__global__ void __launch_bounds__(SA_WARPS * 32)
span_prepare_kernel(float* __restrict__ q_out, TC* __restrict__ pool,
                    const float* __restrict__ proj, int proj_stride, int q_off, int k_off,
                    int v_off, const int* __restrict__ table, int max_pages, int num_pages,
                    const int* __restrict__ tok_pos, const int* __restrict__ tok_req, int H, int G,
                    int D, int V, int qk_norm, float eps, int page_size, int writes,
                    int* __restrict__ status) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TC* row = nullptr;
  if (writes) {
    const int pi = pos / page_size;
    const int page = (pos >= 0 && pi < max_pages) ? table[(size_t)r * max_pages + pi] : -1;
    if (page < 0 || page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    } else {
      row = pool + ((size_t)page * G * page_size + (pos % page_size)) * (size_t)(D + V);
    }
  }
  const float* pr = proj + (size_t)t * proj_stride;
  const int jobs = row ? H + 2 * G : H;            // query heads, key heads, value heads
  for (int job = warp; job < jobs; job += SA_WARPS) {
    const bool is_q = job < H, is_k = !is_q && job < H + G;
    const int g = is_q ? 0 : (is_k ? job - H : job - H - G);
    const int n = (is_q || is_k) ? D : V;
    // the values: columns of their own, or the keys as projected (before any norm)
    const float* src = is_q ? pr + q_off + (size_t)job * D
                     : (is_k || v_off < 0) ? pr + k_off + (size_t)g * D
                                           : pr + v_off + (size_t)g * V;
    float rn = 1.0f;
    if (qk_norm && (is_q || is_k)) {
      float ss = 0.f;
      for (int e = lane; e < n; e += 32) ss = fmaf(src[e], src[e], ss);
      ss = warp_sum(ss);
      rn = 1.0f / sqrtf(ss / (float)n + eps);
    }
    float* qdst = is_q ? q_out + (size_t)t * H * D + (size_t)job * D : nullptr;
    TC* cdst = is_q ? nullptr : row + (size_t)g * page_size * (D + V) + (is_k ? 0 : D);
    for (int e = lane; e < n; e += 32) {
      const float val = src[e] * rn;
      if (qdst) qdst[e] = val;
      else cdst[e] = from_f<TC>(val);
    }
  }
}

__device__ __forceinline__ float sa_dot(const float* __restrict__ k, const float* q, int D,
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
__device__ __forceinline__ float sa_dot(const __nv_bfloat16* __restrict__ k, const float* q,
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

// SA_MAXC: value columns a lane owns (V <= 32 * SA_MAXC); the launcher picks 2, 8 or 32.
template <typename TC, typename TO, int SA_MAXC>
__global__ void __launch_bounds__(SA_WARPS * 32)
span_attention_kernel(TO* __restrict__ out, const float* __restrict__ q,
                      const TC* __restrict__ pool, const int* __restrict__ table, int max_pages,
                      int num_pages, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_req, const float* __restrict__ slopes,
                      const float* __restrict__ gate, int gate_stride, int gate_offset,
                      float out_scale, int n_tokens, int H, int G, int D, int V, int window,
                      int keep_first, float scale, int page_size, int vec,
                      const int* __restrict__ listed, const int* __restrict__ plan_head,
                      int* __restrict__ status) {
  extern __shared__ float s_sa[];                  // q [D] | acc [SA_WARPS][V] | m, l [2 SA_WARPS]
  float* sq = s_sa;
  float* s_acc = s_sa + D;
  float* s_ml = s_acc + (size_t)SA_WARPS * V;
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = blockIdx.x;
  // with a list only the listed tokens are served, as many as the list's head says
  const int n_here = listed ? min(n_tokens, plan_head[0]) : n_tokens;
  if (item >= (long long)n_here * H) return;
  // consecutive tokens of one head are neighbours in the grid: their keys overlap in the L2
  const int h = (int)(item / n_here), entry = (int)(item - (long long)h * n_here);
  const int t = listed ? listed[3 * entry] : entry;
  const int r = tok_req[t];
  if (r < 0) return;
  const int pos = tok_pos[t];
  const int g = h / (H / G);
  const float* qr = q + (size_t)t * H * D + (size_t)h * D;
  for (int e = threadIdx.x; e < D; e += SA_WARPS * 32) sq[e] = qr[e] * scale;
  __syncthreads();
  const int row_len = D + V;
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int kept = min(keep_first, first);          // first tokens that lie behind the window
  const int n_keys = kept + (pos - first + 1);
  const float slope = slopes ? slopes[h] : 0.f;
  const int* tab = table + (size_t)r * max_pages;
  float m = -INFINITY, l = 0.f;
  float acc[SA_MAXC];
#pragma unroll
  for (int c = 0; c < SA_MAXC; ++c) acc[c] = 0.f;
  bool bad = false;
  for (int base = warp * 32; base < n_keys; base += SA_WARPS * 32) {
    const int kk = base + lane;
    const TC* krow = nullptr;
    int j = 0;
    if (kk < n_keys) {
      j = kk < kept ? kk : first + (kk - kept);
      const int pi = j / page_size;
      const int page = pi < max_pages ? tab[pi] : -1;
      if (page < 0 || page >= num_pages) bad = true;
      else krow = pool + (((size_t)page * G + g) * page_size + (j % page_size)) * (size_t)row_len;
    }
    // the bias of the distance is taken off the scaled score
    const float s = krow ? sa_dot(krow, sq, D, vec != 0) - slope * (float)(pos - j) : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;               // no valid key in this round
    const float corr = expf(m - m_new);             // m = -inf: 0
    const float p = krow ? expf(s - m_new) : 0.f;
    l = fmaf(l, corr, warp_sum(p));
    m = m_new;
#pragma unroll
    for (int c = 0; c < SA_MAXC; ++c) acc[c] *= corr;
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
      for (int c = 0; c < SA_MAXC; ++c) {
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
    s_ml[SA_WARPS + warp] = l;
  }
#pragma unroll
  for (int c = 0; c < SA_MAXC; ++c) {
    const int e = c * 32 + lane;
    if (e < V) s_acc[(size_t)warp * V + e] = acc[c];
  }
  __syncthreads();
  float top = -INFINITY;
#pragma unroll
  for (int w = 0; w < SA_WARPS; ++w) top = fmaxf(top, s_ml[w]);
  float total = 0.f, share[SA_WARPS];
#pragma unroll
  for (int w = 0; w < SA_WARPS; ++w) {
    share[w] = s_ml[w] == -INFINITY ? 0.f : expf(s_ml[w] - top);
    total = fmaf(s_ml[SA_WARPS + w], share[w], total);
  }
  const float inv = total > 0.f ? 1.0f / total : 0.f;
  TO* orow = out + (size_t)t * H * V + (size_t)h * V;
  const float* grow = gate ? gate + (size_t)t * gate_stride + gate_offset + (size_t)h * V : nullptr;
  for (int e = threadIdx.x; e < V; e += SA_WARPS * 32) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < SA_WARPS; ++w) o = fmaf(s_acc[(size_t)w * V + e], share[w], o);
    o *= inv;
    if (grow) o *= 1.0f / (1.0f + expf(-grow[e]));
    orow[e] = from_f<TO>(o * out_scale);
  }
}

}  // namespace hs

// proj: float32 rows of `proj_stride` columns with q (H*D) at q_off, k (G*D) at k_off and v (G*V)
// at v_off (v_off < 0: the values are the keys as projected; V must equal D); without `writes`
// only the q columns are read.
HS_EXPORT int hs_span_prepare(float* q_out, void* pool, const float* proj, int proj_stride,
                              int q_off, int k_off, int v_off, const int* table, int max_pages,
                              int num_pages, const int* tok_pos, const int* tok_req,
                              int n_tokens, int H, int G, int D, int V, int qk_norm, float eps,
                              int page_size, int writes, int cache_dtype, int* status,
                              void* stream) {
  if (!q_out || !pool || !proj || !table || !tok_pos || !tok_req || !status)
    return HS_ERR_ARGUMENT;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || page_size <= 0 || q_off < 0 ||
      q_off + H * D > proj_stride)
    return HS_ERR_UNSUPPORTED;
  if (writes && (k_off < 0 || k_off + G * D > proj_stride || (v_off < 0 && V != D) ||
                 (v_off >= 0 && v_off + G * V > proj_stride)))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (cache_dtype == HS_DT_BF16)
    e = hs_launch(hs::span_prepare_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(hs::SA_WARPS * 32),
                  0, st, hs_pdl_enabled(), q_out, (__nv_bfloat16*)pool, proj, proj_stride, q_off,
                  k_off, v_off, table, max_pages, num_pages, tok_pos, tok_req, H, G, D, V, qk_norm,
                  eps, page_size, writes, status);
  else if (cache_dtype == HS_DT_F32)
    e = hs_launch(hs::span_prepare_kernel<float>, dim3(n_tokens), dim3(hs::SA_WARPS * 32), 0, st,
                  hs_pdl_enabled(), q_out, (float*)pool, proj, proj_stride, q_off, k_off, v_off,
                  table, max_pages, num_pages, tok_pos, tok_req, H, G, D, V, qk_norm, eps,
                  page_size, writes, status);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_span_attention(void* out, const float* q, const void* pool, const int* table,
                                int max_pages, int num_pages, const int* tok_pos,
                                const int* tok_req, const float* slopes, const float* gate,
                                int gate_stride, int gate_offset, float out_scale, int n_tokens,
                                int H, int G, int D, int V, int window, int keep_first,
                                float scale, int page_size, int cache_dtype, int out_dtype,
                                const int* listed, const int* plan_head, int* status,
                                void* stream) {
  if (!out || !q || !pool || !table || !tok_pos || !tok_req || !status || (listed && !plan_head))
    return HS_ERR_ARGUMENT;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0 || V > 1024 || window < 0 ||
      keep_first < 0 || page_size <= 0 ||
      (gate && (gate_offset < 0 || gate_offset + H * V > gate_stride)))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = ((size_t)D + (size_t)hs::SA_WARPS * (V + 2)) * sizeof(float);
  if (smem > 48 * 1024) return HS_ERR_UNSUPPORTED;
  const long long items = (long long)n_tokens * H;
  if (items > 0x7fffffffLL) return HS_ERR_TOO_LARGE;
  const dim3 grid((unsigned)items), blk(hs::SA_WARPS * 32);
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = hs_pdl_enabled();
  // 16-byte reads of a key row need rows that start and end on 16 bytes
  const int per16 = cache_dtype == HS_DT_BF16 ? 8 : 4;
  const int vec = (D % per16 == 0 && V % per16 == 0) ? 1 : 0;
  cudaError_t e;
#define HS_SA_LAUNCH_C(TC, TO, C)                                                                \
  e = hs_launch(hs::span_attention_kernel<TC, TO, C>, grid, blk, smem, st, pdl, (TO*)out, q,     \
                (const TC*)pool, table, max_pages, num_pages, tok_pos, tok_req, slopes, gate,    \
                gate_stride, gate_offset, out_scale, n_tokens, H, G, D, V, window, keep_first,   \
                scale, page_size, vec, listed, plan_head, status)
#define HS_SA_LAUNCH(TC, TO)                                                                     \
  do {                                                                                           \
    if (V <= 64) HS_SA_LAUNCH_C(TC, TO, 2);                                                      \
    else if (V <= 256) HS_SA_LAUNCH_C(TC, TO, 8);                                                \
    else HS_SA_LAUNCH_C(TC, TO, 32);                                                             \
  } while (0)
  if (cache_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_SA_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (cache_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_SA_LAUNCH(float, float);
  else return HS_ERR_UNSUPPORTED;
#undef HS_SA_LAUNCH
#undef HS_SA_LAUNCH_C
  return e == cudaSuccess ? HS_OK : (int)e;
}
