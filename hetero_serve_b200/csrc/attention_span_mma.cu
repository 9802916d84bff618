// Prompt portions of the attention with a distance slope, a window and kept first tokens, on
// the tensor cores (bfloat16 cache; key and value sizes that are multiples of 16 up to 128).
//
// The tiling is that of the other prompt-attention kernels of this library: a work item is up to
// 128 consecutive queries of one request x one query head, 8 warps of 16 queries, persistent CTAs
// that take items from a counter, 64 cache rows at a time through the block table into a ring of
// three cp.async stages, S = Q K^T and O += P V on mma.sync m16n8k16 with float32 accumulators,
// an online softmax in float32.  What differs:
//   * a cache row is [key (D) | value (V)] of one token and key/value head;
//   * query i sees j <= i with i - j < window (window 0: all) or j < keep_first.  The walk takes
//     first the kept rows that lie before the window of the item's FIRST query, then the token
//     rows from that window on (kept rows among them count by the second rule); the two ranges
//     are apart, so no key counts twice, and a warp skips tiles none of its rows see;
//   * the score loses slope_h * (i - j), in the accumulators;
//   * the queries arrive in float32 (normed or not) and are rounded once, into shared memory;
//   * the head's output may be multiplied element by element by the sigmoid of gate columns and
//     by a scale before it is rounded.
#include "common.cuh"

namespace hs {

constexpr int SP_BQ = 128, SP_BKV = 64, SP_WARPS = 8, SP_STAGES = 3;

struct SpanPrefillParams {
  const float* q;            // [T, heads * D]
  const __nv_bfloat16* pool;
  __nv_bfloat16* out;        // [T, heads * V]
  const int* table;
  const int* tile_info;      // per tile: first query's flat index, queries, request row, first position
  const int* plan_head;
  const float* slopes;       // [heads] or null
  const float* gate;         // [T, gate_stride] or null: column gate_offset + h * V + e
  int* status;
  int* work_counter;         // next work item; zero at launch
  int n_heads, n_kv_heads, page_size, num_pages, max_pages;
  int window, keep_first, gate_stride, gate_offset;
  float scale, out_scale;
};

// 16-byte chunks of a row of N numbers, permuted by the row inside groups of 8, 4 or 2 chunks
// (the largest power of two that divides the chunks of a row)
template <int N>
__device__ __forceinline__ int sp_swz(int row, int chunk) {
  constexpr int C = N / 8;
  constexpr int S = (C % 8 == 0) ? 8 : (C % 4 == 0) ? 4 : (C % 2 == 0) ? 2 : 1;
  return row * C + (chunk ^ (row & (S - 1)));
}

__device__ __forceinline__ void sp_cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void sp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void sp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void sp_ldsm(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void sp_ldsm_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void sp_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sp_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// kept first rows query i sees apart from its window: those behind it (window 0: none)
__device__ __forceinline__ int sp_seen(int i, int window, int keep_first) {
  if (window <= 0) return 0;
  const int behind = i - window + 1;               // positions wholly behind the window
  return behind > 0 ? min(behind, keep_first) : 0;
}

template <int D, int V>
__global__ void __launch_bounds__(SP_WARPS * 32, (V <= 64 && D <= 64 ? 2 : 1))
span_prefill_kernel(const SpanPrefillParams p) {
  constexpr int QC = D / 8, VC = V / 8;    // 16-byte chunks of a key and of a value
  constexpr int KSTEPS = D / 16;           // k-steps of Q K^T
  constexpr int DT = V / 8;                // n-tiles of the output
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint4* sQ = (uint4*)smem_raw;                          // [128][QC]
  uint4* sK = sQ + SP_BQ * QC;                           // [SP_STAGES][64][QC]
  uint4* sV = sK + SP_STAGES * SP_BKV * QC;              // [SP_STAGES][64][VC]

  __shared__ int s_item;
  pdl_trigger();
  pdl_wait();
  const int n_items = p.plan_head[1] * p.n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const float sc = p.scale * 1.4426950408889634f;        // scores in units of log2(e)
  while (true) {
  __syncthreads();            // the previous item's shared memory has been consumed
  if (threadIdx.x == 0) s_item = atomicAdd(p.work_counter, 1);
  __syncthreads();
  const int item = s_item;
  if (item >= n_items) break;
  const int tile = item / p.n_heads, h = item - tile * p.n_heads;
  const int4 ti = *(const int4*)(p.tile_info + 4 * tile);
  const int tok0 = ti.x, nq = ti.y, r = ti.z, pos0 = ti.w;
  if (r < 0 || nq <= 0 || pos0 < 0) continue;
  const int pos_last = pos0 + nq - 1;
  const int PS = p.page_size;
  if (pos_last / PS >= p.max_pages) {
    if (threadIdx.x == 0) atomicOr(p.status, HS_STATUS_BAD_POSITION);
    continue;
  }
  const int hk = h / (p.n_heads / p.n_kv_heads);
  const int* trow = p.table + (size_t)r * p.max_pages;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  // ---- Q tile -> shared memory, rounded to bfloat16 (rows past nq are zero)
  for (int c = threadIdx.x; c < SP_BQ * QC; c += blockDim.x) {
    const int row = c / QC, ch = c % QC;
    uint4 v = zero4;
    if (row < nq) {
      const float4* src =
          (const float4*)(p.q + ((size_t)(tok0 + row) * p.n_heads + h) * D + ch * 8);
      const float4 a = src[0], b = src[1];
      v = make_uint4(sp_pack(a.x, a.y), sp_pack(a.z, a.w), sp_pack(b.x, b.y), sp_pack(b.z, b.w));
    }
    sQ[sp_swz<D>(row, ch)] = v;
  }

  // the walk: tiles of kept first rows (those the item's last query sees behind its window),
  // then tiles of token rows from the window of the item's first query on.  Token rows between
  // the two are never read: their pages may have been given back already.
  const float slope = p.slopes ? p.slopes[h] * 1.4426950408889634f : 0.f;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int n_mean = min(sp_seen(pos_last, p.window, p.keep_first), key_lo);
  const int n_ct = (n_mean + SP_BKV - 1) / SP_BKV;
  const int kt_first = key_lo / SP_BKV;
  const int n_tiles = n_ct + pos_last / SP_BKV + 1 - kt_first;
  auto load_tile = [&](int u, int stage) {
    uint4* dK = sK + stage * SP_BKV * QC;
    uint4* dV = sV + stage * SP_BKV * VC;
    const bool mean = u < n_ct;
    const int j0 = mean ? u * SP_BKV : (kt_first + u - n_ct) * SP_BKV;
    const __nv_bfloat16* src_pool = p.pool;
    const int* tab = trow;
    const int tab_len = p.max_pages;
    const int n_pages = p.num_pages;
    for (int c = threadIdx.x; c < SP_BKV * (QC + VC); c += blockDim.x) {
      const int row = c / (QC + VC), ch = c % (QC + VC);
      const int j = j0 + row;
      bool ok = mean ? j < n_mean : (j >= key_lo && j <= pos_last);
      int page = 0, slot = 0;
      if (ok) {
        const int pg = j / PS;
        slot = j - pg * PS;
        page = pg < tab_len ? tab[pg] : -1;
        if (page < 0 || page >= n_pages) {
          atomicOr(p.status, HS_STATUS_BAD_PAGE);
          ok = false;
        }
      }
      uint4* dst = ch < QC ? &dK[sp_swz<D>(row, ch)] : &dV[sp_swz<V>(row, ch - QC)];
      if (ok) {
        const __nv_bfloat16* src =
            src_pool + (((size_t)page * p.n_kv_heads + hk) * PS + slot) * (size_t)(D + V) + ch * 8;
        sp_cp_async16(dst, src);
      } else {
        *dst = zero4;
      }
    }
  };

  // the first SP_STAGES-1 tiles are requested up front; one commit group per tile (empty ones too)
#pragma unroll
  for (int st = 0; st < SP_STAGES - 1; ++st) {
    if (st < n_tiles) load_tile(st, st);
    sp_commit();
  }
  __syncthreads();          // Q is in shared memory

  // ---- Q fragments stay in registers
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    sp_ldsm(qf[ks], &sQ[sp_swz<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4))]);

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int pos_a = min(pos0 + row_a, pos_last), pos_b = min(pos0 + row_b, pos_last);
  const int seen_a = min(sp_seen(pos_a, p.window, p.keep_first), n_mean);
  const int seen_b = min(sp_seen(pos_b, p.window, p.keep_first), n_mean);
  const int win = p.window > 0 ? p.window : 0x3fffffff;
  // what any query of this warp sees: mean rows below warp_seen, token rows from the window of
  // its first row to its last row's position; a warp whose rows are all past nq sees nothing
  const bool warp_live = warp * 16 < nq;
  const int warp_last = warp_live ? min(pos0 + warp * 16 + 15, pos_last) : -1;
  const int warp_lo = max(0, min(pos0 + warp * 16, pos_last) - win + 1);
  const int warp_seen = warp_live ? min(sp_seen(warp_last, p.window, p.keep_first), n_mean) : 0;

  for (int u = 0; u < n_tiles; ++u) {
    const int stage = u % SP_STAGES;
    sp_wait<SP_STAGES - 2>();           // tile u has landed (for this thread's copies)
    __syncthreads();                    // ... for everyone's; and tile u-1 has been consumed
    if (u + SP_STAGES - 1 < n_tiles) load_tile(u + SP_STAGES - 1, (u + SP_STAGES - 1) % SP_STAGES);
    sp_commit();
    const bool mean = u < n_ct;
    const int j0 = mean ? u * SP_BKV : (kt_first + u - n_ct) * SP_BKV;
    const bool live = mean ? j0 < warp_seen
                           : (j0 <= warp_last && (j0 + SP_BKV - 1 >= warp_lo || j0 < p.keep_first));
    if (live) {
      const uint4* tK = sK + stage * SP_BKV * QC;
      const uint4* tV = sV + stage * SP_BKV * VC;
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {           // pairs of 8-key tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = np * 16 + (mi >> 1) * 8 + (lane & 7);
          sp_ldsm(b, &tK[sp_swz<D>(key, ks * 2 + (mi & 1))]);
          sp_mma(s[np * 2], qf[ks], b[0], b[1]);
          sp_mma(s[np * 2 + 1], qf[ks], b[2], b[3]);
        }
      }
      // scale, mask, running maximum
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int j = j0 + nt * 8 + t * 2 + (c & 1);
          const int i = c < 2 ? pos_a : pos_b;
          // the kept rows below key_lo are walked first and count for a query that has them
          // behind its window; the token rows from key_lo on count inside the query's window or
          // as kept first rows.  The two ranges are apart, so no key counts twice.
          const bool sees = mean ? j < (c < 2 ? seen_a : seen_b)
                                 : (j <= i && (j > i - win || j < p.keep_first) && j >= key_lo);
          s[nt][c] = sees ? fmaf(s[nt][c], sc, -slope * (float)(i - j)) : -INFINITY;
        }
        mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      // a row whose rows of this tile are all masked keeps its state (mn == m); a row with
      // nothing at all yet (mn == -inf) contributes zeros
      const float ca = (mn_a == -INFINITY) ? 1.f : exp2f(m_a - mn_a);
      const float cb = (mn_b == -INFINITY) ? 1.f : exp2f(m_b - mn_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a;
      const float base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - base_a);
        s[nt][1] = exp2f(s[nt][1] - base_a);
        s[nt][2] = exp2f(s[nt][2] - base_b);
        s[nt][3] = exp2f(s[nt][3] - base_b);
        sum_a += s[nt][0] + s[nt][1];
        sum_b += s[nt][2] + s[nt][3];
      }
      l_a = l_a * ca + sum_a;
      l_b = l_b * cb + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] *= ca; o[i][1] *= ca; o[i][2] *= cb; o[i][3] *= cb;
      }
      // O += P V, 16 rows per k-step
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = sp_pack(s[2 * kk][0], s[2 * kk][1]);
        a[1] = sp_pack(s[2 * kk][2], s[2 * kk][3]);
        a[2] = sp_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = sp_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {      // pairs of 8-wide output tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
          sp_ldsm_t(b, &tV[sp_swz<V>(key, dp * 2 + (mi >> 1))]);
          sp_mma(o[dp * 2], a, b[0], b[1]);
          sp_mma(o[dp * 2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  sp_wait<0>();
  // ---- finish: the per-thread sums cover 2 of a row's 8 columns per tile; add the quad
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16* oa = p.out + ((size_t)(tok0 + row_a) * p.n_heads + h) * V;
  __nv_bfloat16* ob = p.out + ((size_t)(tok0 + row_b) * p.n_heads + h) * V;
  const float* ga = p.gate ? p.gate + (size_t)(tok0 + row_a) * p.gate_stride + p.gate_offset + (size_t)h * V : nullptr;
  const float* gb = p.gate ? p.gate + (size_t)(tok0 + row_b) * p.gate_stride + p.gate_offset + (size_t)h * V : nullptr;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const int e = i * 8 + t * 2;
    float va[2] = {o[i][0] * ia, o[i][1] * ia}, vb[2] = {o[i][2] * ib, o[i][3] * ib};
    if (row_a < nq) {
      if (ga) {
        va[0] *= 1.0f / (1.0f + expf(-ga[e]));
        va[1] *= 1.0f / (1.0f + expf(-ga[e + 1]));
      }
      *(uint32_t*)(oa + e) = sp_pack(va[0] * p.out_scale, va[1] * p.out_scale);
    }
    if (row_b < nq) {
      if (gb) {
        vb[0] *= 1.0f / (1.0f + expf(-gb[e]));
        vb[1] *= 1.0f / (1.0f + expf(-gb[e + 1]));
      }
      *(uint32_t*)(ob + e) = sp_pack(vb[0] * p.out_scale, vb[1] * p.out_scale);
    }
  }
  }   // next work item
}

template <int D, int V>
static int launch_span_prefill(const SpanPrefillParams& p, cudaStream_t st) {
  auto kern = span_prefill_kernel<D, V>;
  const int smem = (SP_BQ * D + SP_STAGES * SP_BKV * (D + V)) * 2;
  static int ctas = 0;   // persistent CTAs: as many as are resident at once
  if (ctas == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, SP_WARPS * 32, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 2) per_sm = 2;
    ctas = per_sm * hs_sm_count();
  }
  cudaError_t e = cudaMemsetAsync(p.work_counter, 0, sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  e = hs_launch(kern, dim3(ctas), dim3(SP_WARPS * 32), (size_t)smem, st, hs_pdl_enabled(), p);
  return e == cudaSuccess ? HS_OK : (int)e;
}

}  // namespace hs

// The tiles of the step's work list (prompt portions): tile_info as the plain prefill kernel's.
// Sizes this kernel does not take are refused with HS_ERR_UNSUPPORTED and nothing is launched.
HS_EXPORT int hs_span_attention_prefill(void* out, const float* q, const void* pool,
                                        const int* table, int max_pages, int num_pages,
                                        const int* tile_info, const int* plan_head, int tile_cap,
                                        int* work_counter, const float* slopes, const float* gate,
                                        int gate_stride, int gate_offset, float out_scale,
                                        int n_heads, int n_kv_heads, int head_dim, int value_dim,
                                        int window, int keep_first, float scale, int page_size,
                                        int* status, void* stream) {
  using namespace hs;
  if (!out || !q || !pool || !table || !tile_info || !plan_head || !status || !work_counter)
    return HS_ERR_ARGUMENT;
  if (tile_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 || window < 0 ||
      keep_first < 0 || max_pages <= 0 ||
      (gate && (gate_offset < 0 || gate_offset + n_heads * value_dim > gate_stride)))
    return HS_ERR_UNSUPPORTED;
  SpanPrefillParams p;
  p.q = q; p.pool = (const __nv_bfloat16*)pool; p.out = (__nv_bfloat16*)out; p.table = table;
  p.tile_info = tile_info; p.plan_head = plan_head; p.slopes = slopes; p.gate = gate;
  p.status = status; p.work_counter = work_counter;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.window = window;
  p.keep_first = keep_first; p.gate_stride = gate_stride; p.gate_offset = gate_offset;
  p.scale = scale; p.out_scale = out_scale;
  cudaStream_t st = (cudaStream_t)stream;
#define HS_SP_CASE(DD, VV) \
  if (head_dim == DD && value_dim == VV) return launch_span_prefill<DD, VV>(p, st)
  HS_SP_CASE(32, 32); HS_SP_CASE(48, 48); HS_SP_CASE(64, 64); HS_SP_CASE(96, 96);
  HS_SP_CASE(128, 128); HS_SP_CASE(64, 128); HS_SP_CASE(128, 64);
#undef HS_SP_CASE
  return HS_ERR_UNSUPPORTED;
}
