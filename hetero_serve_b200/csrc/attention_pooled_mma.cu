// Prompt portions of the attention over a sliding window plus pooled blocks, on the tensor
// cores (bfloat16 cache; key and value sizes 64 or 128, chosen apart).
//
// The tiling is that of the other prompt-attention kernels of this library: a work item is up to
// 128 consecutive queries of one request x one query head, 8 warps of 16 queries, persistent CTAs
// that take items from a counter, 64 cache rows at a time through the block table into a ring of
// three cp.async stages, S = Q K^T and O += P V on mma.sync m16n8k16 with float32 accumulators,
// an online softmax in float32.  What differs:
//   * a cache row is [key (D) | value (V)] of one token and key/value head, and there are two
//     kinds of rows under ONE softmax: the rows of means of the companion pool (row b stands for
//     the positions b*block .. b*block + block - 1), walked first, and the token rows;
//   * query i sees the mean rows b < max(0, (i - window + 1) / block) and the token rows
//     i - window < j <= i; the walk takes the mean rows the item's LAST query sees and the token
//     rows from the window of its FIRST query on, and a warp skips tiles none of its rows see;
//   * the queries arrive in float32 (normed and rotated) and are rounded once, into shared memory;
//   * the head's output is turned back by the query's position over all of V (number e pairs
//     with e + V/2: both halves of a pair sit in the same thread's accumulators).
#include "common.cuh"
#include "rotary.cuh"

namespace hs {

constexpr int PP_BQ = 128, PP_BKV = 64, PP_WARPS = 8, PP_STAGES = 3;

struct PooledPrefillParams {
  const float* q;            // [T, heads * D]
  const __nv_bfloat16* pool;
  const __nv_bfloat16* coarse;
  __nv_bfloat16* out;        // [T, heads * V]
  const int* table;
  const int* ctable;
  const int* tile_info;      // per tile: first query's flat index, queries, request row, first position
  const int* plan_head;
  const float* freq_v;       // [V / 2] or null: the output is not turned
  int* status;
  int* work_counter;         // next work item; zero at launch
  int n_heads, n_kv_heads, page_size, num_pages, max_pages, cnum_pages, cmax_pages;
  int window, block;
  float scale;
};

// 16-byte chunks of a row of N numbers, permuted inside groups of 8 by the row
template <int N>
__device__ __forceinline__ int pp_swz(int row, int chunk) {
  return row * (N / 8) + (chunk ^ (row & 7));
}

__device__ __forceinline__ void pp_cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void pp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void pp_ldsm(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void pp_ldsm_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void pp_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pp_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// mean rows query i sees: the blocks that end at or before i - window
__device__ __forceinline__ int pp_seen(int i, int window, int block) {
  const int behind = i - window + 1;               // positions wholly behind the window
  return behind > 0 ? behind / block : 0;
}

template <int D, int V>
__global__ void __launch_bounds__(PP_WARPS * 32, (V <= 64 ? 2 : 1))
pooled_prefill_kernel(const PooledPrefillParams p) {
  constexpr int QC = D / 8, VC = V / 8;    // 16-byte chunks of a key and of a value
  constexpr int KSTEPS = D / 16;           // k-steps of Q K^T
  constexpr int DT = V / 8;                // n-tiles of the output
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint4* sQ = (uint4*)smem_raw;                          // [128][QC]
  uint4* sK = sQ + PP_BQ * QC;                           // [PP_STAGES][64][QC]
  uint4* sV = sK + PP_STAGES * PP_BKV * QC;              // [PP_STAGES][64][VC]

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
  const int* crow = p.ctable + (size_t)r * p.cmax_pages;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  // ---- Q tile -> shared memory, rounded to bfloat16 (rows past nq are zero)
  for (int c = threadIdx.x; c < PP_BQ * QC; c += blockDim.x) {
    const int row = c / QC, ch = c % QC;
    uint4 v = zero4;
    if (row < nq) {
      const float4* src =
          (const float4*)(p.q + ((size_t)(tok0 + row) * p.n_heads + h) * D + ch * 8);
      const float4 a = src[0], b = src[1];
      v = make_uint4(pp_pack(a.x, a.y), pp_pack(a.z, a.w), pp_pack(b.x, b.y), pp_pack(b.z, b.w));
    }
    sQ[pp_swz<D>(row, ch)] = v;
  }

  // the walk: tiles of mean rows (those the item's last query sees), then tiles of token rows
  // from the window of the item's first query on.  Token rows before it are never read: their
  // pages may have been given back already.
  const int n_mean = pp_seen(pos_last, p.window, p.block);
  const int n_ct = (n_mean + PP_BKV - 1) / PP_BKV;
  const int key_lo = max(0, pos0 - p.window + 1);
  const int kt_first = key_lo / PP_BKV;
  const int n_tiles = n_ct + pos_last / PP_BKV + 1 - kt_first;
  auto load_tile = [&](int u, int stage) {
    uint4* dK = sK + stage * PP_BKV * QC;
    uint4* dV = sV + stage * PP_BKV * VC;
    const bool mean = u < n_ct;
    const int j0 = mean ? u * PP_BKV : (kt_first + u - n_ct) * PP_BKV;
    const __nv_bfloat16* src_pool = mean ? p.coarse : p.pool;
    const int* tab = mean ? crow : trow;
    const int tab_len = mean ? p.cmax_pages : p.max_pages;
    const int n_pages = mean ? p.cnum_pages : p.num_pages;
    for (int c = threadIdx.x; c < PP_BKV * (QC + VC); c += blockDim.x) {
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
      uint4* dst = ch < QC ? &dK[pp_swz<D>(row, ch)] : &dV[pp_swz<V>(row, ch - QC)];
      if (ok) {
        const __nv_bfloat16* src =
            src_pool + (((size_t)page * p.n_kv_heads + hk) * PS + slot) * (size_t)(D + V) + ch * 8;
        pp_cp_async16(dst, src);
      } else {
        *dst = zero4;
      }
    }
  };

  // the first PP_STAGES-1 tiles are requested up front; one commit group per tile (empty ones too)
#pragma unroll
  for (int st = 0; st < PP_STAGES - 1; ++st) {
    if (st < n_tiles) load_tile(st, st);
    pp_commit();
  }
  __syncthreads();          // Q is in shared memory

  // ---- Q fragments stay in registers
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    pp_ldsm(qf[ks], &sQ[pp_swz<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4))]);

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int pos_a = min(pos0 + row_a, pos_last), pos_b = min(pos0 + row_b, pos_last);
  const int seen_a = pp_seen(pos_a, p.window, p.block), seen_b = pp_seen(pos_b, p.window, p.block);
  // what any query of this warp sees: mean rows below warp_seen, token rows from the window of
  // its first row to its last row's position; a warp whose rows are all past nq sees nothing
  const bool warp_live = warp * 16 < nq;
  const int warp_last = warp_live ? min(pos0 + warp * 16 + 15, pos_last) : -1;
  const int warp_lo = max(0, min(pos0 + warp * 16, pos_last) - p.window + 1);
  const int warp_seen = warp_live ? pp_seen(warp_last, p.window, p.block) : 0;

  for (int u = 0; u < n_tiles; ++u) {
    const int stage = u % PP_STAGES;
    pp_wait<PP_STAGES - 2>();           // tile u has landed (for this thread's copies)
    __syncthreads();                    // ... for everyone's; and tile u-1 has been consumed
    if (u + PP_STAGES - 1 < n_tiles) load_tile(u + PP_STAGES - 1, (u + PP_STAGES - 1) % PP_STAGES);
    pp_commit();
    const bool mean = u < n_ct;
    const int j0 = mean ? u * PP_BKV : (kt_first + u - n_ct) * PP_BKV;
    const bool live = mean ? j0 < warp_seen : (j0 <= warp_last && j0 + PP_BKV - 1 >= warp_lo);
    if (live) {
      const uint4* tK = sK + stage * PP_BKV * QC;
      const uint4* tV = sV + stage * PP_BKV * VC;
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
          pp_ldsm(b, &tK[pp_swz<D>(key, ks * 2 + (mi & 1))]);
          pp_mma(s[np * 2], qf[ks], b[0], b[1]);
          pp_mma(s[np * 2 + 1], qf[ks], b[2], b[3]);
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
          const bool sees = mean ? j < (c < 2 ? seen_a : seen_b) : (j <= i && j > i - p.window);
          s[nt][c] = sees ? s[nt][c] * sc : -INFINITY;
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
        a[0] = pp_pack(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pp_pack(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pp_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pp_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {      // pairs of 8-wide output tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
          pp_ldsm_t(b, &tV[pp_swz<V>(key, dp * 2 + (mi >> 1))]);
          pp_mma(o[dp * 2], a, b[0], b[1]);
          pp_mma(o[dp * 2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  pp_wait<0>();
  // ---- finish: the per-thread sums cover 2 of a row's 8 columns per tile; add the quad
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16* oa = p.out + ((size_t)(tok0 + row_a) * p.n_heads + h) * V;
  __nv_bfloat16* ob = p.out + ((size_t)(tok0 + row_b) * p.n_heads + h) * V;
#pragma unroll
  for (int i = 0; i < DT / 2; ++i) {
    // numbers e = i*8 + t*2 (+1) of the first half and their partners e + V/2
    float lo[4] = {o[i][0] * ia, o[i][1] * ia, o[i][2] * ib, o[i][3] * ib};
    float hi[4] = {o[i + DT / 2][0] * ia, o[i + DT / 2][1] * ia, o[i + DT / 2][2] * ib,
                   o[i + DT / 2][3] * ib};
    const int e = i * 8 + t * 2;
    if (p.freq_v != nullptr) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float cs, sn;
        pair_angle(c < 2 ? pos_a : pos_b, p.freq_v[e + (c & 1)], &cs, &sn);
        const float x = lo[c], y = hi[c];
        lo[c] = x * cs + y * sn;                 // the angle negated
        hi[c] = y * cs - x * sn;
      }
    }
    if (row_a < nq) {
      *(uint32_t*)(oa + e) = pp_pack(lo[0], lo[1]);
      *(uint32_t*)(oa + e + V / 2) = pp_pack(hi[0], hi[1]);
    }
    if (row_b < nq) {
      *(uint32_t*)(ob + e) = pp_pack(lo[2], lo[3]);
      *(uint32_t*)(ob + e + V / 2) = pp_pack(hi[2], hi[3]);
    }
  }
  }   // next work item
}

template <int D, int V>
static int launch_pooled_prefill(const PooledPrefillParams& p, cudaStream_t st) {
  auto kern = pooled_prefill_kernel<D, V>;
  const int smem = (PP_BQ * D + PP_STAGES * PP_BKV * (D + V)) * 2;
  static int ctas = 0;   // persistent CTAs: as many as are resident at once
  if (ctas == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, PP_WARPS * 32, smem);
    if (e != cudaSuccess) return (int)e;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 2) per_sm = 2;
    ctas = per_sm * hs_sm_count();
  }
  cudaError_t e = cudaMemsetAsync(p.work_counter, 0, sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  e = hs_launch(kern, dim3(ctas), dim3(PP_WARPS * 32), (size_t)smem, st, hs_pdl_enabled(), p);
  return e == cudaSuccess ? HS_OK : (int)e;
}

}  // namespace hs

// The tiles of the step's work list (prompt portions): tile_info as the plain prefill kernel's.
// Sizes this kernel does not take are refused with HS_ERR_UNSUPPORTED and nothing is launched.
HS_EXPORT int hs_pooled_attention_prefill(void* out, const float* q, const void* pool,
                                          const int* table, int max_pages, int num_pages,
                                          const void* coarse, const int* ctable, int cmax_pages,
                                          int cnum_pages, const int* tile_info,
                                          const int* plan_head, int tile_cap, int* work_counter,
                                          const float* freq_v, int n_heads, int n_kv_heads,
                                          int head_dim, int value_dim, int window, int block,
                                          float scale, int page_size, int* status, void* stream) {
  using namespace hs;
  if (!out || !q || !pool || !table || !coarse || !ctable || !tile_info || !plan_head ||
      !status || !work_counter)
    return HS_ERR_ARGUMENT;
  if (tile_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || page_size <= 0 ||
      window <= 0 || block <= 0 || max_pages <= 0 || cmax_pages <= 0)
    return HS_ERR_UNSUPPORTED;
  PooledPrefillParams p;
  p.q = q; p.pool = (const __nv_bfloat16*)pool; p.coarse = (const __nv_bfloat16*)coarse;
  p.out = (__nv_bfloat16*)out; p.table = table; p.ctable = ctable; p.tile_info = tile_info;
  p.plan_head = plan_head; p.freq_v = freq_v; p.status = status; p.work_counter = work_counter;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.cnum_pages = cnum_pages;
  p.cmax_pages = cmax_pages; p.window = window; p.block = block; p.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  if (head_dim == 64 && value_dim == 64) return launch_pooled_prefill<64, 64>(p, st);
  if (head_dim == 64 && value_dim == 128) return launch_pooled_prefill<64, 128>(p, st);
  if (head_dim == 128 && value_dim == 64) return launch_pooled_prefill<128, 64>(p, st);
  if (head_dim == 128 && value_dim == 128) return launch_pooled_prefill<128, 128>(p, st);
  return HS_ERR_UNSUPPORTED;
}
