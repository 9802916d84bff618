// Block-diagonal linear on the CUDA cores, float32 accumulation:
//
//   out[t, g * n + j] = sum_k a[t, a_off + g * a_gstride + k] * w[g][k][j]
//
// `a` is float32 with row stride a_stride, so a group's input may be a slice of a wider row
// (the unrotated part of one head's query, say); the weights are held k-major ([groups, k, n],
// transposed once at binding) so that a warp's loads of one k are contiguous.  A block covers TT
// tokens x 32 output columns; its four warps each sum a quarter of k for every column, and the
// quarters are added in a fixed order, so a row's result depends on nothing else in the batch.
#include "common.cuh"
#include "mma_tiles.cuh"

namespace hs {

constexpr int GL_TT = 8;          // tokens a block covers
constexpr int GL_THREADS = 128;   // four warps: each takes a quarter of the summed index
constexpr int GL_COLS = 32;       // output columns a block covers (one a lane)

template <typename TW, typename TO>
__global__ void __launch_bounds__(GL_THREADS)
grouped_linear_kernel(TO* __restrict__ out, const float* __restrict__ a,
                      const TW* __restrict__ w, int n_tokens, int a_stride, int a_off,
                      int a_gstride, int groups, int n, int k) {
  extern __shared__ float s_a[];                    // [GL_TT][k]
  __shared__ float s_part[GL_THREADS / 32][GL_TT][GL_COLS];
  const int t0 = blockIdx.x * GL_TT;
  const int g = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.z * GL_COLS + lane;
  const int nt = min(GL_TT, n_tokens - t0);
  for (int i = threadIdx.x; i < GL_TT * k; i += GL_THREADS) {
    const int tt = i / k, kk = i - tt * k;
    s_a[i] = tt < nt ? a[(size_t)(t0 + tt) * a_stride + a_off + (size_t)g * a_gstride + kk] : 0.f;
  }
  __syncthreads();
  float acc[GL_TT];
#pragma unroll
  for (int tt = 0; tt < GL_TT; ++tt) acc[tt] = 0.f;
  const int per = (k + 3) / 4;
  const int k_lo = warp * per, k_hi = min(k, k_lo + per);
  if (j < n) {
    const TW* wg = w + (size_t)g * k * n + j;
#pragma unroll 8
    for (int kk = k_lo; kk < k_hi; ++kk) {
      const float wv = to_f(wg[(size_t)kk * n]);
#pragma unroll
      for (int tt = 0; tt < GL_TT; ++tt) acc[tt] = fmaf(s_a[tt * k + kk], wv, acc[tt]);
    }
  }
#pragma unroll
  for (int tt = 0; tt < GL_TT; ++tt) s_part[warp][tt][lane] = acc[tt];
  __syncthreads();
  // the four quarters are added in a fixed order: a row's sum never depends on the batch
  for (int i = threadIdx.x; i < GL_TT * GL_COLS; i += GL_THREADS) {
    const int tt = i / GL_COLS, c = i - tt * GL_COLS;
    const int col = blockIdx.z * GL_COLS + c;
    if (tt < nt && col < n) {
      const float v = ((s_part[0][tt][c] + s_part[1][tt][c]) + s_part[2][tt][c]) + s_part[3][tt][c];
      out[(size_t)(t0 + tt) * groups * n + (size_t)g * n + col] = from_f<TO>(v);
    }
  }
}

// The same product for many tokens in bfloat16, on the tensor cores: 64 tokens x 64 columns of
// one group a block, mma.sync m16n8k16.  The weights come n-major here ([groups, n, k], the
// summed index fastest); the float32 input slice is rounded to bfloat16 on its way into shared
// memory (fetched into registers a step ahead), the weights are copied asynchronously.
// SPLIT == 3: each input number is written as the sum of three bfloat16 terms (its rounding, the
// rounding of what is left, and again: 24 bits in all, a float32's whole mantissa) and the three
// products are summed in the same float32 accumulators.  A product of two bfloat16 numbers is
// exact in float32, so with weights that ARE bfloat16 numbers the result is the float32 product
// up to the order of its additions.
template <typename TO, int SPLIT>
__global__ void __launch_bounds__(128)
grouped_linear_mma_kernel(TO* __restrict__ out, const float* __restrict__ a,
                          const __nv_bfloat16* __restrict__ w, int n_tokens, int a_stride,
                          int a_off, int a_gstride, int groups, int N, int K, int vec) {
  __shared__ __align__(16) __nv_bfloat16 s_a[2][SPLIT][TM * TS];
  __shared__ __align__(16) __nv_bfloat16 s_b[2][TN * TS];
  const int t0 = blockIdx.x * TM, n0 = blockIdx.y * TN, g = blockIdx.z;
  const int rows = min(TM, n_tokens - t0), ncols = min(TN, N - n0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  const int gq = lane >> 2, tq = lane & 3;
  const float* a_base = a + (size_t)t0 * a_stride + a_off + (size_t)g * a_gstride;
  const __nv_bfloat16* b_base = w + ((size_t)g * N + n0) * K;
  auto b_row = [&](int r) { return b_base + (size_t)r * K; };
  float ra[2][8];
  auto fetch_a = [&](int k0) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = threadIdx.x + 128 * j;
      const int r = c >> 2, col = (c & 3) * 8;
      const float* src = a_base + (size_t)r * a_stride + k0 + col;
      if (r >= rows) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ra[j][i] = 0.f;
      } else if (vec) {
        const float4 u = *(const float4*)src, v = *(const float4*)(src + 4);
        ra[j][0] = u.x; ra[j][1] = u.y; ra[j][2] = u.z; ra[j][3] = u.w;
        ra[j][4] = v.x; ra[j][5] = v.y; ra[j][6] = v.z; ra[j][7] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) ra[j][i] = src[i];
      }
    }
  };
  auto store_a = [&](int buf) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int c = threadIdx.x + 128 * j;
#pragma unroll
      for (int term = 0; term < SPLIT; ++term) {
        __nv_bfloat162 p[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          p[i] = __floats2bfloat162_rn(ra[j][2 * i], ra[j][2 * i + 1]);
          if (term + 1 < SPLIT) {              // what this term leaves for the next (exact)
            ra[j][2 * i] -= __bfloat162float(p[i].x);
            ra[j][2 * i + 1] -= __bfloat162float(p[i].y);
          }
        }
        *(uint4*)(s_a[buf][term] + (c >> 2) * TS + (c & 3) * 8) = *(const uint4*)p;
      }
    }
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
  fetch_a(0);
  store_a(0);
  tile_copy(s_b[0], b_row, ncols, 0, w);
  asm volatile("cp.async.commit_group;");
  const int a_r = lane & 15, a_c = (lane >> 4) * 8;
  const int b_r = (lane & 7) + (lane >> 4) * 8, b_c = ((lane >> 3) & 1) * 8;
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += TK, buf ^= 1) {
    const bool more = k0 + TK < K;
    if (more) {
      fetch_a(k0 + TK);
      tile_copy(s_b[buf ^ 1], b_row, ncols, k0 + TK, w);
      asm volatile("cp.async.commit_group;");
      asm volatile("cp.async.wait_group 1;");
    } else {
      asm volatile("cp.async.wait_group 0;");
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk += 16) {
      uint32_t fb[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        ldmatrix_x4(fb[j], s_b[buf] + (wn + 16 * j + b_r) * TS + kk + b_c);
#pragma unroll
      for (int term = SPLIT - 1; term >= 0; --term) {      // the small terms first
        uint32_t fa[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
          ldmatrix_x4(fa[i], s_a[buf][term] + (wm + 16 * i + a_r) * TS + kk + a_c);
#pragma unroll
        for (int j = 0; j < 4; j += 2)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            mma_bf16(acc[i][j], fa[i], fb[j >> 1]);
            mma_bf16(acc[i][j + 1], fa[i], fb[j >> 1] + 2);
          }
      }
    }
    if (more) store_a(buf ^ 1);      // that stage was last read a turn ago, behind a barrier
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = wm + 16 * i + gq + 8 * half;
        if (r >= rows) continue;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int c = wn + 8 * j + 2 * tq + q;
          if (c < ncols)
            out[(size_t)(t0 + r) * groups * N + (size_t)g * N + n0 + c] =
                from_f<TO>(acc[i][j][2 * half + q]);
        }
      }
}

}  // namespace hs

HS_EXPORT int hs_grouped_linear(void* out, const float* a, const void* w, int n_tokens,
                                int a_stride, int a_off, int a_gstride, int groups, int n, int k,
                                int w_dtype, int out_dtype, void* stream) {
  if (!out || !a || !w) return HS_ERR_ARGUMENT;
  if (groups <= 0 || n <= 0 || k <= 0) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const size_t smem = (size_t)hs::GL_TT * k * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  dim3 grid((n_tokens + hs::GL_TT - 1) / hs::GL_TT, groups, (n + hs::GL_COLS - 1) / hs::GL_COLS);
  cudaStream_t st = (cudaStream_t)stream;
#define HS_GL(TW, TO)                                                                         \
  do {                                                                                        \
    auto kern = hs::grouped_linear_kernel<TW, TO>;                                            \
    if (smem > 48 * 1024)                                                                     \
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    kern<<<grid, hs::GL_THREADS, smem, st>>>((TO*)out, a, (const TW*)w, n_tokens, a_stride,  \
                                             a_off, a_gstride, groups, n, k);                 \
  } while (0)
  if (w_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_GL(float, float);
  else if (w_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32) HS_GL(__nv_bfloat16, float);
  else if (w_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_GL(__nv_bfloat16, __nv_bfloat16);
  else return HS_ERR_UNSUPPORTED;
#undef HS_GL
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// The tensor-core form: weights [groups, n, k] bfloat16; k a multiple of 32.  Returns
// HS_ERR_UNSUPPORTED for what it does not take (the caller then uses the kernel above).
HS_EXPORT int hs_grouped_linear_mma(void* out, const float* a, const void* w_nk, int n_tokens,
                                    int a_stride, int a_off, int a_gstride, int groups, int n,
                                    int k, int out_dtype, int split, void* stream) {
  if (!out || !a || !w_nk) return HS_ERR_ARGUMENT;
  if (groups <= 0 || n <= 0 || k <= 0 || k % hs::TK || (split != 1 && split != 3))
    return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  const int vec = a_stride % 4 == 0 && a_off % 4 == 0 && a_gstride % 4 == 0 && !((uintptr_t)a & 15);
  dim3 grid((n_tokens + hs::TM - 1) / hs::TM, (n + hs::TN - 1) / hs::TN, groups);
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == HS_DT_F32 && split == 3)
    hs::grouped_linear_mma_kernel<float, 3><<<grid, 128, 0, st>>>(
        (float*)out, a, (const __nv_bfloat16*)w_nk, n_tokens, a_stride, a_off, a_gstride, groups,
        n, k, vec);
  else if (split == 3)
    return HS_ERR_UNSUPPORTED;
  else if (out_dtype == HS_DT_F32)
    hs::grouped_linear_mma_kernel<float, 1><<<grid, 128, 0, st>>>(
        (float*)out, a, (const __nv_bfloat16*)w_nk, n_tokens, a_stride, a_off, a_gstride, groups,
        n, k, vec);
  else if (out_dtype == HS_DT_BF16)
    hs::grouped_linear_mma_kernel<__nv_bfloat16, 1><<<grid, 128, 0, st>>>(
        (__nv_bfloat16*)out, a, (const __nv_bfloat16*)w_nk, n_tokens, a_stride, a_off, a_gstride,
        groups, n, k, vec);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
