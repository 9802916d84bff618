// Root-mean-square norms on the float32 residual stream.
//
//   rms_norm       out[i] = x[r] / sqrt(mean(x[r]^2) + eps) * w   (r = rows[i] or i), optionally
//                  with one-plus weights (1 + w) and a sigmoid gate per element,
//                  out *= sigmoid(gate[i, g_off + e]).
//   rms_norm_add   the norm of a sublayer's OUTPUT added into the stream:
//                      y = a                                        (one input), or
//                      y = mix * (rms(a) * wa + rms(b) * wb)        (two inputs side by side)
//                      x += rms(y) * w    (w null: x += y, no outer norm)
//                      h = x in the compute type (optional copy for the projections of the
//                      next sublayer)
//   cast_rows      h = x in the compute type.
//
// One block per row; every sum of squares is taken per row in an order fixed by the width, so a
// row's result does not depend on its neighbours in the batch.  All statistics are float32; the
// divisions and roots are the accurate ones.
#include "common.cuh"

namespace hs {

constexpr int RMS_THREADS = 256;

// sum over the block, the same order for every row: lanes by butterfly, warps in index order
__device__ __forceinline__ float block_sum(float v, float* s_part) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // s_part may still be read from the sum before
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < RMS_THREADS / 32; ++i) total += s_part[i];
  return total;
}

template <typename TO>
__global__ void __launch_bounds__(RMS_THREADS)
rms_norm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                const int* __restrict__ rows, int width, float eps, int one_plus,
                const float* __restrict__ gate, int g_off, int g_stride) {
  __shared__ float s_part[RMS_THREADS / 32];
  pdl_trigger();
  pdl_wait();
  const int o = blockIdx.x;
  const int src = rows ? rows[o] : o;
  const float* xr = x + (size_t)src * width;
  float ss = 0.f;
  for (int e = threadIdx.x; e < width; e += RMS_THREADS) ss = fmaf(xr[e], xr[e], ss);
  const float r = 1.0f / sqrtf(block_sum(ss, s_part) / (float)width + eps);
  TO* orow = out + (size_t)o * width;
  const float* gr = gate ? gate + (size_t)src * g_stride + g_off : nullptr;
  for (int e = threadIdx.x; e < width; e += RMS_THREADS) {
    float v = xr[e] * r * (one_plus ? 1.0f + w[e] : w[e]);
    if (gr) v = v / (1.0f + expf(-gr[e]));
    orow[e] = from_f<TO>(v);
  }
}

template <typename TH>
__global__ void __launch_bounds__(RMS_THREADS)
rms_norm_add_kernel(float* __restrict__ x, TH* __restrict__ h, const float* __restrict__ a,
                    const float* __restrict__ wa, const float* __restrict__ b,
                    const float* __restrict__ wb, float mix, const float* __restrict__ w,
                    int width, float eps_in, float eps, const float* __restrict__ ln_g,
                    const float* __restrict__ ln_b, float ln_eps) {
  extern __shared__ float s_y[];                       // [width]
  __shared__ float s_part[RMS_THREADS / 32];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  const float* ar = a + row;
  if (b) {
    const float* br = b + row;
    float sa = 0.f, sb = 0.f;
    for (int e = threadIdx.x; e < width; e += RMS_THREADS) {
      sa = fmaf(ar[e], ar[e], sa);
      sb = fmaf(br[e], br[e], sb);
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, s_part) / (float)width + eps_in);
    const float rb = 1.0f / sqrtf(block_sum(sb, s_part) / (float)width + eps_in);
    for (int e = threadIdx.x; e < width; e += RMS_THREADS)
      s_y[e] = mix * (ar[e] * ra * wa[e] + br[e] * rb * wb[e]);
  } else {
    for (int e = threadIdx.x; e < width; e += RMS_THREADS) s_y[e] = ar[e];
  }
  float r = 1.0f;
  if (w) {
    float ss = 0.f;                                    // each thread reads back its own entries
    for (int e = threadIdx.x; e < width; e += RMS_THREADS) ss = fmaf(s_y[e], s_y[e], ss);
    r = 1.0f / sqrtf(block_sum(ss, s_part) / (float)width + eps);
  }
  float* xr = x + row;
  for (int e = threadIdx.x; e < width; e += RMS_THREADS) {
    const float v = xr[e] + (w ? s_y[e] * r * w[e] : s_y[e]);
    xr[e] = v;
    if (ln_g) s_y[e] = v;                              // read back below by this thread alone
    else if (h) h[row + e] = from_f<TH>(v);
  }
  if (ln_g == nullptr || h == nullptr) return;
  // h = the layer norm of the new row (the norm in front of the sublayer that runs next): the
  // mean first, then the mean of the squared deviations
  float sm = 0.f;
  for (int e = threadIdx.x; e < width; e += RMS_THREADS) sm += s_y[e];
  const float mean = block_sum(sm, s_part) / (float)width;
  float sq = 0.f;
  for (int e = threadIdx.x; e < width; e += RMS_THREADS) {
    const float d = s_y[e] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, s_part) / (float)width + ln_eps);
  for (int e = threadIdx.x; e < width; e += RMS_THREADS)
    h[row + e] = from_f<TH>(fmaf((s_y[e] - mean) * rstd, ln_g[e], ln_b ? ln_b[e] : 0.f));
}

__global__ void cast_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ x,
                                 long long n) {
  pdl_trigger();
  pdl_wait();
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const long long step = (long long)gridDim.x * blockDim.x * 4;
  for (; i < n; i += step) {
    if (i + 3 < n && ((((uintptr_t)(x + i)) & 15) == 0) && ((((uintptr_t)(out + i)) & 7) == 0)) {
      const float4 v = *(const float4*)(x + i);
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 pk;
      pk.x = *(uint32_t*)&lo;
      pk.y = *(uint32_t*)&hi;
      *(uint2*)(out + i) = pk;
    } else {
      for (int j = 0; j < 4 && i + j < n; ++j) out[i + j] = __float2bfloat16_rn(x[i + j]);
    }
  }
}

}  // namespace hs

HS_EXPORT int hs_rms_norm(void* out, const float* x, const float* w, const int* rows, int n_rows,
                          int width, float eps, int one_plus, const float* gate, int g_off,
                          int g_stride, int out_dtype, void* stream) {
  if (!out || !x || !w) return HS_ERR_ARGUMENT;
  if (width <= 0) return HS_ERR_UNSUPPORTED;
  if (n_rows <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool pdl = hs_pdl_enabled();
  cudaError_t e = cudaSuccess;
  if (out_dtype == HS_DT_F32)
    e = hs_launch(hs::rms_norm_kernel<float>, dim3(n_rows), dim3(hs::RMS_THREADS), 0, st, pdl,
                  (float*)out, x, w, rows, width, eps, one_plus, gate, g_off, g_stride);
  else if (out_dtype == HS_DT_BF16)
    e = hs_launch(hs::rms_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(hs::RMS_THREADS), 0, st,
                  pdl, (__nv_bfloat16*)out, x, w, rows, width, eps, one_plus, gate, g_off,
                  g_stride);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

// h_dtype: the type of the optional copy `h` (ignored when h is null).  With ln_g (and ln_b or
// null), h receives the layer norm of the new rows instead of the rows themselves.
HS_EXPORT int hs_rms_norm_add(float* x, void* h, const float* a, const float* wa, const float* b,
                              const float* wb, float mix, const float* w, int n_rows, int width,
                              float eps_in, float eps, int h_dtype, const float* ln_g,
                              const float* ln_b, float ln_eps, void* stream) {
  if (!x || !a || (b && (!wa || !wb)) || (ln_g && !h)) return HS_ERR_ARGUMENT;
  if (width <= 0) return HS_ERR_UNSUPPORTED;
  if (n_rows <= 0) return HS_OK;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (h && h_dtype == HS_DT_BF16) {
    auto k = hs::rms_norm_add_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = hs_launch(k, dim3(n_rows), dim3(hs::RMS_THREADS), smem, st, hs_pdl_enabled(), x,
                  (__nv_bfloat16*)h, a, wa, b, wb, mix, w, width, eps_in, eps, ln_g, ln_b, ln_eps);
  } else if (!h || h_dtype == HS_DT_F32) {
    auto k = hs::rms_norm_add_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = hs_launch(k, dim3(n_rows), dim3(hs::RMS_THREADS), smem, st, hs_pdl_enabled(), x,
                  (float*)h, a, wa, b, wb, mix, w, width, eps_in, eps, ln_g, ln_b, ln_eps);
  } else {
    return HS_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_cast_rows(void* out, const float* x, long long n, void* stream) {
  if (!out || !x) return HS_ERR_ARGUMENT;
  if (n <= 0) return HS_OK;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  cudaError_t e = hs_launch(hs::cast_rows_kernel, dim3((int)blocks), dim3(256), 0,
                            (cudaStream_t)stream, hs_pdl_enabled(), (__nv_bfloat16*)out, x, n);
  return e == cudaSuccess ? HS_OK : (int)e;
}
