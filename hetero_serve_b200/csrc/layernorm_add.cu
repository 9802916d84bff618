// Layer norm of a sublayer's OUTPUT added into the float32 residual stream, and in the same
// launch the layer norm of the new rows for the sublayer that follows:
//
//   x   += (y - mean(y)) / sqrt(var(y) + eps) * g + b
//   out  = (x - mean(x)) / sqrt(var(x) + eps2) * g2 + b2          (optional; without g2: out = x,
//                                                                   the new rows in out's type)
//
// One block per row, the row in shared memory; mean first, then the mean of the squared
// deviations, each summed in an order fixed by the width: a row's result does not depend on its
// neighbours in the batch.  All statistics are float32.
//
//   learned_act    out = xIELU(z): z > 0: a_pos z^2 + z/2;  z <= 0: a_neg (e^z - 1 - z) + z/2,
//                  the two factors handed in by value (formed once from the learned numbers)
//   scale_softcap  t = cap * tanh(t * s / cap), in place
#include "common.cuh"

namespace hs {

constexpr int LNA_THREADS = 256;

__device__ __forceinline__ float lna_block_sum(float v, float* s_part) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_part[warp] = v;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < LNA_THREADS / 32; ++i) total += s_part[i];
  return total;
}

template <typename TO>
__global__ void __launch_bounds__(LNA_THREADS)
layernorm_add_kernel(float* __restrict__ x, const float* __restrict__ y,
                     const float* __restrict__ g, const float* __restrict__ b, float eps,
                     TO* __restrict__ out, const float* __restrict__ g2,
                     const float* __restrict__ b2, float eps2, int width) {
  extern __shared__ float s_row[];                     // [width]
  __shared__ float s_part[LNA_THREADS / 32];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  const float inv_w = 1.0f / (float)width;
  float s = 0.f;
  for (int e = threadIdx.x; e < width; e += LNA_THREADS) {
    const float v = y[row + e];
    s_row[e] = v;
    s += v;
  }
  const float mean = lna_block_sum(s, s_part) * inv_w;
  float ss = 0.f;
  for (int e = threadIdx.x; e < width; e += LNA_THREADS) {
    const float d = s_row[e] - mean;
    ss = fmaf(d, d, ss);
  }
  const float r = 1.0f / sqrtf(lna_block_sum(ss, s_part) * inv_w + eps);
  float s2 = 0.f;
  for (int e = threadIdx.x; e < width; e += LNA_THREADS) {
    const float v = x[row + e] + ((s_row[e] - mean) * r * g[e] + (b ? b[e] : 0.f));
    x[row + e] = v;
    s_row[e] = v;
    s2 += v;
    if (out != nullptr && g2 == nullptr) out[row + e] = from_f<TO>(v);   // the new rows as they are
  }
  if (out == nullptr || g2 == nullptr) return;
  const float mean2 = lna_block_sum(s2, s_part) * inv_w;
  float ss2 = 0.f;
  for (int e = threadIdx.x; e < width; e += LNA_THREADS) {
    const float d = s_row[e] - mean2;
    ss2 = fmaf(d, d, ss2);
  }
  const float r2 = 1.0f / sqrtf(lna_block_sum(ss2, s_part) * inv_w + eps2);
  for (int e = threadIdx.x; e < width; e += LNA_THREADS)
    out[row + e] = from_f<TO>((s_row[e] - mean2) * r2 * g2[e] + (b2 ? b2[e] : 0.f));
}

template <typename TO>
__global__ void learned_act_kernel(TO* __restrict__ out, const float* __restrict__ z, long long n,
                                   float a_pos, float a_neg) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = z[i];
    const float r = v > 0.f ? fmaf(a_pos * v, v, 0.5f * v)
                            : fmaf(a_neg, expm1f(v) - v, 0.5f * v);
    out[i] = from_f<TO>(r);
  }
}

__global__ void scale_softcap_kernel(float* __restrict__ t, long long n, float s, float cap) {
  pdl_trigger();
  pdl_wait();
  const float k = s / cap;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    t[i] = cap * tanhf(t[i] * k);
}

}  // namespace hs

HS_EXPORT int hs_layernorm_add(float* x, const float* y, const float* g, const float* b, float eps,
                               void* out, const float* g2, const float* b2, float eps2,
                               int n_rows, int width, int out_dtype, void* stream) {
  if (!x || !y || !g) return HS_ERR_ARGUMENT;
  if (width <= 0) return HS_ERR_UNSUPPORTED;
  if (n_rows <= 0) return HS_OK;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (out && out_dtype == HS_DT_BF16) {
    auto k = hs::layernorm_add_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = hs_launch(k, dim3(n_rows), dim3(hs::LNA_THREADS), smem, st, hs_pdl_enabled(), x, y, g, b,
                  eps, (__nv_bfloat16*)out, g2, b2, eps2, width);
  } else if (!out || out_dtype == HS_DT_F32) {
    auto k = hs::layernorm_add_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    e = hs_launch(k, dim3(n_rows), dim3(hs::LNA_THREADS), smem, st, hs_pdl_enabled(), x, y, g, b,
                  eps, (float*)out, g2, b2, eps2, width);
  } else {
    return HS_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_learned_act_xielu(void* out, const float* z, long long n, float a_pos,
                                   float a_neg, int out_dtype, void* stream) {
  if (!out || !z) return HS_ERR_ARGUMENT;
  if (n <= 0) return HS_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if (out_dtype == HS_DT_BF16)
    e = hs_launch(hs::learned_act_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, st,
                  hs_pdl_enabled(), (__nv_bfloat16*)out, z, n, a_pos, a_neg);
  else if (out_dtype == HS_DT_F32)
    e = hs_launch(hs::learned_act_kernel<float>, dim3((int)blocks), dim3(256), 0, st,
                  hs_pdl_enabled(), (float*)out, z, n, a_pos, a_neg);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_scale_softcap(float* t, long long n, float s, float cap, void* stream) {
  if (!t) return HS_ERR_ARGUMENT;
  if (!(cap > 0.f)) return HS_ERR_UNSUPPORTED;
  if (n <= 0) return HS_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  cudaError_t e = hs_launch(hs::scale_softcap_kernel, dim3((int)blocks), dim3(256), 0,
                            (cudaStream_t)stream, hs_pdl_enabled(), t, n, s, cap);
  return e == cudaSuccess ? HS_OK : (int)e;
}
