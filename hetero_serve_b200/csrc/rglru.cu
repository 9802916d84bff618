// The real-gated linear recurrent unit: short convolution, gates, decay and the recurrence.
//
//   rglru_conv   u[t, c] = cb[c] + sum_j cw[c, taps-1-j] * xb[t-j, c]   (causal; rows before the
//                portion's first token come from the request's history of taps-1 inputs, which
//                is zero for a new request)
//   rglru_scan   r = sigmoid(z_r + b_r), i = sigmoid(z_i + b_i)    (z: the block-diagonal
//                products of u, columns [part][r | i][n])
//                log a = -scale * r * rate[c];  a = exp(log a)
//                S <- a S + sqrt(1 - a^2) i u;   out = S * gelu_tanh(y)
//                then the state and the convolution's history are stored for the next step.
//
// Everything here is float32 (only `out`, the input of the output projection, is written in
// the compute type).  The recurrence of one (request, channel) is linear, S <- a S + d, so the
// portion is cut into up to 32 or 64 segments of equal length: every segment is first reduced
// to its pair (product of a, result from zero), the carries are chained in index order, and
// the segment is walked again from its carry.  The cut depends on the portion's length and the layer's channels only;
// sqrt(1 - a^2) is formed as sqrt(-expm1(2 log a)), which keeps its digits when a is near 1.
#include "common.cuh"

namespace hs {

constexpr int RG_THREADS = 1024; // a block: RG_CH channels x RG_THREADS / RG_CH segments
constexpr int RG_WIDE = 1024;    // up to this many channels a block covers 16 of them and cuts a
                                 // portion into 64 segments (more blocks than 32 channels give,
                                 // which few channels need to fill the device); beyond, 32 and 32
constexpr int RG_MIN_SEG = 8;    // shortest segment: short portions use fewer warps
constexpr int RG_AHEAD = 4;      // steps whose inputs are in flight together

__global__ void __launch_bounds__(256)
rglru_conv_kernel(float* __restrict__ u, const float* __restrict__ proj, int proj_stride,
                  int x_off, const float* __restrict__ cw, const float* __restrict__ cb,
                  const float* __restrict__ state, int state_stride,
                  const int* __restrict__ tok_req, const int* __restrict__ req_start,
                  const int* __restrict__ req_slot, int C, int taps) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = tok_req[t];
  if (r < 0 || c >= C) return;
  const int local = t - req_start[r];
  const float* hist = state + (size_t)req_slot[r] * state_stride + C;     // [taps-1][C]
  float acc = cb[c];
  for (int j = 0; j < taps; ++j) {
    const int back = local - j;
    const float v = back >= 0 ? proj[(size_t)(t - j) * proj_stride + x_off + c]
                              : hist[(size_t)(taps - 1 + back) * C + c];
    acc = fmaf(cw[(size_t)c * taps + (taps - 1 - j)], v, acc);
  }
  u[(size_t)t * C + c] = acc;
}

struct RgStep { float a, d; };

__device__ __forceinline__ RgStep rg_step(float zr, float zi, float uu, float rate, float scale) {
  const float rg = 1.0f / (1.0f + expf(-zr));
  const float ig = 1.0f / (1.0f + expf(-zi));
  const float log_a = -scale * rg * rate;
  RgStep s;
  s.a = expf(log_a);
  s.d = sqrtf(-expm1f(2.0f * log_a)) * ig * uu;
  return s;
}

template <typename TO, int RG_CH>
__global__ void __launch_bounds__(RG_THREADS)
rglru_scan_kernel(TO* __restrict__ out, float* __restrict__ state, int state_stride,
                  const float* __restrict__ u, const float* __restrict__ z,
                  const float* __restrict__ proj, int proj_stride, int y_off, int x_off,
                  const float* __restrict__ b_gates, const float* __restrict__ rate,
                  const int* __restrict__ req_start, const int* __restrict__ req_len,
                  const int* __restrict__ req_slot, int C, int n_per, int taps, float scale) {
  constexpr int RG_PARTS = RG_THREADS / RG_CH;
  __shared__ float s_a[RG_PARTS][RG_CH], s_d[RG_PARTS][RG_CH];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int n = req_len[r];
  if (n <= 0) return;
  const int t0 = req_start[r];
  const int lane = threadIdx.x % RG_CH, part = threadIdx.x / RG_CH;
  const int c = blockIdx.x * RG_CH + lane;
  const bool live = c < C;
  int seg = (n + RG_PARTS - 1) / RG_PARTS;
  if (seg < RG_MIN_SEG) seg = RG_MIN_SEG;
  const int lo = part * seg, hi = min(n, lo + seg);
  // column of this channel's gate logits: [part of the channels][r | i][n_per]
  const int blk = live ? c / n_per : 0;
  const int zc = blk * 2 * n_per + (c - blk * n_per);
  float br = 0.f, bi = 0.f, rt = 0.f;
  if (live) { br = b_gates[zc]; bi = b_gates[zc + n_per]; rt = rate[c]; }
  float* st = state + (size_t)req_slot[r] * state_stride;
  // pass 1: the segment as one step (A, D): S_out = A * S_in + D.  A portion that fits into
  // one segment is walked once, in pass 2.
  const bool single = n <= seg;
  const float S0 = live ? st[c] : 0.f;          // read before the barrier: the last segment's
  float A = 1.f, D = 0.f;                        // owner stores the new state behind it
  if (live && !single) {
    // RG_AHEAD steps' inputs are loaded before the first is used (rows past the segment's end
    // read its first row again and are dropped)
    for (int i = lo; i < hi; i += RG_AHEAD) {
      float zr[RG_AHEAD], zi[RG_AHEAD], uu[RG_AHEAD];
#pragma unroll
      for (int k = 0; k < RG_AHEAD; ++k) {
        const size_t t = (size_t)(t0 + (i + k < hi ? i + k : lo));
        zr[k] = z[t * 2 * C + zc];
        zi[k] = z[t * 2 * C + zc + n_per];
        uu[k] = u[t * C + c];
      }
#pragma unroll
      for (int k = 0; k < RG_AHEAD; ++k) {
        if (i + k >= hi) break;
        const RgStep s = rg_step(zr[k] + br, zi[k] + bi, uu[k], rt, scale);
        A *= s.a;
        D = fmaf(s.a, D, s.d);
      }
    }
  }
  s_a[part][lane] = A;
  s_d[part][lane] = D;
  __syncthreads();
  if (!live || lo >= n) return;
  // pass 2: the carries of the segments before, in index order, then the segment itself
  float S = S0;
  for (int p = 0; p < part; ++p) S = fmaf(s_a[p][lane], S, s_d[p][lane]);
  for (int i = lo; i < hi; i += RG_AHEAD) {
    float zr[RG_AHEAD], zi[RG_AHEAD], uu[RG_AHEAD], yy[RG_AHEAD];
#pragma unroll
    for (int k = 0; k < RG_AHEAD; ++k) {
      const size_t t = (size_t)(t0 + (i + k < hi ? i + k : lo));
      zr[k] = z[t * 2 * C + zc];
      zi[k] = z[t * 2 * C + zc + n_per];
      uu[k] = u[t * C + c];
      yy[k] = proj[t * proj_stride + y_off + c];
    }
#pragma unroll
    for (int k = 0; k < RG_AHEAD; ++k) {
      if (i + k >= hi) break;
      const RgStep s = rg_step(zr[k] + br, zi[k] + bi, uu[k], rt, scale);
      S = fmaf(s.a, S, s.d);
      out[(size_t)(t0 + i + k) * C + c] = from_f<TO>(S * gelu_tanh(yy[k]));
    }
  }
  if (hi == n) {
    st[c] = S;
    // the last taps-1 inputs of the convolution, oldest first: old history, then this portion
    float* hist = st + C;
    for (int k = 0; k < taps - 1; ++k) {
      const int idx = n + k;             // place in (old history ++ portion)
      hist[(size_t)k * C + c] = idx < taps - 1
          ? hist[(size_t)idx * C + c]
          : proj[(size_t)(t0 + idx - (taps - 1)) * proj_stride + x_off + c];
    }
  }
}

// One token of every request: convolution, gates, decay, the state's step and the history in
// ONE launch.  A block takes one part of the channels for up to RS_TT tokens (so the part's gate
// matrices are read once for all of them): the part's n convolved inputs of each token go to
// shared memory, the 2n gate sums are formed from them as the block-diagonal kernel forms them
// (a warp sums a quarter of the inputs for 32 columns, the four quarters are added in the same
// order; eight such column groups are in flight), then a thread per (token, channel) steps the
// state.  Every sum has the order it has on the path of three launches, so a token's result is
// the same bits on both.
constexpr int RS_THREADS = 1024;
constexpr int RS_TT = 8;

template <typename TO>
__global__ void __launch_bounds__(RS_THREADS)
rglru_step_kernel(TO* __restrict__ out, float* __restrict__ state, int state_stride,
                  const float* __restrict__ proj, int proj_stride, int y_off, int x_off,
                  const float* __restrict__ cw, const float* __restrict__ cb,
                  const float* __restrict__ w_gates, const float* __restrict__ b_gates,
                  const float* __restrict__ rate, const int* __restrict__ tok_req,
                  const int* __restrict__ req_slot, int n_tokens, int C, int n_per, int taps,
                  float scale) {
  extern __shared__ float s_rs[];            // u [RS_TT][n_per] | partial sums [4][RS_TT][2 n_per]
  __shared__ int s_slot[RS_TT];
  float* s_u = s_rs;
  float* s_z = s_rs + RS_TT * n_per;
  pdl_trigger();
  pdl_wait();
  const int blk = blockIdx.x, t0 = blockIdx.y * RS_TT;
  if (threadIdx.x < RS_TT) {
    const int t = t0 + threadIdx.x;
    const int r = t < n_tokens ? tok_req[t] : -1;
    s_slot[threadIdx.x] = r >= 0 ? req_slot[r] : -1;
  }
  __syncthreads();
  const int c0 = blk * n_per;
  for (int idx = threadIdx.x; idx < RS_TT * n_per; idx += RS_THREADS) {
    const int tt = idx / n_per, i = idx - tt * n_per;
    const int c = c0 + i;
    float acc = 0.f;
    if (s_slot[tt] >= 0) {
      const float* hist = state + (size_t)s_slot[tt] * state_stride + C;   // [taps-1][C]
      const float* row = proj + (size_t)(t0 + tt) * proj_stride;
      acc = cb[c];
      for (int j = 0; j < taps; ++j) {
        const float v = j == 0 ? row[x_off + c] : hist[(size_t)(taps - 1 - j) * C + c];
        acc = fmaf(cw[(size_t)c * taps + (taps - 1 - j)], v, acc);
      }
    }
    s_u[idx] = acc;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quarter = warp & 3, lane_group = warp >> 2;          // 8 column groups in flight
  const int n_out = 2 * n_per;
  const int per = (n_per + 3) / 4;
  const int k_lo = quarter * per, k_hi = min(n_per, k_lo + per);
  const float* wg = w_gates + (size_t)blk * n_per * n_out;
  for (int j0 = lane_group * 32; j0 < n_out; j0 += (RS_THREADS / 128) * 32) {
    const int j = j0 + lane;
    if (j >= n_out) continue;
    float acc[RS_TT];
#pragma unroll
    for (int tt = 0; tt < RS_TT; ++tt) acc[tt] = 0.f;
#pragma unroll 8
    for (int kk = k_lo; kk < k_hi; ++kk) {
      const float wv = wg[(size_t)kk * n_out + j];
#pragma unroll
      for (int tt = 0; tt < RS_TT; ++tt) acc[tt] = fmaf(s_u[tt * n_per + kk], wv, acc[tt]);
    }
#pragma unroll
    for (int tt = 0; tt < RS_TT; ++tt) s_z[(quarter * RS_TT + tt) * n_out + j] = acc[tt];
  }
  __syncthreads();
  const int qs = RS_TT * n_out;                                  // one quarter's sums
  for (int idx = threadIdx.x; idx < RS_TT * n_per; idx += RS_THREADS) {
    const int tt = idx / n_per, i = idx - tt * n_per;
    if (s_slot[tt] < 0) continue;
    const int c = c0 + i, t = t0 + tt;
    const float* zq = s_z + tt * n_out;
    const float zr = ((zq[i] + zq[qs + i]) + zq[2 * qs + i]) + zq[3 * qs + i];
    const float zi = ((zq[n_per + i] + zq[qs + n_per + i]) + zq[2 * qs + n_per + i]) +
                     zq[3 * qs + n_per + i];
    const int zc = blk * n_out + i;
    const RgStep s = rg_step(zr + b_gates[zc], zi + b_gates[zc + n_per], s_u[idx], rate[c], scale);
    float* st = state + (size_t)s_slot[tt] * state_stride;
    float* hist = st + C;
    const float* row = proj + (size_t)t * proj_stride;
    const float S = fmaf(s.a, st[c], s.d);
    out[(size_t)t * C + c] = from_f<TO>(S * gelu_tanh(row[y_off + c]));
    st[c] = S;
    for (int k = 0; k + 1 < taps - 1; ++k) hist[(size_t)k * C + c] = hist[(size_t)(k + 1) * C + c];
    if (taps > 1) hist[(size_t)(taps - 2) * C + c] = row[x_off + c];
  }
}

}  // namespace hs

HS_EXPORT int hs_rglru_conv(float* u, const float* proj, int proj_stride, int x_off,
                            const float* cw, const float* cb, const float* state,
                            int state_stride, const int* tok_req, const int* req_start,
                            const int* req_slot, int n_tokens, int C, int taps, void* stream) {
  if (!u || !proj || !cw || !cb || !state || !tok_req || !req_start || !req_slot)
    return HS_ERR_ARGUMENT;
  if (C <= 0 || taps < 1 || state_stride < C * taps) return HS_ERR_UNSUPPORTED;
  if (n_tokens <= 0) return HS_OK;
  if (n_tokens > 65535) return HS_ERR_TOO_LARGE;
  cudaError_t e = hs_launch(hs::rglru_conv_kernel, dim3((C + 255) / 256, n_tokens), dim3(256), 0,
                            (cudaStream_t)stream, hs_pdl_enabled(), u, proj, proj_stride, x_off,
                            cw, cb, state, state_stride, tok_req, req_start, req_slot, C, taps);
  return e == cudaSuccess ? HS_OK : (int)e;
}

HS_EXPORT int hs_rglru_scan(void* out, float* state, int state_stride, const float* u,
                            const float* z, const float* proj, int proj_stride, int y_off,
                            int x_off, const float* b_gates, const float* rate,
                            const int* req_start, const int* req_len, const int* req_slot,
                            int n_requests, int C, int blocks, int taps, float scale,
                            int out_dtype, void* stream) {
  if (!out || !state || !u || !z || !proj || !b_gates || !rate || !req_start || !req_len ||
      !req_slot)
    return HS_ERR_ARGUMENT;
  if (C <= 0 || blocks <= 0 || C % blocks || taps < 1 || state_stride < C * taps)
    return HS_ERR_UNSUPPORTED;
  if (n_requests <= 0) return HS_OK;
  if (n_requests > 65535) return HS_ERR_TOO_LARGE;
  // the cut depends on the model's channels only, never on the batch
  const int ch = C <= hs::RG_WIDE ? 16 : 32;
  const dim3 grid((C + ch - 1) / ch, n_requests), block(hs::RG_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
#define HS_RG_SCAN(TO, CH)                                                                       \
  e = hs_launch(hs::rglru_scan_kernel<TO, CH>, grid, block, 0, st, hs_pdl_enabled(), (TO*)out,   \
                state, state_stride, u, z, proj, proj_stride, y_off, x_off, b_gates, rate,       \
                req_start, req_len, req_slot, C, C / blocks, taps, scale)
  if (out_dtype == HS_DT_BF16) {
    if (ch == 16) HS_RG_SCAN(__nv_bfloat16, 16); else HS_RG_SCAN(__nv_bfloat16, 32);
  } else if (out_dtype == HS_DT_F32) {
    if (ch == 16) HS_RG_SCAN(float, 16); else HS_RG_SCAN(float, 32);
  } else {
    return HS_ERR_UNSUPPORTED;
  }
#undef HS_RG_SCAN
  return e == cudaSuccess ? HS_OK : (int)e;
}

// One token a request (tokens whose request row is negative are skipped).  The gate matrices
// are float32 [blocks, n (summed), 2n (r | i)].  Refuses parts of more than 256 channels.
HS_EXPORT int hs_rglru_step(void* out, float* state, int state_stride, const float* proj,
                            int proj_stride, int y_off, int x_off, const float* cw,
                            const float* cb, const float* w_gates, const float* b_gates,
                            const float* rate, const int* tok_req, const int* req_slot,
                            int n_tokens, int C, int blocks, int taps, float scale, int out_dtype,
                            void* stream) {
  if (!out || !state || !proj || !cw || !cb || !w_gates || !b_gates || !rate || !tok_req ||
      !req_slot)
    return HS_ERR_ARGUMENT;
  if (C <= 0 || blocks <= 0 || C % blocks || taps < 1 || state_stride < C * taps)
    return HS_ERR_UNSUPPORTED;
  const int n_per = C / blocks;
  // parts of up to 256 channels: beyond that a block's walk over its gate matrices takes
  // longer than the three launches, whose grids spread it over the device
  if (n_per > 256) return HS_ERR_UNSUPPORTED;
  const size_t smem = (size_t)9 * hs::RS_TT * n_per * sizeof(float);
  if (n_tokens <= 0) return HS_OK;
  const int tiles = (n_tokens + hs::RS_TT - 1) / hs::RS_TT;
  if (tiles > 65535) return HS_ERR_TOO_LARGE;
  const dim3 grid(blocks, tiles), block(hs::RS_THREADS);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  static bool sized = false;
  if (!sized) {
    const int most = 9 * hs::RS_TT * 256 * (int)sizeof(float);
    e = cudaFuncSetAttribute(hs::rglru_step_kernel<__nv_bfloat16>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(hs::rglru_step_kernel<float>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, most);
    if (e != cudaSuccess) return (int)e;
    sized = true;
  }
  if (out_dtype == HS_DT_BF16)
    e = hs_launch(hs::rglru_step_kernel<__nv_bfloat16>, grid, block, smem, st, hs_pdl_enabled(),
                  (__nv_bfloat16*)out, state, state_stride, proj, proj_stride, y_off, x_off, cw,
                  cb, w_gates, b_gates, rate, tok_req, req_slot, n_tokens, C, n_per, taps, scale);
  else if (out_dtype == HS_DT_F32)
    e = hs_launch(hs::rglru_step_kernel<float>, grid, block, smem, st, hs_pdl_enabled(),
                  (float*)out, state, state_stride, proj, proj_stride, y_off, x_off, cw, cb,
                  w_gates, b_gates, rate, tok_req, req_slot, n_tokens, C, n_per, taps, scale);
  else
    return HS_ERR_UNSUPPORTED;
  return e == cudaSuccess ? HS_OK : (int)e;
}
