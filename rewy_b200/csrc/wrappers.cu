// Element-wise stages around the core backward: the transformations the reference's autograd wrappers apply before
// the forward and after the family backward (src/fast_delta_rule/_compat/kda.py:56-63,202-210; FLA l2norm_fwd /
// l2norm_bwd, fused_beta_sigmoid(_bwd), kda_gate_chunk_cumsum and kda_gate_bwd).  Each is one pass over its tensor,
// bound by HBM: 16-byte accesses, one warp per 128-wide row, grids sized in multiples of the SM count.
//   l2norm      y = x * rsqrt(sum x^2 + eps)                       dx = (dy - y * sum(dy*y)) * rstd, cast to BF16
//   beta        y = scale * sigmoid(x)                             dx = dy * scale * s * (1 - s)
//   KDA gate    g = -exp(A_log[h]) * softplus(x + dt_bias[h,k])    chunk-local cumulative sum in log2 units
//               dx = -exp(A_log[h]) * dg * sigmoid(x + bias);  dA_log[h] = sum dg * g;  ddt_bias[h,k] = sum dx
#include <cstdio>
#include "common.cuh"

namespace rewy {
namespace {

constexpr float RCP_LN2 = 1.4426950408889634f;

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}

__device__ __forceinline__ void load4_bf16(const bf16* p, float (&x)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
__device__ __forceinline__ void store4_bf16(bf16* p, const float (&x)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]));
}

// One warp per row of 128 BF16 values; lane l owns columns 4l .. 4l+3.
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y,
                                                          float* __restrict__ rstd, long long rows, float eps) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    float v[4];
    load4_bf16(x + r * 128 + 4 * lane, v);
    const float ss = warp_sum(v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]);
    const float rs = rsqrtf(ss + eps);
    float o[4] = {v[0] * rs, v[1] * rs, v[2] * rs, v[3] * rs};
    store4_bf16(y + r * 128 + 4 * lane, o);
    if (lane == 0) rstd[r] = rs;
  }
}

template <bool DY_F32>
__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const bf16* __restrict__ y, const float* __restrict__ rstd,
                                                          const void* __restrict__ dy, bf16* __restrict__ dx,
                                                          long long rows) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    float yv[4], g[4];
    load4_bf16(y + r * 128 + 4 * lane, yv);
    if (DY_F32) {
      const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(dy) + r * 128 + 4 * lane);
      g[0] = t.x; g[1] = t.y; g[2] = t.z; g[3] = t.w;
    } else {
      load4_bf16(static_cast<const bf16*>(dy) + r * 128 + 4 * lane, g);
    }
    const float s = warp_sum(g[0] * yv[0] + g[1] * yv[1] + g[2] * yv[2] + g[3] * yv[3]);
    const float rs = rstd[r];
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; i++) o[i] = (g[i] - yv[i] * s) * rs;
    store4_bf16(dx + r * 128 + 4 * lane, o);
  }
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// x: raw beta logits (BF16 or FP32); y: FP32 (what the backward kernels read) and, optionally, BF16.
template <bool X_F32>
__global__ void __launch_bounds__(256) beta_sigmoid_fwd_kernel(const void* __restrict__ x, float* __restrict__ y32,
                                                                bf16* __restrict__ y16, long long n, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float xv = X_F32 ? static_cast<const float*>(x)[i] : bf2f(static_cast<const bf16*>(x)[i]);
    float y = scale * sigmoidf(xv);
    if (y16 != nullptr) {  // the forward's beta is rounded to the logits' dtype, as the reference's fused sigmoid returns it
      const bf16 yb = f2bf(y);
      y16[i] = yb;
      y = bf2f(yb);
    }
    if (y32 != nullptr) y32[i] = y;
  }
}
template <bool X_F32>
__global__ void __launch_bounds__(256) beta_sigmoid_bwd_kernel(const void* __restrict__ x, const float* __restrict__ dy,
                                                                float* __restrict__ dx, long long n, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float xv = X_F32 ? static_cast<const float*>(x)[i] : bf2f(static_cast<const bf16*>(x)[i]);
    const float s = sigmoidf(xv);
    dx[i] = dy[i] * scale * s * (1.f - s);
  }
}

// Chunk-local inclusive cumulative sum of the per-step gate in log2 units, with the KDA gate activation optionally
// applied first.  One thread per (chunk, head, channel): 64 sequential tokens, channels contiguous across the warp.
// ACT: g = -exp(A_log[h]) * softplus(x + dt_bias[h*128 + k]); otherwise x is the per-step natural-log gate itself.
template <bool ACT, bool X_F32>
__global__ void __launch_bounds__(128) gate_cumsum_fwd_kernel(const void* __restrict__ x, const float* __restrict__ A_log,
                                                               const float* __restrict__ dt_bias, float* __restrict__ out,
                                                               float* __restrict__ g_act, int T, int H, long long chunks_h) {
  const int k = threadIdx.x;
  for (long long ch = blockIdx.x; ch < chunks_h; ch += gridDim.x) {   // ch = (b*NT + n)*H + h
    const int h = (int)(ch % H);
    const long long bn = ch / H;
    const long long row0 = bn * 64;                                    // token row in [B*T] (T is a multiple of 64)
    const float a = ACT ? -__expf(A_log[h]) : 1.f;
    const float bias = ACT && dt_bias != nullptr ? dt_bias[h * 128 + k] : 0.f;
    float run = 0.f;
#pragma unroll 8
    for (int t = 0; t < 64; t++) {
      const long long at = ((row0 + t) * H + h) * 128 + k;
      float g = X_F32 ? static_cast<const float*>(x)[at] : bf2f(static_cast<const bf16*>(x)[at]);
      if (ACT) {
        g = a * softplusf(g + bias);
        if (g_act != nullptr) g_act[at] = g;
      }
      run += g;
      out[at] = run * RCP_LN2;
    }
  }
}

// Backward of the gate activation.  dg: gradient with respect to the activated per-step gate (FP32).  One CTA per
// (batch, chunk, head), one thread per channel; per-CTA partial sums of dA_log and ddt_bias go to
// dA_part[(b*NT+n)*H + h] and dbias_part[((b*NT+n)*H + h)*128 + k] (summed over the leading index by the caller, as
// FLA's kda_gate_bwd does).
template <bool X_F32>
__global__ void __launch_bounds__(128) gate_act_bwd_kernel(const void* __restrict__ x, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, const float* __restrict__ dg,
                                                            float* __restrict__ dx, float* __restrict__ dA_part,
                                                            float* __restrict__ dbias_part, int H, long long chunks_h) {
  __shared__ float red[4];
  const int k = threadIdx.x;
  for (long long ch = blockIdx.x; ch < chunks_h; ch += gridDim.x) {
    const int h = (int)(ch % H);
    const long long row0 = (ch / H) * 64;
    const float a = -__expf(A_log[h]);
    const float bias = dt_bias != nullptr ? dt_bias[h * 128 + k] : 0.f;
    float sa = 0.f, sb = 0.f;
#pragma unroll 8
    for (int t = 0; t < 64; t++) {
      const long long at = ((row0 + t) * H + h) * 128 + k;
      const float xv = (X_F32 ? static_cast<const float*>(x)[at] : bf2f(static_cast<const bf16*>(x)[at])) + bias;
      const float d = dg[at];
      const float gx = a * d * sigmoidf(xv);
      dx[at] = gx;
      sb += gx;
      sa += d * a * softplusf(xv);
    }
    dbias_part[ch * 128 + k] = sb;
    sa = warp_sum(sa);
    __syncthreads();
    if ((k & 31) == 0) red[k >> 5] = sa;
    __syncthreads();
    if (k == 0) dA_part[ch] = red[0] + red[1] + red[2] + red[3];
  }
}

int grid_for(long long work_items, int per_block) {
  long long blocks = (work_items + per_block - 1) / per_block;
  const long long cap = 148ll * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

bool bad16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

}  // namespace
}  // namespace rewy

using namespace rewy;

#define WRAP_REQUIRE(ptr)                                                                                \
  do {                                                                                                   \
    if ((ptr) == nullptr) return report_error(REWY_ERR_NULL, "required pointer '" #ptr "' is NULL");      \
    if (bad16(ptr)) return report_error(REWY_ERR_ALIGN, "pointer '" #ptr "' is not 16-byte aligned");      \
  } while (0)

static int finish(const char* what) {
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return REWY_OK;
  char msg[160];
  snprintf(msg, sizeof(msg), "%s: %s", what, cudaGetErrorString(e));
  return report_error(REWY_ERR_LAUNCH, msg);
}

extern "C" int rewy_l2norm_fwd(const void* x, void* y, float* rstd, int64_t rows, float eps, rewy_stream_t st) {
  WRAP_REQUIRE(x); WRAP_REQUIRE(y); WRAP_REQUIRE(rstd);
  if (rows <= 0) return report_error(REWY_ERR_SHAPE, "rows must be positive");
  l2norm_fwd_kernel<<<grid_for(rows, 8), 256, 0, (cudaStream_t)st>>>((const bf16*)x, (bf16*)y, rstd, rows, eps);
  return finish("l2norm forward");
}

extern "C" int rewy_l2norm_bwd(const void* y, const float* rstd, const void* dy, int dy_is_f32, void* dx, int64_t rows,
                               rewy_stream_t st) {
  WRAP_REQUIRE(y); WRAP_REQUIRE(rstd); WRAP_REQUIRE(dy); WRAP_REQUIRE(dx);
  if (rows <= 0) return report_error(REWY_ERR_SHAPE, "rows must be positive");
  const int grid = grid_for(rows, 8);
  if (dy_is_f32)
    l2norm_bwd_kernel<true><<<grid, 256, 0, (cudaStream_t)st>>>((const bf16*)y, rstd, dy, (bf16*)dx, rows);
  else
    l2norm_bwd_kernel<false><<<grid, 256, 0, (cudaStream_t)st>>>((const bf16*)y, rstd, dy, (bf16*)dx, rows);
  return finish("l2norm backward");
}

extern "C" int rewy_beta_sigmoid_fwd(const void* x, int x_is_f32, float* y32, void* y16, int64_t n, float scale,
                                     rewy_stream_t st) {
  if (x == nullptr || (y32 == nullptr && y16 == nullptr)) return report_error(REWY_ERR_NULL, "x or both outputs are NULL");
  if (n <= 0) return report_error(REWY_ERR_SHAPE, "n must be positive");
  const int grid = grid_for(n, 256);
  if (x_is_f32)
    beta_sigmoid_fwd_kernel<true><<<grid, 256, 0, (cudaStream_t)st>>>(x, y32, (bf16*)y16, n, scale);
  else
    beta_sigmoid_fwd_kernel<false><<<grid, 256, 0, (cudaStream_t)st>>>(x, y32, (bf16*)y16, n, scale);
  return finish("beta sigmoid forward");
}

extern "C" int rewy_beta_sigmoid_bwd(const void* x, int x_is_f32, const float* dy, float* dx, int64_t n, float scale,
                                     rewy_stream_t st) {
  if (x == nullptr || dy == nullptr || dx == nullptr) return report_error(REWY_ERR_NULL, "x, dy or dx is NULL");
  if (n <= 0) return report_error(REWY_ERR_SHAPE, "n must be positive");
  const int grid = grid_for(n, 256);
  if (x_is_f32)
    beta_sigmoid_bwd_kernel<true><<<grid, 256, 0, (cudaStream_t)st>>>(x, dy, dx, n, scale);
  else
    beta_sigmoid_bwd_kernel<false><<<grid, 256, 0, (cudaStream_t)st>>>(x, dy, dx, n, scale);
  return finish("beta sigmoid backward");
}

extern "C" int rewy_gate_cumsum_fwd(const void* x, int x_is_f32, const float* A_log, const float* dt_bias, float* g_cumsum,
                                    float* g_act, int32_t B, int32_t T, int32_t H, rewy_stream_t st) {
  if (x == nullptr || g_cumsum == nullptr) return report_error(REWY_ERR_NULL, "x or g_cumsum is NULL");
  if (B <= 0 || H <= 0 || T < C || T % C != 0) return report_error(REWY_ERR_SHAPE, "bad B/T/H");
  const long long chunks_h = (long long)B * (T / C) * H;
  const int grid = (int)(chunks_h < 148ll * 64 ? chunks_h : 148ll * 64);
  cudaStream_t s = (cudaStream_t)st;
  if (A_log != nullptr) {
    if (x_is_f32) gate_cumsum_fwd_kernel<true, true><<<grid, 128, 0, s>>>(x, A_log, dt_bias, g_cumsum, g_act, T, H, chunks_h);
    else gate_cumsum_fwd_kernel<true, false><<<grid, 128, 0, s>>>(x, A_log, dt_bias, g_cumsum, g_act, T, H, chunks_h);
  } else {
    if (x_is_f32) gate_cumsum_fwd_kernel<false, true><<<grid, 128, 0, s>>>(x, nullptr, nullptr, g_cumsum, nullptr, T, H, chunks_h);
    else gate_cumsum_fwd_kernel<false, false><<<grid, 128, 0, s>>>(x, nullptr, nullptr, g_cumsum, nullptr, T, H, chunks_h);
  }
  return finish("gate cumulative sum");
}

extern "C" int rewy_gate_act_bwd(const void* x, int x_is_f32, const float* A_log, const float* dt_bias, const float* dg,
                                 float* dx, float* dA_part, float* dbias_part, int32_t B, int32_t T, int32_t H,
                                 rewy_stream_t st) {
  if (x == nullptr || A_log == nullptr || dg == nullptr || dx == nullptr || dA_part == nullptr || dbias_part == nullptr)
    return report_error(REWY_ERR_NULL, "a required pointer of the gate backward is NULL");
  if (B <= 0 || H <= 0 || T < C || T % C != 0) return report_error(REWY_ERR_SHAPE, "bad B/T/H");
  const long long chunks_h = (long long)B * (T / C) * H;
  const int grid = (int)(chunks_h < 148ll * 64 ? chunks_h : 148ll * 64);
  cudaStream_t s = (cudaStream_t)st;
  if (x_is_f32) gate_act_bwd_kernel<true><<<grid, 128, 0, s>>>(x, A_log, dt_bias, dg, dx, dA_part, dbias_part, H, chunks_h);
  else gate_act_bwd_kernel<false><<<grid, 128, 0, s>>>(x, A_log, dt_bias, dg, dx, dA_part, dbias_part, H, chunks_h);
  return finish("gate activation backward");
}
