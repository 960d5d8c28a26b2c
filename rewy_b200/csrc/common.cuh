// Shared definitions of the delta-rule backward kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/rewy_b200.h"

namespace rewy {

constexpr int C = 64;    // chunk rows
constexpr int DK = 128;  // key head dim
constexpr int DV = 128;  // value head dim

enum GateMode { GATE_NONE = 0, GATE_SCALAR = 1, GATE_VECTOR = 2 };

using bf16 = __nv_bfloat16;

struct Dims {
  int B, T, H, NT;
};

// Host-side launchers (one per stage); each returns a cudaError_t from the launch.
cudaError_t launch_prepare(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st);                // warp-MMA kernel
cudaError_t launch_prepare_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st);  // TMA + tcgen05
cudaError_t launch_fwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st);
cudaError_t launch_bwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st);      // warp-MMA kernel
// tcgen05 forward scan; final_state (optional) receives the state after the last chunk
cudaError_t launch_fwd_scan_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st,
                               float* final_state = nullptr);
cudaError_t launch_bwd_scan_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st);  // tcgen05
// chunk adjoint: tensor-core kernel (ctrl = device int[2 + chunks]: status word, wide-chunk count, indices)
// followed by the warp-MMA kernel on the listed wide-span chunks; or the warp-MMA kernel on every chunk.
cudaError_t launch_chunk_adjoint_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* ctrl, cudaStream_t st);
cudaError_t launch_chunk_adjoint_warp(const RewyBwdArgs& a, const RewyStageBuffers& s, const int* list, cudaStream_t st);
cudaError_t launch_chunk_output_tc(const RewyFwdArgs& a, int* err, cudaStream_t st);  // forward output, TMA + tcgen05
void count_launch(int n = 1);
int report_error(int code, const char* text);  // stores the text rewy_last_error() returns; gives back `code`
// shape envelope + presence and 16-byte alignment of every pointer of a chunk-stage call (REWY_OK or an error code)
int validate_chunk_stage(const RewyBwdArgs* a, const RewyStageBuffers* s, bool need_ctrl);

__host__ __device__ inline int gate_mode_of(int family) {
  return family == REWY_DELTA ? GATE_NONE : (family == REWY_GDN ? GATE_SCALAR : GATE_VECTOR);
}

// Opt a kernel in to `bytes` of dynamic shared memory once per device (the attribute sticks to the function in that
// device's context), so that a launch costs no extra runtime call afterwards.  Kern is the kernel itself (one guard per
// template instance).
template <auto Kern>
inline cudaError_t ensure_dynamic_smem(size_t bytes) {
  static unsigned long long done = 0;  // bit d: set on device d
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && ((__atomic_load_n(&done, __ATOMIC_ACQUIRE) >> dev) & 1ull)) return cudaSuccess;
  e = cudaFuncSetAttribute(Kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && dev < 64) __atomic_fetch_or(&done, 1ull << dev, __ATOMIC_RELEASE);
  return e;
}

// ---- small device helpers -------------------------------------------------------------------
__device__ __forceinline__ float bf2f(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 f2bf(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t u) {
  __nv_bfloat162 p = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(p);
}

// Copy a [rows x cols] BF16 tile (cols multiple of 8) from global (row pitch g_ld elements) to
// shared (row pitch s_ld elements) with 16-byte accesses by the whole CTA.
template <int ROWS, int COLS>
__device__ __forceinline__ void load_tile_bf16(bf16* __restrict__ s, int s_ld, const bf16* __restrict__ g,
                                               size_t g_ld) {
  constexpr int V8 = COLS / 8;
  for (int i = threadIdx.x; i < ROWS * V8; i += blockDim.x) {
    int r = i / V8, c = (i % V8) * 8;
    *reinterpret_cast<uint4*>(s + r * s_ld + c) = *reinterpret_cast<const uint4*>(g + (size_t)r * g_ld + c);
  }
}
template <int ROWS, int COLS>
__device__ __forceinline__ void store_tile_bf16(bf16* __restrict__ g, size_t g_ld, const bf16* __restrict__ s,
                                                int s_ld) {
  constexpr int V8 = COLS / 8;
  for (int i = threadIdx.x; i < ROWS * V8; i += blockDim.x) {
    int r = i / V8, c = (i % V8) * 8;
    *reinterpret_cast<uint4*>(g + (size_t)r * g_ld + c) = *reinterpret_cast<const uint4*>(s + r * s_ld + c);
  }
}

}  // namespace rewy
