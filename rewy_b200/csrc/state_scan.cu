// The two cross-chunk scans, sequential over the T/64 chunks of one (batch, head) and parallel over
// (batch, head, value-tile).  The 128 x BV FP32 state tile stays in registers for the whole sequence.
//
// Forward (recompute policy):  h[n] stored; v_new = u - w h[n]; h <- lam*h + kg^T v_new
//   replaces FLA chunk_gated_delta_rule_fwd_h as called at src/fast_delta_rule/backends/backward.py:117-118.
// Reverse:  dh[n] stored; dR = kg dh[n] + Aqk^T dO; dh <- lam*dh + scale*qg^T dO - w^T dR; dh0
//   (dh and dR enter their products as BF16 hi+lo pairs so the FP32 state does not drift over long sequences)
//   replaces chunk_gated_delta_rule_bwd_dhu (src/fast_delta_rule/kernels/vector_state_gpu.py:12-67 and the
//   FLA kernel bound at backends/backward.py:120-121) with the dv = Aqk^T dO product of FLA's
//   chunk_kda_bwd_dAv / chunk_bwd_dv_local (backends/backward.py:119) folded in.
#include "warp_mma.cuh"

namespace rewy {
namespace {

constexpr int LD128 = 136;
constexpr int LD64 = 72;
constexpr int BV = 64;  // value columns per CTA

template <int GATE>
__device__ __forceinline__ void load_lambda(float* sLam, const float* g, size_t last_row_base128, size_t last_row_base1) {
  if (threadIdx.x < DK) {
    float l = 1.f;
    if (GATE == GATE_VECTOR) l = exp2f(g[last_row_base128 + threadIdx.x]);
    if (GATE == GATE_SCALAR) l = exp2f(g[last_row_base1]);
    sLam[threadIdx.x] = l;
  }
}

template <int GATE>
__global__ void __launch_bounds__(256) bwd_scan_kernel(
    const bf16* __restrict__ qg, const bf16* __restrict__ kg, const bf16* __restrict__ w, const bf16* __restrict__ Aqk,
    const bf16* __restrict__ dO, const float* __restrict__ g, const float* __restrict__ dht, bf16* __restrict__ dh,
    bf16* __restrict__ dR, bf16* __restrict__ dRlo, float* __restrict__ dh0, int T, int H, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQg = reinterpret_cast<bf16*>(smem_raw);
  bf16* sKg = sQg + C * LD128;
  bf16* sW = sKg + C * LD128;
  bf16* sDO = sW + C * LD128;    // [64][72]
  bf16* sAqk = sDO + C * LD64;   // [64][72]
  bf16* sDh = sAqk + C * LD64;   // [128][72]
  bf16* sDR = sDh + DK * LD64;   // [64][72]
  bf16* sDRlo = sDR + C * LD64;  // [64][72]
  bf16* sDhLo = sDRlo + C * LD64; // [128][72] low part of the state, used only in the dR product
  float* sLam = reinterpret_cast<float*>(sDhLo + DK * LD64);

  const int v0 = blockIdx.x * BV, bh = blockIdx.y, b = bh / H, h = bh % H;
  const int NT = T / C;
  const size_t ldt = (size_t)H * 128;

  Tile<128, 64, 4, 2> state;
  state.zero();
  if (dht != nullptr) {
    const float* p = dht + (size_t)bh * DK * DV;
    state.for_each_pair([&](int r, int c, float& x0, float& x1) {
      float2 t = *reinterpret_cast<const float2*>(p + (size_t)r * DV + v0 + c);
      x0 = t.x; x1 = t.y;
    });
  }

  for (int n = NT - 1; n >= 0; --n) {
    const size_t row0 = (size_t)b * T + (size_t)n * C;
    const size_t base128 = (row0 * H + h) * 128;
    const size_t base64 = (row0 * H + h) * 64;
    load_tile_bf16<C, 128>(sQg, LD128, qg + base128, ldt);
    load_tile_bf16<C, 128>(sKg, LD128, kg + base128, ldt);
    load_tile_bf16<C, 128>(sW, LD128, w + base128, ldt);
    load_tile_bf16<C, BV>(sDO, LD64, dO + base128 + v0, ldt);
    load_tile_bf16<C, 64>(sAqk, LD64, Aqk + base64, (size_t)H * 64);
    load_lambda<GATE>(sLam, g, base128 + (size_t)(C - 1) * ldt, row0 * H + h + (size_t)(C - 1) * H);
    state.for_each_pair([&](int r, int c, float& x0, float& x1) {
      __nv_bfloat162 hi = __floats2bfloat162_rn(x0, x1);
      float2 hf = __bfloat1622float2(hi);
      *reinterpret_cast<__nv_bfloat162*>(sDh + r * LD64 + c) = hi;
      *reinterpret_cast<uint32_t*>(sDhLo + r * LD64 + c) = pack_bf16(x0 - hf.x, x1 - hf.y);
    });
    __syncthreads();
    store_tile_bf16<DK, BV>(dh + (((size_t)b * NT + n) * H + h) * DK * DV + v0, DV, sDh, LD64);

    {
      Tile<64, 64, 2, 4> acc;
      acc.zero();
      acc.mma<128>(Operand<false>{sKg, LD128}, Operand<true>{sDh, LD64});
      acc.mma<128>(Operand<false>{sKg, LD128}, Operand<true>{sDhLo, LD64});
      acc.mma<64>(Operand<true>{sAqk, LD64}, Operand<true>{sDO, LD64});
      acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
        __nv_bfloat162 hi = __floats2bfloat162_rn(x0, x1);
        float2 hf = __bfloat1622float2(hi);
        *reinterpret_cast<__nv_bfloat162*>(sDR + r * LD64 + c) = hi;
        *reinterpret_cast<uint32_t*>(sDRlo + r * LD64 + c) = pack_bf16(x0 - hf.x, x1 - hf.y);
      });
    }
    __syncthreads();
    store_tile_bf16<C, BV>(dR + base128 + v0, ldt, sDR, LD64);
    store_tile_bf16<C, BV>(dRlo + base128 + v0, ldt, sDRlo, LD64);
    {
      Tile<128, 64, 4, 2> tmp;
      tmp.zero();
      tmp.mma<64>(Operand<true>{sQg, LD128}, Operand<true>{sDO, LD64});
#pragma unroll
      for (int i = 0; i < tmp.TM; i++)
#pragma unroll
        for (int j = 0; j < tmp.TN; j++)
#pragma unroll
          for (int e = 0; e < 4; e++) {
            float lam = GATE == GATE_NONE ? 1.f : sLam[state.row(i, e)];
            state.acc[i][j][e] = state.acc[i][j][e] * lam + scale * tmp.acc[i][j][e];
          }
      state.mma<64>(Operand<true, true>{sW, LD128}, Operand<true>{sDR, LD64});
      state.mma<64>(Operand<true, true>{sW, LD128}, Operand<true>{sDRlo, LD64});
    }
    __syncthreads();
  }
  if (dh0 != nullptr) {
    float* p = dh0 + (size_t)bh * DK * DV;
    state.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<float2*>(p + (size_t)r * DV + v0 + c) = make_float2(x0, x1);
    });
  }
}

template <int GATE>
__global__ void __launch_bounds__(256) fwd_scan_kernel(
    const bf16* __restrict__ kg, const bf16* __restrict__ w, const bf16* __restrict__ u, const float* __restrict__ g,
    const float* __restrict__ h0, bf16* __restrict__ hout, bf16* __restrict__ v_new, int T, int H) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sKg = reinterpret_cast<bf16*>(smem_raw);
  bf16* sW = sKg + C * LD128;
  bf16* sU = sW + C * LD128;    // [64][72]
  bf16* sH = sU + C * LD64;     // [128][72]
  bf16* sVn = sH + DK * LD64;   // [64][72]
  float* sLam = reinterpret_cast<float*>(sVn + C * LD64);

  const int v0 = blockIdx.x * BV, bh = blockIdx.y, b = bh / H, h = bh % H;
  const int NT = T / C;
  const size_t ldt = (size_t)H * 128;

  Tile<128, 64, 4, 2> state;
  state.zero();
  if (h0 != nullptr) {
    const float* p = h0 + (size_t)bh * DK * DV;
    state.for_each_pair([&](int r, int c, float& x0, float& x1) {
      float2 t = *reinterpret_cast<const float2*>(p + (size_t)r * DV + v0 + c);
      x0 = t.x; x1 = t.y;
    });
  }
  for (int n = 0; n < NT; ++n) {
    const size_t row0 = (size_t)b * T + (size_t)n * C;
    const size_t base128 = (row0 * H + h) * 128;
    load_tile_bf16<C, 128>(sKg, LD128, kg + base128, ldt);
    load_tile_bf16<C, 128>(sW, LD128, w + base128, ldt);
    load_tile_bf16<C, BV>(sU, LD64, u + base128 + v0, ldt);
    load_lambda<GATE>(sLam, g, base128 + (size_t)(C - 1) * ldt, row0 * H + h + (size_t)(C - 1) * H);
    state.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(sH + r * LD64 + c) = pack_bf16(x0, x1);
    });
    __syncthreads();
    store_tile_bf16<DK, BV>(hout + (((size_t)b * NT + n) * H + h) * DK * DV + v0, DV, sH, LD64);
    {
      Tile<64, 64, 2, 4> acc;
      acc.zero();
      acc.mma<128>(Operand<false, true>{sW, LD128}, Operand<true>{sH, LD64});
      acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
        float2 uu = unpack_bf16(*reinterpret_cast<const uint32_t*>(sU + r * LD64 + c));
        *reinterpret_cast<uint32_t*>(sVn + r * LD64 + c) = pack_bf16(x0 + uu.x, x1 + uu.y);
      });
    }
    __syncthreads();
    store_tile_bf16<C, BV>(v_new + base128 + v0, ldt, sVn, LD64);
    if (GATE != GATE_NONE) {
      state.for_each([&](int r, int c, float& x) { x *= sLam[r]; });
    }
    state.mma<64>(Operand<true>{sKg, LD128}, Operand<true>{sVn, LD64});
    __syncthreads();
  }
}

constexpr size_t BWD_SMEM = (size_t)(3 * C * LD128 + 4 * C * LD64 + 2 * DK * LD64) * sizeof(bf16) + DK * sizeof(float);
constexpr size_t FWD_SMEM = (size_t)(2 * C * LD128 + 2 * C * LD64 + DK * LD64) * sizeof(bf16) + DK * sizeof(float);

template <int GATE>
cudaError_t run_bwd(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  auto kern = bwd_scan_kernel<GATE>;
  cudaError_t e = ensure_dynamic_smem<bwd_scan_kernel<GATE>>(BWD_SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid(DV / BV, a.B * a.H);
  kern<<<grid, 256, BWD_SMEM, st>>>((const bf16*)s.qg, (const bf16*)s.kg, (const bf16*)s.w, (const bf16*)s.Aqk,
                                    (const bf16*)a.d_o, a.g, a.dht, (bf16*)s.dh, (bf16*)s.dR, (bf16*)s.dR_lo, a.dh0, a.T, a.H,
                                    a.scale);
  count_launch();
  return cudaGetLastError();
}
template <int GATE>
cudaError_t run_fwd(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  auto kern = fwd_scan_kernel<GATE>;
  cudaError_t e = ensure_dynamic_smem<fwd_scan_kernel<GATE>>(FWD_SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid(DV / BV, a.B * a.H);
  kern<<<grid, 256, FWD_SMEM, st>>>((const bf16*)s.kg, (const bf16*)s.w, (const bf16*)s.u, a.g, a.h0, (bf16*)s.h,
                                    (bf16*)s.v_new, a.T, a.H);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  switch (gate_mode_of(a.family)) {
    case GATE_NONE: return run_bwd<GATE_NONE>(a, s, st);
    case GATE_SCALAR: return run_bwd<GATE_SCALAR>(a, s, st);
    default: return run_bwd<GATE_VECTOR>(a, s, st);
  }
}
cudaError_t launch_fwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  switch (gate_mode_of(a.family)) {
    case GATE_NONE: return run_fwd<GATE_NONE>(a, s, st);
    case GATE_SCALAR: return run_fwd<GATE_SCALAR>(a, s, st);
    default: return run_fwd<GATE_VECTOR>(a, s, st);
  }
}

}  // namespace rewy
