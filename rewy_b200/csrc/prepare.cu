// Stage "prepare": rebuilds the WY operands of one chunk from the saved triangular inverse.
//   w = Akk (b*k*gamma), u = Akk (w_gate*v), qg = q*gamma, kg = k*exp2(g_last - g)
// and, for the scalar-gate / ungated families (which save no Aqk),
//   Aqk = scale * tril((q k^T) * exp2(g_i - g_j)).
// Replaces FLA recompute_w_u_fwd as called by the reference at src/fast_delta_rule/backends/backward.py:116
// and inside FLA's chunk_kda_bwd / chunk_gdn2_bwd recompute branch.
#include "warp_mma.cuh"

namespace rewy {
namespace {

constexpr int LD128 = 136;  // padded pitch of a 128-wide BF16 tile
constexpr int LD64 = 72;    // padded pitch of a 64-wide BF16 tile

template <int GATE, bool VECTOR_BETA>
__global__ void __launch_bounds__(256) prepare_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, const float* __restrict__ g,
    const float* __restrict__ beta, const bf16* __restrict__ bg, const bf16* __restrict__ wg,
    const bf16* __restrict__ Akk, bf16* __restrict__ w_out, bf16* __restrict__ u_out, bf16* __restrict__ qg_out,
    bf16* __restrict__ kg_out, bf16* __restrict__ Aqk_out, int T, int H, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sA = reinterpret_cast<bf16*>(smem_raw);  // [64][72]
  bf16* sE = sA + C * LD64;                      // [64][136]
  bf16* sZ = sE + C * LD128;
  bf16* sQ = sZ + C * LD128;
  bf16* sK = sQ + C * LD128;
  float* sG = reinterpret_cast<float*>(sK + C * LD128);  // [64] scalar gate rows

  const int n = blockIdx.x, bh = blockIdx.y, b = bh / H, h = bh % H;
  const size_t row0 = (size_t)b * T + (size_t)n * C;  // first token row of the chunk
  const size_t ldt = (size_t)H * 128;                 // token pitch of [B,T,H,128]
  const size_t base128 = (row0 * H + h) * 128;
  const size_t base64 = (row0 * H + h) * 64;
  const size_t base1 = row0 * H + h;

  load_tile_bf16<C, 64>(sA, LD64, Akk + base64, (size_t)H * 64);
  if (GATE == GATE_SCALAR) {
    if (threadIdx.x < C) sG[threadIdx.x] = g[base1 + (size_t)threadIdx.x * H];
  }
  __syncthreads();

  // elementwise operands, 2 columns per thread-iteration
  for (int i = threadIdx.x; i < C * 64; i += blockDim.x) {
    const int r = i >> 6, c = (i & 63) * 2;
    const size_t go = base128 + (size_t)r * ldt + c;
    float2 kk = unpack_bf16(*reinterpret_cast<const uint32_t*>(k + go));
    float2 qq = unpack_bf16(*reinterpret_cast<const uint32_t*>(q + go));
    float2 vv = unpack_bf16(*reinterpret_cast<const uint32_t*>(v + go));
    float g0 = 0.f, g1 = 0.f, gl0 = 0.f, gl1 = 0.f;
    if (GATE == GATE_VECTOR) {
      float2 gg = *reinterpret_cast<const float2*>(g + go);
      float2 gl = *reinterpret_cast<const float2*>(g + base128 + (size_t)(C - 1) * ldt + c);
      g0 = gg.x; g1 = gg.y; gl0 = gl.x; gl1 = gl.y;
    } else if (GATE == GATE_SCALAR) {
      g0 = g1 = sG[r];
      gl0 = gl1 = sG[C - 1];
    }
    float b0, b1, w0, w1;
    if (VECTOR_BETA) {
      float2 bb = unpack_bf16(*reinterpret_cast<const uint32_t*>(bg + go));
      float2 ww = unpack_bf16(*reinterpret_cast<const uint32_t*>(wg + go));
      b0 = bb.x; b1 = bb.y; w0 = ww.x; w1 = ww.y;
    } else {
      b0 = b1 = w0 = w1 = beta[base1 + (size_t)r * H];
    }
    const float e0 = GATE == GATE_NONE ? 1.f : exp2f(g0), e1 = GATE == GATE_NONE ? 1.f : exp2f(g1);
    *reinterpret_cast<uint32_t*>(sE + r * LD128 + c) = pack_bf16(kk.x * b0 * e0, kk.y * b1 * e1);
    *reinterpret_cast<uint32_t*>(sZ + r * LD128 + c) = pack_bf16(vv.x * w0, vv.y * w1);
    *reinterpret_cast<uint32_t*>(qg_out + go) = pack_bf16(qq.x * e0, qq.y * e1);
    const float f0 = GATE == GATE_NONE ? 1.f : exp2f(gl0 - g0), f1 = GATE == GATE_NONE ? 1.f : exp2f(gl1 - g1);
    *reinterpret_cast<uint32_t*>(kg_out + go) = pack_bf16(kk.x * f0, kk.y * f1);
    if (Aqk_out != nullptr) {
      *reinterpret_cast<uint32_t*>(sQ + r * LD128 + c) = *reinterpret_cast<const uint32_t*>(q + go);
      *reinterpret_cast<uint32_t*>(sK + r * LD128 + c) = *reinterpret_cast<const uint32_t*>(k + go);
    }
  }
  __syncthreads();

  {
    Tile<64, 128, 2, 4> acc;
    acc.zero();
    acc.mma<64>(Operand<false>{sA, LD64}, Operand<true>{sE, LD128});
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(w_out + base128 + (size_t)r * ldt + c) = pack_bf16(x0, x1);
    });
    acc.zero();
    acc.mma<64>(Operand<false>{sA, LD64}, Operand<true>{sZ, LD128});
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(u_out + base128 + (size_t)r * ldt + c) = pack_bf16(x0, x1);
    });
  }
  if (Aqk_out != nullptr) {
    Tile<64, 64, 2, 4> acc;
    acc.zero();
    acc.mma<128>(Operand<false>{sQ, LD128}, Operand<false>{sK, LD128});
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      float f0 = scale, f1 = scale;
      if (GATE == GATE_SCALAR) {
        f0 *= exp2f(sG[r] - sG[c <= r ? c : r]);
        f1 *= exp2f(sG[r] - sG[c + 1 <= r ? c + 1 : r]);
      }
      float y0 = c <= r ? x0 * f0 : 0.f, y1 = c + 1 <= r ? x1 * f1 : 0.f;
      *reinterpret_cast<uint32_t*>(Aqk_out + base64 + (size_t)r * H * 64 + c) = pack_bf16(y0, y1);
    });
  }
}

constexpr size_t PREPARE_SMEM = (size_t)(C * LD64 + 4 * C * LD128) * sizeof(bf16) + C * sizeof(float);

template <int GATE, bool VB>
cudaError_t run(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st, bool need_aqk) {
  auto kern = prepare_kernel<GATE, VB>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREPARE_SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid(a.T / C, a.B * a.H);
  kern<<<grid, 256, PREPARE_SMEM, st>>>(
      (const bf16*)a.q, (const bf16*)a.k, (const bf16*)a.v, a.g, a.beta, (const bf16*)a.b_gate, (const bf16*)a.w_gate,
      (const bf16*)a.Akk, (bf16*)s.w, (bf16*)s.u, (bf16*)s.qg, (bf16*)s.kg, need_aqk ? (bf16*)s.Aqk : nullptr, a.T, a.H,
      a.scale);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prepare(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  switch (a.family) {
    case REWY_DELTA: return run<GATE_NONE, false>(a, s, st, true);
    case REWY_GDN: return run<GATE_SCALAR, false>(a, s, st, true);
    case REWY_KDA: return run<GATE_VECTOR, false>(a, s, st, false);
    default: return run<GATE_VECTOR, true>(a, s, st, false);
  }
}

}  // namespace rewy
