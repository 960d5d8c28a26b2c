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
  bf16* sE = sA + C * LD64;                      // [64][136]  b*k*gamma, later w
  bf16* sZ = sE + C * LD128;                     // [64][136]  w_gate*v, later u
  float* sG = reinterpret_cast<float*>(sZ + C * LD128);  // [64] scalar gate rows
  float* sGl = sG + C;                                    // [128] last gate row of the chunk (vector gate)
  bf16* sQ = reinterpret_cast<bf16*>(sGl + 128);          // [64][136] q and k, only when Aqk is rebuilt
  bf16* sK = sQ + C * LD128;

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
  if (GATE == GATE_VECTOR) {
    if (threadIdx.x < 128) sGl[threadIdx.x] = g[base128 + (size_t)(C - 1) * ldt + threadIdx.x];
  }
  __syncthreads();

  // elementwise operands, 8 columns (16 bytes of BF16) per thread-iteration
  for (int i = threadIdx.x; i < C * 16; i += blockDim.x) {
    const int r = i >> 4, c = (i & 15) * 8;
    const size_t go = base128 + (size_t)r * ldt + c;
    const uint4 kr = *reinterpret_cast<const uint4*>(k + go);
    const uint4 qr = *reinterpret_cast<const uint4*>(q + go);
    const uint4 vr = *reinterpret_cast<const uint4*>(v + go);
    float gg[8], gl[8];
    if (GATE == GATE_VECTOR) {
      const float4 ga = *reinterpret_cast<const float4*>(g + go), gb = *reinterpret_cast<const float4*>(g + go + 4);
      gg[0] = ga.x; gg[1] = ga.y; gg[2] = ga.z; gg[3] = ga.w; gg[4] = gb.x; gg[5] = gb.y; gg[6] = gb.z; gg[7] = gb.w;
#pragma unroll
      for (int j = 0; j < 8; j++) gl[j] = sGl[c + j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        gg[j] = GATE == GATE_SCALAR ? sG[r] : 0.f;
        gl[j] = GATE == GATE_SCALAR ? sG[C - 1] : 0.f;
      }
    }
    uint4 br = make_uint4(0, 0, 0, 0), wr = br;
    float bs = 0.f;
    if (VECTOR_BETA) {
      br = *reinterpret_cast<const uint4*>(bg + go);
      wr = *reinterpret_cast<const uint4*>(wg + go);
    } else {
      bs = beta[base1 + (size_t)r * H];
    }
    const uint32_t* ku = reinterpret_cast<const uint32_t*>(&kr);
    const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qr);
    const uint32_t* vu = reinterpret_cast<const uint32_t*>(&vr);
    const uint32_t* bu = reinterpret_cast<const uint32_t*>(&br);
    const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wr);
    uint32_t eo[4], zo[4], qo[4], ko[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 kk = unpack_bf16(ku[j]), qq = unpack_bf16(qu[j]), vv = unpack_bf16(vu[j]);
      float b0 = bs, b1 = bs, w0 = bs, w1 = bs;
      if (VECTOR_BETA) {
        const float2 bb = unpack_bf16(bu[j]), ww = unpack_bf16(wu[j]);
        b0 = bb.x; b1 = bb.y; w0 = ww.x; w1 = ww.y;
      }
      const float g0 = gg[2 * j], g1 = gg[2 * j + 1];
      const float e0 = GATE == GATE_NONE ? 1.f : exp2f(g0), e1 = GATE == GATE_NONE ? 1.f : exp2f(g1);
      const float f0 = GATE == GATE_NONE ? 1.f : exp2f(gl[2 * j] - g0), f1 = GATE == GATE_NONE ? 1.f : exp2f(gl[2 * j + 1] - g1);
      eo[j] = pack_bf16(kk.x * b0 * e0, kk.y * b1 * e1);
      zo[j] = pack_bf16(vv.x * w0, vv.y * w1);
      qo[j] = pack_bf16(qq.x * e0, qq.y * e1);
      ko[j] = pack_bf16(kk.x * f0, kk.y * f1);
    }
    *reinterpret_cast<uint4*>(sE + r * LD128 + c) = make_uint4(eo[0], eo[1], eo[2], eo[3]);
    *reinterpret_cast<uint4*>(sZ + r * LD128 + c) = make_uint4(zo[0], zo[1], zo[2], zo[3]);
    if (qg_out != nullptr) {  // nullptr: a family without a gate, whose scans read q and k themselves
      *reinterpret_cast<uint4*>(qg_out + go) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
      *reinterpret_cast<uint4*>(kg_out + go) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
    }
    if (Aqk_out != nullptr) {
      *reinterpret_cast<uint4*>(sQ + r * LD128 + c) = qr;
      *reinterpret_cast<uint4*>(sK + r * LD128 + c) = kr;
    }
  }
  __syncthreads();

  {
    // w and u go back through the operand tiles they were computed from, so that they leave in 16-byte rows
    Tile<64, 128, 2, 4> acc;
    acc.zero();
    acc.mma<64>(LdmOperand<false>{sA, LD64}, LdmOperand<true>{sE, LD128});
    __syncthreads();  // every warp has read the b*k*gamma tile
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(sE + r * LD128 + c) = pack_bf16(x0, x1);
    });
    acc.zero();
    acc.mma<64>(LdmOperand<false>{sA, LD64}, LdmOperand<true>{sZ, LD128});
    __syncthreads();
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(sZ + r * LD128 + c) = pack_bf16(x0, x1);
    });
    __syncthreads();
    store_tile_bf16<C, 128>(w_out + base128, ldt, sE, LD128);
    store_tile_bf16<C, 128>(u_out + base128, ldt, sZ, LD128);
  }
  if (Aqk_out != nullptr) {
    Tile<64, 64, 2, 4> acc;
    acc.zero();
    acc.mma<128>(LdmOperand<false>{sQ, LD128}, LdmOperand<false>{sK, LD128});
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

constexpr size_t PREPARE_SMEM_BASE = (size_t)(C * LD64 + 2 * C * LD128) * sizeof(bf16) + (C + 128) * sizeof(float);
constexpr size_t PREPARE_SMEM_AQK = PREPARE_SMEM_BASE + (size_t)(2 * C * LD128) * sizeof(bf16);  // + q and k tiles

template <int GATE, bool VB>
cudaError_t run(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st, bool need_aqk) {
  auto kern = prepare_kernel<GATE, VB>;
  const size_t smem = need_aqk ? PREPARE_SMEM_AQK : PREPARE_SMEM_BASE;
  cudaError_t e = ensure_dynamic_smem<prepare_kernel<GATE, VB>>(PREPARE_SMEM_AQK);
  if (e != cudaSuccess) return e;
  dim3 grid(a.T / C, a.B * a.H);
  kern<<<grid, 256, smem, st>>>(
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
