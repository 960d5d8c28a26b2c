// Stage "chunk adjoint": everything of the backward that is local to one 64-token chunk of one head.
//   P = Akk^T (dR + dR_lo);  dv = w*P (dw_gate = v*P);  dAqk = scale*tril(dO R^T);  dAkk = -tril(P R^T, -1)
//   dq = gamma*scale*(dO h^T) + alpha*(dAqk Yc)
//   gamma*eb = gamma*(-P h^T) + alpha*(dAkk Yc)
//   yb/gamma = zeta*(dAqk^T Qc + dAkk^T Ec) + exp2(g_last-g)*(R dh^T)
//   dk = b*(gamma*eb) + yb/gamma;  db = k*(gamma*eb);  dbeta = sum_k db + sum_v v*P
//   dg = reverse chunk cumsum of  q*dq + k*b*(gamma*eb) - k*(yb/gamma)  (+ chunk-end term on the last row)
// with Yc = k*zeta, Qc = q*alpha, Ec = b*k*alpha, alpha = exp2(g-c), zeta = 1/alpha and c the per-channel
// mid-point of the chunk's cumulative gate; chunks whose gate span reaches 80 log2 units take an exact
// pairwise path instead of the centered products.
//
// One kernel replaces, for all four families, the reference's residual-WY producer/consumer
// (src/fast_delta_rule/kernels/kda_residual_tri_beta.py:9-73, kda_residual_local_beta_consumer.py:23-180),
// the matrix intra (kernels/endpoint_intra.py:17-297, kernels/gdn2_consumer_fp32.py:9-75), the scalar-gate
// unified adjoint with its Gram-free gate gradient (kernels/scalar_liveness_gpu.py:12-84), FLA's
// chunk_kda_bwd_dAv dAqk product and FLA's reverse chunk_local_cumsum.
#include "warp_mma.cuh"

namespace rewy {
namespace {

constexpr int LD128 = 136;
constexpr int LD64 = 72;
constexpr int LDG = 132;  // pitch of the FP32 dg tile
constexpr float SPAN_LIMIT = 80.f;

struct ChunkParams {
  const bf16 *q, *k, *v, *bg, *wg, *Akk, *dO, *R, *h, *dh, *dR, *dRlo;
  const float *g, *beta;
  void *dq, *dk, *dbg, *dwg;
  bf16* dv;
  float *dg, *dbeta;
  int T, H, out_f32, passes;
  float scale;
  const int* list;  // nullptr, or [count, chunk indices...] (flattened (batch*head)*NT + chunk)
};

__device__ __forceinline__ void store_out2(void* base, size_t off, float x0, float x1, int out_f32) {
  if (out_f32)
    *reinterpret_cast<float2*>(reinterpret_cast<float*>(base) + off) = make_float2(x0, x1);
  else
    *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(base) + off) = pack_bf16(x0, x1);
}

__device__ __forceinline__ void split_store(bf16* hi, bf16* lo, int idx, float x0, float x1) {
  __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
  float2 hf = __bfloat1622float2(h);
  *reinterpret_cast<__nv_bfloat162*>(hi + idx) = h;
  *reinterpret_cast<uint32_t*>(lo + idx) = pack_bf16(x0 - hf.x, x1 - hf.y);
}

template <int GATE, bool VB>
__device__ __forceinline__ void chunk_body(const ChunkParams& p, const int n, const int bh, unsigned char* smem_raw) {
  bf16* sDO = reinterpret_cast<bf16*>(smem_raw);  // [64][136]
  bf16* sR = sDO + C * LD128;                     // [64][136]
  bf16* sP = sR + C * LD128;                      // [64][136]
  bf16* sHD = sP + C * LD128;                     // [128][136]  h, later dh
  bf16* sXh = sHD + DK * LD128;                   // [64][136]   Yc hi, later Qc hi   (phase A: Akk)
  bf16* sXl = sXh + C * LD128;                    //             Yc lo, later Qc lo   (phase A: dR)
  bf16* sEh = sXl + C * LD128;                    // Ec hi
  bf16* sEl = sEh + C * LD128;                    // Ec lo
  bf16* sHh = sEl + C * LD128;                    // [64][72] dAqk hi
  bf16* sHl = sHh + C * LD64;
  bf16* sDh = sHl + C * LD64;                     // dAkk hi
  bf16* sDl = sDh + C * LD64;
  float* sRow = reinterpret_cast<float*>(sDl + C * LD64);  // [64]  dbeta accumulators
  float* sCol = sRow + C;                                  // [128] chunk-end gate term
  float* sCen = sCol + DK;                                 // [128] centre c
  float* sGs = sCen + DK;                                  // [64]  scalar gate rows
  int* sFlag = reinterpret_cast<int*>(sGs + C);
  float* sG32 = reinterpret_cast<float*>(sDO);             // [64][132] alias of sDO+sR for the cumsum
  bf16* sAkk = sXh;                                        // phase A aliases
  bf16* sDRt = sXl;
  bf16* sDRlo = sEh;

  const int b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H, NT = T / C;
  const size_t row0 = (size_t)b * T + (size_t)n * C;
  const size_t ldt = (size_t)H * 128;
  const size_t base128 = (row0 * H + h) * 128;
  const size_t base64 = (row0 * H + h) * 64;
  const size_t base1 = row0 * H + h;
  const size_t hbase = (((size_t)b * NT + n) * H + h) * DK * DV;
  const int tid = threadIdx.x, lane = tid & 31;
  const float scale = p.scale;
  const bool three = p.passes != 1;

  // ---- phase 0: tiles for P, centres, flags ------------------------------------------------
  load_tile_bf16<C, 64>(sAkk, LD64, p.Akk + base64, (size_t)H * 64);
  load_tile_bf16<C, 128>(sDRt, LD128, p.dR + base128, ldt);
  load_tile_bf16<C, 128>(sDRlo, LD128, p.dRlo + base128, ldt);
  load_tile_bf16<C, 128>(sDO, LD128, p.dO + base128, ldt);
  load_tile_bf16<C, 128>(sR, LD128, p.R + base128, ldt);
  if (tid < C) sRow[tid] = 0.f;
  if (tid < DK) sCol[tid] = 0.f;
  if (tid == 0) *sFlag = 0;
  if (GATE == GATE_SCALAR && tid < C) sGs[tid] = p.g[base1 + (size_t)tid * H];
  __syncthreads();
  if (tid < DK) {
    float c = 0.f;
    if (GATE == GATE_VECTOR) {
      float lo = INFINITY, hi = -INFINITY;
      for (int r = 0; r < C; r++) {
        float x = p.g[base128 + (size_t)r * ldt + tid];
        lo = fminf(lo, x);
        hi = fmaxf(hi, x);
      }
      c = 0.5f * (lo + hi);
      if (!(hi - lo < SPAN_LIMIT)) atomicOr(sFlag, 1);
    } else if (GATE == GATE_SCALAR) {
      float lo = INFINITY, hi = -INFINITY;
      for (int r = 0; r < C; r++) {
        lo = fminf(lo, sGs[r]);
        hi = fmaxf(hi, sGs[r]);
      }
      c = 0.5f * (lo + hi);
      if (tid == 0 && !(hi - lo < SPAN_LIMIT)) atomicOr(sFlag, 1);
    }
    sCen[tid] = c;
  }
  auto gate = [&](int r, int c) -> float {
    if (GATE == GATE_VECTOR) return p.g[base128 + (size_t)r * ldt + c];
    if (GATE == GATE_SCALAR) return sGs[r];
    return 0.f;
  };
  auto gate2 = [&](int r, int c) -> float2 {
    if (GATE == GATE_VECTOR) return *reinterpret_cast<const float2*>(p.g + base128 + (size_t)r * ldt + c);
    if (GATE == GATE_SCALAR) return make_float2(sGs[r], sGs[r]);
    return make_float2(0.f, 0.f);
  };
  auto ld2 = [&](const bf16* t, int r, int c) -> float2 {
    return unpack_bf16(*reinterpret_cast<const uint32_t*>(t + base128 + (size_t)r * ldt + c));
  };
  auto bval2 = [&](int r, int c) -> float2 {
    if (VB) return ld2(p.bg, r, c);
    float x = p.beta[base1 + (size_t)r * H];
    return make_float2(x, x);
  };

  // ---- phase A: P = Akk^T dR ---------------------------------------------------------------
  {
    Tile<64, 128, 2, 4> acc;
    acc.zero();
    acc.mma<64>(Operand<true>{sAkk, LD64}, Operand<true>{sDRt, LD128});
    acc.mma<64>(Operand<true>{sAkk, LD64}, Operand<true>{sDRlo, LD128});
    float part[acc.TM][2];
#pragma unroll
    for (int i = 0; i < acc.TM; i++) part[i][0] = part[i][1] = 0.f;
#pragma unroll
    for (int i = 0; i < acc.TM; i++)
#pragma unroll
      for (int j = 0; j < acc.TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const int r = acc.row(i, e), c = acc.col(j, e);
          const float p0 = acc.acc[i][j][e], p1 = acc.acc[i][j][e + 1];
          const size_t go = base128 + (size_t)r * ldt + c;
          float2 vv = ld2(p.v, r, c);
          float w0, w1;
          if (VB) {
            float2 ww = ld2(p.wg, r, c);
            w0 = ww.x; w1 = ww.y;
            store_out2(p.dwg, go, vv.x * p0, vv.y * p1, p.out_f32);
          } else {
            w0 = w1 = p.beta[base1 + (size_t)r * H];
            part[i][e >> 1] += vv.x * p0 + vv.y * p1;
          }
          *reinterpret_cast<uint32_t*>(p.dv + go) = pack_bf16(w0 * p0, w1 * p1);
          *reinterpret_cast<uint32_t*>(sP + r * LD128 + c) = pack_bf16(p0, p1);
        }
    if (!VB) {
#pragma unroll
      for (int i = 0; i < acc.TM; i++)
#pragma unroll
        for (int hrow = 0; hrow < 2; hrow++) {
          float s = part[i][hrow];
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          if ((lane & 3) == 0) atomicAdd(&sRow[acc.row(i, hrow * 2)], s);
        }
    }
  }
  __syncthreads();
  const bool pairwise = (GATE != GATE_NONE) && (*sFlag != 0);

  // ---- phase B: dAqk, dAkk, centred operand tiles, h tile, sum_v h*dh ----------------------------
  load_tile_bf16<DK, 128>(sHD, LD128, p.h + hbase, DV);
  for (int i = tid; i < C * 64; i += blockDim.x) {
    const int r = i >> 6, c = (i & 63) * 2;
    float2 kk = ld2(p.k, r, c), qq = ld2(p.q, r, c), bb = bval2(r, c);
    float a0 = 1.f, a1 = 1.f, z0 = 1.f, z1 = 1.f;
    if (GATE != GATE_NONE && !pairwise) {
      float2 gg = gate2(r, c);
      float c0 = GATE == GATE_VECTOR ? sCen[c] : sCen[0], c1 = GATE == GATE_VECTOR ? sCen[c + 1] : sCen[0];
      a0 = exp2f(gg.x - c0); a1 = exp2f(gg.y - c1);
      z0 = exp2f(c0 - gg.x); z1 = exp2f(c1 - gg.y);
    }
    split_store(sEh, sEl, r * LD128 + c, bb.x * kk.x * a0, bb.y * kk.y * a1);
    // Yc goes to sX now; Qc replaces it before the third group of products.
    // (sX aliases the phase-A tiles, which are no longer read after the barrier above.)
    split_store(sXh, sXl, r * LD128 + c, kk.x * z0, kk.y * z1);
  }
  if (GATE != GATE_NONE) {
    // chunk-end term, part 1: lam[k] * sum_v h[k,v]*dh[k,v]
    const int warp = tid >> 5;
    for (int kk = warp; kk < DK; kk += 8) {
      const size_t o = hbase + (size_t)kk * DV + lane * 4;
      uint2 a = *reinterpret_cast<const uint2*>(p.h + o), d = *reinterpret_cast<const uint2*>(p.dh + o);
      float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), d0 = unpack_bf16(d.x), d1 = unpack_bf16(d.y);
      float s = a0.x * d0.x + a0.y * d0.y + a1.x * d1.x + a1.y * d1.y;
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
      if (lane == 0) atomicAdd(&sCol[kk], s * exp2f(gate(C - 1, kk)));
    }
  }
  {
    Tile<64, 64, 2, 4> acc;
    acc.zero();
    acc.mma<128>(Operand<false>{sDO, LD128}, Operand<false>{sR, LD128});
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      split_store(sHh, sHl, r * LD64 + c, c <= r ? x0 * scale : 0.f, c + 1 <= r ? x1 * scale : 0.f);
    });
    acc.zero();
    acc.mma<128>(Operand<false>{sP, LD128}, Operand<false>{sR, LD128});
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      split_store(sDh, sDl, r * LD64 + c, c < r ? -x0 : 0.f, c + 1 < r ? -x1 : 0.f);
    });
  }
  __syncthreads();

  // Exact pairwise contraction for chunks whose gate span is too wide for centred factors.
  // kind 0: sum_{j<=i} M[i,j] k[j,c] 2^(g[i,c]-g[j,c])           (M = dAqk or dAkk)
  // kind 1: sum_{i>=j} (L[i,j] q[i,c] + D[i,j] b[i,c] k[i,c]) 2^(g[i,c]-g[j,c])
  auto mat = [&](const bf16* hi, const bf16* lo, int i, int j) -> float {
    return bf2f(hi[i * LD64 + j]) + bf2f(lo[i * LD64 + j]);
  };
  auto pair_rowsum = [&](const bf16* hi, const bf16* lo, int i, int c) -> float {
    float gi = gate(i, c), s = 0.f;
    for (int j = 0; j <= i; j++)
      s += mat(hi, lo, i, j) * bf2f(p.k[base128 + (size_t)j * ldt + c]) * exp2f(gi - gate(j, c));
    return s;
  };
  auto pair_colsum = [&](int j, int c) -> float {
    float gj = gate(j, c), s = 0.f;
    for (int i = j; i < C; i++) {
      const size_t go = base128 + (size_t)i * ldt + c;
      float bi = VB ? bf2f(p.bg[go]) : p.beta[base1 + (size_t)i * H];
      s += (mat(sHh, sHl, i, j) * bf2f(p.q[go]) + mat(sDh, sDl, i, j) * bi * bf2f(p.k[go])) * exp2f(gate(i, c) - gj);
    }
    return s;
  };

  using T128 = Tile<64, 128, 2, 4>;
  float dgrow[T128::TM][T128::TN][4];
  float dkpart[T128::TM][T128::TN][4];
  T128 acc1, acc2;

  // ---- phase C1: dq -------------------------------------------------------------------------
  acc1.zero();
  acc1.mma<128>(Operand<false>{sDO, LD128}, Operand<false>{sHD, LD128});
  acc2.zero();
  if (!pairwise) {
    acc2.mma<64>(Operand<false>{sHh, LD64}, Operand<true>{sXh, LD128});
    if (three) {
      acc2.mma<64>(Operand<false>{sHh, LD64}, Operand<true>{sXl, LD128});
      acc2.mma<64>(Operand<false>{sHl, LD64}, Operand<true>{sXh, LD128});
    }
  } else {
    acc2.for_each([&](int r, int c, float& x) { x = pair_rowsum(sHh, sHl, r, c); });
  }
#pragma unroll
  for (int i = 0; i < T128::TM; i++)
#pragma unroll
    for (int j = 0; j < T128::TN; j++)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int r = acc1.row(i, e), c = acc1.col(j, e);
        float2 gg = gate2(r, c);
        float ga0 = GATE == GATE_NONE ? 1.f : exp2f(gg.x), ga1 = GATE == GATE_NONE ? 1.f : exp2f(gg.y);
        float al0 = 1.f, al1 = 1.f;
        if (GATE != GATE_NONE && !pairwise) {
          al0 = exp2f(gg.x - (GATE == GATE_VECTOR ? sCen[c] : sCen[0]));
          al1 = exp2f(gg.y - (GATE == GATE_VECTOR ? sCen[c + 1] : sCen[0]));
        }
        float d0 = ga0 * scale * acc1.acc[i][j][e] + al0 * acc2.acc[i][j][e];
        float d1 = ga1 * scale * acc1.acc[i][j][e + 1] + al1 * acc2.acc[i][j][e + 1];
        store_out2(p.dq, base128 + (size_t)r * ldt + c, d0, d1, p.out_f32);
        float2 qq = ld2(p.q, r, c);
        dgrow[i][j][e] = qq.x * d0;
        dgrow[i][j][e + 1] = qq.y * d1;
      }

  // ---- phase C2: gamma*eb -> dk part, db -----------------------------------------------------
  acc1.zero();
  acc1.mma<128>(Operand<false, true>{sP, LD128}, Operand<false>{sHD, LD128});
  acc2.zero();
  if (!pairwise) {
    acc2.mma<64>(Operand<false>{sDh, LD64}, Operand<true>{sXh, LD128});
    if (three) {
      acc2.mma<64>(Operand<false>{sDh, LD64}, Operand<true>{sXl, LD128});
      acc2.mma<64>(Operand<false>{sDl, LD64}, Operand<true>{sXh, LD128});
    }
  } else {
    acc2.for_each([&](int r, int c, float& x) { x = pair_rowsum(sDh, sDl, r, c); });
  }
  {
    float part[T128::TM][2];
#pragma unroll
    for (int i = 0; i < T128::TM; i++) part[i][0] = part[i][1] = 0.f;
#pragma unroll
    for (int i = 0; i < T128::TM; i++)
#pragma unroll
      for (int j = 0; j < T128::TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const int r = acc1.row(i, e), c = acc1.col(j, e);
          float2 gg = gate2(r, c);
          float ga0 = GATE == GATE_NONE ? 1.f : exp2f(gg.x), ga1 = GATE == GATE_NONE ? 1.f : exp2f(gg.y);
          float al0 = 1.f, al1 = 1.f;
          if (GATE != GATE_NONE && !pairwise) {
            al0 = exp2f(gg.x - (GATE == GATE_VECTOR ? sCen[c] : sCen[0]));
            al1 = exp2f(gg.y - (GATE == GATE_VECTOR ? sCen[c + 1] : sCen[0]));
          }
          float e0 = ga0 * acc1.acc[i][j][e] + al0 * acc2.acc[i][j][e];
          float e1 = ga1 * acc1.acc[i][j][e + 1] + al1 * acc2.acc[i][j][e + 1];
          float2 kk = ld2(p.k, r, c), bb = bval2(r, c);
          if (VB)
            store_out2(p.dbg, base128 + (size_t)r * ldt + c, kk.x * e0, kk.y * e1, p.out_f32);
          else
            part[i][e >> 1] += kk.x * e0 + kk.y * e1;
          dkpart[i][j][e] = bb.x * e0;
          dkpart[i][j][e + 1] = bb.y * e1;
          dgrow[i][j][e] += kk.x * bb.x * e0;
          dgrow[i][j][e + 1] += kk.y * bb.y * e1;
        }
    if (!VB) {
#pragma unroll
      for (int i = 0; i < T128::TM; i++)
#pragma unroll
        for (int hrow = 0; hrow < 2; hrow++) {
          float s = part[i][hrow];
          s += __shfl_xor_sync(0xffffffffu, s, 1);
          s += __shfl_xor_sync(0xffffffffu, s, 2);
          if ((lane & 3) == 0) atomicAdd(&sRow[acc1.row(i, hrow * 2)], s);
        }
    }
  }
  __syncthreads();  // h and Yc tiles are dead

  // ---- phase C3: yb/gamma -> dk, gate row term -------------------------------------------------
  load_tile_bf16<DK, 128>(sHD, LD128, p.dh + hbase, DV);
  if (!pairwise) {
    for (int i = tid; i < C * 64; i += blockDim.x) {
      const int r = i >> 6, c = (i & 63) * 2;
      float2 qq = ld2(p.q, r, c);
      float a0 = 1.f, a1 = 1.f;
      if (GATE != GATE_NONE) {
        float2 gg = gate2(r, c);
        a0 = exp2f(gg.x - (GATE == GATE_VECTOR ? sCen[c] : sCen[0]));
        a1 = exp2f(gg.y - (GATE == GATE_VECTOR ? sCen[c + 1] : sCen[0]));
      }
      split_store(sXh, sXl, r * LD128 + c, qq.x * a0, qq.y * a1);
    }
  }
  __syncthreads();
  acc1.zero();
  acc1.mma<128>(Operand<false>{sR, LD128}, Operand<false>{sHD, LD128});
  acc2.zero();
  if (!pairwise) {
    acc2.mma<64>(Operand<true>{sHh, LD64}, Operand<true>{sXh, LD128});
    acc2.mma<64>(Operand<true>{sDh, LD64}, Operand<true>{sEh, LD128});
    if (three) {
      acc2.mma<64>(Operand<true>{sHh, LD64}, Operand<true>{sXl, LD128});
      acc2.mma<64>(Operand<true>{sHl, LD64}, Operand<true>{sXh, LD128});
      acc2.mma<64>(Operand<true>{sDh, LD64}, Operand<true>{sEl, LD128});
      acc2.mma<64>(Operand<true>{sDl, LD64}, Operand<true>{sEh, LD128});
    }
  } else {
    acc2.for_each([&](int r, int c, float& x) { x = pair_colsum(r, c); });
  }
  {
    float colpart[T128::TN][2];
#pragma unroll
    for (int j = 0; j < T128::TN; j++) colpart[j][0] = colpart[j][1] = 0.f;
#pragma unroll
    for (int i = 0; i < T128::TM; i++)
#pragma unroll
      for (int j = 0; j < T128::TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
          const int r = acc1.row(i, e), c = acc1.col(j, e);
          float ze0 = 1.f, ze1 = 1.f, f0 = 1.f, f1 = 1.f;
          if (GATE != GATE_NONE) {
            float2 gg = gate2(r, c), gl = gate2(C - 1, c);
            f0 = exp2f(gl.x - gg.x);
            f1 = exp2f(gl.y - gg.y);
            if (!pairwise) {
              ze0 = exp2f((GATE == GATE_VECTOR ? sCen[c] : sCen[0]) - gg.x);
              ze1 = exp2f((GATE == GATE_VECTOR ? sCen[c + 1] : sCen[0]) - gg.y);
            }
          }
          float s0 = f0 * acc1.acc[i][j][e], s1 = f1 * acc1.acc[i][j][e + 1];  // k-state part of yb/gamma
          float y0 = ze0 * acc2.acc[i][j][e] + s0, y1 = ze1 * acc2.acc[i][j][e + 1] + s1;
          store_out2(p.dk, base128 + (size_t)r * ldt + c, dkpart[i][j][e] + y0, dkpart[i][j][e + 1] + y1, p.out_f32);
          if (GATE != GATE_NONE) {
            float2 kk = ld2(p.k, r, c);
            dgrow[i][j][e] -= kk.x * y0;
            dgrow[i][j][e + 1] -= kk.y * y1;
            colpart[j][0] += kk.x * s0;
            colpart[j][1] += kk.y * s1;
          }
        }
    if (GATE != GATE_NONE) {
#pragma unroll
      for (int j = 0; j < T128::TN; j++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          float s = colpart[j][e];
          s += __shfl_xor_sync(0xffffffffu, s, 4);
          s += __shfl_xor_sync(0xffffffffu, s, 8);
          s += __shfl_xor_sync(0xffffffffu, s, 16);
          if (lane < 4) atomicAdd(&sCol[acc1.col(j, e)], s);
        }
    }
  }
  __syncthreads();  // every product that reads sDO / sR is done; reuse them for the dg tile

  if (!VB && tid < C) p.dbeta[base1 + (size_t)tid * H] = sRow[tid];
  if (GATE == GATE_NONE) return;

#pragma unroll
  for (int i = 0; i < T128::TM; i++)
#pragma unroll
    for (int j = 0; j < T128::TN; j++)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int r = acc1.row(i, e), c = acc1.col(j, e);
        *reinterpret_cast<float2*>(sG32 + r * LDG + c) = make_float2(dgrow[i][j][e], dgrow[i][j][e + 1]);
      }
  __syncthreads();
  if (GATE == GATE_VECTOR) {
    if (tid < DK) {
      float run = sCol[tid];
      for (int r = C - 1; r >= 0; --r) {
        run += sG32[r * LDG + tid];
        p.dg[base128 + (size_t)r * ldt + tid] = run;
      }
    }
  } else {
    // scalar gate: sum over the key dimension first, then the reverse cumsum over rows
    const int warp = tid >> 5;
    for (int r = warp; r < C; r += 8) {
      float s = 0.f;
      for (int c = lane; c < DK; c += 32) s += sG32[r * LDG + c] + (r == C - 1 ? sCol[c] : 0.f);
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
      if (lane == 0) sGs[r] = s;
    }
    __syncthreads();
    if (tid == 0) {
      float run = 0.f;
      for (int r = C - 1; r >= 0; --r) {
        run += sGs[r];
        p.dg[base1 + (size_t)r * H] = run;
      }
    }
  }
}

// Grid mode: blockIdx = (chunk, batch*head).  List mode (p.list != nullptr): the CTAs walk over the chunk
// indices list[1 .. list[0]] that the tensor-core kernel left to the exact pairwise path.
template <int GATE, bool VB>
__global__ void __launch_bounds__(256, 1) chunk_adjoint_kernel(const ChunkParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (p.list == nullptr) {
    chunk_body<GATE, VB>(p, blockIdx.x, blockIdx.y, smem_raw);
    return;
  }
  const int count = p.list[0], NT = p.T / C;
  for (int i = blockIdx.x; i < count; i += gridDim.x) {
    const int chunk = p.list[1 + i];
    chunk_body<GATE, VB>(p, chunk % NT, chunk / NT, smem_raw);
    __syncthreads();
  }
}

constexpr size_t CHUNK_SMEM = (size_t)(3 * C * LD128 + DK * LD128 + 4 * C * LD128 + 4 * C * LD64) * sizeof(bf16) +
                              (size_t)(C + DK + DK + C) * sizeof(float) + 16;
static_assert((size_t)C * LDG * sizeof(float) <= (size_t)2 * C * LD128 * sizeof(bf16), "dg tile must fit its alias");

template <int GATE, bool VB>
cudaError_t run(const ChunkParams& p, int B, cudaStream_t st) {
  auto kern = chunk_adjoint_kernel<GATE, VB>;
  cudaError_t e = ensure_dynamic_smem<chunk_adjoint_kernel<GATE, VB>>(CHUNK_SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid(p.T / C, B * p.H);
  if (p.list != nullptr) grid = dim3(min(p.T / C * B * p.H, 296), 1);
  kern<<<grid, 256, CHUNK_SMEM, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_chunk_adjoint_warp(const RewyBwdArgs& a, const RewyStageBuffers& s, const int* list, cudaStream_t st) {
  ChunkParams p;
  p.list = list;
  p.q = (const bf16*)a.q; p.k = (const bf16*)a.k; p.v = (const bf16*)a.v;
  p.bg = (const bf16*)a.b_gate; p.wg = (const bf16*)a.w_gate; p.Akk = (const bf16*)a.Akk;
  p.dO = (const bf16*)a.d_o; p.R = (const bf16*)s.v_new; p.h = (const bf16*)s.h; p.dh = (const bf16*)s.dh;
  p.dR = (const bf16*)s.dR; p.dRlo = (const bf16*)s.dR_lo; p.g = a.g; p.beta = a.beta;
  p.dq = a.dq; p.dk = a.dk; p.dbg = a.db_gate; p.dwg = a.dw_gate; p.dv = (bf16*)a.dv; p.dg = a.dg; p.dbeta = a.dbeta;
  p.T = a.T; p.H = a.H; p.out_f32 = a.out_dtype == REWY_OUT_F32; p.passes = a.intra_passes == 1 ? 1 : 3;
  p.scale = a.scale;
  switch (a.family) {
    case REWY_DELTA: return run<GATE_NONE, false>(p, a.B, st);
    case REWY_GDN: return run<GATE_SCALAR, false>(p, a.B, st);
    case REWY_KDA: return run<GATE_VECTOR, false>(p, a.B, st);
    default: return run<GATE_VECTOR, true>(p, a.B, st);
  }
}

}  // namespace rewy
