// Forward pass of the four families: what the autograd forward needs besides the backward's own stages.
//
//   chunk_fwd_local_kernel   one CTA per chunk, three per SM: Akk = (I + tril(E Y^T, -1))^-1, Aqk = scale tril(Qg Y^T),
//                            w = Akk E, u = Akk Z, qg, kg          (E = b k gamma, Y = k / gamma, Z = w v)
//   fwd_scan_tc_kernel       (state_scan_tc.cu) h[n], v_new, final state
//   chunk_output_tc_kernel   (chunk_output_tc.cu, tcgen05) o = scale qg h[n] + Aqk v_new; chunk_output_kernel here is its
//                            warp-MMA cross-check (rewy_set_forward_variant(1))
// Replaces FLA's chunk_kda_fwd / chunk_gdn2_fwd / chunk_gated_delta_rule_fwd / chunk_delta_rule_fwd as the reference
// binds them (src/fast_delta_rule/_compat/kda.py:89-113, gdn2.py:94-117, gdn.py:33-125, delta.py).
//
// The two 64x64x128 products that build the A matrices use centred gate factors (alpha = 2^(G - c), zeta = 1/alpha with
// c the per-channel mid-point of G over the chunk) and BF16 hi/lo operand pairs in three passes (about 16 mantissa
// bits), accumulated in FP32 by warp-level MMA (operands by ldmatrix); scalar gates apply their pairwise factor 2^(G_i - G_j) to the exact
// q k^T and k k^T products instead.  A chunk whose cumulative gate spans 80 log2 units or more in some channel does not
// use centred factors (they would leave the FP32 range): its two matrices are summed pair by pair on the CUDA cores,
// sum_k q_ik k_jk 2^(G_ik - G_jk), like the exact pairwise path of the backward.  The unit lower-triangular inverse is
// plain FP32 forward substitution, one thread per column with the column held in registers.
#include <atomic>
#include <cstdio>
#include "warp_mma.cuh"

namespace rewy {
namespace {

constexpr int LD128 = 136;  // padded pitch of a 128-wide BF16 tile
constexpr int LD64 = 72;    // padded pitch of a 64-wide BF16 tile
constexpr int LDL = 68;     // padded pitch of the FP32 64x64 matrix (rows stay 16-byte aligned)
constexpr int LDG = 132;    // padded pitch of the FP32 gate tile of a wide-span chunk
constexpr float FWD_SPAN_LIMIT = 80.f;

struct FwdLocalParams {
  const bf16 *q, *k, *v, *bg, *wg;
  const float *g, *beta;
  bf16 *Akk, *Aqk, *w, *u, *qg, *kg;
  int T, H;
  float scale;
};

__device__ __forceinline__ void split_store8(bf16* hi, bf16* lo, const float (&x)[8]) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 hh = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    float2 hf = __bfloat1622float2(hh);
    h[i] = *reinterpret_cast<uint32_t*>(&hh);
    l[i] = pack_bf16(x[2 * i] - hf.x, x[2 * i + 1] - hf.y);
  }
  *reinterpret_cast<uint4*>(hi) = make_uint4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<uint4*>(lo) = make_uint4(l[0], l[1], l[2], l[3]);
}

// 2^x and 1/x in one instruction each (2 ulp / 1 ulp); results below the normal range flush to zero
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const float2 f = unpack_bf16(u[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
}
__device__ __forceinline__ void load_gate8(const float* g, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(g), b = *reinterpret_cast<const float4*>(g + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// Shared memory holds four operand tiles and nothing else of size, so that three CTAs share an SM: the element-wise
// operands are built in three passes over the chunk's inputs (the second and third read them again, from L2), each
// pass reusing the tiles of the one before, and the FP32 matrix I + L and the inverse take the first two tiles once
// the products that read them are complete.
template <int GATE, bool VECTOR_BETA>
__global__ void __launch_bounds__(256, 3) chunk_fwd_local_kernel(const FwdLocalParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TILE = C * LD128;
  bf16* sT = reinterpret_cast<bf16*>(smem_raw);            // four tiles [64][136]:
  //   vector gate, pass 1: Qc hi, Qc lo, Yc hi, Yc lo;  pass 2: Ec hi, Ec lo over the first two
  //   scalar gate / none:  q, k in the last two
  //   wide-span chunk:     k in the second, the FP32 gate rows [64][132] over the last two (q and the key gate are
  //                        read from global memory)
  //   after the A products: I + L (FP32 [64][68]) in the first, Akk (BF16 [64][72]) in the second
  //   last pass, all:      E = b k gamma and Z = w v in the last two (-> w, u)
  static_assert((size_t)C * LDG * sizeof(float) <= 2 * (size_t)TILE * sizeof(bf16), "gate rows fit two tiles");
  static_assert((size_t)C * LDL * sizeof(float) <= (size_t)TILE * sizeof(bf16), "I + L fits one tile");
  static_assert(LD64 <= LD128, "Akk fits one tile");
  float* sL = reinterpret_cast<float*>(sT);                // [64][68]   strictly lower part of E Y^T
  bf16* sA = sT + TILE;                                    // [64][72]   Akk (BF16) once inverted
  bf16* sE = sT + 2 * TILE;
  bf16* sZ = sT + 3 * TILE;
  bf16* sStage = sE;                                       // [64][72]   Aqk between its product and its row-wise store
  float* sG = reinterpret_cast<float*>(sT + 4 * TILE);     // [64]       scalar gate rows
  float* sGl = sG + C;                                     // [128]      last gate row of the chunk (vector gate)
  float* sCen = sGl + 128;                                 // [128]      per-channel centre of the gate (vector gate)
  float* sBeta = sCen + 128;                               // [64]       scalar beta rows

  const int n = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  const size_t row0 = (size_t)b * T + (size_t)n * C;
  const size_t ldt = (size_t)H * 128;
  const size_t base128 = (row0 * H + h) * 128;
  const size_t base64 = (row0 * H + h) * 64;
  const size_t base1 = row0 * H + h;
  const int tid = threadIdx.x;

  bool wide_here = false;
  if (GATE == GATE_SCALAR && tid < C) sG[tid] = p.g[base1 + (size_t)tid * H];
  if (!VECTOR_BETA && tid >= C && tid < 2 * C) sBeta[tid - C] = p.beta[base1 + (size_t)(tid - C) * H];
  if (GATE == GATE_VECTOR && tid < 128) {
    // per-channel range of the cumulative gate over the chunk -> centre; the last row is the chunk decay
    float lo = INFINITY, hi = -INFINITY, last = 0.f;
#pragma unroll
    for (int t = 0; t < C; t++) {  // all 64 loads in flight at once
      last = p.g[base128 + (size_t)t * ldt + tid];
      lo = fminf(lo, last);
      hi = fmaxf(hi, last);
    }
    sGl[tid] = last;
    sCen[tid] = 0.5f * (lo + hi);
    wide_here = !(hi - lo < FWD_SPAN_LIMIT);
  }
  // wide gate span somewhere in the chunk: no centred factors, exact pairwise sums instead (vector gate only)
  const bool wide = __syncthreads_or(wide_here ? 1 : 0) != 0;
  float* sGf = reinterpret_cast<float*>(sT + 2 * TILE);  // [64][132] FP32 gate rows of a wide chunk

  // ---- the two A products: Qc Yc^T (-> Aqk) and Ec Yc^T (-> strictly lower part of I + L) -------------------------
  if (GATE == GATE_VECTOR && !wide) {
    // pass 1: Qc = q alpha and Yc = k / alpha as BF16 hi/lo pairs (alpha = 2^(G - centre))
#pragma unroll
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, c = (i & 15) * 8;
      const size_t go = base128 + (size_t)r * ldt + c;
      float kk[8], qq[8], gg[8], qc[8], yc[8];
      unpack8(*reinterpret_cast<const uint4*>(p.k + go), kk);
      unpack8(*reinterpret_cast<const uint4*>(p.q + go), qq);
      load_gate8(p.g + go, gg);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float al = ex2(gg[j] - sCen[c + j]);  // |exponent| < 40: no flush
        qc[j] = qq[j] * al;
        yc[j] = kk[j] * rcp(al);
      }
      split_store8(sT + 0 * TILE + r * LD128 + c, sT + 1 * TILE + r * LD128 + c, qc);
      split_store8(sT + 2 * TILE + r * LD128 + c, sT + 3 * TILE + r * LD128 + c, yc);
    }
    __syncthreads();
    const LdmOperand<false> Yh{sT + 2 * TILE, LD128}, Yl{sT + 3 * TILE, LD128};
    uint32_t aqp[8];  // this thread's part of Aqk (scaled, masked, BF16 pairs): staged for a row-wise store further down
    {
      const LdmOperand<false> Qh{sT + 0 * TILE, LD128}, Ql{sT + 1 * TILE, LD128};
      Tile<64, 64, 2, 4> aq;
      static_assert(Tile<64, 64, 2, 4>::REGS == 16, "eight column pairs per thread");
      aq.zero();
      aq.mma<128>(Qh, Yh); aq.mma<128>(Ql, Yh); aq.mma<128>(Qh, Yl);
      int n8 = 0;
      aq.for_each_pair([&](int r, int c, float& x0, float& x1) {
        const float y0 = c <= r ? x0 * p.scale : 0.f, y1 = c + 1 <= r ? x1 * p.scale : 0.f;
        aqp[n8++] = pack_bf16(y0, y1);
      });
    }
    __syncthreads();  // every warp has read Qc
    // pass 2: Ec = b k alpha over the Qc tiles
#pragma unroll
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, c = (i & 15) * 8;
      const size_t go = base128 + (size_t)r * ldt + c;
      float kk[8], gg[8], bb[8], ec[8];
      unpack8(*reinterpret_cast<const uint4*>(p.k + go), kk);
      load_gate8(p.g + go, gg);
      if (VECTOR_BETA) unpack8(*reinterpret_cast<const uint4*>(p.bg + go), bb);
      const float bs = VECTOR_BETA ? 0.f : sBeta[r];
#pragma unroll
      for (int j = 0; j < 8; j++) ec[j] = (VECTOR_BETA ? bb[j] : bs) * kk[j] * ex2(gg[j] - sCen[c + j]);
      split_store8(sT + 0 * TILE + r * LD128 + c, sT + 1 * TILE + r * LD128 + c, ec);
    }
    __syncthreads();
    {
      const LdmOperand<false> Eh{sT + 0 * TILE, LD128}, El{sT + 1 * TILE, LD128};
      Tile<64, 64, 2, 4> ak;
      ak.zero();
      ak.mma<128>(Eh, Yh); ak.mma<128>(El, Yh); ak.mma<128>(Eh, Yl);
      __syncthreads();  // every warp has read Ec and Yc: I + L and the Aqk tile take their places
      int n8 = 0;
      ak.for_each_pair([&](int r, int c, float& x0, float& x1) {
        sL[r * LDL + c] = c < r ? x0 : 0.f;
        sL[r * LDL + c + 1] = c + 1 < r ? x1 : 0.f;
        *reinterpret_cast<uint32_t*>(sStage + r * LD64 + c) = aqp[n8++];
      });
    }
  } else {
    // raw q and k tiles (scalar gate / none), or k and the gate rows of a wide-span chunk
    bf16* sQr = sT + 2 * TILE;
    bf16* sKr = GATE == GATE_VECTOR ? sT + TILE : sT + 3 * TILE;
#pragma unroll
    for (int i = tid; i < C * 16; i += 256) {
      const int r = i >> 4, c = (i & 15) * 8;
      const size_t go = base128 + (size_t)r * ldt + c;
      *reinterpret_cast<uint4*>(sKr + r * LD128 + c) = *reinterpret_cast<const uint4*>(p.k + go);
      if (GATE == GATE_VECTOR) {
        *reinterpret_cast<float4*>(sGf + r * LDG + c) = *reinterpret_cast<const float4*>(p.g + go);
        *reinterpret_cast<float4*>(sGf + r * LDG + c + 4) = *reinterpret_cast<const float4*>(p.g + go + 4);
      } else {
        *reinterpret_cast<uint4*>(sQr + r * LD128 + c) = *reinterpret_cast<const uint4*>(p.q + go);
      }
    }
    __syncthreads();
    if (GATE == GATE_VECTOR) {
      // exact pairwise sums, thread = (row i, every fourth column j)
      const int i = tid >> 2;
      const float beta_i = VECTOR_BETA ? 0.f : sBeta[i];
      const bf16* qi = p.q + base128 + (size_t)i * ldt;    // query row of token i
      const bf16* bgi = p.bg + base128 + (size_t)i * ldt;  // key gate row of token i (vector beta)
      for (int j = tid & 3; j < C; j += 4) {
        float aq = 0.f, ak = 0.f;
        if (j <= i) {
          for (int kk = 0; kk < 128; kk++) {
            const float f = exp2f(sGf[i * LDG + kk] - sGf[j * LDG + kk]) * bf2f(sKr[j * LD128 + kk]);
            aq = fmaf(bf2f(qi[kk]), f, aq);
            const float bi = VECTOR_BETA ? bf2f(bgi[kk]) : beta_i;
            ak = fmaf(bi * bf2f(sKr[i * LD128 + kk]), f, ak);
          }
        }
        p.Aqk[base64 + (size_t)i * H * 64 + j] = f2bf(p.scale * aq);
        sL[i * LDL + j] = j < i ? ak : 0.f;
      }
    } else {
      const LdmOperand<false> Q{sQr, LD128}, K{sKr, LD128};
      Tile<64, 64, 2, 4> aq, ak;
      aq.zero();
      ak.zero();
      aq.mma<128>(Q, K);
      ak.mma<128>(K, K);
      __syncthreads();  // every warp has read q and k: the Aqk tile takes the place of q
      aq.for_each_pair([&](int r, int c, float& x0, float& x1) {
        float f0 = p.scale, f1 = p.scale;
        if (GATE == GATE_SCALAR) {
          f0 *= exp2f(sG[r] - sG[c <= r ? c : r]);
          f1 *= exp2f(sG[r] - sG[c + 1 <= r ? c + 1 : r]);
        }
        const float y0 = c <= r ? x0 * f0 : 0.f, y1 = c + 1 <= r ? x1 * f1 : 0.f;
        *reinterpret_cast<uint32_t*>(sStage + r * LD64 + c) = pack_bf16(y0, y1);
      });
      ak.for_each_pair([&](int r, int c, float& x0, float& x1) {
        // exact k k^T: beta and the pairwise gate factor go on afterwards
        float f0 = VECTOR_BETA ? 1.f : sBeta[r], f1 = f0;
        if (GATE == GATE_SCALAR) {
          f0 *= exp2f(sG[r] - sG[c < r ? c : r]);
          f1 *= exp2f(sG[r] - sG[c + 1 < r ? c + 1 : r]);
        }
        sL[r * LDL + c] = c < r ? x0 * f0 : 0.f;
        sL[r * LDL + c + 1] = c + 1 < r ? x1 * f1 : 0.f;
      });
    }
  }
  __syncthreads();

  // ---- last pass, by the threads that do not invert: E = b k gamma and Z = w v into the last two tiles, qg and kg
  //      straight to global memory -----------------------------------------------------------------------------------
  if (tid >= C) {
    if (!(GATE == GATE_VECTOR && wide)) {
      // Aqk leaves in 16-byte pieces of whole rows; the tile is overwritten by this pass, so its 192 threads meet first
      for (int i = tid - C; i < C * 8; i += 256 - C) {
        const int r = i >> 3, c = (i & 7) * 8;
        *reinterpret_cast<uint4*>(p.Aqk + base64 + (size_t)r * H * 64 + c) = *reinterpret_cast<const uint4*>(sStage + r * LD64 + c);
      }
      asm volatile("bar.sync 1, 192;" ::: "memory");
    }
#pragma unroll 2
    for (int i = tid - C; i < C * 16; i += 256 - C) {
      const int r = i >> 4, c = (i & 15) * 8;
      const size_t go = base128 + (size_t)r * ldt + c;
      float kk[8], qq[8], vv[8], gg[8], bb[8], ww[8];
      unpack8(*reinterpret_cast<const uint4*>(p.k + go), kk);
      unpack8(*reinterpret_cast<const uint4*>(p.q + go), qq);
      unpack8(*reinterpret_cast<const uint4*>(p.v + go), vv);
      if (GATE == GATE_VECTOR) load_gate8(p.g + go, gg);
      if (VECTOR_BETA) {
        unpack8(*reinterpret_cast<const uint4*>(p.bg + go), bb);
        unpack8(*reinterpret_cast<const uint4*>(p.wg + go), ww);
      }
      const float bs = VECTOR_BETA ? 0.f : sBeta[r];
      float ev[8], zv[8], qv[8], kv[8];  // E = b k gamma, Z = w v, qg, kg (rounded to BF16 below)
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float gj = GATE == GATE_VECTOR ? gg[j] : (GATE == GATE_SCALAR ? sG[r] : 0.f);
        const float gam = GATE == GATE_NONE ? 1.f : exp2f(gj);
        const float glast = GATE == GATE_VECTOR ? sGl[c + j] : (GATE == GATE_SCALAR ? sG[C - 1] : 0.f);
        ev[j] = (VECTOR_BETA ? bb[j] : bs) * kk[j] * gam;
        zv[j] = vv[j] * (VECTOR_BETA ? ww[j] : bs);
        qv[j] = qq[j] * gam;
        kv[j] = kk[j] * (GATE == GATE_NONE ? 1.f : exp2f(glast - gj));
      }
      *reinterpret_cast<uint4*>(sE + r * LD128 + c) = pack8(ev);
      *reinterpret_cast<uint4*>(sZ + r * LD128 + c) = pack8(zv);
      *reinterpret_cast<uint4*>(p.qg + go) = pack8(qv);
      *reinterpret_cast<uint4*>(p.kg + go) = pack8(kv);
    }
  }

  // ---- Akk = (I + L)^-1: thread c solves column c by forward substitution (x[j] = 0 for j < c comes out by itself) ----
  if (tid < C) {
    float x[C];
#pragma unroll
    for (int i = 0; i < C; i++) {
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int j = 0; j + 3 < i; j += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(sL + i * LDL + j);
        s0 = fmaf(l4.x, x[j], s0); s1 = fmaf(l4.y, x[j + 1], s1); s2 = fmaf(l4.z, x[j + 2], s2); s3 = fmaf(l4.w, x[j + 3], s3);
      }
#pragma unroll
      for (int j = (i / 4) * 4; j < i; j++) s0 = fmaf(sL[i * LDL + j], x[j], s0);
      x[i] = (i == tid ? 1.f : 0.f) - ((s0 + s1) + (s2 + s3));
    }
#pragma unroll
    for (int i = 0; i < C; i++) {
      const bf16 a = f2bf(x[i]);
      sA[i * LD64 + tid] = a;
      p.Akk[base64 + (size_t)i * H * 64 + tid] = a;
    }
  }
  __syncthreads();

  // ---- w = Akk E, u = Akk Z (BF16 operands, as the recompute stage of the backward does) -----------------------------
  {
    Tile<64, 128, 2, 4> acc;
    acc.zero();
    acc.mma<64>(LdmOperand<false>{sA, LD64}, LdmOperand<true>{sE, LD128});
    __syncthreads();
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
    store_tile_bf16<C, 128>(p.w + base128, ldt, sE, LD128);
    store_tile_bf16<C, 128>(p.u + base128, ldt, sZ, LD128);
  }
}

constexpr size_t FWD_LOCAL_SMEM = (size_t)(4 * C * LD128) * sizeof(bf16) + (size_t)(C + 128 + 128 + C) * sizeof(float);
static_assert(3 * (FWD_LOCAL_SMEM + 1024) <= 233472, "three forward chunk CTAs must fit one SM");

// o = scale * qg h[n] + Aqk v_new for one chunk.
__global__ void __launch_bounds__(256) chunk_output_kernel(const bf16* __restrict__ qg, const bf16* __restrict__ Aqk,
                                                           const bf16* __restrict__ v_new, const bf16* __restrict__ hst,
                                                           bf16* __restrict__ o, int T, int H, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);  // [64][136] qg, later the output tile
  bf16* sV = sQ + C * LD128;                     // [64][136] v_new
  bf16* sA = sV + C * LD128;                     // [64][72]  Aqk
  bf16* sH = sA + C * LD64;                      // [128][136] h[n]
  const int n = blockIdx.x, bh = blockIdx.y, b = bh / H, h = bh % H, NT = T / C;
  const size_t row0 = (size_t)b * T + (size_t)n * C;
  const size_t ldt = (size_t)H * 128;
  const size_t base128 = (row0 * H + h) * 128;
  const size_t base64 = (row0 * H + h) * 64;
  load_tile_bf16<C, 128>(sQ, LD128, qg + base128, ldt);
  load_tile_bf16<C, 128>(sV, LD128, v_new + base128, ldt);
  load_tile_bf16<C, 64>(sA, LD64, Aqk + base64, (size_t)H * 64);
  load_tile_bf16<128, 128>(sH, LD128, hst + (((size_t)b * NT + n) * H + h) * 128 * 128, 128);
  __syncthreads();
  Tile<64, 128, 2, 4> acc;
  acc.zero();
  acc.mma<128>(Operand<false>{sQ, LD128}, Operand<true>{sH, LD128});
  acc.for_each([&](int, int, float& x) { x *= scale; });
  acc.mma<64>(Operand<false>{sA, LD64}, Operand<true>{sV, LD128});
  __syncthreads();  // every warp has read qg
  acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
    *reinterpret_cast<uint32_t*>(sQ + r * LD128 + c) = pack_bf16(x0, x1);
  });
  __syncthreads();
  store_tile_bf16<C, 128>(o + base128, ldt, sQ, LD128);
}
constexpr size_t OUTPUT_SMEM = (size_t)(2 * C * LD128 + C * LD64 + 128 * LD128) * sizeof(bf16);

// chunk-local inclusive cumulative sum of a scalar per-head gate in log2 units: one thread per (chunk, head)
__global__ void __launch_bounds__(128) scalar_gate_cumsum_kernel(const void* __restrict__ x, int x_is_f32,
                                                                  float* __restrict__ out, int H, long long chunks_h) {
  const long long ch = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= chunks_h) return;
  const int h = (int)(ch % H);
  const long long row0 = (ch / H) * 64;
  float run = 0.f;
  for (int t = 0; t < 64; t++) {
    const long long at = (row0 + t) * H + h;
    run += x_is_f32 ? static_cast<const float*>(x)[at] : bf2f(static_cast<const bf16*>(x)[at]);
    out[at] = run * 1.4426950408889634f;
  }
}

template <int GATE, bool VB>
cudaError_t run_local(const FwdLocalParams& p, int B, cudaStream_t st) {
  auto kern = chunk_fwd_local_kernel<GATE, VB>;
  const size_t smem = FWD_LOCAL_SMEM;
  cudaError_t e = ensure_dynamic_smem<chunk_fwd_local_kernel<GATE, VB>>(smem);
  if (e != cudaSuccess) return e;
  dim3 grid(p.T / C, B * p.H);
  kern<<<grid, 256, smem, st>>>(p);
  count_launch();
  return cudaGetLastError();
}

bool bad16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

std::atomic<int> g_forward_variant{0};  // output kernel: 0 = TMA + tcgen05, 1 = warp-MMA (cross-check)

}  // namespace
}  // namespace rewy

using namespace rewy;

#define FWD_REQUIRE(field)                                                                                     \
  do {                                                                                                         \
    if (a->field == nullptr) return report_error(REWY_ERR_NULL, "required pointer '" #field "' is NULL");       \
    if (bad16(a->field)) return report_error(REWY_ERR_ALIGN, "pointer '" #field "' is not 16-byte aligned");     \
  } while (0)

extern "C" int rewy_chunk_fwd(const RewyFwdArgs* a, rewy_stream_t stream) {
  if (a == nullptr) return report_error(REWY_ERR_NULL, "args is NULL");
  if (a->family < REWY_DELTA || a->family > REWY_GDN2) return report_error(REWY_ERR_UNSUPPORTED, "unknown family");
  if (a->B <= 0 || a->H <= 0 || a->T < C || a->T % C != 0) return report_error(REWY_ERR_SHAPE, "bad B/T/H");
  if ((long long)a->B * a->H > 65535) return report_error(REWY_ERR_SHAPE, "B*H exceeds the grid limit 65535");
  if ((long long)a->B * a->T * a->H > REWY_MAX_TOKEN_HEADS)
    return report_error(REWY_ERR_SHAPE, "B*T*H exceeds 2^29 token-heads (32-bit tile coordinates)");
  if (a->state_v_first != 0 && a->state_v_first != 1) return report_error(REWY_ERR_UNSUPPORTED, "state_v_first must be 0 or 1");
  if (a->cu_seqlens != nullptr && (a->B != 1 || a->num_seqs <= 0 || (long long)a->num_seqs * a->H > 65535))
    return report_error(REWY_ERR_SHAPE, "packed sequences need B = 1 and 0 < num_seqs*H <= 65535");
  FWD_REQUIRE(q); FWD_REQUIRE(k); FWD_REQUIRE(v); FWD_REQUIRE(o); FWD_REQUIRE(Aqk); FWD_REQUIRE(Akk); FWD_REQUIRE(w);
  FWD_REQUIRE(u); FWD_REQUIRE(qg); FWD_REQUIRE(kg); FWD_REQUIRE(v_new); FWD_REQUIRE(h); FWD_REQUIRE(ctrl);
  if (a->family != REWY_DELTA) FWD_REQUIRE(g);
  if (a->family == REWY_GDN2) { FWD_REQUIRE(b_gate); FWD_REQUIRE(w_gate); }
  else FWD_REQUIRE(beta);
  if (a->h0 != nullptr && bad16(a->h0)) return report_error(REWY_ERR_ALIGN, "pointer 'h0' is not 16-byte aligned");
  if (a->final_state != nullptr && bad16(a->final_state))
    return report_error(REWY_ERR_ALIGN, "pointer 'final_state' is not 16-byte aligned");
  cudaStream_t st = (cudaStream_t)stream;
  FwdLocalParams p;
  p.q = (const bf16*)a->q; p.k = (const bf16*)a->k; p.v = (const bf16*)a->v; p.bg = (const bf16*)a->b_gate;
  p.wg = (const bf16*)a->w_gate; p.g = a->g; p.beta = a->beta;
  p.Akk = (bf16*)a->Akk; p.Aqk = (bf16*)a->Aqk; p.w = (bf16*)a->w; p.u = (bf16*)a->u; p.qg = (bf16*)a->qg; p.kg = (bf16*)a->kg;
  p.T = a->T; p.H = a->H; p.scale = a->scale;
  cudaError_t e = cudaMemsetAsync(a->ctrl, 0, sizeof(int), st);
  if (e == cudaSuccess) {
    switch (a->family) {
      case REWY_DELTA: e = run_local<GATE_NONE, false>(p, a->B, st); break;
      case REWY_GDN: e = run_local<GATE_SCALAR, false>(p, a->B, st); break;
      case REWY_KDA: e = run_local<GATE_VECTOR, false>(p, a->B, st); break;
      default: e = run_local<GATE_VECTOR, true>(p, a->B, st); break;
    }
  }
  if (e == cudaSuccess) {
    RewyBwdArgs ba{};
    ba.family = a->family; ba.B = a->B; ba.T = a->T; ba.H = a->H; ba.state_v_first = a->state_v_first; ba.scale = a->scale;
    ba.g = a->g; ba.h0 = a->h0; ba.cu_seqlens = a->cu_seqlens; ba.num_seqs = a->num_seqs;
    RewyStageBuffers sb{};
    sb.w = a->w; sb.u = a->u; sb.kg = a->kg; sb.h = a->h; sb.v_new = a->v_new;
    e = launch_fwd_scan_tc(ba, sb, static_cast<int*>(a->ctrl), st, a->final_state);
  }
  if (e == cudaSuccess && g_forward_variant.load(std::memory_order_relaxed) == 0) {
    e = launch_chunk_output_tc(*a, static_cast<int*>(a->ctrl), st);
  } else if (e == cudaSuccess) {
    e = ensure_dynamic_smem<chunk_output_kernel>(OUTPUT_SMEM);
    if (e == cudaSuccess) {
      dim3 grid(a->T / C, a->B * a->H);
      chunk_output_kernel<<<grid, 256, OUTPUT_SMEM, st>>>((const bf16*)a->qg, (const bf16*)a->Aqk, (const bf16*)a->v_new,
                                                         (const bf16*)a->h, (bf16*)a->o, a->T, a->H, a->scale);
      count_launch();
      e = cudaGetLastError();
    }
  }
  if (e != cudaSuccess) {
    char msg[160];
    snprintf(msg, sizeof(msg), "chunk forward: %s", cudaGetErrorString(e));
    return report_error(REWY_ERR_LAUNCH, msg);
  }
  return REWY_OK;
}

extern "C" int rewy_set_forward_variant(int variant) {
  if (variant != 0 && variant != 1) return report_error(REWY_ERR_UNSUPPORTED, "forward variant must be 0 or 1");
  g_forward_variant.store(variant, std::memory_order_relaxed);
  return REWY_OK;
}

extern "C" int rewy_scalar_gate_cumsum_fwd(const void* x, int x_is_f32, float* g_cumsum, int32_t B, int32_t T, int32_t H,
                                           rewy_stream_t stream) {
  if (x == nullptr || g_cumsum == nullptr) return report_error(REWY_ERR_NULL, "x or g_cumsum is NULL");
  if (B <= 0 || H <= 0 || T < C || T % C != 0) return report_error(REWY_ERR_SHAPE, "bad B/T/H");
  const long long chunks_h = (long long)B * (T / C) * H;
  scalar_gate_cumsum_kernel<<<(unsigned)((chunks_h + 127) / 128), 128, 0, (cudaStream_t)stream>>>(x, x_is_f32, g_cumsum, H,
                                                                                                 chunks_h);
  count_launch();
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return report_error(REWY_ERR_LAUNCH, cudaGetErrorString(e));
  return REWY_OK;
}
