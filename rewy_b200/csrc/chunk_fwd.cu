// Forward pass of the four families: what the autograd forward needs besides the backward's own stages.
//
//   chunk_fwd_local_kernel   one CTA per chunk: Akk = (I + tril(E Y^T, -1))^-1, Aqk = scale tril(Qg Y^T),
//                            w = Akk E, u = Akk Z, qg, kg          (E = b k gamma, Y = k / gamma, Z = w v)
//   fwd_scan_tc_kernel       (state_scan_tc.cu) h[n], v_new, final state
//   chunk_output_tc_kernel   (chunk_output_tc.cu, tcgen05) o = scale qg h[n] + Aqk v_new; chunk_output_kernel here is its
//                            warp-MMA cross-check (rewy_set_forward_variant(1))
// Replaces FLA's chunk_kda_fwd / chunk_gdn2_fwd / chunk_gated_delta_rule_fwd / chunk_delta_rule_fwd as the reference
// binds them (src/fast_delta_rule/_compat/kda.py:89-113, gdn2.py:94-117, gdn.py:33-125, delta.py).
//
// The two 64x64x128 products that build the A matrices use centred gate factors (alpha = 2^(G - c), zeta = 1/alpha with
// c the per-channel mid-point of G over the chunk) and BF16 hi/lo operand pairs in three passes (about 16 mantissa
// bits), accumulated in FP32 by warp-level MMA; scalar gates apply their pairwise factor 2^(G_i - G_j) to the exact
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

template <int GATE, bool VECTOR_BETA>
__global__ void __launch_bounds__(256) chunk_fwd_local_kernel(const FwdLocalParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sA = reinterpret_cast<bf16*>(smem_raw);            // [64][72]   Akk (BF16) once inverted
  bf16* sE = sA + C * LD64;                                // [64][136]  b*k*gamma, later w
  bf16* sZ = sE + C * LD128;                               // [64][136]  w_gate*v, later u
  float* sL = reinterpret_cast<float*>(sZ + C * LD128);    // [64][68]   strictly lower part of E Y^T
  float* sG = sL + C * LDL;                                // [64]       scalar gate rows
  float* sGl = sG + C;                                     // [128]      last gate row of the chunk (vector gate)
  float* sCen = sGl + 128;                                 // [128]      per-channel centre of the gate (vector gate)
  float* sBeta = sCen + 128;                               // [64]       scalar beta rows
  bf16* sT = reinterpret_cast<bf16*>(sBeta + C);           // operand tiles of the two A products, [64][136] each:
  // vector gate: Qc hi, Qc lo, Ec hi, Ec lo, Yc hi, Yc lo;  scalar gate / none: q, k
  constexpr int TILE = C * LD128;

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
#pragma unroll 8
    for (int t = 0; t < C; t++) {
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
  float* sGf = reinterpret_cast<float*>(sT + 3 * TILE);  // [64][132] FP32 gate tile of a wide chunk

  // element-wise operands, 8 columns (16 bytes of BF16) per thread-iteration
  for (int i = tid; i < C * 16; i += blockDim.x) {
    const int r = i >> 4, c = (i & 15) * 8;
    const size_t go = base128 + (size_t)r * ldt + c;
    const uint4 kr = *reinterpret_cast<const uint4*>(p.k + go);
    const uint4 qr = *reinterpret_cast<const uint4*>(p.q + go);
    const uint4 vr = *reinterpret_cast<const uint4*>(p.v + go);
    float gg[8];
    if (GATE == GATE_VECTOR) {
      const float4 ga = *reinterpret_cast<const float4*>(p.g + go), gb = *reinterpret_cast<const float4*>(p.g + go + 4);
      gg[0] = ga.x; gg[1] = ga.y; gg[2] = ga.z; gg[3] = ga.w; gg[4] = gb.x; gg[5] = gb.y; gg[6] = gb.z; gg[7] = gb.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) gg[j] = GATE == GATE_SCALAR ? sG[r] : 0.f;
    }
    uint4 br = make_uint4(0, 0, 0, 0), wr = br;
    const float bs = VECTOR_BETA ? 0.f : sBeta[r];
    if (VECTOR_BETA) {
      br = *reinterpret_cast<const uint4*>(p.bg + go);
      wr = *reinterpret_cast<const uint4*>(p.wg + go);
    }
    const uint32_t* ku = reinterpret_cast<const uint32_t*>(&kr);
    const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qr);
    const uint32_t* vu = reinterpret_cast<const uint32_t*>(&vr);
    const uint32_t* bu = reinterpret_cast<const uint32_t*>(&br);
    const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wr);
    float ev[8], zv[8], qv[8], kv[8];  // E = b k gamma, Z = w v, qg, kg (rounded to BF16 below)
    float qc[8], ec[8], yc[8];          // centred operands of the A products (vector gate)
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float2 kk2 = unpack_bf16(ku[j >> 1]), qq2 = unpack_bf16(qu[j >> 1]), vv2 = unpack_bf16(vu[j >> 1]);
      const float kk = (j & 1) ? kk2.y : kk2.x, qq = (j & 1) ? qq2.y : qq2.x, vv = (j & 1) ? vv2.y : vv2.x;
      float bb = bs, ww = bs;
      if (VECTOR_BETA) {
        const float2 b2 = unpack_bf16(bu[j >> 1]), w2 = unpack_bf16(wu[j >> 1]);
        bb = (j & 1) ? b2.y : b2.x;
        ww = (j & 1) ? w2.y : w2.x;
      }
      const float gj = gg[j];
      const float gam = GATE == GATE_NONE ? 1.f : exp2f(gj);
      const float glast = GATE == GATE_VECTOR ? sGl[c + j] : (GATE == GATE_SCALAR ? sG[C - 1] : 0.f);
      ev[j] = bb * kk * gam;
      zv[j] = vv * ww;
      qv[j] = qq * gam;
      kv[j] = kk * (GATE == GATE_NONE ? 1.f : exp2f(glast - gj));
      if (GATE == GATE_VECTOR && !wide) {
        const float al = exp2f(gj - sCen[c + j]);
        qc[j] = qq * al;
        ec[j] = bb * kk * al;
        yc[j] = kk * __frcp_rn(al);
      }
    }
    uint32_t eo[4], zo[4], qo[4], ko[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      eo[j] = pack_bf16(ev[2 * j], ev[2 * j + 1]);
      zo[j] = pack_bf16(zv[2 * j], zv[2 * j + 1]);
      qo[j] = pack_bf16(qv[2 * j], qv[2 * j + 1]);
      ko[j] = pack_bf16(kv[2 * j], kv[2 * j + 1]);
    }
    *reinterpret_cast<uint4*>(sE + r * LD128 + c) = make_uint4(eo[0], eo[1], eo[2], eo[3]);
    *reinterpret_cast<uint4*>(sZ + r * LD128 + c) = make_uint4(zo[0], zo[1], zo[2], zo[3]);
    *reinterpret_cast<uint4*>(p.qg + go) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
    *reinterpret_cast<uint4*>(p.kg + go) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
    if (GATE == GATE_VECTOR && !wide) {
      split_store8(sT + 0 * TILE + r * LD128 + c, sT + 1 * TILE + r * LD128 + c, qc);
      split_store8(sT + 2 * TILE + r * LD128 + c, sT + 3 * TILE + r * LD128 + c, ec);
      split_store8(sT + 4 * TILE + r * LD128 + c, sT + 5 * TILE + r * LD128 + c, yc);
    } else {
      *reinterpret_cast<uint4*>(sT + 0 * TILE + r * LD128 + c) = qr;
      *reinterpret_cast<uint4*>(sT + 1 * TILE + r * LD128 + c) = kr;
      if (GATE == GATE_VECTOR) {  // wide chunk: raw key gate and gate rows for the pairwise sums
        if (VECTOR_BETA) *reinterpret_cast<uint4*>(sT + 2 * TILE + r * LD128 + c) = br;
        *reinterpret_cast<float4*>(sGf + r * LDG + c) = make_float4(gg[0], gg[1], gg[2], gg[3]);
        *reinterpret_cast<float4*>(sGf + r * LDG + c + 4) = make_float4(gg[4], gg[5], gg[6], gg[7]);
      }
    }
  }
  __syncthreads();

  // ---- the two A products: Qc Yc^T (-> Aqk) and Ec Yc^T (-> strictly lower part of I + L) -------------------------
  if (GATE == GATE_VECTOR && wide) {
    // exact pairwise sums, thread = (row i, every fourth column j)
    const bf16 *sQr = sT, *sKr = sT + TILE, *sBr = sT + 2 * TILE;
    const int i = tid >> 2;
    const float beta_i = VECTOR_BETA ? 0.f : sBeta[i];
    for (int j = tid & 3; j < C; j += 4) {
      float aq = 0.f, ak = 0.f;
      if (j <= i) {
        for (int kk = 0; kk < 128; kk++) {
          const float f = exp2f(sGf[i * LDG + kk] - sGf[j * LDG + kk]) * bf2f(sKr[j * LD128 + kk]);
          aq = fmaf(bf2f(sQr[i * LD128 + kk]), f, aq);
          const float bi = VECTOR_BETA ? bf2f(sBr[i * LD128 + kk]) : beta_i;
          ak = fmaf(bi * bf2f(sKr[i * LD128 + kk]), f, ak);
        }
      }
      p.Aqk[base64 + (size_t)i * H * 64 + j] = f2bf(p.scale * aq);
      sL[i * LDL + j] = j < i ? ak : 0.f;
    }
  } else {
    Tile<64, 64, 2, 4> aq, ak;
    aq.zero();
    ak.zero();
    if (GATE == GATE_VECTOR) {
      const Operand<false> Qh{sT + 0 * TILE, LD128}, Ql{sT + 1 * TILE, LD128}, Eh{sT + 2 * TILE, LD128},
          El{sT + 3 * TILE, LD128}, Yh{sT + 4 * TILE, LD128}, Yl{sT + 5 * TILE, LD128};
      aq.mma<128>(Qh, Yh); aq.mma<128>(Ql, Yh); aq.mma<128>(Qh, Yl);
      ak.mma<128>(Eh, Yh); ak.mma<128>(El, Yh); ak.mma<128>(Eh, Yl);
    } else {
      const Operand<false> Q{sT + 0 * TILE, LD128}, K{sT + 1 * TILE, LD128};
      aq.mma<128>(Q, K);
      ak.mma<128>(K, K);
    }
    aq.for_each_pair([&](int r, int c, float& x0, float& x1) {
      float f0 = p.scale, f1 = p.scale;
      if (GATE == GATE_SCALAR) {
        f0 *= exp2f(sG[r] - sG[c <= r ? c : r]);
        f1 *= exp2f(sG[r] - sG[c + 1 <= r ? c + 1 : r]);
      }
      const float y0 = c <= r ? x0 * f0 : 0.f, y1 = c + 1 <= r ? x1 * f1 : 0.f;
      *reinterpret_cast<uint32_t*>(p.Aqk + base64 + (size_t)r * H * 64 + c) = pack_bf16(y0, y1);
    });
    ak.for_each_pair([&](int r, int c, float& x0, float& x1) {
      float f0 = 1.f, f1 = 1.f;
      if (GATE != GATE_VECTOR) {  // exact k k^T: beta and the pairwise gate factor go on afterwards
        f0 = f1 = VECTOR_BETA ? 1.f : sBeta[r];
        if (GATE == GATE_SCALAR) {
          f0 *= exp2f(sG[r] - sG[c < r ? c : r]);
          f1 *= exp2f(sG[r] - sG[c + 1 < r ? c + 1 : r]);
        }
      }
      sL[r * LDL + c] = c < r ? x0 * f0 : 0.f;
      sL[r * LDL + c + 1] = c + 1 < r ? x1 * f1 : 0.f;
    });
  }
  __syncthreads();

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
    acc.mma<64>(Operand<false>{sA, LD64}, Operand<true>{sE, LD128});
    __syncthreads();
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(sE + r * LD128 + c) = pack_bf16(x0, x1);
    });
    acc.zero();
    acc.mma<64>(Operand<false>{sA, LD64}, Operand<true>{sZ, LD128});
    __syncthreads();
    acc.for_each_pair([&](int r, int c, float& x0, float& x1) {
      *reinterpret_cast<uint32_t*>(sZ + r * LD128 + c) = pack_bf16(x0, x1);
    });
    __syncthreads();
    store_tile_bf16<C, 128>(p.w + base128, ldt, sE, LD128);
    store_tile_bf16<C, 128>(p.u + base128, ldt, sZ, LD128);
  }
}

constexpr size_t FWD_LOCAL_SMEM_FIXED = (size_t)(C * LD64 + 2 * C * LD128) * sizeof(bf16) +
                                        (size_t)(C * LDL + C + 128 + 128 + C) * sizeof(float);
constexpr size_t FWD_LOCAL_SMEM_VECTOR = FWD_LOCAL_SMEM_FIXED + (size_t)6 * C * LD128 * sizeof(bf16);
constexpr size_t FWD_LOCAL_SMEM_SCALAR = FWD_LOCAL_SMEM_FIXED + (size_t)2 * C * LD128 * sizeof(bf16);
static_assert(FWD_LOCAL_SMEM_VECTOR <= 232448, "shared memory plan of the forward chunk kernel exceeds 227 KB");

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
  const size_t smem = GATE == GATE_VECTOR ? FWD_LOCAL_SMEM_VECTOR : FWD_LOCAL_SMEM_SCALAR;
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
