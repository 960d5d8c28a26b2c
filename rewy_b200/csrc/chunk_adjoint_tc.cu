// Stage "chunk adjoint" on the Blackwell tensor cores (tcgen05 + TMEM accumulators, TMA tile loads and stores).
//
// Same mathematics as chunk_adjoint.cu (the reference functions it replaces are listed there); this file is
// the production path.  One persistent CTA per SM walks over chunks (head fastest, so CTAs that run together
// read the same token rows); per chunk:
//   P        = Akk^T (dR_hi + dR_lo)               M=128 N=128 K=64  both operands MN-major; the A tile is used for
//                                                  both 64-row halves, so lanes 64..127 repeat rows 0..63
//   [H;-D]   = [dO;P] R^T                          M=128 N=64  K=128 one stacked product
//   [X1|X3]  = h [dO;P]^T                          M=128 (key channel) N=128 (token | token) K=128
//   [X2|X4]  = Yc^T [H;D]^T                        N=128 K=64, BF16 hi/lo split operands, three passes
//   X5       = dh R^T                              N=64 K=128
//   X6       = Ec^T D + Qc^T H                     N=64 K=64+64, three passes each
// Yc^T, Ec^T and Qc^T are written by their owner threads straight into tensor memory (A operand from TMEM); every
// other operand is a tile exactly as TMA lands it.  The accumulators of the last products are [key channel x
// token]: epilogue thread (k, token quarter) sees per-channel gate factors as scalars and runs the reverse gate
// cumsum as a running sum.  What keeps the kernel fed:
//   * one elected thread issues every TMA copy, product and commit, from warp-uniform code with descriptor words
//     precomputed (a product costs it two integer adds);
//   * the next chunk's tiles are requested in three instalments (k,q,g / Akk,dR,v / dO,R,h) so that the SM's
//     memory port is never saturated while the epilogue stores need it; k, q, g arrive as tiles and are read
//     into registers once; beta rows are double-buffered and fetched under a tensor-core wait;
//   * dv and dg leave as tiles by bulk stores; per-token sums go through small per-warp arrays, per-channel
//     sums through spare TMEM columns (no shared-memory atomics).
// Chunks whose cumulative gate spans 80 or more log2 units are not processed here: their indices are appended
// to a list that the warp-MMA kernel (exact pairwise path) works off afterwards.
#include <cstdio>
#include "tc05.cuh"

namespace rewy {
namespace {
using namespace tc;

constexpr float SPAN_LIMIT = 80.f;

// Division of a non-negative int below 2^31 by a divisor fixed at launch: quotient = umulhi(x, mul) >> shift.
struct FastDiv {
  uint32_t mul, shift, div;
  __device__ __forceinline__ int quot(int x) const { return div == 1 ? x : (int)(__umulhi((uint32_t)x, mul) >> shift); }
};

struct TcParams {
  const bf16 *q, *k, *v, *bg, *wg, *dh;
  const float *g, *beta;
  void *dq, *dk, *dbg, *dwg;
  bf16* dv;
  float *dg, *dbeta;
  int* wide_list;   // [0] = count, [1..] = flattened chunk indices with a wide gate span
  int* err;         // device status word: non-zero if a bounded wait gave up
  int T, H, NT, total_chunks, out_f32;
  FastDiv div_nt, div_h;
  float scale;
};

// Shared-memory plan (byte offsets from a 1024-byte aligned base).  Regions are reused as soon as the product that
// read them is complete; the aliases are listed after the tiles.
struct Smem {
  static constexpr uint32_t AKK = 0;                   // [64 j][64 i] BF16                      8 KB
  static constexpr uint32_t DRHI = AKK + 8192;         // 2 panels [64 j][64 v]                  16 KB
  static constexpr uint32_t DRLO = DRHI + 16384;       //                                        16 KB
  static constexpr uint32_t DOP = DRLO + 16384;        // per v-panel: dO [64][64] then P [64][64] 32 KB
  static constexpr uint32_t R = DOP + 32768;           // 2 panels [64 j][64 v]                  16 KB
  static constexpr uint32_t HS = R + 16384;            // 2 panels [128 k][64 v]  h              32 KB
  static constexpr uint32_t HHI = HS + 32768;          // dAqk hi [64 i][64 j]                   8 KB
  static constexpr uint32_t DHI = HHI + 8192;          // dAkk hi; [dAqk hi ; dAkk hi] is one 128-row operand
  static constexpr uint32_t HLO = DHI + 8192;          // dAqk lo
  static constexpr uint32_t DLO = HLO + 8192;          // dAkk lo
  static constexpr uint32_t PARK = DLO + 8192;         // float [64 t][128 k]: parked gate-gradient rows, then the dg tile   32 KB
  static constexpr uint32_t GT = PARK + 32768;         // g tile of the NEXT chunk (4 panels [64 t][32 k] FP32)                32 KB
  static constexpr uint32_t DQT = HS;                  // dq and dk tiles (dense [64 t][128 k] BF16, 16 KB each) take the h buffer
  static constexpr uint32_t DKT = HS + 16384;          // once [X1|X3] is complete; they leave by bulk stores before h is reloaded
  static constexpr uint32_t BT = DOP;                  // GDN2: key-gate tile of the NEXT chunk, its two panels in the two dO tiles
                                                       // (16384 apart) once [X1|X3] is complete; read into registers at chunk start
  static constexpr uint32_t DBT = R;                   // GDN2: key-gate gradient tile (dense [64 t][128 k] BF16) during pass B
  static constexpr uint32_t DWT = PARK;                // GDN2: value-gate gradient tile (2 panels [64 i][64 v]) and, behind it,
  static constexpr uint32_t WT = PARK + 16384;         // the value-gate tile of this chunk: PARK is free until pass A
  static constexpr uint32_t DHT = DRHI;                // dh tile (2 panels [128 k][64 v]) takes the dR tiles once P is done
  static constexpr uint32_t KT = HLO;                  // k tile of the NEXT chunk (2 panels [64 t][64 k]) lands in the two lo
                                                       // tiles once they are dead and is read into registers at chunk start
  static constexpr uint32_t DVT = HLO;                 // dv tile (2 panels [64 i][64 v]) between the P epilogue and its bulk store,
                                                       // which has read it before the lo tiles are written
  static constexpr uint32_t VT = HHI;                  // v tile (2 panels [64 i][64 v]) aliases the two hi tiles until P is done
  static constexpr uint32_t TILES_END = GT + 32768;    // 221184
  static constexpr uint32_t QT = DOP + 8192;           // q tile of the NEXT chunk: its two panels [64 t][64 k] land in the two P
                                                       // tiles (16384 apart) once the products that read P are complete, and
                                                       // are read into registers at chunk start, before P is written again
  static constexpr uint32_t BETA = TILES_END;          // float[2][64] beta of this chunk and of the next one
  static constexpr uint32_t DBETA = BETA + 512;        // float[64]
  static constexpr uint32_t GS = DBETA + 256;          // float[2][64] scalar gate rows, this chunk and the next
  static constexpr uint32_t DGS = GS + 512;            // float[64] per-token gate sums (scalar gate)
  static constexpr uint32_t MINMAX = DGS + 256;        // float[4][2][128] per-quarter min / max of the gate rows (chunk start)
  static constexpr uint32_t DBP = MINMAX;              // float[8][64] sum_v v*P per token, one row per 16 value columns
  static constexpr uint32_t DBW = DBP + 2048;          // float[16 warps][16 tokens] sum_k k*(gamma eb) of the warp's channels
  static constexpr uint32_t DGW = DBW + 1024;          // float[16][16] same for the scalar-gate rows
  static constexpr uint32_t GL = MINMAX + 4096;        // float[128] last-row gate of the chunk per channel
  static constexpr uint32_t BARS = GL + 512;        // 8 mbarriers
  static constexpr uint32_t TMEM = BARS + 128;         // uint32 tmem base (+ flags)
  static constexpr uint32_t TOTAL = TMEM + 64;
};
static_assert(Smem::TOTAL + 1024 <= 232448, "shared memory plan exceeds the 227 KB per-CTA limit");

enum { BAR_A = 0, BAR_B, BAR_C, BAR_D, BAR_P, BAR_HD, BAR_C3, BAR_G, BAR_Q, BAR_QR, BAR_W, NUM_BARS };

// TMEM column plan (512 columns allocated).
constexpr uint32_t TM_P = 0, TM_HD = 128, TM_X1 = 192, TM_X3 = 256, TM_X2 = 320, TM_X4 = 384, TM_X5 = 448, TM_X6 = 64;
// Operand tiles of the matrix-intra products, written by their owner threads (lane = key channel; 16 tokens = 8
// packed columns per thread; hi block then lo block, 32 columns each): Yc^T in the last 64 columns until [X2 | X4]
// is complete (X5, issued after it, accumulates there), Ec^T where P was, Qc^T where the
// stacked product was.
// Per-channel scratch of the gate epilogue (lane = key channel) takes the first columns of Ec^T once X6 is complete:
// column TM_SCR + wg holds sum_v h*dh of value quarter wg, +4 the chunk-end sums and +8 the gate-gradient totals
// of token quarter wg.
constexpr uint32_t TM_SCR = 0;
constexpr uint32_t TM_Y = 448, TM_E = 0, TM_QC = 128;

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&r)[16]) {
  uint32_t u[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) r[i] = __uint_as_float(u[i]);
}

__device__ __forceinline__ void tmem_st1(uint32_t taddr, float x) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(__float_as_uint(x)) : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&r)[8]) {
  uint32_t u[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; i++) r[i] = __uint_as_float(u[i]);
}

__device__ __forceinline__ void store_out1(void* base, size_t off, float x, int out_f32) {
  if (out_f32)
    reinterpret_cast<float*>(base)[off] = x;
  else
    reinterpret_cast<bf16*>(base)[off] = f2bf(x);
}

// Pack 8 FP32 values into 8 BF16 "hi" and 8 BF16 "lo" (residual) values.
__device__ __forceinline__ void split8(const float (&x)[8], uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 hh = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
    float2 hf = __bfloat1622float2(hh);
    h[i] = *reinterpret_cast<uint32_t*>(&hh);
    l[i] = pack_bf16(x[2 * i] - hf.x, x[2 * i + 1] - hf.y);
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// K-major BF16 product over KSTEPS K=16 steps; tiles made of 64-element (128-byte) panels `a_panel` / `b_panel` bytes
// apart.  `a` and `b` are descriptor low words (desc_lo) of the tile bases; all offsets fold into immediates.
template <int KSTEPS>
__device__ __forceinline__ void mma_kmajor(uint32_t d, uint32_t a, uint32_t a_panel, uint32_t b, uint32_t b_panel,
                                           uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ks++)
    mma_f16_lo(d, a + (((ks >> 2) * a_panel + (ks & 3) * 32) >> 4), b + (((ks >> 2) * b_panel + (ks & 3) * 32) >> 4), idesc,
               accumulate || ks > 0);
}
// Four K=16 steps with A in tensor memory (8 columns per step) and B in shared memory, K-major (step 32 B) or
// MN-major (step 2048 B).
__device__ __forceinline__ void mma_ts4(uint32_t d, uint32_t a_tmem, uint32_t b, uint32_t b_step, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < 4; ks++) mma_f16_ts(d, a_tmem + ks * 8, b + ((ks * b_step) >> 4), idesc, accumulate || ks > 0);
}

// Sum over the warp of x[lane & 15] for each of the 16 per-thread values (16 shuffles); every lane returns the
// total of value index (lane & 15).
__device__ __forceinline__ float warp_sum16(float (&x)[16], int lane) {
#pragma unroll
  for (int m = 8, n = 16; m >= 1; m >>= 1, n >>= 1) {
    const bool up = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; i++) {
      float send = up ? x[i] : x[i + n / 2];
      float keep = up ? x[i + n / 2] : x[i];
      x[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
    }
  }
  return x[0] + __shfl_xor_sync(0xffffffffu, x[0], 16);
}


// 512 threads: thread = (key channel kch = tid & 127, token quarter wg = tid >> 7).  The four warpgroups share
// the 128 TMEM lanes (warp w reads lanes 32*(w & 3) ..) and split the columns of every accumulator.
constexpr int TPB = 512;
constexpr int NWG = 4;
constexpr int HALF = 16;  // tokens per thread

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
// Same for 8 values: every lane returns the warp total of value index (lane & 7) (9 shuffles).
__device__ __forceinline__ float warp_sum8(float (&x)[8], int lane) {
#pragma unroll
  for (int m = 4, n = 8; m >= 1; m >>= 1, n >>= 1) {
    const bool up = (lane & m) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; i++) {
      float send = up ? x[i] : x[i + n / 2];
      float keep = up ? x[i + n / 2] : x[i];
      x[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
    }
  }
  float s = x[0] + __shfl_xor_sync(0xffffffffu, x[0], 8);
  return s + __shfl_xor_sync(0xffffffffu, s, 16);
}

template <int GATE, bool VB, bool OUTF32>
__global__ void __launch_bounds__(TPB, 1)
chunk_adjoint_tc_kernel(const __grid_constant__ CUtensorMap tmAkk, const __grid_constant__ CUtensorMap tmDRhi,
                        const __grid_constant__ CUtensorMap tmDRlo, const __grid_constant__ CUtensorMap tmDO,
                        const __grid_constant__ CUtensorMap tmR, const __grid_constant__ CUtensorMap tmH,
                        const __grid_constant__ CUtensorMap tmDH, const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmG,
                        const __grid_constant__ CUtensorMap tmDG, const __grid_constant__ CUtensorMap tmQ,
                        const __grid_constant__ CUtensorMap tmDV, const __grid_constant__ CUtensorMap tmDQ,
                        const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmBG,
                        const __grid_constant__ CUtensorMap tmDBG, const __grid_constant__ CUtensorMap tmWG,
                        const __grid_constant__ CUtensorMap tmDW, const TcParams p) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  float* sBeta2 = reinterpret_cast<float*>(sm + Smem::BETA);
  float* sDb = reinterpret_cast<float*>(sm + Smem::DBETA);
  float* sGs2 = reinterpret_cast<float*>(sm + Smem::GS);
  float* sDgs = reinterpret_cast<float*>(sm + Smem::DGS);
  float* sMinMax = reinterpret_cast<float*>(sm + Smem::MINMAX);
  float* sDbP = reinterpret_cast<float*>(sm + Smem::DBP);
  float* sDbW = reinterpret_cast<float*>(sm + Smem::DBW);
  float* sDgW = reinterpret_cast<float*>(sm + Smem::DGW);
  float* sGl = reinterpret_cast<float*>(sm + Smem::GL);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + Smem::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + Smem::TMEM);
  const uint32_t sb = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kch = tid & 127, wg = tid >> 7, t0 = wg * HALF;
  const int T = p.T, H = p.H, NT = p.NT;
  const size_t ldt = (size_t)H * 128;
  const float scale = p.scale;

  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; i++) mbar_init(&bars[i], i == BAR_QR ? TPB / 32 : 1);  // BAR_QR: one arrival per warp
    fence_barrier_init();
    prefetch_tmap(&tmAkk); prefetch_tmap(&tmDRhi); prefetch_tmap(&tmDRlo); prefetch_tmap(&tmDO);
    prefetch_tmap(&tmR); prefetch_tmap(&tmH); prefetch_tmap(&tmDH); prefetch_tmap(&tmV);
    prefetch_tmap(&tmK); prefetch_tmap(&tmG);
    if (GATE == GATE_VECTOR) prefetch_tmap(&tmDG);
    prefetch_tmap(&tmQ); prefetch_tmap(&tmDV);
    if (!OUTF32) { prefetch_tmap(&tmDQ); prefetch_tmap(&tmDK); }
    if (VB) { prefetch_tmap(&tmBG); prefetch_tmap(&tmWG); if (!OUTF32) { prefetch_tmap(&tmDBG); prefetch_tmap(&tmDW); } }
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *tmem_slot;
  const uint32_t tlane = tb + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's TMEM lanes
  // the one thread that issues every TMA copy, tensor-core product and commit (bulk store groups are per thread)
  const bool leader = warp == 0 && elect_one();
  // The last product group is issued from another warp: the leader's warp is still busy with its own share of the
  // operand tiles when the others have finished theirs, and whoever issues is late for the epilogue by that much.
  const bool leader2 = warp == 1 && elect_one();
  uint32_t ph = 0;                                                  // phase bit per barrier
  bool alive = true;                                                // false once a bounded wait gave up

  constexpr uint32_t ID_P = instr_desc(FMT_BF16, 128, 128, true, true);
  constexpr uint32_t ID_KK = instr_desc(FMT_BF16, 128, 64, false, false);
  constexpr uint32_t ID_KK128 = instr_desc(FMT_BF16, 128, 128, false, false);
  constexpr uint32_t ID_KMN = instr_desc(FMT_BF16, 128, 64, false, true);

  // descriptor low word of the tile at byte offset `off` of the plan
  const uint32_t sb4 = sb >> 4;  // the plan's base is 1024-byte aligned, so offsets add without carries
  auto dl = [&](uint32_t off, uint32_t lbo) { return sb4 + (off >> 4) + ((lbo >> 4) << 16); };
  auto wait = [&](int b, int code) {
    if (alive) alive = mbar_wait(&bars[b], (ph >> b) & 1u, p.err, code);
  };
  // Tile loads of one chunk, issued by one thread, in three instalments so that the SM's memory port is never
  // saturated for long while the epilogue's global stores need it:
  //   LOAD_G  {k, q, g}            needed at the start of the chunk     -> issued before the previous chunk's pass B
  //   LOAD_A  {Akk, dR hi/lo, v}   needed by the first product          -> issued after the previous chunk's pass B
  //   LOAD_BC {dO, R} and {h}      needed by the second product group   -> issued at the start of the chunk itself
  constexpr int LOAD_G = 1, LOAD_A = 2, LOAD_BC = 4;
  auto issue_loads = [&](int chunk, int parts) {
    const int bn = p.div_h.quot(chunk), h = chunk - bn * H, b = p.div_nt.quot(bn), n = bn - b * NT;
    const int row0 = b * T + n * C, hrow0 = ((b * NT + n) * H + h) * 128;
    if (parts & LOAD_G) {
      mbar_expect_tx(&bars[BAR_G], 2 * 16384 + (GATE == GATE_VECTOR ? 32768 : 0) + (VB ? 16384 : 0));
      if (VB)
        for (int pn = 0; pn < 2; pn++) tma_load_2d(sm + Smem::BT + pn * 16384, &tmBG, h * 128 + 64 * pn, row0, &bars[BAR_G]);
      tma_load_3d(sm + Smem::KT, &tmK, h * 128, row0, 0, &bars[BAR_G]);
      for (int pn = 0; pn < 2; pn++) tma_load_2d(sm + Smem::QT + pn * 16384, &tmQ, h * 128 + 64 * pn, row0, &bars[BAR_G]);
      if (GATE == GATE_VECTOR) tma_load_3d(sm + Smem::GT, &tmG, h * 128, row0, 0, &bars[BAR_G]);
    }
    if (parts & LOAD_A) {
      mbar_expect_tx(&bars[BAR_A], 8192 + 3 * 16384);
      tma_load_2d(sm + Smem::AKK, &tmAkk, h * 64, row0, &bars[BAR_A]);
      tma_load_3d(sm + Smem::DRHI, &tmDRhi, h * 128, row0, 0, &bars[BAR_A]);
      tma_load_3d(sm + Smem::DRLO, &tmDRlo, h * 128, row0, 0, &bars[BAR_A]);
      tma_load_3d(sm + Smem::VT, &tmV, h * 128, row0, 0, &bars[BAR_A]);
    }
    if (parts & LOAD_BC) {
      mbar_expect_tx(&bars[BAR_B], 2 * 16384);
      for (int pn = 0; pn < 2; pn++) tma_load_2d(sm + Smem::DOP + pn * 16384, &tmDO, h * 128 + 64 * pn, row0, &bars[BAR_B]);
      tma_load_3d(sm + Smem::R, &tmR, h * 128, row0, 0, &bars[BAR_B]);
      mbar_expect_tx(&bars[BAR_C], 32768);
      tma_load_3d(sm + Smem::HS, &tmH, 0, hrow0, 0, &bars[BAR_C]);
      if (VB) {
        mbar_expect_tx(&bars[BAR_W], 16384);
        tma_load_3d(sm + Smem::WT, &tmWG, h * 128, row0, 0, &bars[BAR_W]);
      }
    }
  };

  if (tid == 0 && (int)blockIdx.x < p.total_chunks) issue_loads(blockIdx.x, LOAD_G | LOAD_A);
  auto row_base1 = [&](int chunk) -> size_t {
    const int bn = p.div_h.quot(chunk), h = chunk - bn * H, b = p.div_nt.quot(bn), n = bn - b * NT;
    return ((size_t)b * T + (size_t)n * C) * H + h;
  };
  // beta (and the scalar gate) of a chunk are fetched one chunk ahead, by threads 64..127 at a point of the chunk
  // where they would wait for the tensor core anyway, into the other half of a double buffer
  int buf = 0;
  auto fetch_rows = [&](int chunk, int into) {
    if (tid >= C && tid < 2 * C && chunk < p.total_chunks) {
      const size_t at = row_base1(chunk) + (size_t)(tid - C) * H;
      if (!VB) sBeta2[into * C + tid - C] = p.beta[at];
      if (GATE == GATE_SCALAR) sGs2[into * C + tid - C] = p.g[at];
    }
  };
  fetch_rows(blockIdx.x, 0);
  __syncthreads();  // the rows of the first chunk are in place (later ones are fetched a chunk ahead, before its barriers)

  for (int chunk = blockIdx.x; chunk < p.total_chunks && alive; chunk += gridDim.x) {
    // Work order: head fastest, then chunk, then batch.  CTAs that run at the same time then read the same token rows
    // (the heads of a row are contiguous in memory) and neighbouring state tiles.
    const int bn = p.div_h.quot(chunk), h = chunk - bn * H, b = p.div_nt.quot(bn), n = bn - b * NT;
    const int row0 = b * T + n * C;                       // first token row in [B*T]
    const size_t base128 = ((size_t)row0 * H + h) * 128;
    const size_t base1 = (size_t)row0 * H + h;
    const int hrow0 = ((b * NT + n) * H + h) * 128;        // first row of this chunk's state in [B*NT*H*128]
    const int next_chunk = chunk + gridDim.x;
    uint32_t used = (1u << BAR_A) | (1u << BAR_G);

    const float* sBeta = sBeta2 + buf * C;
    const float* sGs = sGs2 + buf * C;
    // ---- this thread's 32 tokens of its key channel: k and q (packed BF16 pair) and the gate row ------------
    uint32_t kq[HALF];
    uint32_t bgp[VB ? HALF / 2 : 1];  // GDN2: key gate of the thread's tokens, two BF16 per register
    float g[HALF];
    // k, q and g from the tiles TMA brought in while the previous chunk's epilogue ran
    wait(BAR_G, 11);
#pragma unroll
    for (int j = 0; j < HALF; j++) {
      const int t = t0 + j;
      const uint32_t off = swz(t, (kch & 63) >> 3) + (kch & 7) * 2;
      kq[j] = (uint32_t) * reinterpret_cast<const uint16_t*>(sm + Smem::KT + (kch >> 6) * 8192 + off) |
              ((uint32_t) * reinterpret_cast<const uint16_t*>(sm + Smem::QT + (kch >> 6) * 16384 + off) << 16);
      if (VB) {
        const uint32_t bv = *reinterpret_cast<const uint16_t*>(sm + Smem::BT + (kch >> 6) * 16384 + off);
        bgp[j >> 1] = (j & 1) ? (bgp[j >> 1] | (bv << 16)) : bv;
      }
      g[j] = GATE == GATE_VECTOR
                 ? *reinterpret_cast<const float*>(sm + Smem::GT + (kch >> 5) * 8192 + swz(t, (kch & 31) >> 2) + (kch & 3) * 4)
                 : 0.f;
    }
    if (GATE == GATE_VECTOR && wg == NWG - 1) sGl[kch] = g[HALF - 1];
    // (the tiles these values came from are first written again after the barriers below)
    float cen = 0.f;
    bool wide = false;
    if (GATE != GATE_NONE) {
      float lo = INFINITY, hi = -INFINITY;
#pragma unroll
      for (int j = 0; j < HALF; j++) {
        if (GATE == GATE_SCALAR) g[j] = sGs[t0 + j];
        lo = fminf(lo, g[j]);
        hi = fmaxf(hi, g[j]);
      }
      sMinMax[(wg * 2 + 0) * 128 + kch] = lo;
      sMinMax[(wg * 2 + 1) * 128 + kch] = hi;
      __syncthreads();
#pragma unroll
      for (int w2 = 0; w2 < NWG; w2++) {
        lo = fminf(lo, sMinMax[(w2 * 2 + 0) * 128 + kch]);
        hi = fmaxf(hi, sMinMax[(w2 * 2 + 1) * 128 + kch]);
      }
      if (GATE == GATE_VECTOR) {
        cen = 0.5f * (lo + hi);
        wide = !(hi - lo < SPAN_LIMIT);
      } else {
        // A scalar gate is the same for every channel, so its pairwise factor 2^(G_i - G_j), i >= j, is applied to the
        // 64x64 matrices themselves and no operand is scaled by a centred factor.  With a non-increasing cumulative
        // gate (every per-token gate <= 0) that factor is at most 1 whatever the span; only a chunk that both spans
        // 80 log2 units and rises somewhere goes to the pairwise kernel.
        bool rises = t0 > 0 && g[0] > sGs[t0 - 1];
#pragma unroll
        for (int j = 1; j < HALF; j++) rises = rises || g[j] > g[j - 1];
        wide = rises && !(hi - lo < SPAN_LIMIT);
      }
    }
    // the previous chunk's output tiles must have left shared memory before their regions are written again
    if (leader) tma_store_wait_read();
    if (__syncthreads_or(wide ? 1 : 0)) {
      // wide gate span: leave the chunk to the exact pairwise kernel; drain the loads already in flight
      if (tid == 0) {
        wait(BAR_A, 101);
        int idx = atomicAdd(&p.wide_list[0], 1);
        p.wide_list[1 + idx] = (b * H + h) * NT + n;  // the pairwise kernel's chunk numbering: (batch, head) major
      }
      ph ^= used;
      fetch_rows(next_chunk, buf ^ 1);
      buf ^= 1;
      alive = __syncthreads_and(alive ? 1 : 0) != 0;
      if (tid == 0 && alive && next_chunk < p.total_chunks) issue_loads(next_chunk, LOAD_G | LOAD_A);
      continue;
    }
    if (warp == 0) {
      if (leader) issue_loads(chunk, LOAD_BC);
      __syncwarp();
    }
    used |= (1u << BAR_B) | (1u << BAR_C) | (VB ? 1u << BAR_W : 0u);
    // From here on g[] holds the centred factor alpha = 2^(g - c) of each token; zeta = 1 / alpha (vector gate), or
    // gamma = 2^g (scalar gate, c = 0).
    if (GATE != GATE_NONE) {
#pragma unroll
      for (int j = 0; j < HALF; j++) g[j] = ex2(g[j] - cen);
    }
    auto kf = [&](int j) { return __uint_as_float(kq[j] << 16); };          // k of token t0 + j
    auto qf = [&](int j) { return __uint_as_float(kq[j] & 0xFFFF0000u); };  // q of token t0 + j
    auto bgf = [&](int j) {                                                  // key gate of token t0 + j (GDN2)
      return __uint_as_float((j & 1) ? (bgp[VB ? j >> 1 : 0] & 0xFFFF0000u) : (bgp[VB ? j >> 1 : 0] << 16));
    };

    // ---- P = Akk^T (dR_hi + dR_lo) ----------------------------------------------------------------
    if (warp == 0) {
      wait(BAR_A, 1);
      if (alive) {
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
          mma_f16_lo(tb + TM_P, dl(Smem::AKK + ks * 2048, 0), dl(Smem::DRHI + ks * 2048, 8192), ID_P, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
          mma_f16_lo(tb + TM_P, dl(Smem::AKK + ks * 2048, 0), dl(Smem::DRLO + ks * 2048, 8192), ID_P, true);
        mma_commit(&bars[BAR_P]);
        }
      }
      __syncwarp();
    }
    used |= 1u << BAR_P;

    // ---- operand tile Yc^T of the matrix-intra products (row = channel, 16 token columns per thread) ---------
    const float ec = GATE == GATE_NONE ? 1.f : ex2(cen);
#pragma unroll
    for (int t8 = 0; t8 < HALF / 8; t8++) {
      float y[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int jj = t8 * 8 + j;
        y[j] = kf(jj) * (GATE == GATE_VECTOR ? rcp(g[jj]) : 1.f);
      }
      const int ch = wg * (HALF / 8) + t8;
      uint4 hi, lo;
      split8(y, hi, lo);
      tmem_st4(tlane + TM_Y + ch * 4, hi);
      if (GATE == GATE_VECTOR) tmem_st4(tlane + TM_Y + 32 + ch * 4, lo);
    }
    tmem_st_wait();

    // ---- after P: dh takes the place of the dR tiles; P epilogue (rows 0..63 live in TMEM lanes 0..63) ---------
    wait(BAR_P, 2);
    tc_fence_after_sync();
    if (VB) wait(BAR_W, 15);
    if (warp == 0 && alive) {
      if (leader) {
        mbar_expect_tx(&bars[BAR_D], 32768);
        tma_load_3d(sm + Smem::DHT, &tmDH, 0, hrow0, 0, &bars[BAR_D]);
      }
      __syncwarp();
    }
    used |= 1u << BAR_D;
    // The A operand's two 64-row panels are the same tile (leading offset 0), so TMEM lanes 64..127 repeat rows
    // 0..63 and all sixteen warps take part: thread = (token i, 16 value columns).
    if (alive) {
      const int i = kch & 63, hs = kch >> 6;  // row (token) 0..63; value columns 32*wg + 16*hs ..
      const size_t go = base128 + (size_t)i * ldt;
      const float beta_i = sBeta[i];
      float dbv = 0.f;
      {
        float x[16];
        const int v0 = 32 * wg + 16 * hs;  // value column
        const int vp = v0 >> 6, vc = (v0 & 63) >> 3;  // 64-wide panel, 16-byte chunk inside its rows
        tmem_ld16(tlane + TM_P + v0, x);
        tmem_ld_wait();
        uint4 vraw[2] = {*reinterpret_cast<const uint4*>(sm + Smem::VT + vp * 8192 + swz(i, vc)),
                         *reinterpret_cast<const uint4*>(sm + Smem::VT + vp * 8192 + swz(i, vc + 1))};
        const uint32_t* vu = reinterpret_cast<const uint32_t*>(vraw);
        uint32_t dvp[8], pp[8];
        float dwv[16];
        uint4 wraw[2];
        if (VB) {
          wraw[0] = *reinterpret_cast<const uint4*>(sm + Smem::WT + vp * 8192 + swz(i, vc));
          wraw[1] = *reinterpret_cast<const uint4*>(sm + Smem::WT + vp * 8192 + swz(i, vc + 1));
        }
        const uint32_t* wu = reinterpret_cast<const uint32_t*>(wraw);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float2 vv = unpack_bf16(vu[j]);
          float w0 = beta_i, w1 = beta_i;
          if (VB) {
            float2 ww = unpack_bf16(wu[j]);
            w0 = ww.x; w1 = ww.y;
            dwv[2 * j] = vv.x * x[2 * j];
            dwv[2 * j + 1] = vv.y * x[2 * j + 1];
          } else {
            dbv += vv.x * x[2 * j] + vv.y * x[2 * j + 1];
          }
          dvp[j] = pack_bf16(w0 * x[2 * j], w1 * x[2 * j + 1]);
          pp[j] = pack_bf16(x[2 * j], x[2 * j + 1]);
        }
        // dv tile (same panel layout as the v tile) in the dead k tile; it leaves by one bulk store after the barrier
        *reinterpret_cast<uint4*>(sm + Smem::DVT + vp * 8192 + swz(i, vc)) = make_uint4(dvp[0], dvp[1], dvp[2], dvp[3]);
        *reinterpret_cast<uint4*>(sm + Smem::DVT + vp * 8192 + swz(i, vc + 1)) = make_uint4(dvp[4], dvp[5], dvp[6], dvp[7]);
        if (VB) {
          if (OUTF32) {
            float* o = reinterpret_cast<float*>(p.dwg) + go + v0;
#pragma unroll
            for (int j = 0; j < 4; j++)
              *reinterpret_cast<float4*>(o + 4 * j) = make_float4(dwv[4 * j], dwv[4 * j + 1], dwv[4 * j + 2], dwv[4 * j + 3]);
          } else {
            uint32_t dwp[8];
#pragma unroll
            for (int j = 0; j < 8; j++) dwp[j] = pack_bf16(dwv[2 * j], dwv[2 * j + 1]);
            // tile in the parking area (free until pass A); it leaves with the dv tile
            *reinterpret_cast<uint4*>(sm + Smem::DWT + vp * 8192 + swz(i, vc)) = make_uint4(dwp[0], dwp[1], dwp[2], dwp[3]);
            *reinterpret_cast<uint4*>(sm + Smem::DWT + vp * 8192 + swz(i, vc + 1)) = make_uint4(dwp[4], dwp[5], dwp[6], dwp[7]);
          }
        }
        const uint32_t ptile = Smem::DOP + vp * 16384 + 8192;
        *reinterpret_cast<uint4*>(sm + ptile + swz(i, vc)) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
        *reinterpret_cast<uint4*>(sm + ptile + swz(i, vc + 1)) = make_uint4(pp[4], pp[5], pp[6], pp[7]);
      }
      if (!VB) sDbP[(wg * 2 + hs) * 64 + i] = dbv;
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    // ---- [dAqk/scale ; -dAkk] = [dO ; P] R^T ---------------------------------------------------------
    if (warp == 0) {
      wait(BAR_B, 3);
      if (alive) {
        tc_fence_after_sync();
        if (leader) {
          tma_store_3d(&tmDV, sm + Smem::DVT, h * 128, row0, 0);
          if (VB && !OUTF32) tma_store_3d(&tmDW, sm + Smem::DWT, h * 128, row0, 0);
          tma_store_commit();
          mma_kmajor<8>(tb + TM_HD, dl(Smem::DOP, 16), 16384, dl(Smem::R, 16), 8192, ID_KK, false);
          // the dv tile sits where the epilogue of this product writes: everyone waits for this commit first, and
          // it is only issued once the store has read the tile
          tma_store_wait_read();
          mma_commit(&bars[BAR_HD]);
        }
      }
      __syncwarp();
    }
    used |= 1u << BAR_HD;
    // Ec^T tiles while the stacked product runs (first needed by the last product group)
#pragma unroll
    for (int t8 = 0; t8 < HALF / 8; t8++) {
      float e[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int jj = t8 * 8 + j;
        const float bb = VB ? bgf(jj) : sBeta[t0 + jj];
        e[j] = bb * kf(jj) * (GATE == GATE_VECTOR ? g[jj] : 1.f);
      }
      uint4 hi, lo;
      split8(e, hi, lo);
      tmem_st4(tlane + TM_E + (wg * (HALF / 8) + t8) * 4, hi);
      tmem_st4(tlane + TM_E + 32 + (wg * (HALF / 8) + t8) * 4, lo);
    }
    tmem_st_wait();
    // this thread's 32 values of its channel's h row, kept for the chunk-end gate term (the h tile is gone by
    // the time dh arrives)
    uint4 hrow[4];
    if (GATE != GATE_NONE) {
      wait(BAR_C, 6);
#pragma unroll
      for (int ch = 0; ch < 4; ch++)
        hrow[ch] = *reinterpret_cast<const uint4*>(sm + Smem::HS + (wg >> 1) * 16384 + swz(kch, (wg & 1) * 4 + ch));
    } else if (tid == 0) {
      wait(BAR_C, 6);
    }
    wait(BAR_HD, 4);
    tc_fence_after_sync();
    if (alive) {
      const int i = kch & 63;
      const bool lower_incl = kch < C;  // lanes 0..63: dAqk (diagonal kept); lanes 64..127: dAkk (strictly lower)
      const float mul = lower_incl ? scale : -1.f;
      const uint32_t thi = lower_incl ? Smem::HHI : Smem::DHI, tlo = lower_incl ? Smem::HLO : Smem::DLO;
      {
        float x[16];
        const int col0 = 16 * wg;
        tmem_ld16(tlane + TM_HD + col0, x);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; half++) {
          float y[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int col = col0 + 8 * half + j;
            const bool keep = lower_incl ? (col <= i) : (col < i);
            float f = mul;
            if (GATE == GATE_SCALAR) f *= ex2(fminf(sGs[i] - sGs[col], 126.f));  // pairwise gate factor (kept entries: i >= col)
            y[j] = keep ? f * x[8 * half + j] : 0.f;
          }
          uint4 hi, lo;
          split8(y, hi, lo);
          *reinterpret_cast<uint4*>(sm + thi + swz(i, (col0 >> 3) + half)) = hi;
          *reinterpret_cast<uint4*>(sm + tlo + swz(i, (col0 >> 3) + half)) = lo;
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    // ---- second product group: [X1|X3], [X2|X4] and the Ec part of X6 ----------------------------------------
    if (warp == 0 && alive) {
      tc_fence_after_sync();
      if (leader) {
        // [X1 | X3] = h [dO ; P]^T as one N=128 product (the sign of X3 is applied in the epilogue)
        mma_kmajor<8>(tb + TM_X1, dl(Smem::HS, 16), 16384, dl(Smem::DOP, 16), 16384, ID_KK128, false);
        // [X2 | X4] = Yc^T [dAqk ; dAkk]^T, hi/lo split in three passes, Yc^T from tensor memory
        mma_ts4(tb + TM_X2, tb + TM_Y, dl(Smem::HHI, 16), 32, ID_KK128, false);
        if (GATE == GATE_VECTOR)  // without a vector gate Yc = k is exact in BF16: its lo part is zero
          mma_ts4(tb + TM_X2, tb + TM_Y + 32, dl(Smem::HHI, 16), 32, ID_KK128, true);
        mma_ts4(tb + TM_X2, tb + TM_Y, dl(Smem::HLO, 16), 32, ID_KK128, true);
        mma_commit(&bars[BAR_Q]);  // X1 and X2 complete: dq can be finished while the rest still runs
      }
      __syncwarp();
    }
    if (warp == 1 && alive) {
      tc_fence_after_sync();
      if (leader2) {
        // X6, Ec part, from the second issuer at the same time: B stored [reduction row i][n = j contiguous] = MN-major
        mma_ts4(tb + TM_X6, tb + TM_E, dl(Smem::DHI, 8192), 2048, ID_KMN, false);
        mma_ts4(tb + TM_X6, tb + TM_E + 32, dl(Smem::DHI, 8192), 2048, ID_KMN, true);
        mma_ts4(tb + TM_X6, tb + TM_E, dl(Smem::DLO, 8192), 2048, ID_KMN, true);
      }
      __syncwarp();
    }
    used |= (1u << BAR_C3) | (1u << BAR_Q) | (1u << BAR_QR);
    // Qc^T into the columns the stacked product has left
#pragma unroll
    for (int t8 = 0; t8 < HALF / 8; t8++) {
      float x[8];
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const int jj = t8 * 8 + j;
        x[j] = qf(jj) * (GATE == GATE_VECTOR ? g[jj] : 1.f);
      }
      uint4 hi, lo;
      split8(x, hi, lo);
      tmem_st4(tlane + TM_QC + (wg * (HALF / 8) + t8) * 4, hi);
      if (GATE == GATE_VECTOR) tmem_st4(tlane + TM_QC + 32 + (wg * (HALF / 8) + t8) * 4, lo);
    }
    tmem_st_wait();
    tc_fence_before_sync();
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars[BAR_QR]);  // this warp's part of Qc^T is complete in tensor memory
    wait(BAR_D, 8);
    // chunk-end gate term, part 1: sum_v h[k,v] dh[k,v] over this thread's 32 value columns (h from registers,
    // dh from the tile that just landed)
    float hd = 0.f;  // written to the scratch columns once every product is complete
    if (GATE != GATE_NONE && alive) {
#pragma unroll
      for (int ch = 0; ch < 4; ch++) {
        uint4 d = *reinterpret_cast<const uint4*>(sm + Smem::DHT + (wg >> 1) * 16384 + swz(kch, (wg & 1) * 4 + ch));
        const uint32_t* au = reinterpret_cast<const uint32_t*>(&hrow[ch]);
        const uint32_t* du = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float2 x = unpack_bf16(au[j]), y = unpack_bf16(du[j]);
          hd += x.x * y.x + x.y * y.y;
        }
      }
    }
    if (warp == 1) {
      wait(BAR_QR, 13);  // Qc^T complete (all sixteen warps), and the leader has issued everything before it
      if (alive) {
        tc_fence_after_sync();
        if (leader2) {
          // X5 = dh R^T into the columns Yc^T leaves: the leader issued [X2 | X4] before its warp arrived on BAR_QR, so
          // this runs after it
          mma_kmajor<8>(tb + TM_X5, dl(Smem::DHT, 16), 16384, dl(Smem::R, 16), 8192, ID_KK, false);
          mma_ts4(tb + TM_X6, tb + TM_QC, dl(Smem::HHI, 8192), 2048, ID_KMN, true);
          if (GATE == GATE_VECTOR)  // likewise Qc = q
            mma_ts4(tb + TM_X6, tb + TM_QC + 32, dl(Smem::HHI, 8192), 2048, ID_KMN, true);
          mma_ts4(tb + TM_X6, tb + TM_QC, dl(Smem::HLO, 8192), 2048, ID_KMN, true);
          mma_commit(&bars[BAR_C3]);
        }
      }
      __syncwarp();
    }

    // ---- epilogue, thread = (key channel, token quarter) ------------------------------------------------------
    // Factored forms: dq = al*(ec*s*x1 + x2), gamma*eb = al*(ec*x3 + x4), yb/gamma = ze*(x6 + en*x5).
    // Every token quarter lacks the totals of the tokens after it: partial reverse sums are parked in the (dead) Yc
    // tiles and the carry (plus the chunk-end term) is added after the barrier.
    const float gl = GATE == GATE_VECTOR ? sGl[kch] : (GATE == GATE_SCALAR ? sGs[C - 1] : 0.f);
    const float en = GATE == GATE_NONE ? 1.f : ex2(gl - cen);  // exp2(g_last - g) = zeta * en
    float* sPark = reinterpret_cast<float*>(sm + Smem::PARK);  // [64 tokens][128 channels]
    const size_t go0 = base128 + (size_t)t0 * ldt + kch;
    fetch_rows(next_chunk, buf ^ 1);
    // pass A (needs X1, X2 only): dq, and q*dq parked for the gate row
    wait(BAR_Q, 12);
    tc_fence_after_sync();
    if (alive) {
      const float ecs = ec * scale;
      float x1[16], x2[16];
      tmem_ld16(tlane + TM_X1 + t0, x1);
      tmem_ld16(tlane + TM_X2 + t0, x2);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < HALF; j++) {
        const size_t go = go0 + (size_t)j * ldt;
        const float al = GATE == GATE_NONE ? 1.f : g[j];
        const float dq = GATE == GATE_SCALAR ? fmaf(al * ecs, x1[j], x2[j]) : al * fmaf(ecs, x1[j], x2[j]);
        if (OUTF32)
          reinterpret_cast<float*>(p.dq)[go] = dq;
        else
          *reinterpret_cast<bf16*>(sm + Smem::DQT + (t0 + j) * 256 + kch * 2) = f2bf(dq);
        if (GATE != GATE_NONE) sPark[(t0 + j) * 128 + kch] = qf(j) * dq;
      }
    }
    wait(BAR_C3, 10);
    tc_fence_after_sync();
    if (GATE != GATE_NONE && alive) tmem_st1(tlane + TM_SCR + wg, hd);
    // every tile of this chunk has been consumed by the tensor core and (barrier above) by the threads: start the
    // next chunk's loads under the rest of the epilogue
    if (warp == 0 && alive && next_chunk < p.total_chunks) {
      if (leader) issue_loads(next_chunk, LOAD_G);
      __syncwarp();
    }
    // pass B: dk, db, gate rows in reverse token order
    float run = 0.f;
    const float nec = -ec;
    if (alive) {
      float colsum = 0.f;  // chunk-end term, part 2: sum_t k * exp2(g_last-g) * (R dh^T) over this thread's tokens
#pragma unroll
      for (int c8 = HALF / 8 - 1; c8 >= 0; c8--) {
        float x3[8], x4[8], x5[8], x6[8];
        const int col = t0 + 8 * c8;
        tmem_ld8(tlane + TM_X3 + col, x3);
        tmem_ld8(tlane + TM_X4 + col, x4);
        tmem_ld8(tlane + TM_X5 + col, x5);
        tmem_ld8(tlane + TM_X6 + col, x6);
        tmem_ld_wait();
        float dbp[8], dgp[8];
#pragma unroll
        for (int j = 7; j >= 0; j--) {
          const int jj = 8 * c8 + j, t = t0 + jj;
          const size_t go = go0 + (size_t)jj * ldt;
          float al = 1.f, ze = 1.f;
          if (GATE != GATE_NONE) {
            al = g[jj];
            if (GATE == GATE_VECTOR) ze = rcp(al);
          }
          const float kk = kf(jj);
          const float bb = VB ? bgf(jj) : sBeta[t];
          float e, y, tail_f;  // gamma * eb (x3 = +h P^T), yb / gamma, 2^(g_last - g)
          if (GATE == GATE_SCALAR) {
            tail_f = ex2(gl - sGs[t]);
            e = fmaf(al * nec, x3[j], x4[j]);
            y = fmaf(tail_f, x5[j], x6[j]);
          } else {
            tail_f = ze * en;
            e = al * fmaf(nec, x3[j], x4[j]);
            y = ze * fmaf(en, x5[j], x6[j]);
          }
          const float be = bb * e;
          if (OUTF32) {
            reinterpret_cast<float*>(p.dk)[go] = be + y;
            if (VB) reinterpret_cast<float*>(p.dbg)[go] = kk * e;
          } else {
            *reinterpret_cast<bf16*>(sm + Smem::DKT + t * 256 + kch * 2) = f2bf(be + y);
            if (VB) *reinterpret_cast<bf16*>(sm + Smem::DBT + t * 256 + kch * 2) = f2bf(kk * e);
          }
          if (!VB) dbp[j] = kk * e;
          if (GATE != GATE_NONE) {
            colsum = fmaf(kk * tail_f, x5[j], colsum);
            const float row = fmaf(kk, be - y, sPark[t * 128 + kch]);
            if (GATE == GATE_VECTOR) {
              run += row;
              sPark[t * 128 + kch] = run;
            } else {
              dgp[j] = row;
            }
          }
        }
        if (!VB) {
          float s = warp_sum8(dbp, lane);
          if (lane < 8) sDbW[warp * 16 + 8 * c8 + lane] = s;
        }
        if (GATE == GATE_SCALAR) {
          float s = warp_sum8(dgp, lane);
          if (lane < 8) sDgW[warp * 16 + 8 * c8 + lane] = s;
        }
      }
      if (GATE != GATE_NONE) tmem_st1(tlane + TM_SCR + 4 + wg, colsum);
      if (GATE == GATE_VECTOR) tmem_st1(tlane + TM_SCR + 8 + wg, run);
      if (GATE != GATE_NONE) tmem_st_wait();
    }
    if (warp == 0 && alive && next_chunk < p.total_chunks) {
      if (leader) issue_loads(next_chunk, LOAD_A);
      __syncwarp();
    }
    if (!OUTF32) fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (!OUTF32 && leader && alive) {
      tma_store_2d(&tmDQ, sm + Smem::DQT, h * 128, row0);
      tma_store_2d(&tmDK, sm + Smem::DKT, h * 128, row0);
      if (VB) tma_store_2d(&tmDBG, sm + Smem::DBT, h * 128, row0);
      tma_store_commit();
    }
    if (alive) {
      // chunk-end term of this channel: lambda * sum_v h dh + sum_t k 2^(g_last - g) (R dh^T)
      float endk = 0.f;
      float scr[16];
      if (GATE != GATE_NONE) {
        tmem_ld16(tlane + TM_SCR, scr);
        tmem_ld_wait();
        endk = ex2(gl) * (scr[0] + scr[1] + scr[2] + scr[3]) + (scr[4] + scr[5] + scr[6] + scr[7]);
      }
      if (GATE == GATE_VECTOR) {
        float carry = endk;  // the chunk-end term sits on token 63: part of every carry
#pragma unroll
        for (int w2 = 1; w2 < NWG; w2++) carry += w2 > wg ? scr[8 + w2] : 0.f;
        // the finished [64 tokens][128 channels] tile leaves as one bulk store after the barrier below
#pragma unroll
        for (int jj = 0; jj < HALF; jj++) sPark[(t0 + jj) * 128 + kch] += carry;
        fence_async_smem();
      }
      if (!VB && tid < C) {
        float db = 0.f;
#pragma unroll
        for (int m = 0; m < 8; m++) db += sDbP[m * 64 + tid];
#pragma unroll
        for (int m = 0; m < 4; m++) db += sDbW[((tid >> 4) * 4 + m) * 16 + (tid & 15)];
        p.dbeta[base1 + (size_t)tid * H] = db;
      }
      if (GATE == GATE_SCALAR) {
        if (tid < C) {
          float dgt = 0.f;
#pragma unroll
          for (int m = 0; m < 4; m++) dgt += sDgW[((tid >> 4) * 4 + m) * 16 + (tid & 15)];
          sDgs[tid] = dgt;
        }
        if (wg == 0) {
          // scalar gate: the chunk-end term of every channel lands on the last token's sum
          float se = endk;
#pragma unroll
          for (int m = 16; m > 0; m >>= 1) se += __shfl_xor_sync(0xffffffffu, se, m);
          if (lane == 0) sDb[warp] = se;  // sDb is free for the scalar families' four partial sums
        }
      }
    }
    if (GATE == GATE_SCALAR) {
      __syncthreads();
      if (warp == 0 && alive) {
        // reverse cumulative sum over the 64 tokens by one warp: lane l owns tokens 2l and 2l+1
        const float v0 = sDgs[2 * lane], v1 = sDgs[2 * lane + 1];
        float acc = v0 + v1;  // becomes the sum over this lane and every lane above it
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float up = __shfl_down_sync(0xffffffffu, acc, d);
          if (lane + d < 32) acc += up;
        }
        const float end = sDb[0] + sDb[1] + sDb[2] + sDb[3];  // the chunk-end term sits on the last token
        const float r1 = end + (acc - v0);                    // tokens 2l+1 .. 63
        p.dg[base1 + (size_t)(2 * lane + 1) * H] = r1;
        p.dg[base1 + (size_t)(2 * lane) * H] = r1 + v0;
      }
    }
    ph ^= used;
    buf ^= 1;
    alive = __syncthreads_and(alive ? 1 : 0) != 0;
    if (GATE == GATE_VECTOR && leader && alive) {
      tma_store_2d(&tmDG, sPark, h * 128, row0);
      tma_store_commit();
    }
  }

  if (leader) tma_store_wait_read();  // shared memory stays valid until the last store has read it
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 512);
}

constexpr size_t TC_SMEM = Smem::TOTAL + 1024;

// mul = ceil(2^(31 + ceil(log2 d)) / d), shift = ceil(log2 d) - 1: exact for every dividend below 2^31.
FastDiv make_fastdiv(int d) {
  FastDiv f;
  f.div = (uint32_t)d;
  int lg = 0;
  while ((1ll << lg) < d) lg++;
  const int pw = 31 + lg;
  f.mul = (uint32_t)(((1ull << pw) + (uint64_t)d - 1) / (uint64_t)d);
  f.shift = (uint32_t)(pw - 32);
  return f;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 148;
  }
  return n;
}

template <int GATE, bool VB, bool OUTF32>
cudaError_t run1(const CUtensorMap* tm, const TcParams& p, cudaStream_t st) {
  auto kern = chunk_adjoint_tc_kernel<GATE, VB, OUTF32>;
  cudaError_t e = ensure_dynamic_smem<chunk_adjoint_tc_kernel<GATE, VB, OUTF32>>(TC_SMEM);
  if (e != cudaSuccess) return e;
  const int grid = p.total_chunks < sm_count() ? p.total_chunks : sm_count();
  kern<<<grid, TPB, TC_SMEM, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[6], tm[7], tm[8], tm[9], tm[10], tm[11], tm[12], tm[13], tm[14], tm[15], tm[16], tm[17], tm[18], p);
  count_launch();
  return cudaGetLastError();
}

template <int GATE, bool VB>
cudaError_t run(const CUtensorMap* tm, const TcParams& p, cudaStream_t st) {
  return p.out_f32 ? run1<GATE, VB, true>(tm, p, st) : run1<GATE, VB, false>(tm, p, st);
}

}  // namespace

// Encodes the 19 tensor maps of the chunk kernel (tile loads of every operand, tile stores of the gradients).
bool encode_chunk_maps(CUtensorMap* tm, const RewyBwdArgs& a, const RewyStageBuffers& s, uint64_t rows, uint64_t srows) {
  const int H = a.H;
  bool ok = encode_tmap_2d(&tm[0], a.Akk, 2, (uint64_t)H * 64, rows, (uint64_t)H * 128, 64, 64) &&
            encode_tmap_panels(&tm[1], s.dR, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2) &&
            encode_tmap_panels(&tm[2], s.dR_lo, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2) &&
            encode_tmap_2d(&tm[3], a.d_o, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_panels(&tm[4], s.v_new, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2) &&
            encode_tmap_panels(&tm[5], s.h, 2, 128, srows, 256, 128, 2) &&
            encode_tmap_panels(&tm[6], s.dh, 2, 128, srows, 256, 128, 2) &&
            encode_tmap_panels(&tm[7], a.v, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2) &&
            encode_tmap_panels(&tm[8], a.k, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2) &&
            encode_tmap_2d(&tm[11], a.q, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_panels(&tm[12], a.dv, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2);
  if (ok && gate_mode_of(a.family) == GATE_VECTOR)
    ok = encode_tmap_panels(&tm[9], a.g, 4, (uint64_t)H * 128, rows, (uint64_t)H * 512, 64, 4) &&
         encode_tmap_2d(&tm[10], a.dg, 4, (uint64_t)H * 128, rows, (uint64_t)H * 512, 128, 64, false);
  else
    tm[9] = tm[10] = tm[8];  // never dereferenced without a vector gate
  if (ok && a.out_dtype != REWY_OUT_F32)
    ok = encode_tmap_2d(&tm[13], a.dq, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 128, 64, false) &&
         encode_tmap_2d(&tm[14], a.dk, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 128, 64, false);
  else
    tm[13] = tm[14] = tm[8];  // FP32 dq / dk are stored directly
  tm[15] = tm[16] = tm[17] = tm[18] = tm[8];
  if (ok && a.family == REWY_GDN2) {
    ok = encode_tmap_2d(&tm[15], a.b_gate, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
         encode_tmap_panels(&tm[17], a.w_gate, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2);
    if (ok && a.out_dtype != REWY_OUT_F32)
      ok = encode_tmap_2d(&tm[16], a.db_gate, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 128, 64, false) &&
           encode_tmap_panels(&tm[18], a.dw_gate, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 2);
  }
  return ok;
}

// ctrl: device int[2 + total_chunks]: [0] status word (zeroed by the caller), [1] number of wide-span chunks,
// [2..] their indices.
cudaError_t launch_chunk_adjoint_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* ctrl, cudaStream_t st) {
  const int B = a.B, T = a.T, H = a.H, NT = T / C;
  const uint64_t rows = (uint64_t)B * T, srows = (uint64_t)B * NT * H * 128;
  struct Key {
    const void* ptr[20];
    int B, T, H, family, out_dtype;
  } key;
  memset(&key, 0, sizeof(key));
  const void* ptrs[20] = {a.Akk, s.dR, s.dR_lo, a.d_o, s.v_new, s.h, s.dh, a.v, a.k, a.g, a.dg, a.q, a.dv, a.dq, a.dk,
                          a.b_gate, a.db_gate, a.w_gate, a.dw_gate, nullptr};
  memcpy(key.ptr, ptrs, sizeof(ptrs));
  key.B = B; key.T = T; key.H = H; key.family = a.family; key.out_dtype = a.out_dtype;
  thread_local TmapCache<19, sizeof(Key)> cache;
  const CUtensorMap* tm = cache.find(&key);
  if (tm == nullptr) {
    CUtensorMap* w = cache.slot();
    if (!encode_chunk_maps(w, a, s, rows, srows)) return cudaErrorInvalidValue;
    cache.commit(&key);
    tm = w;
  }
  cudaError_t e = cudaMemsetAsync(ctrl + 1, 0, sizeof(int), st);  // wide-chunk count; the status word is kept
  if (e != cudaSuccess) return e;
  TcParams p;
  p.q = (const bf16*)a.q; p.k = (const bf16*)a.k; p.v = (const bf16*)a.v; p.bg = (const bf16*)a.b_gate;
  p.wg = (const bf16*)a.w_gate; p.dh = (const bf16*)s.dh; p.g = a.g; p.beta = a.beta;
  p.dq = a.dq; p.dk = a.dk; p.dbg = a.db_gate; p.dwg = a.dw_gate; p.dv = (bf16*)a.dv; p.dg = a.dg; p.dbeta = a.dbeta;
  p.wide_list = ctrl + 1; p.err = ctrl;
  p.T = T; p.H = H; p.NT = NT; p.total_chunks = B * H * NT; p.out_f32 = a.out_dtype == REWY_OUT_F32;
  p.scale = a.scale;
  p.div_nt = make_fastdiv(NT);
  p.div_h = make_fastdiv(H);
  switch (a.family) {
    case REWY_DELTA: e = run<GATE_NONE, false>(tm, p, st); break;
    case REWY_GDN: e = run<GATE_SCALAR, false>(tm, p, st); break;
    case REWY_KDA: e = run<GATE_VECTOR, false>(tm, p, st); break;
    default: e = run<GATE_VECTOR, true>(tm, p, st); break;
  }
  if (e != cudaSuccess) return e;
  // chunks with a wide gate span: exact pairwise path of the warp-MMA kernel, driven by the list
  return launch_chunk_adjoint_warp(a, s, ctrl + 1, st);
}

}  // namespace rewy

// ---------------------------------------------------------------------------------------------------
// Chunk stage without any caller-provided or allocated scratch.
//
// The chunk stage needs a small control block in global memory (status word, count and list of the chunks
// that go to the pairwise path).  Hosts that drive this library from a fixed, pre-assigned device arena - a
// C or C++ trainer that carved all of its memory up front, or a process whose memory budget forbids any
// further device allocation - have no allocator to take that block from.  For them the block lives in the
// library image itself: one array per device, sized for REWY_STATIC_MAX_CHUNKS chunks.
namespace rewy {
namespace {

constexpr int STATIC_MAX_CHUNKS = 65536;  // B*H*(T/64) the static control block can describe
static __device__ __align__(256) int g_static_ctrl[2 + STATIC_MAX_CHUNKS];

constexpr int MAX_DEVICES = 64;
int* g_static_ctrl_ptr[MAX_DEVICES] = {};  // device address of g_static_ctrl on each device, once resolved

// Resolve the device address of the array for the current device.  The array's name is only a host-side handle;
// kernels must be given the address cudaGetSymbolAddress returns for the device that is current.
int* static_ctrl_for_current_device(char* why, size_t why_len) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    snprintf(why, why_len, "cannot identify the current device: %s", cudaGetErrorString(e));
    return nullptr;
  }
  int* ptr = __atomic_load_n(&g_static_ctrl_ptr[dev], __ATOMIC_ACQUIRE);
  if (ptr != nullptr) return ptr;
  void* addr = nullptr;
  e = cudaGetSymbolAddress(&addr, g_static_ctrl);
  if (e != cudaSuccess || addr == nullptr) {
    snprintf(why, why_len, "cudaGetSymbolAddress(static control block) failed on device %d: %s", dev, cudaGetErrorString(e));
    return nullptr;
  }
  __atomic_store_n(&g_static_ctrl_ptr[dev], static_cast<int*>(addr), __ATOMIC_RELEASE);
  return static_cast<int*>(addr);
}

}  // namespace
}  // namespace rewy

extern "C" int rewy_stage_chunk_adjoint_static(const RewyBwdArgs* a, const RewyStageBuffers* s, rewy_stream_t stream) {
  using namespace rewy;
  char why[256];
  // the size limit of the built-in block first (it needs no pointer), then exactly the host-side checks of
  // rewy_stage_chunk_adjoint (shape envelope, every pointer present and 16-byte aligned) minus RewyStageBuffers.ctrl
  if (a != nullptr && a->B > 0 && a->H > 0 && a->T >= C) {
    const long long chunks = (long long)a->B * a->H * (a->T / C);
    if (chunks > STATIC_MAX_CHUNKS) {
      snprintf(why, sizeof(why),
               "rewy_stage_chunk_adjoint_static handles at most %d chunks (B*H*T/64); this call has %lld - use "
               "rewy_stage_chunk_adjoint with a caller-provided control block",
               STATIC_MAX_CHUNKS, chunks);
      return report_error(REWY_ERR_SHAPE, why);
    }
  }
  const int rc = validate_chunk_stage(a, s, false);
  if (rc != REWY_OK) return rc;
  int* ctrl = static_ctrl_for_current_device(why, sizeof(why));
  if (ctrl == nullptr) return report_error(REWY_ERR_LAUNCH, why);
  cudaStream_t st = (cudaStream_t)stream;
  // The block keeps whatever the previous call left in it: the status word and the count must start at zero
  // (the list entries beyond the count are never read).
  cudaError_t e = cudaMemsetAsync(ctrl, 0, 2 * sizeof(int), st);
  if (e == cudaSuccess) e = launch_chunk_adjoint_tc(*a, *s, ctrl, st);
  if (e != cudaSuccess) {
    snprintf(why, sizeof(why), "chunk adjoint (static control block): %s", cudaGetErrorString(e));
    return report_error(REWY_ERR_LAUNCH, why);
  }
  return REWY_OK;
}

extern "C" int rewy_static_device_status(rewy_stream_t stream) {
  using namespace rewy;
  char why[256];
  int* ctrl = static_ctrl_for_current_device(why, sizeof(why));
  if (ctrl == nullptr) return report_error(REWY_ERR_LAUNCH, why);
  int word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, ctrl, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return report_error(REWY_ERR_LAUNCH, cudaGetErrorString(e));
  if (word != 0) return report_error(REWY_ERR_DEVICE, "a kernel gave up on a bounded wait (static control block)");
  return REWY_OK;
}
