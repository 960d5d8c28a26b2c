// Reverse cross-chunk state-gradient scan on the Blackwell tensor cores.
//
// Same recurrence as bwd_scan_kernel in state_scan.cu (the reference functions it replaces are listed there):
//   dh[n] stored;  dR = kg dh[n] + Aqk^T dO;  dh <- lam*dh + scale*qg^T dO - w^T dR;  dh0
// One CTA owns one (batch, head) for the whole sequence.  The 128x128 FP32 state lives in TMEM for all T/64
// chunks, stored as S' = dh/scale so that the scale never has to be folded into a tensor-core operand:
//   per chunk   thread (key channel, value half) reads its S' row, writes dh = scale*S' as BF16 hi/lo tiles
//               (hi also goes to global dh[n] by a TMA store), writes lam*S' back to TMEM;
//   MMA 1       dR^T[v,i] = sum_k dh[k,v] kg[i,k] (hi and lo) + sum_j dO[j,v] Aqk[j,i]        M=128 N=64
//   epilogue    thread (value channel, token half) stores dR as BF16 hi/lo to global and (dR/scale) hi/lo tiles
//   MMA 2       S'[k,v] += sum_i qg[i,k] dO[i,v] - sum_i w[i,k] (dR/scale)[i,v]                 M=128 N=128
// Every operand that comes from global memory is used exactly as TMA lands it (MN-major or K-major).
#include "tc05.cuh"

namespace rewy {
namespace {
using namespace tc;

struct ScanParams {
  const float *g, *dht;
  bf16 *dR, *dRlo;
  float* dh0;
  int* err;
  int T, H, NT;
  int svf;  // initial / final state tensors (dht, dh0) are stored value-first: [B,H,V,K]
  const int* cu;  // packed sequences: device int32 [sequences + 1] token offsets (multiples of 64), or nullptr
  float scale;
};

// Shared-memory plan, byte offsets from a 1024-byte aligned base.  The 64 KB region X is time-shared inside a chunk:
// first the dh hi/lo tiles (operands of the dR product), then - once that product is done - qg, w and the
// (dR/scale) hi/lo tiles (operands of the state update).  That keeps a CTA at 105 KB so two CTAs share an SM and
// hide each other's waits.
struct SS {
  static constexpr uint32_t KG = 0;               // [64 i][128 k] two panels              16 KB
  static constexpr uint32_t DO0 = KG + 16384;     // [64 i][128 v]                         16 KB
  static constexpr uint32_t AQK = DO0 + 16384;    // [64 j][64 i]                          8 KB
  static constexpr uint32_t DHHI = AQK + 8192;    // X: [128 k][128 v] two panels          32 KB
  static constexpr uint32_t DHLO = DHHI + 32768;  // X:                                    32 KB
  static constexpr uint32_t QG = DHHI;            // X: [64 i][128 k]                      16 KB
  static constexpr uint32_t W = DHHI + 16384;     // X: [64 i][128 k]                      16 KB
  static constexpr uint32_t DRHI = DHLO;          // X: (dR/scale)^T [128 v][64 i]         16 KB
  static constexpr uint32_t DRLO = DHLO + 16384;  // X:                                    16 KB
  static constexpr uint32_t BARS = DHLO + 32768;  // 8 mbarriers
  static constexpr uint32_t TMEM = BARS + 64;
  static constexpr uint32_t TOTAL = TMEM + 64;
};
static_assert(2 * (SS::TOTAL + 2048) <= 233472, "two reverse-scan CTAs must fit one SM");

enum { B_L1 = 0, B_DO, B_L2, B_DR, B_S };
constexpr uint32_t TM_S = 0, TM_DR = 128;
constexpr int TPB = 256;

__device__ __forceinline__ void tmem_ld16f(uint32_t taddr, float (&r)[16]) {
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
__device__ __forceinline__ void tmem_st16f(uint32_t taddr, const float (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(__float_as_uint(r[0])), "r"(__float_as_uint(r[1])), "r"(__float_as_uint(r[2])), "r"(__float_as_uint(r[3])),
      "r"(__float_as_uint(r[4])), "r"(__float_as_uint(r[5])), "r"(__float_as_uint(r[6])), "r"(__float_as_uint(r[7])),
      "r"(__float_as_uint(r[8])), "r"(__float_as_uint(r[9])), "r"(__float_as_uint(r[10])), "r"(__float_as_uint(r[11])),
      "r"(__float_as_uint(r[12])), "r"(__float_as_uint(r[13])), "r"(__float_as_uint(r[14])), "r"(__float_as_uint(r[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// shared -> global tile store through a tensor map (bulk async group of the issuing thread)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, int c0, int c1, const void* src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void split8s(const float (&x)[8], uint4& hi, uint4& lo) {
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

template <int GATE>
__global__ void __launch_bounds__(TPB, 2)
bwd_scan_tc_kernel(const __grid_constant__ CUtensorMap tmKg, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ CUtensorMap tmQg, const __grid_constant__ CUtensorMap tmDO,
                   const __grid_constant__ CUtensorMap tmAqk, const __grid_constant__ CUtensorMap tmDH,
                   const ScanParams p) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SS::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + SS::TMEM);
  const uint32_t sb = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int ch = tid & 127, wg = tid >> 7;  // channel (key row of S / value row of dR^T), column half
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;  // b: batch element, or sequence of a packed batch
  const int H = p.H;
  // token rows [bos, bos + 64 NT) of this sequence; its chunks are chunk0 .. chunk0 + NT - 1 of the h / dh tensors
  int bos = b * p.T, NT = p.NT;
  if (p.cu != nullptr) {
    bos = p.cu[b];
    const int len = p.cu[b + 1] - bos;
    NT = len / C;
    if (len < 0 || len % C != 0 || bos % C != 0) {  // outside the envelope: report, touch nothing
      if (threadIdx.x == 0) atomicCAS(p.err, 0, 90);
      return;
    }
  }
  const int chunk0 = bos / C;
  const size_t ldt = (size_t)H * 128;
  const float scale = p.scale, inv_scale = 1.f / p.scale;
  if (NT == 0) {  // empty sequence: the state gradient passes through unchanged
    if (p.dh0 != nullptr)
      for (int i = threadIdx.x; i < DK * DV; i += blockDim.x)
        p.dh0[(size_t)bh * DK * DV + i] = p.dht == nullptr ? 0.f : p.dht[(size_t)bh * DK * DV + i];
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < 8; i++) mbar_init(&bars[i], 1);
    fence_barrier_init();
    prefetch_tmap(&tmKg); prefetch_tmap(&tmW); prefetch_tmap(&tmQg); prefetch_tmap(&tmDO);
    prefetch_tmap(&tmAqk); prefetch_tmap(&tmDH);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *tmem_slot;
  const uint32_t tlane = tb + ((uint32_t)((warp & 3) * 32) << 16);
  uint32_t ph = 0;
  bool alive = true;
  auto wait = [&](int bar, int code) {
    if (alive) alive = mbar_wait(&bars[bar], (ph >> bar) & 1u, p.err, code);
    ph ^= 1u << bar;
  };

  auto row_of = [&](int n) { return bos + n * C; };
  auto issue_l1 = [&](int n) {  // kg and Aqk of chunk n
    const int row0 = row_of(n);
    mbar_expect_tx(&bars[B_L1], 16384 + 8192);
    for (int pn = 0; pn < 2; pn++) tma_load_2d(sm + SS::KG + pn * 8192, &tmKg, h * 128 + 64 * pn, row0, &bars[B_L1]);
    tma_load_2d(sm + SS::AQK, &tmAqk, h * 64, row0, &bars[B_L1]);
  };
  auto issue_do = [&](int n) {  // dO of chunk n (read by both products of the chunk)
    mbar_expect_tx(&bars[B_DO], 16384);
    for (int pn = 0; pn < 2; pn++)
      tma_load_2d(sm + SS::DO0 + pn * 8192, &tmDO, h * 128 + 64 * pn, row_of(n), &bars[B_DO]);
  };
  auto issue_l2 = [&](int n) {  // qg, w of chunk n
    const int row0 = row_of(n);
    mbar_expect_tx(&bars[B_L2], 32768);
    for (int pn = 0; pn < 2; pn++) {
      tma_load_2d(sm + SS::QG + pn * 8192, &tmQg, h * 128 + 64 * pn, row0, &bars[B_L2]);
      tma_load_2d(sm + SS::W + pn * 8192, &tmW, h * 128 + 64 * pn, row0, &bars[B_L2]);
    }
  };
  if (tid == 0) {
    issue_l1(NT - 1);
    issue_do(NT - 1);
  }

  // initial state S' = dht / scale (element (k, v) at k*128 + v, or at v*128 + k in the value-first layout)
  {
    const float* st0 = p.dht == nullptr ? nullptr : p.dht + (size_t)bh * DK * DV;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      float x[16];
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const int v0 = 64 * wg + 16 * c + j;
        if (st0 != nullptr) {
          if (p.svf)
            v4 = make_float4(st0[(size_t)v0 * DK + ch], st0[(size_t)(v0 + 1) * DK + ch], st0[(size_t)(v0 + 2) * DK + ch],
                             st0[(size_t)(v0 + 3) * DK + ch]);
          else
            v4 = *reinterpret_cast<const float4*>(st0 + (size_t)ch * DV + v0);
        }
        x[j] = v4.x * inv_scale; x[j + 1] = v4.y * inv_scale; x[j + 2] = v4.z * inv_scale; x[j + 3] = v4.w * inv_scale;
      }
      tmem_st16f(tlane + TM_S + 64 * wg + 16 * c, x);
    }
    tmem_st_wait();
  }

  constexpr uint32_t ID_DR_A = instr_desc(FMT_BF16, 128, 64, true, false);   // A MN-major (dh^T), B K-major (kg)
  constexpr uint32_t ID_DR_B = instr_desc(FMT_BF16, 128, 64, true, true);    // A MN-major (dO^T), B MN-major (Aqk)
  constexpr uint32_t ID_S_Q = instr_desc(FMT_BF16, 128, 128, true, true);    // A MN-major (qg^T), B MN-major (dO)
  constexpr uint32_t ID_S_W = instr_desc(FMT_BF16, 128, 128, true, false, true, false);  // -(w^T) (dR/scale)^T K-major

  auto load_lambda = [&](int n) -> float {  // per-channel decay of chunk n (log2 gate of its last row)
    const int last = row_of(n) + C - 1;
    if (GATE == GATE_VECTOR) return p.g[((size_t)last * H + h) * 128 + ch];
    if (GATE == GATE_SCALAR) return p.g[(size_t)last * H + h];
    return 0.f;
  };
  float glast = load_lambda(NT - 1);
  int it = 0;
  for (int n = NT - 1; n >= 0; --n, ++it) {
    const int row0 = row_of(n);
    // ---- (a) state row -> dh tiles (hi to global as well), decayed state back to TMEM ---------------------
    if (it > 0) {
      wait(B_S, 1);
      tc_fence_after_sync();
      if (tid == 0 && alive) issue_do(n);  // the dO buffer is free once the previous state update is complete
    }
    const float lam = GATE == GATE_NONE ? 1.f : exp2f(glast);
    if (n > 0) glast = load_lambda(n - 1);  // in flight for a whole chunk before it is needed
    if (alive) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        float x[16];
        tmem_ld16f(tlane + TM_S + 64 * wg + 16 * c, x);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; half++) {
          float y[8];
#pragma unroll
          for (int j = 0; j < 8; j++) y[j] = scale * x[8 * half + j];
          uint4 hi, lo;
          split8s(y, hi, lo);
          *reinterpret_cast<uint4*>(sm + SS::DHHI + wg * 16384 + swz(ch, 2 * c + half)) = hi;
          *reinterpret_cast<uint4*>(sm + SS::DHLO + wg * 16384 + swz(ch, 2 * c + half)) = lo;
        }
        if (GATE != GATE_NONE) {
#pragma unroll
          for (int j = 0; j < 16; j++) x[j] *= lam;
          tmem_st16f(tlane + TM_S + 64 * wg + 16 * c, x);
        }
      }
      if (GATE != GATE_NONE) tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0) {
      const int hrow0 = ((chunk0 + n) * H + h) * 128;
      if (alive) {
        for (int pn = 0; pn < 2; pn++) tma_store_2d(&tmDH, 64 * pn, hrow0, sm + SS::DHHI + pn * 16384);
        bulk_commit();
      }
      wait(B_L1, 2);
      if (alive) {
        tc_fence_after_sync();
        for (int pass = 0; pass < 2; pass++) {
          const uint32_t a = sb + (pass == 0 ? SS::DHHI : SS::DHLO);
          for (int ks = 0; ks < 8; ks++)
            mma_f16(tb + TM_DR, smem_desc(a + ks * 2048, 16384, 1024),
                    smem_desc(sb + SS::KG + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024), ID_DR_A, pass > 0 || ks > 0);
        }
      }
      wait(B_DO, 3);  // dO was requested at the top of the chunk: its latency hides behind the products above
      if (alive) {
        for (int ks = 0; ks < 4; ks++)
          mma_f16(tb + TM_DR, smem_desc(sb + SS::DO0 + ks * 2048, 8192, 1024),
                  smem_desc(sb + SS::AQK + ks * 2048, 8192, 1024), ID_DR_B, true);
        mma_commit(&bars[B_DR]);
      }
    } else {
      ph ^= (1u << B_L1) | (1u << B_DO);
    }
    // ---- (c) dR^T row -> global dR hi/lo, (dR/scale) tiles ----------------------------------------------
    wait(B_DR, 4);
    tc_fence_after_sync();
    if (tid == 0) {
      bulk_wait_read0();  // the dh store has finished reading the hi tile: region X may now be refilled
      if (alive) {
        issue_l2(n);                    // qg, w into the first half of X
        if (n > 0) issue_l1(n - 1);     // kg / Aqk buffers are free as well
      }
    }
    if (alive) {
      const size_t go = ((size_t)row0 * H + h) * 128 + ch;  // + token * ldt
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float x[16];
        tmem_ld16f(tlane + TM_DR + 32 * wg + 16 * c, x);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; half++) {
          float y[8];
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const float v = x[8 * half + j];
            const int tok = 32 * wg + 16 * c + 8 * half + j;
            const bf16 hi = f2bf(v);
            p.dR[go + (size_t)tok * ldt] = hi;
            p.dRlo[go + (size_t)tok * ldt] = f2bf(v - bf2f(hi));
            y[j] = v * inv_scale;
          }
          uint4 hi4, lo4;
          split8s(y, hi4, lo4);
          const int chunk16 = 4 * wg + 2 * c + half;
          *reinterpret_cast<uint4*>(sm + SS::DRHI + swz(ch, chunk16)) = hi4;
          *reinterpret_cast<uint4*>(sm + SS::DRLO + swz(ch, chunk16)) = lo4;
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    // ---- (d) state update -----------------------------------------------------------------------------
    if (tid == 0) {
      wait(B_L2, 5);
      if (alive) {
        tc_fence_after_sync();
        for (int ks = 0; ks < 4; ks++)
          mma_f16(tb + TM_S, smem_desc(sb + SS::QG + ks * 2048, 8192, 1024),
                  smem_desc(sb + SS::DO0 + ks * 2048, 8192, 1024), ID_S_Q, true);
        for (int pass = 0; pass < 2; pass++)
          for (int ks = 0; ks < 4; ks++)
            mma_f16(tb + TM_S, smem_desc(sb + SS::W + ks * 2048, 8192, 1024),
                    smem_desc(sb + (pass == 0 ? SS::DRHI : SS::DRLO) + ks * 32, 16, 1024), ID_S_W, true);
        mma_commit(&bars[B_S]);
      }
    } else {
      ph ^= 1u << B_L2;
    }
  }
  // ---- dh0 = scale * S' ---------------------------------------------------------------------------------
  wait(B_S, 6);
  tc_fence_after_sync();
  if (p.dh0 != nullptr && alive) {
    float* dst = p.dh0 + (size_t)bh * DK * DV;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      float x[16];
      tmem_ld16f(tlane + TM_S + 64 * wg + 16 * c, x);
      tmem_ld_wait();
      const int v0 = 64 * wg + 16 * c;
      if (p.svf) {
#pragma unroll
        for (int j = 0; j < 16; j++) dst[(size_t)(v0 + j) * DK + ch] = scale * x[j];
      } else {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(dst + (size_t)ch * DV + v0 + j) =
              make_float4(scale * x[j], scale * x[j + 1], scale * x[j + 2], scale * x[j + 3]);
      }
    }
  }
  if (tid == 0) bulk_wait0();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}


// ---------------------------------------------------------------------------------------------------------
// Forward state scan (recompute policy):  h[n] stored;  v_new = u - w h[n];  h <- lam*h + kg^T v_new.
// Replaces FLA chunk_gated_delta_rule_fwd_h (src/fast_delta_rule/backends/backward.py:117-118).  Same layout
// tricks as the reverse scan; operands are single BF16 (h and v_new are exactly the tensors that get saved), so it
// needs 97 KB of shared memory and 192 TMEM columns and two CTAs share an SM.
struct FwdParams {
  const float *g, *h0;
  float* final_state;  // optional: state after the last chunk, FP32 [B,H,K,V] ([B,H,V,K] when svf)
  bf16* v_new;
  int* err;
  int T, H, NT;
  int svf;  // h0 is stored value-first: [B,H,V,K]
  const int* cu;  // packed sequences: device int32 [sequences + 1] token offsets (multiples of 64), or nullptr
};
struct FS {
  static constexpr uint32_t W = 0;                // [64 i][128 k] two panels   16 KB
  static constexpr uint32_t KG = W + 16384;       // [64 i][128 k]              16 KB
  static constexpr uint32_t U = KG + 16384;       // [64 i][128 v]              16 KB
  static constexpr uint32_t HT = U + 16384;       // h tile [128 k][128 v]      32 KB
  static constexpr uint32_t VNT = HT + 32768;     // v_new^T [128 v][64 i]      16 KB
  static constexpr uint32_t BARS = VNT + 16384;
  static constexpr uint32_t TMEM = BARS + 64;
  static constexpr uint32_t TOTAL = TMEM + 64;
};
enum { F_W = 0, F_KG, F_U, F_V, F_S };
constexpr uint32_t TMF_S = 0, TMF_V = 128;

template <int GATE>
__global__ void __launch_bounds__(TPB, 2)
fwd_scan_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmKg,
                   const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmH, const FwdParams p) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + FS::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + FS::TMEM);
  const uint32_t sb = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int ch = tid & 127, wg = tid >> 7;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;  // b: batch element, or sequence of a packed batch
  const int H = p.H;
  int bos = b * p.T, NT = p.NT;
  if (p.cu != nullptr) {
    bos = p.cu[b];
    const int len = p.cu[b + 1] - bos;
    NT = len / C;
    if (len < 0 || len % C != 0 || bos % C != 0) {  // outside the envelope: report, touch nothing
      if (threadIdx.x == 0) atomicCAS(p.err, 0, 91);
      return;
    }
  }
  const int chunk0 = bos / C;
  const size_t ldt = (size_t)H * 128;
  if (NT == 0) {  // empty sequence: the state passes through unchanged
    if (p.final_state != nullptr)
      for (int i = threadIdx.x; i < DK * DV; i += blockDim.x)
        p.final_state[(size_t)bh * DK * DV + i] = p.h0 == nullptr ? 0.f : p.h0[(size_t)bh * DK * DV + i];
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < 8; i++) mbar_init(&bars[i], 1);
    fence_barrier_init();
    prefetch_tmap(&tmW); prefetch_tmap(&tmKg); prefetch_tmap(&tmU); prefetch_tmap(&tmH);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = *tmem_slot;
  const uint32_t tlane = tb + ((uint32_t)((warp & 3) * 32) << 16);
  uint32_t ph = 0;
  bool alive = true;
  auto wait = [&](int bar, int code) {
    if (alive) alive = mbar_wait(&bars[bar], (ph >> bar) & 1u, p.err, code);
    ph ^= 1u << bar;
  };
  auto row_of = [&](int n) { return bos + n * C; };
  auto load2 = [&](uint32_t dst, const CUtensorMap* m, int n, int bar) {
    mbar_expect_tx(&bars[bar], 16384);
    for (int pn = 0; pn < 2; pn++) tma_load_2d(sm + dst + pn * 8192, m, h * 128 + 64 * pn, row_of(n), &bars[bar]);
  };
  if (tid == 0) {
    load2(FS::W, &tmW, 0, F_W);
    load2(FS::U, &tmU, 0, F_U);
    load2(FS::KG, &tmKg, 0, F_KG);
  }
  {  // initial state (element (k, v) at k*128 + v, or at v*128 + k in the value-first layout)
    const float* st0 = p.h0 == nullptr ? nullptr : p.h0 + (size_t)bh * DK * DV;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      float x[16];
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
        const int v0 = 64 * wg + 16 * c + j;
        if (st0 != nullptr) {
          if (p.svf)
            v4 = make_float4(st0[(size_t)v0 * DK + ch], st0[(size_t)(v0 + 1) * DK + ch], st0[(size_t)(v0 + 2) * DK + ch],
                             st0[(size_t)(v0 + 3) * DK + ch]);
          else
            v4 = *reinterpret_cast<const float4*>(st0 + (size_t)ch * DV + v0);
        }
        x[j] = v4.x; x[j + 1] = v4.y; x[j + 2] = v4.z; x[j + 3] = v4.w;
      }
      tmem_st16f(tlane + TMF_S + 64 * wg + 16 * c, x);
    }
    tmem_st_wait();
  }
  constexpr uint32_t ID_V = instr_desc(FMT_BF16, 128, 64, true, false, true, false);  // -(h^T) w^T: A MN-major negated
  constexpr uint32_t ID_S = instr_desc(FMT_BF16, 128, 128, true, false);              // kg^T (v_new^T)^T
  auto load_lambda = [&](int n) -> float {
    const int last = row_of(n) + C - 1;
    if (GATE == GATE_VECTOR) return p.g[((size_t)last * H + h) * 128 + ch];
    if (GATE == GATE_SCALAR) return p.g[(size_t)last * H + h];
    return 0.f;
  };
  float glast = load_lambda(0);
  for (int n = 0; n < NT; ++n) {
    const int row0 = row_of(n);
    if (n > 0) {
      wait(F_S, 1);
      tc_fence_after_sync();
      if (tid == 0 && alive) load2(FS::KG, &tmKg, n, F_KG);  // kg buffer is free once the previous update is done
    }
    const float lam = GATE == GATE_NONE ? 1.f : exp2f(glast);
    if (n + 1 < NT) glast = load_lambda(n + 1);
    if (alive) {
#pragma unroll
      for (int c = 0; c < 4; c++) {
        float x[16];
        tmem_ld16f(tlane + TMF_S + 64 * wg + 16 * c, x);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; half++) {
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 4; j++) pk[j] = pack_bf16(x[8 * half + 2 * j], x[8 * half + 2 * j + 1]);
          *reinterpret_cast<uint4*>(sm + FS::HT + wg * 16384 + swz(ch, 2 * c + half)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        if (GATE != GATE_NONE) {
#pragma unroll
          for (int j = 0; j < 16; j++) x[j] *= lam;
          tmem_st16f(tlane + TMF_S + 64 * wg + 16 * c, x);
        }
      }
      if (GATE != GATE_NONE) tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0) {
      const int hrow0 = ((chunk0 + n) * H + h) * 128;
      if (alive) {
        for (int pn = 0; pn < 2; pn++) tma_store_2d(&tmH, 64 * pn, hrow0, sm + FS::HT + pn * 16384);
        bulk_commit();
      }
      wait(F_W, 2);
      if (alive) {
        tc_fence_after_sync();
        for (int ks = 0; ks < 8; ks++)
          mma_f16(tb + TMF_V, smem_desc(sb + FS::HT + ks * 2048, 16384, 1024),
                  smem_desc(sb + FS::W + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024), ID_V, ks > 0);
        mma_commit(&bars[F_V]);
      }
    } else {
      ph ^= 1u << F_W;
    }
    // v_new^T row = u - (w h)^T: to global (token-major) and to the K-major tile of the state update
    wait(F_V, 3);
    tc_fence_after_sync();
    if (tid == 0 && alive && n + 1 < NT) load2(FS::W, &tmW, n + 1, F_W);
    wait(F_U, 4);
    if (alive) {
      const size_t go = ((size_t)row0 * H + h) * 128 + ch;
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float x[16];
        tmem_ld16f(tlane + TMF_V + 32 * wg + 16 * c, x);
        tmem_ld_wait();
#pragma unroll
        for (int half = 0; half < 2; half++) {
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            bf16 r2[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int tok = 32 * wg + 16 * c + 8 * half + j + e;
              const bf16 uu = *reinterpret_cast<const bf16*>(sm + FS::U + (ch >> 6) * 8192 + swz(tok, (ch & 63) >> 3) + (ch & 7) * 2);
              r2[e] = f2bf(bf2f(uu) + x[8 * half + j + e]);
              p.v_new[go + (size_t)tok * ldt] = r2[e];
            }
            pk[j >> 1] = (uint32_t)(*reinterpret_cast<uint16_t*>(&r2[0])) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&r2[1])) << 16);
          }
          *reinterpret_cast<uint4*>(sm + FS::VNT + swz(ch, 4 * wg + 2 * c + half)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
    if (tid == 0) bulk_wait_read0();
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0) {
      if (alive && n + 1 < NT) load2(FS::U, &tmU, n + 1, F_U);  // every thread is done with this chunk's u tile
      wait(F_KG, 5);
      if (alive) {
        tc_fence_after_sync();
        for (int ks = 0; ks < 4; ks++)
          mma_f16(tb + TMF_S, smem_desc(sb + FS::KG + ks * 2048, 8192, 1024),
                  smem_desc(sb + FS::VNT + ks * 32, 16, 1024), ID_S, true);
        mma_commit(&bars[F_S]);
      }
    } else {
      ph ^= 1u << F_KG;
    }
  }
  wait(F_S, 6);
  tc_fence_after_sync();
  if (p.final_state != nullptr && alive) {
    float* dst = p.final_state + (size_t)bh * DK * DV;
#pragma unroll
    for (int c = 0; c < 4; c++) {
      float x[16];
      tmem_ld16f(tlane + TMF_S + 64 * wg + 16 * c, x);
      tmem_ld_wait();
      const int v0 = 64 * wg + 16 * c;
      if (p.svf) {
#pragma unroll
        for (int j = 0; j < 16; j++) dst[(size_t)(v0 + j) * DK + ch] = x[j];
      } else {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(dst + (size_t)ch * DV + v0 + j) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
      }
    }
  }
  if (tid == 0) bulk_wait0();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}

constexpr size_t FWD_SCAN_SMEM = FS::TOTAL + 1024;
static_assert(2 * (FWD_SCAN_SMEM + 1024) <= 233472, "two forward-scan CTAs must fit one SM");

template <int GATE>
cudaError_t run_fwd(const CUtensorMap* tm, const FwdParams& p, int grid, cudaStream_t st) {
  auto kern = fwd_scan_tc_kernel<GATE>;
  cudaError_t e = ensure_dynamic_smem<fwd_scan_tc_kernel<GATE>>(FWD_SCAN_SMEM);
  if (e != cudaSuccess) return e;
  kern<<<grid, TPB, FWD_SCAN_SMEM, st>>>(tm[0], tm[1], tm[2], tm[3], p);
  count_launch();
  return cudaGetLastError();
}

constexpr size_t SCAN_SMEM = SS::TOTAL + 1024;

template <int GATE>
cudaError_t run(const CUtensorMap* tm, const ScanParams& p, int grid, cudaStream_t st) {
  auto kern = bwd_scan_tc_kernel<GATE>;
  cudaError_t e = ensure_dynamic_smem<bwd_scan_tc_kernel<GATE>>(SCAN_SMEM);
  if (e != cudaSuccess) return e;
  kern<<<grid, TPB, SCAN_SMEM, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// err: device status word.  A bounded wait that gives up records its site there with atomicCAS(err, 0, site), so the
// first failing site of a call survives; the caller zeroes the word once per call, before its first stage.
cudaError_t launch_bwd_scan_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st) {
  const int B = a.B, T = a.T, H = a.H, NT = T / C;
  const uint64_t rows = (uint64_t)B * T, srows = (uint64_t)B * NT * H * 128;
  CUtensorMap tm[6];
  bool ok = encode_tmap_2d(&tm[0], s.kg, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[1], s.w, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[2], s.qg, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[3], a.d_o, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[4], s.Aqk, 2, (uint64_t)H * 64, rows, (uint64_t)H * 128, 64, 64) &&
            encode_tmap_2d(&tm[5], s.dh, 2, 128, srows, 256, 64, 128);
  if (!ok) return cudaErrorInvalidValue;
  ScanParams p;
  p.g = a.g; p.dht = a.dht; p.dR = (bf16*)s.dR; p.dRlo = (bf16*)s.dR_lo; p.dh0 = a.dh0; p.err = err;
  p.T = T; p.H = H; p.NT = NT; p.svf = a.state_v_first; p.cu = a.cu_seqlens; p.scale = a.scale;
  const int seqs = a.cu_seqlens != nullptr ? a.num_seqs : B;  // one CTA per (sequence, head)
  switch (gate_mode_of(a.family)) {
    case GATE_NONE: return run<GATE_NONE>(tm, p, seqs * H, st);
    case GATE_SCALAR: return run<GATE_SCALAR>(tm, p, seqs * H, st);
    default: return run<GATE_VECTOR>(tm, p, seqs * H, st);
  }
}

// err: device status word, same contract as for the reverse scan.
cudaError_t launch_fwd_scan_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st,
                               float* final_state) {
  const int B = a.B, T = a.T, H = a.H, NT = T / C;
  const uint64_t rows = (uint64_t)B * T, srows = (uint64_t)B * NT * H * 128;
  CUtensorMap tm[4];
  bool ok = encode_tmap_2d(&tm[0], s.w, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[1], s.kg, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[2], s.u, 2, (uint64_t)H * 128, rows, (uint64_t)H * 256, 64, 64) &&
            encode_tmap_2d(&tm[3], s.h, 2, 128, srows, 256, 64, 128);
  if (!ok) return cudaErrorInvalidValue;
  FwdParams p;
  p.g = a.g; p.h0 = a.h0; p.final_state = final_state; p.v_new = (bf16*)s.v_new; p.err = err; p.T = T; p.H = H; p.NT = NT; p.svf = a.state_v_first;
  p.cu = a.cu_seqlens;
  const int seqs = a.cu_seqlens != nullptr ? a.num_seqs : B;  // one CTA per (sequence, head)
  switch (gate_mode_of(a.family)) {
    case GATE_NONE: return run_fwd<GATE_NONE>(tm, p, seqs * H, st);
    case GATE_SCALAR: return run_fwd<GATE_SCALAR>(tm, p, seqs * H, st);
    default: return run_fwd<GATE_VECTOR>(tm, p, seqs * H, st);
  }
}

}  // namespace rewy
