// Stage "prepare" on the Blackwell tensor cores: TMA tile loads and stores, tcgen05 products with TMEM accumulators.
//
// Same mathematics as prepare_kernel in prepare.cu (the reference functions it replaces are listed there):
//   w = Akk (b k gamma), u = Akk (w_gate v), qg = q gamma, kg = k 2^(g_last - g)
//   and, for the scalar-gate / ungated families, Aqk = scale tril((q k^T) 2^(g_i - g_j)).
// Persistent CTAs walk over chunks (head fastest); two CTAs share an SM and hide each other's waits.  Per chunk:
//   * one elected thread requests the k, v, q, Akk (and gate) tiles by TMA (GDN2: the key gate lands in the tile that
//     becomes kg; the value gate is read with plain 16-byte loads, which keeps the plan at 105 KB);
//   * scalar families: q k^T runs first on the tiles as they landed (M=128 with only lanes 0..63 meaningful);
//   * every thread turns 16-byte pieces of the k / v / q tiles IN PLACE into E = b k gamma, Z = w_gate v and qg (the
//     tiles keep the 128-byte-swizzled layout TMA wrote, which is what the products and the tile stores read), and
//     writes kg into a tile of its own;
//   * w^T = E^T Akk^T and u^T = Z^T Akk^T are two M=128 (channel), N=64 (token), K=64 products: A is the E / Z tile read
//     MN-major, B the Akk tile K-major.  qg and kg leave by TMA while they run;
//   * epilogue thread (channel, token half) reads its accumulator rows and writes the dense [token][channel] BF16
//     tiles of w and u, which leave by TMA.
#include "tc05.cuh"

namespace rewy {
namespace {
using namespace tc;

struct PrepParams {
  const float *g, *beta;
  const bf16* wg;  // GDN2 value gate, read with plain 16-byte loads
  bf16* Aqk;
  int* err;
  int T, H, NT, total_chunks;
  int write_qk;  // 0: qg and kg are not stored (a family without a gate, whose scans read q and k themselves)
  float scale;
};

// Shared-memory plan, byte offsets from a 1024-byte aligned base.
struct PS {
  static constexpr uint32_t KT = 0;                // k tile, 2 panels [64 t][64 k]; becomes E in place        16 KB
  static constexpr uint32_t VT = KT + 16384;       // v tile; becomes Z in place                               16 KB
  static constexpr uint32_t QT = VT + 16384;       // q tile; becomes qg in place                              16 KB
  static constexpr uint32_t KGT = QT + 16384;      // kg tile, same layout; GDN2: the key gate tile lands here 16 KB
                                                   // first (each thread reads its piece of it before writing kg there)
  static constexpr uint32_t AK = KGT + 16384;      // Akk [64 i][64 j]                                         8 KB
  static constexpr uint32_t GT = AK + 8192;        // vector gate: 4 panels [64 t][32 k] FP32                  32 KB
  static constexpr uint32_t WO = GT;               // dense [64 t][128 k] BF16 output tiles of w and u take the gate
  static constexpr uint32_t UO = GT + 16384;       // tile once every thread has its factors
  static constexpr uint32_t ROWS = GT + 32768;     // float[64] beta rows, float[64] scalar gate rows
  static constexpr uint32_t BARS = ROWS + 512;
  static constexpr uint32_t TMEM = BARS + 64;
  static constexpr uint32_t TOTAL = TMEM + 64;
};
constexpr uint32_t TM_W = 0, TM_U = 64, TM_AQK = 128;
enum { PB_LOAD = 0, PB_AQK, PB_MMA, PB_COUNT };
constexpr int TPB = 256;

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

template <int GATE, bool VB>
__global__ void __launch_bounds__(TPB, 2)
prepare_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                  const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmAkk,
                  const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmBG,
                  const __grid_constant__ CUtensorMap tmQg,
                  const __grid_constant__ CUtensorMap tmKg, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmU, const PrepParams p) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  float* sBeta = reinterpret_cast<float*>(sm + PS::ROWS);
  float* sGs = sBeta + C;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + PS::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + PS::TMEM);
  const uint32_t sb = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int ch = tid & 127, half = tid >> 7;
  const int T = p.T, H = p.H, NT = p.NT;
  constexpr bool SCALAR_FAMILY = GATE != GATE_VECTOR;  // these save no Aqk: it is rebuilt here

  if (tid == 0) {
    for (int i = 0; i < PB_COUNT; i++) mbar_init(&bars[i], 1);
    fence_barrier_init();
    prefetch_tmap(&tmK); prefetch_tmap(&tmV); prefetch_tmap(&tmQ); prefetch_tmap(&tmAkk);
    prefetch_tmap(&tmQg); prefetch_tmap(&tmKg); prefetch_tmap(&tmW); prefetch_tmap(&tmU);
    if (GATE == GATE_VECTOR) prefetch_tmap(&tmG);
    if (VB) prefetch_tmap(&tmBG);
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
  const bool leader = warp == 0 && elect_one();
  uint32_t ph = 0;
  bool alive = true;
  auto wait = [&](int b, int code) {
    if (alive) alive = mbar_wait(&bars[b], (ph >> b) & 1u, p.err, code);
  };
  const uint32_t sb4 = sb >> 4;
  auto dl = [&](uint32_t off, uint32_t lbo) { return sb4 + (off >> 4) + ((lbo >> 4) << 16); };

  constexpr uint32_t ID_WU = instr_desc(FMT_BF16, 128, 64, true, false);   // A MN-major (E / Z), B K-major (Akk)
  constexpr uint32_t ID_QK = instr_desc(FMT_BF16, 128, 64, false, false);  // A K-major (q), B K-major (k)

  for (int chunk = blockIdx.x; chunk < p.total_chunks && alive; chunk += gridDim.x) {
    const int bn = chunk / H, h = chunk - bn * H, b = bn / NT, n = bn - b * NT;  // head fastest
    const int row0 = b * T + n * C;
    const size_t base1 = (size_t)row0 * H + h;
    uint32_t used = (1u << PB_LOAD) | (1u << PB_MMA) | (SCALAR_FAMILY ? 1u << PB_AQK : 0u);

    if (warp == 0) {
      if (leader) {
        mbar_expect_tx(&bars[PB_LOAD], 3 * 16384 + 8192 + (GATE == GATE_VECTOR ? 32768 : 0) + (VB ? 16384 : 0));
        tma_load_3d(sm + PS::KT, &tmK, h * 128, row0, 0, &bars[PB_LOAD]);
        tma_load_3d(sm + PS::VT, &tmV, h * 128, row0, 0, &bars[PB_LOAD]);
        tma_load_3d(sm + PS::QT, &tmQ, h * 128, row0, 0, &bars[PB_LOAD]);
        tma_load_2d(sm + PS::AK, &tmAkk, h * 64, row0, &bars[PB_LOAD]);
        if (GATE == GATE_VECTOR) tma_load_3d(sm + PS::GT, &tmG, h * 128, row0, 0, &bars[PB_LOAD]);
        if (VB) tma_load_3d(sm + PS::KGT, &tmBG, h * 128, row0, 0, &bars[PB_LOAD]);
      }
      __syncwarp();
    }
    if (tid < C) {
      if (!VB) sBeta[tid] = p.beta[base1 + (size_t)tid * H];
      if (GATE == GATE_SCALAR) sGs[tid] = p.g[base1 + (size_t)tid * H];
    }
    wait(PB_LOAD, 1);
    __syncthreads();  // beta / scalar gate rows visible

    // ---- scalar families: q k^T on the tiles as they landed, before they are rewritten in place --------------------
    if (SCALAR_FAMILY) {
      if (warp == 0 && alive) {
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ks++)
            mma_f16_lo(tb + TM_AQK, dl(PS::QT + (ks >> 2) * 8192 + (ks & 3) * 32, 16),
                       dl(PS::KT + (ks >> 2) * 8192 + (ks & 3) * 32, 16), ID_QK, ks > 0);
          mma_commit(&bars[PB_AQK]);
        }
        __syncwarp();
      }
      wait(PB_AQK, 2);
      tc_fence_after_sync();
      if (alive && ch < C) {
        // lanes 0..63 hold rows i of q k^T; thread (i, half) finishes 32 columns j
        const int i = ch;
        const float gi = GATE == GATE_SCALAR ? sGs[i] : 0.f;
        bf16* dst = p.Aqk + (base1 + (size_t)i * H) * 64 + 32 * half;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          float x[16];
          tmem_ld16(tlane + TM_AQK + 32 * half + 16 * c, x);
          tmem_ld_wait();
          uint32_t pk[8];
#pragma unroll
          for (int j2 = 0; j2 < 8; j2++) {
            float y[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
              const int j = 32 * half + 16 * c + 2 * j2 + e;
              float f = p.scale;
              if (GATE == GATE_SCALAR) f *= exp2f(gi - sGs[j <= i ? j : i]);
              y[e] = j <= i ? x[2 * j2 + e] * f : 0.f;
            }
            pk[j2] = pack_bf16(y[0], y[1]);
          }
          *reinterpret_cast<uint4*>(dst + 16 * c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint4*>(dst + 16 * c + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
      tc_fence_before_sync();
      __syncthreads();  // the product has read q and k: they may be rewritten now
      tc_fence_after_sync();
    }

    // ---- element-wise operands, in place: 16-byte pieces (row r, 8 channels) ---------------------------------------
    if (alive) {
#pragma unroll
      for (int it = 0; it < (C * 16) / TPB; it++) {
        const int i = tid + it * TPB;
        const int r = i >> 4, c16 = i & 15;                       // row, 16-byte piece of the 128 channels
        const uint32_t off = (c16 >> 3) * 8192 + swz(r, c16 & 7);  // same place in every BF16 tile
        const uint4 kr = *reinterpret_cast<const uint4*>(sm + PS::KT + off);
        const uint4 vr = *reinterpret_cast<const uint4*>(sm + PS::VT + off);
        const uint4 qr = *reinterpret_cast<const uint4*>(sm + PS::QT + off);
        float gg[8], gl[8];
        if (GATE == GATE_VECTOR) {
          // FP32 gate tile: panels of 32 channels; 8 channels = two 16-byte pieces
          const uint32_t gp = PS::GT + (c16 >> 2) * 8192, gc = (c16 & 3) * 2;
          const float4 ga = *reinterpret_cast<const float4*>(sm + gp + swz(r, gc));
          const float4 gb = *reinterpret_cast<const float4*>(sm + gp + swz(r, gc + 1));
          const float4 la = *reinterpret_cast<const float4*>(sm + gp + swz(C - 1, gc));
          const float4 lb = *reinterpret_cast<const float4*>(sm + gp + swz(C - 1, gc + 1));
          gg[0] = ga.x; gg[1] = ga.y; gg[2] = ga.z; gg[3] = ga.w; gg[4] = gb.x; gg[5] = gb.y; gg[6] = gb.z; gg[7] = gb.w;
          gl[0] = la.x; gl[1] = la.y; gl[2] = la.z; gl[3] = la.w; gl[4] = lb.x; gl[5] = lb.y; gl[6] = lb.z; gl[7] = lb.w;
        } else {
#pragma unroll
          for (int j = 0; j < 8; j++) {
            gg[j] = GATE == GATE_SCALAR ? sGs[r] : 0.f;
            gl[j] = GATE == GATE_SCALAR ? sGs[C - 1] : 0.f;
          }
        }
        uint4 br = make_uint4(0, 0, 0, 0), wr = br;
        const float bs = VB ? 0.f : sBeta[r];
        if (VB) {
          br = *reinterpret_cast<const uint4*>(sm + PS::KGT + off);
          wr = *reinterpret_cast<const uint4*>(p.wg + ((size_t)(row0 + r) * H + h) * 128 + c16 * 8);
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
          if (VB) {
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
        *reinterpret_cast<uint4*>(sm + PS::KT + off) = make_uint4(eo[0], eo[1], eo[2], eo[3]);
        *reinterpret_cast<uint4*>(sm + PS::VT + off) = make_uint4(zo[0], zo[1], zo[2], zo[3]);
        *reinterpret_cast<uint4*>(sm + PS::QT + off) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
        *reinterpret_cast<uint4*>(sm + PS::KGT + off) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();

    // ---- w^T = E^T Akk^T, u^T = Z^T Akk^T; qg and kg leave meanwhile -------------------------------------------------
    if (warp == 0 && alive) {
      if (leader) {
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
          mma_f16_lo(tb + TM_W, dl(PS::KT + ks * 2048, 8192), dl(PS::AK + ks * 32, 16), ID_WU, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ks++)
          mma_f16_lo(tb + TM_U, dl(PS::VT + ks * 2048, 8192), dl(PS::AK + ks * 32, 16), ID_WU, ks > 0);
        mma_commit(&bars[PB_MMA]);
        if (p.write_qk) {
          tma_store_3d(&tmQg, sm + PS::QT, h * 128, row0, 0);
          tma_store_3d(&tmKg, sm + PS::KGT, h * 128, row0, 0);
          tma_store_commit();
        }
      }
      __syncwarp();
    }
    wait(PB_MMA, 3);
    tc_fence_after_sync();
    if (alive) {
      // thread (channel ch, token half): 32 tokens of w^T and of u^T -> dense [token][channel] BF16 tiles
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float xw[16], xu[16];
        tmem_ld16(tlane + TM_W + 32 * half + 16 * c, xw);
        tmem_ld16(tlane + TM_U + 32 * half + 16 * c, xu);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int t = 32 * half + 16 * c + j;
          *reinterpret_cast<bf16*>(sm + PS::WO + t * 256 + ch * 2) = f2bf(xw[j]);
          *reinterpret_cast<bf16*>(sm + PS::UO + t * 256 + ch * 2) = f2bf(xu[j]);
        }
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 0) {
      if (leader) {
        if (alive) {
          tma_store_2d(&tmW, sm + PS::WO, h * 128, row0);
          tma_store_2d(&tmU, sm + PS::UO, h * 128, row0);
          tma_store_commit();
        }
        tma_store_wait_read();  // every output tile has been read before the next chunk's loads land on them
      }
      __syncwarp();
    }
    ph ^= used;
    alive = __syncthreads_and(alive ? 1 : 0) != 0;
  }

  if (leader) tma_store_wait_read();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}

constexpr size_t PREP_TC_SMEM = PS::TOTAL + 1024;
static_assert(2 * (PREP_TC_SMEM + 1024) <= 233472, "two prepare CTAs must fit one SM");

int sm_count_prepare() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 148;
  }
  return n;
}

template <int GATE, bool VB>
cudaError_t run(const CUtensorMap* tm, const PrepParams& p, cudaStream_t st) {
  const size_t smem = PREP_TC_SMEM;
  cudaError_t e = ensure_dynamic_smem<prepare_tc_kernel<GATE, VB>>(smem);
  if (e != cudaSuccess) return e;
  const int cap = sm_count_prepare() * 2;  // two CTAs per SM
  const int grid = p.total_chunks < cap ? p.total_chunks : cap;
  prepare_tc_kernel<GATE, VB><<<grid, TPB, smem, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], tm[5], tm[7], tm[8], tm[9], tm[10], p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace

// err: device status word (first failing bounded wait of the call is recorded there).
cudaError_t launch_prepare_tc(const RewyBwdArgs& a, const RewyStageBuffers& s, int* err, cudaStream_t st) {
  const int B = a.B, T = a.T, H = a.H, NT = T / C;
  const uint64_t rows = (uint64_t)B * T, cols = (uint64_t)H * 128, pitch = (uint64_t)H * 256;
  const bool vector = gate_mode_of(a.family) == GATE_VECTOR, vb = a.family == REWY_GDN2;
  CUtensorMap tm[11];
  bool ok = encode_tmap_panels(&tm[0], a.k, 2, cols, rows, pitch, 64, 2) &&
            encode_tmap_panels(&tm[1], a.v, 2, cols, rows, pitch, 64, 2) &&
            encode_tmap_panels(&tm[2], a.q, 2, cols, rows, pitch, 64, 2) &&
            encode_tmap_2d(&tm[3], a.Akk, 2, (uint64_t)H * 64, rows, (uint64_t)H * 128, 64, 64) &&
            encode_tmap_2d(&tm[9], s.w, 2, cols, rows, pitch, 128, 64, false) &&
            encode_tmap_2d(&tm[10], s.u, 2, cols, rows, pitch, 128, 64, false);
  tm[4] = tm[5] = tm[6] = tm[7] = tm[8] = tm[0];  // never dereferenced unless the family has the tensor
  const bool write_qk = s.qg != nullptr && s.kg != nullptr;
  if (ok && write_qk)
    ok = encode_tmap_panels(&tm[7], s.qg, 2, cols, rows, pitch, 64, 2) &&
         encode_tmap_panels(&tm[8], s.kg, 2, cols, rows, pitch, 64, 2);
  if (ok && vector) ok = encode_tmap_panels(&tm[4], a.g, 4, cols, rows, (uint64_t)H * 512, 64, 4);
  if (ok && vb) ok = encode_tmap_panels(&tm[5], a.b_gate, 2, cols, rows, pitch, 64, 2);
  if (!ok) return cudaErrorInvalidValue;
  PrepParams p;
  p.g = a.g; p.beta = a.beta; p.wg = (const bf16*)a.w_gate; p.Aqk = (bf16*)s.Aqk; p.err = err;
  p.T = T; p.H = H; p.NT = NT; p.total_chunks = B * H * NT; p.scale = a.scale;
  p.write_qk = write_qk ? 1 : 0;
  switch (a.family) {
    case REWY_DELTA: return run<GATE_NONE, false>(tm, p, st);
    case REWY_GDN: return run<GATE_SCALAR, false>(tm, p, st);
    case REWY_KDA: return run<GATE_VECTOR, false>(tm, p, st);
    default: return run<GATE_VECTOR, true>(tm, p, st);
  }
}

}  // namespace rewy
