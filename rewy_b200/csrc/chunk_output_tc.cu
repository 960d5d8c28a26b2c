// Forward output of one chunk on the Blackwell tensor cores:  o = scale * qg h[n] + Aqk v_new.
//
// Computed transposed so that every accumulator has M = 128 rows (value channel = TMEM lane):
//   o1^T[v, i] = sum_k h[k, v] qg[i, k]          A = h tile read MN-major, B = qg tile K-major     M=128 N=64 K=128
//   o2^T[v, i] = sum_j v_new[j, v] Aqk[i, j]     A = v_new tile read MN-major, B = Aqk K-major     M=128 N=64 K=64
// Every operand is a tile exactly as TMA lands it.  Epilogue thread (value channel, token half) combines
// scale * o1 + o2 and writes the dense [token][channel] BF16 tile, which leaves by TMA.  Persistent CTAs walk over
// chunks (head fastest); two CTAs share an SM and hide each other's load waits.
// Replaces FLA's chunk_gla_fwd_o_gk / chunk_fwd_o as called inside chunk_kda_fwd and its siblings
// (src/fast_delta_rule/_compat/kda.py:89-113).
#include "tc05.cuh"

namespace rewy {
namespace {
using namespace tc;

struct OutParams {
  int* err;
  int T, H, NT, total_chunks;
  float scale;
};

struct OS {
  static constexpr uint32_t HT = 0;               // h tile, 2 panels [128 k][64 v]           32 KB
  static constexpr uint32_t QG = HT + 32768;      // qg tile, 2 panels [64 i][64 k]           16 KB
  static constexpr uint32_t VN = QG + 16384;      // v_new tile, 2 panels [64 j][64 v]        16 KB
  static constexpr uint32_t AQ = VN + 16384;      // Aqk [64 i][64 j]                         8 KB
  static constexpr uint32_t OT = AQ + 8192;       // dense [64 t][128 v] BF16 output tile     16 KB
  static constexpr uint32_t BARS = OT + 16384;
  static constexpr uint32_t TMEM = BARS + 64;
  static constexpr uint32_t TOTAL = TMEM + 64;
};
constexpr uint32_t TM_O1 = 0, TM_O2 = 64;
enum { OB_LOAD = 0, OB_MMA, OB_COUNT };
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

__global__ void __launch_bounds__(TPB, 2)
chunk_output_tc_kernel(const __grid_constant__ CUtensorMap tmH, const __grid_constant__ CUtensorMap tmQg,
                       const __grid_constant__ CUtensorMap tmVn, const __grid_constant__ CUtensorMap tmAqk,
                       const __grid_constant__ CUtensorMap tmO, const OutParams p) {
  extern __shared__ __align__(1024) unsigned char raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OS::BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OS::TMEM);
  const uint32_t sb = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5;
  const int ch = tid & 127, half = tid >> 7;
  const int T = p.T, H = p.H, NT = p.NT;

  if (tid == 0) {
    for (int i = 0; i < OB_COUNT; i++) mbar_init(&bars[i], 1);
    fence_barrier_init();
    prefetch_tmap(&tmH); prefetch_tmap(&tmQg); prefetch_tmap(&tmVn); prefetch_tmap(&tmAqk); prefetch_tmap(&tmO);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 128);
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
  constexpr uint32_t ID_O = instr_desc(FMT_BF16, 128, 64, true, false);  // A MN-major, B K-major

  for (int chunk = blockIdx.x; chunk < p.total_chunks && alive; chunk += gridDim.x) {
    const int bn = chunk / H, h = chunk - bn * H, b = bn / NT, n = bn - b * NT;  // head fastest
    const int row0 = b * T + n * C;
    const int hrow0 = ((b * NT + n) * H + h) * 128;
    if (warp == 0) {
      if (leader) {
        mbar_expect_tx(&bars[OB_LOAD], 32768 + 2 * 16384 + 8192);
        tma_load_3d(sm + OS::HT, &tmH, 0, hrow0, 0, &bars[OB_LOAD]);
        tma_load_3d(sm + OS::QG, &tmQg, h * 128, row0, 0, &bars[OB_LOAD]);
        tma_load_3d(sm + OS::VN, &tmVn, h * 128, row0, 0, &bars[OB_LOAD]);
        tma_load_2d(sm + OS::AQ, &tmAqk, h * 64, row0, &bars[OB_LOAD]);
      }
      __syncwarp();
    }
    if (warp == 0) {
      wait(OB_LOAD, 31);
      if (alive) {
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 8; ks++)   // K = key channel: 16 rows of the h tile per step
            mma_f16_lo(tb + TM_O1, dl(OS::HT + ks * 2048, 16384), dl(OS::QG + (ks >> 2) * 8192 + (ks & 3) * 32, 16), ID_O, ks > 0);
#pragma unroll
          for (int ks = 0; ks < 4; ks++)   // K = token j: 16 rows of the v_new tile per step
            mma_f16_lo(tb + TM_O2, dl(OS::VN + ks * 2048, 8192), dl(OS::AQ + ks * 32, 16), ID_O, ks > 0);
          mma_commit(&bars[OB_MMA]);
        }
      }
      __syncwarp();
    }
    wait(OB_MMA, 32);
    tc_fence_after_sync();
    if (alive) {
#pragma unroll
      for (int c = 0; c < 2; c++) {
        float x1[16], x2[16];
        tmem_ld16(tlane + TM_O1 + 32 * half + 16 * c, x1);
        tmem_ld16(tlane + TM_O2 + 32 * half + 16 * c, x2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j++) {
          const int t = 32 * half + 16 * c + j;
          *reinterpret_cast<bf16*>(sm + OS::OT + t * 256 + ch * 2) = f2bf(fmaf(p.scale, x1[j], x2[j]));
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
          tma_store_2d(&tmO, sm + OS::OT, h * 128, row0);
          tma_store_commit();
        }
        tma_store_wait_read();  // the output tile has been read before the next chunk's epilogue writes it
      }
      __syncwarp();
    }
    ph ^= (1u << OB_LOAD) | (1u << OB_MMA);
    alive = __syncthreads_and(alive ? 1 : 0) != 0;
  }
  if (leader) tma_store_wait_read();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 128);
}

constexpr size_t OUT_TC_SMEM = OS::TOTAL + 1024;
static_assert(2 * (OUT_TC_SMEM + 1024) <= 233472, "two output CTAs must fit one SM");

}  // namespace

// err: device status word (first failing bounded wait of the call is recorded there).
cudaError_t launch_chunk_output_tc(const RewyFwdArgs& a, int* err, cudaStream_t st) {
  const int B = a.B, T = a.T, H = a.H, NT = T / C;
  const uint64_t rows = (uint64_t)B * T, cols = (uint64_t)H * 128, pitch = (uint64_t)H * 256;
  const uint64_t srows = (uint64_t)B * NT * H * 128;
  CUtensorMap tm[5];
  const bool ok = encode_tmap_panels(&tm[0], a.h, 2, 128, srows, 256, 128, 2) &&
                  encode_tmap_panels(&tm[1], a.qg, 2, cols, rows, pitch, 64, 2) &&
                  encode_tmap_panels(&tm[2], a.v_new, 2, cols, rows, pitch, 64, 2) &&
                  encode_tmap_2d(&tm[3], a.Aqk, 2, (uint64_t)H * 64, rows, (uint64_t)H * 128, 64, 64) &&
                  encode_tmap_2d(&tm[4], a.o, 2, cols, rows, pitch, 128, 64, false);
  if (!ok) return cudaErrorInvalidValue;
  cudaError_t e = ensure_dynamic_smem<chunk_output_tc_kernel>(OUT_TC_SMEM);
  if (e != cudaSuccess) return e;
  OutParams p;
  p.err = err; p.T = T; p.H = H; p.NT = NT; p.total_chunks = B * H * NT; p.scale = a.scale;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int cap = 2 * sms;
  const int grid = p.total_chunks < cap ? p.total_chunks : cap;
  chunk_output_tc_kernel<<<grid, TPB, OUT_TC_SMEM, st>>>(tm[0], tm[1], tm[2], tm[3], tm[4], p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace rewy
