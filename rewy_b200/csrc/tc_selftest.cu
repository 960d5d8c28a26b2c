// Self-test of the tensor-core plumbing: one CTA runs each shared-memory operand form the backward stages use
// (TMA-written K-major and MN-major BF16 tiles, thread-written K-major and MN-major TF32 tiles, operand
// negation) through tcgen05.mma and writes the FP32 accumulators to global memory for comparison with a
// plain matrix product.  Exported as rewy_selftest_tensor_core (no counterpart in the reference).
#include <cstdio>
#include "tc05.cuh"

namespace rewy {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}
}  // namespace

bool encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                    uint32_t box_cols, uint32_t box_rows, bool swizzle128) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool encode_tmap_panels(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_rows, uint32_t panels) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const uint32_t box_cols = 128u / (uint32_t)elem_bytes;
  cuuint64_t dims[3] = {cols, rows, panels};
  cuuint64_t strides[2] = {pitch_bytes, 128};  // the panel index moves 128 bytes along the row
  cuuint32_t box[3] = {box_cols, box_rows, panels};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {
using namespace tc;

struct SelfTestSmem {
  alignas(1024) unsigned char a128[2][128 * 128];  // A [128 x 128] BF16, two 64-column panels
  alignas(1024) unsigned char b64[2][64 * 128];    // B [64 x 128] BF16, two panels
  alignas(1024) unsigned char akk[64 * 128];       // Akk [64 j x 64 i] BF16
  alignas(1024) unsigned char dr[2][64 * 128];     // dR [64 j x 128 v] BF16 two panels
  alignas(1024) unsigned char yf[2][128 * 128];    // Y [128 k x 64 j] FP32, two 32-column panels
  alignas(1024) unsigned char hf[2][64 * 128];     // H [64 i x 64 j] FP32, two 32-column panels
  uint64_t bar_in, bar_mma;
  uint32_t tmem_base;
};

__global__ void __launch_bounds__(128) selftest_kernel(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmAkk,
                                                       const __grid_constant__ CUtensorMap tmDR, const float* __restrict__ Y,
                                                       const float* __restrict__ Hm, float* __restrict__ out, int* err) {
  extern __shared__ __align__(1024) unsigned char raw[];
  SelfTestSmem& s = *reinterpret_cast<SelfTestSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&s.bar_in, 1);
    mbar_init(&s.bar_mma, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(&s.tmem_base, 512);
    tmem_relinquish();
  }
  // thread-written TF32 tiles: thread = row
  for (int j = 0; j < 64; j += 4) {
    float4 v = make_float4(round_tf32(Y[tid * 64 + j]), round_tf32(Y[tid * 64 + j + 1]), round_tf32(Y[tid * 64 + j + 2]),
                           round_tf32(Y[tid * 64 + j + 3]));
    *reinterpret_cast<float4*>(s.yf[j >> 5] + swz(tid, (j & 31) >> 2)) = v;
    if (tid < 64) {
      float4 w = make_float4(round_tf32(Hm[tid * 64 + j]), round_tf32(Hm[tid * 64 + j + 1]),
                             round_tf32(Hm[tid * 64 + j + 2]), round_tf32(Hm[tid * 64 + j + 3]));
      *reinterpret_cast<float4*>(s.hf[j >> 5] + swz(tid, (j & 31) >> 2)) = w;
    }
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tb = s.tmem_base;
  bool ok = true;
  if (tid == 0) {
    mbar_expect_tx(&s.bar_in, 2 * 128 * 128 + 2 * 64 * 128 + 64 * 128 + 2 * 64 * 128);
    for (int p = 0; p < 2; p++) {
      tma_load_2d(s.a128[p], &tmA, 64 * p, 0, &s.bar_in);
      tma_load_2d(s.b64[p], &tmB, 64 * p, 0, &s.bar_in);
      tma_load_2d(s.dr[p], &tmDR, 64 * p, 0, &s.bar_in);
    }
    tma_load_2d(s.akk, &tmAkk, 0, 0, &s.bar_in);
    ok = mbar_wait(&s.bar_in, 0, err, 1);
    if (ok) {
      tc_fence_after_sync();
      // T1: cols 0..63 = A B^T; T1n: cols 64..127 = (-A) B^T  (K-major BF16, K = 128)
      constexpr uint32_t id1 = instr_desc(FMT_BF16, 128, 64, false, false);
      constexpr uint32_t id1n = instr_desc(FMT_BF16, 128, 64, false, false, true, false);
      for (int ks = 0; ks < 8; ks++) {
        uint64_t ad = smem_desc(smem_u32(s.a128[ks >> 2]) + (ks & 3) * 32, 16, 1024);
        uint64_t bd = smem_desc(smem_u32(s.b64[ks >> 2]) + (ks & 3) * 32, 16, 1024);
        mma_f16(tb + 0, ad, bd, id1, ks > 0);
        mma_f16(tb + 64, ad, bd, id1n, ks > 0);
      }
      // T2: cols 128..255 = Akk^T dR (both MN-major BF16, K = 64, M padded to 128, N = 128)
      constexpr uint32_t id2 = instr_desc(FMT_BF16, 128, 128, true, true);
      for (int ks = 0; ks < 4; ks++) {
        uint64_t ad = smem_desc(smem_u32(s.akk) + ks * 2048, 8192, 1024);
        uint64_t bd = smem_desc(smem_u32(s.dr[0]) + ks * 2048, 8192, 1024);
        mma_f16(tb + 128, ad, bd, id2, ks > 0);
      }
      // T3: cols 256..319 = Y H^T (TF32, both K-major, K = 64).  (TF32 with an MN-major B operand produced zeros
      // on B200 and is not used.)
      constexpr uint32_t id3 = instr_desc(FMT_TF32, 128, 64, false, false);
      for (int ks = 0; ks < 8; ks++) {
        uint64_t ad = smem_desc(smem_u32(s.yf[ks >> 2]) + (ks & 3) * 32, 16, 1024);
        uint64_t bd = smem_desc(smem_u32(s.hf[ks >> 2]) + (ks & 3) * 32, 16, 1024);
        mma_tf32(tb + 256, ad, bd, id3, ks > 0);
      }
      // T4: cols 320..383 = B64 (as [k = 64 rows][n = 128]) ... BF16 B MN-major with a K-major A:
      //     out[m, n] = sum_r A[m, r] * Bt[r, n] for r < 64, n < 64, with Bt = first 64x64 block of B (n contiguous)
      constexpr uint32_t id4 = instr_desc(FMT_BF16, 128, 64, false, true);
      for (int ks = 0; ks < 4; ks++) {
        uint64_t ad = smem_desc(smem_u32(s.a128[0]) + ks * 32, 16, 1024);
        uint64_t bd = smem_desc(smem_u32(s.b64[0]) + ks * 2048, 8192, 1024);
        mma_f16(tb + 320, ad, bd, id4, ks > 0);
      }
      mma_commit(&s.bar_mma);
    }
  }
  ok = mbar_wait(&s.bar_mma, 0, err, 2);
  tc_fence_after_sync();
  if (ok && *reinterpret_cast<volatile int*>(err) == 0) {
    // out layout: [128 rows][384 columns]
    for (int c0 = 0; c0 < 384; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tb, warp * 32, c0), r);
      tmem_ld_wait();
      for (int j = 0; j < 32; j++) out[(size_t)tid * 384 + c0 + j] = __uint_as_float(r[j]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 512);
}

// Self-test of the give-up path of the bounded waits: every thread waits, with a short limit, for a phase of an
// mbarrier that nobody ever arrives on (no copy and no product is in flight), records the site, folds the per-thread
// flags exactly like the stages do and returns normally.
__global__ void bounded_wait_selftest_kernel(int* err, int* done, unsigned long long limit_ns, int site) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  bool alive = mbar_wait_limit(&bar, 0, err, site, limit_ns);
  alive = __syncthreads_and(alive ? 1 : 0) != 0;
  if (threadIdx.x == 0) *done = alive ? 1 : 2;  // 2: the wait ran out and the CTA left through the give-up path
}

}  // namespace
}  // namespace rewy

using namespace rewy;

extern "C" int rewy_selftest_bounded_wait(int* err, int* done, uint32_t limit_us, int site, rewy_stream_t stream) {
  if (err == nullptr || done == nullptr) return report_error(REWY_ERR_NULL, "err or done is NULL");
  if (limit_us == 0 || limit_us > 1000000u || site == 0)
    return report_error(REWY_ERR_UNSUPPORTED, "limit_us must be 1..1000000 and site non-zero");
  bounded_wait_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(err, done, (unsigned long long)limit_us * 1000ull, site);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? REWY_OK : REWY_ERR_LAUNCH;
}

// A [128x128] bf16, B [64x128] bf16, Akk [64x64] bf16, dR [64x128] bf16, Y [128x64] f32, H [64x64] f32 (row-major,
// device); out [128x384] f32: columns 0-63 A B^T, 64-127 -(A B^T), 128-255 rows 0-63 Akk^T dR, 256-319 Y H^T,
// 320-383 A[:, :64] B[:64, :64] (BF16, B MN-major).  err: device int, set non-zero if a bounded wait gave up.
extern "C" int rewy_selftest_tensor_core(const void* A, const void* B, const void* Akk, const void* dR, const float* Y,
                                         const float* H, float* out, int* err, rewy_stream_t stream) {
  CUtensorMap tmA, tmB, tmAkk, tmDR;
  if (!encode_tmap_2d(&tmA, A, 2, 128, 128, 256, 64, 128) || !encode_tmap_2d(&tmB, B, 2, 128, 64, 256, 64, 64) ||
      !encode_tmap_2d(&tmAkk, Akk, 2, 64, 64, 128, 64, 64) || !encode_tmap_2d(&tmDR, dR, 2, 128, 64, 256, 64, 64))
    return REWY_ERR_LAUNCH;
  const size_t smem = sizeof(SelfTestSmem) + 1024;
  if (cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return REWY_ERR_LAUNCH;
  selftest_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(tmA, tmB, tmAkk, tmDR, Y, H, out, err);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? REWY_OK : REWY_ERR_LAUNCH;
}
