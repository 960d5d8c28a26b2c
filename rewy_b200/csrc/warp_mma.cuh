// CTA-level BF16 matrix products on shared-memory tiles with warp-level mma.sync (m16n8k16, FP32
// accumulate).  Used by the stages that are not on the tcgen05 path and as their cross-check.
#pragma once
#include "common.cuh"

namespace rewy {

// Operand view over a BF16 shared-memory tile.
//   TRANS == false: element (mn, k) at p[mn*ld + k]   (reduction index contiguous)
//   TRANS == true : element (mn, k) at p[k*ld + mn]   (reduction index strided)
// NEG flips the sign of every element as it is fetched.
template <bool TRANS, bool NEG = false>
struct Operand {
  static constexpr bool LDM = false;
  const bf16* p;
  int ld;
  __device__ __forceinline__ uint32_t pair(int mn, int k) const {  // elements (mn,k) and (mn,k+1)
    uint32_t u;
    if (!TRANS) {
      u = *reinterpret_cast<const uint32_t*>(p + mn * ld + k);
    } else {
      uint16_t lo = *reinterpret_cast<const uint16_t*>(p + k * ld + mn);
      uint16_t hi = *reinterpret_cast<const uint16_t*>(p + (k + 1) * ld + mn);
      u = (uint32_t)lo | ((uint32_t)hi << 16);
    }
    if (NEG) u ^= 0x80008000u;
    return u;
  }
};

// The same view, fetched with ldmatrix: four 8x8 BF16 matrices per instruction instead of one 32-bit (or two 16-bit)
// shared-memory loads per fragment register.  Requires p 16-byte aligned and ld a multiple of 8 elements.
template <bool TRANS, bool NEG = false>
struct LdmOperand {
  static constexpr bool LDM = true;
  static constexpr bool TRANSPOSED = TRANS;
  static constexpr bool NEGATE = NEG;
  const bf16* p;
  int ld;
};

template <bool TRANS>
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const bf16* at) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(at));
  if (TRANS)
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
  else
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Warp arrangement of a CTA-level product D[M x N] += A[M x KD] * B[KD x N].
// WM x WN warps (WM*WN == warps in the CTA), each warp owns an (M/WM) x (N/WN) sub-tile made of
// 16x8 fragments.  Accumulator element e of fragment (i, j) of the calling thread sits at
//   row = m0 + i*16 + (lane>>2) + (e>=2 ? 8 : 0),  col = n0 + j*8 + (lane&3)*2 + (e&1).
template <int M, int N, int WM, int WN>
struct Tile {
  static constexpr int TM = M / WM / 16;
  static constexpr int TN = N / WN / 8;
  static constexpr int REGS = TM * TN * 4;
  static_assert(M % (WM * 16) == 0 && N % (WN * 8) == 0, "tile does not divide");
  float acc[TM][TN][4];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
      for (int j = 0; j < TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;
  }
  __device__ __forceinline__ static int m0() { return ((threadIdx.x >> 5) / WN) * (M / WM); }
  __device__ __forceinline__ static int n0() { return ((threadIdx.x >> 5) % WN) * (N / WN); }
  __device__ __forceinline__ static int row(int i, int e) {
    return m0() + i * 16 + ((threadIdx.x & 31) >> 2) + ((e >> 1) << 3);
  }
  __device__ __forceinline__ static int col(int j, int e) { return n0() + j * 8 + ((threadIdx.x & 3) << 1) + (e & 1); }

  // ldmatrix operands.  Lane l of a warp supplies the address of one 8-element row of one of the four matrices of
  // an instruction (matrix l>>3, row l&7):
  //   A, m16 x k16:  a0 (m 0-7, k 0-7), a1 (m 8-15, k 0-7), a2 (m 0-7, k 8-15), a3 (m 8-15, k 8-15)
  //   B, two n8 x k16 fragments:  b[j][0] (k 0-7), b[j][1] (k 8-15), b[j+1][0], b[j+1][1]
  // A transposed view is stored [k][mn] and read with .trans, which hands every thread the same elements.
  template <int KD, class OA, class OB>
  __device__ __forceinline__ void mma_ldm(const OA& A, const OB& B) {
    static_assert(TN % 2 == 0, "B fragments are fetched two at a time");
    const int l = threadIdx.x & 31;
    const int rm = m0(), rn = n0();
    const bf16* pa = OA::TRANSPOSED ? A.p + ((l & 7) + (l >> 4) * 8) * A.ld + rm + ((l >> 3) & 1) * 8
                                    : A.p + (rm + (l & 7) + ((l >> 3) & 1) * 8) * A.ld + (l >> 4) * 8;
    const bf16* pb = OB::TRANSPOSED ? B.p + ((l & 7) + ((l >> 3) & 1) * 8) * B.ld + rn + (l >> 4) * 8
                                    : B.p + (rn + (l & 7) + (l >> 4) * 8) * B.ld + ((l >> 3) & 1) * 8;
    const int a_i = OA::TRANSPOSED ? 16 : 16 * A.ld, a_k = OA::TRANSPOSED ? A.ld : 1;
    const int b_j = OB::TRANSPOSED ? 16 : 16 * B.ld, b_k = OB::TRANSPOSED ? B.ld : 1;
#pragma unroll 2
    for (int k0 = 0; k0 < KD; k0 += 16) {
      uint32_t a[TM][4], b[TN][2];
#pragma unroll
      for (int i = 0; i < TM; i++) {
        ldmatrix_x4<OA::TRANSPOSED>(a[i], pa + i * a_i + k0 * a_k);
        if (OA::NEGATE) {
#pragma unroll
          for (int e = 0; e < 4; e++) a[i][e] ^= 0x80008000u;
        }
      }
#pragma unroll
      for (int j = 0; j < TN; j += 2) {
        uint32_t r[4];
        ldmatrix_x4<OB::TRANSPOSED>(r, pb + (j >> 1) * b_j + k0 * b_k);
        if (OB::NEGATE) {
#pragma unroll
          for (int e = 0; e < 4; e++) r[e] ^= 0x80008000u;
        }
        b[j][0] = r[0]; b[j][1] = r[1]; b[j + 1][0] = r[2]; b[j + 1][1] = r[3];
      }
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) mma_16816(acc[i][j], a[i], b[j]);
    }
  }

  template <int KD, class OA, class OB>
  __device__ __forceinline__ void mma(const OA& A, const OB& B) {
    if constexpr (OA::LDM && OB::LDM) {
      mma_ldm<KD>(A, B);
    } else {
      mma_lds<KD>(A, B);
    }
  }

  template <int KD, class OA, class OB>
  __device__ __forceinline__ void mma_lds(const OA& A, const OB& B) {
    const int g = (threadIdx.x & 31) >> 2, t = threadIdx.x & 3;
    const int rm = m0(), rn = n0();
#pragma unroll 2
    for (int k0 = 0; k0 < KD; k0 += 16) {
      uint32_t a[TM][4], b[TN][2];
#pragma unroll
      for (int i = 0; i < TM; i++) {
        int r = rm + i * 16 + g;
        a[i][0] = A.pair(r, k0 + 2 * t);
        a[i][1] = A.pair(r + 8, k0 + 2 * t);
        a[i][2] = A.pair(r, k0 + 2 * t + 8);
        a[i][3] = A.pair(r + 8, k0 + 2 * t + 8);
      }
#pragma unroll
      for (int j = 0; j < TN; j++) {
        int c = rn + j * 8 + g;
        b[j][0] = B.pair(c, k0 + 2 * t);
        b[j][1] = B.pair(c, k0 + 2 * t + 8);
      }
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) mma_16816(acc[i][j], a[i], b[j]);
    }
  }

  // f(row, col, value&) over every accumulator element of the calling thread.
  template <class F>
  __device__ __forceinline__ void for_each(F&& f) {
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
      for (int j = 0; j < TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) f(row(i, e), col(j, e), acc[i][j][e]);
  }
  // f(row, col, v0&, v1&) over adjacent column pairs (col even).
  template <class F>
  __device__ __forceinline__ void for_each_pair(F&& f) {
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
      for (int j = 0; j < TN; j++)
#pragma unroll
        for (int e = 0; e < 4; e += 2) f(row(i, e), col(j, e), acc[i][j][e], acc[i][j][e + 1]);
  }
};

}  // namespace rewy
