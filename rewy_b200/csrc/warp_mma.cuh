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

  template <int KD, class OA, class OB>
  __device__ __forceinline__ void mma(const OA& A, const OB& B) {
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
