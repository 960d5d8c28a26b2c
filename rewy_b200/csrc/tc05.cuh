// Blackwell (sm_100a) plumbing used by the tensor-core stages: mbarriers with bounded waits, TMA tile
// loads (every CTA fetches its own tiles), tcgen05 MMA with TMEM accumulators, shared-memory matrix descriptors.
#pragma once
#include <cuda.h>
#include <cstring>
#include "common.cuh"

namespace rewy {
namespace tc {

// ---- error word ------------------------------------------------------------------------------
// A wait that gives up records where it was and the kernel carries on to its exit path; the host reads
// the word after the launch.  Nothing here traps or spins without a bound.
constexpr unsigned long long WAIT_LIMIT_NS = 400ull * 1000 * 1000;  // give up on a phase after 0.4 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code` in *err, first failing site wins) if the phase has not completed
// after limit_ns nanoseconds of %globaltimer.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int* err, int code, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) break;
  }
  if (err != nullptr) atomicCAS(err, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err, int code) {
  return mbar_wait_limit(bar, parity, err, code, WAIT_LIMIT_NS);
}

// One lane of a fully active warp (used inside warp-uniform branches, so that the operands of the single-thread
// instructions issued under it stay warp-uniform values).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- proxies and fences ------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA -------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared of the box the tensor map was encoded with; c0 is the innermost coordinate
// (must keep c0 * element size a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async group of the issuing thread).  The shared tile must have been
// written (generic proxy), fenced with fence_async_smem() and made visible by a barrier before this is issued.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until every committed store group of this thread has finished READING shared memory.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// 3-D tiled load (see encode_tmap_panels: the third coordinate walks over 128-byte column panels of the same rows).
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// ---- TMEM ------------------------------------------------------------------------------------
// Allocation is warp-wide (all 32 lanes execute it); ncols is a power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// TMEM address = (lane << 16) | column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}
// 32 lanes x 32 consecutive columns: thread t of the warp gets lane (lane_base + t), r[j] = column (col + j).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor (sm_100 format): start address, leading/stride byte offsets in 16-byte
// units, version 1, 128-byte swizzle.  Tiles are stored as rows of 128 bytes, 8 rows per 1024-byte swizzle
// atom, base 1024-byte aligned (exactly what a TMA box with 128-byte inner extent and SWIZZLE_128B writes):
//   K-major operand  (reduction index contiguous):  rows = M/N index;  SBO = 1024 (next 8 rows), LBO unused.
//     A K=16 (BF16) / K=8 (TF32) step advances the start address by 32 bytes inside the 128-byte row;
//     the next 128 bytes of the reduction dimension live in the next panel.
//   MN-major operand (M/N index contiguous): rows = reduction index; SBO = 1024 (next 8 reduction rows),
//     LBO = byte distance between panels of 64 (BF16) / 32 (TF32) M/N elements.
//     A K=16 step covers two 8-row atoms: the start address advances by 2048 bytes (1024 for TF32 K=8).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

enum { FMT_F16 = 0, FMT_BF16 = 1, FMT_TF32 = 2 };
// Instruction descriptor for kind::f16 / kind::tf32 with FP32 accumulation.
__host__ __device__ constexpr uint32_t instr_desc(int fmt, int M, int N, bool a_mn_major, bool b_mn_major,
                                                  bool neg_a = false, bool neg_b = false) {
  return (1u << 4)                     // D format F32
         | ((uint32_t)fmt << 7)        // A format
         | ((uint32_t)fmt << 10)       // B format
         | ((neg_a ? 1u : 0u) << 13) | ((neg_b ? 1u : 0u) << 14)
         | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16)
         | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// The same instruction with both descriptors given as (low, high) words.  For the fixed tile plan of a kernel the
// high word is a constant and the low word is "tile base >> 4" plus a compile-time offset, so that issuing a
// product costs the single thread that does it a couple of integer adds per instruction instead of rebuilding
// two 64-bit descriptors.
constexpr uint32_t DESC_HI_SW128 = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);  // SBO 1024 B, version 1, SWIZZLE_128B
// low word of the descriptor of a tile at shared address `saddr` (below 256 KB) with leading byte offset `lbo`
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo_bytes) { return (saddr >> 4) | ((lbo_bytes >> 4) << 16); }
__device__ __forceinline__ void mma_f16_lo(uint32_t d_tmem, uint32_t alo, uint32_t blo, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(alo), "r"(blo), "r"(idesc), "r"((uint32_t)accumulate), "r"(DESC_HI_SW128)
      : "memory");
}
// A operand in tensor memory: row m of A is TMEM lane m, element k sits in column a_tmem + k / 2 (two BF16 per 32-bit
// column, even k in the low half), exactly as a thread that owns lane m writes it with tcgen05.st; B from shared memory.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t blo, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(blo), "r"(idesc), "r"((uint32_t)accumulate), "r"(DESC_HI_SW128)
      : "memory");
}
// Arrive on an mbarrier when every MMA issued so far by this thread has completed (implies
// tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Byte offset of element chunk (row r, 16-byte chunk c) inside a 128-byte-swizzled panel of 128-byte rows.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

// Round an FP32 value to the nearest TF32 (10-bit mantissa) so that the tensor core's truncation is exact.
__device__ __forceinline__ float round_tf32(float x) {
  uint32_t u = __float_as_uint(x);
  u = (u + 0x1000u) & 0xFFFFE000u;
  return __uint_as_float(u);
}

}  // namespace tc

// Host side: encode a 2-D tiled tensor map (row-major tensor of `rows` x `cols` elements, `pitch_bytes` between
// rows) whose box is box_cols x box_rows with 128-byte swizzle (or, with swizzle128 = false, dense rows of box_cols
// elements).  Returns false if the driver entry point is
// unavailable or the encode fails.
bool encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                    uint32_t box_cols, uint32_t box_rows, bool swizzle128 = true);

// Same tensor seen as `panels` column panels of 128 bytes each: one load of the box (128 bytes x box_rows x panels)
// at coordinates (first column, first row, 0) writes the panels one after the other, each as box_rows rows of 128
// swizzled bytes - the operand layout of a K extent (or an MN extent) wider than one swizzle atom.
bool encode_tmap_panels(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_rows, uint32_t panels);

// Host-side cache of encoded tensor maps, one instance per launcher and host thread.  A call whose key (the pointers
// and the shape the maps depend on, as raw bytes) matches one of the last SLOTS calls reuses the encoded maps, so
// repeated launches on the same buffers (training steps, benchmark loops, graph re-captures) cost no driver calls.
template <int N, int KEY_BYTES, int SLOTS = 4>
struct TmapCache {
  struct Entry {
    unsigned char key[KEY_BYTES];
    CUtensorMap tm[N];
    bool valid = false;
  } entry[SLOTS];
  int next = 0;
  const CUtensorMap* find(const void* key) const {
    for (int i = 0; i < SLOTS; i++)
      if (entry[i].valid && memcmp(entry[i].key, key, KEY_BYTES) == 0) return entry[i].tm;
    return nullptr;
  }
  // the slot to encode into; call commit(key) once every map of the slot has been encoded
  CUtensorMap* slot() {
    entry[next].valid = false;
    return entry[next].tm;
  }
  void commit(const void* key) {
    memcpy(entry[next].key, key, KEY_BYTES);
    entry[next].valid = true;
    next = (next + 1) % SLOTS;
  }
};

}  // namespace rewy
