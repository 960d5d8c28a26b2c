// C ABI of the library: argument validation, workspace carving and stage sequencing.
// No allocation, no synchronisation; every launch goes to the caller's stream.
#include <atomic>
#include <cstdio>
#include <cstring>
#include "common.cuh"

namespace rewy {
namespace {

thread_local char g_error[512] = "";
std::atomic<int> g_launches{0};

int fail(int code, const char* fmt, const char* what = "", long long x = 0) {
  snprintf(g_error, sizeof(g_error), fmt, what, x);
  return code;
}

size_t align_up(size_t x) { return (x + 255) & ~size_t(255); }

struct Plan {
  bool prepare;       // rebuild w,u,qg,kg (+ forward scan for v_new,h)
  bool build_aqk;     // scalar families save no Aqk
  size_t off_ctrl, off_dh, off_dR, off_dRlo, off_w, off_u, off_qg, off_kg, off_vnew, off_h, off_aqk, total;
};

Plan make_plan(int family, int policy, long long B, long long T, long long H) {
  Plan p{};
  const size_t n = (size_t)B * T * H;  // token-heads
  p.build_aqk = family == REWY_DELTA || family == REWY_GDN;
  p.prepare = p.build_aqk || policy == REWY_RECOMPUTE;
  size_t o = 0;
  p.off_ctrl = o; o += align_up(sizeof(int) * (size_t)(2 + B * H * (T / C)));
  p.off_dh = o; o += align_up(n * 512);
  p.off_dR = o; o += align_up(n * 256);
  p.off_dRlo = o; o += align_up(n * 256);
  if (p.prepare) {
    p.off_w = o; o += align_up(n * 256);
    p.off_u = o; o += align_up(n * 256);
    p.off_qg = o; o += align_up(n * 256);
    p.off_kg = o; o += align_up(n * 256);
    p.off_vnew = o; o += align_up(n * 256);
    p.off_h = o; o += align_up(n * 512);
  }
  if (p.build_aqk) { p.off_aqk = o; o += align_up(n * 128); }
  p.total = o;
  return p;
}

bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

#define REQUIRE_PTR(name)                                                                  \
  do {                                                                                     \
    if (a->name == nullptr) return fail(REWY_ERR_NULL, "required pointer '%s' is NULL", #name); \
    if (misaligned(a->name)) return fail(REWY_ERR_ALIGN, "pointer '%s' is not 16-byte aligned", #name); \
  } while (0)
#define OPTIONAL_PTR(name)                                                                 \
  do {                                                                                     \
    if (a->name != nullptr && misaligned(a->name))                                         \
      return fail(REWY_ERR_ALIGN, "pointer '%s' is not 16-byte aligned", #name);           \
  } while (0)

std::atomic<int> g_chunk_variant{0};  // 0 = tensor-core kernel (+ pairwise list), 1 = warp-MMA kernel everywhere
std::atomic<int> g_scan_variant{0};   // 0 = tensor-core scans, 1 = warp-MMA scans

// intra_passes is an option of the warp-MMA chunk kernel (1 or 3 split passes); the tensor-core kernel always runs 3.
int rc_passes(int passes) {
  const bool warp_variant = g_chunk_variant.load(std::memory_order_relaxed) == 1;
  if (passes == 0 || passes == 3 || (passes == 1 && warp_variant)) return REWY_OK;
  return fail(REWY_ERR_UNSUPPORTED,
              warp_variant ? "intra_passes must be 0, 1 or 3%s" : "intra_passes must be 0 or 3 with the tensor-core chunk kernel%s");
}

int validate_common(const RewyBwdArgs* a, int family) {
  if (a == nullptr) return fail(REWY_ERR_NULL, "args is NULL%s");
  if (a->family != family) return fail(REWY_ERR_UNSUPPORTED, "args->family does not match the entry point%s");
  if (a->policy != REWY_RECOMPUTE && a->policy != REWY_SAVED) return fail(REWY_ERR_UNSUPPORTED, "unknown policy%s");
  if (a->out_dtype != REWY_OUT_BF16 && a->out_dtype != REWY_OUT_F32)
    return fail(REWY_ERR_UNSUPPORTED, "unknown out_dtype%s");
  if ((rc_passes(a->intra_passes)) != REWY_OK) return REWY_ERR_UNSUPPORTED;
  if (a->state_v_first != 0 && a->state_v_first != 1) return fail(REWY_ERR_UNSUPPORTED, "state_v_first must be 0 or 1%s");
  if (a->state_v_first && g_scan_variant.load(std::memory_order_relaxed) == 1)
    return fail(REWY_ERR_UNSUPPORTED, "the warp-MMA scan variant reads [K,V] states only (state_v_first)%s");
  if (a->B <= 0 || a->H <= 0) return fail(REWY_ERR_SHAPE, "B and H must be positive%s");
  if (a->cu_seqlens != nullptr) {
    if (a->B != 1 || a->num_seqs <= 0) return fail(REWY_ERR_SHAPE, "packed sequences need B = 1 and num_seqs > 0%s");
    if ((long long)a->num_seqs * a->H > 65535) return fail(REWY_ERR_SHAPE, "num_seqs*H exceeds the grid limit 65535%s");
    if (g_scan_variant.load(std::memory_order_relaxed) == 1)
      return fail(REWY_ERR_UNSUPPORTED, "the warp-MMA scan variant does not take packed sequences%s");
  }
  if (a->T < C || a->T % C != 0) return fail(REWY_ERR_SHAPE, "T must be a positive multiple of 64 (got %s%lld)", "", a->T);
  if ((long long)a->B * a->H > 65535) return fail(REWY_ERR_SHAPE, "B*H exceeds the grid limit 65535%s");
  if ((long long)a->B * a->T * a->H > REWY_MAX_TOKEN_HEADS)
    return fail(REWY_ERR_SHAPE, "B*T*H exceeds 2^29 token-heads (32-bit tile coordinates)%s");
  REQUIRE_PTR(q); REQUIRE_PTR(k); REQUIRE_PTR(v); REQUIRE_PTR(Akk); REQUIRE_PTR(d_o);
  REQUIRE_PTR(dq); REQUIRE_PTR(dk); REQUIRE_PTR(dv);
  OPTIONAL_PTR(h0); OPTIONAL_PTR(dht); OPTIONAL_PTR(dh0);
  if (family == REWY_DELTA) {
    if (a->g != nullptr || a->dg != nullptr) return fail(REWY_ERR_UNSUPPORTED, "DeltaNet takes no gate%s");
  } else {
    REQUIRE_PTR(g); REQUIRE_PTR(dg);
  }
  if (family == REWY_GDN2) {
    REQUIRE_PTR(b_gate); REQUIRE_PTR(w_gate); REQUIRE_PTR(db_gate); REQUIRE_PTR(dw_gate);
  } else {
    REQUIRE_PTR(beta); REQUIRE_PTR(dbeta);
  }
  if (family == REWY_KDA || family == REWY_GDN2) {
    REQUIRE_PTR(Aqk);
    if (a->policy == REWY_SAVED) { REQUIRE_PTR(w); REQUIRE_PTR(qg); REQUIRE_PTR(kg); REQUIRE_PTR(v_new); REQUIRE_PTR(h); }
  } else if (a->policy == REWY_SAVED) {
    return fail(REWY_ERR_UNSUPPORTED, "the scalar-gate families always recompute (no saved WY tensors)%s");
  }
  return REWY_OK;
}

// Optional per-stage device timing of the whole-family calls (off by default): a ring of CUDA-event sets,
// one set per call, recorded on the caller's stream between the stage launches.
constexpr int TIMING_SETS = 256;
constexpr int TIMING_STAGES = 4;  // prepare, forward scan, reverse scan, chunk adjoint
struct Timing {
  bool enabled = false;
  int used = 0;
  cudaEvent_t ev[TIMING_SETS][TIMING_STAGES + 1];
  bool have[TIMING_SETS][TIMING_STAGES + 1];
  bool created = false;
} g_timing;

void timing_mark(int set, int idx, cudaStream_t st) {
  if (set < 0) return;
  cudaEventRecord(g_timing.ev[set][idx], st);
  g_timing.have[set][idx] = true;
}

std::atomic<int> g_prepare_variant{0};  // 0 = by measurement, 1 = warp-MMA kernel, 2 = TMA + tcgen05 kernel

// Default choice, by measurement on B200: the TMA + tcgen05 kernel for DeltaNet, GDN and KDA (0.83 ms against 0.91 ms at
// KDA B=8 T=8192 H=32); for GDN2, whose chunk reads seven operand tiles, the warp-MMA kernel with four CTAs per SM
// keeps more loads in flight and is faster (4.2 ms against 5.3 ms at B=8 T=32768 H=32).
cudaError_t run_prepare(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  const int variant = g_prepare_variant.load(std::memory_order_relaxed);
  const bool warp = variant == 1 || s.ctrl == nullptr || (variant == 0 && a.family == REWY_GDN2);
  if (warp) return launch_prepare(a, s, st);
  return launch_prepare_tc(a, s, static_cast<int*>(s.ctrl), st);
}

cudaError_t run_fwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  const bool warp_variant = g_scan_variant.load(std::memory_order_relaxed) == 1 || s.ctrl == nullptr;
  if (warp_variant && (a.cu_seqlens != nullptr || a.state_v_first)) return cudaErrorNotSupported;  // tcgen05 scans only
  if (warp_variant) return launch_fwd_scan(a, s, st);
  return launch_fwd_scan_tc(a, s, static_cast<int*>(s.ctrl), st);
}

cudaError_t run_bwd_scan(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  const bool warp_variant = g_scan_variant.load(std::memory_order_relaxed) == 1 || s.ctrl == nullptr;
  if (warp_variant && (a.cu_seqlens != nullptr || a.state_v_first)) return cudaErrorNotSupported;  // tcgen05 scans only
  if (warp_variant) return launch_bwd_scan(a, s, st);
  return launch_bwd_scan_tc(a, s, static_cast<int*>(s.ctrl), st);
}

// The status word is zeroed ONCE per call, before its first stage: every kernel records a give-up with
// atomicCAS(word, 0, site), so the first failing site of the call is what the host reads afterwards.
cudaError_t clear_status(void* ctrl, cudaStream_t st) {
  return ctrl == nullptr ? cudaSuccess : cudaMemsetAsync(ctrl, 0, sizeof(int), st);
}

cudaError_t run_chunk_adjoint(const RewyBwdArgs& a, const RewyStageBuffers& s, cudaStream_t st) {
  if (g_chunk_variant.load(std::memory_order_relaxed) == 1) {
    if (s.ctrl != nullptr) {  // keep the control block readable: no wide chunks
      cudaError_t e = cudaMemsetAsync(static_cast<int*>(s.ctrl) + 1, 0, sizeof(int), st);
      if (e != cudaSuccess) return e;
    }
    return launch_chunk_adjoint_warp(a, s, nullptr, st);
  }
  return launch_chunk_adjoint_tc(a, s, static_cast<int*>(s.ctrl), st);
}

// Side stream and the two events of the fork/join around the forward scan: one set per host thread and device, created
// at first use and kept for the life of the thread (host-side handles only, no device memory).  Per-thread sets keep
// two host threads that drive the same device from waiting on each other's events.
struct ForkJoin {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ready = false, failed = false;
};
std::atomic<int> g_overlap_scans{1};  // 1: forward scan on a side stream, concurrent with the reverse scan
thread_local ForkJoin g_fork_join[64];

ForkJoin* fork_join_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  ForkJoin& f = g_fork_join[dev];
  if (!f.ready && !f.failed) {
    f.failed = cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking) != cudaSuccess ||
               cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming) != cudaSuccess ||
               cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming) != cudaSuccess;
    f.ready = !f.failed;
  }
  return f.ready ? &f : nullptr;
}

int check_cuda(cudaError_t e, const char* stage) {
  if (e == cudaSuccess) return REWY_OK;
  snprintf(g_error, sizeof(g_error), "%s: %s", stage, cudaGetErrorString(e));
  return REWY_ERR_LAUNCH;
}

int run_family(const RewyBwdArgs* a, int family, cudaStream_t st) {
  int rc = validate_common(a, family);
  if (rc != REWY_OK) return rc;
  const Plan p = make_plan(family, a->policy, a->B, a->T, a->H);
  if (a->workspace == nullptr) return fail(REWY_ERR_NULL, "required pointer '%s' is NULL", "workspace");
  if (misaligned(a->workspace)) return fail(REWY_ERR_ALIGN, "pointer '%s' is not 16-byte aligned", "workspace");
  if (a->workspace_bytes < p.total)
    return fail(REWY_ERR_WORKSPACE, "workspace too small: need %s%lld bytes", "", (long long)p.total);
  char* ws = static_cast<char*>(a->workspace);
  RewyStageBuffers s{};
  s.ctrl = ws + p.off_ctrl;
  s.dh = ws + p.off_dh;
  s.dR = ws + p.off_dR;
  s.dR_lo = ws + p.off_dRlo;
  if (p.prepare) {
    s.w = ws + p.off_w; s.u = ws + p.off_u; s.qg = ws + p.off_qg; s.kg = ws + p.off_kg;
    s.v_new = ws + p.off_vnew; s.h = ws + p.off_h;
  } else {
    s.w = const_cast<void*>(a->w); s.qg = const_cast<void*>(a->qg); s.kg = const_cast<void*>(a->kg);
    s.v_new = const_cast<void*>(a->v_new); s.h = const_cast<void*>(a->h);
  }
  s.Aqk = p.build_aqk ? static_cast<void*>(ws + p.off_aqk) : const_cast<void*>(a->Aqk);
  int set = -1;
  if (g_timing.enabled && g_timing.used < TIMING_SETS) {
    set = g_timing.used++;
    for (int i = 0; i <= TIMING_STAGES; i++) g_timing.have[set][i] = false;
  }
  if ((rc = check_cuda(clear_status(s.ctrl, st), "status word")) != REWY_OK) return rc;
  timing_mark(set, 0, st);
  if (p.prepare) {
    // Without a gate qg = q and kg = k: the prepare stage writes neither and the scans read the inputs themselves
    const bool gateless = a->family == REWY_DELTA;
    if (gateless) s.qg = s.kg = nullptr;
    if ((rc = check_cuda(run_prepare(*a, s, st), "prepare")) != REWY_OK) return rc;
    if (gateless) {
      s.qg = const_cast<void*>(a->q);
      s.kg = const_cast<void*>(a->k);
    }
    timing_mark(set, 1, st);
    // The forward scan (h, v_new: read by the chunk stage) and the reverse scan (reads qg, kg, w of the prepare stage
    // only) do not depend on each other: the forward scan goes to a side stream and joins before the chunk stage.  One
    // CTA of each fits an SM together (shared memory and TMEM), so two latency-bound chains share the machine.
    // Worth it while both kernels together leave SMs idle (at most one CTA per SM each); at larger sizes both are bound
    // by HBM and running them together gains nothing.
    const long long scan_ctas = (long long)(a->cu_seqlens != nullptr ? a->num_seqs : a->B) * a->H;
    ForkJoin* fj = g_overlap_scans.load(std::memory_order_relaxed) && scan_ctas <= 148 ? fork_join_for_current_device() : nullptr;
    if (fj != nullptr) {
      cudaError_t e = cudaEventRecord(fj->fork, st);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(fj->side, fj->fork, 0);
      if (e == cudaSuccess) e = run_fwd_scan(*a, s, fj->side);
      if (e == cudaSuccess) e = cudaEventRecord(fj->join, fj->side);
      if ((rc = check_cuda(e, "forward state scan (side stream)")) != REWY_OK) return rc;
      timing_mark(set, 2, st);
      e = run_bwd_scan(*a, s, st);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(st, fj->join, 0);
      if ((rc = check_cuda(e, "reverse state scan")) != REWY_OK) return rc;
    } else {
      if ((rc = check_cuda(run_fwd_scan(*a, s, st), "forward state scan")) != REWY_OK) return rc;
      timing_mark(set, 2, st);
      if ((rc = check_cuda(run_bwd_scan(*a, s, st), "reverse state scan")) != REWY_OK) return rc;
    }
  } else {
    timing_mark(set, 2, st);
    if ((rc = check_cuda(run_bwd_scan(*a, s, st), "reverse state scan")) != REWY_OK) return rc;
  }
  timing_mark(set, 3, st);
  if ((rc = check_cuda(run_chunk_adjoint(*a, s, st), "chunk adjoint")) != REWY_OK) return rc;
  timing_mark(set, 4, st);
  return REWY_OK;
}

int validate_stage(const RewyBwdArgs* a, const RewyStageBuffers* s) {
  if (a == nullptr || s == nullptr) return fail(REWY_ERR_NULL, "args or buffers is NULL%s");
  if (a->family < REWY_DELTA || a->family > REWY_GDN2) return fail(REWY_ERR_UNSUPPORTED, "unknown family%s");
  if (a->B <= 0 || a->H <= 0 || a->T < C || a->T % C != 0) return fail(REWY_ERR_SHAPE, "bad B/T/H%s");
  if ((long long)a->B * a->H > 65535) return fail(REWY_ERR_SHAPE, "B*H exceeds the grid limit 65535%s");
  if ((long long)a->B * a->T * a->H > REWY_MAX_TOKEN_HEADS)
    return fail(REWY_ERR_SHAPE, "B*T*H exceeds 2^29 token-heads (32-bit tile coordinates)%s");
  if (a->cu_seqlens != nullptr && (a->B != 1 || a->num_seqs <= 0 || (long long)a->num_seqs * a->H > 65535))
    return fail(REWY_ERR_SHAPE, "packed sequences need B = 1 and 0 < num_seqs*H <= 65535%s");
  return REWY_OK;
}

#define STAGE_PTR(expr, name)                                                               \
  do {                                                                                      \
    if ((expr) == nullptr) return fail(REWY_ERR_NULL, "required pointer '%s' is NULL", name); \
    if (misaligned(expr)) return fail(REWY_ERR_ALIGN, "pointer '%s' is not 16-byte aligned", name); \
  } while (0)

}  // namespace

// Host-side validation of a chunk-stage call (shape envelope, every pointer present and 16-byte aligned);
// shared by rewy_stage_chunk_adjoint and rewy_stage_chunk_adjoint_static.
int validate_chunk_stage(const RewyBwdArgs* a, const RewyStageBuffers* s, bool need_ctrl) {
  int rc = validate_stage(a, s);
  if (rc != REWY_OK) return rc;
  if (a->out_dtype != REWY_OUT_BF16 && a->out_dtype != REWY_OUT_F32) return fail(REWY_ERR_UNSUPPORTED, "unknown out_dtype%s");
  if (rc_passes(a->intra_passes) != REWY_OK) return REWY_ERR_UNSUPPORTED;
  STAGE_PTR(a->q, "q"); STAGE_PTR(a->k, "k"); STAGE_PTR(a->v, "v"); STAGE_PTR(a->Akk, "Akk"); STAGE_PTR(a->d_o, "d_o");
  STAGE_PTR(s->v_new, "v_new"); STAGE_PTR(s->h, "h"); STAGE_PTR(s->dh, "dh"); STAGE_PTR(s->dR, "dR");
  STAGE_PTR(s->dR_lo, "dR_lo");
  if (need_ctrl) STAGE_PTR(s->ctrl, "ctrl");
  STAGE_PTR(a->dq, "dq"); STAGE_PTR(a->dk, "dk"); STAGE_PTR(a->dv, "dv");
  if (a->family != REWY_DELTA) { STAGE_PTR(a->g, "g"); STAGE_PTR(a->dg, "dg"); }
  if (a->family == REWY_GDN2) {
    STAGE_PTR(a->b_gate, "b_gate"); STAGE_PTR(a->w_gate, "w_gate"); STAGE_PTR(a->db_gate, "db_gate");
    STAGE_PTR(a->dw_gate, "dw_gate");
  } else {
    STAGE_PTR(a->beta, "beta"); STAGE_PTR(a->dbeta, "dbeta");
  }
  return REWY_OK;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int report_error(int code, const char* text) {
  snprintf(g_error, sizeof(g_error), "%s", text);
  return code;
}

}  // namespace rewy

using namespace rewy;

extern "C" {

int rewy_kda_bwd(const RewyBwdArgs* a, rewy_stream_t st) { return run_family(a, REWY_KDA, (cudaStream_t)st); }
int rewy_gdn2_bwd(const RewyBwdArgs* a, rewy_stream_t st) { return run_family(a, REWY_GDN2, (cudaStream_t)st); }
int rewy_gdn_bwd(const RewyBwdArgs* a, rewy_stream_t st) { return run_family(a, REWY_GDN, (cudaStream_t)st); }
int rewy_delta_bwd(const RewyBwdArgs* a, rewy_stream_t st) { return run_family(a, REWY_DELTA, (cudaStream_t)st); }

size_t rewy_bwd_workspace_bytes(int32_t family, int32_t policy, int32_t B, int32_t T, int32_t H) {
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  return make_plan(family, policy, B, T, H).total;
}

int rewy_stage_prepare(const RewyBwdArgs* a, const RewyStageBuffers* s, rewy_stream_t st) {
  int rc = validate_stage(a, s);
  if (rc != REWY_OK) return rc;
  STAGE_PTR(a->q, "q"); STAGE_PTR(a->k, "k"); STAGE_PTR(a->v, "v"); STAGE_PTR(a->Akk, "Akk");
  STAGE_PTR(s->w, "w"); STAGE_PTR(s->u, "u"); STAGE_PTR(s->qg, "qg"); STAGE_PTR(s->kg, "kg");
  if (a->family != REWY_DELTA) STAGE_PTR(a->g, "g");
  if (a->family == REWY_GDN2) { STAGE_PTR(a->b_gate, "b_gate"); STAGE_PTR(a->w_gate, "w_gate"); }
  else STAGE_PTR(a->beta, "beta");
  if (a->family == REWY_DELTA || a->family == REWY_GDN) STAGE_PTR(s->Aqk, "Aqk");
  if ((rc = check_cuda(clear_status(s->ctrl, (cudaStream_t)st), "status word")) != REWY_OK) return rc;
  return check_cuda(run_prepare(*a, *s, (cudaStream_t)st), "prepare");
}

int rewy_stage_fwd_scan(const RewyBwdArgs* a, const RewyStageBuffers* s, rewy_stream_t st) {
  int rc = validate_stage(a, s);
  if (rc != REWY_OK) return rc;
  STAGE_PTR(s->kg, "kg"); STAGE_PTR(s->w, "w"); STAGE_PTR(s->u, "u"); STAGE_PTR(s->h, "h"); STAGE_PTR(s->v_new, "v_new");
  if (a->family != REWY_DELTA) STAGE_PTR(a->g, "g");
  if ((rc = check_cuda(clear_status(s->ctrl, (cudaStream_t)st), "status word")) != REWY_OK) return rc;
  return check_cuda(run_fwd_scan(*a, *s, (cudaStream_t)st), "forward state scan");
}

int rewy_stage_bwd_scan(const RewyBwdArgs* a, const RewyStageBuffers* s, rewy_stream_t st) {
  int rc = validate_stage(a, s);
  if (rc != REWY_OK) return rc;
  STAGE_PTR(s->qg, "qg"); STAGE_PTR(s->kg, "kg"); STAGE_PTR(s->w, "w"); STAGE_PTR(s->Aqk, "Aqk");
  STAGE_PTR(a->d_o, "d_o"); STAGE_PTR(s->dh, "dh"); STAGE_PTR(s->dR, "dR"); STAGE_PTR(s->dR_lo, "dR_lo");
  if (a->family != REWY_DELTA) STAGE_PTR(a->g, "g");
  if ((rc = check_cuda(clear_status(s->ctrl, (cudaStream_t)st), "status word")) != REWY_OK) return rc;
  return check_cuda(run_bwd_scan(*a, *s, (cudaStream_t)st), "reverse state scan");
}

int rewy_stage_chunk_adjoint(const RewyBwdArgs* a, const RewyStageBuffers* s, rewy_stream_t st) {
  int rc = validate_chunk_stage(a, s, g_chunk_variant.load(std::memory_order_relaxed) != 1);
  if (rc != REWY_OK) return rc;
  // standalone stage call: start from a clean status word
  if ((rc = check_cuda(clear_status(s->ctrl, (cudaStream_t)st), "status word")) != REWY_OK) return rc;
  return check_cuda(run_chunk_adjoint(*a, *s, (cudaStream_t)st), "chunk adjoint");
}

int rewy_stage_timing_enable(int enable) {
  if (enable && !g_timing.created) {
    for (int i = 0; i < TIMING_SETS; i++)
      for (int j = 0; j <= TIMING_STAGES; j++)
        if (cudaEventCreate(&g_timing.ev[i][j]) != cudaSuccess) return fail(REWY_ERR_LAUNCH, "cudaEventCreate failed%s");
    g_timing.created = true;
  }
  g_timing.enabled = enable != 0;
  g_timing.used = 0;
  return REWY_OK;
}

int rewy_stage_timing_read(float* ms_sum, int* calls) {
  if (ms_sum == nullptr || calls == nullptr) return fail(REWY_ERR_NULL, "ms_sum or calls is NULL%s");
  for (int j = 0; j < TIMING_STAGES; j++) ms_sum[j] = 0.f;
  *calls = g_timing.used;
  for (int i = 0; i < g_timing.used; i++) {
    // stage j runs between mark j and the next recorded mark
    int prev = 0;
    for (int j = 1; j <= TIMING_STAGES; j++) {
      if (!g_timing.have[i][j]) continue;
      float ms = 0.f;
      cudaError_t e = cudaEventElapsedTime(&ms, g_timing.ev[i][prev], g_timing.ev[i][j]);
      if (e != cudaSuccess) return check_cuda(e, "stage timing (synchronise the stream first)");
      ms_sum[j - 1] += ms;
      prev = j;
    }
  }
  return REWY_OK;
}

int rewy_set_scan_variant(int variant) {
  if (variant != 0 && variant != 1) return fail(REWY_ERR_UNSUPPORTED, "scan variant must be 0 or 1%s");
  g_scan_variant.store(variant, std::memory_order_relaxed);
  return REWY_OK;
}

int rewy_set_scan_overlap(int enable) {
  g_overlap_scans.store(enable != 0, std::memory_order_relaxed);
  return REWY_OK;
}

int rewy_set_prepare_variant(int variant) {
  if (variant < 0 || variant > 2) return fail(REWY_ERR_UNSUPPORTED, "prepare variant must be 0, 1 or 2%s");
  g_prepare_variant.store(variant, std::memory_order_relaxed);
  return REWY_OK;
}

int rewy_set_chunk_variant(int variant) {
  if (variant != 0 && variant != 1) return fail(REWY_ERR_UNSUPPORTED, "chunk variant must be 0 or 1%s");
  g_chunk_variant.store(variant, std::memory_order_relaxed);
  return REWY_OK;
}

int rewy_device_status(const void* ctrl, rewy_stream_t st) {
  if (ctrl == nullptr) return fail(REWY_ERR_NULL, "required pointer '%s' is NULL", "ctrl");
  int word[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(word, ctrl, sizeof(word), cudaMemcpyDeviceToHost, (cudaStream_t)st);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)st);
  if (e != cudaSuccess) return check_cuda(e, "device status read");
  if (word[0] != 0) return fail(REWY_ERR_DEVICE, "a kernel gave up on a bounded wait at site %s%lld", "", word[0]);
  return REWY_OK;
}

int rewy_wide_chunk_count(const void* ctrl, rewy_stream_t st) {
  if (ctrl == nullptr) return -1;
  int word[2] = {0, 0};
  cudaError_t e = cudaMemcpyAsync(word, ctrl, sizeof(word), cudaMemcpyDeviceToHost, (cudaStream_t)st);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)st);
  return e == cudaSuccess ? word[1] : -1;
}

const char* rewy_last_error(void) { return g_error; }
const char* rewy_version(void) { return "rewy_b200 0.1.0 (sm_100a)"; }
int rewy_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
