/*
 * rewy_b200 — C ABI of the B200-native chunked delta-rule backward.
 *
 * One shared library (librewy_b200.so, sm_100a) exports the whole-family backward functions
 * that the reference's four autograd backwards call, plus the stage functions they are made of.
 * Every pointer is a DEVICE pointer to a contiguous token-major tensor; the library never
 * allocates, frees or synchronises; all work is enqueued on the stream that is passed in.
 * Fixed envelope (the reference's release envelope, src/fast_delta_rule/runtime.py:75-106):
 * K = V = 128, chunk = 64, T a positive multiple of 64, equal q/k/v head counts.
 *
 * Layouts (element offsets):
 *   [B,T,H,D]      ((b*T + t)*H + h)*D + d            q,k,v,do,w,u,qg,kg,v_new,dR,b_gate,w_gate and gradients
 *   [B,T,H,64]     ((b*T + t)*H + h)*64 + j           Aqk, Akk: row t%64, column j of the chunk's 64x64 matrix
 *   [B,T,H]        (b*T + t)*H + h                    beta, scalar gate, dbeta
 *   [B,NT,H,K,V]   (((b*NT + n)*H + h)*128 + k)*128+v h, dh (NT = T/64)
 *   [B,H,K,V]      ((b*H + h)*128 + k)*128 + v        initial_state, dht, dh0 ([B,H,V,K] with state_v_first)
 * Gates are chunk-local inclusive cumulative sums in LOG2 units (FP32), as the forward saves them.
 */
#ifndef REWY_B200_H
#define REWY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* rewy_stream_t; /* a cudaStream_t */

/* Envelope: T a positive multiple of 64, B*H (or num_seqs*H) <= 65535, and B*T*H at most this many token-heads
 * (tile coordinates are 32-bit: the rows of the [B,NT,H,128,128] state tensors are 2*B*T*H).  Larger problems are
 * REWY_ERR_SHAPE; 180 GB of device memory hold far fewer. */
#define REWY_MAX_TOKEN_HEADS (1LL << 29)

enum {
  REWY_OK = 0,
  REWY_ERR_NULL = 1,       /* a required pointer is NULL */
  REWY_ERR_SHAPE = 2,      /* B,T,H outside the envelope */
  REWY_ERR_ALIGN = 3,      /* a pointer is not 16-byte aligned */
  REWY_ERR_WORKSPACE = 4,  /* workspace smaller than rewy_bwd_workspace_bytes() */
  REWY_ERR_LAUNCH = 5,     /* a CUDA launch or API call failed */
  REWY_ERR_DEVICE = 6,     /* a kernel gave up on a bounded wait (see rewy_read_device_status) */
  REWY_ERR_UNSUPPORTED = 7 /* family/policy/flag combination not supported */
};

enum { REWY_DELTA = 0, REWY_GDN = 1, REWY_KDA = 2, REWY_GDN2 = 3 };
enum { REWY_RECOMPUTE = 0, REWY_SAVED = 1 };
enum { REWY_OUT_BF16 = 0, REWY_OUT_F32 = 1 };

/* Arguments of one whole-family backward.  Unused pointers are NULL. */
typedef struct RewyBwdArgs {
  int32_t family;      /* REWY_DELTA / REWY_GDN / REWY_KDA / REWY_GDN2 */
  int32_t policy;      /* REWY_RECOMPUTE: w,qg,kg,v_new,h are rebuilt; REWY_SAVED: they are passed in */
  int32_t B, T, H;
  int32_t out_dtype;   /* dtype of dq, dk (and db_gate, dw_gate): REWY_OUT_BF16 or REWY_OUT_F32 */
  int32_t intra_passes;/* 0 = default.  Option of chunk variant 1 (warp-MMA kernel) only: 1 or 3 BF16 split passes of
                          the matrix-intra products; the tensor-core kernel always runs 3 and refuses other values */
  int32_t state_v_first; /* 0: h0, dht, dh0 are [B,H,K,V]; 1: they are [B,H,V,K] (FLA's state_v_first / transposed state
                            layout).  The per-chunk states h and dh keep the [K,V] layout either way: they are produced and
                            consumed inside this library (its own forward saves h). */
  float scale;
  /* inputs */
  const void* q;       /* bf16 [B,T,H,128] */
  const void* k;       /* bf16 [B,T,H,128] */
  const void* v;       /* bf16 [B,T,H,128] */
  const float* g;      /* fp32 log2 cumsum: [B,T,H,128] (KDA, GDN2), [B,T,H] (GDN), NULL (DeltaNet) */
  const float* beta;   /* fp32 [B,T,H] (DeltaNet, GDN, KDA), NULL (GDN2) */
  const void* b_gate;  /* bf16 [B,T,H,128] erase gate (GDN2 only) */
  const void* w_gate;  /* bf16 [B,T,H,128] write gate (GDN2 only) */
  const void* Aqk;     /* bf16 [B,T,H,64] (KDA, GDN2); NULL for DeltaNet/GDN (rebuilt) */
  const void* Akk;     /* bf16 [B,T,H,64] */
  const float* h0;     /* fp32 [B,H,128,128] or NULL */
  const void* d_o;     /* bf16 [B,T,H,128] gradient of the output */
  const float* dht;    /* fp32 [B,H,128,128] gradient of the final state, or NULL */
  /* saved forward tensors (policy REWY_SAVED, KDA/GDN2 only) */
  const void* w;       /* bf16 [B,T,H,128] = Akk (b*k*gamma) */
  const void* qg;      /* bf16 [B,T,H,128] = q*gamma */
  const void* kg;      /* bf16 [B,T,H,128] = k*exp2(g_last - g) */
  const void* v_new;   /* bf16 [B,T,H,128] */
  const void* h;       /* bf16 [B,T/64,H,128,128] state entering each chunk */
  /* outputs */
  void* dq;            /* out_dtype [B,T,H,128] */
  void* dk;            /* out_dtype [B,T,H,128] */
  void* dv;            /* bf16 [B,T,H,128] */
  float* dg;           /* fp32, shape of g; NULL for DeltaNet */
  float* dbeta;        /* fp32 [B,T,H]; NULL for GDN2 */
  void* db_gate;       /* out_dtype [B,T,H,128] (GDN2) */
  void* dw_gate;       /* out_dtype [B,T,H,128] (GDN2) */
  float* dh0;          /* fp32 [B,H,128,128] or NULL (must be non-NULL iff h0 is) */
  /* packed sequences (FLA's cu_seqlens): device int32 [num_seqs + 1] token offsets into a batch with B = 1, or NULL.
   * Every sequence length must be a multiple of 64 (chunks never straddle sequences; a kernel that finds another
   * length records it in the status word and leaves its sequence untouched); h0, dht and dh0 are then
   * [num_seqs,H,128,128].  Only the two state scans look at sequence boundaries. */
  const int32_t* cu_seqlens;
  int32_t num_seqs;
  /* scratch */
  void* workspace;
  size_t workspace_bytes;
} RewyBwdArgs;

/* Inter-stage tensors; the whole-family functions carve them out of the workspace (or alias the
 * saved tensors), the stage functions take them explicitly so each stage can be driven alone. */
typedef struct RewyStageBuffers {
  void* w;      /* bf16 [B,T,H,128] */
  void* u;      /* bf16 [B,T,H,128]   (prepare -> forward scan only) */
  void* qg;     /* bf16 [B,T,H,128] */
  void* kg;     /* bf16 [B,T,H,128] */
  void* v_new;  /* bf16 [B,T,H,128] */
  void* h;      /* bf16 [B,NT,H,128,128] */
  void* Aqk;    /* bf16 [B,T,H,64] */
  void* dh;     /* bf16 [B,NT,H,128,128] */
  void* dR;     /* bf16 [B,T,H,128]  high part of dR = kg dh + Aqk^T dO */
  void* dR_lo;  /* bf16 [B,T,H,128]  low part: bf16(dR - dR_hi); P = Akk^T (dR + dR_lo) keeps dv, dbeta inside 2e-3 */
  void* ctrl;   /* int32 [2 + B*H*T/64] control block of the chunk stage: [0] device status word, [1] number of
                   chunks whose gate span was too wide for the centred products, [2..] their indices */
} RewyStageBuffers;

/* Whole-family backward.  Replace, one for one, the functions the reference's autograd backwards call:
 *   rewy_kda_bwd    <- chunk_kda_bwd            as bound at src/fast_delta_rule/_compat/kda.py:169-201
 *                      (implemented by backends/backward.py:63-73, kda_backward)
 *   rewy_gdn2_bwd   <- chunk_gdn2_bwd           _compat/gdn2.py:145-171 (backends/backward.py:75-81)
 *   rewy_gdn_bwd    <- chunk_gated_delta_rule_bwd  _compat/gdn.py:240-260 (backends/backward.py:133-134)
 *   rewy_delta_bwd  <- chunk_delta_rule_bwd     _compat/delta.py:125-138 (backends/backward.py:136-137)
 * Return REWY_OK or an error code; rewy_last_error() gives the text. */
int rewy_kda_bwd(const RewyBwdArgs* args, rewy_stream_t stream);
int rewy_gdn2_bwd(const RewyBwdArgs* args, rewy_stream_t stream);
int rewy_gdn_bwd(const RewyBwdArgs* args, rewy_stream_t stream);
int rewy_delta_bwd(const RewyBwdArgs* args, rewy_stream_t stream);

/* Bytes of workspace a whole-family call needs (the reference's orchestrators allocate the same
 * intermediates with torch: FLA chunk_kda_bwd stages 1-5, cf. backends/backward.py:15-43,96-131). */
size_t rewy_bwd_workspace_bytes(int32_t family, int32_t policy, int32_t B, int32_t T, int32_t H);

/* Stage functions.
 *   rewy_stage_prepare  <- FLA recompute_w_u_fwd (+ Aqk rebuild for the scalar families), called at
 *                          backends/backward.py:116 and inside FLA chunk_kda_bwd/chunk_gdn2_bwd
 *   rewy_stage_fwd_scan <- FLA chunk_gated_delta_rule_fwd_h, backends/backward.py:117-118
 *   rewy_stage_bwd_scan <- chunk_gated_delta_rule_bwd_dhu (FLA; kernels/vector_state_gpu.py:47-67 for GDN2)
 *                          fused with chunk_kda_bwd_dAv's dv = Aqk^T dO / chunk_bwd_dv_local (backward.py:119-121)
 *   rewy_stage_chunk_adjoint <- residual WY + matrix intra + reverse gate cumsum:
 *                          kernels/kda_residual_local_beta.py:8-23, kernels/endpoint_intra.py:306-326,
 *                          kernels/gdn2_consumer_fp32.py:76-98, kernels/scalar_liveness_gpu.py:87-102,
 *                          FLA chunk_local_cumsum(reverse=True)
 */
int rewy_stage_prepare(const RewyBwdArgs* args, const RewyStageBuffers* buf, rewy_stream_t stream);
int rewy_stage_fwd_scan(const RewyBwdArgs* args, const RewyStageBuffers* buf, rewy_stream_t stream);
int rewy_stage_bwd_scan(const RewyBwdArgs* args, const RewyStageBuffers* buf, rewy_stream_t stream);
int rewy_stage_chunk_adjoint(const RewyBwdArgs* args, const RewyStageBuffers* buf, rewy_stream_t stream);

/* Forward pass.  rewy_chunk_fwd replaces FLA's chunk_kda_fwd / chunk_gdn2_fwd / chunk_gated_delta_rule_fwd /
 * chunk_delta_rule_fwd as the reference's autograd forwards call them (src/fast_delta_rule/_compat/kda.py:89-113,
 * gdn2.py:94-117, gdn.py:33-125, delta.py): from q, k, v, the cumulative gate and beta (or the two vector gates) it
 * writes the output o, the final state and the whole saved set of the backward.  Three launches on the stream: the
 * chunk-local kernel (Akk, Aqk, w, u, qg, kg), the forward state scan (h, v_new, final state) and the output kernel.
 * g is the chunk-local cumulative gate in log2 units (rewy_gate_cumsum_fwd / rewy_scalar_gate_cumsum_fwd write it).
 * Every output pointer except final_state is required; ctrl is an int32[2] control block whose first word is the
 * device status word (rewy_device_status). */
typedef struct RewyFwdArgs {
  int32_t family;          /* REWY_DELTA / REWY_GDN / REWY_KDA / REWY_GDN2 */
  int32_t B, T, H;
  int32_t state_v_first;   /* h0 and final_state are [B,H,V,K] instead of [B,H,K,V] */
  float scale;
  const void* q;           /* bf16 [B,T,H,128] */
  const void* k;           /* bf16 [B,T,H,128] */
  const void* v;           /* bf16 [B,T,H,128] */
  const float* g;          /* fp32 log2 cumsum: [B,T,H,128] (KDA, GDN2), [B,T,H] (GDN), NULL (DeltaNet) */
  const float* beta;       /* fp32 [B,T,H] (DeltaNet, GDN, KDA), NULL (GDN2) */
  const void* b_gate;      /* bf16 [B,T,H,128] (GDN2) */
  const void* w_gate;      /* bf16 [B,T,H,128] (GDN2) */
  const float* h0;         /* fp32 [B,H,128,128] or NULL */
  void* o;                 /* bf16 [B,T,H,128] */
  float* final_state;      /* fp32 [B,H,128,128] or NULL */
  void* Aqk;               /* bf16 [B,T,H,64] */
  void* Akk;               /* bf16 [B,T,H,64] */
  void* w;                 /* bf16 [B,T,H,128] */
  void* u;                 /* bf16 [B,T,H,128] */
  void* qg;                /* bf16 [B,T,H,128] */
  void* kg;                /* bf16 [B,T,H,128] */
  void* v_new;             /* bf16 [B,T,H,128] */
  void* h;                 /* bf16 [B,T/64,H,128,128] */
  void* ctrl;              /* int32 [2] */
  const int32_t* cu_seqlens; /* packed sequences, as in RewyBwdArgs (h0, final_state [num_seqs,H,128,128]); or NULL */
  int32_t num_seqs;
} RewyFwdArgs;
int rewy_chunk_fwd(const RewyFwdArgs* args, rewy_stream_t stream);
/* Output kernel of the forward: 0 (default) TMA + tcgen05, 1 warp-MMA (cross-check).  Process-wide. */
int rewy_set_forward_variant(int variant);
/* Chunk-local cumulative sum in log2 units of a scalar per-head gate x [B,T,H] (BF16 or FP32), FLA chunk_local_cumsum
 * as used by chunk_gated_delta_rule_fwd (_compat/gdn.py:52-69). */
int rewy_scalar_gate_cumsum_fwd(const void* x, int x_is_f32, float* g_cumsum, int32_t B, int32_t T, int32_t H,
                                rewy_stream_t stream);

/* Element-wise stages of the autograd wrappers (one HBM pass each; rows = B*T*H rows of 128 values).
 *   rewy_l2norm_fwd / _bwd       <- FLA l2norm_fwd / l2norm_bwd as used at src/fast_delta_rule/_compat/kda.py:56-59,202-204
 *                                   (same in _compat/gdn.py, gdn2.py, delta.py).  x, y BF16 [rows,128]; rstd FP32 [rows];
 *                                   dy BF16 or FP32 (the dq/dk of the family backward); dx BF16: the cast to the input
 *                                   dtype (_compat/kda.py:208) is part of the same pass.
 *   rewy_beta_sigmoid_fwd / _bwd <- fused_beta_sigmoid / fused_beta_sigmoid_bwd, _compat/kda.py:61-63,205-206.
 *                                   x raw logits (BF16 or FP32) [n]; forward writes scale*sigmoid(x) as FP32 (y32) and/or
 *                                   BF16 (y16; then y32 holds the BF16-rounded value); backward dx FP32 [n].
 *   rewy_gate_cumsum_fwd         <- FLA chunk_local_cumsum(scale=RCP_LN2) and, with A_log != NULL, kda_gate_chunk_cumsum
 *                                   (chunk_kda_fwd with use_gate_in_kernel, _compat/kda.py:89-113): the per-step gate
 *                                   g = -exp(A_log[h]) * softplus(x + dt_bias[h*128+k]) (dt_bias may be NULL) is written to
 *                                   g_act (optional) and its chunk-local inclusive cumulative sum in log2 units to g_cumsum.
 *                                   x [B,T,H,128] BF16 or FP32; A_log FP32 [H]; dt_bias FP32 [H*128].
 *   rewy_gate_act_bwd            <- FLA kda_gate_bwd (chunk_kda_bwd with use_gate_in_kernel): dg is the gradient of the
 *                                   activated per-step gate; dx FP32 [B,T,H,128]; per-chunk partial sums
 *                                   dA_part FP32 [B*T/64*H] and dbias_part FP32 [B*T/64*H*128] whose sums over the leading
 *                                   (batch, chunk) index are dA_log[h] and ddt_bias[h*128+k]. */
int rewy_l2norm_fwd(const void* x, void* y, float* rstd, int64_t rows, float eps, rewy_stream_t stream);
int rewy_l2norm_bwd(const void* y, const float* rstd, const void* dy, int dy_is_f32, void* dx, int64_t rows,
                    rewy_stream_t stream);
int rewy_beta_sigmoid_fwd(const void* x, int x_is_f32, float* y32, void* y16, int64_t n, float scale, rewy_stream_t stream);
int rewy_beta_sigmoid_bwd(const void* x, int x_is_f32, const float* dy, float* dx, int64_t n, float scale,
                          rewy_stream_t stream);
int rewy_gate_cumsum_fwd(const void* x, int x_is_f32, const float* A_log, const float* dt_bias, float* g_cumsum,
                         float* g_act, int32_t B, int32_t T, int32_t H, rewy_stream_t stream);
int rewy_gate_act_bwd(const void* x, int x_is_f32, const float* A_log, const float* dt_bias, const float* dg, float* dx,
                      float* dA_part, float* dbias_part, int32_t B, int32_t T, int32_t H, rewy_stream_t stream);

/* Optional per-stage device timing of the whole-family calls (no counterpart in the reference, which
 * times stages by re-capturing them: research/operators/a800_ablation/audit.py:38-47).  While enabled, each
 * whole-family call records CUDA events on its stream around its stage launches (up to 256 calls).
 * rewy_stage_timing_read sums the elapsed milliseconds per stage {prepare, forward scan, reverse scan,
 * chunk adjoint} over the recorded calls; the stream must have been synchronised by the caller. */
int rewy_stage_timing_enable(int enable);
int rewy_stage_timing_read(float* ms_sum4, int* calls);

/* Control block.  A whole-family call keeps it at offset 0 of its workspace; the stage function takes it in
 * RewyStageBuffers.ctrl.  rewy_device_status copies the status word to the host (this call SYNCHRONISES the
 * stream) and returns REWY_ERR_DEVICE if a kernel gave up on a bounded wait; rewy_wide_chunk_count returns how
 * many chunks took the exact pairwise path (the analogue of the reference's per-tile fallback flags,
 * kernels/endpoint_intra.py:301-304), or -1 on error.  No counterpart in the reference for the status word. */
int rewy_device_status(const void* ctrl, rewy_stream_t stream);
int rewy_wide_chunk_count(const void* ctrl, rewy_stream_t stream);

/* Chunk stage for hosts that cannot allocate device memory.  It has no counterpart in the reference (whose
 * orchestrators allocate every intermediate with torch).  Same inputs, outputs and arithmetic as
 * rewy_stage_chunk_adjoint (always the tensor-core kernel), but the control block is NOT taken from
 * RewyStageBuffers.ctrl (that field is ignored): it is an array inside the library, one copy per device,
 * large enough for REWY_STATIC_MAX_CHUNKS = 65536 chunks (B*H*T/64; 256 KB of device memory that every GPU
 * which loads the library holds until the process exits).  Meant for callers that run out of a device arena
 * they carved up front and therefore have nothing to allocate the block with: a C/C++ host without a caching
 * allocator, or a job whose memory plan leaves no room for allocations after start-up.  The call makes no
 * cudaMalloc/cudaFree and no allocating library call.
 *  - Calls with more than REWY_STATIC_MAX_CHUNKS chunks are refused with REWY_ERR_SHAPE.
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device
 *    current); make that first call outside of any stream capture.
 *  - All calls on one device share the one array, and it keeps the previous call's contents; each call clears
 *    the two words that must start at zero.  Two calls whose kernels may overlap on the GPU (different
 *    streams) race on it - serialise them.
 *  - The array's device address is cached per device at that first call; a cudaDeviceReset invalidates it (the
 *    library must be reloaded afterwards).
 *  - The host-side checks are those of rewy_stage_chunk_adjoint (shape envelope, every pointer non-NULL and 16-byte
 *    aligned), so a misaligned pointer is REWY_ERR_ALIGN before anything is launched.
 * rewy_static_device_status reads the array's status word on the current device (SYNCHRONISES the stream). */
#define REWY_STATIC_MAX_CHUNKS 65536
int rewy_stage_chunk_adjoint_static(const RewyBwdArgs* args, const RewyStageBuffers* buf, rewy_stream_t stream);
int rewy_static_device_status(rewy_stream_t stream);

/* Kernel variant of the chunk stage: 0 (default) tensor-core kernel, 1 warp-MMA kernel on every chunk
 * (cross-check).  Process-wide; no counterpart in the reference. */
int rewy_set_chunk_variant(int variant);
/* Same for the reverse state scan: 0 (default) tensor-core kernel (needs RewyStageBuffers.ctrl for its status
 * word; without it the stage function uses the warp-MMA kernel), 1 warp-MMA kernel. */
int rewy_set_scan_variant(int variant);
/* Under the recompute policy (and always for the scalar families) the forward state scan and the reverse state scan are
 * independent; by default (1) a whole-family call with at most 148 (sequence, head) pairs enqueues the forward scan on a side stream of the library (one
 * non-blocking stream and two events per host thread and device, created at the first such call) that forks from and joins the
 * caller's stream through events, so the two scans run concurrently and the call stays capturable in a CUDA graph.
 * 0 keeps every stage on the caller's stream.  Process-wide; no counterpart in the reference. */
int rewy_set_scan_overlap(int enable);
/* Same for the prepare stage: 0 (default) the faster kernel per family as measured on B200 (TMA + tcgen05 for DeltaNet,
 * GDN and KDA, warp-MMA for GDN2), 1 warp-MMA kernel, 2 TMA + tcgen05 kernel.  The tcgen05 kernel needs
 * RewyStageBuffers.ctrl for its status word; without it the stage function uses the warp-MMA kernel. */
int rewy_set_prepare_variant(int variant);

/* Self-test of the tensor-core plumbing (no counterpart in the reference): one CTA pushes every shared-memory
 * operand form the stages use through tcgen05.mma.  Inputs row-major on the device: A [128x128] bf16,
 * B [64x128] bf16, Akk [64x64] bf16, dR [64x128] bf16, Y [128x64] f32, H [64x64] f32.  out [128x384] f32:
 * columns 0-63 A B^T, 64-127 -(A B^T), 128-255 (rows 0-63) Akk^T dR, 256-319 Y H^T (TF32),
 * 320-383 A[:, :64] B[:64, :64] (BF16 with B read MN-major).
 * err: device int, non-zero if a bounded wait inside the kernel gave up. */
int rewy_selftest_tensor_core(const void* A, const void* B, const void* Akk, const void* dR, const float* Y,
                              const float* H, float* out, int* err, rewy_stream_t stream);

/* Self-test of the failure path (no counterpart in the reference): one CTA waits, for at most limit_us
 * microseconds (1..1000000), on an mbarrier phase that nothing completes - no copy or product is in flight - then
 * records `site` (non-zero) in *err exactly as the stages do, writes 2 to *done (1 if the wait had succeeded) and
 * returns normally.  err, done: device ints, zero on entry.  rewy_device_status(err, stream) then reports
 * REWY_ERR_DEVICE. */
int rewy_selftest_bounded_wait(int* err, int* done, uint32_t limit_us, int site, rewy_stream_t stream);

/* Diagnostics. */
const char* rewy_last_error(void);       /* thread-local text of the last non-zero status */
const char* rewy_version(void);
int rewy_kernel_launch_count(void);      /* kernels launched by this library in this process so far */

#ifdef __cplusplus
}
#endif
#endif /* REWY_B200_H */
