#!/usr/bin/env python
"""Times the reference's own Triton backward for KDA on the current GPU, stage by stage.

    python baseline/triton_reference.py [--batch 8] [--seq 8192] [--heads 32] [--steps 10] [--warmup 3]
                                        [--policy saved|recompute] [--dump PATH]

The reference (fast-delta-rule) is taken UNMODIFIED from ``baseline/_ref`` (``pip install --target``); its Triton
kernels are the residual-WY producer/consumer (kernels/kda_residual_local_beta.py:8-23) and the endpoint matrix
intra (kernels/endpoint_intra.py:306-326), bound into FLA's ``chunk_kda_bwd`` orchestrator exactly as
backends/backward.py:18-29 does (FunctionType clone with overridden globals).  The reference pins
flash-linear-attention at commit a59bc5df...; the FLA that is installed here is a different release, so three
adaptations are needed and every one is listed in the JSON this prints ("adaptations"):
  * ``fla.utils.IS_NVIDIA_SM100`` (imported by the consumer kernel, absent from this FLA) is set from the device's
    compute capability;
  * ``fla.ops.utils.op.unflatten_program_id`` (imported by the intra kernel, absent from this FLA) is supplied as
    ``(pid % n, pid // n)`` of program axis 0 - any bijection over the flattened (tile, chunk) grid gives the same
    result, only the launch order of the tiles could differ;
  * this FLA's wrapper passes the kernel keyword TRANSPOSE_STATE and no USE_GRAPH; they are renamed / defaulted to the
    STATE_V_FIRST / USE_GRAPH keywords the reference's launcher reads.
The other stages (dAv, the reverse state scan, the final reverse cumsum; recompute_w_u_fwd and the forward scan under
the recompute policy) are this FLA's stock Triton kernels, as in the reference.  Also timed: this FLA's stock
``chunk_kda_bwd`` ("fla_original"), the baseline the reference reports its speed-ups against.
Inputs are the synthetic benchmark tensors and the saved set of this repository's forward.  Timing: CUDA events on the
current stream, warm-up first (Triton compiles and autotunes there), one JSON line on stdout.
GDN2 (no ``fla.ops.gdn2`` in this FLA) and the scalar families (the reference's ``_scalar`` passes ``state_v_first`` to
FLA functions that do not take it here) are reported as not assembled, not substituted.
"""
import argparse
import importlib
import json
import sys
import warnings
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"


def unavailable(why):
    print(json.dumps({"unavailable": why}), flush=True)
    return 0


def load_reference():
    """Import the reference's kernels from baseline/_ref against the installed FLA; returns (modules, adaptations)."""
    import torch
    import triton
    import triton.language as tl
    adaptations = []
    import fla.utils as fu
    if not hasattr(fu, "IS_NVIDIA_SM100"):
        fu.IS_NVIDIA_SM100 = torch.cuda.get_device_capability()[0] == 10
        adaptations.append("fla.utils.IS_NVIDIA_SM100 set from the device capability")
    import fla.ops.utils.op as fop
    if not hasattr(fop, "unflatten_program_id"):
        @triton.jit
        def unflatten_program_id(n):
            pid = tl.program_id(0)
            return pid % n, pid // n
        fop.unflatten_program_id = unflatten_program_id
        adaptations.append("fla.ops.utils.op.unflatten_program_id supplied as (pid % n, pid // n)")
    sys.path.insert(0, str(REF))
    from fast_delta_rule.backends.backward import _clone
    from fast_delta_rule.kernels.kda_residual_local_beta import LocalBetaResidual
    from fast_delta_rule.kernels.endpoint_intra import EndpointMatrixIntra
    return _clone, LocalBetaResidual, EndpointMatrixIntra, adaptations


class KeywordAdapter:
    """Stands where FLA's ``chunk_kda_bwd_kernel_wy_dqkg_fused`` stands (kernel[grid](**kw)) and forwards to the
    reference's two-kernel launcher with the keyword names that launcher reads."""

    def __init__(self, inner):
        self.inner = inner

    def __getitem__(self, grid):
        launch = self.inner[grid]

        def run(**kw):
            kw = dict(kw)
            if "TRANSPOSE_STATE" in kw:
                kw["STATE_V_FIRST"] = kw.pop("TRANSPOSE_STATE")
            kw.setdefault("USE_GRAPH", False)
            return launch(**kw)
        return run


class StageTimer:
    """Wraps a stage function of the orchestrator with CUDA events on the current stream."""

    def __init__(self):
        self.events = {}
        self.enabled = False

    def wrap(self, name, fn):
        import torch

        def timed(*a, **k):
            if not self.enabled:
                return fn(*a, **k)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **k)
            e1.record()
            self.events.setdefault(name, []).append((e0, e1))
            return out
        return timed

    def read(self, calls):
        return {n: sum(a.elapsed_time(b) for a, b in ev) / max(calls, 1) for n, ev in self.events.items()}


def build_backwards():
    """Returns (reference_bwd, fla_bwd, timer, adaptations): the reference's optimized KDA backward assembled on the
    installed FLA, and FLA's stock one."""
    _clone, LocalBetaResidual, EndpointMatrixIntra, adaptations = load_reference()
    base = importlib.import_module("fla.ops.kda.chunk_bwd")
    adaptations.append("kernel keywords TRANSPOSE_STATE -> STATE_V_FIRST, USE_GRAPH defaulted to False")
    timer = StageTimer()
    intra = EndpointMatrixIntra(base.chunk_kda_bwd_intra, base.chunk_kda_bwd_intra, True)
    wy = _clone(base.chunk_kda_bwd_wy_dqkg_fused,
                dict(chunk_kda_bwd_kernel_wy_dqkg_fused=KeywordAdapter(LocalBetaResidual())))
    overrides = dict(
        chunk_kda_bwd_wy_dqkg_fused=timer.wrap("residual_wy (reference K1+K2)", wy),
        chunk_kda_bwd_intra=timer.wrap("matrix_intra (reference K3)", intra),
        chunk_kda_bwd_dAv=timer.wrap("dAv (FLA)", base.chunk_kda_bwd_dAv),
        chunk_gated_delta_rule_bwd_dhu=timer.wrap("bwd_dhu (FLA)", base.chunk_gated_delta_rule_bwd_dhu),
        chunk_local_cumsum=timer.wrap("reverse cumsum (FLA)", base.chunk_local_cumsum),
        recompute_w_u_fwd=timer.wrap("recompute_w_u (FLA)", base.recompute_w_u_fwd),
        chunk_gated_delta_rule_fwd_h=timer.wrap("fwd_h (FLA)", base.chunk_gated_delta_rule_fwd_h),
    )
    reference_bwd = _clone(base.chunk_kda_bwd, overrides)
    reference_bwd._fdr_intra = intra
    return reference_bwd, base.chunk_kda_bwd, timer, adaptations


def make_problem(B, T, H, device, seed=42, gate_scale=0.1, state=False):
    import torch
    sys.path.insert(0, str(ROOT))
    from rewy_b200.forward import chunk_forward
    from rewy_b200.synthetic import make_inputs
    xs = make_inputs("kda", B, T, H, seed=seed, device=device, gate_scale=gate_scale, state=state)
    sv = chunk_forward("kda", xs["q"], xs["k"], xs["v"], g=xs["g"], beta=xs["beta"], initial_state=xs["initial_state"],
                       output_final_state=False)
    return xs, sv


def call_kwargs(xs, sv, saved):
    kw = dict(q=xs["q"], k=xs["k"], v=xs["v"], beta=xs["beta"], Aqk=sv["Aqk"], Akk=sv["Akk"], scale=128 ** -0.5,
              initial_state=xs["initial_state"], do=xs["do"], dht=xs["dht"], g=sv["g_cumsum"], disable_recompute=saved)
    if saved:
        kw.update(w=sv["w"], u=sv["u"], qg=sv["qg"], kg=sv["kg"], v_new=sv["v_new"], h=sv["h"])
    return kw


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--policy", default="saved", choices=("saved", "recompute"))
    args = ap.parse_args()
    warnings.filterwarnings("ignore")
    if not (REF / "fast_delta_rule").is_dir():
        return unavailable("baseline/_ref holds no installed reference (pip install --target baseline/_ref)")
    try:
        import torch
        import triton  # noqa: F401
        import fla
    except Exception as exc:
        return unavailable(f"triton / flash-linear-attention not importable: {exc}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    try:
        reference_bwd, fla_bwd, timer, adaptations = build_backwards()
    except Exception as exc:
        return unavailable(f"the reference's kernels do not import against FLA {fla.__version__}: {type(exc).__name__}: {exc}")
    dev = torch.device("cuda", torch.cuda.current_device())
    B, T, H = args.batch, args.seq, args.heads
    xs, sv = make_problem(B, T, H, dev)
    saved = args.policy == "saved"
    kw = call_kwargs(xs, sv, saved)
    out = {"workload": f"KDA backward B={B} T={T} H={H} K=V=128 chunk=64, policy {args.policy}",
           "fla_version": fla.__version__, "triton_version": importlib.import_module("triton").__version__,
           "reference_fla_pin": "a59bc5df8c5841dce2169bb00e4027287197ba77 (not installed; version-skewed run)",
           "adaptations": adaptations,
           "not_assembled": {
               "gdn2": "the installed FLA has no fla.ops.gdn2 (orchestrator, forward and dAv are missing)",
               "gdn, delta": "the reference's _scalar binding passes state_v_first to FLA functions that take "
                             "transpose_state_layout in this release"},
           "steps": args.steps, "warmup": args.warmup}

    def time_arm(fn, name, with_stages):
        try:
            for _ in range(max(args.warmup, 1)):
                fn(**kw)
            torch.cuda.synchronize()
            timer.events.clear()
            timer.enabled = with_stages
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn(**kw)
            e1.record()
            torch.cuda.synchronize()
            timer.enabled = False
            ms = e0.elapsed_time(e1) / args.steps
            r = {"ms": ms, "tokens_per_s": B * T / (ms * 1e-3)}
            if with_stages:
                r["stages_ms"] = timer.read(args.steps)
            return r
        except Exception as exc:  # a kernel that fails to compile or launch is reported, not retried
            timer.enabled = False
            return {"unavailable": f"{name}: {type(exc).__name__}: {str(exc)[:300]}"}

    out["reference_optimized"] = time_arm(reference_bwd, "reference optimized backward", True)
    if hasattr(reference_bwd, "_fdr_intra"):
        out["reference_intra_fallback_calls"] = reference_bwd._fdr_intra.fallback_calls
    out["fla_original"] = time_arm(fla_bwd, "FLA stock backward", False)
    # the forward the reference runs is FLA's own, unchanged (src/fast_delta_rule/_compat/kda.py:89-113)
    from fla.ops.kda import chunk as fla_chunk
    kw = dict(q=xs["q"], k=xs["k"], v=xs["v"], g=xs["g"], beta=xs["beta"], scale=128 ** -0.5,
              initial_state=xs["initial_state"], output_final_state=False, disable_recompute=saved)
    out["fla_forward"] = time_arm(fla_chunk.chunk_kda_fwd, "FLA forward", False)
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
