"""GPU parity at the shapes the benchmark configurations name, with the kernel instances the benchmark times.

Every case runs the whole-family backward through the C ABI on a problem with far more chunks than SMs (each
persistent CTA of the chunk kernel walks over many chunks, every state-scan CTA over a long chain), in BF16 and in
FP32 output mode, and compares one (batch, head) slice with the FP64 closed-form oracle run on that slice alone
(the path has no cross-batch or cross-head term).  The acceptance follows the reference's own
(src/fast_delta_rule/validation.py:47-76: both activation policies, relative L2 per gradient) on the shape grid of
research/operators/a800_ablation/run.py:19.

Tolerances (normalised RMSE):
  FP32 outputs           <= 2e-3 for every gradient against the FP64 oracle;
  BF16 outputs (dq, dk, and GDN2's db, dw): compared in the BF16 domain.  The rounding floor is measured, not argued:
                         floor = NRMSE(bf16(FP32-output run), bf16(oracle)); the BF16-output run must stay within
                         floor + 2e-4 (it rounds the same FP32 values once), and both numbers are printed.
  two runs on the same inputs are bitwise equal (the kernels have no atomics on their outputs).
Under the recompute policy (always, for the scalar-gate families) the backward rebuilds w, u, qg, kg, h and v_new
itself.  BF16 roundings make those tensors a function of the accumulation order, so two correct forwards differ in
last bits, and without a decay (DeltaNet) such differences stay in the state for the rest of the sequence.  The oracle
is therefore fed with the recomputed tensors as the library's own recompute stages produce them (called through the
C ABI on the full problem); the recompute stages themselves are checked against the oracle in test_gpu_parity.py.
"""
import pytest
import torch

from gpu_util import base_args, call_stage, nrmse, oracle_backward, stage_buffers
from rewy_b200 import _capi
from rewy_b200 import backward as bw
from rewy_b200.forward import chunk_forward
from rewy_b200.synthetic import CONFIGS, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3
BF16_SLACK = 2e-4
SCALE = 128 ** -0.5


def _call(op, xs, sv, saved, out_dtype):
    r = _call_family(op, xs, sv, saved, out_dtype)
    torch.cuda.synchronize()
    return r


def _call_family(op, xs, sv, saved, out_dtype):
    B, T, H, _ = xs["k"].shape
    ws = torch.empty(_capi.workspace_bytes(_capi.FAMILY_ID[op], _capi.SAVED if saved else _capi.RECOMPUTE, B, T, H),
                     dtype=torch.uint8, device=DEV)
    common = dict(q=xs["q"], k=xs["k"], v=xs["v"], scale=SCALE, initial_state=xs.get("initial_state"), do=xs["do"],
                  dht=xs.get("dht"), out_dtype=out_dtype, workspace=ws, check_status=True)
    out = _call_op(op, xs, sv, saved, common)
    out["wide_chunks"] = _capi.load().rewy_wide_chunk_count(_capi.ptr(ws), _capi.current_stream(torch.device(DEV)))
    return out


def _call_op(op, xs, sv, saved, common):
    if op == "kda":
        r = bw.kda_backward(beta=xs["beta"], Aqk=sv["Aqk"], Akk=sv["Akk"], g=sv["g_cumsum"], disable_recompute=saved,
                            w=sv["w"], u=sv["u"], qg=sv["qg"], kg=sv["kg"], v_new=sv["v_new"], h=sv["h"], **common)
        return dict(dq=r[0], dk=r[1], dv=r[2], dbeta=r[3], dg=r[4], dh0=r[5])
    if op == "gdn2":
        r = bw.gdn2_backward(b=xs["b"], w_gate=xs["w"], Aqk=sv["Aqk"], Akk=sv["Akk"], g=sv["g_cumsum"],
                             disable_recompute=saved, w_wy=sv["w"], u_wy=sv["u"], qg=sv["qg"], kg=sv["kg"],
                             v_new=sv["v_new"], h=sv["h"], **common)
        return dict(dq=r[0], dk=r[1], dv=r[2], db=r[3], dw=r[4], dg=r[5], dh0=r[6])
    if op == "gdn":
        r = bw.gdn_backward(g=sv["g_cumsum"], beta=xs["beta"], A=sv["Akk"], **common)
        return dict(dq=r[0], dk=r[1], dv=r[2], dbeta=r[3], dg=r[4], dh0=r[5])
    r = bw.delta_backward(beta=xs["beta"], A=sv["Akk"], **common)
    return dict(dq=r[0], dk=r[1], dv=r[2], dbeta=r[3], dh0=r[4])


def _slice(t, b, h, is_state=False):
    if t is None:
        return None
    if is_state:                      # [B,H,K,V]
        return t[b:b + 1, h:h + 1].contiguous()
    return t[b:b + 1, :, h:h + 1].contiguous()   # [B,T,H,...] and h [B,NT,H,K,V]


def _oracle_slice(op, xs, sv, b, h):
    xs_s = {n: _slice(t, b, h, n in ("initial_state", "dht")) for n, t in xs.items()}
    sv_s = {n: _slice(t, b, h) for n, t in sv.items() if t is not None and n not in ("o", "final_state")}
    return oracle_backward(op, xs_s, sv_s)


def _recomputed(op, xs, sv):
    """The saved set with w, u, qg, kg, h, v_new (and Aqk for the scalar families) replaced by what the library's
    recompute stages produce from the same inputs."""
    a, keep = base_args(op, xs, sv)
    like = lambda n: torch.full_like(sv[n], float("nan"))
    w, u, qg, kg, aqk, h, v_new = (like(n) for n in ("w", "u", "qg", "kg", "Aqk", "h", "v_new"))
    ctrl = torch.zeros(8, dtype=torch.int32, device=DEV)
    call_stage("rewy_stage_prepare", a, stage_buffers(w=w, u=u, qg=qg, kg=kg, Aqk=aqk), DEV)
    call_stage("rewy_stage_fwd_scan", a, stage_buffers(w=w, u=u, kg=kg, h=h, v_new=v_new, ctrl=ctrl), DEV)
    assert ctrl[0].item() == 0
    out = dict(sv, w=w, u=u, qg=qg, kg=kg, h=h, v_new=v_new)
    if op in ("gdn", "delta"):
        out["Aqk"] = aqk
    return out


def _slice_out(out, b, h):
    return {n: _slice(t, b, h, n == "dh0") for n, t in out.items() if torch.is_tensor(t)}


def _check_case(op, B, T, H, cfg, policies, b0, h0):
    xs = make_inputs(op, B, T, H, seed=42, device=DEV, gate=cfg["gate"], gate_scale=cfg["gate_scale"],
                     state=cfg["state"])
    sv = chunk_forward(op, xs["q"], xs["k"], xs["v"], g=xs.get("g"), beta=xs.get("beta"), b=xs.get("b"), w=xs.get("w"),
                       initial_state=xs.get("initial_state"), output_final_state=False)
    low = ("dq", "dk") + (("db", "dw") if op == "gdn2" else ())       # outputs that follow out_dtype
    report = {}
    for saved in policies:
        ref = _oracle_slice(op, xs, sv if saved else _recomputed(op, xs, sv), b0, h0)
        o32 = _slice_out(_call(op, xs, sv, saved, torch.float32), b0, h0)
        full16 = _call(op, xs, sv, saved, torch.bfloat16)
        again16 = _call(op, xs, sv, saved, torch.bfloat16)
        torch.cuda.synchronize()
        assert full16["wide_chunks"] == 0, "the benchmark shapes are meant to stay on the tensor-core chunk kernel"
        for n, t in full16.items():
            if torch.is_tensor(t):
                assert torch.equal(t, again16[n]), f"{op} {n}: two runs on the same inputs differ"
        o16 = _slice_out(full16, b0, h0)
        del full16, again16
        errs32, errs16, floor = {}, {}, {}
        for n, got in o32.items():
            r = ref[n]
            errs32[n] = nrmse(r.to(got.dtype), got)
            assert torch.isfinite(got.float()).all(), (op, n)
        for n in low:
            rb = ref[n].to(torch.bfloat16)
            floor[n] = nrmse(rb, o32[n].to(torch.bfloat16))
            errs16[n] = nrmse(rb, o16[n])
        for n, got in o16.items():
            if n not in low:          # same dtype in both modes: must not depend on the output mode of dq/dk
                errs16[n] = nrmse(ref[n].to(got.dtype), got)
        report[saved] = dict(fp32=errs32, bf16=errs16, bf16_rounding_floor=floor)
        print(f"{op} B={B} T={T} H={H} policy_saved={saved} slice=({b0},{h0}): {report[saved]}")
        bad = {n: e for n, e in errs32.items() if not e <= TOL}
        assert not bad, f"FP32-output run above {TOL}: {bad}; all {errs32}"
        bad = {n: (errs16[n], floor[n]) for n in low if not errs16[n] <= floor[n] + BF16_SLACK}
        assert not bad, f"BF16-output run above the measured rounding floor + {BF16_SLACK}: {bad}"
        bad = {n: e for n, e in errs16.items() if n not in low and not e <= TOL}
        assert not bad, f"BF16-output run, gradients that keep their dtype, above {TOL}: {bad}"
    return report


def test_cfg2_kda_headline_shape_both_policies_bf16_and_fp32():
    """KDA B=8, T=8192, H=32 (32768 chunks: 221 per persistent CTA; 128-chunk scan chains)."""
    cfg = CONFIGS["cfg2_kda"]
    _check_case("kda", cfg["B"], cfg["T"], cfg["H"], cfg, (True, False), b0=5, h0=17)


def test_cfg4_gdn2_long_sequence_both_policies_bf16_and_fp32():
    """GDN2 at T=32768 (512-chunk chains, where the state's hi/lo operand pairs matter), H=32, initial state and
    final-state gradient present; the batch is reduced to 2 to bound the torch forward that produces the saved set."""
    cfg = CONFIGS["cfg4_gdn2"]
    _check_case("gdn2", 2, cfg["T"], cfg["H"], cfg, (True, False), b0=1, h0=9)


def test_cfg1_gdn_shape_head_exp_gate_with_states():
    """Gated DeltaNet B=4, T=4096, H=16 with the per-head exponential gate law (75-200 log2 units per chunk)."""
    cfg = CONFIGS["cfg1_gdn"]
    _check_case("gdn", cfg["B"], cfg["T"], cfg["H"], cfg, (False,), b0=2, h0=11)


def test_cfg3_delta_shape():
    """DeltaNet B=16, T=2048, H=16: no gate, no state; residual WY only."""
    cfg = CONFIGS["cfg3_delta"]
    _check_case("delta", cfg["B"], cfg["T"], cfg["H"], cfg, (False,), b0=13, h0=3)
