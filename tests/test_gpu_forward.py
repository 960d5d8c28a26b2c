"""The CUDA forward (chunk-local kernel, tcgen05 state scan, output kernel) against the FP64 chunked forward of the
oracle on the raw inputs, and against the torch statement of the same forward (second implementation).

Tolerances (normalised RMSE, in the BF16 domain of the tensors): the A matrices, qg and kg are single roundings of
FP32-accurate values (3e-3); w, u, v_new, h, o and the final state pass through BF16 operands (the saved Akk, the
state of each chunk) like FLA's forward does, which the reference's acceptance covers with 0.008
(src/fast_delta_rule/validation.py:68-71); 6e-3 is used here, the same limit as for the torch statement on the host.
"""
import pytest
import torch

from gpu_util import nrmse
from rewy_b200.forward import chunk_forward, chunk_forward_torch
from rewy_b200.synthetic import make_inputs, operator_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
OPS = ("kda", "gdn2", "gdn", "delta")
TIGHT = ("Aqk", "Akk", "qg", "kg")
NAMES = ("o", "final_state", "Aqk", "Akk", "w", "u", "qg", "kg", "v_new", "h")


def _kw(op, xs):
    kw = dict(q=xs["q"], k=xs["k"], v=xs["v"], initial_state=xs.get("initial_state"))
    if op != "delta":
        kw["g"] = xs["g"]
    if op == "gdn2":
        kw["b"], kw["w"] = xs["b"], xs["w"]
    else:
        kw["beta"] = xs["beta"]
    return kw


def _oracle(op, xs):
    from oracle import chunk_forward as oracle_forward
    return oracle_forward(op, {n: (t.detach().cpu() if t is not None else None) for n, t in operator_inputs(op, xs).items()})


@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("state", (True, False))
def test_cuda_forward_matches_the_oracle_and_the_torch_statement(op, state):
    xs = make_inputs(op, 2, 256, 2, seed=8, device=DEV, state=state, gate_scale=0.1 if op != "gdn" else 1.0,
                     gate="softplus" if op != "gdn" else "head_exp")
    got = chunk_forward(op, check_status=True, **_kw(op, xs))
    ref = _oracle(op, xs)
    other = chunk_forward_torch(op, **_kw(op, xs))
    errs, cross = {}, {}
    for n in NAMES:
        r = ref[n]
        errs[n] = nrmse(r.to(got[n].dtype), got[n])
        cross[n] = nrmse(other[n], got[n])
        assert torch.isfinite(got[n].float()).all(), n
    if op != "delta":
        assert torch.allclose(got["g_cumsum"].double().cpu(), ref["g_cumsum"], atol=1e-4, rtol=1e-5)
    print(f"forward {op} state={state}: vs oracle {errs}; vs torch statement {cross}")
    bad = {n: e for n, e in errs.items() if not e <= (3e-3 if n in TIGHT else 6e-3)}
    assert not bad, bad
    bad = {n: e for n, e in cross.items() if not e <= 4e-3}
    assert not bad, f"CUDA forward and torch statement disagree: {bad}"


def test_output_kernel_variants_agree():
    """The TMA + tcgen05 output kernel against its warp-MMA cross-check (same operands, FP32 accumulation)."""
    from rewy_b200 import _capi
    lib = _capi.load()
    xs = make_inputs("gdn2", 2, 512, 3, seed=12, device=DEV)
    tc = chunk_forward("gdn2", check_status=True, **_kw("gdn2", xs))
    try:
        assert lib.rewy_set_forward_variant(1) == 0
        warp = chunk_forward("gdn2", check_status=True, **_kw("gdn2", xs))
    finally:
        lib.rewy_set_forward_variant(0)
    assert torch.isfinite(tc["o"].float()).all()
    assert nrmse(warp["o"], tc["o"]) < 1e-3, nrmse(warp["o"], tc["o"])
    assert torch.equal(warp["h"], tc["h"]) and torch.equal(warp["v_new"], tc["v_new"])


def test_cuda_forward_value_first_states_and_no_final_state():
    xs = make_inputs("kda", 1, 192, 3, seed=9, device=DEV)
    plain = chunk_forward("kda", check_status=True, **_kw("kda", xs))
    kw = _kw("kda", xs)
    kw["initial_state"] = xs["initial_state"].transpose(-1, -2).contiguous()
    vf = chunk_forward("kda", state_v_first=True, check_status=True, **kw)
    assert torch.equal(vf["final_state"].transpose(-1, -2), plain["final_state"])
    for n in ("o", "h", "v_new"):
        assert torch.equal(vf[n], plain[n]), n
    none = chunk_forward("kda", output_final_state=False, check_status=True, **_kw("kda", xs))
    assert none["final_state"] is None and torch.equal(none["o"], plain["o"])


@pytest.mark.parametrize("case", ("strong", "mixed"))
def test_cuda_forward_wide_gate_spans_take_the_pairwise_path(case):
    """Cumulative gates spanning 80 log2 units or more per chunk (about 150 everywhere, or far above 200 in a few
    channels of one chunk next to ordinary chunks): centred factors would leave the FP32 range, the chunk-local kernel
    sums those chunks pair by pair."""
    if case == "strong":
        xs = make_inputs("kda", 1, 192, 2, seed=10, device=DEV, gate_scale=2.0)
    else:
        xs = make_inputs("kda", 1, 192, 2, seed=10, device=DEV, gate_scale=0.1)
        xs["g"][:, 64:128, 0, :32] *= 30
    span = (xs["g"].float().reshape(1, 3, 64, 2, 128).sum(2).abs().max() * 1.4427).item()
    assert span > 100, span
    got = chunk_forward("kda", check_status=True, **_kw("kda", xs))
    ref = _oracle("kda", xs)
    errs = {n: nrmse(ref[n].to(got[n].dtype), got[n]) for n in NAMES}
    print(f"forward kda wide spans ({case}, max span {span:.0f}): {errs}")
    assert all(torch.isfinite(got[n].float()).all() for n in NAMES)
    bad = {n: e for n, e in errs.items() if not e <= 8e-3}
    assert not bad, bad


def test_cuda_forward_headline_shape_slice():
    """One (batch, head) slice of the CUDA forward at B=8, T=8192, H=32 against the oracle run on that slice."""
    xs = make_inputs("kda", 8, 8192, 32, seed=42, device=DEV, gate_scale=0.1, state=False)
    got = chunk_forward("kda", check_status=True, **_kw("kda", xs))
    b0, h0 = 3, 21
    sl = {n: (t[b0:b0 + 1, :, h0:h0 + 1].contiguous() if t is not None else None) for n, t in xs.items()}
    ref = _oracle("kda", sl)
    errs = {n: nrmse(ref[n].to(got[n].dtype), got[n][b0:b0 + 1, :, h0:h0 + 1] if n != "final_state" else got[n][b0:b0 + 1, h0:h0 + 1])
            for n in NAMES}
    print(f"forward kda headline slice: {errs}")
    bad = {n: e for n, e in errs.items() if not e <= (3e-3 if n in TIGHT else 6e-3)}
    assert not bad, bad
