"""Envelope extensions handled in the operators, around the autograd functions (rewy_b200/functions.py):
lengths that are not multiples of the 64-token chunk (fixed batch and packed; neutral padding tokens), grouped value
heads (q and k repeated per group) and head dimensions below 128 (zero channels).

Checked: forward outputs, final states and every gradient against the FP64 token recurrence with the reference's own
acceptance limits (validation.py:40-45,68-71); a packed ragged batch against its sequences run one at a time; the
padding tokens of a fused-gate call leave the final state alone; a grouped call equals the call with repeated heads.
FLA covers these cases inside its kernels; the reference's release envelope rejects them
(src/fast_delta_rule/runtime.py:84-88).
"""
import pytest
import torch

from gpu_util import nrmse
from rewy_b200.synthetic import make_inputs, operator_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
OPS = ("kda", "gdn2", "gdn", "delta")
NAMES = {"kda": "chunk_kda", "gdn2": "chunk_gdn2", "gdn": "chunk_gated_delta_rule", "delta": "chunk_delta_rule"}


def _call(op, ins, do, dht, **kw):
    import rewy_b200 as fdr
    leaves = {n: x.detach().clone().requires_grad_() for n, x in ins.items() if x is not None}
    with fdr.use_backend("optimized", ops=(op,)):
        o, fin = getattr(fdr, NAMES[op])(**leaves, output_final_state=True, **kw)
    grads = torch.autograd.grad((o, fin), tuple(leaves.values()), (do, dht))
    return o, fin, dict(zip(leaves, grads))


@pytest.mark.parametrize("T", (100, 37))
@pytest.mark.parametrize("op", OPS)
def test_length_that_is_not_a_multiple_of_the_chunk_against_the_recurrence(op, T):
    from oracle import recurrence_grads
    xs = make_inputs(op, 2, T, 2, seed=7, device=DEV, gate_scale=0.05, gate="softplus")
    ins = operator_inputs(op, xs)
    ref, o_ref, fin_ref = recurrence_grads(op, {n: (x.detach().cpu() if x is not None else None) for n, x in ins.items()},
                                           xs["do"].cpu(), xs["dht"].cpu())
    for saved in ((False, True) if op in ("kda", "gdn2") else (False,)):
        kw = dict(disable_recompute=saved) if op in ("kda", "gdn2") else {}
        o, fin, grads = _call(op, ins, xs["do"], xs["dht"], **kw)
        assert o.shape == xs["do"].shape
        errs = {n: nrmse(ref[n], g) for n, g in grads.items()}
        errs["o"], errs["final_state"] = nrmse(o_ref, o), nrmse(fin_ref, fin)
        print("NRMSE", op, T, saved, {n: float(f"{e:.3g}") for n, e in errs.items()})
        for n, e in errs.items():
            assert e <= (0.02 if n in ("g", "beta", "b", "w") else 0.008), (op, T, n, e)


@pytest.mark.parametrize("op", OPS)
def test_packed_ragged_batch_equals_its_sequences_run_one_at_a_time(op):
    lengths = (100, 37, 200)
    seqs = [make_inputs(op, 1, T, 2, seed=60 + i, device=DEV, gate_scale=0.1, gate="softplus") for i, T in enumerate(lengths)]
    names = [n for n, x in operator_inputs(op, seqs[0]).items() if x is not None and n != "initial_state"]
    cat = lambda n: torch.cat([s[n] for s in seqs], 1)
    packed = {n: cat(n) for n in names}
    packed["initial_state"] = torch.cat([s["initial_state"] for s in seqs], 0)
    cu = torch.tensor([0, 100, 137, 337], dtype=torch.int64, device=DEV)
    o, fin, grads = _call(op, packed, cat("do"), torch.cat([s["dht"] for s in seqs], 0), cu_seqlens=cu)
    assert o.shape[1] == 337 and fin.shape[0] == 3
    at = 0
    for i, (s, T) in enumerate(zip(seqs, lengths)):
        one = {n: s[n] for n in names}
        one["initial_state"] = s["initial_state"]
        o1, fin1, g1 = _call(op, one, s["do"], s["dht"])
        assert torch.equal(o[:, at:at + T], o1), (op, i, "o")
        assert torch.equal(fin[i:i + 1], fin1), (op, i, "final_state")
        for n in names:
            assert torch.equal(grads[n][:, at:at + T], g1[n]), (op, i, n)
        assert torch.equal(grads["initial_state"][i:i + 1], g1["initial_state"]), (op, i, "initial_state")
        at += T


def test_padding_tokens_of_a_fused_gate_call_do_not_decay_the_state():
    """With use_gate_in_kernel the gate input goes through -exp(A_log) softplus(g + dt_bias); the padding must still mean
    "no decay".  The fused call on 100 tokens has to agree with the call that is given the activated gate."""
    import rewy_b200 as fdr
    T, H = 100, 2
    xs = make_inputs("kda", 1, T, H, seed=11, device=DEV, gate_scale=0.05, gate="softplus")
    gen = torch.Generator(device="cpu").manual_seed(3)
    raw = torch.randn(1, T, H, 128, generator=gen).to(DEV)
    A_log = (0.3 * torch.randn(H, generator=gen)).to(DEV)
    dt_bias = (0.1 * torch.randn(H * 128, generator=gen)).to(DEV)
    act = -torch.exp(A_log).view(1, 1, H, 1) * torch.nn.functional.softplus(raw + dt_bias.view(1, 1, H, 128))
    with fdr.use_backend("optimized", ops=("kda",)):
        o_f, fin_f = fdr.chunk_kda(xs["q"], xs["k"], xs["v"], raw, xs["beta"], initial_state=xs["initial_state"],
                                   output_final_state=True, use_gate_in_kernel=True, A_log=A_log, dt_bias=dt_bias)
        o_a, fin_a = fdr.chunk_kda(xs["q"], xs["k"], xs["v"], act, xs["beta"], initial_state=xs["initial_state"],
                                   output_final_state=True)
    assert nrmse(o_a, o_f) <= 2e-3 and nrmse(fin_a, fin_f) <= 1e-3, (nrmse(o_a, o_f), nrmse(fin_a, fin_f))


@pytest.mark.parametrize("op", ("kda", "gdn"))
def test_grouped_value_heads_equal_the_call_with_repeated_query_and_key_heads(op):
    """HV = 2 H: value head hv reads query/key head hv // 2 (FLA's convention); dq and dk are sums over each group."""
    xs = make_inputs(op, 1, 128, 4, seed=21, device=DEV, gate_scale=0.1, gate="softplus")
    ins = {n: x for n, x in operator_inputs(op, xs).items() if x is not None}
    grouped = dict(ins, q=ins["q"][:, :, ::2].contiguous(), k=ins["k"][:, :, ::2].contiguous())
    repeated = dict(ins, q=grouped["q"].repeat_interleave(2, 2), k=grouped["k"].repeat_interleave(2, 2))
    o_g, fin_g, g_g = _call(op, grouped, xs["do"], xs["dht"])
    o_r, fin_r, g_r = _call(op, repeated, xs["do"], xs["dht"])
    assert g_g["q"].shape == grouped["q"].shape and torch.equal(o_g, o_r) and torch.equal(fin_g, fin_r)
    for n in ins:
        if n in ("q", "k"):
            want = g_r[n].float().view(1, 128, 2, 2, 128).sum(3)
            assert nrmse(want, g_g[n]) <= 4e-3, (op, n, nrmse(want, g_g[n]))     # one BF16 rounding of the sum
        else:
            assert torch.equal(g_g[n], g_r[n]), (op, n)


@pytest.mark.parametrize("op", OPS)
def test_head_dimensions_below_128_against_the_recurrence(op):
    """K = 64, V = 96: zero channels are added for the kernels and cut from the results; the scale stays 64^-0.5."""
    from oracle import recurrence_grads
    xs = make_inputs(op, 1, 128, 2, K=64, V=96, seed=5, device=DEV, gate_scale=0.05, gate="softplus")
    ins = operator_inputs(op, xs)
    ref, o_ref, fin_ref = recurrence_grads(op, {n: (x.detach().cpu() if x is not None else None) for n, x in ins.items()},
                                           xs["do"].cpu(), xs["dht"].cpu())
    o, fin, grads = _call(op, ins, xs["do"], xs["dht"])
    assert o.shape[-1] == 96 and fin.shape[-2:] == (64, 96)
    errs = {n: nrmse(ref[n], g) for n, g in grads.items()}
    errs["o"], errs["final_state"] = nrmse(o_ref, o), nrmse(fin_ref, fin)
    print("NRMSE", op, {n: float(f"{e:.3g}") for n, e in errs.items()})
    for n, e in errs.items():
        assert e <= (0.02 if n in ("g", "beta", "b", "w") else 0.008), (op, n, e)


@pytest.mark.parametrize("op", ("kda", "delta"))
def test_non_contiguous_inputs_give_the_contiguous_result(op):
    """The reference's accelerator test passes a non-contiguous q (tests/test_accelerator.py:41)."""
    xs = make_inputs(op, 2, 128, 2, seed=9, device=DEV, gate_scale=0.1, gate="softplus")
    ins = {n: x for n, x in operator_inputs(op, xs).items() if x is not None}
    strided = dict(ins)
    strided["q"] = torch.stack([ins["q"], ins["q"]], -1)[..., 0]                 # channel stride 2
    strided["v"] = ins["v"].transpose(1, 2).contiguous().transpose(1, 2)          # head-major storage
    assert not strided["q"].is_contiguous() and not strided["v"].is_contiguous()
    o, fin, g = _call(op, ins, xs["do"], xs["dht"])
    o2, fin2, g2 = _call(op, strided, xs["do"].transpose(1, 2).contiguous().transpose(1, 2), xs["dht"])
    assert torch.equal(o, o2) and torch.equal(fin, fin2)
    for n in g:
        assert torch.equal(g[n], g2[n]), (op, n)
