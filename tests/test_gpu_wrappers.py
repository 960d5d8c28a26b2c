"""Wrapper-level stages (q/k L2 normalisation, beta sigmoid, fused KDA gate, value-first states) on the GPU.

The element-wise CUDA passes are compared with their FP64 formulas; the public operators with every wrapper option
switched on are compared with FP64 autograd through the same transformations followed by the token recurrence - the
reference's fused-option acceptance (tests/test_accelerator.py:65-83, limits 0.008 and 0.02 for gate, beta, A_log and
dt_bias gradients).
"""
import pytest
import torch

from gpu_util import nrmse
from rewy_b200 import elementwise as ew
from rewy_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _gen(seed):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    return g


def test_l2norm_forward_and_backward_match_fp64():
    g = _gen(1)
    x = (torch.randn(3, 200, 5, 128, generator=g, device=DEV) * 3).bfloat16()
    y, rstd = ew.l2norm_fwd(x)
    xd = x.double()
    rs = (xd.pow(2).sum(-1, keepdim=True) + 1e-6).rsqrt()
    assert nrmse((xd * rs).to(torch.bfloat16), y) < 1e-3 and nrmse(rs[..., 0], rstd) < 1e-6
    for dt in (torch.float32, torch.bfloat16):
        dy = torch.randn(3, 200, 5, 128, generator=g, device=DEV).to(dt)
        dx = ew.l2norm_bwd(y, rstd, dy)
        yd, dyd = y.double(), dy.double()
        want = (dyd - yd * (dyd * yd).sum(-1, keepdim=True)) * rstd.double()[..., None]
        assert dx.dtype == torch.bfloat16 and nrmse(want.to(torch.bfloat16), dx) < 1e-3, dt


@pytest.mark.parametrize("dt", (torch.bfloat16, torch.float32))
def test_beta_sigmoid_forward_and_backward_match_fp64(dt):
    g = _gen(2)
    x = torch.randn(2, 130, 7, generator=g, device=DEV).to(dt)
    dy = torch.randn(2, 130, 7, generator=g, device=DEV)
    for scale in (1.0, 2.0):
        y = ew.beta_sigmoid_fwd(x, scale)
        s = torch.sigmoid(x.double())
        assert y.dtype == dt and nrmse((scale * s).to(dt), y) < 1e-6 + (4e-3 if dt == torch.bfloat16 else 0)
        dx = ew.beta_sigmoid_bwd(x, dy, scale)
        assert nrmse(dy.double() * scale * s * (1 - s), dx) < 1e-5


@pytest.mark.parametrize("dt", (torch.bfloat16, torch.float32))
def test_gate_cumsum_and_activation_match_fp64(dt):
    g = _gen(3)
    B, T, H = 2, 192, 3
    x = torch.randn(B, T, H, 128, generator=g, device=DEV).to(dt)
    A_log = torch.randn(H, generator=g, device=DEV) * 0.5 - 1.0
    bias = torch.randn(H * 128, generator=g, device=DEV) * 0.3
    ln2 = torch.log(torch.tensor(2.0, dtype=torch.float64))
    chunks = lambda t: t.reshape(B, T // 64, 64, H, 128)
    # plain chunk-local cumulative sum in log2 units
    got = ew.gate_cumsum_fwd(x)
    want = (chunks(x.double()).cumsum(2) / ln2).reshape(B, T, H, 128)
    assert nrmse(want, got) < 1e-6
    # with the gate activation, with and without the bias
    for b in (bias, None):
        act = -A_log.double().exp()[None, None, :, None] * torch.nn.functional.softplus(
            x.double() + (0 if b is None else b.double().view(H, 128)))
        got = ew.gate_cumsum_fwd(x, A_log, b)
        assert nrmse((chunks(act).cumsum(2) / ln2).reshape(B, T, H, 128), got) < 1e-5
        dg = torch.randn(B, T, H, 128, generator=g, device=DEV)
        dx, dA, dbias = ew.gate_act_bwd(x, A_log, b, dg)
        sig = torch.sigmoid(x.double() + (0 if b is None else b.double().view(H, 128)))
        want_dx = -A_log.double().exp()[None, None, :, None] * dg.double() * sig
        assert nrmse(want_dx, dx) < 1e-5
        assert nrmse((dg.double() * act).sum((0, 1, 3)), dA) < 1e-5
        if b is None:
            assert dbias is None
        else:
            assert nrmse(want_dx.sum((0, 1)).reshape(-1), dbias) < 1e-5


def _fp64_reference(op, raw, do, dht, l2norm, sigmoid, gate, v_first):
    """FP64 autograd through the wrapper transformations and the token recurrence; gradients w.r.t. the raw inputs."""
    from oracle import recurrence
    leaf = {n: t.detach().double().cpu().clone().requires_grad_() for n, t in raw.items() if t is not None}
    xs = dict(leaf)
    if l2norm:
        for n in ("q", "k"):
            xs[n] = leaf[n] * (leaf[n].pow(2).sum(-1, keepdim=True) + 1e-6).rsqrt()
    if sigmoid:
        xs["beta"] = torch.sigmoid(leaf["beta"])
    if gate:
        H = leaf["q"].shape[2]
        bias = leaf["dt_bias"].view(H, 128) if "dt_bias" in leaf else 0
        xs["g"] = -leaf["A_log"].exp()[None, None, :, None] * torch.nn.functional.softplus(leaf["g"] + bias)
    if "initial_state" in leaf and v_first:
        xs["initial_state"] = leaf["initial_state"].transpose(-1, -2)
    o, fin = recurrence(op, {n: xs[n] for n in xs if n not in ("A_log", "dt_bias")})
    if v_first:
        fin = fin.transpose(-1, -2)
    grads = torch.autograd.grad((o, fin), tuple(leaf.values()), (do.double().cpu(), dht.double().cpu()))
    return dict(zip(leaf, grads)), o.detach(), fin.detach()


def test_kda_with_every_wrapper_option_against_fp64_autograd():
    """The reference's fused-option case: raw gate with A_log and dt_bias, beta logits, unnormalised q/k, value-first
    initial and final states."""
    import rewy_b200 as fdr
    B, T, H = 1, 128, 2
    g = _gen(4)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    raw = dict(q=rn(B, T, H, 128).bfloat16(), k=rn(B, T, H, 128).bfloat16(), v=rn(B, T, H, 128).bfloat16(),
               g=rn(B, T, H, 128).bfloat16(), beta=rn(B, T, H).bfloat16(),
               A_log=torch.full((H,), -2.0, device=DEV), dt_bias=rn(H * 128) * 0.1,
               initial_state=rn(B, H, 128, 128) * 0.1)       # [B,H,V,K]
    do, dht = rn(B, T, H, 128).bfloat16(), rn(B, H, 128, 128) * 0.1
    ref, o_ref, fin_ref = _fp64_reference("kda", raw, do, dht, True, True, True, True)
    fdr.stats(reset=True)
    for saved in (False, True):
        ins = {n: t.detach().clone().requires_grad_() for n, t in raw.items()}
        with fdr.use_backend("optimized", ops=("kda",)):
            o, fin = fdr.chunk_kda(**ins, output_final_state=True, use_gate_in_kernel=True,
                                   use_beta_sigmoid_in_kernel=True, use_qk_l2norm_in_kernel=True, state_v_first=True,
                                   disable_recompute=saved)
        grads = torch.autograd.grad((o, fin), tuple(ins.values()), (do, dht))
        errs = {n: nrmse(ref[n], gr) for n, gr in zip(ins, grads)}
        errs["o"], errs["final_state"] = nrmse(o_ref, o), nrmse(fin_ref, fin)
        print(f"kda fused options, policy_saved={saved}: {errs}")
        bad = {n: e for n, e in errs.items() if not e <= (0.02 if n in ("g", "beta", "A_log", "dt_bias") else 0.008)}
        assert not bad, bad
        assert grads[0].dtype == torch.bfloat16 and grads[5].shape == (H,) and grads[6].shape == (H * 128,)
    assert fdr.stats()["kda.optimized_backward"] == 2


@pytest.mark.parametrize("op", ("gdn", "gdn2", "delta"))
def test_other_families_with_their_wrapper_options_against_fp64_autograd(op):
    """q/k normalisation for every family, beta sigmoid (doubled) for Gated DeltaNet, value-first states where the
    operator takes them."""
    import rewy_b200 as fdr
    xs = make_inputs(op, 1, 128, 2, seed=17, device=DEV, gate_scale=0.1, gate="softplus")
    g = _gen(5)
    raw = {n: xs[n] for n in ("q", "k", "v")}
    raw["q"] = (raw["q"].float() * 3).bfloat16()        # not unit length: the operator normalises
    raw["k"] = (raw["k"].float() * 2).bfloat16()
    if op != "delta":
        raw["g"] = xs["g"]
    if op == "gdn2":
        raw["b"], raw["w"] = xs["b"], xs["w"]
    elif op == "gdn":
        raw["beta"] = torch.randn(1, 128, 2, generator=g, device=DEV).bfloat16()
    else:
        raw["beta"] = xs["beta"]
    v_first = op != "delta"
    raw["initial_state"] = xs["initial_state"].transpose(-1, -2).contiguous() if v_first else xs["initial_state"]
    dht = xs["dht"].transpose(-1, -2).contiguous() if v_first else xs["dht"]
    sigmoid = op == "gdn"
    ref, o_ref, fin_ref = _fp64_reference(op, raw, xs["do"], dht, True, False, False, v_first) if not sigmoid else \
        _fp64_reference_scaled_sigmoid(op, raw, xs["do"], dht, v_first)
    ins = {n: t.detach().clone().requires_grad_() for n, t in raw.items()}
    kw = dict(output_final_state=True, use_qk_l2norm_in_kernel=True)
    if v_first:
        kw["state_v_first"] = True
    if sigmoid:
        kw.update(use_beta_sigmoid_in_kernel=True, allow_neg_eigval=True)
    name = {"gdn": "chunk_gated_delta_rule", "gdn2": "chunk_gdn2", "delta": "chunk_delta_rule"}[op]
    with fdr.use_backend("optimized", ops=(op,)):
        o, fin = getattr(fdr, name)(**ins, **kw)
    grads = torch.autograd.grad((o, fin), tuple(ins.values()), (xs["do"], dht))
    errs = {n: nrmse(ref[n], gr) for n, gr in zip(ins, grads)}
    errs["o"], errs["final_state"] = nrmse(o_ref, o), nrmse(fin_ref, fin)
    print(f"{op} wrapper options: {errs}")
    bad = {n: e for n, e in errs.items() if not e <= (0.02 if n in ("g", "beta", "b", "w") else 0.008)}
    assert not bad, bad


def _fp64_reference_scaled_sigmoid(op, raw, do, dht, v_first):
    """As _fp64_reference with beta = 2 * sigmoid(logits) (allow_neg_eigval) and normalised q/k."""
    from oracle import recurrence
    leaf = {n: t.detach().double().cpu().clone().requires_grad_() for n, t in raw.items() if t is not None}
    xs = dict(leaf)
    for n in ("q", "k"):
        xs[n] = leaf[n] * (leaf[n].pow(2).sum(-1, keepdim=True) + 1e-6).rsqrt()
    xs["beta"] = 2.0 * torch.sigmoid(leaf["beta"])
    if v_first:
        xs["initial_state"] = leaf["initial_state"].transpose(-1, -2)
    o, fin = recurrence(op, xs)
    if v_first:
        fin = fin.transpose(-1, -2)
    grads = torch.autograd.grad((o, fin), tuple(leaf.values()), (do.double().cpu(), dht.double().cpu()))
    return dict(zip(leaf, grads)), o.detach(), fin.detach()
