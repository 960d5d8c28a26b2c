"""Whole-family backward and forward on shapes that are not round: odd head counts and batch sizes, a single chunk,
chunk counts that are not multiples of the number of persistent CTAs, more (batch, head) pairs than one wave of scan
CTAs.  Every gradient against the FP64 oracle (2e-3; 3e-3 for the scalar-gate dg on fewer than 1024 token-heads), both policies, BF16 outputs checked for finiteness and closeness.
Index arithmetic (head-fastest chunk order, per-(batch, head) scan chains, tile coordinates) is what these cases probe.
"""
import pytest
import torch

from gpu_util import forward_saved, nrmse, oracle_backward
from rewy_b200 import backward as bw
from rewy_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SHAPES = [(1, 64, 1), (3, 64, 5), (1, 448, 7), (5, 192, 3), (2, 1088, 1), (1, 128, 37), (7, 128, 11), (2, 320, 19)]


def _call(op, xs, sv, saved, out_dtype):
    common = dict(q=xs["q"], k=xs["k"], v=xs["v"], scale=128 ** -0.5, initial_state=xs.get("initial_state"), do=xs["do"],
                  dht=xs.get("dht"), out_dtype=out_dtype, check_status=True)
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


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%d_T%d_H%d" % s)
@pytest.mark.parametrize("op", ("kda", "gdn2", "gdn", "delta"))
def test_odd_shapes_against_the_oracle(op, shape):
    B, T, H = shape
    xs = make_inputs(op, B, T, H, seed=1000 + B * 131 + T + H, device=DEV, gate_scale=0.1, gate="softplus")
    sv = forward_saved(op, xs)
    ref = oracle_backward(op, xs, sv)
    for saved in ((True, False) if op in ("kda", "gdn2") else (False,)):
        out = _call(op, xs, sv, saved, torch.float32)
        errs = {n: nrmse(ref[n].to(t.dtype), t) for n, t in out.items() if torch.is_tensor(t)}
        # the scalar-gate dg is a key-sum of terms that largely cancel; over a handful of tokens its relative error
        # scatters more than over a benchmark-sized tensor (measured 2.2e-3 on 64 values, 1.2e-3 on 1024)
        bad = {n: e for n, e in errs.items() if not e <= (3e-3 if (op == "gdn" and n == "dg" and B * T * H < 1024) else 2e-3)}
        assert not bad, f"{op} {shape} saved={saved}: {bad}; all {errs}"
        out16 = _call(op, xs, sv, saved, torch.bfloat16)
        for n, t in out16.items():
            if torch.is_tensor(t):
                assert torch.isfinite(t.float()).all(), (op, shape, n)
                assert nrmse(out[n].to(t.dtype), t) <= 1e-6, (op, shape, n)   # the same values, rounded once
