"""Pins the CPU oracle against fixtures produced by the reference's own CPU code
(tests/golden/make_golden.py) and against the reference's own test constructions."""
import numpy as np
import pytest
import torch

from oracle import (chunk_backward, chunk_forward, matrix_intra_centered, matrix_intra_pairwise,
                    naive_chunk_backward_fp32, recurrence, recurrence_grads)

OPS = ("kda", "gdn", "gdn2", "delta")
GRAD_NAME = dict(q="dq", k="dk", v="dv", g="dg", beta="dbeta", b="db", w="dw", initial_state="dh0")


def _load_recurrence(golden_dir, op):
    with np.load(golden_dir / f"recurrence_{op}.npz") as z:
        a = {n: torch.from_numpy(z[n]) for n in z.files}
    xs = {n[3:]: x.double() for n, x in a.items() if n.startswith("in_") and n not in ("in_do", "in_dht")}
    grads = {n[5:]: x.double() for n, x in a.items() if n.startswith("grad_")}
    return xs, a["in_do"].double(), a["in_dht"].double(), grads, a["out_o"].double(), a["out_final_state"].double()


def _rel(ref, got):
    return ((got - ref).norm() / ref.norm()).item()


@pytest.mark.parametrize("op", OPS)
def test_recurrence_matches_reference_recurrence(golden_dir, op):
    xs, do, dht, grads, o, final = _load_recurrence(golden_dir, op)
    got, o2, final2 = recurrence_grads(op, xs, do, dht)
    assert _rel(o, o2) < 1e-6 and _rel(final, final2) < 1e-6
    for n, g in grads.items():
        assert _rel(g, got[n]) < 1e-6, n


@pytest.mark.parametrize("op", OPS)
def test_closed_form_chunk_backward_matches_reference_recurrence(golden_dir, op):
    """Two chunks chained (T=128): forward intermediates + closed-form backward vs the reference gradients."""
    xs, do, dht, grads, o, final = _load_recurrence(golden_dir, op)
    fwd = chunk_forward(op, xs)
    assert _rel(o, fwd["o"]) < 1e-6 and _rel(final, fwd["final_state"]) < 1e-6
    bwd = chunk_backward(op, xs, fwd, do, dht)
    for n, g in grads.items():
        assert _rel(g, bwd[GRAD_NAME[n]]) < 1e-6, n


@pytest.mark.parametrize("family", ("delta", "gdn", "kda", "gdn2"))
def test_closed_form_matches_reference_manuscript_backward(golden_dir, family):
    """One chunk of 8 rows, K=6, V=5, incoming state and state gradient, beta row 0 = 0."""
    with np.load(golden_dir / "closed_form_seed79.npz") as z:
        a = {n[len(family) + 1:]: torch.from_numpy(z[n]) for n in z.files if n.startswith(family + "_")}
    t = lambda x: x[None, :, None]            # [n,d] -> [1,n,1,d]
    xs = dict(q=t(a["in_Q"]), k=t(a["in_K"]), v=t(a["in_V"]), initial_state=a["in_S"][None, None])
    if family == "gdn":
        xs["g"] = t(a["in_g"])[..., 0]
    elif family != "delta":
        xs["g"] = t(a["in_g"])
    if family == "gdn2":
        xs["b"], xs["w"] = t(a["in_b"]), t(a["in_w"])
    else:
        xs["beta"] = t(a["in_b"])[..., 0]
    fwd = chunk_forward(family, xs, scale=1.0, chunk=8)
    bwd = chunk_backward(family, xs, fwd, t(a["in_do"]), a["in_ds"][None, None], scale=1.0, chunk=8)
    sq = lambda x: x[0, :, 0]
    assert torch.allclose(sq(fwd["v_new"]), a["out_R"], atol=1e-12)
    assert torch.allclose(sq(bwd["P"]), a["out_P"], atol=1e-12)
    assert torch.allclose(sq(bwd["dq"]), a["out_qb"], atol=1e-12)
    assert torch.allclose(sq(bwd["dk"]), a["out_kb"], atol=1e-12)
    assert torch.allclose(sq(bwd["dv"]), a["out_vb"], atol=1e-12)
    assert torch.allclose(bwd["dh0"][0, 0], a["out_sb"], atol=1e-12)
    if family == "gdn2":
        assert torch.allclose(sq(bwd["db"]), a["out_bb"], atol=1e-12)
        assert torch.allclose(sq(bwd["dw"]), a["out_wb"], atol=1e-12)
    else:
        assert torch.allclose(sq(bwd["dbeta"][..., None])[:, 0], a["out_bb"].sum(1) + a["out_wb"].sum(1), atol=1e-12)
    if family == "gdn":
        assert torch.allclose(bwd["dg"][0, :, 0], a["out_gb"].sum(1), atol=1e-12)
    elif family != "delta":
        assert torch.allclose(sq(bwd["dg"]), a["out_gb"], atol=1e-12)


@pytest.mark.parametrize("family", ("kda", "gdn2"))
@pytest.mark.parametrize("scale", (1.0, 3.0))
def test_matrix_intra_oracles_match_reference_oracle_on_captured_inputs(golden_dir, family, scale):
    with np.load(golden_dir / f"intra_{family}_inputs.npz") as z:
        x = {n: z[n].copy() for n in z.files}
    with np.load(golden_dir / f"intra_{family}_expected.npz") as z:
        exp = [z[f"scale{scale:g}_{n}"] for n in ("dq", "dk", "db", "dg")]
    x["g"] = x["g"] * scale
    for fn in (matrix_intra_pairwise, matrix_intra_centered):
        got = fn(x, family)
        for e, g in zip(exp, got):
            assert np.linalg.norm(g - e) <= 2e-6 * np.linalg.norm(e) + 1e-12


def _fd_objective(q, k, gate, beta, l, d):
    value = 0.0
    for i in range(len(q)):
        for j in range(i + 1):
            fac = np.exp2(gate[i] - gate[j])
            value += l[i, j] * np.sum(q[i] * k[j] * fac)
            if j < i:
                value += d[i, j] * np.sum(beta[i] * k[i] * k[j] * fac)
    return value


@pytest.mark.parametrize("vector_beta", (False, True))
@pytest.mark.parametrize("span", (3.0, 96.0))
def test_matrix_intra_vjp_against_finite_differences(vector_beta, span):
    """Same construction as the reference's finite-difference VJP test (tests/test_npu950.py:52-98):
    an independent scalar double-loop objective differentiated numerically, beta rows zeroed."""
    rng = np.random.default_rng(950)
    c, kd = 16, 32
    q, k = rng.normal(size=(2, c, kd))
    gate = -np.linspace(0.0, span, c)[:, None] * np.ones((1, kd))
    beta = rng.uniform(0.1, 0.9, (c, kd if vector_beta else 1))
    beta[::3] = 0.0
    l = np.tril(rng.normal(size=(c, c)))
    d = np.tril(rng.normal(size=(c, c)), -1)
    fam = "gdn2" if vector_beta else "kda"
    x = dict(q=q[None, :, None], k=k[None, :, None], g=gate[None, :, None], dAqk=l[None, :, None], dAkk=d[None, :, None],
             dq=np.zeros((1, c, 1, kd)), dk=np.zeros((1, c, 1, kd)), dg=np.zeros((1, c, 1, kd)))
    if vector_beta:
        x["b"], x["db"] = beta[None, :, None], np.zeros((1, c, 1, kd))
    else:
        x["beta"], x["db"] = beta[None, :, None, 0], np.zeros((1, c, 1))
    fn = matrix_intra_centered if span < 80 else matrix_intra_pairwise
    dq, dk, db, dg = (a[0, :, 0] for a in fn(x, fam))
    if not vector_beta:
        db = db[:, None]
    ln2 = np.log(2.0)
    for i, grad in enumerate((dq, dk, dg * ln2, db)):   # dg is per natural-log unit; objective gate is log2
        inputs = (q, k, gate, beta)
        direction = rng.normal(size=inputs[i].shape)
        pos, neg = list(inputs), list(inputs)
        eps = 1e-5
        pos[i] = inputs[i] + eps * direction
        neg[i] = inputs[i] - eps * direction
        numerical = (_fd_objective(*pos, l, d) - _fd_objective(*neg, l, d)) / (2 * eps)
        np.testing.assert_allclose(numerical, np.sum(grad * direction), rtol=2e-6, atol=2e-6)


def test_naive_chunk_fp32_backward_agrees_with_recurrence():
    """The CPU baseline path (FP32 autograd through the naive chunked forward) at a small shape."""
    from rewy_b200.synthetic import make_inputs, operator_inputs
    xs = make_inputs("kda", 1, 128, 1, seed=5)
    ins = operator_inputs("kda", xs)
    ref, _, _ = recurrence_grads("kda", ins, xs["do"], xs["dht"])
    got, _, _ = naive_chunk_backward_fp32("kda", ins, xs["do"], xs["dht"])
    for n, g in ref.items():
        assert _rel(g, got[n].double()) < 1e-4, n


def test_partition_invariance_of_chunking():
    """Chunk size 32 and 64 give the same gradients (the reference's partition-invariance check,
    benchmarks/plotting/check_manuscript_math.py:102-124)."""
    from rewy_b200.synthetic import make_inputs, operator_inputs
    xs = make_inputs("gdn2", 1, 128, 1, seed=9)
    ins = {n: (x.double() if x is not None else None) for n, x in operator_inputs("gdn2", xs).items()}
    a = chunk_backward("gdn2", ins, chunk_forward("gdn2", ins, chunk=32), xs["do"], xs["dht"], chunk=32)
    b = chunk_backward("gdn2", ins, chunk_forward("gdn2", ins, chunk=64), xs["do"], xs["dht"], chunk=64)
    for n in ("dq", "dk", "dv", "db", "dw", "dg", "dh0"):
        assert _rel(a[n], b[n]) < 1e-10, n
