"""Seeded synthetic inputs for the four operator families.

The reference measures and validates on synthetic tensors only
(src/fast_delta_rule/validation.py:6-21, research/operators/run_cuda.py:21-35); these
generators reproduce the distributions of the benchmark configurations: q,k ~ N(0,1)
L2-normalised over the head dimension and rounded to BF16, v ~ N(0,1) BF16,
beta = sigmoid(N(0,1)), log-decay gates negative, states ~ N(0, 0.1^2) FP32.
Every (batch, head) slice is drawn from its own generator keyed by (seed, b, h), so any
(batch, head) shard of a problem equals the same slice of the unsharded problem.
"""
import math
import torch

FAMILIES = ("delta", "gdn", "kda", "gdn2")

# The benchmark configurations of this operator (family, B, T, H and gate law).
CONFIGS = {
    "cfg0_kda_cpu": dict(op="kda", B=1, T=256, H=2, gate="softplus", gate_scale=0.1, state=False),
    "cfg1_gdn": dict(op="gdn", B=4, T=4096, H=16, gate="head_exp", gate_scale=1.0, state=True),
    "cfg2_kda": dict(op="kda", B=8, T=8192, H=32, gate="softplus", gate_scale=0.1, state=False),
    "cfg3_delta": dict(op="delta", B=16, T=2048, H=16, gate=None, gate_scale=0.0, state=False),
    "cfg4_gdn2": dict(op="gdn2", B=8, T=32768, H=32, gate="softplus", gate_scale=0.05, state=True),
}


def _gen(seed, b, h, device):
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + b * 1009 + h) & 0x7FFFFFFFFFFFFFFF)
    return g


def make_inputs(op, B, T, H, *, K=128, V=128, seed=42, device="cpu", gate="softplus", gate_scale=0.1,
                state=True, grad_state=None, heads=None, batches=None):
    """Returns dict(q,k,v,[g],[beta | b,w],initial_state,do,dht).

    heads / batches: optional iterables selecting a (batch, head) shard; slices are generated
    independently so the shard equals the matching slice of the full problem."""
    if op not in FAMILIES:
        raise ValueError(f"unknown family {op!r}")
    batches = list(range(B)) if batches is None else list(batches)
    heads = list(range(H)) if heads is None else list(heads)
    grad_state = state if grad_state is None else grad_state
    nb, nh = len(batches), len(heads)
    dev = torch.device(device)
    out = dict(
        q=torch.empty(nb, T, nh, K, dtype=torch.bfloat16, device=dev),
        k=torch.empty(nb, T, nh, K, dtype=torch.bfloat16, device=dev),
        v=torch.empty(nb, T, nh, V, dtype=torch.bfloat16, device=dev),
        do=torch.empty(nb, T, nh, V, dtype=torch.bfloat16, device=dev),
    )
    if op == "gdn":
        out["g"] = torch.empty(nb, T, nh, dtype=torch.float32, device=dev)
    elif op in ("kda", "gdn2"):
        out["g"] = torch.empty(nb, T, nh, K, dtype=torch.float32, device=dev)
    if op == "gdn2":
        out["b"] = torch.empty(nb, T, nh, K, dtype=torch.bfloat16, device=dev)
        out["w"] = torch.empty(nb, T, nh, V, dtype=torch.bfloat16, device=dev)
    else:
        out["beta"] = torch.empty(nb, T, nh, dtype=torch.bfloat16, device=dev)
    out["initial_state"] = torch.empty(nb, nh, K, V, dtype=torch.float32, device=dev) if state else None
    out["dht"] = torch.empty(nb, nh, K, V, dtype=torch.float32, device=dev) if grad_state else None
    for ib, b in enumerate(batches):
        for ih, h in enumerate(heads):
            gen = _gen(seed, b, h, dev)
            rn = lambda *s: torch.randn(*s, generator=gen, device=dev, dtype=torch.float32)
            out["q"][ib, :, ih] = torch.nn.functional.normalize(rn(T, K), dim=-1).to(torch.bfloat16)
            out["k"][ib, :, ih] = torch.nn.functional.normalize(rn(T, K), dim=-1).to(torch.bfloat16)
            out["v"][ib, :, ih] = rn(T, V).to(torch.bfloat16)
            out["do"][ib, :, ih] = rn(T, V).to(torch.bfloat16)
            if op == "gdn":
                a_h = torch.rand(1, generator=gen, device=dev)
                if gate == "head_exp":
                    out["g"][ib, :, ih] = -torch.exp(a_h) * torch.nn.functional.softplus(rn(T)) * gate_scale
                else:
                    out["g"][ib, :, ih] = -torch.nn.functional.softplus(rn(T)) * gate_scale
            elif op in ("kda", "gdn2"):
                out["g"][ib, :, ih] = -torch.nn.functional.softplus(rn(T, K)) * gate_scale
            if op == "gdn2":
                out["b"][ib, :, ih] = torch.sigmoid(rn(T, K)).to(torch.bfloat16)
                out["w"][ib, :, ih] = torch.sigmoid(rn(T, V)).to(torch.bfloat16)
            else:
                out["beta"][ib, :, ih] = torch.sigmoid(rn(T)).to(torch.bfloat16)
            if state:
                out["initial_state"][ib, ih] = rn(K, V) * 0.1
            if grad_state:
                out["dht"][ib, ih] = rn(K, V) * 0.1
    return out


def make_config(name, **overrides):
    cfg = dict(CONFIGS[name])
    cfg.update(overrides)
    op = cfg.pop("op")
    B, T, H = cfg.pop("B"), cfg.pop("T"), cfg.pop("H")
    return op, make_inputs(op, B, T, H, **cfg)


def operator_inputs(op, xs):
    """The subset of ``xs`` the family's forward takes (drops do/dht)."""
    names = {"delta": ("q", "k", "v", "beta"), "gdn": ("q", "k", "v", "g", "beta"),
             "kda": ("q", "k", "v", "g", "beta"), "gdn2": ("q", "k", "v", "g", "b", "w")}[op]
    d = {n: xs[n] for n in names}
    d["initial_state"] = xs.get("initial_state")
    return d
