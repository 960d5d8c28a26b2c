"""The reference's CPU-runnable path: autograd through a naive chunked forward in FP32.

The reference's CPU baseline for this operator is ``torch.autograd`` through FLA's
``naive_chunk_kda`` (third-party flash-linear-attention @ a59bc5df, fla/ops/kda/naive.py:69-166;
scalar-gate and ungated analogues fla/ops/gated_delta_rule/naive.py:67 and
fla/ops/delta_rule/naive.py:40; the GDN2 form follows src/fast_delta_rule/validation.py:32-36).
This file restates that path on top of ``oracle.chunked.chunk_forward`` evaluated in FP32
with autograd enabled.  Test / baseline infrastructure: never imported by the product.
"""
import torch
from .chunked import chunk_forward


def naive_chunk_forward(op, xs, scale=None, chunk=64, dtype=torch.float32):
    """Returns (o [B,T,H,V], final_state [B,H,K,V]); differentiable w.r.t. tensors in xs."""
    out = chunk_forward(op, xs, scale=scale, chunk=chunk, dtype=dtype)
    return out["o"], out["final_state"]


def naive_chunk_backward_fp32(op, xs, do, dht=None, scale=None, chunk=64):
    """FP32 forward + autograd backward on CPU; returns (grads dict, seconds fwd, seconds bwd)."""
    import time
    leaf = {n: x.detach().float().clone().requires_grad_() for n, x in xs.items() if x is not None}
    t0 = time.perf_counter()
    o, final = naive_chunk_forward(op, leaf, scale=scale, chunk=chunk)
    t1 = time.perf_counter()
    outputs, seeds = [o], [do.float()]
    if dht is not None:
        outputs.append(final)
        seeds.append(dht.float())
    grads = torch.autograd.grad(outputs, tuple(leaf.values()), tuple(seeds), allow_unused=True)
    t2 = time.perf_counter()
    result = {n: (g if g is not None else torch.zeros_like(x)) for (n, x), g in zip(leaf.items(), grads)}
    return result, t1 - t0, t2 - t1
