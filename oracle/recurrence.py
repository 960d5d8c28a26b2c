"""FP64 token recurrence of the four delta-rule families and its autograd gradients.

Restates the reference's acceptance oracle
(src/fast_delta_rule/validation.py:23-38, ``recurrence``) and the research
harness' variant (research/operators/run_cuda.py:37-51).  Test infrastructure:
never imported by the product package.

Families (``op``):
  'delta' : S_t = S_{t-1} + k_t (beta_t (v_t - k_t^T S_{t-1}))^T
  'gdn'   : as delta, after S_{t-1} <- exp(g_t) S_{t-1}, g_t scalar per head
  'kda'   : as gdn with g_t a vector over the key dimension
  'gdn2'  : S_t = D_t S_{t-1} + k_t (w_t * v_t - (b_t * k_t)^T D_t S_{t-1})^T,
            vector erase gate b_t [K] and write gate w_t [V]
Output o_t = (scale * q_t)^T S_t, scale = K^-1/2.  Gates are natural-log per step.
"""
import torch


def recurrence(op, xs, scale=None):
    """xs: dict with q,k,v [B,T,H,D]; g ([B,T,H] gdn, [B,T,H,K] kda/gdn2);
    beta [B,T,H] or b,w [B,T,H,D] (gdn2); initial_state [B,H,K,V] or None.
    Returns (o [B,T,H,V], final_state [B,H,K,V]) in the dtype of q (use float64)."""
    q, k, v = xs["q"], xs["k"], xs["v"]
    B, T, H, K = k.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    state = xs.get("initial_state")
    if state is None:
        state = torch.zeros(B, H, K, V, dtype=q.dtype)
    outs = []
    for t in range(T):
        if op != "delta":
            g = xs["g"][:, t]
            if op == "gdn":
                g = g[..., None]
            state = state * g.exp()[..., None]
        kt = k[:, t]
        if op == "gdn2":
            residual = xs["w"][:, t] * v[:, t] - torch.einsum("bhk,bhkv->bhv", xs["b"][:, t] * kt, state)
        else:
            residual = xs["beta"][:, t, :, None] * (v[:, t] - torch.einsum("bhk,bhkv->bhv", kt, state))
        state = state + kt[..., None] * residual[..., None, :]
        outs.append(torch.einsum("bhk,bhkv->bhv", q[:, t] * scale, state))
    return torch.stack(outs, 1), state


def recurrence_grads(op, xs, do, dht=None, scale=None):
    """Gradients of sum(o*do) + sum(final_state*dht) w.r.t. every tensor in xs, in FP64."""
    leaf = {n: x.detach().double().clone().requires_grad_() for n, x in xs.items() if x is not None}
    o, final = recurrence(op, leaf, scale)
    outputs, seeds = [o], [do.double()]
    if dht is not None:
        outputs.append(final)
        seeds.append(dht.double())
    grads = torch.autograd.grad(outputs, tuple(leaf.values()), tuple(seeds), allow_unused=True)
    result = {n: (g if g is not None else torch.zeros_like(x)) for (n, x), g in zip(leaf.items(), grads)}
    return result, o.detach(), final.detach()
