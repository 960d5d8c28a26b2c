"""Chunked forward pass that produces the tensors the backward contract needs.

The reference keeps FLA's Triton forward (``chunk_kda_fwd`` etc., bound at
src/fast_delta_rule/_compat/kda.py:89-113, _compat/gdn2.py:94-117, _compat/gdn.py:33-125,
_compat/delta.py); that library revision is not part of this package, so the forward half is
stated here with batched torch ops on the inputs' device.  It is outside the timed backward.
What it returns follows FLA's saved set exactly:
  g_cumsum  FP32 chunk-local cumulative gate in LOG2 units (scale RCP_LN2, _compat/gdn.py:52-69)
  Aqk, Akk  BF16 [B,T,H,64]; Akk = (I + tril(E Y^T,-1))^-1 without beta, Aqk = scale*tril(Qg Y^T)
  w,u,qg,kg,v_new  BF16 [B,T,H,128]; h BF16 [B,T/64,H,128,128] (state entering each chunk)
Operands of every product are rounded to BF16 and accumulated in FP32 like the tensor-core path.
"""
import math
import torch

RCP_LN2 = 1.0 / math.log(2.0)
CHUNK = 64


def _chunks(x):
    B, T, H = x.shape[:3]
    return x.reshape(B, T // CHUNK, CHUNK, H, *x.shape[3:]).movedim(3, 1)      # [B,H,NT,C,...]


def _unchunks(x):
    x = x.movedim(1, 3)
    B, NT, C, H = x.shape[:4]
    return x.reshape(B, NT * C, H, *x.shape[4:])


def _bf(x):
    return x.to(torch.bfloat16).to(torch.float32)


@torch.no_grad()
def chunk_forward(op, q, k, v, g=None, beta=None, b=None, w=None, scale=None, initial_state=None,
                  output_final_state=True, g_is_cumsum=False):
    """Returns dict(o, final_state, g_cumsum, Aqk, Akk, w, u, qg, kg, v_new, h).

    q,k,v BF16 [B,T,H,128]; g per-step natural-log gate FP32 ([B,T,H] for 'gdn', [B,T,H,128] for
    'kda'/'gdn2', None for 'delta'); beta [B,T,H] or (b [B,T,H,128], w [B,T,H,128]) for 'gdn2'."""
    B, T, H, K = k.shape
    V = v.shape[-1]
    if T % CHUNK or K != 128 or V != 128:
        raise ValueError("chunk_forward needs T % 64 == 0 and K = V = 128")
    scale = K ** -0.5 if scale is None else scale
    outs = []
    for ib in range(B):  # one batch element at a time bounds the FP32 temporaries
        sl = slice(ib, ib + 1)
        outs.append(_forward_one(op, q[sl], k[sl], v[sl], None if g is None else g[sl],
                                 None if beta is None else beta[sl], None if b is None else b[sl],
                                 None if w is None else w[sl], scale,
                                 None if initial_state is None else initial_state[sl], g_is_cumsum))
    res = {n: (None if outs[0][n] is None else torch.cat([o[n] for o in outs], 0)) for n in outs[0]}
    if not output_final_state:
        res["final_state"] = None
    return res


def _forward_one(op, q, k, v, g, beta, b, w, scale, h0, g_is_cumsum):
    f32 = torch.float32
    dev = k.device
    qc, kc, vc = (_chunks(x.to(f32)) for x in (q, k, v))              # [1,H,NT,C,D]
    _, H, NT, C, K = kc.shape
    V = vc.shape[-1]
    if op == "delta":
        G = torch.zeros(1, H, NT, C, 1, dtype=f32, device=dev)
        g_cumsum = None
    else:
        gc = _chunks(g.to(f32))
        if op == "gdn":
            gc = gc[..., None]
        G = gc if g_is_cumsum else gc.cumsum(3) * RCP_LN2
        g_cumsum = _unchunks(G if op != "gdn" else G[..., 0]).contiguous()
    if op == "gdn2":
        bc, wc = _chunks(b.to(f32)), _chunks(w.to(f32))
    else:
        bc = wc = _chunks(beta.to(f32))[..., None]
    # centred gate factors keep exp2 in range; very wide chunks fall back to FP64 for the two matrices
    lo, hi = G.amin(3, keepdim=True), G.amax(3, keepdim=True)
    cen = 0.5 * (lo + hi)
    wide = bool(((hi - lo) >= 80).any()) if op != "delta" else False
    mt = torch.float64 if wide else f32
    alpha, zeta = torch.exp2((G - cen).to(mt)), torch.exp2((cen - G).to(mt))
    ka, kz = kc.to(mt) * alpha, kc.to(mt) * zeta
    M = torch.tril((bc.to(mt) * ka) @ kz.transpose(-1, -2), -1)
    eye = torch.eye(C, dtype=mt, device=dev)
    Akk = torch.linalg.solve_triangular(M + eye, eye.expand_as(M), upper=False).to(f32)
    Aqk = (scale * torch.tril((qc.to(mt) * alpha) @ kz.transpose(-1, -2))).to(f32)
    del M, ka, kz, alpha, zeta
    Akk_b, Aqk_b = _bf(Akk), _bf(Aqk)
    gamma = torch.exp2(G)
    Glast = G[..., -1:, :]
    E_b = _bf(bc * kc * gamma)
    Z_b = _bf(wc * vc)
    w_wy = _bf(Akk_b @ E_b)
    u = _bf(Akk_b @ Z_b)
    qg = _bf(qc * gamma)
    kg = _bf(kc * torch.exp2(Glast - G))
    lam = torch.exp2(Glast).transpose(-1, -2)                           # [1,H,NT,K|1,1]
    S = torch.zeros(1, H, K, V, dtype=f32, device=dev) if h0 is None else h0.to(f32).clone()
    h = torch.empty(1, NT, H, K, V, dtype=torch.bfloat16, device=dev)
    v_new = torch.empty(1, H, NT, C, V, dtype=f32, device=dev)
    o = torch.empty(1, H, NT, C, V, dtype=f32, device=dev)
    for n in range(NT):
        Sb = S.to(torch.bfloat16)
        h[:, n] = Sb
        Sb = Sb.to(f32)
        R = _bf(u[:, :, n] - w_wy[:, :, n] @ Sb)
        v_new[:, :, n] = R
        o[:, :, n] = scale * (qg[:, :, n] @ Sb) + Aqk_b[:, :, n] @ R
        S = lam[:, :, n] * S + kg[:, :, n].transpose(-1, -2) @ R
    bf = lambda x: _unchunks(x).to(torch.bfloat16).contiguous()
    return dict(o=bf(o), final_state=S, g_cumsum=g_cumsum, Aqk=bf(Aqk_b), Akk=bf(Akk_b), w=bf(w_wy), u=bf(u),
                qg=bf(qg.expand_as(qc)), kg=bf(kg.expand_as(kc)), v_new=bf(v_new), h=h)
