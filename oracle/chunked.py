"""Closed-form chunked forward intermediates and backward in FP64, in the layouts the
backward operators exchange.  Test infrastructure: never imported by the product.

Algebra follows the reference's NumPy statement of one chunk
(benchmarks/plotting/check_manuscript_math.py:21-43, ``backward``) and its chunk chaining
(:102-124, ``backward_partitioned``); layouts and what is saved follow the autograd
contracts (src/fast_delta_rule/_compat/kda.py:89-157, _compat/gdn2.py:94-127,
_compat/gdn.py:166-205, _compat/delta.py) and the kernels' data contracts
(kernels/kda_residual_local_beta_consumer.py:80-96 for token-major indexing,
kernels/vector_state_gpu.py:31-44 for ``dh``/``dR``/``dh0``).

Conventions (per chunk of C=64 rows, per head):
  G      chunk-local inclusive cumulative gate in LOG2 units (``g_cumsum`` as FLA saves it),
         gamma = exp2(G); scalar families broadcast G over K; 'delta' has G = 0.
  E = b*k*gamma, Y = k/gamma, Z = w*v, Qg = q*gamma (unscaled), lam = gamma[last row]
  Akk = (I + tril(E Y^T, -1))^-1          (beta NOT folded in)
  Aqk = scale * tril(Qg Y^T)              (diagonal included)
  w_wy = Akk E, u = Akk Z, qg = Qg, kg = k*exp2(G_last - G)
  v_new = R = u - w_wy h[n],  h[n+1] = lam*h[n] + kg^T R,  o = scale*Qg h[n] + Aqk R
Backward given do and the gradient dS of the state leaving the chunk:
  dR = Aqk^T do + kg dS;  P = Akk^T dR;  dAqk = scale*tril(do R^T);  dAkk = -tril(P R^T, -1)
  qgb = scale*do h^T + dAqk Y;  eb = -P h^T + dAkk Y;  fb = R dS^T
  yb = dAqk^T Qg + dAkk^T E + fb*lam;  dS_in = lam*dS + scale*qg^T do - w_wy^T dR
  dq = gamma*qgb;  dk = gamma*b*eb + yb/gamma;  db = gamma*k*eb;  dv = w*P;  dw = v*P
  dG_row = Qg*qgb + E*eb - Y*yb;  last row += lam*(sum_v h*dS + sum_rows Y*fb)
  dg (per-step natural-log gate) = reverse chunk-local cumsum of dG_row.
"""
import math
import torch

FAMILIES = ("delta", "gdn", "kda", "gdn2")
RCP_LN2 = 1.0 / math.log(2.0)


def _chunks(x, C):
    """[B,T,H,...] -> [B,H,NT,C,...]"""
    B, T, H = x.shape[:3]
    x = x.reshape(B, T // C, C, H, *x.shape[3:])
    return x.movedim(3, 1)


def _unchunks(x):
    """[B,H,NT,C,...] -> [B,T,H,...]"""
    x = x.movedim(1, 3)
    B, NT, C, H = x.shape[:4]
    return x.reshape(B, NT * C, H, *x.shape[4:])


def _gates(op, xs, C, dtype):
    """Return (G log2 cumsum in chunk layout broadcastable to K, b, w) in chunk layout."""
    k = xs["k"]
    B, T, H, K = k.shape
    V = xs["v"].shape[-1]
    if op == "delta":
        G = torch.zeros(B, H, T // C, C, 1, dtype=dtype)
    elif "g_cumsum" in xs and xs["g_cumsum"] is not None:
        G = _chunks(xs["g_cumsum"].to(dtype), C)
        if op == "gdn":
            G = G[..., None]
    else:
        g = _chunks(xs["g"].to(dtype), C)
        if op == "gdn":
            g = g[..., None]
        G = g.cumsum(3) * RCP_LN2
    if op == "gdn2":
        b = _chunks(xs["b"].to(dtype), C)
        w = _chunks(xs["w"].to(dtype), C)
    else:
        beta = _chunks(xs["beta"].to(dtype), C)[..., None]
        b, w = beta, beta
    return G, b, w


def chunk_forward(op, xs, scale=None, chunk=64, dtype=torch.float64):
    """Forward pass in chunked form; returns every tensor the backward contract names.

    xs: q,k,v [B,T,H,D]; g per-step natural-log gate ([B,T,H] gdn, [B,T,H,K] kda/gdn2);
    beta [B,T,H] or b [B,T,H,K], w [B,T,H,V]; initial_state [B,H,K,V] or None."""
    C = chunk
    q, k, v = (_chunks(xs[n].to(dtype), C) for n in ("q", "k", "v"))
    B, H, NT, _, K = k.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    G, b, w = _gates(op, xs, C, dtype)
    gamma = torch.exp2(G)
    E = b * k * gamma
    Y = k / gamma
    Z = w * v
    Qg = q * gamma
    eye = torch.eye(C, dtype=dtype)
    M = eye + torch.tril(E @ Y.transpose(-1, -2), -1)
    Akk = torch.linalg.solve_triangular(M, eye.expand_as(M), upper=False)
    Aqk = scale * torch.tril(Qg @ Y.transpose(-1, -2))
    w_wy = Akk @ E
    u = Akk @ Z
    Glast = G[..., -1:, :]
    lam = torch.exp2(Glast)                      # [B,H,NT,1,K or 1]
    kg = k * torch.exp2(Glast - G)
    h0 = xs.get("initial_state")
    S = torch.zeros(B, H, K, V, dtype=dtype) if h0 is None else h0.to(dtype).clone()
    hs, Rs, os_ = [], [], []
    for n in range(NT):
        hs.append(S)
        R = u[:, :, n] - w_wy[:, :, n] @ S
        Rs.append(R)
        os_.append(scale * Qg[:, :, n] @ S + Aqk[:, :, n] @ R)
        S = lam[:, :, n].transpose(-1, -2) * S + kg[:, :, n].transpose(-1, -2) @ R
    h = torch.stack(hs, 2)                       # [B,H,NT,K,V]
    R = torch.stack(Rs, 2)
    o = torch.stack(os_, 2)
    Gout = G if op in ("kda", "gdn2") else G[..., 0]
    out = dict(
        g_cumsum=None if op == "delta" else _unchunks(Gout),
        Aqk=_unchunks(Aqk), Akk=_unchunks(Akk), w=_unchunks(w_wy), u=_unchunks(u),
        qg=_unchunks(Qg.expand_as(q)), kg=_unchunks(kg.expand_as(k)), v_new=_unchunks(R),
        h=h.transpose(1, 2).contiguous(),        # [B,NT,H,K,V]
        o=_unchunks(o), final_state=S,
    )
    return out


def chunk_backward(op, xs, saved, do, dht=None, scale=None, chunk=64, dtype=torch.float64):
    """Closed-form backward from the saved tensors of ``chunk_forward`` (or any forward that
    honours the same contract, e.g. BF16-rounded ones upcast by the caller).

    saved must hold g_cumsum (unless 'delta'), Aqk, Akk, w, qg, kg, v_new, h.
    Returns dict with dq,dk,dv,dg and dbeta (or db,dw for gdn2), dh0, plus the inter-stage
    tensors dAqk,dAkk [B,T,H,64], dR (=dv2 of the scan), P [B,T,H,V], dh [B,NT,H,K,V]."""
    C = chunk
    q, k, v = (_chunks(xs[n].to(dtype), C) for n in ("q", "k", "v"))
    B, H, NT, _, K = k.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    xg = dict(xs)
    xg["g_cumsum"] = saved.get("g_cumsum")
    G, b, w = _gates(op, xg, C, dtype)
    gamma = torch.exp2(G)
    Glast = G[..., -1:, :]
    lam = torch.exp2(Glast)
    Aqk, Akk, w_wy, qg, kg, R = (_chunks(saved[n].to(dtype), C) for n in ("Aqk", "Akk", "w", "qg", "kg", "v_new"))
    h = saved["h"].to(dtype).transpose(1, 2)     # [B,H,NT,K,V]
    dO = _chunks(do.to(dtype), C)
    E = b * k * gamma
    Y = k / gamma
    Qg = q * gamma
    dS = torch.zeros(B, H, K, V, dtype=dtype) if dht is None else dht.to(dtype).clone()
    T_ = lambda x: x.transpose(-1, -2)
    outs = {n: [None] * NT for n in ("dq", "dk", "dv", "db", "dw", "dgrow", "dAqk", "dAkk", "dR", "P", "dh")}
    for n in reversed(range(NT)):
        outs["dh"][n] = dS
        dR = T_(Aqk[:, :, n]) @ dO[:, :, n] + kg[:, :, n] @ dS
        P = T_(Akk[:, :, n]) @ dR
        Hm = scale * torch.tril(dO[:, :, n] @ T_(R[:, :, n]))
        Dm = -torch.tril(P @ T_(R[:, :, n]), -1)
        fb = R[:, :, n] @ T_(dS)
        qgb = scale * dO[:, :, n] @ T_(h[:, :, n]) + Hm @ Y[:, :, n]
        eb = -P @ T_(h[:, :, n]) + Dm @ Y[:, :, n]
        lam_n = lam[:, :, n]                      # [B,H,1,K|1]
        yb = T_(Hm) @ Qg[:, :, n] + T_(Dm) @ E[:, :, n] + fb * lam_n
        gam = gamma[:, :, n]
        outs["dq"][n] = gam * qgb
        outs["dk"][n] = gam * b[:, :, n] * eb + yb / gam
        outs["db"][n] = gam * k[:, :, n] * eb
        outs["dv"][n] = w[:, :, n] * P
        outs["dw"][n] = v[:, :, n] * P
        grow = Qg[:, :, n] * qgb + E[:, :, n] * eb - Y[:, :, n] * yb
        end = lam_n[..., 0, :] * ((h[:, :, n] * dS).sum(-1) + (Y[:, :, n] * fb).sum(-2))
        grow = grow.clone()
        grow[..., -1, :] = grow[..., -1, :] + end
        outs["dgrow"][n] = grow
        outs["dAqk"][n], outs["dAkk"][n], outs["dR"][n], outs["P"][n] = Hm, Dm, dR, P
        dS = T_(lam_n) * dS + scale * T_(qg[:, :, n]) @ dO[:, :, n] - T_(w_wy[:, :, n]) @ dR
    st = {n: torch.stack(x, 2) for n, x in outs.items()}
    res = dict(dq=_unchunks(st["dq"]), dk=_unchunks(st["dk"]), dv=_unchunks(st["dv"]),
               dAqk=_unchunks(st["dAqk"]), dAkk=_unchunks(st["dAkk"]), dR=_unchunks(st["dR"]),
               P=_unchunks(st["P"]), dh=st["dh"].transpose(1, 2).contiguous(), dh0=dS)
    if op == "gdn2":
        res["db"] = _unchunks(st["db"])
        res["dw"] = _unchunks(st["dw"])
    else:
        res["dbeta"] = _unchunks(st["db"].sum(-1) + st["dw"].sum(-1))
    if op != "delta":
        grow = st["dgrow"]
        if op == "gdn":
            grow = grow.sum(-1)
            dg = grow.flip(3).cumsum(3).flip(3)
        else:
            dg = grow.flip(3).cumsum(3).flip(3)
        res["dg"] = _unchunks(dg)
    return res
