"""Chunked forward pass that produces the output and the tensors the backward contract needs.

The reference keeps FLA's Triton forward (``chunk_kda_fwd`` etc., bound at
src/fast_delta_rule/_compat/kda.py:89-113, _compat/gdn2.py:94-117, _compat/gdn.py:33-125,
_compat/delta.py).  Here ``chunk_forward`` runs the CUDA forward of librewy_b200.so (``rewy_chunk_fwd``: chunk-local
kernel, tcgen05 state scan, output kernel; the chunk-local cumulative gate is ``rewy_gate_cumsum_fwd``); CPU tensors
are refused.  ``chunk_forward_torch`` states the same forward with batched torch ops: it is the second implementation
the CUDA forward is cross-checked against and what the host-only tests run; no operator calls it.
What both return follows FLA's saved set exactly:
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
                  output_final_state=True, g_is_cumsum=False, state_v_first=False, check_status=False, cu_seqlens=None):
    """CUDA forward.  Returns dict(o, final_state, g_cumsum, Aqk, Akk, w, u, qg, kg, v_new, h).

    q,k,v BF16 [B,T,H,128]; g per-step natural-log gate ([B,T,H] for 'gdn', [B,T,H,128] for 'kda'/'gdn2', None for
    'delta') or, with ``g_is_cumsum``, already the chunk-local cumulative gate in log2 units; beta [B,T,H] or
    (b [B,T,H,128], w [B,T,H,128]) for 'gdn2'; ``state_v_first``: initial and final state are [B,H,V,K];
    ``check_status`` synchronises and raises if a kernel gave up on a bounded wait; ``cu_seqlens`` (int tensor
    [sequences + 1], lengths multiples of 64, batch of 1): packed sequences, states are [sequences,H,128,128]."""
    from . import _capi, elementwise
    if not q.is_cuda:
        raise RuntimeError("rewy_b200 chunk_forward needs CUDA tensors (there is no CPU fallback); "
                           "chunk_forward_torch is the host restatement used for cross-checks")
    B, T, H, K = k.shape
    if T % CHUNK or K != 128 or v.shape[-1] != 128 or q.dtype != torch.bfloat16:
        raise ValueError("chunk_forward needs BF16 inputs, T % 64 == 0 and K = V = 128")
    scale = K ** -0.5 if scale is None else scale
    dev = q.device
    lib = _capi.load()
    bf = lambda t: None if t is None else t.to(torch.bfloat16).contiguous()
    q, k, v = bf(q), bf(k), bf(v)
    g_cumsum = None
    with torch.cuda.device(dev):
        if op in ("kda", "gdn2"):
            g_cumsum = g.float().contiguous() if g_is_cumsum else elementwise.gate_cumsum_fwd(g)
        elif op == "gdn":
            if g_is_cumsum:
                g_cumsum = g.float().contiguous()
            else:
                gin = g if g.dtype in (torch.bfloat16, torch.float32) else g.float()
                gin = gin.contiguous()
                g_cumsum = torch.empty(gin.shape, dtype=torch.float32, device=dev)
                _capi.check(lib.rewy_scalar_gate_cumsum_fwd(_capi.ptr(gin), int(gin.dtype == torch.float32), _capi.ptr(g_cumsum),
                                                            B, T, H, _capi.current_stream(dev)), "rewy_scalar_gate_cumsum_fwd")
        big = lambda: torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=dev)
        a64 = lambda: torch.empty(B, T, H, 64, dtype=torch.bfloat16, device=dev)
        out = dict(o=big(), Aqk=a64(), Akk=a64(), w=big(), u=big(), qg=big(), kg=big(), v_new=big(),
                   h=torch.empty(B, T // CHUNK, H, 128, 128, dtype=torch.bfloat16, device=dev))
        cu = None if cu_seqlens is None else cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        if cu is not None and B != 1:
            raise ValueError("chunk_forward: packed sequences (cu_seqlens) need a batch of 1")
        nseq = B if cu is None else cu.numel() - 1
        final = torch.empty(nseq, H, 128, 128, dtype=torch.float32, device=dev) if output_final_state else None
        ctrl = torch.empty(2, dtype=torch.int32, device=dev)
        a = _capi.FwdArgs()
        a.family, a.B, a.T, a.H, a.state_v_first, a.scale = _capi.FAMILY_ID[op], B, T, H, int(bool(state_v_first)), float(scale)
        keep = [q, k, v, g_cumsum, None if beta is None else beta.float().contiguous(), bf(b), bf(w),
                None if initial_state is None else initial_state.float().contiguous()]
        for name, t in zip(("q", "k", "v", "g", "beta", "b_gate", "w_gate", "h0"), keep):
            setattr(a, name, _capi.ptr(t))
        for name, t in out.items():
            setattr(a, name, _capi.ptr(t))
        a.final_state, a.ctrl = _capi.ptr(final), _capi.ptr(ctrl)
        if cu is not None:
            a.cu_seqlens, a.num_seqs = _capi.ptr(cu), nseq
        _capi.check(lib.rewy_chunk_fwd(a, _capi.current_stream(dev)), "rewy_chunk_fwd")
        if check_status:
            _capi.check(lib.rewy_device_status(_capi.ptr(ctrl), _capi.current_stream(dev)), "device status (forward)")
    out.update(final_state=final, g_cumsum=g_cumsum)
    return out


@torch.no_grad()
def chunk_forward_torch(op, q, k, v, g=None, beta=None, b=None, w=None, scale=None, initial_state=None,
                        output_final_state=True, g_is_cumsum=False):
    """The same forward with batched torch ops on the inputs' device (cross-check implementation).
    Returns dict(o, final_state, g_cumsum, Aqk, Akk, w, u, qg, kg, v_new, h).

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
