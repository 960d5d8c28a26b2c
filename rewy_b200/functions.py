"""Autograd functions and public operators of the four families.

Same contracts as the reference's private autograd copies (src/fast_delta_rule/_compat/kda.py:23-210,
gdn.py:128-267, gdn2.py:43-201, delta.py:19-141): the forward saves FLA's tensor set (policy
``disable_recompute`` decides whether w,u,qg,kg,v_new,h are kept), the backward hands them to the
whole-family backward of ``rewy_b200.backward`` and casts to the input dtypes.  The wrapper-level options the
reference accepts for KDA on CUDA (fused gate activation, beta sigmoid, q/k L2 normalisation, value-first state
layout: docs/compatibility.md:12-13, tests/test_accelerator.py:65-83) run as CUDA passes of ``rewy_b200.elementwise``.  The backward stays bound
to this implementation after a ``use_backend`` context exits, like the reference's.
"""
import torch

from . import backward as _bwd
from .forward import chunk_forward


from . import elementwise as _ew


def _cumulative_gate(g, A_log=None, dt_bias=None):
    """Chunk-local cumulative gate in log2 units on the device (vector gates), optionally with the KDA gate activation."""
    return _ew.gate_cumsum_fwd(g, A_log, dt_bias)


class ChunkKDAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
                use_gate_in_kernel, use_beta_sigmoid_in_kernel, allow_neg_eigval, disable_recompute, state_v_first,
                cu_seqlens):
        q_rstd = k_rstd = None
        if use_qk_l2norm_in_kernel:
            q, q_rstd = _ew.l2norm_fwd(q)
            k, k_rstd = _ew.l2norm_fwd(k)
        beta_raw = beta
        if use_beta_sigmoid_in_kernel:
            beta = _ew.beta_sigmoid_fwd(beta_raw, 2.0 if allow_neg_eigval else 1.0)
        # with use_gate_in_kernel, g is the raw gate input: -exp(A_log) * softplus(g + dt_bias) and the chunk cumsum are
        # one pass; otherwise g is the per-step natural-log decay
        g_cumsum = _cumulative_gate(g, A_log if use_gate_in_kernel else None, dt_bias if use_gate_in_kernel else None)
        f = chunk_forward("kda", q, k, v, g=g_cumsum, beta=beta, scale=scale, initial_state=initial_state,
                          output_final_state=output_final_state, g_is_cumsum=True, state_v_first=state_v_first,
                          cu_seqlens=cu_seqlens)
        keep = (lambda x: x) if disable_recompute else (lambda x: None)
        ctx.save_for_backward(q, q_rstd, k, k_rstd, v, g_cumsum, g, beta_raw, beta, A_log, dt_bias, f["Aqk"], f["Akk"],
                              keep(f["w"]), keep(f["u"]), keep(f["qg"]), keep(f["kg"]), keep(f["v_new"]),
                              keep(f["h"]), initial_state, cu_seqlens)
        ctx.scale, ctx.disable_recompute = scale, disable_recompute
        ctx.use_qk_l2norm_in_kernel, ctx.use_beta_sigmoid_in_kernel = use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel
        ctx.use_gate_in_kernel, ctx.allow_neg_eigval, ctx.state_v_first = use_gate_in_kernel, allow_neg_eigval, state_v_first
        return f["o"].type_as(q), f["final_state"]

    @staticmethod
    def backward(ctx, do, dht):
        (q, q_rstd, k, k_rstd, v, g_cumsum, g_input, beta_raw, beta, A_log, dt_bias, Aqk, Akk, w, u, qg, kg, v_new, h,
         initial_state, cu_seqlens) = ctx.saved_tensors
        dq, dk, dv, db, dg, dh0, _, _ = _bwd.kda_backward(
            q=q, k=k, v=v, beta=beta, Aqk=Aqk, Akk=Akk, scale=ctx.scale, initial_state=initial_state, do=do, dht=dht,
            g=g_cumsum, state_v_first=ctx.state_v_first, cu_seqlens=cu_seqlens, disable_recompute=ctx.disable_recompute, w=w, u=u, qg=qg, kg=kg,
            v_new=v_new, h=h, out_dtype=torch.float32 if ctx.use_qk_l2norm_in_kernel else torch.bfloat16)
        dA = dbias = None
        if ctx.use_gate_in_kernel:
            dg, dA, dbias = _ew.gate_act_bwd(g_input, A_log, dt_bias, dg)
            dA = dA.view_as(A_log).to(A_log.dtype)
            dbias = None if dbias is None else dbias.view_as(dt_bias).to(dt_bias.dtype)
        if ctx.use_qk_l2norm_in_kernel:
            dq = _ew.l2norm_bwd(q, q_rstd, dq)
            dk = _ew.l2norm_bwd(k, k_rstd, dk)
        if ctx.use_beta_sigmoid_in_kernel:
            db = _ew.beta_sigmoid_bwd(beta_raw, db, 2.0 if ctx.allow_neg_eigval else 1.0)
        return (dq.to(q), dk.to(k), dv.to(v), dg.to(g_input), db.to(beta_raw), dA, dbias, None, dh0, None, None, None,
                None, None, None, None, None)


class ChunkGDN2Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, b, w, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
                disable_recompute, state_v_first, cu_seqlens):
        q_rstd = k_rstd = None
        if use_qk_l2norm_in_kernel:
            q, q_rstd = _ew.l2norm_fwd(q)
            k, k_rstd = _ew.l2norm_fwd(k)
        g_cumsum = _cumulative_gate(g)
        f = chunk_forward("gdn2", q, k, v, g=g_cumsum, b=b, w=w, scale=scale, initial_state=initial_state,
                          output_final_state=output_final_state, g_is_cumsum=True, state_v_first=state_v_first,
                          cu_seqlens=cu_seqlens)
        keep = (lambda x: x) if disable_recompute else (lambda x: None)
        ctx.save_for_backward(q, q_rstd, k, k_rstd, v, g_cumsum, g, b, w, f["Aqk"], f["Akk"], keep(f["w"]),
                              keep(f["u"]), keep(f["qg"]), keep(f["kg"]), keep(f["v_new"]), keep(f["h"]), initial_state,
                              cu_seqlens)
        ctx.scale, ctx.disable_recompute, ctx.use_qk_l2norm_in_kernel = scale, disable_recompute, use_qk_l2norm_in_kernel
        ctx.state_v_first = state_v_first
        return f["o"].type_as(q), f["final_state"]

    @staticmethod
    def backward(ctx, do, dht):
        (q, q_rstd, k, k_rstd, v, g_cumsum, g_input, b, w, Aqk, Akk, w_wy, u_wy, qg, kg, v_new, h,
         initial_state, cu_seqlens) = ctx.saved_tensors
        dq, dk, dv, db, dw, dg, dh0, _, _ = _bwd.gdn2_backward(
            q=q, k=k, v=v, b=b, w_gate=w, Aqk=Aqk, Akk=Akk, scale=ctx.scale, initial_state=initial_state, do=do,
            dht=dht, g=g_cumsum, state_v_first=ctx.state_v_first, cu_seqlens=cu_seqlens, w_wy=w_wy, u_wy=u_wy, qg=qg, kg=kg, v_new=v_new, h=h,
            disable_recompute=ctx.disable_recompute,
            out_dtype=torch.float32 if ctx.use_qk_l2norm_in_kernel else torch.bfloat16)
        if ctx.use_qk_l2norm_in_kernel:
            dq = _ew.l2norm_bwd(q, q_rstd, dq)
            dk = _ew.l2norm_bwd(k, k_rstd, dk)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dg.to(g_input.dtype), db.to(b.dtype), dw.to(w.dtype),
                None, dh0, None, None, None, None, None)


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel,
                use_beta_sigmoid_in_kernel, allow_neg_eigval, state_v_first, cu_seqlens):
        q_rstd = k_rstd = None
        if use_qk_l2norm_in_kernel:
            q, q_rstd = _ew.l2norm_fwd(q)
            k, k_rstd = _ew.l2norm_fwd(k)
        beta_raw = beta
        if use_beta_sigmoid_in_kernel:
            beta = _ew.beta_sigmoid_fwd(beta_raw, 2.0 if allow_neg_eigval else 1.0)
        f = chunk_forward("gdn", q, k, v, g=g, beta=beta, scale=scale, initial_state=initial_state,
                          output_final_state=output_final_state, state_v_first=state_v_first, cu_seqlens=cu_seqlens)
        ctx.save_for_backward(q, q_rstd, k, k_rstd, v, f["g_cumsum"], g, beta_raw, beta, f["Akk"], initial_state, cu_seqlens)
        ctx.scale, ctx.use_qk_l2norm_in_kernel = scale, use_qk_l2norm_in_kernel
        ctx.use_beta_sigmoid_in_kernel, ctx.allow_neg_eigval = use_beta_sigmoid_in_kernel, allow_neg_eigval
        ctx.state_v_first = state_v_first
        return f["o"].to(q.dtype), f["final_state"]

    @staticmethod
    def backward(ctx, do, dht):
        q, q_rstd, k, k_rstd, v, g, g_input, beta_raw, beta, A, initial_state, cu_seqlens = ctx.saved_tensors
        dq, dk, dv, db, dg, dh0, _, _ = _bwd.gdn_backward(
            q=q, k=k, v=v, g=g, beta=beta, A=A, scale=ctx.scale, initial_state=initial_state, do=do, dht=dht,
            state_v_first=ctx.state_v_first, cu_seqlens=cu_seqlens,
            out_dtype=torch.float32 if ctx.use_qk_l2norm_in_kernel else torch.bfloat16)
        if ctx.use_qk_l2norm_in_kernel:
            dq = _ew.l2norm_bwd(q, q_rstd, dq)
            dk = _ew.l2norm_bwd(k, k_rstd, dk)
        if ctx.use_beta_sigmoid_in_kernel:
            db = _ew.beta_sigmoid_bwd(beta_raw, db, 2.0 if ctx.allow_neg_eigval else 1.0)
        return (dq.to(q), dk.to(k), dv.to(v), dg.to(g_input), db.to(beta_raw), None, dh0, None, None, None, None, None,
                None)


class ChunkDeltaRuleFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, beta, scale, initial_state, output_final_state, use_qk_l2norm_in_kernel, cu_seqlens):
        q_rstd = k_rstd = None
        if use_qk_l2norm_in_kernel:
            q, q_rstd = _ew.l2norm_fwd(q)
            k, k_rstd = _ew.l2norm_fwd(k)
        f = chunk_forward("delta", q, k, v, beta=beta, scale=scale, initial_state=initial_state,
                          output_final_state=output_final_state, cu_seqlens=cu_seqlens)
        ctx.save_for_backward(q, q_rstd, k, k_rstd, v, beta, f["Akk"], initial_state, cu_seqlens)
        ctx.scale, ctx.use_qk_l2norm_in_kernel = scale, use_qk_l2norm_in_kernel
        return f["o"].to(q.dtype), f["final_state"]

    @staticmethod
    def backward(ctx, do, dht):
        q, q_rstd, k, k_rstd, v, beta, A, initial_state, cu_seqlens = ctx.saved_tensors
        dq, dk, dv, db, dh0 = _bwd.delta_backward(
            q=q, k=k, v=v, beta=beta, A=A, scale=ctx.scale, initial_state=initial_state, do=do, dht=dht,
            cu_seqlens=cu_seqlens,
            out_dtype=torch.float32 if ctx.use_qk_l2norm_in_kernel else torch.bfloat16)
        if ctx.use_qk_l2norm_in_kernel:
            dq = _ew.l2norm_bwd(q, q_rstd, dq)
            dk = _ew.l2norm_bwd(k, k_rstd, dk)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), db.to(beta.dtype), None, dh0, None, None, None


def _packed(cu_seqlens, q):
    """cu_seqlens as an int32 device tensor (the dispatch layer has already checked that every length is a multiple
    of 64), or None."""
    return None if cu_seqlens is None else cu_seqlens.to(device=q.device, dtype=torch.int32).contiguous()


class _Ragged:
    """Lengths that are not multiples of the chunk: every sequence is extended to the next multiple of 64 by neutral
    tokens (q = k = v = 0, no decay), which change neither the state nor any real token's output, and the results are
    cut back.  The padding and the cut are ordinary differentiable tensor operations around the autograd function, so
    the gradients of the real tokens come out by themselves.  FLA handles such lengths by bounds checks inside its
    kernels (the reference's release envelope rejects them: src/fast_delta_rule/runtime.py:87-88)."""

    def __init__(self, T, device, cu_seqlens=None, cu_seqlens_cpu=None):
        self.T, self.index, self.cu = T, None, None
        if cu_seqlens is None:
            self.total = -(-T // 64) * 64
            self.needed = self.total != T
            return
        host = (cu_seqlens if cu_seqlens_cpu is None else cu_seqlens_cpu).detach().cpu().to(torch.int64)
        lengths = host[1:] - host[:-1]
        padded = (lengths + 63) // 64 * 64
        self.needed = bool((padded != lengths).any())
        if not self.needed:
            return
        starts = torch.cumsum(padded, 0) - padded
        self.total = int(padded.sum())
        self.index = torch.cat([torch.arange(int(n)) + int(s) for n, s in zip(lengths, starts)]).to(device)
        self.cu = torch.cat([starts, starts[-1:] + padded[-1:]]).to(device=device, dtype=torch.int32)

    def pad(self, x, fill=0.0):
        """x [B, T, ...] -> [B, padded T, ...]"""
        if x is None or not self.needed:
            return x
        if self.index is None:
            tail = x.new_full((x.shape[0], self.total - self.T) + tuple(x.shape[2:]), fill)
            return torch.cat([x, tail], 1)
        return x.new_full((x.shape[0], self.total) + tuple(x.shape[2:]), fill).index_copy(1, self.index, x)

    def cut(self, o):
        if not self.needed:
            return o
        return o[:, :self.T] if self.index is None else o.index_select(1, self.index)


def _common_checks(q, k, v, initial_state):
    if q.shape != k.shape:
        raise ValueError(f"q and k must have the same shape, got q={tuple(q.shape)} vs k={tuple(k.shape)}")
    if initial_state is not None and initial_state.dtype != torch.float32:
        raise ValueError("initial_state must be in float32.")
    if v.shape[2] != q.shape[2] and (v.shape[2] < q.shape[2] or v.shape[2] % q.shape[2] != 0):
        raise ValueError(f"the value heads ({v.shape[2]}) must be a multiple of the query/key heads ({q.shape[2]})")


class _Narrow:
    """Head dimensions below 128: the key and value channels are filled up with zeros (exact: a zero channel adds
    nothing to any product and its state rows stay zero) and outputs and states are cut back.  The scale keeps the
    caller's K.  Everything here is differentiable tensor code around the autograd function."""

    def __init__(self, q, v):
        self.K, self.V = q.shape[-1], v.shape[-1]
        if self.K > 128 or self.V > 128:
            raise ValueError(f"head dimensions above 128 are not supported (K={self.K}, V={self.V})")
        self.needed = self.K != 128 or self.V != 128

    def key(self, x):    # [..., K] -> [..., 128]
        return x if x is None or not self.needed else torch.nn.functional.pad(x, (0, 128 - self.K))

    def value(self, x):  # [..., V] -> [..., 128]
        return x if x is None or not self.needed else torch.nn.functional.pad(x, (0, 128 - self.V))

    def state(self, h, v_first=False):  # [N,H,K,V] (or [N,H,V,K]) -> [N,H,128,128]
        if h is None or not self.needed:
            return h
        last, first = (self.K, self.V) if v_first else (self.V, self.K)
        return torch.nn.functional.pad(h, (0, 128 - last, 0, 128 - first))

    def cut(self, o, final_state, v_first=False):
        if not self.needed:
            return o, final_state
        if final_state is not None:
            final_state = final_state[..., :self.V, :self.K] if v_first else final_state[..., :self.K, :self.V]
        return o[..., :self.V], final_state


def _grouped(q, k, v):
    """Grouped value heads (HV = G * H; value head hv reads query/key head hv // G, as in FLA's kernels): q and k are
    repeated to HV heads, and autograd's backward of the repeat sums dq and dk over each group.  The kernels then see
    equal head counts; the price is G copies of q and k."""
    G = v.shape[2] // q.shape[2]
    return (q, k) if G == 1 else (q.repeat_interleave(G, 2), k.repeat_interleave(G, 2))


@torch.compiler.disable
def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              allow_neg_eigval=False, safe_gate=False, lower_bound=None, disable_recompute=False,
              return_intermediate_states=False, state_v_first=False, cu_seqlens=None, cu_seqlens_cpu=None,
              cp_context=None, use_graph=False, max_num_seqs=None, **kwargs):
    """KDA (per-channel gated delta rule).  q,k [B,T,H,128] BF16, v [B,T,H,128], g [B,T,H,128] per-step
    natural-log decay (or, with ``use_gate_in_kernel``, the raw gate input together with ``A_log`` [H] and the optional
    ``dt_bias`` [H*128] keyword arguments), beta [B,T,H].  Returns (o, final_state)."""
    _common_checks(q, k, v, initial_state)
    if allow_neg_eigval and not use_beta_sigmoid_in_kernel:
        raise ValueError("`allow_neg_eigval=True` requires `use_beta_sigmoid_in_kernel=True`.")
    A_log, dt_bias = kwargs.get("A_log"), kwargs.get("dt_bias")
    if use_gate_in_kernel:
        if A_log is None:
            raise ValueError("A_log must be provided when use_gate_in_kernel=True.")
        if lower_bound is not None:
            raise ValueError("rewy_b200 chunk_kda: the lower_bound gate law belongs to safe_gate, which is not supported")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    nw = _Narrow(q, v)
    if nw.needed:
        if use_gate_in_kernel:
            raise ValueError("rewy_b200 chunk_kda: the fused gate needs K = 128 (dt_bias is laid out per channel)")
        q, k, g, v, initial_state = nw.key(q), nw.key(k), nw.key(g), nw.value(v), nw.state(initial_state, state_v_first)
    q, k = _grouped(q, k, v)
    rg = _Ragged(q.shape[1], q.device, cu_seqlens, cu_seqlens_cpu)
    if rg.needed:
        # a raw gate input goes through -exp(A_log) softplus(g + dt_bias): a very negative value gives decay 0
        q, k, v, beta, g = rg.pad(q), rg.pad(k), rg.pad(v), rg.pad(beta), rg.pad(g, -1e4 if use_gate_in_kernel else 0.0)
        cu_seqlens = rg.cu
    o, final_state = ChunkKDAFunction.apply(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state,
                                            use_qk_l2norm_in_kernel, use_gate_in_kernel, use_beta_sigmoid_in_kernel,
                                            allow_neg_eigval, disable_recompute, state_v_first, _packed(cu_seqlens, q))
    return nw.cut(rg.cut(o), final_state, state_v_first)


@torch.compiler.disable
def chunk_gdn2(q, k, v, g, b, w, scale=None, initial_state=None, output_final_state=False,
               use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None,
               safe_gate=False, lower_bound=None, disable_recompute=False, return_intermediate_states=False,
               state_v_first=False, cp_context=None, **kwargs):
    """GDN2 (vector erase gate b [B,T,H,128], vector write gate w [B,T,H,128]).  Returns (o, final_state)."""
    _common_checks(q, k, v, initial_state)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    nw = _Narrow(q, v)
    if nw.needed:
        q, k, g, b = nw.key(q), nw.key(k), nw.key(g), nw.key(b)
        v, w, initial_state = nw.value(v), nw.value(w), nw.state(initial_state, state_v_first)
    q, k = _grouped(q, k, v)
    rg = _Ragged(q.shape[1], q.device, cu_seqlens, cu_seqlens_cpu)
    if rg.needed:
        q, k, v, g, b, w = (rg.pad(x) for x in (q, k, v, g, b, w))
        cu_seqlens = rg.cu
    o, final_state = ChunkGDN2Function.apply(q, k, v, g, b, w, scale, initial_state, output_final_state,
                                             use_qk_l2norm_in_kernel, disable_recompute, state_v_first,
                                             _packed(cu_seqlens, q))
    return nw.cut(rg.cut(o), final_state, state_v_first)


@torch.compiler.disable
def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, use_beta_sigmoid_in_kernel=False, allow_neg_eigval=False,
                           state_v_first=False, cu_seqlens=None, cu_seqlens_cpu=None, chunk_indices=None,
                           cp_context=None, **kwargs):
    """Gated DeltaNet (scalar per-head gate g [B,T,H]).  Returns (o, final_state)."""
    _common_checks(q, k, v, initial_state)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    nw = _Narrow(q, v)
    if nw.needed:
        q, k, v, initial_state = nw.key(q), nw.key(k), nw.value(v), nw.state(initial_state, state_v_first)
    q, k = _grouped(q, k, v)
    rg = _Ragged(q.shape[1], q.device, cu_seqlens, cu_seqlens_cpu)
    if rg.needed:
        q, k, v, g, beta = (rg.pad(x) for x in (q, k, v, g, beta))
        cu_seqlens = rg.cu
    o, final_state = ChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state,
                                                       use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel,
                                                       allow_neg_eigval, state_v_first, _packed(cu_seqlens, q))
    return nw.cut(rg.cut(o), final_state, state_v_first)


@torch.compiler.disable
def chunk_delta_rule(q, k, v, beta, scale=None, initial_state=None, output_final_state=False,
                     use_qk_l2norm_in_kernel=False, cu_seqlens=None, cu_seqlens_cpu=None, **kwargs):
    """DeltaNet (ungated delta rule).  Returns (o, final_state)."""
    _common_checks(q, k, v, initial_state)
    if scale is None:
        scale = k.shape[-1] ** -0.5
    nw = _Narrow(q, v)
    if nw.needed:
        q, k, v, initial_state = nw.key(q), nw.key(k), nw.value(v), nw.state(initial_state)
    q, k = _grouped(q, k, v)
    rg = _Ragged(q.shape[1], q.device, cu_seqlens, cu_seqlens_cpu)
    if rg.needed:
        q, k, v, beta = (rg.pad(x) for x in (q, k, v, beta))
        cu_seqlens = rg.cu
    o, final_state = ChunkDeltaRuleFunction.apply(q, k, v, beta, scale, initial_state, output_final_state,
                                                  use_qk_l2norm_in_kernel, _packed(cu_seqlens, q))
    return nw.cut(rg.cut(o), final_state)
