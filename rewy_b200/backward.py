"""Whole-family backward functions with the reference's names, arguments and return order.

They stand where the reference's ``kda_backward``, ``gdn2_backward``, ``gdn_backward`` and
``delta_backward`` stand (src/fast_delta_rule/backends/backward.py:63-137), i.e. they are what the
autograd backwards call as ``chunk_kda_bwd`` / ``chunk_gdn2_bwd`` / ``chunk_gated_delta_rule_bwd`` /
``chunk_delta_rule_bwd`` (src/fast_delta_rule/_compat/kda.py:169-201, gdn2.py:145-171, gdn.py:240-260,
delta.py:125-138).  All arithmetic happens in librewy_b200.so; this module only checks the envelope,
allocates outputs and workspace with torch and marshals raw pointers.

The call into the library is a torch custom operator, ``torch.ops.rewy_b200.family_bwd`` (registered with
``torch.library`` for CUDA tensors, with a shape-only fake implementation): the four functions below are
thin bindings of it, so the backward is a single opaque node for ``torch.compile`` / export, and the C ABI
stays the only thing underneath.
"""
from typing import Optional

import torch
from torch import Tensor

from . import _capi
from .runtime import record

_FAMILY_FN = {_capi.KDA: "rewy_kda_bwd", _capi.GDN2: "rewy_gdn2_bwd", _capi.GDN: "rewy_gdn_bwd",
              _capi.DELTA: "rewy_delta_bwd"}
_NONE = None


def _empty(dev):
    return torch.empty(0, device=dev)


@torch.library.custom_op("rewy_b200::family_bwd", mutates_args=("workspace",), device_types="cuda")
def _family_bwd(family: int, policy: int, out_f32: bool, intra_passes: int, state_v_first: bool, scale: float,
                q: Tensor, k: Tensor, v: Tensor, d_o: Tensor, Akk: Tensor, workspace: Tensor,
                g: Optional[Tensor], beta: Optional[Tensor], b_gate: Optional[Tensor], w_gate: Optional[Tensor],
                Aqk: Optional[Tensor], h0: Optional[Tensor], dht: Optional[Tensor], w: Optional[Tensor],
                qg: Optional[Tensor], kg: Optional[Tensor], v_new: Optional[Tensor], h: Optional[Tensor],
                cu_seqlens: Optional[Tensor]) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """(dq, dk, dv, dg, dbeta, db_gate, dw_gate, dh0); outputs a family does not have are empty tensors.
    Tensors must be contiguous, on one CUDA device, in the dtypes of RewyBwdArgs."""
    lib = _capi.load()
    B, T, H, _ = k.shape
    dev = q.device
    odt = torch.float32 if out_f32 else torch.bfloat16
    shape = (B, T, H, 128)
    vector_gates = family == _capi.GDN2
    out = dict(
        dq=torch.empty(shape, dtype=odt, device=dev), dk=torch.empty(shape, dtype=odt, device=dev),
        dv=torch.empty(shape, dtype=torch.bfloat16, device=dev),
        dg=torch.empty_like(g) if g is not None else None,
        dbeta=torch.empty((B, T, H), dtype=torch.float32, device=dev) if not vector_gates else None,
        db_gate=torch.empty(shape, dtype=odt, device=dev) if vector_gates else None,
        dw_gate=torch.empty(shape, dtype=odt, device=dev) if vector_gates else None,
        dh0=torch.empty_like(h0) if h0 is not None else None,   # [B,H,128,128], or [sequences,H,128,128] when packed
    )
    a = _capi.BwdArgs()
    a.family, a.policy, a.B, a.T, a.H = family, policy, B, T, H
    a.out_dtype = _capi.OUT_F32 if out_f32 else _capi.OUT_BF16
    a.intra_passes = intra_passes
    a.state_v_first = int(state_v_first)
    a.scale = scale
    if cu_seqlens is not None:   # int32, on the device, [sequences + 1]
        a.cu_seqlens, a.num_seqs = _capi.ptr(cu_seqlens), cu_seqlens.numel() - 1
    for name, t in dict(q=q, k=k, v=v, d_o=d_o, Akk=Akk, g=g, beta=beta, b_gate=b_gate, w_gate=w_gate, Aqk=Aqk, h0=h0,
                        dht=dht, w=w, qg=qg, kg=kg, v_new=v_new, h=h).items():
        setattr(a, name, _capi.ptr(t))
    for name, t in out.items():
        setattr(a, name, _capi.ptr(t))
    a.workspace = _capi.ptr(workspace)
    a.workspace_bytes = workspace.numel() * workspace.element_size()
    fn = getattr(lib, _FAMILY_FN[family])
    with torch.cuda.device(dev):
        # Inputs, outputs and workspace are allocated on (or already in use by) the current stream, the same
        # stream the launches go to, so the caching allocator's stream-ordered reuse keeps them valid.
        _capi.check(fn(a, _capi.current_stream(dev)), fn.__name__)
    return tuple(out[n] if out[n] is not None else _empty(dev)
                 for n in ("dq", "dk", "dv", "dg", "dbeta", "db_gate", "dw_gate", "dh0"))


@_family_bwd.register_fake
def _family_bwd_fake(family, policy, out_f32, intra_passes, state_v_first, scale, q, k, v, d_o, Akk, workspace, g, beta, b_gate, w_gate,
                     Aqk, h0, dht, w, qg, kg, v_new, h, cu_seqlens):
    B, T, H, _ = k.shape
    odt = torch.float32 if out_f32 else torch.bfloat16
    big = lambda dt: q.new_empty((B, T, H, 128), dtype=dt)
    none = lambda: q.new_empty(0, dtype=torch.float32)   # a fresh tensor each time: outputs must not alias each other
    vec = family == _capi.GDN2
    return (big(odt), big(odt), big(torch.bfloat16), torch.empty_like(g) if g is not None else none(),
            q.new_empty((B, T, H), dtype=torch.float32) if not vec else none(), big(odt) if vec else none(),
            big(odt) if vec else none(), torch.empty_like(h0) if h0 is not None else none())


def _unsupported(name, value, allowed=(None, False)):
    if value not in allowed:
        raise RuntimeError(f"rewy_b200 backward: argument {name}={value!r} is outside the supported envelope")


def _check_common(q, k, v, do, chunk_size, cu_seqlens, cp_context, state_v_first, use_gate_in_kernel):
    if not q.is_cuda:
        raise RuntimeError("rewy_b200 backward needs CUDA tensors (there is no CPU fallback)")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise RuntimeError("rewy_b200 backward: q, k, v must be BF16")
    B, T, H, K = k.shape
    if q.shape != k.shape or v.shape != (B, T, H, 128) or K != 128:
        raise RuntimeError("rewy_b200 backward: needs q.shape == k.shape, equal heads and K = V = 128")
    if T < 64 or T % 64:
        raise RuntimeError("rewy_b200 backward: sequence length must be a positive multiple of 64")
    if chunk_size != 64:
        raise RuntimeError("rewy_b200 backward: chunk_size must be 64")
    if cu_seqlens is not None and B != 1:
        raise RuntimeError("rewy_b200 backward: packed sequences (cu_seqlens) need a batch of 1")
    _unsupported("cp_context", cp_context, (None,))
    _unsupported("use_gate_in_kernel", use_gate_in_kernel)   # the gate activation is a wrapper stage (elementwise.py)
    if do.shape != v.shape:
        raise RuntimeError("rewy_b200 backward: do must have the shape of v")
    return B, T, H


def _cu(cu_seqlens, device):
    """cu_seqlens as the library takes them: int32, contiguous, on the device.  Lengths must be multiples of 64; the
    operators check that on the host at forward time, the scan kernels again on the device."""
    if cu_seqlens is None:
        return None
    return cu_seqlens.to(device=device, dtype=torch.int32).contiguous()


def _c(t, dtype=None):
    if t is None:
        return None
    if dtype is not None and t.dtype != dtype:
        t = t.to(dtype)
    return t.contiguous()


def _run(family, policy, B, T, H, scale, tensors, out_dtype, intra_passes, workspace, want_dg, want_dbeta, vector_gates,
         check_status=False, state_v_first=False):
    """tensors: dict name -> tensor or None for every input pointer of RewyBwdArgs."""
    lib = _capi.load()
    dev = tensors["q"].device
    if out_dtype not in (None, torch.float32, torch.bfloat16):
        raise RuntimeError("rewy_b200 backward: out_dtype must be torch.float32 or torch.bfloat16")
    out_f32 = out_dtype in (None, torch.float32)
    need = _capi.workspace_bytes(family, policy, B, T, H)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    elif workspace.numel() * workspace.element_size() < need or workspace.device != dev:
        raise RuntimeError(f"rewy_b200 backward: workspace must hold {need} bytes on {dev}")
    t = tensors
    r = torch.ops.rewy_b200.family_bwd(
        family, policy, out_f32, int(intra_passes or 0), bool(state_v_first), float(scale), t["q"], t["k"], t["v"], t["d_o"], t["Akk"],
        workspace, t["g"], t["beta"], t["b_gate"], t["w_gate"], t["Aqk"], t["h0"], t["dht"], t["w"], t["qg"], t["kg"],
        t["v_new"], t["h"], t.get("cu_seqlens"))
    names = ("dq", "dk", "dv", "dg", "dbeta", "db_gate", "dw_gate", "dh0")
    out = {n: (x if x.numel() else None) for n, x in zip(names, r)}
    if check_status:  # synchronises: reads the device status word at the start of the workspace
        with torch.cuda.device(dev):
            _capi.check(lib.rewy_device_status(_capi.ptr(workspace), _capi.current_stream(dev)), "device status")
            out["wide_chunks"] = int(lib.rewy_wide_chunk_count(_capi.ptr(workspace), _capi.current_stream(dev)))
    return out


def kda_backward(q, k, v, beta, Aqk, Akk, scale, initial_state, do, dht, g=None, g_org=None, state_v_first=False,
                 cu_seqlens=None, chunk_indices=None, chunk_size=64, safe_gate=False, lower_bound=None,
                 use_gate_in_kernel=False, A_log=None, dt_bias=None, disable_recompute=False, cp_context=None,
                 w=None, u=None, qg=None, kg=None, v_new=None, h=None, use_graph=False, chunk_offsets=None,
                 *, out_dtype=None, intra_passes=None, workspace=None, check_status=False):
    """KDA backward.  Returns (dq, dk, dv, db, dg, dh0, dA, dbias) like FLA's ``chunk_kda_bwd``;
    ``g`` is the chunk-local cumulative gate in log2 units that the forward saved."""
    B, T, H = _check_common(q, k, v, do, chunk_size, cu_seqlens, cp_context, state_v_first, use_gate_in_kernel)
    _unsupported("safe_gate", safe_gate)
    _unsupported("use_graph", use_graph)
    if g is None:
        raise RuntimeError("rewy_b200 kda backward: g (cumulative gate) is required")
    saved = bool(disable_recompute)
    tensors = dict(
        q=_c(q), k=_c(k), v=_c(v), g=_c(g, torch.float32), beta=_c(beta, torch.float32), b_gate=None, w_gate=None,
        Aqk=_c(Aqk, torch.bfloat16), Akk=_c(Akk, torch.bfloat16), h0=_c(initial_state, torch.float32),
        d_o=_c(do, torch.bfloat16), dht=_c(dht, torch.float32),
        w=_c(w, torch.bfloat16) if saved else None, qg=_c(qg, torch.bfloat16) if saved else None,
        kg=_c(kg, torch.bfloat16) if saved else None, v_new=_c(v_new, torch.bfloat16) if saved else None,
        h=_c(h, torch.bfloat16) if saved else None, cu_seqlens=_cu(cu_seqlens, q.device))
    out = _run(_capi.KDA, _capi.SAVED if saved else _capi.RECOMPUTE, B, T, H, scale, tensors, out_dtype,
               intra_passes, workspace, True, True, False, check_status, state_v_first)
    record("kda", "optimized_backward")
    return out["dq"], out["dk"], out["dv"], out["dbeta"], out["dg"], out["dh0"], None, None


def gdn2_backward(q, k, v, b, w_gate, Aqk, Akk, scale, initial_state, do, dht, g=None, g_org=None, cu_seqlens=None,
                  chunk_indices=None, chunk_size=64, safe_gate=False, lower_bound=None, use_gate_in_kernel=False,
                  A_log=None, dt_bias=None, state_v_first=False, w_wy=None, u_wy=None, qg=None, kg=None, v_new=None,
                  h=None, disable_recompute=False, cp_context=None,
                  *, out_dtype=None, intra_passes=None, workspace=None, check_status=False):
    """GDN2 backward.  Returns (dq, dk, dv, db, dw, dg, dh0, dA_log, ddt_bias) like ``chunk_gdn2_bwd``."""
    B, T, H = _check_common(q, k, v, do, chunk_size, cu_seqlens, cp_context, state_v_first, use_gate_in_kernel)
    _unsupported("safe_gate", safe_gate)
    if g is None:
        raise RuntimeError("rewy_b200 gdn2 backward: g (cumulative gate) is required")
    saved = bool(disable_recompute)
    tensors = dict(
        q=_c(q), k=_c(k), v=_c(v), g=_c(g, torch.float32), beta=None, b_gate=_c(b, torch.bfloat16),
        w_gate=_c(w_gate, torch.bfloat16), Aqk=_c(Aqk, torch.bfloat16), Akk=_c(Akk, torch.bfloat16),
        h0=_c(initial_state, torch.float32), d_o=_c(do, torch.bfloat16), dht=_c(dht, torch.float32),
        w=_c(w_wy, torch.bfloat16) if saved else None, qg=_c(qg, torch.bfloat16) if saved else None,
        kg=_c(kg, torch.bfloat16) if saved else None, v_new=_c(v_new, torch.bfloat16) if saved else None,
        h=_c(h, torch.bfloat16) if saved else None, cu_seqlens=_cu(cu_seqlens, q.device))
    out = _run(_capi.GDN2, _capi.SAVED if saved else _capi.RECOMPUTE, B, T, H, scale, tensors, out_dtype,
               intra_passes, workspace, True, False, True, check_status, state_v_first)
    record("gdn2", "optimized_backward")
    return out["dq"], out["dk"], out["dv"], out["db_gate"], out["dw_gate"], out["dg"], out["dh0"], None, None


def gdn_backward(q, k, v, g, beta, A, scale, initial_state, do, dht, cu_seqlens=None, cp_context=None,
                 chunk_indices=None, state_v_first=False, use_gate_in_kernel=False, g_input=None, A_log=None,
                 dt_bias=None, chunk_size=64, *, out_dtype=None, intra_passes=None, workspace=None, check_status=False):
    """Gated DeltaNet backward.  Returns (dq, dk, dv, db, dg, dh0, dA_log, ddt_bias) — ``db`` before ``dg``
    as at src/fast_delta_rule/backends/backward.py:130."""
    B, T, H = _check_common(q, k, v, do, chunk_size, cu_seqlens, cp_context, state_v_first, use_gate_in_kernel)
    tensors = dict(
        q=_c(q), k=_c(k), v=_c(v), g=_c(g, torch.float32), beta=_c(beta, torch.float32), b_gate=None, w_gate=None,
        Aqk=None, Akk=_c(A, torch.bfloat16), h0=_c(initial_state, torch.float32), d_o=_c(do, torch.bfloat16),
        dht=_c(dht, torch.float32), w=None, qg=None, kg=None, v_new=None, h=None, cu_seqlens=_cu(cu_seqlens, q.device))
    out = _run(_capi.GDN, _capi.RECOMPUTE, B, T, H, scale, tensors, out_dtype, intra_passes, workspace,
               True, True, False, check_status, state_v_first)
    record("gdn", "optimized_backward")
    return out["dq"], out["dk"], out["dv"], out["dbeta"], out["dg"], out["dh0"], None, None


def delta_backward(q, k, v, beta, A, scale, initial_state, do, dht, cu_seqlens=None, chunk_indices=None,
                   chunk_size=64, *, out_dtype=None, intra_passes=None, workspace=None, check_status=False):
    """DeltaNet backward.  Returns (dq, dk, dv, db, dh0) like ``chunk_delta_rule_bwd``."""
    B, T, H = _check_common(q, k, v, do, chunk_size, cu_seqlens, None, False, False)
    tensors = dict(
        q=_c(q), k=_c(k), v=_c(v), g=None, beta=_c(beta, torch.float32), b_gate=None, w_gate=None,
        Aqk=None, Akk=_c(A, torch.bfloat16), h0=_c(initial_state, torch.float32), d_o=_c(do, torch.bfloat16),
        dht=_c(dht, torch.float32), w=None, qg=None, kg=None, v_new=None, h=None, cu_seqlens=_cu(cu_seqlens, q.device))
    out = _run(_capi.DELTA, _capi.RECOMPUTE, B, T, H, scale, tensors, out_dtype, intra_passes, workspace,
               False, True, False, check_status)
    record("delta", "optimized_backward")
    return out["dq"], out["dk"], out["dv"], out["dbeta"], out["dh0"]
