"""Element-wise stages of the autograd wrappers, bound to the CUDA library.

These are what the reference's autograd functions run around the core operator
(src/fast_delta_rule/_compat/kda.py:56-63 and :202-210: FLA ``l2norm_fwd`` / ``l2norm_bwd``,
``fused_beta_sigmoid`` / ``fused_beta_sigmoid_bwd``; ``kda_gate_chunk_cumsum`` / ``kda_gate_bwd`` inside
``chunk_kda_fwd`` / ``chunk_kda_bwd`` when ``use_gate_in_kernel`` is set).  One CUDA pass each; there is no
CPU or PyTorch fallback: non-CUDA tensors raise.
"""
import torch

from . import _capi


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("rewy_b200 element-wise stages need CUDA tensors (there is no CPU fallback)")


def _stream(t):
    return _capi.current_stream(t.device)


def _as_input(x):
    """BF16 and FP32 are read directly; anything else is converted to FP32 first."""
    if x.dtype not in (torch.bfloat16, torch.float32):
        x = x.float()
    return x.contiguous(), int(x.dtype == torch.float32)


def l2norm_fwd(x, eps=1e-6):
    """x BF16 [..., 128] -> (y BF16, rstd FP32 [...])."""
    _need_cuda(x)
    if x.dtype != torch.bfloat16 or x.shape[-1] != 128:
        raise RuntimeError("rewy_b200 l2norm: expects BF16 rows of 128 values")
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().rewy_l2norm_fwd(_capi.ptr(x), _capi.ptr(y), _capi.ptr(rstd), x.numel() // 128, eps,
                                                 _stream(x)), "rewy_l2norm_fwd")
    return y, rstd


def l2norm_bwd(y, rstd, dy):
    """Gradient of the normalisation, written in BF16 (the cast to the input dtype is part of the pass)."""
    _need_cuda(y, rstd, dy)
    if dy.dtype not in (torch.bfloat16, torch.float32):
        dy = dy.float()
    y, dy, rstd = y.contiguous(), dy.contiguous(), rstd.contiguous()
    dx = torch.empty_like(y)
    with torch.cuda.device(y.device):
        _capi.check(_capi.load().rewy_l2norm_bwd(_capi.ptr(y), _capi.ptr(rstd), _capi.ptr(dy),
                                                 int(dy.dtype == torch.float32), _capi.ptr(dx), y.numel() // 128,
                                                 _stream(y)), "rewy_l2norm_bwd")
    return dx


def beta_sigmoid_fwd(x, scale=1.0):
    """scale * sigmoid(x) in the dtype of x (BF16 logits give a BF16 beta, like the reference's fused sigmoid)."""
    _need_cuda(x)
    xin, is_f32 = _as_input(x)
    y16 = torch.empty_like(xin) if not is_f32 else None
    y32 = torch.empty(xin.shape, dtype=torch.float32, device=x.device) if is_f32 else None
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().rewy_beta_sigmoid_fwd(_capi.ptr(xin), is_f32, _capi.ptr(y32), _capi.ptr(y16), xin.numel(),
                                                       float(scale), _stream(x)), "rewy_beta_sigmoid_fwd")
    return y32 if is_f32 else y16


def beta_sigmoid_bwd(x, dy, scale=1.0):
    """dx (FP32) for y = scale * sigmoid(x); dy FP32."""
    _need_cuda(x, dy)
    xin, is_f32 = _as_input(x)
    dy = dy.float().contiguous()
    dx = torch.empty(xin.shape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().rewy_beta_sigmoid_bwd(_capi.ptr(xin), is_f32, _capi.ptr(dy), _capi.ptr(dx), xin.numel(),
                                                       float(scale), _stream(x)), "rewy_beta_sigmoid_bwd")
    return dx


def gate_cumsum_fwd(g, A_log=None, dt_bias=None):
    """g [B,T,H,128] (BF16 or FP32).  Returns the chunk-local cumulative gate in log2 units (FP32).  With ``A_log`` the KDA
    gate activation -exp(A_log[h]) * softplus(g + dt_bias[h*128+k]) is applied first (``dt_bias`` optional)."""
    _need_cuda(g, A_log, dt_bias)
    B, T, H, K = g.shape
    if K != 128 or T % 64:
        raise RuntimeError("rewy_b200 gate cumsum: expects [B,T,H,128] with T a multiple of 64")
    gin, is_f32 = _as_input(g)
    out = torch.empty(gin.shape, dtype=torch.float32, device=g.device)
    a = None if A_log is None else A_log.float().contiguous().view(-1)
    bias = None if dt_bias is None else dt_bias.float().contiguous().view(-1)
    if a is not None and a.numel() != H or bias is not None and bias.numel() != H * 128:
        raise RuntimeError("rewy_b200 gate cumsum: A_log must hold H values and dt_bias H*128")
    if a is None and bias is not None:
        raise RuntimeError("rewy_b200 gate cumsum: dt_bias needs A_log")
    with torch.cuda.device(g.device):
        _capi.check(_capi.load().rewy_gate_cumsum_fwd(_capi.ptr(gin), is_f32, _capi.ptr(a), _capi.ptr(bias), _capi.ptr(out),
                                                      None, B, T, H, _stream(g)), "rewy_gate_cumsum_fwd")
    return out


def gate_act_bwd(g_raw, A_log, dt_bias, dg):
    """Backward of the KDA gate activation.  dg: FP32 gradient of the activated per-step gate.
    Returns (dg_raw FP32 [B,T,H,128], dA_log FP32 [H], ddt_bias FP32 [H*128] or None)."""
    _need_cuda(g_raw, A_log, dt_bias, dg)
    B, T, H, K = g_raw.shape
    gin, is_f32 = _as_input(g_raw)
    dg = dg.float().contiguous()
    a = A_log.float().contiguous().view(-1)
    bias = None if dt_bias is None else dt_bias.float().contiguous().view(-1)
    nt = T // 64
    dx = torch.empty(gin.shape, dtype=torch.float32, device=g_raw.device)
    dA_part = torch.empty(B * nt, H, dtype=torch.float32, device=g_raw.device)
    db_part = torch.empty(B * nt, H * 128, dtype=torch.float32, device=g_raw.device)
    with torch.cuda.device(g_raw.device):
        _capi.check(_capi.load().rewy_gate_act_bwd(_capi.ptr(gin), is_f32, _capi.ptr(a), _capi.ptr(bias), _capi.ptr(dg),
                                                   _capi.ptr(dx), _capi.ptr(dA_part), _capi.ptr(db_part), B, T, H,
                                                   _stream(g_raw)), "rewy_gate_act_bwd")
    # the per-(batch, chunk) partial sums are added up in a fixed order (deterministic), as FLA's kda_gate_bwd does
    return dx, dA_part.sum(0), (db_part.sum(0) if dt_bias is not None else None)
