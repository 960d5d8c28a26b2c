"""Helpers shared by the GPU parity tests: run the product forward, call single stages through the
C ABI and compare with the FP64 oracle."""
import torch

from rewy_b200 import _capi
from rewy_b200.forward import chunk_forward
from rewy_b200.synthetic import make_inputs, operator_inputs


def nrmse(ref, got):
    ref = ref.detach().double().cpu()
    got = got.detach().double().cpu()
    return ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()


def forward_saved(op, xs):
    """Product forward on the device of xs; returns its dict of saved tensors."""
    kw = dict(q=xs["q"], k=xs["k"], v=xs["v"], initial_state=xs.get("initial_state"))
    if op != "delta":
        kw["g"] = xs["g"]
    if op == "gdn2":
        kw["b"], kw["w"] = xs["b"], xs["w"]
    else:
        kw["beta"] = xs["beta"]
    return chunk_forward(op, check_status=True, **kw)


def base_args(op, xs, saved, out_dtype=_capi.OUT_F32, intra_passes=0):
    """BwdArgs with the boundary inputs filled in; returns (args, keepalive list)."""
    B, T, H, _ = xs["k"].shape
    a = _capi.BwdArgs()
    a.family, a.policy, a.B, a.T, a.H = _capi.FAMILY_ID[op], _capi.SAVED, B, T, H
    a.out_dtype, a.intra_passes, a.scale = out_dtype, intra_passes, 128 ** -0.5
    keep = []

    def put(name, t, dtype=None):
        if t is None:
            return
        if dtype is not None:
            t = t.to(dtype)
        t = t.contiguous()
        keep.append(t)
        setattr(a, name, _capi.ptr(t))

    put("q", xs["q"]); put("k", xs["k"]); put("v", xs["v"])
    if op != "delta":
        put("g", saved["g_cumsum"], torch.float32)
    if op == "gdn2":
        put("b_gate", xs["b"]); put("w_gate", xs["w"])
    else:
        put("beta", xs["beta"], torch.float32)
    put("Akk", saved["Akk"]); put("d_o", xs["do"])
    put("h0", xs.get("initial_state")); put("dht", xs.get("dht"))
    return a, keep


def stage_buffers(**tensors):
    s = _capi.StageBuffers()
    for n, t in tensors.items():
        setattr(s, n, _capi.ptr(t))
    return s


def call_stage(name, a, s, device):
    lib = _capi.load()
    fn = getattr(lib, name)
    with torch.cuda.device(device):
        _capi.check(fn(a, s, _capi.current_stream(device)), name)
    torch.cuda.synchronize(device)


def oracle_backward(op, xs, saved, policy_saved=True):
    """FP64 closed-form backward from the (BF16) saved tensors, on CPU."""
    from oracle import chunk_backward
    cpu = lambda t: None if t is None else t.detach().cpu()
    ins = {n: cpu(x) for n, x in operator_inputs(op, xs).items()}
    sv = {n: cpu(x) for n, x in saved.items()}
    return chunk_backward(op, ins, sv, cpu(xs["do"]), cpu(xs.get("dht")))
