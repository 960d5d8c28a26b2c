"""The chunk stage for hosts that cannot allocate device memory (rewy_stage_chunk_adjoint_static).

Some users of the C ABI run entirely out of a device arena they reserved at start-up (a plain C or C++ training
loop, or a job whose memory plan forbids allocations once it is running); they cannot hand the chunk stage the
small control block it normally receives in RewyStageBuffers.ctrl.  The static variant keeps that block inside the
library.  This test drives it through the C ABI twice in a row - the second time on inputs whose wide-gate chunk
leaves entries in the shared block that the next call must not trip over - and checks every output against the
regular entry point.  It lives in a file that sorts last so that a run stopping at the first failure has already
exercised everything else.
"""
import pytest
import torch

from gpu_util import base_args, call_stage, forward_saved, nrmse, oracle_backward, stage_buffers
from rewy_b200 import _capi
from rewy_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(entry, xs, saved, dh, dR, dR_lo, with_ctrl):
    a, keep = base_args("kda", xs, saved, _capi.OUT_F32, 0)
    B, T, H, _ = xs["k"].shape
    nan = lambda shape, dt: torch.full(shape, float("nan"), dtype=dt, device=DEV)
    out = dict(dq=nan((B, T, H, 128), torch.float32), dk=nan((B, T, H, 128), torch.float32),
               dv=nan((B, T, H, 128), torch.bfloat16), dg=nan((B, T, H, 128), torch.float32),
               dbeta=nan((B, T, H), torch.float32))
    for n, t in out.items():
        setattr(a, n, _capi.ptr(t))
    bufs = dict(v_new=saved["v_new"], h=saved["h"], dh=dh, dR=dR, dR_lo=dR_lo)
    ctrl = None
    if with_ctrl:
        ctrl = torch.zeros(2 + B * H * (T // 64), dtype=torch.int32, device=DEV)
        bufs["ctrl"] = ctrl
    call_stage(entry, a, stage_buffers(**bufs), DEV)
    if ctrl is not None:
        assert ctrl[0].item() == 0
    return out


def _case(seed, widen):
    xs = make_inputs("kda", 1, 192, 2, seed=seed, device=DEV, gate_scale=0.1)
    if widen:
        xs["g"][:, 64:128, 0, :32] *= 30   # one chunk takes the pairwise path: the control block's list is used
    saved = forward_saved("kda", xs)
    ref = oracle_backward("kda", xs, saved)
    dh = ref["dh"].to(torch.bfloat16).to(DEV)
    hi = ref["dR"].to(torch.bfloat16)
    lo = (ref["dR"] - hi.double()).to(torch.bfloat16)
    return xs, saved, dh, hi.to(DEV).contiguous(), lo.to(DEV).contiguous()


def _oracle_errors(ref, out):
    return dict(dq=nrmse(ref["dq"], out["dq"]), dk=nrmse(ref["dk"], out["dk"]), dv=nrmse(ref["dv"].to(torch.bfloat16), out["dv"]),
                dg=nrmse(ref["dg"], out["dg"]), dbeta=nrmse(ref["dbeta"], out["dbeta"]))


def test_static_control_block_matches_regular_entry_point_twice_in_a_row():
    lib = _capi.load()
    stream = _capi.current_stream(torch.device(DEV))
    for seed, widen in ((31, True), (32, False)):       # two calls in a row share the library's block
        xs, saved, dh, dR, dR_lo = _case(seed, widen)
        ref = oracle_backward("kda", xs, saved)
        want = _run("rewy_stage_chunk_adjoint", xs, saved, dh, dR, dR_lo, with_ctrl=True)
        got = _run("rewy_stage_chunk_adjoint_static", xs, saved, dh, dR, dR_lo, with_ctrl=False)
        with torch.cuda.device(DEV):
            assert lib.rewy_static_device_status(stream) == 0, lib.rewy_last_error()
        for n in want:
            assert torch.isfinite(got[n].float()).all(), n
            # same kernels on the same inputs
            assert nrmse(want[n], got[n]) <= 1e-5, (seed, n, nrmse(want[n], got[n]))
        # and against the FP64 oracle itself (the case with a chunk on the pairwise path included)
        errs = _oracle_errors(ref, got)
        bad = {n: e for n, e in errs.items() if not e <= 2e-3}
        assert not bad, (seed, bad)


def test_static_entry_point_allocates_no_device_memory():
    """What the entry point exists for: between the moment its arguments are ready and the moment its results are,
    the amount of free device memory does not move (no cudaMalloc / cudaFree by the library, no allocator behind it).
    The first call on the device (which resolves the address of the built-in block) is made beforehand."""
    lib = _capi.load()
    xs, saved, dh, dR, dR_lo = _case(33, False)
    _run("rewy_stage_chunk_adjoint_static", xs, saved, dh, dR, dR_lo, with_ctrl=False)      # first call: set-up
    a, keep = base_args("kda", xs, saved, _capi.OUT_F32, 0)
    B, T, H, _ = xs["k"].shape
    out = dict(dq=torch.empty(B, T, H, 128, device=DEV), dk=torch.empty(B, T, H, 128, device=DEV),
               dv=torch.empty(B, T, H, 128, dtype=torch.bfloat16, device=DEV), dg=torch.empty(B, T, H, 128, device=DEV),
               dbeta=torch.empty(B, T, H, device=DEV))
    for n, t in out.items():
        setattr(a, n, _capi.ptr(t))
    s = stage_buffers(v_new=saved["v_new"], h=saved["h"], dh=dh, dR=dR, dR_lo=dR_lo)
    stream = _capi.current_stream(torch.device(DEV))
    torch.cuda.synchronize()
    with torch.cuda.device(DEV):
        free_before, _ = torch.cuda.mem_get_info()
        for _ in range(3):
            assert lib.rewy_stage_chunk_adjoint_static(a, s, stream) == 0, lib.rewy_last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert lib.rewy_static_device_status(stream) == 0
    assert free_after == free_before, (free_before, free_after)
    assert torch.isfinite(out["dq"]).all()


def test_static_variant_rejects_problems_beyond_its_block():
    lib = _capi.load()
    a = _capi.BwdArgs()
    a.family, a.B, a.T, a.H = _capi.KDA, 64, 8192, 32      # 262144 chunks > 65536
    s = _capi.StageBuffers()
    assert lib.rewy_stage_chunk_adjoint_static(a, s, None) == 2
    assert b"at most 65536 chunks" in lib.rewy_last_error()
