"""Self-test of the tcgen05/TMA plumbing against plain matrix products (GPU)."""
import ctypes

import pytest
import torch

from rewy_b200 import _capi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tf32(x):
    u = x.contiguous().view(torch.int32)
    return ((u + 0x1000) & ~0x1FFF).view(torch.float32)


def test_tensor_core_operand_forms():
    g = torch.Generator(device=DEV); g.manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=g, device=DEV)
    A, B = rn(128, 128).bfloat16(), rn(64, 128).bfloat16()
    Akk, dR = rn(64, 64).bfloat16(), rn(64, 128).bfloat16()
    Y, H = rn(128, 64), rn(64, 64)
    out = torch.full((128, 384), float("nan"), device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    lib = _capi.load()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.rewy_selftest_tensor_core(p(A), p(B), p(Akk), p(dR), p(Y), p(H), p(out), p(err),
                                       _capi.current_stream(torch.device(DEV)))
    assert rc == 0
    torch.cuda.synchronize()
    assert err.item() == 0, f"a bounded wait gave up at site {err.item()}"
    Af, Bf = A.double(), B.double()
    Yt, Ht = _tf32(Y).double(), _tf32(H).double()
    want = {
        "A B^T (K-major BF16)": (out[:, 0:64], Af @ Bf.T),
        "-(A B^T) (negated A)": (out[:, 64:128], -(Af @ Bf.T)),
        "Akk^T dR (MN-major BF16)": (out[:64, 128:256], Akk.double().T @ dR.double()),
        "Y H^T (TF32 K-major)": (out[:, 256:320], Yt @ Ht.T),
        "A B (BF16, B MN-major)": (out[:, 320:384], Af[:, :64] @ Bf[:64, :64]),
    }
    errs = {n: ((got.double() - ref).norm() / ref.norm()).item() for n, (got, ref) in want.items()}
    assert all(e < 1e-5 for e in errs.values()), errs


def test_a_bounded_wait_that_runs_out_returns_and_is_reported():
    """The failure path of every device-side wait: a wait on an mbarrier phase that nothing completes gives up after
    its limit (2 ms here), records its site in the status word, the CTA folds the per-thread flags and returns
    normally; the host then reads REWY_ERR_DEVICE.  Nothing faults, traps or spins without a bound, and the context
    stays usable (the operand self-test runs afterwards in the same process)."""
    lib = _capi.load()
    words = torch.zeros(2, dtype=torch.int32, device=DEV)      # [status word, wide-chunk count] like a control block
    done = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = _capi.current_stream(torch.device(DEV))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    with torch.cuda.device(DEV):
        assert lib.rewy_selftest_bounded_wait(p(words), p(done), 2000, 77, stream) == 0
        torch.cuda.synchronize()
        assert done.item() == 2 and words[0].item() == 77
        assert lib.rewy_device_status(p(words), stream) == 6          # REWY_ERR_DEVICE
        assert b"site 77" in lib.rewy_last_error()
        # the first failing site is kept: a second give-up does not overwrite it
        assert lib.rewy_selftest_bounded_wait(p(words), p(done), 1000, 78, stream) == 0
        torch.cuda.synchronize()
        assert words[0].item() == 77
    test_tensor_core_operand_forms()
