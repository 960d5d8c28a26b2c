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
