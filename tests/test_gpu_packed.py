"""Packed sequences (FLA's cu_seqlens) whose lengths are multiples of 64 (the form the library itself takes; other
lengths are padded to it by the operators): the chunk-local kernels do not see sequence
boundaries, the two state scans take per-sequence bounds.  A packed batch must give, sequence by sequence, exactly what
the same sequences give when they are run one at a time (same kernels, same arithmetic order), for the forward outputs
and every gradient, with initial states and final-state gradients per sequence.  The reference's kernels take cu_seqlens
on the same terms (kernels/vector_state_gpu.py:20-23,50-57; research/operators/a800_ablation/run.py:19) although its
release envelope rejects them.
"""
import pytest
import torch

from rewy_b200 import _capi
from rewy_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LENGTHS = (128, 64, 192)
NAMES = {"kda": "chunk_kda", "gdn2": "chunk_gdn2", "gdn": "chunk_gated_delta_rule", "delta": "chunk_delta_rule"}
ARGS = {"kda": ("q", "k", "v", "g", "beta"), "gdn2": ("q", "k", "v", "g", "b", "w"), "gdn": ("q", "k", "v", "g", "beta"),
        "delta": ("q", "k", "v", "beta")}


def _sequences(op):
    return [make_inputs(op, 1, T, 2, seed=50 + i, device=DEV, gate_scale=0.1, gate="softplus") for i, T in enumerate(LENGTHS)]


def _run(op, tensors, h0, do, dht, saved, cu=None):
    import rewy_b200 as fdr
    ins = {n: t.detach().clone().requires_grad_() for n, t in tensors.items()}
    h0 = h0.detach().clone().requires_grad_()
    kw = dict(output_final_state=True, initial_state=h0)
    if op in ("kda", "gdn2"):
        kw["disable_recompute"] = saved
    if cu is not None:
        kw["cu_seqlens"] = cu
    with fdr.use_backend("optimized", ops=(op,)):
        o, fin = getattr(fdr, NAMES[op])(**ins, **kw)
    grads = torch.autograd.grad((o, fin), tuple(ins.values()) + (h0,), (do, dht))
    return o, fin, dict(zip(tuple(ins) + ("initial_state",), grads))


@pytest.mark.parametrize("op,saved", [("kda", True), ("kda", False), ("gdn2", True), ("gdn", False), ("delta", False)])
def test_packed_batch_equals_its_sequences_run_one_at_a_time(op, saved):
    seqs = _sequences(op)
    cat = lambda n: torch.cat([s[n] for s in seqs], 1)
    packed = {n: cat(n) for n in ARGS[op]}
    h0 = torch.cat([s["initial_state"] for s in seqs], 0)          # [sequences, H, K, V]
    dht = torch.cat([s["dht"] for s in seqs], 0)
    do = cat("do")
    cu = torch.tensor([0, 128, 192, 384], dtype=torch.int64, device=DEV)
    o, fin, grads = _run(op, packed, h0, do, dht, saved, cu)
    assert fin.shape == (3, 2, 128, 128) and grads["initial_state"].shape == (3, 2, 128, 128)
    at = 0
    for i, s in enumerate(seqs):
        T = LENGTHS[i]
        o1, fin1, g1 = _run(op, {n: s[n] for n in ARGS[op]}, s["initial_state"], s["do"], s["dht"], saved)
        assert torch.equal(o[:, at:at + T], o1), (op, i, "o")
        assert torch.equal(fin[i:i + 1], fin1), (op, i, "final_state")
        for n in ARGS[op]:
            assert torch.equal(grads[n][:, at:at + T], g1[n]), (op, i, n)
        assert torch.equal(grads["initial_state"][i:i + 1], g1["initial_state"]), (op, i, "initial_state")
        at += T


def test_offsets_that_do_not_match_the_token_count_are_refused_and_the_kernels_check_lengths():
    """The operators refuse offsets that do not add up on the host (lengths that are not multiples of 64 are padded
    there, tests/test_gpu_envelope.py); the scan kernels, given such offsets directly, record the length in the status
    word and leave their sequence untouched."""
    import rewy_b200 as fdr
    from rewy_b200.forward import chunk_forward
    xs = make_inputs("kda", 1, 256, 2, seed=3, device=DEV)
    with fdr.use_backend("optimized"):
        with pytest.raises(RuntimeError, match="packed sequences need"):
            fdr.chunk_kda(xs["q"], xs["k"], xs["v"], xs["g"], xs["beta"],
                          cu_seqlens=torch.tensor([0, 100, 200], device=DEV))
    with pytest.raises(RuntimeError, match="device status"):
        chunk_forward("kda", xs["q"], xs["k"], xs["v"], g=xs["g"], beta=xs["beta"], check_status=True,
                      cu_seqlens=torch.tensor([0, 100, 256], device=DEV))
