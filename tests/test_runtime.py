"""CPU tests of the host layer: selection, dispatch report, rejection envelope, C-ABI exports.
Mirrors the reference's control-plane tests (tests/test_runtime.py:6-33)."""
import ctypes
import re
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_import_has_no_side_effects():
    code = ("import sys; import rewy_b200; "
            "assert 'torch' not in sys.modules and 'fla' not in sys.modules and 'ctypes' not in sys.modules; print('ok')")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_nested_use_backend_restores_on_exception():
    from rewy_b200 import runtime, use_backend
    assert runtime.selection().backend == "original"
    with use_backend("optimized", ops=("kda",)):
        assert runtime.selection().ops == ("kda",)
        with pytest.raises(ZeroDivisionError):
            with use_backend("original"):
                assert runtime.selection().backend == "original"
                1 / 0
        assert runtime.selection().backend == "optimized"
    assert runtime.selection().backend == "original"


def test_unknown_backend_and_operator_rejected():
    from rewy_b200 import runtime
    with pytest.raises(ValueError):
        runtime.configure("fastest")
    with pytest.raises(ValueError):
        runtime.configure("optimized", ops=("kda", "mamba"))
    with pytest.raises(ValueError):
        runtime.operator("mamba")


def test_assert_used_reports_missing_backward():
    import rewy_b200 as fdr
    fdr.stats(reset=True)
    with pytest.raises(RuntimeError, match="No optimized_backward calls"):
        fdr.assert_used(("kda",))
    fdr.runtime.record("kda", "optimized_backward")
    fdr.assert_used(("kda",))
    assert fdr.stats(reset=True) == {"kda.optimized_backward": 1}
    rep = fdr.dispatch_report()
    assert set(rep) == {"backend", "counts", "count_boundary"}


@pytest.mark.parametrize("mutate,reason", [
    (lambda a: a.update(q=a["q"].float()), "BF16"),
    (lambda a: a.update(q=a["q"][:, :0], k=a["k"][:, :0], v=a["v"][:, :0]), "must be positive"),
    (lambda a: a.update(chunk_size=32), "chunk_size=64"),
    (lambda a: a.update(cu_seqlens=torch.tensor([0, 100, 120])), "packed sequences need"),
    (lambda a: a.update(scale=0.5), "custom scale"),
    (lambda a: a.update(safe_gate=True), "safe_gate"),
    (lambda a: a.update(v=torch.zeros(1, 128, 2, 256, dtype=torch.bfloat16)), "above K=V=128"),
    (lambda a: a.update(q=a["q"][..., :64], k=a["k"][..., :64], use_gate_in_kernel=True), "fused gate needs K=128"),
    (lambda a: a.update(v=a["v"][:, :, :1]), "unequal q/k/v"),
    (lambda a: a.update(v=a["v"][:, :64]), "unequal q/k/v"),
])
def test_rejection_envelope(mutate, reason):
    from rewy_b200.runtime import rejection_reason
    t = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    args = dict(q=t, k=t, v=t)
    assert rejection_reason("kda", args, device_types=("cpu",)) is None
    mutate(args)
    got = rejection_reason("kda", args, device_types=("cpu",))
    assert got is not None and reason in got, got


def test_fused_gate_and_value_first_states_follow_the_reference_envelope():
    """KDA accepts the fused gate activation and the value-first state layout (docs/compatibility.md:12-13 of the
    reference); GDN and GDN2 reject the fused gate with the reference's wording (runtime.py:103-104)."""
    from rewy_b200.runtime import rejection_reason
    t = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    args = dict(q=t, k=t, v=t, use_gate_in_kernel=True, state_v_first=True)
    assert rejection_reason("kda", args, device_types=("cpu",)) is None
    assert rejection_reason("gdn", args, device_types=("cpu",)) == "GDN fused gate is not release-validated"
    assert rejection_reason("gdn2", args, device_types=("cpu",)) == "GDN2 fused gate is not release-validated"
    assert rejection_reason("gdn", dict(q=t, k=t, v=t, state_v_first=True), device_types=("cpu",)) is None


def test_packed_sequences_and_ragged_lengths_are_accepted():
    from rewy_b200.runtime import rejection_reason
    t = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16)
    ok = dict(q=t, k=t, v=t, cu_seqlens=torch.tensor([0, 64, 256]))
    assert rejection_reason("kda", ok, device_types=("cpu",)) is None
    assert rejection_reason("delta", dict(ok, cu_seqlens_cpu=torch.tensor([0, 128, 256])), device_types=("cpu",)) is None
    assert rejection_reason("kda", dict(ok, cu_seqlens=torch.tensor([0, 37, 256])), device_types=("cpu",)) is None
    four = torch.zeros(1, 256, 4, 128, dtype=torch.bfloat16)           # grouped value heads: HV = 2 H
    assert rejection_reason("kda", dict(q=t, k=t, v=four), device_types=("cpu",)) is None
    narrow = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16)         # K = 64 keys, V = 128 values
    assert rejection_reason("gdn", dict(q=narrow, k=narrow, v=t), device_types=("cpu",)) is None
    odd = torch.zeros(2, 100, 2, 128, dtype=torch.bfloat16)
    assert rejection_reason("gdn", dict(q=odd, k=odd, v=odd), device_types=("cpu",)) is None
    for bad in ([0, 64, 200], [0, 256, 256], [64, 256], [0, 128]):
        assert "packed sequences need" in rejection_reason("kda", dict(ok, cu_seqlens=torch.tensor(bad)), device_types=("cpu",))
    two = torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16)
    assert "packed sequences need" in rejection_reason("kda", dict(q=two, k=two, v=two, cu_seqlens=torch.tensor([0, 256])),
                                                       device_types=("cpu",))


def test_ragged_lengths_are_padded_to_the_chunk_and_cut_back():
    """Host logic of the neutral padding: indices, padded offsets, differentiable pad and cut."""
    from rewy_b200.functions import _Ragged
    assert not _Ragged(128, "cpu").needed
    rg = _Ragged(100, "cpu")
    x = torch.arange(2 * 100 * 3, dtype=torch.float32).reshape(2, 100, 3).requires_grad_()
    y = rg.pad(x, -1.0)
    assert y.shape == (2, 128, 3) and torch.equal(y[:, :100], x) and bool((y[:, 100:] == -1).all())
    assert torch.equal(rg.cut(y), x)
    assert not _Ragged(256, "cpu", torch.tensor([0, 64, 256])).needed
    rg = _Ragged(167, "cpu", torch.tensor([0, 37, 101, 167]))          # lengths 37, 64, 66 -> 64, 64, 128
    assert rg.needed and rg.total == 256 and rg.cu.tolist() == [0, 64, 128, 256]
    x = torch.randn(1, 167, 2, requires_grad=True)
    y = rg.pad(x)
    assert torch.equal(y[0, :37], x[0, :37]) and torch.equal(y[0, 64:128], x[0, 37:101]) and torch.equal(y[0, 128:194], x[0, 101:])
    assert bool((y[0, 37:64] == 0).all()) and bool((y[0, 194:] == 0).all())
    (rg.cut(y) * 2).sum().backward()
    assert torch.equal(x.grad, torch.full_like(x, 2.0))


def test_rejection_on_cpu_tensors_is_device():
    from rewy_b200.runtime import rejection_reason
    t = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    assert rejection_reason("kda", dict(q=t, k=t, v=t)) == "CUDA required"
    assert rejection_reason("kda", dict(q=t[0], k=t, v=t)) == "expected rank-4 q/k/v"


def test_strict_rejection_raises_and_counts():
    import rewy_b200 as fdr
    fdr.stats(reset=True)
    t = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    with fdr.use_backend("optimized"):
        with pytest.raises(RuntimeError, match="rewy_b200 kda: CUDA required"):
            fdr.chunk_kda(t, t, t, torch.zeros(1, 128, 2, 128), torch.zeros(1, 128, 2))
    assert fdr.stats(reset=True) == {"kda.rejected:CUDA required": 1}


def test_backward_functions_refuse_cpu_tensors():
    from rewy_b200 import backward
    t = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        backward.delta_backward(t, t, t, torch.zeros(1, 128, 2), torch.zeros(1, 128, 2, 64), 1.0, None, t, None)


def test_shared_library_exports_every_declared_symbol():
    """Every function declared in include/rewy_b200.h is exported by the built library."""
    from rewy_b200 import _capi
    header = (ROOT / "include" / "rewy_b200.h").read_text()
    declared = set(re.findall(r"^\s*(?:const\s+char\*|int|size_t)\s+(rewy_\w+)\s*\(", header, re.M))
    assert declared == set(_capi.EXPORTS), declared ^ set(_capi.EXPORTS)
    lib = ctypes.CDLL(str(_capi.library_path()))
    for name in declared:
        assert hasattr(lib, name), name
    assert b"sm_100a" in _capi.load().rewy_version()


def test_struct_layout_matches_header_field_order():
    from rewy_b200 import _capi
    header = (ROOT / "include" / "rewy_b200.h").read_text()
    body = header[header.index("typedef struct RewyBwdArgs {"):header.index("} RewyBwdArgs;")]
    fields = re.findall(r"^\s*(?:const\s+)?(?:void|float|int32_t|size_t)\s*\*?\s*([\w, ]+);", body, re.M)
    names = [n.strip() for f in fields for n in f.split(",")]
    assert names == [n for n, _ in _capi.BwdArgs._fields_]
    body = header[header.index("typedef struct RewyStageBuffers {"):header.index("} RewyStageBuffers;")]
    names = re.findall(r"^\s*void\*\s+(\w+);", body, re.M)
    assert names == [n for n, _ in _capi.StageBuffers._fields_]


def test_argument_validation_without_a_gpu():
    """Status codes for bad arguments are produced before any CUDA call."""
    from rewy_b200 import _capi
    lib = _capi.load()
    a = _capi.BwdArgs()
    a.family, a.B, a.T, a.H = _capi.KDA, 1, 100, 1
    assert lib.rewy_kda_bwd(a, None) == 2 and b"multiple of 64" in lib.rewy_last_error()
    a.T = 128
    assert lib.rewy_kda_bwd(a, None) == 1 and b"'q'" in lib.rewy_last_error()
    assert lib.rewy_gdn_bwd(a, None) == 7
    # maximum size: 2^29 token-heads is the last accepted problem (then the first missing pointer is reported)
    a.B, a.T, a.H = 64, 1 << 17, 64
    assert lib.rewy_kda_bwd(a, None) == 1
    a.T = (1 << 17) + 64
    assert lib.rewy_kda_bwd(a, None) == 2 and b"2^29" in lib.rewy_last_error()
    f = _capi.FwdArgs()
    f.family, f.B, f.T, f.H = _capi.KDA, 64, (1 << 17) + 64, 64
    assert lib.rewy_chunk_fwd(f, None) == 2 and b"2^29" in lib.rewy_last_error()
    a.B, a.T, a.H = 1, 128, 1
    assert lib.rewy_bwd_workspace_bytes(_capi.KDA, _capi.SAVED, 1, 128, 1) == 256 + 128 * (512 + 2 * 256)
    assert lib.rewy_bwd_workspace_bytes(_capi.GDN, _capi.RECOMPUTE, 1, 128, 1) == 256 + 128 * (512 + 2 * 256 + 5 * 256 + 512 + 128)


def test_forward_producer_matches_oracle_forward_on_cpu():
    """The torch statement of the forward (BF16 operands; the cross-check of the CUDA forward) against the FP64 chunked
    forward of the oracle; the CUDA forward itself refuses CPU tensors."""
    from rewy_b200.forward import chunk_forward as cuda_forward
    t = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        cuda_forward("delta", t, t, t, beta=torch.zeros(1, 64, 1))
    from oracle import chunk_forward as oracle_forward
    from rewy_b200.forward import chunk_forward_torch as chunk_forward
    from rewy_b200.synthetic import make_inputs, operator_inputs
    for op in ("kda", "gdn", "gdn2", "delta"):
        xs = make_inputs(op, 1, 128, 2, seed=8)
        ins = operator_inputs(op, xs)
        kw = {n: ins[n] for n in ins if n not in ("initial_state",)}
        got = chunk_forward(op, initial_state=ins["initial_state"], **kw)
        ref = oracle_forward(op, ins)
        for n in ("o", "final_state", "Aqk", "Akk", "w", "u", "qg", "kg", "v_new", "h"):
            err = ((got[n].double() - ref[n]).norm() / ref[n].norm()).item()
            assert err < 6e-3, (op, n, err)
        if op != "delta":
            assert torch.allclose(got["g_cumsum"].double(), ref["g_cumsum"], atol=1e-5)


def _fake_stage_call(family, skew=None):
    """A chunk-stage call whose pointers are made-up, 16-byte aligned addresses (never dereferenced: validation
    happens on the host before any CUDA call); `skew` names one pointer that is moved off the 16-byte grid."""
    from rewy_b200 import _capi
    a, s = _capi.BwdArgs(), _capi.StageBuffers()
    a.family, a.B, a.T, a.H, a.out_dtype, a.scale = family, 1, 128, 2, _capi.OUT_F32, 1.0
    names_a = ["q", "k", "v", "Akk", "d_o", "dq", "dk", "dv", "g", "dg"]
    names_a += ["b_gate", "w_gate", "db_gate", "dw_gate"] if family == _capi.GDN2 else ["beta", "dbeta"]
    addr = 0x10000
    for n in names_a:
        setattr(a, n, addr + (4 if n == skew else 0))
        addr += 0x1000
    for n in ("v_new", "h", "dh", "dR", "dR_lo", "ctrl"):
        setattr(s, n, addr + (4 if n == skew else 0))
        addr += 0x1000
    return a, s


@pytest.mark.parametrize("entry", ("rewy_stage_chunk_adjoint", "rewy_stage_chunk_adjoint_static"))
@pytest.mark.parametrize("family,skew", [("KDA", "g"), ("KDA", "dg"), ("GDN2", "dw_gate"), ("GDN2", "b_gate"),
                                         ("KDA", "dR_lo"), ("KDA", "dbeta")])
def test_chunk_stage_entries_report_misaligned_pointers_before_any_launch(entry, family, skew):
    """Both chunk-stage entry points run the same host-side checks: a pointer off the 16-byte grid is
    REWY_ERR_ALIGN (3), naming the pointer, and nothing is launched."""
    from rewy_b200 import _capi
    lib = _capi.load()
    a, s = _fake_stage_call(getattr(_capi, family), skew)
    before = lib.rewy_kernel_launch_count()
    assert getattr(lib, entry)(a, s, None) == 3
    assert skew.encode() in lib.rewy_last_error()
    assert lib.rewy_kernel_launch_count() == before


def test_static_chunk_stage_checks_the_grid_limit_and_missing_pointers():
    from rewy_b200 import _capi
    lib = _capi.load()
    a, s = _fake_stage_call(_capi.KDA)
    a.B, a.H, a.T = 2048, 32, 64            # B*H = 65536 is beyond the grid limit, yet within the block's chunk count
    assert lib.rewy_stage_chunk_adjoint_static(a, s, None) == 2 and b"65535" in lib.rewy_last_error()
    a, s = _fake_stage_call(_capi.KDA)
    a.dbeta = None
    assert lib.rewy_stage_chunk_adjoint_static(a, s, None) == 1 and b"dbeta" in lib.rewy_last_error()


def test_intra_passes_is_an_option_of_the_warp_mma_variant_only():
    from rewy_b200 import _capi
    lib = _capi.load()
    a, s = _fake_stage_call(_capi.KDA)
    for passes, want in ((1, 7), (2, 7), (4, 7)):
        a.intra_passes = passes
        assert lib.rewy_stage_chunk_adjoint(a, s, None) == want, passes
    assert b"intra_passes" in lib.rewy_last_error()
    a.intra_passes, a.family, a.policy, a.T = 2, _capi.KDA, _capi.SAVED, 128
    assert lib.rewy_kda_bwd(a, None) == 7


def test_selftest_bounded_wait_rejects_bad_arguments():
    from rewy_b200 import _capi
    lib = _capi.load()
    assert lib.rewy_selftest_bounded_wait(None, None, 1000, 5, None) == 1
    assert lib.rewy_selftest_bounded_wait(0x1000, 0x2000, 0, 5, None) == 7
    assert lib.rewy_selftest_bounded_wait(0x1000, 0x2000, 2000000, 5, None) == 7


def test_fla_integration_patches_and_restores_public_aliases():
    """enable(integrations=('fla',)) makes FLA's public names resolve to the dispatching entries; the captured
    originals stay reachable; uninstall puts the aliases back.  Families the installed FLA lacks are reported."""
    fla = pytest.importorskip("fla")
    import importlib
    from rewy_b200 import integrations, runtime
    mod = importlib.import_module("fla.ops.kda")
    before = mod.chunk_kda
    try:
        report = integrations.install()
        assert "kda" in report["patched"] and "gdn" in report["patched"] and "delta" in report["patched"]
        assert mod.chunk_kda is runtime.operator("kda")
        assert importlib.import_module("fla.ops.kda.chunk").chunk_kda is runtime.operator("kda")
        assert importlib.import_module("fla.ops.delta_rule").chunk_delta_rule is runtime.operator("delta")
        assert runtime.original_operator("kda") is not runtime.operator("kda")
        assert integrations.install() is report                      # idempotent
        for op, why in report["skipped"].items():
            assert "no original (FLA) operator" in why, (op, why)
    finally:
        integrations.uninstall()
    assert mod.chunk_kda is before


def test_model_bindings_change_one_attribute_and_are_restored():
    """The two model bindings of the reference (integrations/models.py:5-15): one attribute of one module each."""
    import sys
    import types
    import rewy_b200 as fdr
    from rewy_b200 import integrations, runtime
    pkg, layer = types.ModuleType("lit_gpt"), types.ModuleType("lit_gpt.gdn2")
    theirs = lambda *a, **k: None
    layer.chunk_gdn2 = theirs
    pkg.gdn2 = layer
    sys.modules["lit_gpt"], sys.modules["lit_gpt.gdn2"] = pkg, layer
    try:
        fdr.enable("original", integrations=("gdn2",))
        assert layer.chunk_gdn2 is runtime.operator("gdn2")
        integrations.uninstall()
        assert layer.chunk_gdn2 is theirs
        del layer.chunk_gdn2
        with pytest.raises(RuntimeError, match="has no chunk_gdn2"):
            fdr.enable("original", integrations=("gdn2",))
    finally:
        integrations.uninstall()
        fdr.disable()
        del sys.modules["lit_gpt"], sys.modules["lit_gpt.gdn2"]
    with pytest.raises(RuntimeError, match="not importable"):
        fdr.enable("original", integrations=("gdn2",))
    fdr.disable()
    qwen = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
    before = qwen.torch_chunk_gated_delta_rule
    try:
        fdr.enable("original", integrations=("qwen3_5",))
        assert qwen.torch_chunk_gated_delta_rule is runtime.operator("gdn")
    finally:
        integrations.uninstall()
        fdr.disable()
    assert qwen.torch_chunk_gated_delta_rule is before


def test_launcher_runs_a_script_and_writes_the_dispatch_report(tmp_path):
    """`python -m rewy_b200 run`: the script runs unmodified with its own argv, the report is written, and an optimized
    run without any optimized backward is an error unless it is declared forward-only (reference: cli.py:70-95)."""
    import json
    import sys
    pytest.importorskip("fla")
    from rewy_b200 import disable, integrations, launcher
    script = tmp_path / "train.py"
    script.write_text("import sys, pathlib\npathlib.Path(sys.argv[1]).write_text(' '.join(sys.argv[1:]))\n")
    marker, report = tmp_path / "ran.txt", tmp_path / "out" / "report.json"
    argv_before = sys.argv[:]
    try:
        assert launcher.main(["run", "--backend", "original", "--report", str(report), str(script), str(marker), "--lr", "3"]) == 0
        assert marker.read_text() == f"{marker} --lr 3" and sys.argv == argv_before
        got = json.loads(report.read_text())
        assert got["backend"] == "original" and got["counts"] == {} and "count_boundary" in got
        with pytest.raises(RuntimeError, match="No optimized backward ran"):
            launcher.main(["run", "--report", str(report), str(script), str(marker)])
        assert json.loads(report.read_text())["backend"] == "optimized"     # written even when the run is refused
        assert launcher.main(["run", "--allow-no-backward", str(script), str(marker)]) == 0
        failing = tmp_path / "fail.py"
        failing.write_text("raise SystemExit(3)\n")
        with pytest.raises(SystemExit):
            launcher.main(["run", "--backend", "original", str(failing)])
    finally:
        integrations.uninstall()
        disable()
    assert set(launcher.doctor()) >= {"python", "torch", "library", "cuda_available"}


def test_unknown_integration_is_rejected():
    import rewy_b200 as fdr
    with pytest.raises(ValueError, match="Unknown integration"):
        fdr.enable("original", integrations=("jax",))


def test_custom_op_is_registered_with_a_shape_only_implementation():
    """The backward is one torch custom operator over the C ABI; its fake implementation gives the output shapes and
    dtypes of every family without touching a device."""
    from rewy_b200 import _capi, backward
    assert "rewy_b200::family_bwd" in str(torch.ops.rewy_b200.family_bwd.default._schema)
    B, T, H = 2, 128, 3
    m = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="meta")
    big, a64 = m(B, T, H, 128), m(B, T, H, 64)
    ws = m(1024, dt=torch.uint8)
    g = m(B, T, H, 128, dt=torch.float32)
    h0 = m(B, H, 128, 128, dt=torch.float32)
    r = backward._family_bwd_fake(_capi.KDA, _capi.RECOMPUTE, False, 0, False, 1.0, big, big, big, big, a64, ws, g,
                                  m(B, T, H, dt=torch.float32), None, None, a64, h0, h0, None, None, None, None, None, None)
    assert [tuple(x.shape) for x in r] == [(B, T, H, 128)] * 4 + [(B, T, H), (0,), (0,), (B, H, 128, 128)]
    assert r[0].dtype == torch.bfloat16 and r[3].dtype == torch.float32
    r = backward._family_bwd_fake(_capi.GDN2, _capi.SAVED, True, 0, True, 1.0, big, big, big, big, a64, ws, g, None, big, big,
                                  a64, None, None, big, big, big, big, m(B, T // 64, H, 128, 128), None)
    assert [tuple(x.shape) for x in r] == [(B, T, H, 128)] * 4 + [(0,)] + [(B, T, H, 128)] * 2 + [(0,)]
    assert r[0].dtype == torch.float32 and r[5].dtype == torch.float32
