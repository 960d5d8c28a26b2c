"""Regenerates the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN CPU CODE.

Needs the reference checkout (read-only) and runs only where it is mounted; the tests read the
committed .npz files and never the reference tree.  Usage:
    python tests/golden/make_golden.py /path/to/reference

What is produced:
  recurrence_<op>.npz   seeded inputs of src/fast_delta_rule/validation.py:6-21 (``inputs``, seed 42,
                        T=128, H=1) and the FP64 gradients of its token ``recurrence`` (:23-38) obtained
                        exactly as ``verify`` does (:55-58).
  closed_form_seed79.npz  inputs/outputs of ``backward`` in benchmarks/plotting/check_manuscript_math.py:21-54
                        (function text executed from the reference file; the script part is not run).
  intra_<family>.npz    the reference's captured matrix-intra inputs validation/npu950_intra/<family>.npz
                        (copied verbatim as data) and the outputs of ``oracle`` in
                        scripts/npu950_intra_regression.py:25-46 at gate scales 1 and 3.
"""
import hashlib
import importlib.util
import json
import shutil
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def recurrence_fixtures(ref):
    sys.path.insert(0, str(ref / "src"))
    sys.dont_write_bytecode = True
    from fast_delta_rule import validation
    for op in ("kda", "gdn", "gdn2", "delta"):
        xs = validation.inputs(op, "cpu", length=128, heads=1)
        cpu = {n: x.detach().cpu().double().requires_grad_() for n, x in xs.items()}
        do = torch.randn_like(xs["v"])
        dh = torch.randn_like(xs["initial_state"])
        expected = validation.recurrence(op, cpu)
        grads = torch.autograd.grad(expected, tuple(cpu.values()), (do.double(), dh.double()))
        arrays = {f"in_{n}": x.detach().float().numpy() for n, x in xs.items()}
        arrays["in_do"] = do.float().numpy()
        arrays["in_dht"] = dh.float().numpy()
        arrays.update({f"grad_{n}": g.numpy().astype(np.float32) for n, g in zip(cpu, grads)})
        arrays["out_o"] = expected[0].detach().numpy().astype(np.float32)
        arrays["out_final_state"] = expected[1].detach().numpy().astype(np.float32)
        np.savez_compressed(HERE / f"recurrence_{op}.npz", **arrays)


def closed_form_fixture(ref):
    text = (ref / "benchmarks/plotting/check_manuscript_math.py").read_text()
    start = text.index("def recurrence(")
    stop = text.index("rng=np.random.default_rng(79)")
    scope = {"np": np}
    exec(compile(text[start:stop], "check_manuscript_math_functions", "exec"), scope)
    backward = scope["backward"]
    rng = np.random.default_rng(79)
    arrays = {}
    for family in ("delta", "gdn", "kda", "gdn2"):
        n, k, v = 8, 6, 5
        Q = rng.normal(size=(n, k)) * .3
        K = rng.normal(size=(n, k)) * .2
        V = rng.normal(size=(n, v))
        S = rng.normal(size=(k, v)) * .2
        g = rng.uniform(-.3, .08, size=(n, k))
        if family == "delta":
            g[:] = 0
        if family == "gdn":
            g[:] = g[:, :1]
        beta = rng.uniform(.1, .9, size=(n, 1))
        beta[0] = 0
        b = np.broadcast_to(beta, (n, k)).copy()
        w = np.broadcast_to(beta, (n, v)).copy()
        if family == "gdn2":
            b = rng.uniform(-.1, .9, size=(n, k))
            w = rng.uniform(-.1, .9, size=(n, v))
        do = rng.normal(size=(n, v))
        ds = rng.normal(size=(k, v))
        bars, _, P, R = backward(Q, K, V, g, b, w, S, do, ds)
        for name, x in zip(("Q", "K", "V", "g", "b", "w", "S", "do", "ds"), (Q, K, V, g, b, w, S, do, ds)):
            arrays[f"{family}_in_{name}"] = x
        for name, x in zip(("qb", "kb", "vb", "gb", "bb", "wb", "sb"), bars):
            arrays[f"{family}_out_{name}"] = x
        arrays[f"{family}_out_P"] = P
        arrays[f"{family}_out_R"] = R
    np.savez_compressed(HERE / "closed_form_seed79.npz", **arrays)


def intra_fixtures(ref):
    mod = _load(ref / "scripts/npu950_intra_regression.py", "ref_intra_regression")
    meta = json.loads((ref / "validation/npu950_intra/metadata.json").read_text())
    for family in ("kda", "gdn2"):
        src = ref / f"validation/npu950_intra/{family}.npz"
        assert hashlib.sha256(src.read_bytes()).hexdigest() == meta[family]["fixture_sha256"]
        shutil.copyfile(src, HERE / f"intra_{family}_inputs.npz")
        (HERE / f"intra_{family}_inputs.npz").chmod(0o644)
        data, _ = mod.load_fixture(family)
        arrays = {}
        for scale in (1.0, 3.0):
            x = {n: a.copy() for n, a in data.items()}
            x["g"] = x["g"] * scale
            for name, out in zip(("dq", "dk", "db", "dg"), mod.oracle(x, family)):
                arrays[f"scale{scale:g}_{name}"] = out.astype(np.float32)
        np.savez_compressed(HERE / f"intra_{family}_expected.npz", **arrays)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python make_golden.py <checkout of the reference (flashserve/ReWY)>")
    ref = Path(sys.argv[1])
    recurrence_fixtures(ref)
    closed_form_fixture(ref)
    intra_fixtures(ref)
    print("golden fixtures written to", HERE)
