"""``python -m rewy_b200 run [options] script.py [args...]``: run an unmodified training script with the backend
selected, then write the dispatch report.  ``python -m rewy_b200 doctor`` prints what is installed.

Counterpart of the reference's launcher (src/fast_delta_rule/cli.py:27-95, the ``run`` and ``doctor`` commands):
same options and the same rule that an "optimized" run in which no optimized backward was counted is an error
unless ``--allow-no-backward`` is given.  The report is ``{"backend", "counts", "count_boundary"}`` as a JSON file
and as one line on stderr.
"""
import argparse
import importlib.metadata
import json
import os
import runpy
import sys
from pathlib import Path


def doctor():
    """Versions of what the package builds on, whether the CUDA library is built and whether a GPU is visible."""
    from . import _capi
    found = {"python": sys.version.split()[0], "platform": sys.platform}
    for name in ("torch", "triton", "flash-linear-attention", "transformers"):
        try:
            found[name] = importlib.metadata.version(name)
        except importlib.metadata.PackageNotFoundError:
            found[name] = None
    found["library"] = str(_capi.LIB_PATH) if _capi.LIB_PATH.exists() else None
    try:
        import torch
        found["cuda_available"] = torch.cuda.is_available()
        if found["cuda_available"]:
            found["device"] = torch.cuda.get_device_name()
    except Exception as exc:  # a broken torch install is a finding, not a crash of the diagnosis
        found["cuda_available"] = f"torch not importable: {exc}"
    return found


def run(backend, fallback, ops, integrations, report, allow_no_backward, script, script_args):
    from . import enable, stats
    from .runtime import dispatch_report
    enable(backend, strict=fallback == "error", ops=ops, integrations=integrations)
    stats(reset=True)
    print(f"[rewy_b200] backend={backend} ops={','.join(ops)} fallback={fallback}", file=sys.stderr)
    saved_argv, saved_path = sys.argv[:], sys.path[:]
    sys.argv = [script] + list(script_args)
    sys.path.insert(0, str(Path(script).resolve().parent))
    try:
        try:
            runpy.run_path(script, run_name="__main__")
        except SystemExit as stop:
            if stop.code not in (None, 0):
                raise
        counts = stats()
        if backend == "optimized" and not allow_no_backward and not any(counts.get(f"{op}.optimized_backward", 0) for op in ops):
            raise RuntimeError("No optimized backward ran. Check --integration/--ops; use --allow-no-backward only for "
                               "forward-only scripts.")
    finally:
        result = dispatch_report()
        print("[rewy_b200] " + json.dumps(result), file=sys.stderr)
        if report is not None:
            report.parent.mkdir(parents=True, exist_ok=True)
            report.write_text(json.dumps(result, indent=2) + "\n")
        sys.argv, sys.path[:] = saved_argv, saved_path


def main(argv=None):
    parser = argparse.ArgumentParser(prog="python -m rewy_b200",
                                     description="Select the delta-rule backend without editing the training script.")
    commands = parser.add_subparsers(dest="command", required=True)
    commands.add_parser("doctor")
    r = commands.add_parser("run")
    r.add_argument("--backend", choices=("original", "optimized"), default=os.getenv("REWY_BACKEND", "optimized"))
    r.add_argument("--fallback", choices=("error", "original"), default="error")
    r.add_argument("--ops", default="kda,gdn,gdn2,delta")
    r.add_argument("--integration", action="append", choices=("fla", "qwen3_5", "gdn2"))
    r.add_argument("--report", type=Path)
    r.add_argument("--allow-no-backward", action="store_true")
    r.add_argument("script")
    r.add_argument("args", nargs=argparse.REMAINDER)
    a = parser.parse_args(argv)
    if a.command == "doctor":
        print(json.dumps(doctor(), indent=2))
        return 0
    run(a.backend, a.fallback, tuple(a.ops.split(",")), tuple(a.integration or ("fla",)), a.report, a.allow_no_backward,
        a.script, a.args)
    return 0
