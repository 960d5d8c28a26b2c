"""Explicit backend selection and the dispatch report.

Mirrors the reference's selection/audit runtime (src/fast_delta_rule/runtime.py:22-149): a
context-local ``Selection``, process-global counters keyed ``<op>.<event>`` with the events
``optimized_forward``, ``optimized_backward``, ``original_forward``, ``fallback_forward`` and
``rejected:<reason>``, ``stats()``, ``assert_used()`` and the capability-based rejection envelope.
Differences: there is no FLA fingerprint check (this package does not patch FLA), and there is no
silent fallback — a rejected call raises in strict mode and, in non-strict mode, is forwarded to the
installed FLA operator only if one exists.
"""
from collections import Counter
from contextlib import contextmanager
from contextvars import ContextVar
from dataclasses import dataclass
from functools import lru_cache
import importlib
import inspect
import warnings

OPERATORS = {
    "kda": ("kda", "chunk_kda"),
    "gdn": ("gated_delta_rule", "chunk_gated_delta_rule"),
    "gdn2": ("gdn2", "chunk_gdn2"),
    "delta": ("delta_rule", "chunk_delta_rule"),
}


@dataclass(frozen=True)
class Selection:
    backend: str = "original"
    strict: bool = True
    ops: tuple = tuple(OPERATORS)


_selection = ContextVar("rewy_b200_selection", default=Selection())
_counts = Counter()
_warned = set()


def record(op, event):
    _counts[f"{op}.{event}"] += 1


def stats(reset=False):
    result = dict(sorted(_counts.items()))
    if reset:
        _counts.clear()
    return result


def selection():
    return _selection.get()


def configure(backend="optimized", *, strict=True, ops=None):
    if backend not in ("original", "optimized"):
        raise ValueError("backend must be original or optimized")
    ops = tuple(OPERATORS) if ops is None else tuple(ops)
    unknown = set(ops) - OPERATORS.keys()
    if unknown:
        raise ValueError(f"Unknown operators: {sorted(unknown)}")
    return _selection.set(Selection(backend, strict, ops))


@contextmanager
def use_backend(backend, *, strict=True, ops=None):
    token = configure(backend, strict=strict, ops=ops)
    try:
        yield
    finally:
        _selection.reset(token)


def dispatch_report():
    """The dispatch report the reference's launcher writes (src/fast_delta_rule/cli.py:86-95)."""
    return {"backend": _selection.get().backend, "counts": stats(),
            "count_boundary": "Python autograd function calls, not kernel launches"}


def assert_used(ops=None, *, backward=True):
    ops = _selection.get().ops if ops is None else ops
    suffix = "optimized_backward" if backward else "optimized_forward"
    missing = [op for op in ops if not _counts.get(f"{op}.{suffix}", 0)]
    if missing:
        raise RuntimeError(f"No {suffix} calls for {missing}; check integration and whether backward ran.")


def rejection_reason(op, arguments, device_types=("cuda",)):
    """Capability envelope, in the reference's order and wording (runtime.py:75-106).
    ``device_types`` exists so the envelope can be exercised on a machine without a GPU."""
    import torch
    q, k, v = (arguments.get(n) for n in ("q", "k", "v"))
    if not all(isinstance(x, torch.Tensor) and x.ndim == 4 for x in (q, k, v)):
        return "expected rank-4 q/k/v"
    if q.device.type not in device_types:
        return "CUDA required"
    if any(x.device != q.device for x in (k, v)):
        return "mixed devices"
    if any(x.dtype != torch.bfloat16 for x in (q, k, v)):
        return "release envelope uses BF16 q/k/v"
    if k.shape[-1] > 128 or v.shape[-1] > 128:
        return "head dimensions above K=V=128 are not supported"  # below: the operators fill up with zero channels
    if q.shape != k.shape or k.shape[:2] != v.shape[:2] or v.shape[2] < k.shape[2] or v.shape[2] % k.shape[2]:
        return "unequal q/k/v shapes"  # grouped value heads (a multiple of the q/k heads) are accepted
    if k.shape[1] < 1:
        return "sequence length must be positive"  # other lengths: the operators pad to the chunk with neutral tokens
    if arguments.get("chunk_size", 64) != 64:
        return "release envelope requires chunk_size=64"
    cu = arguments.get("cu_seqlens")
    if cu is not None:
        # packed sequences are accepted (the reference's release envelope rejects them all: "packed/variable sequences
        # are not release-validated"); lengths that are not multiples of 64 are padded by the operators
        host = arguments.get("cu_seqlens_cpu")
        host = cu.detach().cpu() if host is None else host
        lengths = host[1:] - host[:-1]
        if q.shape[0] != 1 or host.numel() < 2 or int(host[0]) != 0 or int(host[-1]) != k.shape[1] \
                or bool((lengths <= 0).any()):
            return "packed sequences need a batch of 1 and positive lengths that add up to the token count"
    if arguments.get("cp_context") is not None:
        return "context parallelism is not release-validated"
    if arguments.get("safe_gate", False):
        return "safe_gate transform is not release-validated"
    if arguments.get("use_graph", False):
        return "static variable-length graph buffers are not supported"
    if arguments.get("return_intermediate_states", False):
        return "intermediate inference states are not supported"
    scale = arguments.get("scale")
    if scale is not None and scale != k.shape[-1] ** -0.5:
        return "custom scale is not release-validated"
    if op == "kda" and arguments.get("use_gate_in_kernel", False) and k.shape[-1] != 128:
        return "the KDA fused gate needs K=128"
    if op == "gdn" and arguments.get("use_gate_in_kernel", False):
        return "GDN fused gate is not release-validated"
    if op == "gdn2" and arguments.get("use_gate_in_kernel", False):
        return "GDN2 fused gate is not release-validated"
    if op == "delta" and arguments.get("head_first", False):
        return "head-first layout is not supported"
    return None


@lru_cache(None)
def original_operator(op):
    """The installed FLA operator, if any ('original' backend / non-strict forwarding).  Cached at first use, so
    aliases patched later by ``rewy_b200.integrations`` do not shadow it."""
    family, name = OPERATORS[op]
    try:
        module = importlib.import_module(f"fla.ops.{family}.chunk")
    except Exception as exc:  # FLA absent or too old for this family
        raise RuntimeError(f"rewy_b200 {op}: no original (FLA) operator is importable: {exc}") from exc
    return inspect.unwrap(getattr(module, name))


def optimized_operator(op):
    from . import functions
    return getattr(functions, OPERATORS[op][1])


@lru_cache(None)
def operator(op):
    if op not in OPERATORS:
        raise ValueError(f"Unknown operator {op!r}")
    optimized = optimized_operator(op)
    signature = inspect.signature(optimized)

    def call(*args, **kwargs):
        config = _selection.get()
        if config.backend == "original" or op not in config.ops:
            record(op, "original_forward")
            return original_operator(op)(*args, **kwargs)
        bound = signature.bind(*args, **kwargs)
        bound.apply_defaults()
        arguments = dict(bound.arguments)
        arguments.update(arguments.pop("kwargs", {}))
        reason = rejection_reason(op, arguments)
        if reason:
            record(op, "rejected:" + reason)
            if config.strict:
                raise RuntimeError(f"rewy_b200 {op}: {reason}")
            key = (op, reason)
            if key not in _warned:
                warnings.warn(f"rewy_b200 {op} using original: {reason}", RuntimeWarning, stacklevel=2)
                _warned.add(key)
            record(op, "fallback_forward")
            return original_operator(op)(*args, **kwargs)
        result = optimized(*args, **kwargs)
        record(op, "optimized_forward")
        return result

    call.__name__ = OPERATORS[op][1]
    call.__doc__ = optimized.__doc__
    return call
