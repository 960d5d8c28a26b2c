"""Make flash-linear-attention's public operator names resolve to this package's operators.

Counterpart of the reference's FLA integration (src/fast_delta_rule/integrations/fla.py:7-35).  The reference
registers ``chunk_kda`` and ``chunk_gated_delta_rule`` in the backend registry of the FLA revision it pins
(``fla.backends``) and patches the public aliases of the other two families.  Installed FLA releases differ in
whether they have that registry, so this module uses the mechanism that exists in all of them: it replaces the
public aliases ``fla.ops.<family>.<name>`` and ``fla.ops.<family>.chunk.<name>`` (and the same name inside FLA
layer modules that are already imported) by the dispatching entry of ``rewy_b200.runtime.operator``.  The
original functions are captured first, so the "original" backend and non-strict forwarding still reach FLA's
own implementation.  Families the installed FLA does not have are skipped and reported.

Model bindings (the reference's src/fast_delta_rule/integrations/models.py:5-15): ``bind_qwen3_5`` points the chunked
gated delta rule of transformers' Qwen3.5 modelling file at the ``gdn`` operator, ``bind_gdn2`` does the same for the
``chunk_gdn2`` of the GDN2 authors' ``lit_gpt.gdn2`` layer.  Both change exactly one attribute of one module and
refuse a module that does not have it; ``uninstall()`` puts every patched attribute back.
"""
import importlib
import sys

_LAYERS = {"kda": ("kda",), "gdn": ("gated_deltanet", "gated_delta_net"), "gdn2": ("gdn2",), "delta": ("delta_net",)}
_patched = []       # (module, attribute, previous value)
_installed = None   # result of the last install()


def install():
    """Patch FLA's public aliases; returns {"patched": [...ops], "skipped": {op: reason}}.  Idempotent."""
    global _installed
    if _installed is not None:
        return _installed
    try:
        importlib.import_module("fla")
    except Exception as exc:
        raise RuntimeError(f"rewy_b200 integration 'fla': flash-linear-attention is not importable: {exc}") from exc
    from .runtime import OPERATORS, operator, original_operator
    originals, skipped = {}, {}
    for op in OPERATORS:  # capture every original before any alias changes
        try:
            originals[op] = original_operator(op)
        except RuntimeError as exc:
            skipped[op] = str(exc)
    for op in originals:
        family, name = OPERATORS[op]
        entry = operator(op)
        targets = [f"fla.ops.{family}", f"fla.ops.{family}.chunk"] + [f"fla.layers.{m}" for m in _LAYERS[op]]
        for path in targets:
            module = sys.modules.get(path) if path.startswith("fla.layers.") else importlib.import_module(path)
            if module is not None and hasattr(module, name):
                _patched.append((module, name, getattr(module, name)))
                setattr(module, name, entry)
    _installed = {"patched": sorted(originals), "skipped": skipped}
    return _installed


def _bind(module_path, attribute, op, what):
    try:
        module = importlib.import_module(module_path)
    except Exception as exc:
        raise RuntimeError(f"rewy_b200 integration {what!r}: {module_path} is not importable: {exc}") from exc
    if not hasattr(module, attribute):
        raise RuntimeError(f"rewy_b200 integration {what!r}: {module_path} has no {attribute}")
    from .runtime import operator
    entry = operator(op)
    if getattr(module, attribute) is not entry:
        _patched.append((module, attribute, getattr(module, attribute)))
        setattr(module, attribute, entry)


def bind_qwen3_5():
    """transformers' Qwen3.5: layers built after this call run the ``gdn`` operator for their chunked delta rule.  The
    modelling file takes FLA's ``chunk_gated_delta_rule`` when flash-linear-attention is importable and its own
    ``torch_chunk_gated_delta_rule`` otherwise; whichever it would pick is pointed at the operator."""
    path = "transformers.models.qwen3_5.modeling_qwen3_5"
    _bind(path, "torch_chunk_gated_delta_rule", "gdn", "qwen3_5")
    if getattr(importlib.import_module(path), "chunk_gated_delta_rule", None) is not None:
        from .runtime import original_operator
        try:
            original_operator("gdn")  # capture FLA's own function before its alias in the modelling file changes
        except RuntimeError:
            pass
        _bind(path, "chunk_gated_delta_rule", "gdn", "qwen3_5")


def bind_gdn2():
    """The GDN2 authors' layer (their project must be importable as ``lit_gpt``)."""
    _bind("lit_gpt.gdn2", "chunk_gdn2", "gdn2", "gdn2")


INTEGRATIONS = {"fla": install, "qwen3_5": bind_qwen3_5, "gdn2": bind_gdn2}


def uninstall():
    """Put every patched alias back."""
    global _installed
    while _patched:
        module, name, previous = _patched.pop()
        setattr(module, name, previous)
    _installed = None
