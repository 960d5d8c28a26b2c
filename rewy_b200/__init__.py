"""rewy_b200 — B200-native chunked delta-rule backward behind the fast-delta-rule operator surface.

Importing this package loads neither torch nor the CUDA library (like the reference,
src/fast_delta_rule/__init__.py: "No framework imports or patches on import").
Public surface (same names and meaning as the reference's, __init__.py:6-40):
    enable(backend="optimized", strict=True, ops=None, integrations=())   select the backend for this context
    disable()                                                             back to "original"
    use_backend(backend, strict=True, ops=None)                           context manager
    stats(reset=False), assert_used(ops=None, backward=True)              dispatch report / audit
    chunk_kda, chunk_gated_delta_rule, chunk_gdn2, chunk_delta_rule       the four operators
"""
from .runtime import use_backend, stats, assert_used, dispatch_report

__version__ = "0.1.0"


def enable(backend="optimized", *, strict=True, ops=None, integrations=()):
    """Select the CUDA backward for the given operators.  ``integrations`` names what else should reach them without
    source edits (``rewy_b200.integrations``): "fla" replaces flash-linear-attention's public operator aliases,
    "qwen3_5" and "gdn2" bind the two model files the reference binds.  An unknown name raises."""
    from .runtime import configure
    from . import _capi
    unknown = [name for name in integrations if name not in ("fla", "qwen3_5", "gdn2")]
    if unknown:
        raise ValueError(f"Unknown integration: {unknown[0]}")
    if backend == "optimized":
        _capi.load()  # fail here, loudly, if the CUDA library has not been built
    if integrations:
        from .integrations import INTEGRATIONS
        for name in integrations:
            INTEGRATIONS[name]()
    configure(backend, strict=strict, ops=ops)


def disable():
    from .runtime import configure
    configure("original")


def chunk_kda(*args, **kwargs):
    from .runtime import operator
    return operator("kda")(*args, **kwargs)


def chunk_gated_delta_rule(*args, **kwargs):
    from .runtime import operator
    return operator("gdn")(*args, **kwargs)


def chunk_gdn2(*args, **kwargs):
    from .runtime import operator
    return operator("gdn2")(*args, **kwargs)


def chunk_delta_rule(*args, **kwargs):
    from .runtime import operator
    return operator("delta")(*args, **kwargs)
