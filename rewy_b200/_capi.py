"""ctypes binding of librewy_b200.so (the C ABI declared in include/rewy_b200.h).

There is no fallback: if the shared library is missing or a call returns a non-zero status a
RuntimeError is raised.  Tensors are passed as raw device pointers; the launches go to torch's
current CUDA stream.
"""
import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_size_t, c_void_p
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "librewy_b200.so"

DELTA, GDN, KDA, GDN2 = 0, 1, 2, 3
FAMILY_ID = {"delta": DELTA, "gdn": GDN, "kda": KDA, "gdn2": GDN2}
RECOMPUTE, SAVED = 0, 1
OUT_BF16, OUT_F32 = 0, 1

EXPORTS = (
    "rewy_kda_bwd", "rewy_gdn2_bwd", "rewy_gdn_bwd", "rewy_delta_bwd", "rewy_bwd_workspace_bytes",
    "rewy_stage_prepare", "rewy_stage_fwd_scan", "rewy_stage_bwd_scan", "rewy_stage_chunk_adjoint",
    "rewy_stage_timing_enable", "rewy_stage_timing_read", "rewy_selftest_tensor_core", "rewy_selftest_bounded_wait",
    "rewy_device_status", "rewy_wide_chunk_count", "rewy_set_chunk_variant", "rewy_set_scan_variant",
    "rewy_set_prepare_variant", "rewy_set_scan_overlap",
    "rewy_stage_chunk_adjoint_static", "rewy_static_device_status",
    "rewy_l2norm_fwd", "rewy_l2norm_bwd", "rewy_beta_sigmoid_fwd", "rewy_beta_sigmoid_bwd", "rewy_gate_cumsum_fwd",
    "rewy_gate_act_bwd", "rewy_chunk_fwd", "rewy_scalar_gate_cumsum_fwd", "rewy_set_forward_variant",
    "rewy_last_error", "rewy_version", "rewy_kernel_launch_count",
)


class BwdArgs(ctypes.Structure):
    _fields_ = [
        ("family", c_int32), ("policy", c_int32), ("B", c_int32), ("T", c_int32), ("H", c_int32),
        ("out_dtype", c_int32), ("intra_passes", c_int32), ("state_v_first", c_int32), ("scale", c_float),
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("g", c_void_p), ("beta", c_void_p),
        ("b_gate", c_void_p), ("w_gate", c_void_p), ("Aqk", c_void_p), ("Akk", c_void_p), ("h0", c_void_p),
        ("d_o", c_void_p), ("dht", c_void_p),
        ("w", c_void_p), ("qg", c_void_p), ("kg", c_void_p), ("v_new", c_void_p), ("h", c_void_p),
        ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p), ("dg", c_void_p), ("dbeta", c_void_p),
        ("db_gate", c_void_p), ("dw_gate", c_void_p), ("dh0", c_void_p),
        ("cu_seqlens", c_void_p), ("num_seqs", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class FwdArgs(ctypes.Structure):
    _fields_ = [("family", c_int32), ("B", c_int32), ("T", c_int32), ("H", c_int32), ("state_v_first", c_int32),
                ("scale", c_float)] + [(n, c_void_p) for n in (
                    "q", "k", "v", "g", "beta", "b_gate", "w_gate", "h0", "o", "final_state", "Aqk", "Akk", "w", "u", "qg",
                    "kg", "v_new", "h", "ctrl", "cu_seqlens")] + [("num_seqs", c_int32)]


class StageBuffers(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("w", "u", "qg", "kg", "v_new", "h", "Aqk", "dh", "dR", "dR_lo", "ctrl")]


_lib = None


def library_path():
    return LIB_PATH


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m rewy_b200.build` (needs nvcc). "
            "rewy_b200 has no CPU or PyTorch fallback for the backward.")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name in ("rewy_kda_bwd", "rewy_gdn2_bwd", "rewy_gdn_bwd", "rewy_delta_bwd"):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(BwdArgs), c_void_p]
        fn.restype = c_int
    for name in ("rewy_stage_prepare", "rewy_stage_fwd_scan", "rewy_stage_bwd_scan", "rewy_stage_chunk_adjoint",
                 "rewy_stage_chunk_adjoint_static"):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.POINTER(BwdArgs), ctypes.POINTER(StageBuffers), c_void_p]
        fn.restype = c_int
    lib.rewy_bwd_workspace_bytes.argtypes = [c_int32, c_int32, c_int32, c_int32, c_int32]
    lib.rewy_bwd_workspace_bytes.restype = c_size_t
    lib.rewy_stage_timing_enable.argtypes = [c_int]
    lib.rewy_stage_timing_enable.restype = c_int
    lib.rewy_stage_timing_read.argtypes = [ctypes.POINTER(c_float), ctypes.POINTER(c_int)]
    lib.rewy_stage_timing_read.restype = c_int
    lib.rewy_selftest_tensor_core.argtypes = [c_void_p] * 9
    lib.rewy_selftest_tensor_core.restype = c_int
    i64 = ctypes.c_int64
    lib.rewy_chunk_fwd.argtypes = [ctypes.POINTER(FwdArgs), c_void_p]
    lib.rewy_chunk_fwd.restype = c_int
    lib.rewy_scalar_gate_cumsum_fwd.argtypes = [c_void_p, c_int, c_void_p, c_int32, c_int32, c_int32, c_void_p]
    lib.rewy_scalar_gate_cumsum_fwd.restype = c_int
    lib.rewy_l2norm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, i64, c_float, c_void_p]
    lib.rewy_l2norm_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, i64, c_void_p]
    lib.rewy_beta_sigmoid_fwd.argtypes = [c_void_p, c_int, c_void_p, c_void_p, i64, c_float, c_void_p]
    lib.rewy_beta_sigmoid_bwd.argtypes = [c_void_p, c_int, c_void_p, c_void_p, i64, c_float, c_void_p]
    lib.rewy_gate_cumsum_fwd.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32,
                                         c_void_p]
    lib.rewy_gate_act_bwd.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32,
                                      c_int32, c_int32, c_void_p]
    for name in ("rewy_l2norm_fwd", "rewy_l2norm_bwd", "rewy_beta_sigmoid_fwd", "rewy_beta_sigmoid_bwd",
                 "rewy_gate_cumsum_fwd", "rewy_gate_act_bwd"):
        getattr(lib, name).restype = c_int
    lib.rewy_selftest_bounded_wait.argtypes = [c_void_p, c_void_p, ctypes.c_uint32, c_int, c_void_p]
    lib.rewy_selftest_bounded_wait.restype = c_int
    lib.rewy_device_status.argtypes = [c_void_p, c_void_p]
    lib.rewy_device_status.restype = c_int
    lib.rewy_wide_chunk_count.argtypes = [c_void_p, c_void_p]
    lib.rewy_wide_chunk_count.restype = c_int
    lib.rewy_static_device_status.argtypes = [c_void_p]
    lib.rewy_static_device_status.restype = c_int
    lib.rewy_set_scan_variant.argtypes = [c_int]
    lib.rewy_set_scan_variant.restype = c_int
    lib.rewy_set_forward_variant.argtypes = [c_int]
    lib.rewy_set_forward_variant.restype = c_int
    lib.rewy_set_scan_overlap.argtypes = [c_int]
    lib.rewy_set_scan_overlap.restype = c_int
    lib.rewy_set_prepare_variant.argtypes = [c_int]
    lib.rewy_set_prepare_variant.restype = c_int
    lib.rewy_set_chunk_variant.argtypes = [c_int]
    lib.rewy_set_chunk_variant.restype = c_int
    lib.rewy_last_error.restype = c_char_p
    lib.rewy_version.restype = c_char_p
    lib.rewy_kernel_launch_count.restype = c_int
    _lib = lib
    return lib


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def check(status, what):
    if status != 0:
        msg = load().rewy_last_error().decode()
        raise RuntimeError(f"rewy_b200 {what} failed with status {status}: {msg}")


def current_stream(device):
    import torch
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def workspace_bytes(family, policy, B, T, H):
    return int(load().rewy_bwd_workspace_bytes(family, policy, B, T, H))


STAGE_NAMES = ("prepare", "fwd_scan", "bwd_scan", "chunk_adjoint")


def stage_timing_enable(on=True):
    check(load().rewy_stage_timing_enable(1 if on else 0), "rewy_stage_timing_enable")


def stage_timing_read():
    """Returns ({stage: total ms}, calls) for the whole-family calls recorded since enabling."""
    ms = (c_float * 4)()
    calls = c_int(0)
    check(load().rewy_stage_timing_read(ms, ctypes.byref(calls)), "rewy_stage_timing_read")
    return {n: float(ms[i]) for i, n in enumerate(STAGE_NAMES)}, int(calls.value)


def launch_count():
    return int(load().rewy_kernel_launch_count())
