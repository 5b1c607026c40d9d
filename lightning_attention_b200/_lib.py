"""ctypes binding of liblightning_b200.so. There is no fallback: a missing library is an error."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LIGHTNING_B200_LIB overrides the in-tree library (e.g. to try an experimental build).
LIB_PATH = os.environ.get("LIGHTNING_B200_LIB") or os.path.join(_HERE, "liblightning_b200.so")

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

_lib = None


def lib():
    """The loaded library (loads it on first use)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m lightning_attention_b200.build` "
                "(needs nvcc; there is no non-CUDA code path)"
            )
        L = ctypes.CDLL(LIB_PATH)
        vp, i, ll, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_size_t
        L.lab200_version.restype = i
        L.lab200_version.argtypes = []
        L.lab200_launch_count.restype = ll
        L.lab200_launch_count.argtypes = []
        L.lab200_la_debug_trace.restype = None
        L.lab200_la_debug_trace.argtypes = [vp, i]
        L.lab200_error_string.restype = ctypes.c_char_p
        L.lab200_error_string.argtypes = [i]
        L.lab200_la_plan_chunks.restype = i
        L.lab200_la_plan_chunks.argtypes = [i, i, i, i]
        L.lab200_la_workspace_bytes.restype = sz
        L.lab200_la_workspace_bytes.argtypes = [i, i, i, i, i]
        L.lab200_la_generic.restype = i
        L.lab200_la_generic.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, i, i, vp]
        L.lab200_la_generic_resume.restype = i
        L.lab200_la_generic_resume.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, i, vp]
        L.lab200_la_generic_resume_swapped.restype = i
        L.lab200_la_generic_resume_swapped.argtypes = [vp, vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, i, i, vp]
        L.lab200_la_combine_states.restype = i
        L.lab200_la_combine_states.argtypes = [vp, vp, vp, vp, i, i, i, i, i, i, ctypes.c_longlong, i, vp]
        L.lab200_la_decode_step.restype = i
        L.lab200_la_decode_step.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, vp]
        L.lab200_srmsnorm_gate_fwd.restype = i
        L.lab200_srmsnorm_gate_fwd.argtypes = [vp, vp, vp, vp, ll, i, f, i, vp]
        L.lab200_srmsnorm_gate_bwd.restype = i
        L.lab200_srmsnorm_gate_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ll, i, i, vp]
        L.lab200_la2_fwd.restype = i
        L.lab200_la2_fwd.argtypes = [vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, vp]
        L.lab200_la2_fwd_static.restype = i
        L.lab200_la2_fwd_static.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, vp]
        L.lab200_la2_dkdv.restype = i
        L.lab200_la2_dkdv.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, i, vp]
        L.lab200_la2_bwd_workspace_bytes.restype = sz
        L.lab200_la2_bwd_workspace_bytes.argtypes = [i, i, i, i, i, i]
        L.lab200_la2_bwd.restype = i
        L.lab200_la2_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i, i, i, i, i, i, i, vp]
        L.lab200_last_status.restype = i
        L.lab200_last_status.argtypes = []
        L.lab200_static_status.restype = i
        L.lab200_static_status.argtypes = [vp]
        L.lab200_debug_wait_expiry.restype = i
        L.lab200_debug_wait_expiry.argtypes = [vp, sz, ll, vp]
        L.lab200_read_status.restype = i
        L.lab200_read_status.argtypes = [vp, vp]
        L.lab200_srmsnorm_fwd.restype = i
        L.lab200_srmsnorm_fwd.argtypes = [vp, vp, vp, ll, i, f, i, vp]
        L.lab200_srmsnorm_bwd.restype = i
        L.lab200_srmsnorm_bwd.argtypes = [vp, vp, vp, vp, ll, i, i, vp]
        _lib = L
    return _lib


EXPORTS = [
    "lab200_version", "lab200_launch_count", "lab200_la_debug_trace", "lab200_error_string", "lab200_la_plan_chunks", "lab200_la_workspace_bytes",
    "lab200_la_generic", "lab200_la_generic_resume", "lab200_la_generic_resume_swapped", "lab200_la_combine_states", "lab200_la_decode_step", "lab200_la2_fwd", "lab200_la2_fwd_static", "lab200_la2_bwd", "lab200_la2_bwd_workspace_bytes", "lab200_la2_dkdv", "lab200_read_status", "lab200_last_status", "lab200_static_status", "lab200_debug_wait_expiry",
    "lab200_srmsnorm_fwd", "lab200_srmsnorm_bwd", "lab200_srmsnorm_gate_fwd", "lab200_srmsnorm_gate_bwd",
]


def dtype_code(dtype):
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}") from None


def check(rc, what):
    if rc != 0:
        msg = lib().lab200_error_string(rc).decode()
        raise RuntimeError(f"{what} failed with code {rc}: {msg}")


def raise_on_device_status(device):
    """Raises if a bounded wait of an earlier attention call on `device` ran out (lab200_last_status): the kernels then
    return early with an error word instead of hanging, and the outputs of that call are invalid. Non-blocking; called by
    the operators before they enqueue new work, so the report comes one call late."""
    with torch.cuda.device(device):
        rc = lib().lab200_last_status()
    if rc != 0:
        msg = lib().lab200_error_string(rc).decode()
        raise RuntimeError(f"an earlier lightning attention call on {device} failed on the device with code {rc} ({msg}); "
                           "its outputs are invalid")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("lightning_attention_b200 ops run on CUDA tensors only (no CPU path exists)")
