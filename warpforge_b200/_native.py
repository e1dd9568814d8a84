"""ctypes binding of libwfb200.so -- the stand-in for the Panama FFM binding class a
WarpForge backend would carry (the reference binds libcuda the same way,
warpforge-backend-nvidia/src/main/java/io/surfworks/warpforge/backend/nvidia/cuda/CudaRuntime.java:64-162:
one downcall handle per symbol, int status returned, `checkError` turning non-zero into
an exception).

The library is never built at import time and there is no fallback: a missing
``libwfb200.so`` raises ImportError-like ``NativeLibraryMissing`` with the build command.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwfb200.so")

c_int, c_i64, c_vp, c_f32 = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_float
c_char_p = ctypes.c_char_p
P = ctypes.POINTER

# name -> (restype, argtypes); must list every function declared in include/wfb200.h
SIGNATURES = {
    "wf_version": (c_int, []),
    "wf_device_count": (c_int, [P(c_int)]),
    "wf_init": (c_int, [c_int, P(c_i64)]),
    "wf_destroy": (c_int, [c_i64]),
    "wf_device_info": (c_int, [c_i64, P(c_int), P(c_int), P(c_int), P(c_i64), P(c_i64)]),
    "wf_stream_create": (c_int, [c_i64, P(c_i64)]),
    "wf_stream_destroy": (c_int, [c_i64, c_i64]),
    "wf_stream_sync": (c_int, [c_i64, c_i64]),
    "wf_malloc": (c_int, [c_i64, c_i64, P(c_i64)]),
    "wf_free": (c_int, [c_i64, c_i64]),
    "wf_host_alloc": (c_int, [c_i64, c_i64, P(c_vp)]),
    "wf_host_free": (c_int, [c_i64, c_vp]),
    "wf_memcpy_h2d": (c_int, [c_i64, c_i64, c_vp, c_i64, c_i64, c_int]),
    "wf_memcpy_d2h": (c_int, [c_i64, c_vp, c_i64, c_i64, c_i64, c_int]),
    "wf_weight_upload": (c_int, [c_i64, c_int, c_vp, c_i64, c_i64, c_int, c_int, P(c_i64)]),
    "wf_set_exact_exp": (c_int, [c_i64, c_int]),
    "wf_rms_norm": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f32, c_i64]),
    "wf_layer_norm": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_f32, c_i64]),
    "wf_softmax": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_silu": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_dot_f32": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_gelu": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_swiglu": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_add": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_embedding": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_gguf_open": (c_int, [c_char_p, P(c_i64), c_char_p, c_i64]),
    "wf_gguf_close": (c_int, [c_i64]),
    "wf_gguf_info": (c_int, [c_i64, P(c_int), P(c_i64), P(c_i64), P(c_i64), P(c_int), P(c_i64)]),
    "wf_gguf_tensor_name": (c_int, [c_i64, c_i64, c_char_p, c_i64]),
    "wf_gguf_tensor_info": (c_int, [c_i64, c_char_p, P(c_int), P(c_int), P(c_i64), P(c_i64), P(c_i64)]),
    "wf_gguf_tensor_data": (c_int, [c_i64, c_char_p, P(c_vp), P(c_i64)]),
    "wf_gguf_metadata": (c_int, [c_i64, c_i64, c_char_p, c_i64, c_char_p, c_i64]),
    "wf_gguf_upload": (c_int, [c_i64, c_i64, c_char_p, c_int, c_int, c_int, P(c_i64)]),
    "wf_weight_free": (c_int, [c_i64, c_i64]),
    "wf_weight_info": (c_int, [c_i64, c_i64, P(c_int), P(c_i64), P(c_i64), P(c_i64), P(c_i64)]),
    "wf_dequant_rows": (c_int, [c_i64, c_i64, c_i64, c_i64, c_vp]),
    "wf_qlinear": (c_int, [c_i64, c_i64, c_vp, c_int, c_int, c_i64, c_vp, c_int, c_i64]),
    "wf_qlinear_noalloc": (c_int, [c_i64, c_i64, c_i64, c_int, c_i64, c_i64, c_i64]),
    "wf_qlinear_allgather": (c_int, [c_i64, c_i64, c_i64, c_vp, c_int, c_i64, c_vp, c_i64]),
    "wf_comm_get_unique_id": (c_int, [c_vp]),
    "wf_comm_init": (c_int, [c_i64, c_vp, c_int, c_int, P(c_i64)]),
    "wf_comm_destroy": (c_int, [c_i64, c_i64]),
    "wf_comm_info": (c_int, [c_i64, c_i64, c_vp, c_vp, c_vp]),
    "wf_allgather": (c_int, [c_i64, c_i64, c_i64, c_i64, c_i64, c_i64]),
    "wf_program_create": (c_int, [c_i64, c_int, P(c_i64), P(c_i64), P(c_i64), P(c_int), c_i64, c_int, c_int, P(c_i64), P(c_i64)]),
    "wf_plan_several_tokens": (c_int, [c_int, c_i64, c_i64, c_int, c_int, c_int, P(c_int), P(c_int), P(c_int), P(c_int), P(c_i64)]),
    "wf_program_step_host": (c_int, [c_i64, c_i64, c_int, P(c_vp), P(c_i64), P(c_i64), c_vp, c_i64, c_i64, c_i64]),
    "wf_program_create_fused": (c_int, [c_i64, c_int, P(c_i64), P(c_i64), P(c_i64), P(c_int), P(c_int), P(c_i64), P(ctypes.c_float),
                                        P(c_i64), c_i64, c_int, c_int, P(c_i64), P(c_i64)]),
    "wf_program_run": (c_int, [c_i64, c_i64, c_i64]),
    "wf_program_destroy": (c_int, [c_i64, c_i64]),
    "wf_program_read_timing": (c_int, [c_i64, c_i64, P(c_i64), c_i64]),
    "wf_ipc_export": (c_int, [c_i64, c_i64, c_vp]),
    "wf_ipc_import": (c_int, [c_i64, c_vp, P(c_i64)]),
    "wf_ipc_close": (c_int, [c_i64, c_i64]),
    "wf_graph_begin": (c_int, [c_i64, c_i64]),
    "wf_graph_end": (c_int, [c_i64, c_i64, P(c_i64)]),
    "wf_graph_launch": (c_int, [c_i64, c_i64, c_i64]),
    "wf_graph_destroy": (c_int, [c_i64, c_i64]),
    "wf_error_string": (ctypes.c_char_p, [c_int]),
    "wf_last_error": (c_int, [c_i64, ctypes.c_char_p, c_i64]),
    "wf_event_create": (c_int, [c_i64, P(c_i64)]),
    "wf_event_destroy": (c_int, [c_i64, c_i64]),
    "wf_event_record": (c_int, [c_i64, c_i64, c_i64]),
    "wf_event_elapsed_ms": (c_int, [c_i64, c_i64, c_i64, P(c_f32)]),
    "wf_set_salt": (c_int, [c_i64, c_int]),
    "wf_read_timing": (c_int, [c_i64, P(c_i64), c_i64]),
    "wf_launch_count": (c_int, [c_i64, P(c_i64)]),
}

WF_OK = 0
WF_ERR_INVALID_ARGUMENT, WF_ERR_INVALID_HANDLE, WF_ERR_UNSUPPORTED_TYPE, WF_ERR_SHAPE = -1, -2, -3, -4
WF_ERR_SHARD, WF_ERR_BUSY, WF_ERR_NO_DEVICE, WF_ERR_NOT_SM100 = -5, -6, -7, -8
WF_ERR_NCCL_UNAVAILABLE, WF_ERR_DEVICE_WAIT, WF_ERR_TOO_LARGE, WF_ERR_GGUF = -9, -10, -11, -12
WF_ERR_INDEX = -13
WF_ERR_RECORDING, WF_ERR_IN_USE = -14, -15
WF_X_BF16, WF_X_F32, WF_X_RMSNORM_F32, WF_X_SWIGLU_F32 = 0, 1, 2, 3
WF_Q4_0_ORDER_REFERENCE, WF_Q4_0_ORDER_GGML = 0, 1
WF_DTYPE_F32, WF_DTYPE_BF16 = 0, 1
WF_OP_NEW_X, WF_OP_DEPENDS = 1, 2


class NativeLibraryMissing(RuntimeError):
    pass


class WfError(RuntimeError):
    """Non-zero status from the native library (CudaException's role, CudaRuntime.java:615-633)."""

    def __init__(self, op: str, status: int, name: str, detail: str = ""):
        self.op, self.status, self.name, self.detail = op, status, name, detail
        super().__init__(f"{op} failed: {name} ({status})" + (f": {detail}" if detail else ""))


_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NativeLibraryMissing(
                f"{LIB_PATH} is missing; build it with `python -m warpforge_b200.build` (needs nvcc). "
                "There is no CPU fallback for this library.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def error_name(status: int) -> str:
    return load().wf_error_string(status).decode()


def check(op: str, status: int, ctx: int = 0) -> None:
    if status == WF_OK:
        return
    detail = ""
    if ctx:
        buf = ctypes.create_string_buffer(512)
        if load().wf_last_error(ctx, buf, 512) == WF_OK:
            detail = buf.value.decode(errors="replace")
    raise WfError(op, status, error_name(status), detail)
