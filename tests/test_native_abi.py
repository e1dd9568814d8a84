"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU, exports
every function include/wfb200.h declares, the ctypes table covers the same set, and the
calls that need no device behave (argument errors, missing-device errors)."""
import ctypes
import os
import re

import pytest

from warpforge_b200 import _native as N

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = open(os.path.join(ROOT, "include", "wfb200.h")).read()


def declared_functions():
    code = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(wf_[a-z0-9_]+)\s*\(", code)))


def test_library_builds_and_loads():
    if not os.path.exists(N.LIB_PATH):
        from warpforge_b200 import build

        build.build()
    assert N.load().wf_version() >= 100


def test_header_library_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 30
    assert sorted(N.SIGNATURES) == names
    lib = ctypes.CDLL(N.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/wfb200.h but not exported"


def test_every_declaration_cites_the_reference():
    """Each group of entry points says which reference interface it replaces."""
    for token in ("CudaRuntime.java", "CudaContext.java", "GpuBackend.java", "Dequantizer.java", "DotGeneralKernel.java",
                  "CollectiveApi.java", "GGUF.java"):
        assert token in HEADER


def test_status_names():
    lib = N.load()
    assert lib.wf_error_string(0) == b"WF_OK"
    assert lib.wf_error_string(N.WF_ERR_SHAPE) == b"WF_ERR_SHAPE"
    assert lib.wf_error_string(N.WF_ERR_UNSUPPORTED_TYPE) == b"WF_ERR_UNSUPPORTED_TYPE"
    assert lib.wf_error_string(1002) == b"cudaErrorMemoryAllocation"
    assert lib.wf_error_string(N.WF_ERR_RECORDING) == b"WF_ERR_RECORDING"
    assert lib.wf_error_string(N.WF_ERR_IN_USE) == b"WF_ERR_IN_USE"


def test_invalid_handles_and_arguments_without_a_device():
    lib = N.load()
    assert lib.wf_destroy(0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_destroy(0x1234) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_stream_sync(77, 0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_qlinear(77, 1, None, 1, 0, 1, None, 0, 0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_program_step_host(77, 1, 0, None, None, None, None, 0, 0, 0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_dot_f32(77, 1, 1, 1, 1, 1, 1, 0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_gelu(77, 1, 1, 1, 0) == N.WF_ERR_INVALID_HANDLE
    assert lib.wf_init(0, None) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_device_count(None) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_comm_get_unique_id(None) == N.WF_ERR_INVALID_ARGUMENT


def test_no_device_means_no_context_and_no_fallback():
    """Without a CUDA device the library refuses to create a context; nothing computes on the CPU."""
    n = ctypes.c_int(-1)
    rc = N.load().wf_device_count(ctypes.byref(n))
    if rc == N.WF_OK and n.value > 0:
        pytest.skip("a CUDA device is present")
    h = ctypes.c_int64(1)
    assert N.load().wf_init(0, ctypes.byref(h)) == N.WF_ERR_NO_DEVICE and h.value == 0
    from warpforge_b200.backend import NvidiaBackend

    with pytest.raises(N.WfError) as e:
        NvidiaBackend(0)
    assert e.value.status == N.WF_ERR_NO_DEVICE


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "warpforge_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "quant.py" and "oracle" not in text, f"{f} mentions the oracle"
