"""CPU-side checks of the operator layer's C ABI (include/paddock_exec.h): the library loads,
exports every declared symbol, and refuses to come up without a CUDA device (there is no host path)."""
import ctypes as C
import os
import re

import pytest

from paddock_b200 import executor as X

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "paddock_exec.h")


def test_library_exports_every_declared_symbol():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(pdx_\w+)\s*\(", text)))
    assert len(names) >= 28 and "pdx_open" in names and "pdx_nvf4_gemm_f4" in names
    lib = C.CDLL(X.lib_path())
    for n in names:
        assert hasattr(lib, n), f"{n} declared in paddock_exec.h but not exported"


def test_plane_info_struct_matches_the_header():
    # kind, ggml_type, in, out, bytes, three pointers, scale2, layout
    assert C.sizeof(X.PlaneInfo) == 4 + 4 + 8 + 8 + 8 + 3 * 8 + 4 + 4


def test_executor_needs_a_device_or_a_pack():
    import torch
    if torch.cuda.is_available():
        with pytest.raises(X.GpuError) as e:
            X.GpuExecutor(pack_path="/nonexistent/libnothing.so")
        assert e.value.kind == "Pack"
    else:
        with pytest.raises(X.GpuError) as e:
            X.GpuExecutor()
        assert e.value.kind == "Driver"
