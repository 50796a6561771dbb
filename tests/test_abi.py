"""The C-ABI library: loads, exports every symbol the public header declares, and refuses to
compute without an sm_100 device (no CPU fallback)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "triton_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_header_declares_the_entry_points():
    syms = declared_symbols()
    for need in ("b200_matmul", "b200_attention_fwd", "b200_attention_bwd", "b200_status", "b200_last_error",
                 "b200_version"):
        assert need in syms


def test_library_exports_every_declared_symbol():
    from triton_b200 import _lib
    L = _lib.lib()
    for s in declared_symbols():
        assert hasattr(L, s), f"{s} is declared in the header but not exported"
        assert s in _lib.SIGNATURES, f"{s} has no ctypes signature in triton_b200/_lib.py"
    assert L.b200_version() >= 100


def test_header_compiles_as_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "triton_b200.h"\nint (*fp)(void) = b200_version;\nint main(void) { return fp == 0; }\n')
    import subprocess
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), "-c", str(src),
                        "-o", str(tmp_path / "t.o")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour on a machine without a GPU")
def test_no_cpu_fallback():
    from triton_b200 import _lib
    L = _lib.lib()
    rc = L.b200_matmul(None, 16, 16, 16, 4, 4, 4, 4, 1, 4, 1, 4, 1, 0, 0, 0, None, None)
    assert rc == 4, "compute entry points must fail with B200_ERR_DEVICE when no sm_100 device is current"
    assert "device" in _lib.last_error().lower()
    import triton_b200
    a = torch.zeros(4, 4, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        triton_b200.matmul(a, a)
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        triton_b200.attention(q, q, q, True, 0.5)


def test_argument_errors_do_not_need_a_device():
    from triton_b200 import _lib
    L = _lib.lib()
    assert L.b200_matmul(None, 16, 16, 16, -1, 4, 4, 4, 1, 4, 1, 4, 1, 0, 0, 0, None, None) == 1
    assert L.b200_matmul(None, 16, 16, 16, 4, 4, 4, 4, 1, 4, 1, 4, 1, 7, 0, 0, None, None) == 1
    s4 = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    assert L.b200_attention_fwd(None, 16, 16, 16, 16, 16, 1, 1, 128, 48, s4, s4, s4, s4, 0.5, 1, 0) == 2  # head dim
    assert L.b200_attention_fwd(None, 16, 16, 16, 16, 16, 1, 1, 128, 64, s4, s4, s4, s4, -1.0, 1, 0) == 1  # sm_scale
    assert L.b200_attention_bwd(None, *([16] * 10), 1, 1, 100, 64, *([s4] * 8), 0.5, 1, 0) == 1  # N % 128
