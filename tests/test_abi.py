"""The C ABI without a GPU: the library loads, exports every symbol the header
declares, and its host-only entry points behave."""
import ctypes as C
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from izwi_b200 import build
    build.build()
    import izwi_b200
    return izwi_b200.lib()


def declared_symbols():
    text = (ROOT / "include" / "izwi_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(izb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/izwi_b200.h but not exported"


def test_binding_table_matches_header():
    from izwi_b200 import exported_symbols
    assert exported_symbols() == declared_symbols()


def test_status_strings(lib):
    assert lib.izb_status_string(0) == b"ok"
    assert b"wait" in lib.izb_status_string(-4)
    assert lib.izb_version() >= 100


def test_quantized_storage_bytes(lib):
    out = C.c_size_t()
    assert lib.izb_quantized_storage_bytes(1, 3, 32, C.byref(out)) == 0 and out.value == 102
    assert lib.izb_quantized_storage_bytes(2, 4096, 1024, C.byref(out)) == 0 and out.value == 4096 * 1024 // 256 * 144
    assert lib.izb_quantized_storage_bytes(2, 3, 100, C.byref(out)) == -1   # not a multiple of the block size
    assert lib.izb_quantized_storage_bytes(7, 1, 32, C.byref(out)) == -1    # unknown format
    assert lib.izb_quantized_storage_bytes(1, 2**40, 2**40, C.byref(out)) == -1  # overflow
    assert lib.izb_quantized_storage_bytes(1, 1, 32, None) == -1


def test_null_context_is_rejected_not_dereferenced(lib):
    assert lib.izb_ctx_destroy(None) == -1
    assert lib.izb_ctx_check(None, None) == -1
    assert lib.izb_linear(None, None, None) == -1
    assert lib.izb_silu_mul(None, None, None, None, None, 1, 1, 1, 1, 1) == -1
    assert lib.izb_dequantize(None, None, 1, None, 32, 1, None) == -1
    assert lib.izb_linear_group_plan_bytes(0) == 0
    assert lib.izb_linear_group_plan_bytes(3) > 0


def test_ctx_create_without_device_reports_no_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    assert lib.izb_ctx_create(0, C.byref(h)) == -5
    assert not h.value
    assert lib.izb_ctx_create(-1, C.byref(h)) == -1


def test_kernel_gate_follows_the_reference_rule():
    """IZWI_B200_KERNELS: unset = on; set = on only for 1 / true / yes / on (kernels/mod.rs:46-57).  Read once per
    process, so every value is tried in a process of its own."""
    import os
    import subprocess
    import sys
    code = "import izwi_b200; print(int(izwi_b200.use_b200_kernels()))"
    for value, want in ((None, "1"), ("1", "1"), (" TRUE ", "1"), ("on", "1"), ("Yes", "1"), ("0", "0"), ("off", "0"),
                        ("", "0"), ("2", "0")):
        env = {k: v for k, v in os.environ.items() if k != "IZWI_B200_KERNELS"}
        if value is not None:
            env["IZWI_B200_KERNELS"] = value
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=str(ROOT), timeout=120)
        assert out.stdout.strip() == want, (value, out.stdout, out.stderr)
