"""The C++ host layer (izwi_b200/host/izwi_host.hpp): its self-test program restates the reference's
projection unit tests against the C ABI.  Without a GPU only the host-side behaviour runs."""
import subprocess

import pytest


@pytest.fixture(scope="module")
def selftest():
    from izwi_b200 import build
    build.build()
    return build.build_host_selftest()


def test_host_layer_without_gpu(selftest):
    proc = subprocess.run([str(selftest), "--no-gpu"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "host_selftest: ok" in proc.stdout


def test_ctypes_structs_match_the_header(selftest):
    """The Python binding declares the ABI structs by hand: their sizes must equal what the C++
    compiler makes of include/izwi_b200.h."""
    import ctypes
    import re
    from izwi_b200 import _lib
    proc = subprocess.run([str(selftest), "--no-gpu"], capture_output=True, text=True, timeout=120)
    sizes = dict((k, int(v)) for k, v in re.findall(r"(izb_\w+)=(\d+)", proc.stdout))
    assert sizes["izb_linear_args"] == ctypes.sizeof(_lib.LinearArgs)
    assert sizes["izb_moe_args"] == ctypes.sizeof(_lib.MoeArgs)
    assert sizes["izb_gguf_tensor"] == ctypes.sizeof(_lib.GgufTensor)


@pytest.mark.gpu
def test_host_layer_on_gpu(cuda, selftest):
    proc = subprocess.run([str(selftest)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "host_selftest: ok" in proc.stdout
