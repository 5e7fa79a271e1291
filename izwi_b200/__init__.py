"""izwi_b200: B200 (sm_100a) kernels for the izwi-core matrix-multiplication
hot path behind a C ABI (include/izwi_b200.h), plus the host-side mirror of the
reference's projection types used by the tests."""
from ._lib import LIB_PATH, IzbError, exported_symbols, lib  # noqa: F401

__all__ = ["LIB_PATH", "IzbError", "exported_symbols", "lib"]
