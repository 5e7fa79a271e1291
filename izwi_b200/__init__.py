"""izwi_b200: B200 (sm_100a) kernels for the izwi-core matrix-multiplication
hot path behind a C ABI (include/izwi_b200.h), plus the host-side mirror of the
reference's projection types used by the tests."""
from ._lib import LIB_PATH, IzbError, exported_symbols, lib  # noqa: F401



def use_b200_kernels() -> bool:
    """The IZWI_B200_KERNELS gate (default on), read once per process by the library with the rule of
    the reference's `use_fused_kernels` (kernels/mod.rs:46-57)."""
    return bool(lib().izb_kernels_enabled())


__all__ = ["LIB_PATH", "IzbError", "exported_symbols", "lib", "use_b200_kernels"]
