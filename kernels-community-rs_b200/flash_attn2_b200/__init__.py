"""B200 (sm_100a) FlashAttention-2 behind the flash-attn2-rs operator surface.

`cabi_ops` talks to the C ABI (include/fa2_b200.h) through ctypes; `interface` (imported lazily,
it needs tvm_ffi) goes through the tvm-ffi operator symbols exactly like the reference package.
"""
from . import cabi_ops  # noqa: F401

_INTERFACE_NAMES = (
    "fwd_explicit", "fwd", "bwd", "varlen_fwd", "varlen_bwd", "flash_attn_func", "flash_attn_varlen_func",
)


def __getattr__(name):
    if name in _INTERFACE_NAMES or name in ("interface", "ops"):
        import importlib

        interface = importlib.import_module(__name__ + ".interface")
        if name == "interface":
            return interface
        if name == "ops":
            return interface.ops
        return getattr(interface, name)
    raise AttributeError(name)
