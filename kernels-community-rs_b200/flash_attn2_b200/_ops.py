"""Loads the tvm-ffi operator library (the file kernel-builder generates for the reference
package): `ops.<name>` are the `__tvm_ffi_<name>` symbols of libflash_attn2_b200.so."""
from pathlib import Path

import tvm_ffi

_LIB = Path(__file__).resolve().parent.parent / "lib" / "libflash_attn2_b200.so"
if not _LIB.exists():
    raise ImportError(
        f"{_LIB} is missing: build it with `python kernels-community-rs_b200/build.py` "
        "(the operators have no fallback implementation)")

ops = tvm_ffi.load_module(str(_LIB))

# Names the reference's tvm-ffi exports carry (flash-attn2-rs/src/host/**): checked by the CPU tests.
OP_NAMES = (
    "fwd", "fwd_lse", "bwd_preprocess", "bwd_dq", "bwd_dkv", "bwd_all",
    "varlen_fwd_explicit", "varlen_bwd_explicit",
    "varlen_fwd_descriptor", "rng_state", "cache_merge_explicit", "cache_update_explicit",
    "cache_validate_layouts",
)


def torch_add_op_namespace_prefix(name: str) -> str:
    """Qualified torch custom-op name, as kernel-builder's generated helper returns it."""
    return f"_flash_attn2_b200::{name}"
