"""CPU: the native libraries load and export every symbol the headers / the reference name.
No compute call is made here (there is no GPU)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_cabi_exports_every_declared_symbol(built_libs):
    header = (ROOT / "include" / "fa2_b200.h").read_text()
    declared = re.findall(r"FA2_API\s+[\w\s\*]+?\b(fa2_\w+)\s*\(", header)
    assert len(declared) >= 8
    lib = ctypes.CDLL(str(built_libs / "libfa2_b200.so"))
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/fa2_b200.h but not exported"
    from flash_attn2_b200 import _cabi

    assert set(_cabi.EXPORTS) == set(declared)


def test_cabi_struct_layout_matches_header(built_libs):
    """The ctypes mirrors must have the C structs' sizes (checked with a tiny compiled probe)."""
    import subprocess
    import tempfile

    src = '#include <stdio.h>\n#include "fa2_b200.h"\nint main(){printf("%zu %zu %zu", sizeof(fa2_fwd_args), ' \
          'sizeof(fa2_bwd_preprocess_args), sizeof(fa2_bwd_args));return 0;}'
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "p.c").write_text(src)
        subprocess.run(["gcc", f"-I{ROOT / 'include'}", str(Path(d) / "p.c"), "-o", str(Path(d) / "p")], check=True)
        sizes = [int(x) for x in subprocess.run([str(Path(d) / "p")], capture_output=True, text=True).stdout.split()]
    from flash_attn2_b200 import _cabi

    assert sizes == [ctypes.sizeof(_cabi.FwdArgs), ctypes.sizeof(_cabi.BwdPreprocessArgs), ctypes.sizeof(_cabi.BwdArgs)]


def test_tvm_ffi_library_exports_reference_operator_names(built_libs):
    from flash_attn2_b200 import _ops

    lib = ctypes.CDLL(str(built_libs / "libflash_attn2_b200.so"))
    for name in _ops.OP_NAMES:
        assert hasattr(lib, f"__tvm_ffi_{name}")
        assert hasattr(_ops.ops, name)
    assert _ops.torch_add_op_namespace_prefix("x").endswith("::x")


def test_argument_contract_without_gpu(built_libs):
    """Bad calls fail before any launch with the reference's error kinds."""
    import flash_attn2_b200 as fa

    z = torch.zeros(1, 8, 2, 64, dtype=torch.float16)
    with pytest.raises(NotImplementedError):  # CPU tensors: no CPU implementation
        fa.fwd(z, z, z)
    with pytest.raises(NotImplementedError):
        fa.cabi_ops.fwd(z, z, z)
    with pytest.raises(ValueError):  # wrong positional count
        fa.ops.fwd(z, z)
    with pytest.raises(ValueError):  # CUDA tensors required by the operator itself
        fa.ops.fwd(z, z, z, None, None, False, -1, -1, 0.0)
    with pytest.raises(TypeError):  # scalar of the wrong type
        fa.ops.fwd(z, z, z, None, None, "yes", -1, -1, 0.0)
    with pytest.raises(RuntimeError):  # exports outside the built path fail loudly
        fa.ops.rng_state()
    with pytest.raises(RuntimeError):
        fa.fwd(z.cuda() if torch.cuda.is_available() else z, z, z, p_dropout="0.1")


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flash_attn2_b200 import _cabi

    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "libfa2_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _cabi.load()
