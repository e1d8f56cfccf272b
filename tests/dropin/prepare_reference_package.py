"""Puts the reference's own Python package on top of this repository's operator library.

  python tests/dropin/prepare_reference_package.py <path to the reference checkout>

Copies, unmodified, `flash-attn2-rs/tvm-ffi-ext/flash_attn2_rs/` (the package kernel-builder ships)
and `flash-attn2-rs/tests/test_fwd.py` + `test_gold.py` from the reference checkout into
`baseline/_ref/` (ignored by git; not product source) and adds the two files kernel-builder would
generate or the Hub would provide:

  baseline/_ref/flash_attn2_rs/_ops.py   `ops` = the tvm-ffi module of lib/libflash_attn2_b200.so and
                                         `torch_add_op_namespace_prefix`, the two names the package imports
  baseline/_ref/kernels/__init__.py      a stand-in for the Hub loader: `get_kernel(...)` returns the
                                         local package instead of downloading a build (and, for the
                                         "gold" kernel of test_gold.py, the flash_attn wheel of the image)

tests/test_dropin_gpu.py then runs the reference's test files against the sm_100a library.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
DEST = ROOT / "baseline" / "_ref"

OPS_PY = '''"""Stand-in for the `_ops.py` kernel-builder generates: binds the package to the sm_100a library."""
from pathlib import Path

import tvm_ffi

_LIB = Path(__file__).resolve().parents[3] / "kernels-community-rs_b200" / "lib" / "libflash_attn2_b200.so"
if not _LIB.exists():
    raise ImportError(f"{_LIB} is missing: run `python kernels-community-rs_b200/build.py`")
ops = tvm_ffi.load_module(str(_LIB))


def torch_add_op_namespace_prefix(name: str) -> str:
    return f"_flash_attn2_b200_dropin::{name}"
'''

KERNELS_PY = '''"""Stand-in for the Hugging Face `kernels` loader: returns the local copy of the reference package."""
import importlib
import types


def _gold():
    """The "gold" kernel of test_gold.py (kernels-community/flash-attn2): the flash_attn wheel of this image,
    which wraps the same FA2 CUDA kernels. Its Python module has the flash_attn_func family; the raw operators
    the Hub package also exports (fwd, bwd, varlen_fwd, varlen_bwd: keyword forms of the extension's positional
    entry points) are added here."""
    iface = importlib.import_module("flash_attn.flash_attn_interface")
    ext = importlib.import_module("flash_attn_2_cuda")
    gold = types.ModuleType("flash_attn2_gold")
    gold.__dict__.update({k: v for k, v in vars(iface).items() if not k.startswith("__")})

    def scale_of(q, softmax_scale):
        return q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale

    def fwd(q, k, v, out=None, alibi_slopes=None, p_dropout=0.0, softmax_scale=None, is_causal=False,
            window_size_left=-1, window_size_right=-1, softcap=0.0, return_softmax=False, gen=None):
        return ext.fwd(q, k, v, out, alibi_slopes, p_dropout, scale_of(q, softmax_scale), is_causal,
                       window_size_left, window_size_right, softcap, return_softmax, gen)

    def bwd(dout, q, k, v, out, softmax_lse, dq=None, dk=None, dv=None, alibi_slopes=None, p_dropout=0.0,
            softmax_scale=None, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
            deterministic=False, gen=None, rng_state=None):
        return ext.bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, alibi_slopes, p_dropout,
                       scale_of(q, softmax_scale), is_causal, window_size_left, window_size_right, softcap,
                       deterministic, gen, rng_state)

    def varlen_fwd(q, k, v, cu_seqlens_q, cu_seqlens_k, out=None, seqused_k=None, leftpad_k=None, block_table=None,
                   alibi_slopes=None, max_seqlen_q=0, max_seqlen_k=0, p_dropout=0.0, softmax_scale=None,
                   zero_tensors=False, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
                   return_softmax=False, gen=None):
        return ext.varlen_fwd(q, k, v, out, cu_seqlens_q, cu_seqlens_k, seqused_k, leftpad_k, block_table,
                              alibi_slopes, max_seqlen_q, max_seqlen_k, p_dropout, scale_of(q, softmax_scale),
                              zero_tensors, is_causal, window_size_left, window_size_right, softcap, return_softmax, gen)

    def varlen_bwd(dout, q, k, v, out, softmax_lse, cu_seqlens_q, cu_seqlens_k, dq=None, dk=None, dv=None,
                   alibi_slopes=None, max_seqlen_q=0, max_seqlen_k=0, p_dropout=0.0, softmax_scale=None,
                   zero_tensors=False, is_causal=False, window_size_left=-1, window_size_right=-1, softcap=0.0,
                   deterministic=False, gen=None, rng_state=None):
        return ext.varlen_bwd(dout, q, k, v, out, softmax_lse, dq, dk, dv, cu_seqlens_q, cu_seqlens_k, alibi_slopes,
                              max_seqlen_q, max_seqlen_k, p_dropout, scale_of(q, softmax_scale), zero_tensors,
                              is_causal, window_size_left, window_size_right, softcap, deterministic, gen, rng_state)

    gold.fwd, gold.bwd, gold.varlen_fwd, gold.varlen_bwd = fwd, bwd, varlen_fwd, varlen_bwd
    return gold


def get_kernel(repo_id, version=None, revision=None, **_):
    if "flash-attn2-rs" in repo_id:
        return importlib.import_module("flash_attn2_rs")
    if repo_id.endswith("/flash-attn2"):
        return _gold()
    raise ValueError(f"no local stand-in for {repo_id}")
'''


def main(argv) -> int:
    if len(argv) != 2:
        print(__doc__)
        return 2
    src = Path(argv[1]) / "flash-attn2-rs"
    pkg = src / "tvm-ffi-ext" / "flash_attn2_rs"
    if not pkg.is_dir():
        print(f"{pkg} not found")
        return 1
    if DEST.exists():
        shutil.rmtree(DEST)
    (DEST / "tests").mkdir(parents=True)
    shutil.copytree(pkg, DEST / "flash_attn2_rs")
    for name in ("test_fwd.py", "test_gold.py"):
        shutil.copy(src / "tests" / name, DEST / "tests" / name)
    (DEST / "flash_attn2_rs" / "_ops.py").write_text(OPS_PY)
    (DEST / "kernels").mkdir()
    (DEST / "kernels" / "__init__.py").write_text(KERNELS_PY)
    print(f"reference package prepared under {DEST}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
