"""GPU: the reference's own Python package and its own test files, unmodified, on top of this
repository's operator library.

`tests/dropin/prepare_reference_package.py` copies flash-attn2-rs/tvm-ffi-ext/flash_attn2_rs and
flash-attn2-rs/tests/test_{fwd,gold}.py into baseline/_ref/ (not tracked) next to a two-name `_ops.py`
and a stand-in for the Hub loader. These tests run the copied test files in a child pytest:

  * tests/test_fwd.py completely (18 parity cases against the crate's naive fp32 attention and
    3 rejection cases);
  * of tests/test_gold.py the forward cases that need only `flash_attn_func` of the gold kernel
    (the flash_attn wheel of the image stands in for kernels-community/flash-attn2), every head dim
    of its parity list (8 ... 256).
"""
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _run(test_file, *extra):
    if not (REF / "flash_attn2_rs" / "__init__.py").exists():
        pytest.fail("baseline/_ref is missing: run tests/dropin/prepare_reference_package.py <reference checkout>")
    env = dict(os.environ, PYTHONPATH=str(REF))
    cmd = [sys.executable, "-m", "pytest", str(REF / "tests" / test_file), "-q", "-p", "no:cacheprovider",
           "-W", "ignore::pytest.PytestUnknownMarkWarning", *extra]
    proc = subprocess.run(cmd, cwd=str(REF), env=env, capture_output=True, text=True, timeout=900)
    tail = (proc.stdout + proc.stderr)[-3000:]
    return proc.returncode, tail


def _counts(tail):
    m = re.search(r"(\d+) passed", tail)
    f = re.search(r"(\d+) failed", tail)
    return (int(m.group(1)) if m else 0), (int(f.group(1)) if f else 0)


def test_reference_package_runs_its_forward_tests_unmodified():
    rc, tail = _run("test_fwd.py")
    passed, failed = _counts(tail)
    assert rc == 0 and failed == 0 and passed == 21, tail


def test_reference_gold_forward_cases_against_the_flash_attn_wheel():
    rc, tail = _run("test_gold.py", "-k",
                    "test_forward_parity or test_strided_views or test_rejects_head_size")
    passed, failed = _counts(tail)
    assert rc == 0 and failed == 0 and passed >= 60, tail
