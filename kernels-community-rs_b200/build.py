"""Builds the native libraries in-tree with nvcc / g++ for sm_100a.

  lib/libfa2_b200.so            CUDA kernels + the C ABI declared in include/fa2_b200.h
  lib/libflash_attn2_b200.so    tvm-ffi operator symbols (__tvm_ffi_fwd, ...) on top of the C ABI

Run as `python build.py` or call build(); a library is rebuilt only when a source is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "lib"
INCLUDE = HERE.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-DFA2_BUILD",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]

KERNEL_SOURCES = ["fwd_sm100.cu", "fwd_wide_sm100.cu", "bwd_sm100.cu", "bwd_wide_sm100.cu", "bwd_aux.cu", "fa2_host.cu"]


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} (exit {proc.returncode})")


def build_kernels(verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libfa2_b200.so"
    srcs = [CSRC / s for s in KERNEL_SOURCES if (CSRC / s).exists()]
    deps = srcs + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [INCLUDE / "fa2_b200.h"]
    if _newer(out, deps):
        objs, jobs = [], []
        for s in srcs:
            o = LIB / (s.stem + ".o")
            if _newer(o, deps):
                cmd = ["nvcc", *NVCC_FLAGS, "-c", str(s), "-o", str(o)]
                if verbose:
                    cmd.insert(1, "-Xptxas=-v")
                jobs.append(cmd)
            objs.append(str(o))
        # one nvcc per translation unit, side by side: every kernel file holds 16 instantiations
        if jobs:
            with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
                list(pool.map(_run, jobs))
        _run(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(out), *objs,
              "-Xcompiler", "-fPIC"])
    return out


def build_tvm_ffi() -> Path | None:
    src = CSRC / "tvm_ffi_ops.cc"
    if not src.exists():
        return None
    import tvm_ffi  # the operator ABI headers and libtvm_ffi.so come with the Python package

    root = Path(tvm_ffi.__file__).resolve().parent
    inc = root / "include"
    libdir = root / "lib"
    out = LIB / "libflash_attn2_b200.so"
    deps = [src, INCLUDE / "fa2_b200.h"]
    if _newer(out, deps) or _newer(out, [LIB / "libfa2_b200.so"]):
        dlpack = [p for p in [inc, root / "include" / "dlpack", root / "3rdparty" / "dlpack" / "include"] if p.exists()]
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
               *[f"-I{p}" for p in dlpack], f"-I{INCLUDE}", "-I/usr/local/cuda/include",
               str(src), "-o", str(out),
               f"-L{LIB}", "-lfa2_b200", f"-L{libdir}", "-ltvm_ffi",
               "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{libdir}"]
        _run(cmd)
    return out


def build(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_tvm_ffi()


if __name__ == "__main__":
    build(verbose="-v" in sys.argv)
    print("built:", *sorted(p.name for p in LIB.glob("*.so")))
