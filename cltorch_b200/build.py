"""Builds cltorch_b200/lib/libthb200.so for sm_100a with nvcc and g++.

Run as `python -m cltorch_b200.build` (add `-v` for the ptxas resource report,
`-f` to rebuild everything). Compilation units build in parallel; a unit is
rebuilt when any source or header is newer than its object file.

Flags that matter for results: no fast-math and `-fmad=false`, so that
`a + b * c` rounds twice exactly as the CPU oracle does.
"""
from __future__ import annotations

import concurrent.futures
import os
import shlex
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
BUILD = PKG / "build"
LIBDIR = PKG / "lib"
LIB = LIBDIR / "libthb200.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

APPLY_PARTS = 8

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "--expt-relaxed-constexpr",
    f"-I{ROOT / 'include'}", f"-I{CSRC}",
]
CXX_FLAGS = [
    "-O2", "-std=c++17", "-fPIC", "-Wall", f"-I{ROOT / 'include'}", f"-I{CSRC}",
    f"-I{CUDA_HOME / 'include'}",
]


def _embed_kernel_source() -> Path:
    """Writes the text NVRTC compiles (math policy, apply kernels, TMA helpers, TMA tile kernel) as a C++ raw string."""
    BUILD.mkdir(parents=True, exist_ok=True)
    out = BUILD / "apply_kernels_src.inc"
    text = "".join((CSRC / "kernels" / n).read_text() for n in ("math_policy.cuh", "apply_kernels.cuh", "tma_pipeline.cuh", "apply_tma_kernels.cuh"))
    text = text.replace("#pragma once", "")
    body = 'R"THBSRC(' + text + ')THBSRC"\n'
    if not out.exists() or out.read_text() != body:
        out.write_text(body)
    return out


def _units():
    """(object name, source, extra flags, compiler) for every compilation unit."""
    units = []
    for k in range(APPLY_PARTS):
        units.append((f"thb_apply_builtin_{k}.o", CSRC / "abi" / "thb_apply_builtin.cu",
                      [f"-DTHB_PART={k}", f"-DTHB_NPARTS={APPLY_PARTS}"], "nvcc"))
    for src in sorted((CSRC / "abi").glob("*.cu")):
        if src.name != "thb_apply_builtin.cu":
            units.append((src.stem + ".o", src, [], "nvcc"))
    for src in sorted((CSRC / "abi").glob("*.cpp")) + sorted((CSRC / "thcl").glob("*.cpp")):
        units.append((src.stem + ".o", src, [], "cxx"))
    return units


def _newest_header_mtime() -> float:
    paths = list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.def")) \
        + list((ROOT / "include").glob("*.h")) + [BUILD / "apply_kernels_src.inc", Path(__file__)]
    return max(p.stat().st_mtime for p in paths if p.exists())


def _compile(unit, verbose: bool) -> str:
    obj, src, extra, comp = unit
    if comp == "nvcc":
        cmd = [NVCC, *NVCC_FLAGS, *extra, f"-I{BUILD}", "-c", str(src), "-o", str(BUILD / obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = ["g++", *CXX_FLAGS, *extra, f"-I{BUILD}", "-c", str(src), "-o", str(BUILD / obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"build failed: {shlex.join(cmd)}\n{res.stdout}\n{res.stderr}")
    return res.stderr if verbose else ""


def build(verbose: bool = False, force: bool = False) -> Path:
    _embed_kernel_source()
    LIBDIR.mkdir(parents=True, exist_ok=True)
    hdr_time = _newest_header_mtime()
    units = _units()
    todo = []
    for u in units:
        obj = BUILD / u[0]
        if force or not obj.exists() or obj.stat().st_mtime < max(hdr_time, u[1].stat().st_mtime):
            todo.append(u)
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
            for log in pool.map(lambda u: _compile(u, verbose), todo):
                if log:
                    sys.stderr.write(log)
    objs = [str(BUILD / u[0]) for u in units]
    if todo or not LIB.exists():
        # cudart is linked statically; NVRTC and NCCL-free: libnvrtc comes from the CUDA toolkit.
        cmd = [NVCC, "-shared", "-o", str(LIB), *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static", f"-L{CUDA_HOME / 'lib64'}", "-lnvrtc",
               "-Xlinker", f"-rpath={CUDA_HOME / 'lib64'}", "-Xlinker", "--no-undefined"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed: {shlex.join(cmd)}\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
