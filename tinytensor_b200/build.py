"""Builds libttb.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: ``python -m tinytensor_b200.build [--force] [--verbose]``.

Each ``csrc/*.cu`` is compiled to an object next to the sources (``csrc/_obj``)
and the objects are linked into ``tinytensor_b200/libttb.so``.  Objects are
rebuilt only when a source or header is newer.  nvcc cross-compiles sm_100a
without a GPU, so this runs anywhere the toolkit is installed.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "_obj"
LIB = PKG / "libttb.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]

# Sources that make up the library.  tt_runner_shim.cu is NOT part of it: it is the
# tinytensor-side adapter and needs the tinytensor headers to compile.
SOURCES = [
    "ttb_api.cu",
    "tma_desc.cu",
    "gemm_simt.cu",
    "gemm_f32_tcgen05.cu",
    "gemm_f64_dmma.cu",
    "gemm_i32_tcgen05.cu",
    "conv2d.cu",
    "device_memory.cu",
]


# Host-only sources (no device code), compiled by the host compiler: C++20, and the floating-point
# contraction default of a release build, which the restated input generator must share with the
# reference library it is pinned against.
HOST_SOURCES = ["generator.cpp"]
HOST_FLAGS = ["-std=c++20", "-O3", "-DNDEBUG", "-march=x86-64-v3", "-fPIC", "-fvisibility=hidden", "-pthread"]


def _cxx() -> str:
    exe = os.environ.get("CXX") or shutil.which("g++")
    if not exe:
        raise RuntimeError("g++ not found; a C++20 host compiler is required to build libttb.so")
    return exe


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libttb.so")
    return exe


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(src: Path, verbose: bool) -> tuple[str, str]:
    obj = OBJ / (src.stem + ".o")
    if src.name in HOST_SOURCES:
        cmd = [_cxx(), *HOST_FLAGS, "-c", str(src), "-o", str(obj)]
    else:
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compiling {src.name} failed:\n{r.stdout}\n{r.stderr}")
    return src.name, r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    srcs = [CSRC / s for s in SOURCES + HOST_SOURCES if (CSRC / s).exists()]
    hdr_t = _newest_header()
    todo = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_t):
            todo.append(s)
    logs = {}
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for name, log in ex.map(lambda s: _compile(s, verbose), todo):
                logs[name] = log
    objs = [OBJ / (s.stem + ".o") for s in srcs]
    if todo or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fPIC", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        for name, log in logs.items():
            sys.stderr.write(f"==== {name}\n{log}\n")
    return LIB


def compile_check_shim(reference_root: Path, export_header_dir: Path) -> list[Path]:
    """Compiles the tinytensor-side adapters (csrc/tt_runner_shim.cu for matmul,
    csrc/tt_conv_shim.cu for conv2d) to objects against tinytensor's headers, the way
    tinytensor's own CUDA backend is compiled (C++20, --expt-relaxed-constexpr, TT_CUDA).
    `export_header_dir` holds a tt/export.h (the file tinytensor's CMake generates)."""
    OBJ.mkdir(exist_ok=True)
    objs = []
    for name in ("tt_runner_shim", "tt_conv_shim"):
        obj = OBJ / f"{name}.o"
        cmd = [
            _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++20", "--expt-relaxed-constexpr",
            "-DTT_CUDA", "-DTINYTENSOR_STATIC_DEFINE", "-O2", "-Xcompiler", "-fPIC",
            f"-I{reference_root}/include", f"-I{reference_root}/tinytensor", f"-I{export_header_dir}",
            "-c", str(CSRC / f"{name}.cu"), "-o", str(obj),
        ]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{name}.cu does not compile against {reference_root}:\n{r.stdout}\n{r.stderr}")
        objs.append(obj)
    return objs


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
