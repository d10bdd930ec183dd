"""In-tree build of the native libraries (no cmake, no JIT cache).

Three artefacts land in ``heterofusedkernels_b200/lib``:

* ``libhfk_b200.so``   — CUDA kernels for sm_100a + the C ABI of ``include/hfk_b200.h``
  (nvcc, static cudart, no torch dependency);
* ``libpcie_through.so`` — the torch operator library ``pcie_through`` (g++), the
  counterpart of the reference's ``pcie_through/lib/libpcie_through.so``
  (pcieThrough/pcie_through/_load.py:8-11);
* ``memory.<abi>.so``  — the pybind11 module behind ``heterofusedkernels.memory``
  (common/csrc/pybind.cpp:7-11).

The reference builds ``common`` first and ``pcie_through`` against it
(pcieThrough/pyproject.toml:8); the same order holds here because both shims link
``libhfk_b200.so``, which owns the registry singleton.

Run ``python -m heterofusedkernels_b200.build`` to build everything.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
INCLUDE = ROOT / "include"

CAPI_SOURCES = ["hfk_capi.cu", "host_registry.cpp"]
CAPI_DEPS = ["common.cuh", "kv_swap.cuh", "paged_gather.cuh", "row_gather.cuh", "block_transfer.cuh", "relayout_swap.cuh",
             "kv_migrate.cuh", "ptr_check.h", "host_util.h"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> Path:
    for key in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(key):
            return Path(os.environ[key])
    return Path("/usr/local/cuda")


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(shlex.quote(c) for c in cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, flush=True)


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build_capi(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """nvcc: kernels + C ABI -> libhfk_b200.so (sm_100a only)."""
    LIB.mkdir(exist_ok=True)
    out = LIB / "libhfk_b200.so"
    deps = [CSRC / s for s in CAPI_SOURCES + CAPI_DEPS] + [INCLUDE / "hfk_b200.h", Path(__file__)]
    if not force and not _stale(out, deps):
        return out
    nvcc = str(_cuda_home() / "bin" / "nvcc")
    cmd = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-shared", "-Xcompiler",
           "-fPIC,-Wall", "-cudart", "static"]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in CAPI_SOURCES] + ["-o", str(out), "-lpthread", "-ldl", "-lrt"]
    _run(cmd, verbose or ptxas_info)
    return out


def _torch_flags() -> tuple[list[str], list[str]]:
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{_cuda_home() / 'include'}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-Wno-deprecated-declarations", *inc]
    tlib = Path(torch.__file__).parent / "lib"
    ldflags = [f"-L{tlib}", f"-Wl,-rpath,{tlib}", f"-L{LIB}", "-Wl,-rpath,$ORIGIN", "-lhfk_b200",
               "-lc10", "-ltorch_cpu", "-ltorch"]
    return cflags, ldflags


def build_torch_ops(force: bool = False, verbose: bool = False) -> Path:
    """g++: TORCH_LIBRARY(pcie_through) shim -> libpcie_through.so."""
    out = LIB / "libpcie_through.so"
    src = CSRC / "torch_ops.cpp"
    if not force and not _stale(out, [src, INCLUDE / "hfk_b200.h", LIB / "libhfk_b200.so"]):
        return out
    cflags, ldflags = _torch_flags()
    cmd = ["g++", "-shared", *cflags, str(src), "-o", str(out), *ldflags, "-lc10_cuda", "-ltorch_cuda"]
    _run(cmd, verbose)
    return out


def memory_module_path() -> Path:
    return LIB / ("memory" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_memory_module(force: bool = False, verbose: bool = False) -> Path:
    """g++: pybind11 module `memory` (heterofusedkernels.memory)."""
    out = memory_module_path()
    src = CSRC / "memory_pybind.cpp"
    if not force and not _stale(out, [src, INCLUDE / "hfk_b200.h", LIB / "libhfk_b200.so"]):
        return out
    cflags, ldflags = _torch_flags()
    py_inc = sysconfig.get_paths()["include"]
    cmd = ["g++", "-shared", *cflags, f"-I{py_inc}", "-DTORCH_EXTENSION_NAME=memory",
           "-DTORCH_API_INCLUDE_EXTENSION_H", str(src), "-o", str(out), *ldflags, "-ltorch_python"]
    _run(cmd, verbose)
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {
        "capi": build_capi(force, verbose),
        "torch_ops": build_torch_ops(force, verbose),
        "memory": build_memory_module(force, verbose),
    }


if __name__ == "__main__":
    force = "--force" in sys.argv
    if "--ptxas" in sys.argv:
        build_capi(force=True, verbose=True, ptxas_info=True)
    for name, path in build_all(force=force, verbose=True).items():
        print(f"{name}: {path}")
