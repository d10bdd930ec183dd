"""B200-native KV-cache data path with the operator surface of HeteroFusedKernels.

* ``heterofusedkernels_b200.capi``    — ctypes view of the C ABI (``include/hfk_b200.h``)
* ``heterofusedkernels_b200.memory``  — NUMA-pinned allocation / host registration
  (the reference's ``heterofusedkernels.memory``, common/csrc/pybind.cpp:7-11)
* ``heterofusedkernels_b200.load_ops()`` — registers ``torch.ops.pcie_through.*``
  (the reference's ``import pcie_through``, pcieThrough/pcie_through/_load.py:8-11)

The drop-in import names ``pcie_through`` and ``heterofusedkernels`` at the
repository root are aliases of these.  Everything computes on the GPU through
``lib/libhfk_b200.so``; a missing library raises, it is never replaced by a CPU path.
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
from pathlib import Path

from . import capi

__all__ = ["capi", "load_ops", "memory", "ops_library_path"]

_LIB_DIR = Path(__file__).resolve().parent / "lib"
_ops_loaded = False


def ops_library_path() -> Path:
    return _LIB_DIR / "libpcie_through.so"


def load_ops() -> None:
    """dlopen the torch operator library so that its TORCH_LIBRARY blocks run."""
    global _ops_loaded
    if _ops_loaded:
        return
    import torch

    path = ops_library_path()
    if not path.exists():
        raise ImportError(f"{path} is missing: run `python -m heterofusedkernels_b200.build`")
    capi.lib()  # the registry singleton lives in libhfk_b200.so; load it first
    torch.ops.load_library(str(path))
    _ops_loaded = True


def _load_memory_module():
    import torch  # noqa: F401  (the extension links libtorch_python)

    suffix = importlib.machinery.EXTENSION_SUFFIXES[0]
    path = _LIB_DIR / ("memory" + suffix)
    if not path.exists():
        raise ImportError(f"{path} is missing: run `python -m heterofusedkernels_b200.build`")
    capi.lib()
    spec = importlib.util.spec_from_file_location("memory", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def __getattr__(name: str):
    if name == "memory":
        mod = _load_memory_module()
        globals()["memory"] = mod
        return mod
    raise AttributeError(name)
