"""Compiles and runs the CPU-only C++ checks in tests/cpp: the address / stride predicates shared by
the kernels and the host validation, and a consumer of include/managed_mem.h (the reference's C++
registry names, common/csrc/managed_memory/managed_mem.h:75-88) linked against libhfk_b200.so."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_cpp_host_checks_compile_and_pass(hfk, tmp_path):
    hfk.lib()  # built
    lib_dir = ROOT / "heterofusedkernels_b200" / "lib"
    exe = tmp_path / "host_checks"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", f"-I{ROOT / 'include'}",
           f"-I{ROOT / 'heterofusedkernels_b200' / 'csrc'}", str(ROOT / "tests" / "cpp" / "host_checks.cpp"),
           "-o", str(exe), f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}", "-lhfk_b200"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stdout + build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and "host checks ok" in run.stdout, run.stdout + run.stderr
