"""Builds and runs the C++ ports of the reference's tests (tests/cpp/mirror_tests.cpp),
which use the C++ host face include/saragossa_kv.hpp over the C ABI."""
import os
import subprocess

import pytest

from oracle import sgo
from saragossa_b200 import _ffi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "mirror_tests.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "_build", "mirror_tests")


def _build():
    _ffi.lib()
    sgo.build()
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    deps = [SRC, os.path.join(ROOT, "include", "saragossa_kv.hpp"), os.path.join(ROOT, "include", "sgk.h")]
    if os.path.exists(EXE) and all(os.path.getmtime(d) < os.path.getmtime(EXE) for d in deps):
        return EXE
    lib_dir = os.path.dirname(_ffi.LIB_PATH)
    oracle_dir = os.path.dirname(sgo._SO)
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-o", EXE, SRC, f"-L{lib_dir}", "-lsgk", f"-L{oracle_dir}",
                           "-lsgo", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{oracle_dir}", "-pthread"])
    return EXE


def test_cpp_mirror_cpu_cases():
    out = subprocess.run([_build(), "cpu"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_cpp_mirror_gpu_cases():
    out = subprocess.run([_build(), "gpu"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
