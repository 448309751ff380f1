"""The C++ facade (ling-engine_b200/csrc/host/ling_engine.hpp): a caller written against the reference's own names,
compiled with g++ and linked to the C-ABI library.  Host logic runs anywhere; the Engine part needs the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ling-engine_b200")
EXE = os.path.join(ROOT, "tests", "cpp", "facade_test")


def build(lb):
    src = os.path.join(ROOT, "tests", "cpp", "facade_test.cpp")
    hdr = os.path.join(PKG, "csrc", "host", "ling_engine.hpp")
    if os.path.exists(EXE) and os.path.getmtime(EXE) > max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(lb.LIB_PATH)):
        return
    subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "csrc", "host"),
                    src, "-o", EXE, lb.LIB_PATH, "-Wl,-rpath," + PKG], check=True)


def test_facade_host_logic(lb):
    build(lb)
    out = subprocess.run([EXE, "host"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_facade_engine_speculate_batch(gpu, lb):
    build(lb)
    out = subprocess.run([EXE, "gpu"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
