"""The C++ facade (ling-engine_b200/csrc/host/ling_engine.hpp): a caller written against the reference's own names,
compiled with g++ and linked to the C-ABI library.  Host logic runs anywhere; the Engine part needs the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ling-engine_b200")
EXE = os.path.join(ROOT, "tests", "cpp", "facade_test")
SCHED = os.path.join(ROOT, "tests", "cpp", "scheduler_test")
PREFIX = os.path.join(ROOT, "tests", "cpp", "prefix_test")


def build(lb, exe=EXE):
    src = exe + ".cpp"
    hdrs = [os.path.join(PKG, "csrc", "host", h) for h in ("ling_engine.hpp", "ling_scheduler.hpp")]
    if os.path.exists(exe) and os.path.getmtime(exe) > max([os.path.getmtime(f) for f in [src, lb.LIB_PATH] + hdrs]):
        return
    subprocess.run(["g++", "-std=c++20", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(PKG, "csrc", "host"),
                    src, "-o", exe, lb.LIB_PATH, "-Wl,-rpath," + PKG], check=True)


def test_facade_host_logic(lb):
    build(lb)
    out = subprocess.run([EXE, "host"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_facade_engine_speculate_batch(gpu, lb):
    build(lb)
    out = subprocess.run([EXE, "gpu"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr


def test_scheduler_loop_on_a_host_engine(lb):
    """The headless scheduler (admission, turns, batching, pairing, page pressure, last resort) against a host-only engine."""
    build(lb, SCHED)
    out = subprocess.run([SCHED, "host"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_scheduler_continuous_batching_equals_serving_alone(gpu, lb):
    """Six requests through four sessions under the scheduler's continuous batching give, token for token, what each gives alone."""
    build(lb, SCHED)
    out = subprocess.run([SCHED, "gpu"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr


def test_prefix_store_classes_on_the_host(lb):
    """PrefixKvTree and ArenaAlloc as C++ classes over a KvPool: page references and the copy of a page two prompts share."""
    build(lb, PREFIX)
    out = subprocess.run([PREFIX, "host"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr


@pytest.mark.gpu
def test_prefix_store_resume_equals_prefill_from_nothing(gpu, lb):
    """A prompt that resumes from the prefix KV store (pages by reference, state restored, shared page copied before the write)
    reaches the same state bits and the same tokens as the prompt prefilled from nothing on an engine without a store."""
    build(lb, PREFIX)
    out = subprocess.run([PREFIX, "gpu"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
