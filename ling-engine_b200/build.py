"""Builds libling_b200.so (the C-ABI library of the verify step) in-tree with nvcc for sm_100a.

    python ling-engine_b200/build.py          # or: from the package, build()

The library is self-contained CUDA C++ (no PyTorch, no Triton); it links the CUDA runtime statically and takes the
one driver entry point it needs (cuTensorMapEncodeTiled) at run time, so it builds on a machine without a GPU.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libling_b200.so")
SOURCES = ["gemm.cu", "nvfp4.cu", "nvfp4_abi.cu", "chain.cu", "kernels.cu", "attention_tc.cu", "context.cu", "kernel_abi.cu", "noalloc.cu", "draft_head.cu", "draft_sparse.cu", "gdn_chunk.cu", "host_logic.cpp", "prefix_store.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=default"]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def build(force=False, verbose=False):
    """Compiles every source to an object (in parallel) and links the shared library. Returns its path."""
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "ling_b200.h"))
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(objdir, src + ".o")
        if force or _newer([s] + headers, o):
            extra = ["-Xptxas", "-v"] if verbose else []
            jobs.append((src, [NVCC] + FLAGS + extra + ["-c", s, "-o", o]))
    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (name, r.stdout, r.stderr))
        return name, r.stderr
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as ex:
        for name, err in ex.map(run, jobs):
            if verbose and err:
                sys.stderr.write(err)
    objs = [os.path.join(objdir, s + ".o") for s in SOURCES]
    if force or jobs or _newer(objs, OUT):
        r = subprocess.run([NVCC, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                            # keep the statically linked C++/CUDA runtimes private to this library: a host process
                            # (Python with other native extensions) may carry different copies of the same symbols
                            "-Xlinker", "-Bsymbolic", "-Xlinker", "--exclude-libs,ALL"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    build_serve(force)
    return OUT


SERVE = os.path.join(HERE, "ling_serve_headless")


def build_serve(force=False):
    """The headless serving driver (csrc/host/serve_headless.cpp): plain C++ over the C ABI, linked to the library beside it."""
    src = os.path.join(CSRC, "host", "serve_headless.cpp")
    deps = [src, OUT] + [os.path.join(CSRC, "host", h) for h in ("ling_engine.hpp", "ling_scheduler.hpp")]
    if not (force or _newer(deps, SERVE)):
        return SERVE
    r = subprocess.run([os.environ.get("CXX", "g++"), "-std=c++20", "-O2", "-Wall", "-I", os.path.join(HERE, "..", "include"),
                        "-I", os.path.join(CSRC, "host"), src, "-o", SERVE, OUT, "-Wl,-rpath,$ORIGIN"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("serve_headless failed to build:\n%s\n%s" % (r.stdout, r.stderr))
    return SERVE


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
