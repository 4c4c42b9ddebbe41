"""Builds ``librllama_b200.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m rllama_b200.build [--force] [--verbose]``
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "librllama_b200.so")
CLI = os.path.join(HERE, "bin", "rllama-b200")
SOURCES = ["context.cu", "gemv.cu", "gemv_stream.cu", "attention.cu", "attention_tc.cu", "elementwise.cu", "gemm.cu", "gemm_tc.cu", "model.cu", "tp.cu", "loader.cu", "host.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "--expt-relaxed-constexpr"]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, trace=False):
    """Builds the library (and the command-line program). ``trace=True`` builds a second library,
    ``librllama_b200_trace.so``, whose prefill GEMM stamps a per-CTA timeline (``bench.py --gemm-trace`` reads it;
    select it with ``RLLAMA_B200_LIB``); the product library is left alone."""
    if trace:
        return _build_trace(verbose)
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "rllama_b200.h"))
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs)))) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose and r.stderr:
                sys.stderr.write(r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if jobs or force or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl", "-lz"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s" % (r.stdout, r.stderr))
    build_cli(force)
    return LIB


def _build_trace(verbose=False):
    obj = os.path.join(OBJ, "trace")
    os.makedirs(obj, exist_ok=True)
    lib = os.path.join(HERE, "librllama_b200_trace.so")
    objs = []
    for src in SOURCES:
        o = os.path.join(obj, src.replace(".cu", ".o"))
        objs.append(o)
        cmd = [NVCC] + FLAGS + ["-DRLB_GEMM_TRACE", "-c", os.path.join(CSRC, src), "-o", o]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    cmd = [NVCC, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl", "-lz"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (r.stdout, r.stderr))
    return lib


def build_cli(force=False):
    """The command-line program (host C++ over the C ABI): ``rllama_b200/bin/rllama-b200``."""
    src = os.path.join(HERE, "cli", "rllama_cli.cpp")
    os.makedirs(os.path.dirname(CLI), exist_ok=True)
    deps = [src, os.path.join(HERE, "cli", "inference_server.hpp"), LIB, os.path.join(HERE, "..", "include", "rllama_b200.h")]
    if force or _stale(CLI, deps):
        cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-Wall", src, "-o", CLI, "-L" + HERE, "-lrllama_b200",
               "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + os.path.join(os.path.dirname(NVCC), "..", "lib64")]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("building the command-line program failed: %s\n%s" % (r.stdout, r.stderr))
    return CLI


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
