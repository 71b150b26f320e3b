"""Build libvlr.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libvlr.so")
LIB_TRACE = os.path.join(HERE, "libvlr_trace.so")     # debugging build with the stage trace compiled in
SOURCES = ["api.cu", "bgmv.cu", "bgmv_decode.cu", "pack.cu", "atmm_sm100.cu", "step.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libvlr.so cannot be built")


def _sources():
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(os.path.dirname(HERE), "include", "vlr.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """trace=True (or VLR_TRACE=1 in the environment) compiles the clock64 stage trace
    into the tensor-core kernels and exports vlr_debug_set_trace: a debugging build, not
    the one that ships or is benchmarked."""
    trace = trace or os.environ.get("VLR_TRACE") == "1"
    lib = LIB_TRACE if trace else LIB
    if not force and not needs_build(lib):
        return lib
    nvcc = _nvcc()
    objs = []
    procs = []
    bdir = os.path.join(HERE, "build", "trace" if trace else "")
    os.makedirs(bdir, exist_ok=True)
    for src in _sources():
        obj = os.path.join(bdir, os.path.basename(src) + ".o")
        cmd = ([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + (["-DVLR_TRACE"] if trace else [])
               + ["-c", src, "-o", obj])
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objs.append(obj)
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            print(out.decode())
        if p.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cmd = [nvcc, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
