"""In-tree build of the CUDA library (sm_100a only).

    python -m orin_llm_b200.build          # -> orin_llm_b200/lib/liborin_attn_b200.so

nvcc cross-compiles without a GPU.  The CUDA runtime is linked statically so that the library
does not depend on which libcudart the host process has loaded.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "liborin_attn_b200.so")
SOURCES = ["capi.cu", "decode.cu", "prefill_mma.cu", "prefill_tc.cu", "rope_kv.cu"]
HEADERS = ["common.cuh", "attn_internal.h", os.path.join("..", "..", "include", "orin_attn_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--threads", "0",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


HOST_LIB = os.path.join(LIBDIR, "liborin_attn_host.so")
HOST_SRC = os.path.join(HERE, "host", "kernels.cpp")


def build_host(force=False):
    """The C++ wrappers with the reference's names (host/kernels.h), linked against the C-ABI library."""
    build(force=False)
    deps = [HOST_SRC, os.path.join(HERE, "host", "kernels.h"), LIB]
    if not force and os.path.exists(HOST_LIB) and all(os.path.getmtime(d) <= os.path.getmtime(HOST_LIB) for d in deps):
        return HOST_LIB
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fno-exceptions", "-fno-rtti", "-o", HOST_LIB, HOST_SRC,
           "-L" + LIBDIR, "-lorin_attn_b200", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("g++ failed:\n" + r.stdout + r.stderr)
    return HOST_LIB


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not needs_build():
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-shared", "-o", LIB]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_host(force="--force" in sys.argv))
