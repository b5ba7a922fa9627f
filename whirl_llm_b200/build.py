"""Builds libwhirl_b200.so (the CUDA kernels and the C ABI) in-tree with nvcc for sm_100a.

    python -m whirl_llm_b200.build            # build if sources are newer than the library
    python -m whirl_llm_b200.build --force
    python -m whirl_llm_b200.build -v         # print registers / spills / shared memory per kernel
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libwhirl_b200.so")
OBJ = os.path.join(HERE, "build")
SOURCES = ["api.cu", "host_api.cu", "rowscan.cu", "select_generic.cu", "single_pass.cu", "merge.cu", "spec_accept.cu", "rng.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-cudart", "shared"]


def _newer_than_lib(lib: str) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "whirl_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), out: str | None = None) -> str:
    """Compiles every source to an object (in parallel) and links the shared library.  `defines` ("NAME=VALUE" strings)
    and `out` build a variant of the library beside the default one."""
    lib = out or LIB
    if not force and not defines and not _newer_than_lib(lib):
        return lib
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    tag = os.path.splitext(os.path.basename(lib))[0]
    objdir = os.path.join(OBJ, tag)
    os.makedirs(objdir, exist_ok=True)
    dflags = [f"-D{d}" for d in defines]

    def compile_one(src: str):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *dflags, "-Xptxas", "-v" if verbose else "-warn-spills", "-c", "-o", obj, os.path.join(CSRC, src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, res

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        done = list(ex.map(compile_one, SOURCES))
    for src, _, res in done:
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
        if verbose:
            print(f"==== {src}\n{res.stderr}")
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "shared", "-o", lib] + [o for _, o, _ in done]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
