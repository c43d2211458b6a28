"""Builds libq4b200.so in place with nvcc for sm_100a (no JIT cache, no torch)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBRARY = os.path.join(HERE, "libq4b200.so")
SOURCES = ["q4b_api.cu", "q4b_pack.cu", "q4b_gemm.cu", "q4b_comm.cu", "q4b_probe.cu", "q4b_decode.cu", "q4b_image.cu", "q4b_layer.cu"]
HEADERS = ["q4b_common.cuh", "q4b_kernels.h", os.path.join("..", "..", "include", "q4b200.h")]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libq4b200.so cannot be built")
    return found


def _sources() -> list[str]:
    return [name for name in SOURCES if os.path.exists(os.path.join(CSRC, name))]


def stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    inputs = [os.path.join(CSRC, name) for name in _sources() + HEADERS]
    return any(os.path.exists(path) and os.path.getmtime(path) > built for path in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu of the package into libq4b200.so; returns its path."""
    if not force and not stale():
        return LIBRARY
    nvcc = _nvcc()
    objects = []
    flags = list(FLAGS)
    procs = []
    for name in _sources():
        obj = os.path.join(CSRC, name.replace(".cu", ".o"))
        command = [nvcc, *flags, "-c", os.path.join(CSRC, name), "-o", obj]
        if verbose:
            command.insert(1, "-Xptxas=-v")
        procs.append((name, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
        objects.append(obj)
    for name, proc in procs:
        output = proc.communicate()[0].decode()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {name}:\n{output}")
        if verbose:
            print(output)
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIBRARY,
                           *objects, "-lcudart", "-ldl"])
    return LIBRARY


if __name__ == "__main__":
    print(build(force=True, verbose=False))
