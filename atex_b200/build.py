"""Builds libnvnorms.so (the C-ABI library with every CUDA kernel) for sm_100a.

Run as ``python -m atex_b200.build`` or call :func:`build`.  Each translation
unit is compiled by its own ``nvcc`` process (the row-cached kernels are split
by dtype and direction so they build in parallel) and the objects are linked
in-tree into ``atex_b200/libnvnorms.so``.  A stamp file with a hash of the
sources and flags makes repeated calls cheap.

This takes the place of the reference's CMake flow
(atex/nv_norms/CMakeLists.txt:1-61, setup.py:21-160), which targets
sm_52...sm_90 and needs TensorFlow headers; this library needs neither.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJDIR = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libnvnorms.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-I", INCLUDE,
]


def _units():
    units = []
    for t, tname in ((0, "f32"), (1, "f16"), (2, "bf16")):
        for b, dname in ((0, "fwd"), (1, "bwd")):
            units.append((f"rows_{tname}_{dname}.o", "rows_inst.cu", [f"-DNVN_T={t}", f"-DNVN_BWD={b}"]))
        units.append((f"rows_res_{tname}.o", "rows_res_inst.cu", [f"-DNVN_T={t}"]))
    units.append(("rows_wide.o", "rows_wide.cu", []))
    units.append(("twophase.o", "twophase.cu", []))
    units.append(("colreduce.o", "colreduce.cu", []))
    units.append(("colreduce_dp.o", "colreduce_dp.cu", []))
    units.append(("nlc_onchip.o", "nlc_onchip.cu", []))
    units.append(("nlc_small.o", "nlc_small.cu", []))
    units.append(("nlc_stream.o", "nlc_stream.cu", []))
    units.append(("nvnorms_api.o", "nvnorms_api.cu", []))
    units.append(("noalloc.o", "noalloc.cu", []))
    return units


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _source_hash() -> str:
    h = hashlib.sha256()
    names = sorted(os.listdir(CSRC)) + [os.path.join(INCLUDE, "nvnorms.h")]
    for name in names:
        path = name if os.path.isabs(name) else os.path.join(CSRC, name)
        if os.path.isfile(path) and path.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link the library if it is missing or stale; returns its path."""
    os.makedirs(OBJDIR, exist_ok=True)
    stamp = os.path.join(OBJDIR, "stamp")
    digest = _source_hash()
    if not force and os.path.exists(LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return LIB
    nvcc = _nvcc()

    def compile_one(unit):
        obj, src, defs = unit
        cmd = [nvcc, *NVCC_FLAGS, *defs, "-c", os.path.join(CSRC, src), "-o", os.path.join(OBJDIR, obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src} {defs}:\n{r.stdout}\n{r.stderr}")
        return os.path.join(OBJDIR, obj)

    units = _units()
    with ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, units))
    # link beside the target and rename: a reader never sees a half-written library
    tmp = LIB + ".tmp"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
