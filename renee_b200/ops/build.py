"""In-tree build of the CUDA kernel library for sm_100a.

``python -m renee_b200.ops.build`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and links ``_kernels.so`` next to this
file.  The library exposes a plain C ABI (``extern "C"`` functions taking raw device pointers and a
stream) and is loaded with ``ctypes`` by :mod:`renee_b200.ops.cuda`; it has no dependency on the
PyTorch headers, so a full rebuild takes seconds and cross-compiles on a machine without a GPU.
(The reference builds its one extension with ``torch.utils.cpp_extension`` and no architecture
flags, setup.py:5-19.)
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "_kernels.so")
STAMP = os.path.join(HERE, "_kernels.hash")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# --use_fast_math only where the approximations are part of the design and covered by 16-bit tolerances: the
# sigmoid / softmax exponentials of the classifier and attention kernels and the GEMM epilogues.  LayerNorm
# statistics, AdamW (division, square root), the loss-scale state machine, the peer-memory reductions and the
# fp32 attention of the debugging mode are compiled with IEEE division and square root.
FAST_MATH = {"xfc.cu", "attention_mma.cu", "attention_tc.cu", "gemm.cu"}


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH + FLAGS + sorted(FAST_MATH)).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == source_hash()


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> str:
    if not force and is_current():
        return LIB
    nvcc = nvcc_path()
    obj_dir = os.path.join(HERE, "build")
    os.makedirs(obj_dir, exist_ok=True)
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        fast = ["--use_fast_math"] if os.path.basename(src) in FAST_MATH else []
        cmd = [nvcc, *ARCH, *FLAGS, *fast, *extra, "-I", CSRC, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    tmp = LIB + ".tmp"
    r = subprocess.run([nvcc, "-shared", *ARCH, "-o", tmp, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    with open(STAMP, "w") as f:
        f.write(source_hash())
    return LIB


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
