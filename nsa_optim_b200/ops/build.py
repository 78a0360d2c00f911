"""Builds the native library ``libnsa_b200.so`` from ``ops/csrc/*.cu`` for sm_100a, in-tree.

    python -m nsa_optim_b200.ops.build [--force] [--verbose] [--debug]

Each ``.cu`` file is one translation unit (no relocatable device code is needed: kernels
receive every pointer they use as an argument).  Objects go to ``ops/_build/``; the shared
library is written beside this file so that it is found by ``ops/native.py``.  nvcc
cross-compiles without a GPU.  ``--debug`` builds ``libnsa_b200_debug.so`` with
``-DNSA_DEBUG_BOUNDS``: indices that kernels read from tensors (token ids, labels, selected block
numbers) are checked where they are used and a bad one is recorded in the status block
(code 302) while the kernel continues with the clamped value; set ``NSA_B200_LIB`` to that file to
run a program on it.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libnsa_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found (set NVCC or add /usr/local/cuda/bin to PATH)")
    return cand


def sources() -> List[str]:
    return sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))


def _newest_header() -> float:
    return max((os.path.getmtime(os.path.join(SRC, f)) for f in os.listdir(SRC)
                if f.endswith((".cuh", ".h"))), default=0.0)


def _compile(nvcc: str, name: str, extra: List[str], verbose: bool, obj_dir: str = OBJ) -> str:
    src = os.path.join(SRC, name)
    obj = os.path.join(obj_dir, name[:-3] + ".o")
    cmd = [nvcc] + ARCH + COMMON + extra + ["-I", SRC, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {name}:\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        print(r.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, debug: bool = False, out: str = None,
          only: List[str] = None) -> str:
    """Builds the library.  ``debug`` adds -DNSA_DEBUG_BOUNDS; a debug build goes to its own object
    directory and, unless ``out`` names another file, to ``libnsa_b200_debug.so`` beside the release
    library (which stays in place).  ``only`` restricts the build to some translation units (a
    partial library for a test that needs few entry points; ``runtime.cu`` is always included)."""
    nvcc = nvcc_path()
    obj_dir = os.path.join(OBJ, "debug") if debug else OBJ
    lib = out or (os.path.join(HERE, "libnsa_b200_debug.so") if debug else LIB)
    os.makedirs(obj_dir, exist_ok=True)
    extra = ["-DNSA_DEBUG_BOUNDS"] if debug else []
    hdr = _newest_header()
    todo, objs = [], []
    names = sources() if only is None else sorted(set(only) | {"runtime.cu"})
    for name in names:
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        objs.append(obj)
        stale = (force or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(SRC, name)), hdr))
        if stale:
            todo.append(name)
    if todo:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(lambda n: _compile(nvcc, n, extra, verbose, obj_dir), todo))
    if todo or not os.path.exists(lib):
        cmd = [nvcc, "-shared", "-o", lib] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--debug", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.debug))


if __name__ == "__main__":
    main()
