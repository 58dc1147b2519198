"""In-tree build and staleness-checked loading of the native library.

Parity: reference ``metal_marlin/metallib_loader.py`` (precompiled-library load with
version/checksum staleness detection) and ``cpp/src/library_manager.mm``.  Here the
library is one shared object, ``metal_marlin_b200/_C.so``: pure-CUDA kernel
translation units (no torch headers, compiled in seconds each) behind an
``extern "C"`` ABI, plus one C++ file registering ``torch.ops.mmb200.*``.  A content
hash of every source is stored beside the library; a mismatch triggers a rebuild
when a compiler is present and a loud error otherwise.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "_C.so")
HASH_PATH = LIB_PATH + ".hash"
OBJ_DIR = os.path.join(_HERE, "csrc", "_obj")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _sources() -> List[str]:
    out = []
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cpp", ".h", ".cuh")):
            out.append(os.path.join(CSRC, f))
    return out


def source_hash() -> str:
    h = hashlib.sha256()
    for p in _sources():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(HASH_PATH):
        return True
    with open(HASH_PATH) as f:
        return f.read().strip() != source_hash()


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build metal_marlin_b200/_C.so")
    return cand


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel for sm_100a and link ``_C.so``.  Returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    import torch
    from torch.utils import cpp_extension

    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    cu = [p for p in _sources() if p.endswith(".cu")]
    cpp = [p for p in _sources() if p.endswith(".cpp")]
    inc = ["-I" + CSRC, "-I" + os.path.join(cuda_home, "include")]
    torch_inc = ["-I" + p for p in cpp_extension.include_paths()]
    jobs = []
    objs = []
    for p in cu:
        o = os.path.join(OBJ_DIR, os.path.basename(p) + ".o")
        objs.append(o)
        jobs.append([nvcc, *NVCC_FLAGS, *inc, "-c", p, "-o", o])
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for p in cpp:
        o = os.path.join(OBJ_DIR, os.path.basename(p) + ".o")
        objs.append(o)
        jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                     "-DTORCH_EXTENSION_NAME=_C", *inc, *torch_inc, "-c", p, "-o", o])
    if verbose:
        for j in jobs:
            print(" ".join(j), file=sys.stderr)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    link = ["g++", "-shared", "-o", LIB_PATH + ".tmp", *objs, "-L" + torch_lib, "-L" + os.path.join(cuda_home, "lib64"),
            "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda", "-lcudart",
            "-Wl,-rpath," + torch_lib, "-Wl,-rpath," + os.path.join(cuda_home, "lib64")]
    _run(link)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    with open(HASH_PATH, "w") as f:
        f.write(source_hash())
    return LIB_PATH


_loaded = False


def load(require: bool = False) -> bool:
    """Load ``_C.so`` into this process (registers ``torch.ops.mmb200``).

    Returns False when the library is missing and ``require`` is False (CPU-only
    use of the package).  On a machine with a GPU the ops layer calls this with
    ``require=True`` so a missing or stale library is an error, never a silent
    fallback."""
    global _loaded
    if _loaded:
        return True
    import torch
    if is_stale():
        have_nvcc = shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc")
        if have_nvcc and (require or os.environ.get("MMB200_AUTOBUILD", "0") == "1"):
            build()
        elif not os.path.exists(LIB_PATH):
            if require:
                raise RuntimeError("metal_marlin_b200/_C.so is missing; run `python -m metal_marlin_b200._build`")
            return False
        elif require and os.environ.get("MMB200_ALLOW_STALE", "0") != "1":
            raise RuntimeError("metal_marlin_b200/_C.so is older than its sources; rebuild it "
                               "(python -m metal_marlin_b200._build) or set MMB200_ALLOW_STALE=1")
    torch.ops.load_library(LIB_PATH)
    _loaded = True
    return True


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
