"""In-tree build of the two native artefacts (no JIT cache, no installation step):

* ``libbf16_huffman_b200.so`` - the CUDA kernels behind the C ABI of ``include/bf16_huffman_b200.h``
  (``nvcc`` for sm_100a only; it has no torch or Python dependency);
* ``_C.abi3.so`` - the PyTorch stable-ABI operator library that forwards to it (host C++ only).

``python bf16_huffman_infer_b200/_build.py`` builds both; ``build()`` is also what
``__graft_entry__.build`` calls.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libbf16_huffman_b200.so")
EXT_PATH = os.path.join(PKG_DIR, "_C.abi3.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xptxas", "-v", "-Xptxas", "--warn-on-spills",
    "-shared", "-Xcompiler", "-fPIC",
]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _run(cmd, log_name):
    r = subprocess.run(cmd, capture_output=True, text=True)
    os.makedirs(os.path.join(PKG_DIR, "build"), exist_ok=True)
    with open(os.path.join(PKG_DIR, "build", log_name), "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build failed ({' '.join(cmd[:3])} ...):\n{r.stdout}\n{r.stderr}")


def build_library(force: bool = False) -> str:
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))]
    sources.append(os.path.join(PKG_DIR, "..", "include", "bf16_huffman_b200.h"))
    if not force and _newer(LIB_PATH, sources):
        return LIB_PATH
    units = [s for s in sources if s.endswith(".cu")]
    _run([_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *units], "build_lib.log")
    return LIB_PATH


def build_extension(force: bool = False) -> str:
    src = os.path.join(CSRC, "bhi_torch_ext.cpp")
    if not force and _newer(EXT_PATH, [src, LIB_PATH]):
        return EXT_PATH
    import torch
    from torch.utils import cpp_extension

    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DPy_LIMITED_API=0x03090000",
        "-DTORCH_TARGET_VERSION=0x020b000000000000",
        *inc, src, "-o", EXT_PATH,
        f"-L{PKG_DIR}", "-l:libbf16_huffman_b200.so", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{torch_lib}",
    ]
    try:
        _run(cmd, "build_ext.log")
    except RuntimeError:
        cmd.remove("-DTORCH_TARGET_VERSION=0x020b000000000000")
        _run(cmd, "build_ext.log")
    return EXT_PATH


def build(force: bool = False) -> None:
    build_library(force)
    build_extension(force)


if __name__ == "__main__":
    build(force="--force" in sys.argv)
    print(LIB_PATH)
    print(EXT_PATH)
