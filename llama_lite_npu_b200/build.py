"""Build libb200kv.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run as ``python -m llama_lite_npu_b200.build`` or call :func:`build_library`.
The library is compiled next to this file so that it is found by ``_lib.py``
without any installation step.  nvcc cross-compiles, so no GPU is needed.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libb200kv.so"
STAMP_PATH = PKG_DIR / "libb200kv.stamp"

SOURCES = (
    "b200kv_capi.cu",
    "kv_append.cu",
    "qk_prologue.cu",
    "batch_metadata.cu",
    "paged_decode.cu",
    "tma.cu",
    "paged_prefill_sm100.cu",
    "prefix_cache.cpp",
    "host_step.cu",
)

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--use_fast_math",
    "-Xptxas", "-v",
)


def _find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libb200kv.so cannot be built")
    return nvcc


def _source_digest() -> str:
    h = hashlib.sha256()
    files = (sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
             + sorted(CSRC.glob("*.cpp")))
    files += sorted(INCLUDE.glob("*.h"))
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into ``libb200kv.so``; skip when sources are unchanged."""
    digest = _source_digest()
    if not force and LIB_PATH.exists() and STAMP_PATH.exists():
        if STAMP_PATH.read_text().strip() == digest:
            return LIB_PATH
    nvcc = _find_nvcc()
    build_dir = PKG_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    objects = []
    procs = []
    for src in SOURCES:
        obj = build_dir / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    log = []
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        log.append(f"==== {src} ====\n{out}")
        if proc.returncode != 0:
            failed = True
    (build_dir / "nvcc.log").write_text("\n".join(log))
    if failed:
        sys.stderr.write("\n".join(log))
        raise RuntimeError("nvcc failed while building libb200kv.so")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objects, "-lcudart"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("linking libb200kv.so failed")
    STAMP_PATH.write_text(digest)
    if verbose:
        sys.stdout.write("\n".join(log))
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose=True)
    print(path)
