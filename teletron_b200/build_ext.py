"""Builds the native sm_100a library in-tree with nvcc.

Every ``csrc/*.cu`` file is compiled to an object (in parallel) and linked into
``teletron_b200/_C/libtt_b200.so``.  The library exposes plain C symbols and is
loaded with ctypes (``teletron_b200.ops._lib``), so it does not depend on the
PyTorch C++ ABI and builds in seconds.  nvcc cross-compiles without a GPU.

The reference builds its two extensions with ``python *_setup.py install`` for sm_90
only (teletron_op/fused_adaln/adaln_setup.py:18-25, teletron_op/install.sh:1-9); this
is the single-library sm_100a counterpart.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT_DIR = PKG / "_C"
LIB_NAME = "libtt_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


def _digest(paths: list[Path], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def lib_path() -> Path:
    return OUT_DIR / LIB_NAME


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library."""
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = find_nvcc()
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    hdr_digest = _digest(_headers(), " ".join(flags))
    srcs = _sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")

    def compile_one(src: Path):
        obj = obj_dir / (src.stem + ".o")
        stamp = obj_dir / (src.stem + ".sha")
        want = _digest([src], hdr_digest)
        if not force and obj.exists() and stamp.exists() and stamp.read_text() == want:
            return obj, False, ""
        cmd = [nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        stamp.write_text(want)
        return obj, True, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if verbose or ptxas_info:
        for (_, did, log), src in zip(results, srcs):
            if did and log.strip():
                print(f"--- {src.name}\n{log}")
    lib = lib_path()
    if rebuilt or force or not lib.exists():
        tmp = lib.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(p)
