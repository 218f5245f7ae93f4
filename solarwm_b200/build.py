"""Build the native library (sm_100a only) in-tree with nvcc.

Every ``csrc/*.cu`` / ``csrc/*.cpp`` file is compiled to an object under
``_native/obj`` and linked into ``_native/libsolar_b200.so``; the Python side loads
that file with ctypes (``solarwm_b200.ops._lib``).  nvcc cross-compiles without a GPU,
so the same call is the CPU-side "does it build" check.

    python -m solarwm_b200.build [--force] [--verbose]
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
OUT = PKG / "_native"
LIB = OUT / "libsolar_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
HOST_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fno-fast-math", "-ffp-contract=off"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _digest(paths) -> str:
    h = hashlib.blake2s()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + HOST_FLAGS).encode())
    return h.hexdigest()


def sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def build_all(force: bool = False, verbose: bool = False) -> Path:
    srcs = sources()
    headers = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    OUT.mkdir(exist_ok=True)
    obj_dir = OUT / "obj"
    obj_dir.mkdir(exist_ok=True)
    stamp = OUT / "build.stamp"
    want = _digest(srcs + headers)
    if not force and LIB.exists() and stamp.exists() and stamp.read_text() == want:
        return LIB
    nvcc = _nvcc()
    hdr_digest = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.name + ".o")
        tag = obj_dir / (src.name + ".tag")
        key = _digest([src]) + hdr_digest
        if not force and obj.exists() and tag.exists() and tag.read_text() == key:
            return obj
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
        else:
            cmd = ["g++", *HOST_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose and (res.stdout or res.stderr):
            print(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        tag.write_text(key)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = OUT / "libsolar_b200.so.tmp"
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed: {res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB)
    stamp.write_text(want)
    return LIB


if __name__ == "__main__":
    path = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
