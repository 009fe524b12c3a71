"""Builds the native libraries of ghost_flow_b200 in-tree with nvcc / g++.

``libgfb200.so``   - every CUDA kernel (sm_100a only) behind a C ABI, loaded with ctypes.
``libghostflow.so`` - the C ABI of the reference's ``ghostflow.h`` plus the checkpoint
                      readers/writers (host C++ only, no CUDA needed to load it).

Usage: ``python -m ghost_flow_b200.csrc.build [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
LIB_DIR = PKG / "lib"
OBJ_DIR = HERE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

# CUDA sources that travel to every run (none of them uses a TMA load with cluster multicast).
CUDA_SOURCES = [
    "gf_host.cu",
    "gemm_bf16.cu",
    "gemm2sm_bf16.cu",
    "norm.cu",
    "pointwise.cu",
    "xent_adamw.cu",
    "attn_fwd.cu",
    "attn_fwd2.cu",
    "attn_fwd3.cu",
    "attn_bwd.cu",
    "attn_bwd2.cu",
    "attn_decode.cu",
    "comm_kernels.cu",
    "moe_kernels.cu",
    "quant_fp8.cu",
    "misc_kernels.cu",
    "noalloc.cu",
    "runtime.cu",
]

HOST_SOURCES = ["cabi.cpp", "formats.cpp", "cpu_ref.cpp", "symm_alloc.cpp"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha1()
    h.update(path.read_bytes())
    for hdr in sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(extra.encode())
    return h.hexdigest()


def _compile_one(cmd: list[str], src: Path, obj: Path, stamp: Path, digest: str, verbose: bool) -> str:
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return f"up to date  {src.name}"
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)
    return f"compiled    {src.name}"


# Sources that contain checked accesses (GF_CHECK_IDX): only these are compiled a second time for the checked library;
# the other objects are shared between the two libraries.
CHECKED_SOURCES = ["gf_host.cu", "gemm_bf16.cu", "moe_kernels.cu"]


def build(force: bool = False, verbose: bool = False, checked: bool = True) -> dict[str, Path]:
    """Compiles what is out of date and links the libraries. Returns their paths. ``checked`` also links
    ``libgfb200_checked.so`` (``-DGF_CHECKED``: data-dependent indices are range-checked on the device and the first
    offender is reported through the status buffer), which ``GF_CHECKED=1`` makes the package load."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    cuda_objs, host_objs, checked_objs = [], [], []
    for name in CUDA_SOURCES:
        src = HERE / name
        if not src.exists():
            continue
        obj = OBJ_DIR / (name + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, src, obj))
        cuda_objs.append(obj)
        if checked and name in CHECKED_SOURCES:
            cobj = OBJ_DIR / (name + ".checked.o")
            jobs.append(([nvcc, *NVCC_FLAGS, "-DGF_CHECKED", "-I", str(HERE), "-c", str(src), "-o", str(cobj)], src,
                         cobj))
            checked_objs.append(cobj)
        elif checked:
            checked_objs.append(obj)
    for name in HOST_SOURCES:
        src = HERE / name
        if not src.exists():
            continue
        obj = OBJ_DIR / (name + ".o")
        cuda_inc = Path(nvcc).resolve().parent.parent / "include"      # headers only (ABI checks); nothing is linked
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-I", str(HERE),
               *(["-I", str(cuda_inc), "-DGF_HAVE_CUDA_H"] if (cuda_inc / "cuda.h").exists() else []),
               "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, src, obj))
        host_objs.append(obj)
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        futs = []
        for cmd, src, obj in jobs:
            stamp = obj.with_suffix(".stamp")
            digest = _digest(src, " ".join(cmd))
            if force and stamp.exists():
                stamp.unlink()
            futs.append(ex.submit(_compile_one, cmd, src, obj, stamp, digest, verbose))
        for f in futs:
            msg = f.result()
            if verbose:
                print(msg)
    out = {}
    if cuda_objs:
        lib = LIB_DIR / "libgfb200.so"
        newest = max(o.stat().st_mtime for o in cuda_objs)
        if force or not lib.exists() or lib.stat().st_mtime < newest:
            cmd = [nvcc, "-shared", "-o", str(lib), *map(str, cuda_objs)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        out["cuda"] = lib
        if checked:
            lib = LIB_DIR / "libgfb200_checked.so"
            newest = max(o.stat().st_mtime for o in checked_objs)
            if force or not lib.exists() or lib.stat().st_mtime < newest:
                r = subprocess.run([nvcc, "-shared", "-o", str(lib), *map(str, checked_objs)], capture_output=True,
                                   text=True)
                if r.returncode != 0:
                    raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
            out["cuda_checked"] = lib
    if host_objs:
        lib = LIB_DIR / "libghostflow.so"
        newest = max(o.stat().st_mtime for o in host_objs)
        if force or not lib.exists() or lib.stat().st_mtime < newest:
            cmd = ["g++", "-shared", "-o", str(lib), *map(str, host_objs), "-lpthread", "-ldl"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        out["host"] = lib
    return out


if __name__ == "__main__":
    libs = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv)
    for k, v in libs.items():
        print(f"{k}: {v}")
