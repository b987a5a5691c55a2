"""In-tree build of the native libraries.

Two artefacts, both placed inside the package so that they travel with a source snapshot:

* ``tesseract_b200/_lib/libtesseract_b200_cuda.so`` -- every ``csrc/*.cu`` compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a -lineinfo``) and linked into one
  shared library that exports a C ABI (loaded with ctypes; no torch headers, so a full rebuild takes
  well under a minute).
* ``tesseract_b200/_lib/_tsb_host*.so`` -- the host runtime (safetensors reads, BPE merge loop, sampler, regex
  compiler and token mask, block allocator, CPU GEMV and GEMM), a pybind11 module built from ``csrc/host``.

``python -m tesseract_b200.build`` rebuilds whatever is out of date (``--force`` rebuilds everything).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
OBJ_DIR = PKG.parent / "build" / "obj"

CUDA_LIB = LIB_DIR / "libtesseract_b200_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-march=x86-64-v3", "-fopenmp"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built on this machine")
    return cand


def _host_ext_path() -> Path:
    return LIB_DIR / ("_tsb_host" + sysconfig.get_config_var("EXT_SUFFIX"))


def _digest(paths, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"command failed: {' '.join(map(str, cmd))}")
    return r.stdout + r.stderr


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile csrc/*.cu for sm_100a and link libtesseract_b200_cuda.so. Returns its path."""
    nvcc = _nvcc()
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else [])
    hdr_digest = _digest(headers, flags)
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        stamp = OBJ_DIR / (src.stem + ".stamp")
        want = _digest([src], [hdr_digest])
        objs.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != want:
            jobs.append((src, obj, stamp, want))

    def compile_one(job):
        src, obj, stamp, want = job
        out = _run([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], verbose)
        stamp.write_text(want)
        return src.name, out

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for name, out in ex.map(compile_one, jobs):
                if ptxas_info and out:
                    print(f"== {name}\n{out}")
    link_stamp = OBJ_DIR / "link.stamp"
    want_link = hashlib.sha256("".join((OBJ_DIR / (s.stem + ".stamp")).read_text() for s in sources).encode()).hexdigest()
    if jobs or not CUDA_LIB.exists() or not link_stamp.exists() or link_stamp.read_text() != want_link:
        _run([nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-Xcompiler", "-fPIC", "-lcudart"], verbose)
        link_stamp.write_text(want_link)
    return CUDA_LIB


def build_host(force: bool = False, verbose: bool = False) -> Path:
    """Build the pybind11 host-runtime module from csrc/host/*.cpp. Returns its path."""
    import pybind11

    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    host_dir = CSRC / "host"
    sources = sorted(host_dir.glob("*.cpp"))
    if not sources:
        return _host_ext_path()
    headers = sorted(host_dir.glob("*.hpp")) + sorted(host_dir.glob("*.h"))
    cxx = shutil.which("g++") or "g++"
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(host_dir)]
    hdr_digest = _digest(headers, CXX_FLAGS)
    jobs, objs = [], []
    for src in sources:
        obj = OBJ_DIR / ("host_" + src.stem + ".o")
        stamp = OBJ_DIR / ("host_" + src.stem + ".stamp")
        want = _digest([src], [hdr_digest])
        objs.append(obj)
        if force or not obj.exists() or not stamp.exists() or stamp.read_text() != want:
            jobs.append((src, obj, stamp, want))

    def compile_one(job):
        src, obj, stamp, want = job
        _run([cxx, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)], verbose)
        stamp.write_text(want)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    out = _host_ext_path()
    if jobs or not out.exists():
        _run([cxx, "-shared", "-o", str(out), *map(str, objs), "-fopenmp"], verbose)
    return out


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False):
    return build_cuda(force, verbose, ptxas_info), build_host(force, verbose)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--only", choices=["cuda", "host"], default=None)
    a = ap.parse_args(argv)
    if a.only in (None, "cuda"):
        print(build_cuda(a.force, a.verbose, a.ptxas_info))
    if a.only in (None, "host"):
        print(build_host(a.force, a.verbose))


if __name__ == "__main__":
    main()
