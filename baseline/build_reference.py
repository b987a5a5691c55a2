#!/usr/bin/env python
"""Offline build of the UNMODIFIED reference (Scifan/Tesseract) into ``baseline/_ref`` for ``bench.py --impl reference``.

The reference is a CMake/C++ project (no ``setup.py`` / ``pyproject.toml``), so ``pip install`` of its source tree
fails; this script configures it with CMake out of tree instead:

* ``find_package(fmt 9)`` (cmake/Dependencies.cmake:7-17) is satisfied by ``baseline/cmake/fmt``: a header-only
  ``fmt::fmt`` over the fmt headers that ship inside the installed torch wheel -- no FetchContent, no network;
* tests (Catch2) off; benchmarks, examples and the pybind11 module on; CUDA + NCCL on, compiled for sm_100;
* ``baseline/harness`` adds two small executables that call the reference's public C++ API (LlamaModel /
  cross_entropy / Engine::backward / Adam, and ContinuousBatchingScheduler) at a shape given on the command line.

Installed layout (git-ignored, travels with a source snapshot):
    baseline/_ref/bin/{ref_train_bench,ref_serve_bench,bench_cuda_llama_serving,bench_cuda_nccl_tp,tesseract_llama_train,...}
    baseline/_ref/python/tesseract/   the reference's own ``tesseract._core`` (CPU tensors only)
    baseline/_ref/BUILD_INFO.json

    python baseline/build_reference.py [--reference /root/reference] [--build-dir /tmp/tesseract_ref_build]
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
INSTALL = os.path.join(HERE, "_ref")
KEEP_BINARIES = ["ref_train_bench", "ref_serve_bench"]
KEEP_REFERENCE_BINARIES = ["benchmarks/bench_cuda_llama_serving", "benchmarks/bench_cuda_nccl_tp",
                           "benchmarks/bench_cuda_matmul", "benchmarks/bench_cuda_fp8_gemm",
                           "examples/tesseract_llama_train", "examples/tesseract_llama_serve"]


def _torch_include() -> str:
    import importlib.util
    spec = importlib.util.find_spec("torch")
    if spec is None or not spec.submodule_search_locations:
        raise SystemExit("torch is not installed: its bundled fmt headers are the offline fmt source")
    inc = os.path.join(list(spec.submodule_search_locations)[0], "include")
    if not os.path.exists(os.path.join(inc, "fmt", "format.h")):
        raise SystemExit(f"no fmt headers under {inc}")
    return inc


def _nccl_args() -> list[str]:
    for inc, lib in (("/usr/include", "/usr/lib/x86_64-linux-gnu/libnccl.so.2"),):
        if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(lib):
            return ["-DTESSERACT_ENABLE_NCCL=ON", "-DNCCL_ROOT=/usr", f"-DNCCL_INCLUDE_DIR={inc}", f"-DNCCL_LIBRARY={lib}"]
    try:
        import nvidia.nccl as n  # namespace package of the pip wheel
        root = list(n.__path__)[0]
        if os.path.exists(os.path.join(root, "include", "nccl.h")):
            return ["-DTESSERACT_ENABLE_NCCL=ON", f"-DNCCL_ROOT={root}"]
    except Exception:
        pass
    return ["-DTESSERACT_ENABLE_NCCL=OFF"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("TESSERACT_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--build-dir", default="/tmp/tesseract_ref_build")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--arch", default="100")
    a = ap.parse_args()
    if not os.path.exists(os.path.join(a.reference, "CMakeLists.txt")):
        raise SystemExit(f"no reference source tree at {a.reference}")
    t0 = time.time()
    os.makedirs(a.build_dir, exist_ok=True)
    ref_build, harness_build = os.path.join(a.build_dir, "reference"), os.path.join(a.build_dir, "harness")
    fmt_inc, nccl = _torch_include(), _nccl_args()
    cfg = ["cmake", "-S", a.reference, "-B", ref_build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release",
           f"-Dfmt_DIR={os.path.join(HERE, 'cmake', 'fmt')}", f"-DFMT_INCLUDE_DIR={fmt_inc}",
           "-DTESSERACT_BUILD_TESTS=OFF", "-DTESSERACT_BUILD_BENCHMARKS=ON", "-DTESSERACT_BUILD_EXAMPLES=ON",
           "-DTESSERACT_BUILD_PYTHON=ON", "-DTESSERACT_ENABLE_CUDA=ON", f"-DTESSERACT_CUDA_ARCHITECTURES={a.arch}",
           "-DCMAKE_CUDA_COMPILER=/usr/local/cuda/bin/nvcc"] + nccl
    nccl_lib = next((x.split("=", 1)[1] for x in nccl if x.startswith("-DNCCL_LIBRARY=")), "")
    cfg_h = ["cmake", "-S", os.path.join(HERE, "harness"), "-B", harness_build, "-G", "Ninja",
             "-DCMAKE_BUILD_TYPE=Release", f"-DREFERENCE_DIR={a.reference}", f"-DREFERENCE_BUILD_DIR={ref_build}",
             f"-DFMT_INCLUDE_DIR={fmt_inc}", f"-DNCCL_LIBRARY={nccl_lib}"]
    log = os.path.join(a.build_dir, "build_reference.log")
    with open(log, "w") as f:
        for cmd in (cfg, ["ninja", "-C", ref_build, f"-j{a.jobs}"], cfg_h, ["ninja", "-C", harness_build, f"-j{a.jobs}"]):
            f.write("$ " + " ".join(cmd) + "\n")
            f.flush()
            rc = subprocess.call(cmd, stdout=f, stderr=subprocess.STDOUT)
            if rc != 0:
                print(f"reference build failed (rc {rc}); log: {log}", file=sys.stderr)
                with open(log) as g:
                    sys.stderr.write("".join(g.readlines()[-30:]))
                return rc
    if os.path.isdir(INSTALL):
        shutil.rmtree(INSTALL)
    os.makedirs(os.path.join(INSTALL, "bin"))
    for b in KEEP_BINARIES:
        shutil.copy2(os.path.join(harness_build, b), os.path.join(INSTALL, "bin", b))
    for b in KEEP_REFERENCE_BINARIES:
        src = os.path.join(a.build_dir, "reference", b)
        if os.path.exists(src):
            shutil.copy2(src, os.path.join(INSTALL, "bin", os.path.basename(b)))
    for f in os.listdir(os.path.join(INSTALL, "bin")):
        subprocess.call(["strip", os.path.join(INSTALL, "bin", f)])
    py_src = os.path.join(a.build_dir, "reference", "python", "tesseract")
    if os.path.isdir(py_src):
        shutil.copytree(py_src, os.path.join(INSTALL, "python", "tesseract"))
    info = {"reference": a.reference, "arch": f"sm_{a.arch}", "built_in_s": round(time.time() - t0, 1),
            "cmake_args": cfg[8:], "binaries": sorted(os.listdir(os.path.join(INSTALL, "bin")))}
    with open(os.path.join(INSTALL, "BUILD_INFO.json"), "w") as f:
        json.dump(info, f, indent=1)
    print(json.dumps(info))
    return 0


if __name__ == "__main__":
    sys.exit(main())
