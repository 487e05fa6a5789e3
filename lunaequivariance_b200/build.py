"""Builds the C-ABI shared library ``_lib/libluna_b200.so`` from ``csrc/*.cu`` with nvcc for sm_100a.

Usage: ``python -m lunaequivariance_b200.build [--force] [--verbose]``.  Objects are rebuilt only when a source or
header is newer; files compile in parallel.  No GPU is needed to build.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PACKAGE_DIR, "csrc")
LIB_DIR = os.path.join(PACKAGE_DIR, "_lib")
BUILD_DIR = os.path.join(PACKAGE_DIR, "_lib", "obj")
LIBRARY = os.path.join(LIB_DIR, "libluna_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or CUDA_HOME")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, name) for name in os.listdir(CSRC) if name.endswith(".cu"))


def headers_mtime() -> float:
    paths = [os.path.join(CSRC, n) for n in os.listdir(CSRC) if n.endswith((".h", ".cuh"))]
    paths.append(os.path.join(os.path.dirname(PACKAGE_DIR), "include", "luna_b200.h"))
    return max(os.path.getmtime(p) for p in paths if os.path.exists(p))


def compile_one(nvcc: str, source: str, verbose: bool, ptxas_info: bool) -> tuple[str, str]:
    obj = os.path.join(BUILD_DIR, os.path.basename(source)[:-3] + ".o")
    command = [nvcc, *NVCC_FLAGS, "-c", source, "-o", obj]
    if ptxas_info:
        command[1:1] = ["-Xptxas", "-v"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")
    return obj, result.stderr if (verbose or ptxas_info) else ""


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    nvcc = find_nvcc()
    os.makedirs(BUILD_DIR, exist_ok=True)
    newest_header = headers_mtime()
    todo, objects = [], []
    for source in sources():
        obj = os.path.join(BUILD_DIR, os.path.basename(source)[:-3] + ".o")
        objects.append(obj)
        stale = (force or ptxas_info or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(os.path.getmtime(source), newest_header))
        if stale:
            todo.append(source)
    if todo:
        workers = min(len(todo), max(1, (os.cpu_count() or 2)))
        with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as pool:
            for obj, log in pool.map(lambda s: compile_one(nvcc, s, verbose, ptxas_info), todo):
                if log:
                    print(log, file=sys.stderr)
    wanted = {os.path.basename(o) for o in objects}
    for name in os.listdir(BUILD_DIR):  # drop objects of deleted sources
        if name.endswith(".o") and name not in wanted:
            os.remove(os.path.join(BUILD_DIR, name))
    if todo or not os.path.exists(LIBRARY):
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                "-o", LIBRARY, *objects]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIBRARY


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--ptxas-info", action="store_true", help="print registers/spills/shared memory per kernel")
    arguments = parser.parse_args()
    print(build(arguments.force, arguments.verbose, arguments.ptxas_info))
