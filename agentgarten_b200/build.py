"""Builds the in-tree CUDA extension ``agentgarten_b200/_C.so`` for sm_100a.

``python -m agentgarten_b200.build [--force] [--verbose]`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and every ``csrc/*.cpp`` with the
host compiler, in parallel, then links one shared object next to the Python sources (a JIT
cache outside the tree would not travel with the repository).  Objects are rebuilt only
when a source or header is newer.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "csrc" / "build"
TARGET = ROOT / "_C.so"
IO_TARGET = ROOT / "_io.so"  # host-only helpers: no CUDA or torch libraries are linked

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C",
             "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1", "-w"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found")
    return found


def _include_flags() -> list[str]:
    from torch.utils.cpp_extension import include_paths

    paths = include_paths(device_type="cuda") if "device_type" in include_paths.__code__.co_varnames \
        else include_paths(cuda=True)
    paths.append(sysconfig.get_paths()["include"])
    paths.append(str(CSRC))
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    paths.append(os.path.join(cuda_home, "include"))
    return [f"-I{p}" for p in dict.fromkeys(paths)]


def _stale(obj: Path, source: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    newest = max(p.stat().st_mtime for p in [source, *headers, Path(__file__)])
    return obj.stat().st_mtime < newest


def build_host(force: bool = False) -> Path:
    """``csrc/host/*.cpp`` -> ``_io.so`` (plain pybind11 module, loadable on any machine)."""
    sources = sorted((CSRC / "host").glob("*.cpp"))
    newest = max(p.stat().st_mtime for p in [*sources, Path(__file__)])
    if not force and IO_TARGET.exists() and IO_TARGET.stat().st_mtime >= newest:
        return IO_TARGET
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-w",
           *_include_flags(), *map(str, sources), "-o", str(IO_TARGET)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("compilation of the host helpers failed")
    return IO_TARGET


def build(force: bool = False, verbose: bool = False) -> Path:
    build_host(force)
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted([*CSRC.glob("*.h"), *CSRC.glob("*.cuh")])
    sources = sorted([*CSRC.glob("*.cu"), *CSRC.glob("*.cpp")])
    includes = _include_flags()
    jobs = []
    for src in sources:
        obj = OBJ / (src.name + ".o")
        if not (force or _stale(obj, src, headers)):
            continue
        if src.suffix == ".cu":
            cmd = [_nvcc(), *NVCC_FLAGS, *includes, "-c", str(src), "-o", str(obj)]
        else:
            cmd = [os.environ.get("CXX", "g++"), *CXX_FLAGS, *includes, "-c", str(src), "-o", str(obj)]
        jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return src, proc

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, proc in pool.map(run, jobs):
            if proc.returncode != 0:
                sys.stderr.write(proc.stdout + proc.stderr)
                raise RuntimeError(f"compilation of {src.name} failed")
            if verbose:
                sys.stderr.write(f"== {src.name}\n{proc.stderr}")
    objects = [OBJ / (s.name + ".o") for s in sources]
    if jobs or force or not TARGET.exists():
        import torch

        lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
        cuda_lib = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "lib64")
        cmd = [os.environ.get("CXX", "g++"), "-shared", "-o", str(TARGET), *map(str, objects),
               f"-L{lib_dir}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
               "-ltorch", "-ltorch_python", "-lcudart",
               f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{cuda_lib}"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("link failed")
    return TARGET


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))
