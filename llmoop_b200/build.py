"""In-tree build of libnerve_b200.so (sm_100a only): nvcc for .cu, g++ for .cpp,
objects cached under llmoop_b200/build/ by source+header mtime."""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB = HERE / "libnerve_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; libnerve_b200.so cannot be built")
    return found


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.hpp")) + sorted(CSRC.glob("*.cuh")) + sorted((HERE.parent / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    jobs = []
    objects = []
    for source in sources:
        obj = BUILD / (source.name + ".o")
        objects.append(obj)
        if not _stale(obj, [source, *headers]):
            continue
        if source.suffix == ".cu":
            command = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if ptxas_info else []), "-c", str(source), "-o", str(obj)]
        else:
            command = ["g++", *CXX_FLAGS, "-c", str(source), "-o", str(obj)]
        jobs.append(command)

    def run(command):
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError("build failed: " + " ".join(command) + "\n" + result.stdout + result.stderr)
        return command, result.stdout + result.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        for command, output in pool.map(run, jobs):
            if verbose or ptxas_info:
                print(" ".join(command[-3:]))
                if output.strip():
                    print(output)
    if jobs or _stale(LIB, objects):
        link = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a",
                "-Xcompiler", "-fPIC", "-lcudart"]
        run(link)
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv))
