"""Builds the sm_100a kernel library in-tree: ``python -m ajllm_b200.build``.

One ``nvcc -gencode arch=compute_100a,code=sm_100a`` invocation per ``.cu`` file (in parallel), then a
shared-library link into ``ajllm_b200/_native/libajllm_b200.so``. Objects are rebuilt only when their
source or a header is newer. ``-Xptxas -v`` output is kept next to the objects (``*.ptxas.txt``) so
register and shared-memory use can be read without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
OUT = PACKAGE / "_native"
LIB = OUT / "libajllm_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return found


def _needs_build(source: Path, obj: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    stamp = obj.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in [source, *headers])


def _compile(nvcc: str, source: Path, obj: Path) -> tuple[Path, str]:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(source), "-o", str(obj)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    log = done.stdout + done.stderr
    obj.with_suffix(".ptxas.txt").write_text(log)
    if done.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source.name}:\n{log[-6000:]}")
    return obj, log


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = find_nvcc()
    OUT.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    jobs = []
    for source in sources:
        obj = OUT / (source.stem + ".o")
        if force or _needs_build(source, obj, headers):
            jobs.append((source, obj))
    if jobs:
        workers = min(len(jobs), max(1, (os.cpu_count() or 2)))
        with ThreadPoolExecutor(max_workers=workers) as pool:
            for obj, log in pool.map(lambda job: _compile(nvcc, *job), jobs):
                if verbose:
                    print(f"[build] {obj.name}\n{log}")
    objects = [OUT / (source.stem + ".o") for source in sources]
    if jobs or not LIB.exists():
        link = [nvcc, "-shared", "-o", str(LIB), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a",
                "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        done = subprocess.run(link, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}{done.stderr}")
    return LIB


def main() -> None:
    force = "--force" in sys.argv
    path = build(force=force, verbose="-v" in sys.argv)
    print(path)


if __name__ == "__main__":
    main()
