"""Build ``libmindpipe_b200.so`` in-tree with nvcc for sm_100a.

``python -m mindpipe_b200.build`` (or :func:`build`) compiles every ``.cu``
under ``csrc/`` to an object file in parallel and links one shared library
at ``mindpipe_b200/lib/libmindpipe_b200.so``.  nvcc cross-compiles without a
GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libmindpipe_b200.so"
OBJ_DIR = PKG / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    return cand


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted((PKG.parent / "include").glob("*.h"))
    srcs = sources()
    jobs = []
    for src in srcs:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, *( ["-Xptxas", "-v"] if ptxas_info else []), "-c", str(src), "-o", str(obj)]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for src, res in ex.map(run, jobs):
            if verbose or ptxas_info or res.returncode != 0:
                sys.stderr.write(f"[{src.name}]\n{res.stdout}{res.stderr}\n")
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}")
    objs = [OBJ_DIR / (s.stem + ".o") for s in srcs]
    if force or jobs or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(path)
