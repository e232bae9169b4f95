"""Builds the sm_100a shared library of the package, in tree, with nvcc.

    python -m strixite_b200.build            # -> strixite_b200/libstrix_b200.so

Every translation unit under csrc/ is compiled for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`) and
linked into one library whose exported symbols are the C ABI declared in include/strix_b200.h.
"""
from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

PKG = pathlib.Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OUT = PKG / "libstrix_b200.so"
OBJ = PKG / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", str(ROOT / "include"), "-I", str(CSRC),
    "-DSXB_BUILDING=1",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the sm_100a library cannot be built")
    return exe


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: pathlib.Path, deps: list[pathlib.Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> pathlib.Path:
    headers = sorted(CSRC.glob("*.cuh")) + sorted((ROOT / "include").glob("*.h")) + [pathlib.Path(__file__)]
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append((src, cmd))
    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, res in pool.map(run, jobs):
            if verbose or ptxas_info or res.returncode:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [OBJ / (s.stem + ".o") for s in sources()]
    if force or jobs or _stale(OUT, objs):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(OUT), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("linking libstrix_b200.so failed")
    return OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
