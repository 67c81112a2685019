"""In-tree build of ``liballoy_b200.so`` (sm_100a) with nvcc.

``python -m alloy_b200.build`` compiles every ``csrc/*.cu`` to an object file
and links them into ``alloy_b200/liballoy_b200.so`` next to this file.  Objects
are rebuilt only when their source (or a header) is newer.  nvcc cross-compiles
without a GPU, so this runs on CPU-only machines too.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "_obj"
LIB = HERE / "liballoy_b200.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--use_fast_math=false",
              "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and pathlib.Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _compile(nvcc: str, src: pathlib.Path, obj: pathlib.Path, verbose: bool) -> str:
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    cmd = [nvcc, *ARCH, *flags, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    (obj.with_suffix(".ptxas.txt")).write_text(res.stderr)
    return res.stderr if verbose else ""


def build_library(force: bool = False, verbose: bool = False) -> pathlib.Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    newest_hdr = max((h.stat().st_mtime for h in headers), default=0.0)
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_hdr)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs):
                if out:
                    print(out, file=sys.stderr)
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if jobs or not LIB.exists():
        cmd = [nvcc, *ARCH, "-shared", "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
