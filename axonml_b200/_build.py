"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_lib/libaxonml_cuda.so``  - every ``csrc/kernels/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), exported through ``extern "C"`` launchers that
  take raw device pointers and a stream, loaded with ctypes (no torch headers, so a full rebuild
  takes seconds per file and cross-compiles on a machine without a GPU).
* ``_lib/libaxonml_host.so``  - ``csrc/host/*.cpp``: the C++ runtime pieces (codecs for the
  checkpoint containers, block quantisation, CPU reference kernels, the data-loader and server
  queues), compiled by g++ with OpenMP.

Objects are cached by source hash, so ``build()`` is incremental.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = ROOT / "_lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fopenmp", "-fvisibility=hidden", "-march=x86-64-v3"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(path.parent.glob("*.cuh")) + sorted(path.parent.glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def _build_lib(sources: list[Path], out: Path, compiler: list[str], flags: list[str],
               link: list[str], verbose: bool) -> bool:
    OBJ.mkdir(parents=True, exist_ok=True)
    objs, jobs = [], []
    for src in sources:
        tag = _digest(src, " ".join(compiler + flags))
        # the library's name is part of the object's: sources of the two libraries share stems
        stem = f"{out.stem}-{src.stem}"
        obj = OBJ / f"{stem}.{tag}.o"
        objs.append(obj)
        if not obj.exists():
            for old in OBJ.glob(f"{stem}.*.o"):
                old.unlink()
            jobs.append(compiler + flags + ["-c", str(src), "-o", str(obj)])
    if jobs:
        if verbose:
            print(f"[axonml_b200] compiling {len(jobs)} file(s) for {out.name}", file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            list(ex.map(_compile, jobs))
    stamp = OBJ / (out.name + ".stamp")
    want = "\n".join(o.name for o in objs)
    if jobs or not out.exists() or not stamp.exists() or stamp.read_text() != want:
        _compile(compiler + link + ["-shared", "-o", str(out)] + [str(o) for o in objs])
        stamp.write_text(want)
        return True
    return False


def build_cuda(verbose: bool = True, bounds: bool = False) -> Path:
    """``bounds=True`` builds ``libaxonml_cuda_bounds.so``: the same sources with ``-DAX_BOUNDS=1``
    (index checks that report instead of accessing, see ``common.cuh``) as relocatable device code,
    because the violation word is one device symbol shared by all translation units."""
    out = LIB / ("libaxonml_cuda_bounds.so" if bounds else "libaxonml_cuda.so")
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    flags = NVCC_FLAGS + (["-DAX_BOUNDS=1", "-rdc=true"] if bounds else [])
    link = ["-Xcompiler", "-fPIC", "-cudart", "static"] + (["-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true"] if bounds else [])
    _build_lib(srcs, out, [_nvcc()], flags, link, verbose)
    return out


def build_host(verbose: bool = True) -> Path:
    out = LIB / "libaxonml_host.so"
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        return out
    _build_lib(srcs, out, [shutil.which("g++") or "g++"], CXX_FLAGS, ["-fopenmp"], verbose)
    return out


def build(verbose: bool = True, bounds: bool = True) -> None:
    LIB.mkdir(exist_ok=True)
    build_host(verbose)
    build_cuda(verbose)
    if bounds:
        build_cuda(verbose, bounds=True)


if __name__ == "__main__":
    build()
    print("ok")
