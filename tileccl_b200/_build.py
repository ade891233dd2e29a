"""Builds ``libtileccl_b200.so`` in-tree with nvcc for sm_100a.

The library is plain C ABI (see ``csrc/api.h``), so there is no dependency on
the PyTorch C++ headers and a full rebuild takes well under a minute.  Objects
go to ``build/`` at the repository root; the shared object is written next to
this file under ``lib/`` so that it travels with the source tree.

Run ``python -m tileccl_b200._build`` (add ``--force`` to rebuild everything,
``--ptxas-v`` to print register / shared-memory usage of every kernel).
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libtileccl_b200.so"
DEBUG_LIB_PATH = LIB_DIR / "libtileccl_b200_debug.so"     # -DTILECCL_DEBUG_CHECKS
BUILD_DIR = PKG_DIR.parent / "build" / "tileccl_b200"
DEBUG_BUILD_DIR = PKG_DIR.parent / "build" / "tileccl_b200_debug"
DEBUG_FLAGS = ["-DTILECCL_DEBUG_CHECKS=1"]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def sources() -> list[Path]:
    out: list[Path] = []
    for pattern in ("**/*.cu", "**/*.cc"):
        out.extend(sorted(CSRC.glob(pattern)))
    return out


def _headers_mtime() -> float:
    latest = 0.0
    for pattern in ("**/*.h", "**/*.cuh"):
        for h in CSRC.glob(pattern):
            latest = max(latest, h.stat().st_mtime)
    return latest


def _compile_one(nvcc: str, src: Path, obj: Path, extra: list[str]) -> tuple[Path, str]:
    cmd = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cc":
        # Host-only translation units still include cuda.h / cuda_runtime.h.
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return src, proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False,
          debug: bool = False) -> Path:
    """Compile every translation unit under ``csrc/`` and link the shared object.

    ``debug=True`` builds the second library, ``libtileccl_b200_debug.so``: the same sources
    with ``-DTILECCL_DEBUG_CHECKS``, in which pointer translations and the symmetric tiles
    the verbs and collectives touch are bounds-checked on the device and violations are
    recorded instead of faulting (``tileccl_b200.debug``; ``TILECCL_DEBUG=1`` loads it)."""
    nvcc = _nvcc()
    build_dir = DEBUG_BUILD_DIR if debug else BUILD_DIR
    lib_path = DEBUG_LIB_PATH if debug else LIB_PATH
    build_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    hdr_mtime = _headers_mtime()
    extra = (["-Xptxas", "-v"] if ptxas_v else []) + (DEBUG_FLAGS if debug else [])
    jobs = []
    objs = []
    for src in sources():
        rel = src.relative_to(CSRC)
        obj = build_dir / (str(rel).replace(os.sep, "__") + ".o")
        objs.append(obj)
        stale = (
            force
            or ptxas_v
            or not obj.exists()
            or obj.stat().st_mtime < src.stat().st_mtime
            or obj.stat().st_mtime < hdr_mtime
        )
        if stale:
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, extra) for s, o in jobs]
            for f in futs:
                src, log = f.result()
                if verbose or ptxas_v:
                    print(f"[tileccl_b200 build] {src.relative_to(CSRC)}")
                    if log.strip():
                        print(log)
    need_link = bool(jobs) or not lib_path.exists()
    if need_link:
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(lib_path), *map(str, objs), "-lpthread", "-ldl"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(f"[tileccl_b200 build] linked {lib_path}")
    return lib_path


def build_all(force: bool = False, verbose: bool = False) -> list[Path]:
    """The release library and the debug library."""
    return [build(force=force, verbose=verbose), build(force=force, verbose=verbose, debug=True)]


if __name__ == "__main__":
    if "--all" in sys.argv:
        for p in build_all(force="--force" in sys.argv, verbose=True):
            print(p)
    else:
        path = build(force="--force" in sys.argv, verbose=True, ptxas_v="--ptxas-v" in sys.argv,
                     debug="--debug" in sys.argv)
        print(path)
