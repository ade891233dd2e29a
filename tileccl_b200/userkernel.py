"""Write your own sm_100a kernel with the tile primitives and run it on the heap.

In the reference any ``@triton.jit`` kernel can import ``tile_put``,
``tile_signal``, ``tile_allreduce`` ... (tileccl/primitives/__init__.py:49-81).
Here the primitives are CUDA ``__device__`` functions in
``tileccl_b200/csrc/device/*.cuh``; this module compiles a user ``.cu`` file
against them with nvcc and launches it with the symmetric-heap window of a
context:

.. code-block:: cpp

    // my_kernel.cu
    #include <tile_collectives.cuh>            // or tile_comm.cuh, tile_sync.cuh, ...
    using namespace tileccl;

    __global__ void my_kernel(SymmWindow w, uint64_t* args) { ... tile_put(w, ...); }

    // The entry point the loader calls: one launch acts as rank `w->rank`.
    extern "C" int tileccl_user_launch(const SymmWindow* w, const uint64_t* args, int n_args,
                                       int grid, int block, void* stream) {
      ...copy args, launch, return (int)cudaGetLastError();
    }

.. code-block:: python

    from tileccl_b200 import userkernel
    mod = userkernel.compile("my_kernel.cu")
    mod.launch(ctx, [buf.data_ptr(), flags.data_ptr()], grid=4, block=256)

``TILECCL_USER_KERNEL_MAIN(kernel)`` in ``user_kernel.cuh`` writes that entry point
for a kernel with the signature ``(SymmWindow, UserArgs)``.
"""

from __future__ import annotations

import ctypes as C
import hashlib
import subprocess
from pathlib import Path
from typing import Optional, Sequence

from . import _build

INCLUDE_DIR = _build.CSRC / "device"
CACHE_DIR = _build.BUILD_DIR.parent / "user_kernels"
MAX_ARGS = 16


class SymmWindow(C.Structure):
    """Mirror of ``tileccl::SymmWindow`` (csrc/device/symm_ptr.cuh)."""

    _fields_ = [("base", C.c_uint64), ("stride", C.c_uint64), ("mc_base", C.c_uint64),
                ("rank", C.c_int32), ("world_size", C.c_int32)]


def include_dir() -> Path:
    """Directory to pass to ``nvcc -I`` so that ``#include <tile_comm.cuh>`` etc. resolve."""
    return INCLUDE_DIR


def window_of(heap, rank: Optional[int] = None) -> SymmWindow:
    """The heap's address window as the device functions expect it, seen from `rank`."""
    return SymmWindow(heap.window_base, heap.stride, heap.multicast_base,
                      heap.rank if rank is None else rank, heap.world_size)


class UserKernelModule:
    def __init__(self, path: Path, entry: str = "tileccl_user_launch"):
        self.path = Path(path)
        self._lib = C.CDLL(str(self.path))
        fn = getattr(self._lib, entry, None)
        if fn is None:
            raise AttributeError(f"{self.path} does not export `{entry}` (see "
                                 "TILECCL_USER_KERNEL_MAIN in user_kernel.cuh)")
        fn.argtypes = [C.POINTER(SymmWindow), C.POINTER(C.c_uint64), C.c_int, C.c_int, C.c_int,
                       C.c_void_p]
        fn.restype = C.c_int
        self._fn = fn
        self._debug_read = getattr(self._lib, "tileccl_user_debug_read", None)
        if self._debug_read is not None:
            self._debug_read.argtypes = [C.c_void_p, C.c_int]
            self._debug_read.restype = C.c_int

    def debug_record(self, *, clear: bool = True):
        """The bounds-violation record of this object on the current device (see
        ``tileccl_b200.debug``); None if the object was built without the entry macros."""
        if self._debug_read is None:
            return None
        from .debug import DebugRecord

        rec = DebugRecord()
        rc = self._debug_read(C.byref(rec), 1 if clear else 0)
        if rc != 0:
            raise RuntimeError(f"reading the debug record failed with CUDA error {rc}")
        return rec

    def launch(self, ctx_or_heap, args: Sequence[int], *, grid: int = 1, block: int = 256,
               rank: Optional[int] = None, stream=None) -> None:
        """Launch on the heap's device as `rank` (default: the heap's own rank).

        ``args``: up to 16 integers (device addresses, sizes, epochs); the kernel receives
        them as ``UserArgs::v[i]``.  Addresses that name symmetric objects are addresses in
        the CALLING rank's heap, as for every primitive.
        """
        import torch

        heap = getattr(ctx_or_heap, "heap", ctx_or_heap)
        if len(args) > MAX_ARGS:
            raise ValueError(f"at most {MAX_ARGS} arguments, got {len(args)}")
        w = window_of(heap, rank)
        arr = (C.c_uint64 * max(1, len(args)))(*[int(a) & 0xFFFFFFFFFFFFFFFF for a in args])
        with torch.cuda.device(heap.device):
            s = stream if stream is not None else torch.cuda.current_stream()
            rc = self._fn(C.byref(w), arr, len(args), int(grid), int(block),
                          C.c_void_p(s.cuda_stream))
        if rc != 0:
            raise RuntimeError(f"user kernel launch failed with CUDA error {rc}")


def compile(source, *, extra_flags: Sequence[str] = (), force: bool = False,
            entry: str = "tileccl_user_launch", debug: bool = False) -> UserKernelModule:
    """Compile ``source`` (a ``.cu`` path) for sm_100a against the device headers and load it.

    ``debug=True`` adds ``-DTILECCL_DEBUG_CHECKS``: translations and symmetric tiles are
    bounds-checked on the device and violations recorded (``module.debug_record()``).

    The shared object is cached under ``build/user_kernels/`` keyed by the source text, the
    headers' time stamps and the flags, so repeated calls cost nothing.
    """
    if debug:
        extra_flags = tuple(extra_flags) + tuple(_build.DEBUG_FLAGS)
    src = Path(source).resolve()
    text = src.read_bytes()
    stamp = max((h.stat().st_mtime_ns for h in INCLUDE_DIR.glob("*.cuh")), default=0)
    key = hashlib.sha256(text + repr((tuple(extra_flags), stamp)).encode()).hexdigest()[:16]
    CACHE_DIR.mkdir(parents=True, exist_ok=True)
    out = CACHE_DIR / f"{src.stem}_{key}.so"
    if force or not out.exists():
        cmd = [_build._nvcc(), *_build.ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-shared",
               "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", str(INCLUDE_DIR),
               *extra_flags, str(src), "-o", str(out)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return UserKernelModule(out, entry)
