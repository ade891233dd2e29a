"""ctypes binding of ``libtileccl_b200.so`` (C ABI declared in ``csrc/api.h``).

The shared object is built in-tree by :mod:`tileccl_b200._build`.  Importing
this module never needs a GPU: the library resolves CUDA driver entry points
lazily, so planning code, the CPU emulator and the CLI work on a machine that
has neither a GPU nor ``libcuda``.  Anything that does need the GPU fails with
:class:`NativeError` carrying the library's own message.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

from . import _build

MAX_RANKS = 8


class NativeError(RuntimeError):
    """A call into libtileccl_b200 returned a non-zero status."""

    def __init__(self, fn: str, code: int, message: str):
        super().__init__(f"{fn} failed (code {code}): {message}")
        self.fn = fn
        self.code = code
        self.message = message


class DeviceProps(C.Structure):
    _fields_ = [
        ("name", C.c_char * 128),
        ("ordinal", C.c_int32),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("sm_count", C.c_int32),
        ("warp_size", C.c_int32),
        ("max_smem_per_block_optin", C.c_int32),
        ("l2_bytes", C.c_int32),
        ("clock_khz", C.c_int32),
        ("mem_clock_khz", C.c_int32),
        ("mem_bus_bits", C.c_int32),
        ("vmm_supported", C.c_int32),
        ("posix_fd_handles", C.c_int32),
        ("fabric_handles", C.c_int32),
        ("multicast_supported", C.c_int32),
        ("total_mem", C.c_int64),
    ]


class HeapInfo(C.Structure):
    _fields_ = [
        ("window_base", C.c_uint64),
        ("stride", C.c_uint64),
        ("mc_base", C.c_uint64),
        ("requested_size", C.c_uint64),
        ("granularity", C.c_uint64),
        ("rank", C.c_int32),
        ("world_size", C.c_int32),
        ("device", C.c_int32),
        ("mode", C.c_int32),
        ("transport", C.c_int32),
        ("nvls_bound", C.c_int32),
    ]


class GemmDesc(C.Structure):
    _fields_ = [
        ("mode", C.c_int32),
        ("dtype", C.c_int32),
        ("b_kmajor", C.c_int32),
        ("epi_op", C.c_int32),
        ("push_mode", C.c_int32),
        ("rank", C.c_int32),
        ("world_size", C.c_int32),
        ("split_axis", C.c_int32),
        ("a_rows", C.c_int64),
        ("b_cols", C.c_int64),
        ("k", C.c_int64),
        ("a_ptr", C.c_uint64),
        ("lda", C.c_int64),
        ("b_ptr", C.c_uint64),
        ("ldb", C.c_int64),
        ("sub_m", C.c_int64),
        ("sub_n", C.c_int64),
        ("out_ptr", C.c_uint64 * MAX_RANKS),
        ("out_mc_ptr", C.c_uint64),
        ("ldo", C.c_int64),
        ("out_rows", C.c_int64),
        ("out_cols", C.c_int64),
        ("out_slot_elems", C.c_int64),
        ("out_slots", C.c_int32),
        ("group_m_tiles", C.c_int32),
        ("sig_local", C.c_uint64),
        ("heap_stride", C.c_int64),
        ("sig_stride", C.c_int32),
        ("rot_m_tiles", C.c_int32),
        ("stage_local", C.c_uint64),
        ("a_gate", C.c_uint64),
        ("a_gate_rows_per_rank", C.c_int32),
        ("ag_src", C.c_uint64),
        ("ag_dst", C.c_uint64),
        ("ag_mc_dst", C.c_uint64),
        ("ag_bytes", C.c_uint64),
        ("scatter_col_begin", C.c_int32),
        ("scatter_col_end", C.c_int32),
        ("grid", C.c_int32),
        ("stats", C.c_uint64),
        ("status", C.c_uint64),
        ("trace", C.c_uint64),
        ("wait_budget_ns", C.c_uint64),
        ("tuning", C.c_int32),
        ("rs_own_lag", C.c_int32),
        ("ident_ptr", C.c_uint64),
        ("disable_cta_pairs", C.c_int32),
        ("comm_ctas", C.c_int32),
        ("dynamic_tiles", C.c_int32),
        ("reserved0", C.c_int32),
        ("entry_local", C.c_uint64),
    ]


STREAM_MAX_RANGES = 64


class StreamChunk(C.Structure):
    _fields_ = [
        ("tile_begin", C.c_int32),
        ("tile_end", C.c_int32),
        ("n_ranges", C.c_int32),
        ("reserved", C.c_int32),
        ("dst", C.c_uint64 * STREAM_MAX_RANGES),
        ("src", C.c_uint64 * STREAM_MAX_RANGES),
        ("bytes", C.c_uint64 * STREAM_MAX_RANGES),
    ]


class GemmPlanInfo(C.Structure):
    _fields_ = [
        ("grid", C.c_int32),
        ("tiles_total", C.c_int32),
        ("tiles_per_owner", C.c_int32),
        ("m_tiles_local", C.c_int32),
        ("n_tiles_local", C.c_int32),
        ("groups", C.c_int32),
        ("k_blocks", C.c_int32),
        ("smem_bytes", C.c_int32),
        ("push_grid", C.c_int32),
        ("pair_kernel", C.c_int32),
        ("pair_grid", C.c_int32),
        ("trace_words", C.c_int64),
    ]


_lib = None
_lib_lock = threading.Lock()


def lib_path() -> Path:
    """The shared object to load: ``TILECCL_NATIVE_LIB`` names another build of it,
    ``TILECCL_DEBUG=1`` selects the build with recorded bounds checks."""
    from .utils.config import current

    cfg = current()
    if cfg.native_lib:
        return Path(cfg.native_lib)
    return _build.DEBUG_LIB_PATH if cfg.debug else _build.LIB_PATH


def _declare(lib: C.CDLL) -> None:
    u64, i32, u32, vp = C.c_uint64, C.c_int32, C.c_uint32, C.c_void_p
    lib.tccl_last_error.restype = C.c_char_p
    lib.tccl_version.restype = C.c_char_p
    sigs = {
        "tccl_gemm_plan_create": [C.POINTER(GemmDesc), C.POINTER(vp)],
        "tccl_gemm_plan_info": [vp, C.POINTER(GemmPlanInfo)],
        "tccl_gemm_plan_launch": [vp, u32, u32, i32, i32, i32, u64],
        "tccl_gemm_plan_launch_streamed": [vp, u32, u32, i32, C.POINTER(StreamChunk), i32, u64, u64,
                                           u64],
        "tccl_gemm_plan_destroy": [vp],
        "tccl_wait_groups": [u64, i32, i32, i32, u64, u32, i32, u64, u64, i32, u64],
        "tccl_device_count": [C.POINTER(i32)],
        "tccl_device_props": [i32, C.POINTER(DeviceProps)],
        "tccl_peer_matrix": [i32, C.POINTER(i32), C.POINTER(i32)],
        "tccl_heap_create_local": [i32, u64, C.POINTER(i32), i32, C.POINTER(vp)],
        "tccl_heap_create_multiprocess": [i32, i32, u64, i32, C.c_char_p, i32, i32, C.POINTER(vp)],
        "tccl_heap_info": [vp, C.POINTER(HeapInfo)],
        "tccl_heap_destroy": [vp],
        "tccl_heap_alloc": [vp, u64, C.POINTER(u64)],
        "tccl_heap_reset": [vp],
        "tccl_heap_bytes_allocated": [vp, C.POINTER(u64)],
        "tccl_collective_launch": [i32, i32, i32, i32, i32, i32, i32, i32, u32, u64, u64, u64, u64, u64,
                                   u64, u64, C.c_int64, u64, i32, u64, u64, u64],
        "tccl_prim_test": [i32, i32, i32, i32, i32, u64, u64, u64, u64, u64, u64, u32, u32, u64, u64,
                           u64],
        "tccl_collective_ll_launch": [i32, i32, i32, i32, i32, i32, u32, u64, u64, u64, u64,
                                      C.c_int64, u64, u64, i32, u64, u64, u64],
        "tccl_p2p_copy": [i32, i32, i32, i32, u64, u64, u64, u64, u64, i32, u64],
        "tccl_broadcast_relay_launch": [i32, i32, i32, i32, u32, u64, u64, u64, u64, u64, u64,
                                        C.c_int64, i32, i32, u64, u64, u64],
        "tccl_debug_read_primitives": [vp, i32],
        "tccl_debug_read_collectives": [vp, i32],
        "tccl_push_region": [u64, u64, C.c_int64, i32, i32, i32, i32, i32, C.c_int64, u64, u32, u64,
                             u32, i32, i32, u64, u64, u64],
        "tccl_plan_tile_groups": [C.c_int64, C.c_int64, C.c_int64, C.c_int64, i32, i32, i32, i32,
                                  C.c_int64, C.POINTER(C.c_int64), i32, C.POINTER(C.c_int64), i32,
                                  C.POINTER(i32)],
        "tccl_plan_group_table": [C.c_int64, C.c_int64, C.POINTER(C.c_int64), i32, i32, i32, i32,
                                  C.POINTER(i32), C.c_int64],
        "tccl_emul_gemm_allgather": [i32, i32, i32, i32, C.c_void_p, C.c_void_p, C.c_void_p, i32, i32,
                                     i32, i32, i32, i32, i32, C.POINTER(i32)],
        "tccl_emul_gemm_reducescatter": [i32, i32, i32, i32, C.c_void_p, C.c_void_p, C.c_void_p, i32,
                                         i32, i32, i32, i32, i32, i32, C.POINTER(i32)],
        "tccl_emul_gemm_reducescatter_ex": [i32, i32, i32, i32, C.c_void_p, C.c_void_p, C.c_void_p, i32,
                                            i32, i32, i32, i32, i32, i32, i32, i32, i32, C.POINTER(i32)],
        "tccl_preload_kernels": [],
        "tccl_plan_tile_order": [i32, i32, i32, i32, i32, i32, C.POINTER(i32), i32],
        "tccl_plan_tile_order_ex": [i32, i32, i32, i32, i32, i32, i32, C.POINTER(i32), i32],
        "tccl_bootstrap_allgather": [i32, i32, C.c_char_p, i32, u64, i32, C.POINTER(u64),
                                     C.POINTER(i32)],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = C.c_int


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first if necessary) the native library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not path.exists():
            from .utils.config import current

            if not build_if_missing or current().no_build:
                raise NativeError("load", -1, f"{path} is missing; run `python -m tileccl_b200._build`")
            _build.build(debug=(path == _build.DEBUG_LIB_PATH))
        lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
        _declare(lib)
        _lib = lib
        return lib


def available() -> bool:
    try:
        load()
        return True
    except Exception:
        return False


def check(fn_name: str, code: int) -> None:
    if code != 0:
        msg = load().tccl_last_error()
        raise NativeError(fn_name, code, msg.decode("utf-8", "replace") if msg else "")


def call(fn_name: str, *args) -> None:
    """Call ``lib.<fn_name>(*args)`` and raise :class:`NativeError` on failure."""
    fn = getattr(load(), fn_name, None)
    if fn is None:
        raise NativeError(fn_name, -1, "symbol not present in this build of libtileccl_b200")
    check(fn_name, fn(*args))


def version() -> str:
    return load().tccl_version().decode()
