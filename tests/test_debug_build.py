"""Debug build (recorded bounds checks) and the per-call epoch invariants: host side."""

import ctypes as C

from tileccl_b200 import _build, debug
from tileccl_b200.utils.config import RuntimeConfig


def test_debug_record_layout_matches_the_device_struct():
    assert C.sizeof(debug.DebugRecord) == 40
    assert debug.DebugRecord.addr.offset == 24 and debug.DebugRecord.enabled.offset == 20


def test_debug_switch_selects_the_debug_library(monkeypatch):
    from tileccl_b200 import _native

    assert RuntimeConfig.from_env({}).debug is False
    assert RuntimeConfig.from_env({"TILECCL_DEBUG": "1"}).debug is True
    monkeypatch.delenv("TILECCL_NATIVE_LIB", raising=False)
    monkeypatch.setenv("TILECCL_DEBUG", "1")
    assert _native.lib_path() == _build.DEBUG_LIB_PATH
    monkeypatch.setenv("TILECCL_DEBUG", "0")
    assert _native.lib_path() == _build.LIB_PATH


def test_release_library_reports_checks_disabled():
    """The release build answers the reader calls with an empty, disabled record (no GPU
    needed: the release readers touch no device)."""
    from tileccl_b200 import _native

    lib = C.CDLL(str(_build.build()))
    rec = debug.DebugRecord(count=9, enabled=9)
    lib.tccl_debug_read_collectives.argtypes = [C.c_void_p, C.c_int32]
    assert lib.tccl_debug_read_collectives(C.byref(rec), 1) == 0
    assert rec.count == 0 and rec.enabled == 0
    assert _native is not None


def test_debug_library_builds_with_the_checks_compiled_in():
    path = _build.build(debug=True)
    assert path == _build.DEBUG_LIB_PATH and path.exists()
    lib = C.CDLL(str(path))
    assert hasattr(lib, "tccl_debug_read_primitives") and hasattr(lib, "tccl_collective_launch")


def test_epoch_invariants_all_to_all():
    ok = [0] * 32
    for src in (1, 2, 3):
        ok[src] = 5
        ok[8 + src] = 5
    assert debug.epoch_invariant_errors(ok, 5, 0, 4) == []
    ahead = list(ok)
    ahead[2] = 6                      # a faster peer already announced call 6
    assert debug.epoch_invariant_errors(ahead, 5, 0, 4) == []
    stale = list(ok)
    stale[8 + 3] = 4                  # rank 3 never completed call 5
    errs = debug.epoch_invariant_errors(stale, 5, 0, 4)
    assert len(errs) == 1 and "done[3] = 4" in errs[0]
    runaway = list(ok)
    runaway[1] = 9
    assert "ready[1] = 9" in debug.epoch_invariant_errors(runaway, 5, 0, 4)[0]


def test_epoch_invariants_rooted():
    # root 1 of 4 after call 3: it has seen everyone's announcement; nobody signals "done" to it
    root_block = [0] * 32
    for src in (0, 2, 3):
        root_block[src] = 3
    assert debug.epoch_invariant_errors(root_block, 3, 1, 4, root=1) == []
    # a receiver only sees the root's completion
    recv = [0] * 32
    recv[8 + 1] = 3
    assert debug.epoch_invariant_errors(recv, 3, 2, 4, root=1) == []
    recv[8 + 1] = 2
    assert "done[1] = 2" in debug.epoch_invariant_errors(recv, 3, 2, 4, root=1)[0]
    recv[8 + 1] = 3
    recv[0] = 1                       # an announcement that should have gone to the root
    assert "non-root" in debug.epoch_invariant_errors(recv, 3, 2, 4, root=1)[0]
