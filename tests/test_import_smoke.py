"""Everything must import on a machine without a GPU or a CUDA driver."""

import importlib

import pytest


def test_package_imports_and_exposes_public_api():
    import tileccl_b200

    assert isinstance(tileccl_b200.__version__, str)
    for name in ("init", "init_local", "current_context", "get_rank", "get_world_size",
                 "describe_runtime_support", "TileCCLContext"):
        assert hasattr(tileccl_b200, name)
    assert callable(tileccl_b200.init) and callable(tileccl_b200.init_local)


@pytest.mark.parametrize("mod", [
    "tileccl_b200.ops", "tileccl_b200.patterns", "tileccl_b200.planning", "tileccl_b200.primitives",
    "tileccl_b200.sync", "tileccl_b200.memory", "tileccl_b200.utils", "tileccl_b200.models",
    "tileccl_b200.parallel", "tileccl_b200.kernels.fused_gemm", "tileccl_b200.backends",
    "tileccl_b200.support", "tileccl_b200.cli", "tileccl_b200.benchmarks", "tileccl_b200.emulation",
])
def test_submodules_import(mod):
    importlib.import_module(mod)


def test_reference_package_names_resolve_to_this_library():
    import tileccl
    import tileccl_b200
    import tileccl_v2

    assert tileccl.ops is tileccl_b200.ops
    assert tileccl.init is tileccl_b200.init
    assert tileccl.Tile is tileccl.SymmetricHeap
    from tileccl.memory.symmetric_heap import SymmetricHeap
    from tileccl.primitives import tile_put, tile_remote_load
    from tileccl.sync import tile_signal, tile_wait
    from tileccl_v2 import build_p2p_transport_plan, build_tile_group_plan, reduce_scatter_spec

    assert SymmetricHeap is tileccl_b200.memory.SymmetricHeap
    assert tileccl_v2.reduce_scatter_spec is reduce_scatter_spec
    with pytest.raises(RuntimeError):
        tile_put()  # device function: not callable from the host


def test_uninitialised_context_raises():
    import tileccl_b200

    saved = tileccl_b200._ctx
    tileccl_b200._ctx = None
    try:
        with pytest.raises(RuntimeError, match="not been initialised"):
            tileccl_b200.current_context()
        with pytest.raises(RuntimeError):
            tileccl_b200.get_rank()
    finally:
        tileccl_b200._ctx = saved


def test_init_argument_validation():
    import tileccl_b200

    with pytest.raises(ValueError):
        tileccl_b200.init(heap=object(), heap_size=1024, force_backend=True)
    with pytest.raises(ValueError):
        tileccl_b200.init(backend="hip", force_backend=True)
    with pytest.raises(ValueError):
        tileccl_b200.init_local(0, 1024)
    with pytest.raises(ValueError):
        tileccl_b200.init_local(2, 0)


def test_native_library_loads_without_gpu(native_lib):
    from tileccl_b200 import _native

    assert _native.version().startswith("0.1")
    n = __import__("ctypes").c_int32(-1)
    _native.call("tccl_device_count", __import__("ctypes").byref(n))
    assert n.value >= 0
