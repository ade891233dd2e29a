"""The user-kernel path builds without a GPU: headers are self-contained and nvcc accepts the example."""
import os
import shutil

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                    reason="nvcc not installed")
def test_example_kernel_compiles_against_the_device_headers():
    from tileccl_b200 import userkernel

    mod = userkernel.compile(os.path.join(ROOT, "examples", "custom_kernel.cu"))
    assert mod.path.exists() and mod.path.suffix == ".so"
    assert (userkernel.include_dir() / "tile_collectives.cuh").exists()


def test_device_api_names_point_at_real_functions():
    from tileccl_b200 import userkernel
    from tileccl_b200.primitives import device_api as d

    for name in d.COLLECTIVE_DEVICE:
        prim = getattr(d, name)
        assert prim.header == "tile_collectives.cuh"
        text = (userkernel.include_dir() / prim.header).read_text()
        assert f" {name}(" in text, name
    with pytest.raises(RuntimeError, match="userkernel"):
        d.tile_allreduce()


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                    reason="nvcc not installed")
def test_example_kernel_compiles_with_the_recorded_bounds_checks():
    from tileccl_b200 import userkernel

    rel = userkernel.compile(os.path.join(ROOT, "examples", "custom_kernel.cu"))
    dbg = userkernel.compile(os.path.join(ROOT, "examples", "custom_kernel.cu"), debug=True)
    assert dbg.path != rel.path and dbg.path.exists()
    assert dbg._debug_read is not None and rel._debug_read is not None
