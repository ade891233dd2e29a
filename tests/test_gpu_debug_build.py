"""The debug build on a GPU: bounds violations are recorded and skipped, nothing faults."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def test_debug_build_records_and_skips_out_of_heap_accesses():
    env = dict(os.environ, TILECCL_DEBUG="1")
    env.pop("TILECCL_NATIVE_LIB", None)
    proc = subprocess.run([sys.executable, os.path.join(HERE, "debug_worker.py")], env=env,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "debug worker ok" in proc.stdout
