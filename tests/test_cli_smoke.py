"""The command line must work without a GPU."""

import json
import subprocess
import sys


def _run(*args):
    return subprocess.run([sys.executable, "-m", "tileccl", *args], capture_output=True, text=True,
                          timeout=300)


def test_help():
    out = _run("--help")
    assert out.returncode == 0
    assert "usage:" in out.stdout
    for sub in ("info", "support", "bench", "compare"):
        assert sub in out.stdout


def test_version():
    out = _run("--version")
    assert out.returncode == 0 and "tileccl_b200" in out.stdout


def test_info_runs():
    out = _run("info")
    assert out.returncode == 0
    assert "native library" in out.stdout


def test_support_json():
    out = _run("support", "--json")
    assert out.returncode == 0, out.stderr
    data = json.loads(out.stdout)
    assert {"context", "ops", "contracts", "execution_paths", "collectives", "memory"} <= set(data)
    assert data["ops"]["gemm_allgather"]["state"] in ("supported", "partial", "unsupported")
