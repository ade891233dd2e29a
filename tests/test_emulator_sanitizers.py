"""The CPU emulation of the fused operators' protocol under ThreadSanitizer and
AddressSanitizer + UBSan (tests/native/emul_sanitize.cc): the on-record sanitizer run of
the signalling protocol, since no device-side sanitizer is available for the kernels."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "tests", "native", "emul_sanitize.cc")
EMULATOR = os.path.join(ROOT, "tileccl_b200", "csrc", "cpu_emul", "fake_device.cc")


def _cuda_include() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "include", "cuda.h")):
            return os.path.join(cand, "include")
    pytest.skip("cuda.h not found (the emulator's error header includes it)")


def _sanitizer_works(flag: str, tmp_path) -> bool:
    src = tmp_path / "probe.cc"
    src.write_text("int main() { return 0; }\n")
    exe = tmp_path / "probe"
    ok = subprocess.run(["g++", f"-fsanitize={flag}", str(src), "-o", str(exe)],
                        capture_output=True).returncode == 0
    return ok and subprocess.run([str(exe)], capture_output=True).returncode == 0


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not installed")
@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_emulated_ranks_are_clean_under_sanitizers(sanitizer, tmp_path):
    if not _sanitizer_works(sanitizer, tmp_path):
        pytest.skip(f"-fsanitize={sanitizer} does not work with this toolchain")
    exe = tmp_path / "emul_sanitize"
    build = subprocess.run(
        ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer",
         "-I", _cuda_include(), DRIVER, EMULATOR, "-lpthread", "-o", str(exe)],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66",
               ASAN_OPTIONS="detect_leaks=1 exitcode=67", UBSAN_OPTIONS="halt_on_error=1")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    out = run.stdout + run.stderr
    assert run.returncode == 0, out[-4000:]
    assert "all cases ok" in run.stdout
    assert "ThreadSanitizer" not in out and "AddressSanitizer" not in out and "runtime error" not in out
