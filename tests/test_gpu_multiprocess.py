"""One process per GPU (torchrun): needs at least two GPUs, skipped otherwise."""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_multiprocess_ranks(ws):
    if not torch.cuda.is_available() or torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "MP_WORKER_OK" in out.stdout, (out.stdout[-3000:], out.stderr[-3000:])


@pytest.mark.parametrize("ws", [2, 4, 8])
def test_stress_thousands_of_calls_with_changing_inputs(ws):
    """Every result of 2000 back-to-back all-gather and reduce-scatter calls is checked on
    the device, with the relaxed and with the release form of the TileGroup signal."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_stress.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker, "--calls", "2000"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0 and "MP_STRESS_OK" in out.stdout, (out.stdout[-3000:], out.stderr[-3000:])


@pytest.mark.parametrize("ws", [2, 4])
def test_debug_mode_checks_every_collective_call(ws):
    """TILECCL_DEBUG=1: the library with recorded bounds checks, and after every collective
    call the status words, the bounds record and the epoch invariants of its counters."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_debug_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker]
    env = dict(os.environ, TILECCL_DEBUG="1")
    env.pop("TILECCL_NATIVE_LIB", None)
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0 and "MP_DEBUG_OK" in out.stdout, (out.stdout[-3000:], out.stderr[-3000:])


@pytest.mark.parametrize("bulk", [0, 1])
@pytest.mark.parametrize("ws", [4, 8])
def test_large_relayed_broadcasts_are_checked_call_by_call(ws, bulk):
    """512 MiB and 96 MiB broadcasts with alternating roots; every element of every call is
    compared on the device (a piece flag that overtakes its data would forward stale pieces)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < ws:
        pytest.skip(f"needs {ws} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_relay_stress.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ws}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), worker,
           "--bulk", str(bulk)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "MP_RELAY_OK" in out.stdout, (out.stdout[-3000:], out.stderr[-3000:])
