"""Where benchmark results live and whether the machine was quiet enough to trust them.

Mirrors the helpers of the reference (tileccl/utils/benchmark_results.py:17-407):
canonical ``figures/data/*_latest.json`` paths guarded by a file lock, JSON
read/write, a pre-run snapshot of what else is running on the GPUs (they are
shared), and runtime metadata / support snapshots to embed in result files.
All GPU queries are read-only.
"""

from __future__ import annotations

import contextlib
import fcntl
import json
import os
import shutil
import subprocess
import time
from pathlib import Path
from typing import Any, Iterator, Optional


def project_root() -> Path:
    return Path(__file__).resolve().parents[2]


def figures_data_dir() -> Path:
    return project_root() / "figures" / "data"


def _latest(name: str) -> Path:
    return figures_data_dir() / f"{name}_latest.json"


def default_pattern_benchmark_path() -> Path:
    return _latest("pattern_overlap")


def default_gemm_benchmark_path() -> Path:
    return _latest("gemm")


def default_p2p_benchmark_path() -> Path:
    return _latest("p2p")


def default_collective_comm_only_benchmark_path() -> Path:
    return _latest("collective_comm_only")


def default_collective_bulk_sync_benchmark_path() -> Path:
    return _latest("collective_bulk_sync")


def default_fused_gate_benchmark_path() -> Path:
    return _latest("fused_gates")


def canonical_benchmark_lock_path() -> Path:
    return figures_data_dir() / ".canonical_benchmark.lock"


def is_canonical_benchmark_output(path) -> bool:
    p = Path(path).resolve()
    return p.parent == figures_data_dir().resolve() and p.name.endswith("_latest.json")


@contextlib.contextmanager
def acquire_canonical_benchmark_lock(timeout_s: float = 600.0, poll_s: float = 0.5) -> Iterator[Path]:
    """Exclusive lock for runs that overwrite the canonical result files."""
    lock_path = canonical_benchmark_lock_path()
    lock_path.parent.mkdir(parents=True, exist_ok=True)
    deadline = time.monotonic() + timeout_s
    with open(lock_path, "a+") as fh:
        while True:
            try:
                fcntl.flock(fh.fileno(), fcntl.LOCK_EX | fcntl.LOCK_NB)
                break
            except BlockingIOError:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"another canonical benchmark run holds {lock_path}") from None
                time.sleep(poll_s)
        try:
            fh.seek(0)
            fh.truncate()
            fh.write(json.dumps({"pid": os.getpid(), "since": time.time()}))
            fh.flush()
            yield lock_path
        finally:
            fcntl.flock(fh.fileno(), fcntl.LOCK_UN)


@contextlib.contextmanager
def canonical_benchmark_run(output_path, **lock_kwargs) -> Iterator[None]:
    """Take the lock only when ``output_path`` is one of the canonical files."""
    if is_canonical_benchmark_output(output_path):
        with acquire_canonical_benchmark_lock(**lock_kwargs):
            yield
    else:
        yield


def write_json(path, payload: dict) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(payload, indent=2, default=str))
    tmp.replace(path)
    return path


def read_json(path) -> dict:
    return json.loads(Path(path).read_text())


def _nvidia_smi_csv_query(scope: str, fields: str, timeout_s: float = 10.0) -> Optional[list]:
    exe = shutil.which("nvidia-smi")
    if exe is None:
        return None
    try:
        out = subprocess.run([exe, f"--query-{scope}={fields}", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=timeout_s)
    except (OSError, subprocess.TimeoutExpired):
        return None
    if out.returncode != 0:
        return None
    return [[c.strip() for c in line.split(",")] for line in out.stdout.strip().splitlines() if line]


def _parse_optional_int(value: Optional[str]) -> Optional[int]:
    try:
        return int(float(value)) if value not in (None, "", "N/A", "[N/A]") else None
    except ValueError:
        return None


def _numeric_visible_gpu_indices() -> Optional[list]:
    raw = os.environ.get("CUDA_VISIBLE_DEVICES")
    if raw is None or not raw.strip():
        return None
    try:
        return [int(x) for x in raw.split(",") if x.strip()]
    except ValueError:
        return None  # UUID form: cannot be matched to indices here


def benchmark_environment_health(*, max_util_percent: int = 5, own_pid: Optional[int] = None) -> dict:
    """Snapshot of other activity on the visible GPUs before a run.

    ``contaminated`` is true when a compute process other than this one is
    resident, or when a GPU already shows utilisation above ``max_util_percent``.
    """
    own_pid = own_pid or os.getpid()
    gpus = _nvidia_smi_csv_query("gpu", "index,utilization.gpu,memory.used,clocks.sm,clocks.max.sm")
    procs = _nvidia_smi_csv_query("compute-apps", "pid,used_memory,gpu_uuid")
    if gpus is None:
        return {"available": False, "contaminated": False, "reason": "nvidia-smi not available",
                "gpus": [], "foreign_processes": []}
    visible = _numeric_visible_gpu_indices()
    gpu_rows, busy = [], []
    for row in gpus:
        idx = _parse_optional_int(row[0])
        if visible is not None and idx not in visible:
            continue
        util = _parse_optional_int(row[1])
        rec = {"index": idx, "utilization_percent": util, "memory_used_mib": _parse_optional_int(row[2]),
               "sm_mhz": _parse_optional_int(row[3]), "sm_max_mhz": _parse_optional_int(row[4])}
        gpu_rows.append(rec)
        if util is not None and util > max_util_percent:
            busy.append(idx)
    foreign = []
    for row in procs or []:
        pid = _parse_optional_int(row[0])
        if pid is not None and pid != own_pid:
            foreign.append({"pid": pid, "used_memory_mib": _parse_optional_int(row[1]),
                            "gpu_uuid": row[2] if len(row) > 2 else None})
    return {"available": True, "contaminated": bool(busy or foreign), "busy_gpus": busy,
            "gpus": gpu_rows, "foreign_processes": foreign, "visible_devices": visible,
            "max_util_percent": max_util_percent}


def emit_benchmark_environment_warnings(health: dict, *, printer=print) -> None:
    if not health.get("available"):
        printer(f"[env] GPU state unknown: {health.get('reason')}")
        return
    if health.get("busy_gpus"):
        printer(f"[env] GPUs already busy before the run: {health['busy_gpus']}")
    if health.get("foreign_processes"):
        printer(f"[env] other compute processes resident: {health['foreign_processes']}")


def runtime_support_snapshot(ctx: Any) -> dict:
    return ctx.support_matrix().to_dict()


def runtime_metadata_snapshot(ctx: Any) -> dict:
    meta = ctx.runtime_metadata()
    heap = meta.get("heap")
    if heap:  # the peer tables are long and not useful in result files
        for key in ("peer_exports", "peer_imports", "peer_memory_map", "segments"):
            heap.pop(key, None)
    return meta


def describe_runtime_support_snapshot(ctx: Any = None) -> dict:
    from ..support import describe_runtime_support

    return describe_runtime_support(ctx).to_dict()


def describe_runtime_metadata_snapshot(ctx: Any = None) -> dict:
    if ctx is not None:
        return runtime_metadata_snapshot(ctx)
    from .. import __version__

    return {"version": __version__, "context": None}
