"""Device layer.  One backend (CUDA on B200); ``backend="auto"`` and ``"cuda"``
are accepted everywhere for API parity with the reference's factory
(tileccl/backends/__init__.py:39-118), ``"hip"`` is rejected with a clear error.
"""

from __future__ import annotations

from .base import BackendInterface, DeviceProperties, TopologyInfo
from .cuda import CUDABackend

_BACKEND: CUDABackend | None = None


def detect_hardware() -> str:
    """``"cuda"`` when a CUDA device is visible, else ``"none"``."""
    try:
        import torch

        return "cuda" if torch.cuda.is_available() else "none"
    except Exception:
        return "none"


def get_backend(name: str = "auto", force: bool = False) -> CUDABackend:
    """Return the process-wide backend object.

    ``force=True`` skips the hardware check (used to build contexts for planning
    on a machine without a GPU).
    """
    global _BACKEND
    name = (name or "auto").lower()
    if name == "hip":
        raise ValueError("the HIP/ROCm backend is not part of this library: it targets NVIDIA B200 only")
    if name not in ("auto", "cuda"):
        raise ValueError(f"unknown backend {name!r}; expected 'auto' or 'cuda'")
    if not force and detect_hardware() != "cuda":
        raise RuntimeError("no CUDA device is visible; pass force_backend=True for host-only use")
    if _BACKEND is None:
        _BACKEND = CUDABackend()
    return _BACKEND


__all__ = ["BackendInterface", "CUDABackend", "DeviceProperties", "TopologyInfo",
           "detect_hardware", "get_backend"]
