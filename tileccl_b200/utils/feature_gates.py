"""Which runtime combinations device-side collectives are validated for.

Function and environment-variable names follow the reference
(tileccl/utils/feature_gates.py:8-186).  There the validated multi-process surface
is one transport (``ctypes_ipc``) at world size 2 and device collectives hide
behind an opt-in variable.  Here device collectives are the only implementation,
validated for the VMM transports at world sizes 1, 2, 4 and 8, so the opt-in
variable is accepted but not required.
"""

from __future__ import annotations

from typing import Optional

_TRUTHY_VALUES = {"1", "true", "yes", "on"}

MULTIPROCESS_DEVICE_COLLECTIVES_ENV = "TileCCL_ENABLE_EXPERIMENTAL_MULTIPROCESS_DEVICE_COLLECTIVES"
FORCE_MULTIPROCESS_TRANSPORT_ENV = "TileCCL_FORCE_MULTIPROCESS_TRANSPORT"

_MULTIPROCESS_TRANSPORT_VALUES = {"auto", "vmm_fd", "vmm_fabric"}
# names the reference understands, mapped onto what exists here
_LEGACY_TRANSPORT_ALIASES = {"ctypes_ipc": "vmm_fd", "pytorch_ipc": "vmm_fd",
                             "peer_access_pointer_exchange": "vmm_fd"}
_VALIDATED_MULTIPROCESS_DEVICE_TRANSPORTS = {"vmm_fd", "vmm_single_process", "local_only"}
_VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES = {1, 2, 4, 8}


def multiprocess_device_validated_public_surface() -> dict:
    return {"transports": sorted(_VALIDATED_MULTIPROCESS_DEVICE_TRANSPORTS),
            "world_sizes": sorted(_VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES),
            "transport": "vmm_fd", "world_size": max(_VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES)}


def multiprocess_device_collectives_enabled() -> bool:
    """Always true here; the variable only matters to code that checks it explicitly."""
    return True


def multiprocess_device_collectives_requested() -> bool:
    """Whether the opt-in variable of the reference is set to a truthy value."""
    from .config import current

    return current().experimental_multiprocess_device_collectives


def forced_multiprocess_transport() -> Optional[str]:
    """Transport forced through the environment, or ``None`` for automatic choice."""
    from .config import current

    raw = current().force_multiprocess_transport
    if raw is None or not raw.strip():
        return None
    value = raw.strip().lower()
    value = _LEGACY_TRANSPORT_ALIASES.get(value, value)
    if value not in _MULTIPROCESS_TRANSPORT_VALUES:
        raise ValueError(f"{FORCE_MULTIPROCESS_TRANSPORT_ENV}={raw!r} is not one of "
                         f"{sorted(_MULTIPROCESS_TRANSPORT_VALUES | set(_LEGACY_TRANSPORT_ALIASES))}")
    if value == "vmm_fabric":
        raise ValueError("vmm_fabric handles need an IMEX domain (multi-node NVLink); this build "
                         "exchanges POSIX file descriptors inside one node")
    return None if value == "auto" else value


def multiprocess_device_remote_access_transport_supported(transport_strategy: str) -> bool:
    return transport_strategy in _VALIDATED_MULTIPROCESS_DEVICE_TRANSPORTS


def multiprocess_device_remote_access_runtime_supported(*, transport_strategy: str,
                                                        world_size: int) -> bool:
    return (multiprocess_device_remote_access_transport_supported(transport_strategy)
            and world_size in _VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES)


def multiprocess_device_remote_access_detail(*, transport_strategy: str,
                                             world_size: Optional[int] = None,
                                             operation: str = "this operation") -> str:
    ok_t = multiprocess_device_remote_access_transport_supported(transport_strategy)
    ok_w = world_size is None or world_size in _VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES
    if ok_t and ok_w:
        return (f"{operation}: device-side remote access is validated for transport "
                f"{transport_strategy!r}" + (f" at world_size {world_size}" if world_size else ""))
    why = []
    if not ok_t:
        why.append(f"transport {transport_strategy!r} is not one of "
                   f"{sorted(_VALIDATED_MULTIPROCESS_DEVICE_TRANSPORTS)}")
    if not ok_w:
        why.append(f"world_size {world_size} is not one of "
                   f"{sorted(_VALIDATED_MULTIPROCESS_DEVICE_WORLD_SIZES)}")
    return f"{operation} cannot use device-side remote access: " + "; ".join(why)


def multiprocess_device_collectives_transport_supported(transport_strategy: str) -> bool:
    return multiprocess_device_remote_access_transport_supported(transport_strategy)


def multiprocess_device_collectives_runtime_supported(*, transport_strategy: str,
                                                      world_size: int) -> bool:
    return multiprocess_device_remote_access_runtime_supported(
        transport_strategy=transport_strategy, world_size=world_size)


def multiprocess_device_collectives_detail(*, transport_strategy: str, world_size: int,
                                           operation: str = "device collectives") -> str:
    return multiprocess_device_remote_access_detail(transport_strategy=transport_strategy,
                                                    world_size=world_size, operation=operation)
