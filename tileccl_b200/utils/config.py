"""Every environment switch of the library in one frozen snapshot.

The reference reads two environment variables in ``tileccl/utils/feature_gates.py:10-11``
and takes everything else as keyword arguments; here the knobs that tune the sm_100a
kernels are environment variables as well, and ``RuntimeConfig.from_env()`` is the one
place that lists them (``python -m tileccl info`` prints it).
"""

from __future__ import annotations

import os
from dataclasses import asdict, dataclass
from typing import Mapping, Optional


def _flag(env: Mapping[str, str], name: str, default: bool = False) -> bool:
    v = env.get(name)
    if v is None or v == "":
        return default
    return v not in ("0", "false", "False", "no")


def _opt_int(env: Mapping[str, str], name: str) -> Optional[int]:
    v = env.get(name)
    return int(v) if v not in (None, "") else None


@dataclass(frozen=True)
class RuntimeConfig:
    # fused GEMM + collective kernel
    push_mode: str = "tma"                 # TILECCL_PUSH_MODE: tma | stores | multimem
    tuning: int = 1                        # TILECCL_TUNING: bit 0 = relaxed signal after a completed bulk store
    gemm_cta_pairs: bool = True            # TILECCL_GEMM_2SM: whole-order launches on CTA pairs
    rs_own_lag: Optional[int] = None       # TILECCL_RS_OWN_LAG: rounds the own rows trail (None = heuristic)
    wait_budget_us: Optional[float] = None  # TILECCL_WAIT_BUDGET_US: budget of every device wait (None = 2 s)
    # NVLS / multicast
    disable_nvls: bool = False             # TILECCL_DISABLE_NVLS
    force_nvls: bool = False               # TILECCL_FORCE_NVLS: also with two ranks
    # planning, bootstrap, build
    calibration: Optional[str] = None      # TILECCL_CALIBRATION: link-model JSON (default: calibration/b200.json)
    bootstrap_timeout_ms: Optional[int] = None  # TILECCL_BOOTSTRAP_TIMEOUT_MS
    native_lib: Optional[str] = None       # TILECCL_NATIVE_LIB: another build of the shared object
    # feature gates kept from the reference
    experimental_multiprocess_device_collectives: bool = False
    force_multiprocess_transport: Optional[str] = None

    @classmethod
    def from_env(cls, env: Optional[Mapping[str, str]] = None) -> "RuntimeConfig":
        e = os.environ if env is None else env
        push = (e.get("TILECCL_PUSH_MODE") or "tma").lower()
        if push not in ("tma", "stores", "multimem"):
            raise ValueError(f"TILECCL_PUSH_MODE must be tma, stores or multimem, got {push!r}")
        budget = e.get("TILECCL_WAIT_BUDGET_US")
        return cls(
            push_mode=push,
            tuning=int(e.get("TILECCL_TUNING") or 1),
            gemm_cta_pairs=_flag(e, "TILECCL_GEMM_2SM", True),
            rs_own_lag=_opt_int(e, "TILECCL_RS_OWN_LAG"),
            wait_budget_us=float(budget) if budget not in (None, "") else None,
            disable_nvls=_flag(e, "TILECCL_DISABLE_NVLS"),
            force_nvls=_flag(e, "TILECCL_FORCE_NVLS"),
            calibration=e.get("TILECCL_CALIBRATION") or None,
            bootstrap_timeout_ms=_opt_int(e, "TILECCL_BOOTSTRAP_TIMEOUT_MS"),
            native_lib=e.get("TILECCL_NATIVE_LIB") or None,
            experimental_multiprocess_device_collectives=_flag(
                e, "TileCCL_ENABLE_EXPERIMENTAL_MULTIPROCESS_DEVICE_COLLECTIVES"),
            force_multiprocess_transport=e.get("TileCCL_FORCE_MULTIPROCESS_TRANSPORT") or None,
        )

    def to_dict(self) -> dict:
        return asdict(self)
