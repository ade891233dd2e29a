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
    call_stats: bool = True                # TILECCL_STATS: fused kernels add per-call counters (ops.call_stats)
    dynamic_tiles: bool = False            # TILECCL_DYNAMIC_TILES: tiles handed to CTAs from a global counter
    rs_cta_pairs: Optional[bool] = None    # TILECCL_RS_CTA_PAIRS: kernel form of a multi-rank reduce-scatter (None = measured choice)
    rs_own_lag: Optional[int] = None       # TILECCL_RS_OWN_LAG: rounds the own rows trail (None = heuristic)
    wait_budget_us: Optional[float] = None  # TILECCL_WAIT_BUDGET_US: budget of every device wait (None = 2 s)
    # NVLS / multicast
    disable_nvls: bool = False             # TILECCL_DISABLE_NVLS
    force_nvls: bool = False               # TILECCL_FORCE_NVLS: also with two ranks
    # planning, bootstrap, build
    calibration: Optional[str] = None      # TILECCL_CALIBRATION: link-model JSON (default: calibration/b200.json)
    bootstrap_timeout_ms: Optional[int] = None  # TILECCL_BOOTSTRAP_TIMEOUT_MS
    native_lib: Optional[str] = None       # TILECCL_NATIVE_LIB: another build of the shared object
    no_build: bool = False                 # TILECCL_NO_BUILD: never compile the shared object on import
    debug: bool = False                    # TILECCL_DEBUG: load the build with recorded bounds checks and check every collective call
    stream_run_shares: Optional[tuple] = None  # TILECCL_STREAM_SHARES: "0.85,0.15" - runs of a host-streamed operand
    stream_copy_streams: int = 1           # TILECCL_STREAM_COPY_STREAMS: copy streams of a host-streamed operand (1 | 2)
    ll_max_bytes: int = 1 << 20            # TILECCL_LL_MAX_BYTES: largest per-peer message of the low-latency collectives (0 = off, at most 1 MiB)
    bcast_relay_min_bytes: int = 256 << 20  # TILECCL_BCAST_RELAY_MIN_BYTES: from this size a broadcast on >= 3 ranks is relayed piece by piece (0 = never)
    bcast_relay_piece_kib: int = 64        # TILECCL_BCAST_RELAY_PIECE_KIB: largest piece of a relayed broadcast (16 .. 1024 KiB; grows only to keep the piece count within 16384)
    bcast_relay_root_workers: int = 148    # TILECCL_BCAST_RELAY_ROOT_WORKERS: copy pipelines the root runs (few, so that each piece completes soon and the relays start early)
    bcast_relay_ctas_per_sm: int = 1       # TILECCL_BCAST_RELAY_CTAS_PER_SM: CTAs per SM of the relay kernel (1 .. 4)
    bcast_relay_bulk: bool = False         # TILECCL_BCAST_RELAY_BULK: 1 = bulk copies through shared memory instead of register copies (measured slower once its flags are release stores)
    comm_sms: Optional[int] = None         # TILECCL_COMM_SMS: SMs of a fused launch that only communicate (None = policy)
    push_mode_explicit: bool = False       # TILECCL_PUSH_MODE was set (it then overrides a pattern's own choice)
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
            call_stats=_flag(e, "TILECCL_STATS", True),
            dynamic_tiles=_flag(e, "TILECCL_DYNAMIC_TILES", False),
            rs_cta_pairs=(None if e.get("TILECCL_RS_CTA_PAIRS") in (None, "")
                          else _flag(e, "TILECCL_RS_CTA_PAIRS")),
            rs_own_lag=_opt_int(e, "TILECCL_RS_OWN_LAG"),
            wait_budget_us=float(budget) if budget not in (None, "") else None,
            disable_nvls=_flag(e, "TILECCL_DISABLE_NVLS"),
            force_nvls=_flag(e, "TILECCL_FORCE_NVLS"),
            calibration=e.get("TILECCL_CALIBRATION") or None,
            bootstrap_timeout_ms=_opt_int(e, "TILECCL_BOOTSTRAP_TIMEOUT_MS"),
            native_lib=e.get("TILECCL_NATIVE_LIB") or None,
            no_build=_flag(e, "TILECCL_NO_BUILD"),
            debug=_flag(e, "TILECCL_DEBUG"),
            stream_run_shares=(tuple(float(x) for x in e["TILECCL_STREAM_SHARES"].split(","))
                               if e.get("TILECCL_STREAM_SHARES") else None),
            stream_copy_streams=2 if (e.get("TILECCL_STREAM_COPY_STREAMS") or "1") == "2" else 1,
            ll_max_bytes=min(1 << 20, max(0, int(e.get("TILECCL_LL_MAX_BYTES") or (1 << 20)))),
            bcast_relay_min_bytes=max(0, int(e["TILECCL_BCAST_RELAY_MIN_BYTES"]) if e.get("TILECCL_BCAST_RELAY_MIN_BYTES") not in (None, "") else (256 << 20)),
            bcast_relay_piece_kib=min(1024, max(16, int(e.get("TILECCL_BCAST_RELAY_PIECE_KIB") or 64))),
            bcast_relay_root_workers=max(4, int(e.get("TILECCL_BCAST_RELAY_ROOT_WORKERS") or 148)),
            bcast_relay_ctas_per_sm=min(4, max(1, int(e.get("TILECCL_BCAST_RELAY_CTAS_PER_SM") or 1))),
            bcast_relay_bulk=_flag(e, "TILECCL_BCAST_RELAY_BULK", False),
            comm_sms=_opt_int(e, "TILECCL_COMM_SMS"),
            push_mode_explicit=bool(e.get("TILECCL_PUSH_MODE")),
            experimental_multiprocess_device_collectives=(
                (e.get("TileCCL_ENABLE_EXPERIMENTAL_MULTIPROCESS_DEVICE_COLLECTIVES") or "")
                .strip().lower() in ("1", "true", "yes", "on")),
            force_multiprocess_transport=e.get("TileCCL_FORCE_MULTIPROCESS_TRANSPORT") or None,
        )

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def wait_budget_ns(self) -> int:
        """Budget of every device-side wait in nanoseconds; 0 = the kernels' default (2 s)."""
        return int(self.wait_budget_us * 1000) if self.wait_budget_us else 0

    @property
    def nvls_allowed(self) -> bool:
        return not self.disable_nvls


# Every variable from_env() looks at.  current() compares their raw values with those of the
# last snapshot, so a launch pays a couple of microseconds instead of a full parse.
ENV_NAMES = (
    "TILECCL_PUSH_MODE", "TILECCL_TUNING", "TILECCL_GEMM_2SM", "TILECCL_STATS",
    "TILECCL_DYNAMIC_TILES", "TILECCL_RS_CTA_PAIRS", "TILECCL_RS_OWN_LAG",
    "TILECCL_WAIT_BUDGET_US", "TILECCL_DISABLE_NVLS", "TILECCL_FORCE_NVLS", "TILECCL_CALIBRATION",
    "TILECCL_BOOTSTRAP_TIMEOUT_MS", "TILECCL_NATIVE_LIB", "TILECCL_NO_BUILD", "TILECCL_DEBUG",
    "TILECCL_STREAM_SHARES", "TILECCL_STREAM_COPY_STREAMS", "TILECCL_LL_MAX_BYTES",
    "TILECCL_BCAST_RELAY_MIN_BYTES", "TILECCL_BCAST_RELAY_PIECE_KIB",
    "TILECCL_BCAST_RELAY_ROOT_WORKERS",
    "TILECCL_BCAST_RELAY_CTAS_PER_SM", "TILECCL_BCAST_RELAY_BULK", "TILECCL_COMM_SMS",
    "TileCCL_ENABLE_EXPERIMENTAL_MULTIPROCESS_DEVICE_COLLECTIVES",
    "TileCCL_FORCE_MULTIPROCESS_TRANSPORT",
)
_ENV_KEYS_RAW = tuple(os.fsencode(n) for n in ENV_NAMES)
_cached: Optional[tuple] = None      # (fingerprint, RuntimeConfig)
_generation = 0                      # how many times the snapshot has been re-parsed


def _fingerprint() -> tuple:
    raw = getattr(os.environ, "_data", None)      # CPython on POSIX: bytes -> bytes
    if isinstance(raw, dict):
        return tuple(map(raw.get, _ENV_KEYS_RAW))
    return tuple(map(os.environ.get, ENV_NAMES))


def current() -> RuntimeConfig:
    """The configuration in force right now.  Every module of the library that depends on an
    environment switch asks here (nothing else reads ``TILECCL_*`` variables).  A variable
    set mid-program takes effect at the next plan or launch that consults it: the snapshot is
    re-parsed whenever the raw value of one of ``ENV_NAMES`` differs from the last call's."""
    global _cached, _generation
    fp = _fingerprint()
    c = _cached
    if c is not None and c[0] == fp:
        return c[1]
    cfg = RuntimeConfig.from_env()
    _cached = (fp, cfg)
    _generation += 1
    return cfg


def generation() -> int:
    """A number that changes whenever ``current()`` would return a different snapshot: part of
    the key of launchers that bake configuration-dependent choices in."""
    current()
    return _generation
