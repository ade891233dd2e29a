"""Command line: ``python -m tileccl`` / ``python -m tileccl_b200``.

Sub-commands as in the reference (tileccl/cli.py:492-597): ``info``, ``support``,
``bench [p2p|collective|pattern|gemm|all]``, ``compare``, ``--version``.  The
reference's ``bench <sub>`` shells out to scripts that are not part of its tree;
here every benchmark lives in ``tileccl_b200/benchmarks`` and runs in-process.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path
from typing import Optional


def _results_dir() -> Path:
    d = Path.home() / ".tileccl" / "benchmark_results"
    d.mkdir(parents=True, exist_ok=True)
    return d


def _save(name: str, payload: dict, output: Optional[str]) -> Path:
    path = Path(output) if output else _results_dir() / f"{name}_{int(time.time())}.json"
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(payload, indent=2, default=str))
    return path


def _handle_info(args) -> int:
    import tileccl_b200
    from tileccl_b200 import _native
    from tileccl_b200.backends import detect_hardware

    print(f"tileccl_b200 {tileccl_b200.__version__}")
    try:
        print(f"native library: {_native.lib_path()} ({_native.version()})")
    except Exception as exc:
        print(f"native library: unavailable ({exc})")
    try:
        from tileccl_b200.utils.config import RuntimeConfig

        cfg = RuntimeConfig.from_env().to_dict()
        print("config: " + ", ".join(f"{k}={v}" for k, v in cfg.items()))
    except ValueError as exc:
        print(f"config: invalid environment ({exc})")
    hw = detect_hardware()
    print(f"hardware: {hw}")
    if hw != "cuda":
        print("no CUDA device visible: planning, cost model and the CPU emulator still work")
        return 0
    try:
        from tileccl_b200.backends import get_backend
        from tileccl_b200.utils.topology import print_topology_info

        be = get_backend()
        for i in range(be.device_count()):
            p = be.get_device_properties(i)
            print(f"gpu{i}: {p.name} {p.arch} SMs={p.compute_units} mem={p.total_memory / 2**30:.0f} GiB "
                  f"L2={p.l2_cache_bytes / 2**20:.0f} MiB vmm={p.vmm_supported} fd={p.posix_fd_handles} "
                  f"fabric={p.fabric_handles} multicast={p.multicast_supported}")
        print_topology_info(be.detect_topology())
    except Exception as exc:  # never let a query failure hide the rest of the output
        print(f"device query failed: {type(exc).__name__}: {exc}")
        return 1
    return 0


def _handle_support(args) -> int:
    import tileccl_b200

    heap_size = args.heap_size_mb * 1024 * 1024 if args.heap_size_mb else None
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if args.world_size > 1 and have_gpu and heap_size:
        ctx = tileccl_b200.init_local(args.world_size, heap_size)[0]
    else:
        ctx = tileccl_b200.init(backend=args.backend, rank=0, world_size=1,
                                heap_size=heap_size if have_gpu else None, force_backend=True)
    matrix = ctx.support_matrix()
    if args.json:
        print(json.dumps(matrix.to_dict(), indent=2, default=str))
        return 0
    d = matrix.to_dict()
    print(f"context: {d['context']}")
    for section in ("ops", "contracts", "execution_paths", "collectives", "memory"):
        print(f"\n[{section}]")
        for name, st in d[section].items():
            print(f"  {name:<42s} {st['state']:<12s} {st['detail']}")
    print(f"\nsummary: {matrix.summary()}")
    return 0


def _handle_bench(args) -> int:
    from tileccl_b200 import benchmarks

    which = args.suite or ("pattern" if args.pattern else "all")
    common = dict(world_size=args.world_size, quick=args.quick)
    runs = {
        "p2p": lambda: benchmarks.bench_p2p(**common),
        "collective": lambda: benchmarks.bench_collectives(**common),
        "pattern": lambda: benchmarks.bench_patterns(M=args.M, N=args.N, K=args.K,
                                                     pattern=args.pattern, **common),
        "gemm": lambda: benchmarks.bench_gemm(quick=args.quick),
    }
    names = list(runs) if which == "all" else [which]
    rc = 0
    for name in names:
        try:
            payload = runs[name]()
        except Exception as exc:
            print(f"[bench {name}] failed: {type(exc).__name__}: {exc}")
            rc = 1
            continue
        path = _save(f"bench_{name}", payload, args.output if len(names) == 1 else None)
        print(benchmarks.render(payload))
        print(f"[bench {name}] saved to {path}")
    return rc


def _handle_compare(args) -> int:
    a, b = (json.loads(Path(p).read_text()) for p in (args.a, args.b))
    rows_a = {r.get("name"): r for r in a.get("rows", [])}
    rows_b = {r.get("name"): r for r in b.get("rows", [])}
    print(f"{'name':<44s} {'a ms':>10s} {'b ms':>10s} {'b/a':>8s}")
    for name in rows_a:
        if name in rows_b and rows_a[name].get("ms") and rows_b[name].get("ms"):
            ra, rb = rows_a[name]["ms"], rows_b[name]["ms"]
            print(f"{name:<44s} {ra:>10.4f} {rb:>10.4f} {rb / ra:>8.3f}")
    return 0


def build_parser() -> argparse.ArgumentParser:
    import tileccl_b200

    ap = argparse.ArgumentParser(prog="tileccl", description="Tile collective library for B200")
    ap.add_argument("--version", action="version", version=f"tileccl_b200 {tileccl_b200.__version__}")
    sub = ap.add_subparsers(dest="command")
    sub.add_parser("info", help="library, device and topology information")
    sp = sub.add_parser("support", help="runtime support matrix")
    sp.add_argument("--backend", default="auto")
    sp.add_argument("--world-size", type=int, default=1)
    sp.add_argument("--heap-size-mb", type=int, default=64)
    sp.add_argument("--json", action="store_true")
    bp = sub.add_parser("bench", help="run benchmarks")
    bp.add_argument("suite", nargs="?", choices=["p2p", "collective", "pattern", "gemm", "all"])
    bp.add_argument("--pattern", default=None)
    bp.add_argument("--M", type=int, default=8192)
    bp.add_argument("--N", type=int, default=4096)
    bp.add_argument("--K", type=int, default=2048)
    bp.add_argument("--world-size", type=int, default=0, help="0 = all visible GPUs")
    bp.add_argument("--quick", action="store_true")
    bp.add_argument("--output", default=None)
    cp = sub.add_parser("compare", help="compare two saved benchmark files")
    cp.add_argument("a")
    cp.add_argument("b")
    return ap


def main(argv: Optional[list] = None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.command is None:
        ap.print_help()
        return 0
    handler = {"info": _handle_info, "support": _handle_support, "bench": _handle_bench,
               "compare": _handle_compare}[args.command]
    return handler(args)


if __name__ == "__main__":
    sys.exit(main())
