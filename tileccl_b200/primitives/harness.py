"""Drive one device primitive from Python (one launch = one rank doing one thing).

Used by the GPU tests of pointer translation, remote load/store, put/get, the
signal/wait family, remote atomics and the bounded-wait time-out path.  Works on
any heap, including emulated ranks that share one GPU: a launch never waits on
another launch unless the test asks for a wait, and every wait is bounded.
"""

from __future__ import annotations

import torch

from .. import _native

OPS = {"put": 0, "get": 1, "remote_store": 2, "remote_load": 3, "signal": 4, "wait": 5, "poll": 6,
       "signal_add": 7, "wait_ge": 8, "atomic": 9, "barrier": 10, "credit": 11, "try_wait": 12,
       "translate": 13, "put_mc": 14, "get_reduce": 15}
ATOMICS = {"add": 0, "cas": 1, "xchg": 2, "min": 3, "max": 4, "and": 5, "or": 6, "xor": 7}


def run(heap, op: str, *, peer: int = 0, a: int = 0, b: int = 0, nbytes: int = 0, value: int = 0,
        value2: int = 0, sub_op: int = 0, budget_us: float = 1e6) -> list:
    """Launch as ``heap.rank`` and return the four result words (synchronises)."""
    result = torch.zeros(4, dtype=torch.int32, device=heap.device)
    with torch.cuda.device(heap.device):
        _native.call("tccl_prim_test", OPS[op], sub_op, heap.rank, heap.world_size, peer,
                     heap.window_base, heap.stride, heap.multicast_base, a, b, nbytes,
                     value & 0xFFFFFFFF, value2 & 0xFFFFFFFF, result.data_ptr(),
                     int(budget_us * 1000), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
    return [x & 0xFFFFFFFF for x in result.tolist()]


def run_concurrent(calls) -> list:
    """Launch one primitive per entry of ``calls`` (``(heap, op, kwargs)``), all before the
    first synchronise, and return each launch's result words.  For primitives whose ranks
    wait for one another (``barrier``): only on heaps whose ranks own different GPUs, since
    launches that share a GPU must never wait on each other."""
    devs = [h.device for h, _, _ in calls]
    if len({str(d) for d in devs}) != len(devs):
        raise ValueError("run_concurrent needs every rank on its own GPU")
    results = []
    for heap, op, kw in calls:
        kw = dict(kw)
        budget_us = kw.pop("budget_us", 1e6)
        result = torch.zeros(4, dtype=torch.int32, device=heap.device)
        results.append(result)
        with torch.cuda.device(heap.device):
            _native.call("tccl_prim_test", OPS[op], kw.get("sub_op", 0), heap.rank, heap.world_size,
                         kw.get("peer", 0), heap.window_base, heap.stride, heap.multicast_base,
                         kw.get("a", 0), kw.get("b", 0), kw.get("nbytes", 0),
                         kw.get("value", 0) & 0xFFFFFFFF, kw.get("value2", 0) & 0xFFFFFFFF,
                         result.data_ptr(), int(budget_us * 1000),
                         torch.cuda.current_stream().cuda_stream)
    for d in devs:
        torch.cuda.synchronize(d)
    return [[x & 0xFFFFFFFF for x in r.tolist()] for r in results]


def translate(heap, ptr: int, to_rank: int) -> int:
    words = run(heap, "translate", peer=to_rank, a=ptr)
    return words[0] | (words[1] << 32)


def atomic(heap, name: str, flag_ptr: int, value: int, to_rank: int, value2: int = 0) -> int:
    return run(heap, "atomic", peer=to_rank, a=flag_ptr, value=value, value2=value2,
               sub_op=ATOMICS[name])[0]
