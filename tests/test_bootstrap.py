"""Rendezvous layer of the symmetric heap: ranks are plain processes that exchange
file descriptors over abstract Unix sockets (no GPU)."""

import ctypes as C
import multiprocessing as mp
import os
import uuid

import pytest


def _rank_main(rank, ws, job, q, misbehave):
    from tileccl_b200 import _native

    if misbehave == "absent" and rank == ws - 1:
        q.put((rank, "absent"))
        return
    r = os.memfd_create(f"tccl-test-{rank}")   # readable by every peer, unlike a pipe
    os.write(r, f"hello from {rank}".encode())
    payloads = (C.c_uint64 * ws)()
    fds = (C.c_int32 * ws)()
    try:
        _native.call("tccl_bootstrap_allgather", rank, ws, job.encode(), 1500 if misbehave else 20000,
                     1000 + rank, r, payloads, fds)
    except _native.NativeError as exc:
        q.put((rank, f"error: {exc.message}"))
        return
    got = {}
    for peer in range(ws):
        if peer == rank:
            continue
        got[peer] = os.pread(fds[peer], 64, 0).decode()
    q.put((rank, [int(p) for p in payloads], got))


def _spawn(ws, misbehave=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    job = uuid.uuid4().hex[:10]
    procs = [ctx.Process(target=_rank_main, args=(r, ws, job, q, misbehave)) for r in range(ws)]
    for p in procs:
        p.start()
    out = [q.get(timeout=60) for _ in range(ws)]
    for p in procs:
        p.join(timeout=30)
    return sorted(out, key=lambda x: x[0])


@pytest.mark.parametrize("ws", [2, 4])
def test_fd_allgather_between_processes(ws):
    results = _spawn(ws)
    for rank, payloads, got in results:
        assert payloads == [1000 + r for r in range(ws)]
        assert got == {p: f"hello from {p}" for p in range(ws) if p != rank}


def test_missing_rank_is_reported_not_hung():
    results = _spawn(2, misbehave="absent")
    by_rank = {r[0]: r[1] for r in results}
    assert by_rank[1] == "absent"
    assert isinstance(by_rank[0], str) and by_rank[0].startswith("error:") and "timed out" in by_rank[0]
