"""Helpers to run a function on several CPU ranks (gloo) in child processes."""
from __future__ import annotations

import os
import socket
import traceback
from typing import Any, Callable

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def _entry(rank: int, world: int, port: int, fn: Callable[..., Any], args: tuple[Any, ...], out: Any,
           dump_after: float = 0.0) -> None:
    if dump_after > 0:
        import faulthandler
        import sys

        faulthandler.enable(file=sys.stderr)                                         # a crashing rank says where
        faulthandler.dump_traceback_later(dump_after, exit=False, file=sys.stderr)   # where is a stuck rank?
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank),
                       "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank), "LOCAL_WORLD_SIZE": str(world)})
    torch.set_num_threads(2)
    try:
        res = fn(rank, world, *args)
        out.put((rank, "ok", res))
    except BaseException as ex:  # noqa: BLE001
        out.put((rank, "error", f"{type(ex).__name__}: {ex}\n{traceback.format_exc()}"))


def run_distributed(fn: Callable[..., Any], world: int, *args: Any, timeout: float = 240.0) -> list[Any]:
    """Runs ``fn(rank, world, *args)`` on ``world`` processes; returns results by rank."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, out, 0.6 * timeout)) for r in range(world)]
    for p in procs:
        p.start()
    results: dict[int, Any] = {}
    errors: list[str] = []
    try:
        for _ in range(world):
            try:
                rank, status, payload = out.get(timeout=timeout)
            except Exception:  # noqa: BLE001 - queue.Empty: a rank never reported
                missing = sorted(set(range(world)) - set(results) - {int(e.split("]")[0][6:]) for e in errors})
                errors.append(f"rank(s) {missing} did not report within {timeout} s")
                break
            if status == "ok":
                results[rank] = payload
            else:
                errors.append(f"[rank {rank}] {payload}")
                if world > 1:
                    timeout = min(timeout, 20.0)    # the others are probably stuck waiting for the failed rank
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if errors:
        raise AssertionError("\n".join(errors))
    return [results[r] for r in range(world)]
