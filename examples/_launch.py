"""Tiny launcher shared by the examples: runs ``fn(rank, world, *args)`` in ``world`` spawned processes, or
inside the current process when the script was started by torchrun (RANK / WORLD_SIZE set)."""
import multiprocessing as mp
import os
import socket
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _child(fn, rank, world, args, q):
    try:
        q.put((rank, None, fn(rank, world, *args)))
    except BaseException as e:  # noqa: BLE001
        import traceback
        q.put((rank, f"{e!r}\n{traceback.format_exc()}", None))


def run(fn, world: int, *args, timeout: float = 180):
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        return [fn(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), *args)]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_child, args=(fn, r, world, args, q)) for r in range(world)]
    [p.start() for p in ps]
    out, errs = {}, []
    for _ in range(world):
        r, err, val = q.get(timeout=timeout)
        (errs.append(f"rank {r}: {err}") if err else out.__setitem__(r, val))
    [p.join(10) for p in ps]
    if errs:
        raise SystemExit("\n".join(errs))
    return [out[r] for r in range(world)]
