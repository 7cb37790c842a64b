"""Helpers to run an N-rank scenario as spawned child processes on one machine."""
import multiprocessing as mp
import os
import traceback


def _child(fn, rank, world, args, q, env, barrier):
    try:
        os.environ.update(env)
        if barrier is not None:
            args = tuple(args) + (barrier,)
        q.put((rank, "ok", fn(rank, world, *args)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{e!r}\n{traceback.format_exc()}"))


def run_ranks(fn, world, args=(), timeout=120, env=None, with_barrier=False):
    """Runs fn(rank, world, *args[, barrier]) in `world` spawned processes; returns results by rank or raises."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    barrier = ctx.Barrier(world) if with_barrier else None
    procs = [ctx.Process(target=_child, args=(fn, r, world, args, q, env or {}, barrier)) for r in range(world)]
    for p in procs:
        p.start()
    results, errors = {}, []
    try:
        for _ in range(world):
            rank, st, val = q.get(timeout=timeout)
            if st == "ok":
                results[rank] = val
            else:
                errors.append(f"rank {rank}: {val}")
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if errors:
        raise AssertionError("\n".join(errors))
    return [results[r] for r in range(world)]
