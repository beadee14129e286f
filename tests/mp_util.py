"""Runs a function in ``world`` fresh processes and collects per-rank results or errors."""
import multiprocessing as mp
import os
import traceback


def _entry(fn, rank, world, args, q):
    try:
        q.put((rank, "ok", fn(rank, world, *args)))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_ranks(fn, world, args=(), timeout=120, env=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    old = {}
    for k, v in (env or {}).items():
        old[k] = os.environ.get(k)
        os.environ[k] = v
    procs = [ctx.Process(target=_entry, args=(fn, r, world, args, q)) for r in range(world)]
    try:
        for p in procs:
            p.start()
        results = {}
        for _ in range(world):
            try:
                rank, kind, val = q.get(timeout=timeout)
            except Exception:
                break
            results[rank] = (kind, val)
        for p in procs:
            p.join(timeout=10)
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()  # exact child handles only
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    return results


def free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port
