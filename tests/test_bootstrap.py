"""Host-side rendezvous: all-gather, barrier, descriptor passing, and failure detection (timeouts)."""
import ctypes
import os
import time
import uuid

import pytest

from mp_util import run_ranks


def _boot(rank, world, key, timeout_ms=10000):
    from ooverlap_b200 import _lib
    lib = _lib.lib()
    h = ctypes.c_void_p()
    rc = lib.oob_bootstrap_create(rank, world, key.encode(), timeout_ms, ctypes.byref(h))
    return lib, h, rc


def _rank_allgather_and_fds(rank, world, key, tmpdir):
    lib, h, rc = _boot(rank, world, key)
    assert rc == 0, lib.oob_last_error()
    mine = (ctypes.c_uint64 * 2)(rank, rank * rank + 7)
    out = (ctypes.c_uint64 * (2 * world))()
    assert lib.oob_bootstrap_allgather(h, mine, out, 16) == 0
    got = [(out[2 * r], out[2 * r + 1]) for r in range(world)]
    # descriptor exchange: every rank shares a file whose content names it
    path = os.path.join(tmpdir, f"rank{rank}.txt")
    with open(path, "w") as f:
        f.write(f"hello from {rank}")
    fd = os.open(path, os.O_RDONLY)
    fds = (ctypes.c_int * world)()
    assert lib.oob_bootstrap_exchange_fds(h, fd, fds) == 0, lib.oob_last_error()
    texts = []
    for r in range(world):
        # positional read: a passed descriptor shares its file offset with the sender and the other receivers
        texts.append(os.pread(fds[r], 64, 0).decode())
        os.close(fds[r])
    os.close(fd)
    # broadcast of one descriptor from rank 1
    bfd = ctypes.c_int(os.open(path, os.O_RDONLY) if rank == 1 else -1)
    assert lib.oob_bootstrap_broadcast_fd(h, 1, ctypes.byref(bfd)) == 0
    btext = os.pread(bfd.value, 64, 0).decode()
    os.close(bfd.value)
    assert lib.oob_bootstrap_barrier(h) == 0
    lib.oob_bootstrap_destroy(h)
    return got, texts, btext


@pytest.mark.parametrize("world", [2, 4])
def test_allgather_barrier_and_fd_passing(world, tmp_path):
    key = "t_" + uuid.uuid4().hex[:12]
    res = run_ranks(_rank_allgather_and_fds, world, (key, str(tmp_path)))
    assert len(res) == world
    for r in range(world):
        kind, val = res[r]
        assert kind == "ok", val
        got, texts, btext = val
        assert got == [(i, i * i + 7) for i in range(world)]
        assert texts == [f"hello from {i}" for i in range(world)]
        assert btext == "hello from 1"


def _rank_missing_peer(rank, world, key):
    # Rank 1 never joins: rank 0 must give up with an error instead of hanging.
    if rank == 1:
        return "absent"
    from ooverlap_b200 import _lib
    _lib.lib()  # loading the library is not part of the rendezvous time measured below
    t0 = time.time()
    lib, h, rc = _boot(rank, world, key, timeout_ms=700)
    return rc, lib.oob_last_error().decode(), time.time() - t0


def test_missing_rank_times_out():
    key = "t_" + uuid.uuid4().hex[:12]
    res = run_ranks(_rank_missing_peer, 2, (key,))
    kind, val = res[0]
    assert kind == "ok", val
    rc, msg, dt = val
    assert rc == -3 and "joined" in msg
    assert dt < 5


def _rank_dies_before_collective(rank, world, key):
    lib, h, rc = _boot(rank, world, key, timeout_ms=1500)
    assert rc == 0
    if rank == 1:
        os._exit(0)  # leaves between steps, without taking part in the next exchange
    buf = (ctypes.c_char * world)()
    rc = lib.oob_bootstrap_allgather(h, b"x", buf, 1)
    return rc, lib.oob_last_error().decode()


def test_peer_exit_is_detected():
    key = "t_" + uuid.uuid4().hex[:12]
    res = run_ranks(_rank_dies_before_collective, 2, (key,), timeout=30)
    kind, val = res[0]
    assert kind == "ok", val
    rc, msg = val
    assert rc == -3
    assert "closed" in msg or "timeout" in msg


def test_key_validation(lib):
    h = ctypes.c_void_p()
    assert lib.oob_bootstrap_create(0, 1, b"", 100, ctypes.byref(h)) == -3
    assert lib.oob_bootstrap_create(0, 1, b"k" * 200, 100, ctypes.byref(h)) == -3
    assert lib.oob_bootstrap_create(3, 2, b"ok", 100, ctypes.byref(h)) == -3
    assert lib.oob_bootstrap_create(0, 1, b"weird key/with:chars", 100, ctypes.byref(h)) == 0
    lib.oob_bootstrap_destroy(h)
