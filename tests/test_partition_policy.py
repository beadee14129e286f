import ctypes
import json

import pytest

from ooverlap_b200 import _lib
from ooverlap_b200.utils.partition import bus_bandwidth_gbs, max_shard, partition, partition_sizes


@pytest.mark.parametrize("count", [0, 1, 7, 16, 4097, 1048576])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8, 16])
def test_partition_covers_everything(count, world):
    sizes = partition_sizes(count, world)
    assert sum(sizes) == count
    assert max(sizes) - min(sizes) <= 1
    assert sizes == sorted(sizes, reverse=True)  # the first `count % world` ranks get base + 1
    assert max(sizes) == (max_shard(count, world) if count else 0)
    prev = 0
    for r in range(world):
        b, e = partition(count, world, r)
        assert b == prev
        prev = e
    assert prev == count


def test_partition_rejects_bad_rank():
    with pytest.raises(ValueError):
        partition(10, 4, 4)


def test_bus_bandwidth_definition():
    # all-reduce: 2(n-1)/n * S / t ; reduce-scatter / all-gather: (n-1)/n * S / t
    assert bus_bandwidth_gbs("all_reduce", 8, 1 << 30, 1.0) == pytest.approx(2 * 7 / 8 * (1 << 30) / 1e9)
    assert bus_bandwidth_gbs("reduce_scatter", 4, 1000, 1e-6) == pytest.approx(0.75)
    assert bus_bandwidth_gbs("all_gather", 2, 1000, 1e-6) == pytest.approx(0.5)


def _select(lib, world, coll, nbytes, nvls):
    algo, ctas = ctypes.c_int(), ctypes.c_int()
    assert lib.oob_policy_select(world, coll, nbytes, nvls, ctypes.byref(algo), ctypes.byref(ctas)) == 0
    return algo.value, ctas.value


def test_policy_builtin_defaults(lib, monkeypatch):
    monkeypatch.delenv("OOB_MAX_CTAS", raising=False)
    assert lib.oob_policy_load(b"") == 0
    algo, ctas = _select(lib, 8, 0, 16 << 10, 0)
    assert algo == _lib.AR_ONESHOT_P2P and ctas >= 1
    algo, _ = _select(lib, 8, 0, 64 << 20, 0)
    assert algo == _lib.AR_TWOSHOT_P2P
    algo, _ = _select(lib, 8, 0, 64 << 20, 1)
    assert algo == _lib.AR_TWOSHOT_NVLS
    assert _select(lib, 8, 1, 1 << 20, 1)[0] == _lib.RS_NVLS
    assert _select(lib, 8, 2, 1 << 20, 0)[0] == _lib.AG_PUSH_P2P


def test_policy_file_nearest_point_and_cap(lib, tmp_path, monkeypatch):
    pts = {"comment": "ignored", "points": [
        {"world": 8, "collective": "allreduce", "nvls": 0, "bytes": 1 << 20, "algo": 1, "ctas": 12},
        {"world": 8, "collective": "allreduce", "nvls": 0, "bytes": 1 << 26, "algo": 1, "ctas": 40, "extra": [1, {"a": 2}]},
        {"world": 8, "collective": "all_gather", "nvls": 1, "bytes": 1 << 20, "algo": 1, "ctas": 6},
    ]}
    path = tmp_path / "policy.json"
    path.write_text(json.dumps(pts))
    monkeypatch.delenv("OOB_MAX_CTAS", raising=False)
    assert lib.oob_policy_load(str(path).encode()) == 0
    assert _select(lib, 8, 0, 3 << 20, 0) == (1, 12)   # nearest in log-ratio: 1 MiB
    assert _select(lib, 8, 0, 1 << 25, 0) == (1, 40)
    assert _select(lib, 8, 2, 1 << 10, 1) == (1, 6)
    # no point for this world size -> built-in
    assert _select(lib, 4, 0, 1 << 10, 0)[0] == _lib.AR_ONESHOT_P2P
    monkeypatch.setenv("OOB_MAX_CTAS", "5")
    assert _select(lib, 8, 0, 1 << 25, 0) == (1, 5)
    monkeypatch.delenv("OOB_MAX_CTAS")
    assert lib.oob_policy_load(b"") == 0


def test_policy_rejects_malformed(lib, tmp_path):
    bad = tmp_path / "bad.json"
    bad.write_text('{"points": [{"world": 8, "collective": "allreduce"}]}')
    assert lib.oob_policy_load(str(bad).encode()) == _lib.ERR_INVALID
    assert b"missing" in lib.oob_last_error()
    bad.write_text('{"points": [')
    assert lib.oob_policy_load(str(bad).encode()) == _lib.ERR_INVALID
    assert lib.oob_policy_load(b"/nonexistent/policy.json") == _lib.ERR_INVALID
    assert lib.oob_policy_load(b"") == 0


def test_gemm_bookkeeping_helpers(lib):
    assert lib.oob_gemm_partial_bytes(8192, 8192) == (64 * 32 + 16) * 128 * 256 * 2
    assert lib.oob_gemm_partial_bytes(100, 100) == (1 + 16) * 128 * 256 * 2
    # two-SM kernel: arrivals + finished work items per owned half tile (2 * 2048 / 8) + ticket; one-SM kernel: 256 tiles + ticket
    assert lib.oob_gemm_counters_needed(_lib.GEMM_AR, 8192, 8192, 8) == 513
    assert lib.oob_gemm_counters_needed(_lib.GEMM_RS_NORM, 4096, 8192, 8) == 9
    assert lib.oob_gemm_counters_needed(_lib.GEMM_AG, 4096, 3584, 8) == 33


def test_packaged_policy_loads_and_covers_two_four_and_eight_ranks(lib, monkeypatch):
    """The measured (algorithm, CTA budget) table that ships with the package parses with the native loader, has
    points for 2, 4 and 8 ranks with and without NVLS, names only algorithms that exist, and a lookup at one of its
    points returns that point."""
    import os
    monkeypatch.delenv("OOB_MAX_CTAS", raising=False)
    path = os.path.join(os.path.dirname(_lib.__file__), "policy", "b200_nvswitch.json")
    data = json.load(open(path))
    pts = data["points"]
    assert {p["world"] for p in pts} == {2, 4, 8}
    assert {p["collective"] for p in pts} == {"all_reduce", "reduce_scatter", "all_gather"}
    valid = {"all_reduce": {_lib.AR_ONESHOT_P2P, _lib.AR_TWOSHOT_P2P, _lib.AR_ONESHOT_NVLS, _lib.AR_TWOSHOT_NVLS},
             "reduce_scatter": {_lib.RS_P2P, _lib.RS_NVLS}, "all_gather": {_lib.AG_PUSH_P2P, _lib.AG_PUSH_NVLS}}
    for p in pts:
        assert p["algo"] in valid[p["collective"]], p
        assert 1 <= p["ctas"] <= 160 and p["bytes"] >= 1024 and p["nvls"] in (0, 1), p
        if not p["nvls"]:
            assert p["algo"] not in (_lib.AR_ONESHOT_NVLS, _lib.AR_TWOSHOT_NVLS) or p["collective"] != "all_reduce", p
    for world in (2, 4, 8):
        assert any(p["world"] == world and p["nvls"] == 1 for p in pts)
    assert lib.oob_policy_load(path.encode()) == 0
    try:
        code = {"all_reduce": 0, "reduce_scatter": 1, "all_gather": 2}
        for p in pts[:: max(1, len(pts) // 25)]:
            algo, ctas = _select(lib, p["world"], code[p["collective"]], p["bytes"], p["nvls"])
            assert (algo, ctas) == (p["algo"], p["ctas"]), p
    finally:
        assert lib.oob_policy_load(b"") == 0


def test_policy_files_merge_later_file_wins(tmp_path):
    from ooverlap_b200.bench.collective_sweep import merge_policies
    a = {"comment": "first", "points": [
        {"world": 8, "collective": "all_reduce", "nvls": 1, "bytes": 1024, "algo": 3, "ctas": 8},
        {"world": 8, "collective": "all_reduce", "nvls": 1, "bytes": 2048, "algo": 3, "ctas": 8}]}
    b = {"comment": "second", "points": [
        {"world": 8, "collective": "all_reduce", "nvls": 1, "bytes": 2048, "algo": 4, "ctas": 16},
        {"world": 4, "collective": "all_gather", "nvls": 0, "bytes": 4096, "algo": 0, "ctas": 4}]}
    pa, pb, out = tmp_path / "a.json", tmp_path / "b.json", tmp_path / "m.json"
    pa.write_text(json.dumps(a))
    pb.write_text(json.dumps(b))
    assert merge_policies([str(pa), str(pb)], str(out)) == 3
    m = json.load(open(out))
    assert m["comment"] == "first"
    assert [(p["world"], p["bytes"], p["algo"]) for p in m["points"]] == [(4, 4096, 0), (8, 1024, 3), (8, 2048, 4)]
    assert merge_policies([str(pb), str(pa)], str(out), comment="mine") == 3
    m = json.load(open(out))
    assert m["comment"] == "mine" and [p["algo"] for p in m["points"] if p["bytes"] == 2048] == [3]
