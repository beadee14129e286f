"""The strategy rule of GemmAllReduce is a pure function: the choices that were measured on 8 x B200 are pinned here."""
import pytest

from ooverlap_b200.ops.overlap import plan_gemm_all_reduce as plan


def test_measured_choices_on_nvswitch():
    # tp8, N = 8192: one partial wave of tiles on the one-SM kernel with the in-switch pull ...
    assert plan(8, 512, 8192, False) == ("fused", 1, 2, 16, "one_sm")
    # ... a few waves: the GEMM and the in-switch all-reduce back to back ...
    assert plan(8, 2048, 8192, False)[0] == "unfused"
    # ... above 64 MiB the two-SM kernel that reduces in place through the switch, 8 communication CTAs
    assert plan(8, 8192, 8192, False) == ("fused", 1, 1, 8, "pair")
    # four ranks: pushed tiles for one partial wave, the two-SM kernel through the switch (16 CTAs) above
    assert plan(4, 512, 8192, False) == ("fused", 1, 0, 16, "one_sm")
    assert plan(4, 2048, 8192, False) == ("fused", 1, 1, 16, "pair") and plan(4, 8192, 8192, False)[3:] == (16, "pair")
    # two ranks: always a fused kernel; one or two waves of tiles on the one-SM kernel with pushed tiles, 64 MiB and
    # more on the two-SM kernel that reduces in place through the switch with 24 communication CTAs
    assert plan(2, 512, 8192, False) == ("fused", 1, None, 16, "one_sm")
    assert plan(2, 2048, 8192, False)[4] == "one_sm"
    assert plan(2, 8192, 8192, False) == ("fused", 1, 1, 24, "pair")
    # what the caller fixed stays
    assert plan(2, 8192, 8192, False, "auto", None, 0, 8, None, "one_sm") == ("fused", 1, 0, 8, "one_sm")
    # emulation runs one launch per op
    assert plan(8, 512, 8192, True)[0] == "fused"


def test_chunked_strategy_resolution():
    assert plan(8, 8192, 8192, False, "chunked")[:2] == ("chunked", 4)          # slabs of 2048 rows
    assert plan(8, 512, 8192, False, "chunked")[0] == "unfused"                 # a single slab: nothing to pipeline
    assert plan(8, 512, 8192, False, "chunked", 2)[:2] == ("chunked", 2)        # explicit slab count
    assert plan(1, 8192, 8192, False, "chunked")[0] == "unfused"
    assert plan(8, 8192, 8192, True, "chunked")[0] == "fused"
    with pytest.raises(ValueError):
        plan(8, 1000, 8192, False, "chunked", 3)
    with pytest.raises(ValueError):
        plan(8, 512, 8192, False, "pipelined")


def test_tuned_solution_overrides_the_rule():
    sol = {"strategy": "fused", "comm_ctas": 24, "use_nvls": 2}
    assert plan(8, 512, 8192, False, "auto", None, None, None, sol) == ("fused", 1, 2, 24, None)
    # explicit arguments win over the solution's
    assert plan(8, 512, 8192, False, "auto", None, 0, 8, sol) == ("fused", 1, 0, 8, None)
    assert plan(8, 8192, 8192, False, "auto", None, None, None, {"strategy": "chunked", "chunks": 8})[:2] == ("chunked", 8)
    # a solution is ignored in emulation and when the caller named a strategy
    assert plan(8, 512, 8192, True, "auto", None, None, None, sol)[0] == "fused"
    assert plan(8, 512, 8192, False, "unfused", None, None, None, sol)[0] == "unfused"
    assert plan(8, 512, 8192, False, "auto", None, None, None, dict(sol, kernel="pair"))[4] == "pair"
    with pytest.raises(ValueError):
        plan(8, 512, 8192, False, "auto", None, None, None, {"strategy": "bogus"})


def test_autotune_candidate_list():
    """What strategy="autotune" measures: the unfused pair, the two-SM kernel over CTA budgets (through the switch when
    there is one; with peer loads too between two ranks), the one-SM kernel, and from four ranks on its in-switch pull
    and, for tall outputs, the slab pipeline."""
    from types import SimpleNamespace
    from ooverlap_b200.ops.overlap import GemmAllReduce

    def cands(world, nvls, M):
        op = SimpleNamespace(comm=SimpleNamespace(world=world, nvls=nvls), M=M, N=8192)
        return GemmAllReduce._candidates(op)

    c8 = cands(8, True, 8192)
    assert c8[0] == ("unfused", None, None, None)
    assert [c for c in c8 if c[1] == "pair"] == [("fused", "pair", 1, n) for n in (4, 8, 10, 16, 24, 32)]  # 10: wave-aligned
    assert ("fused", "one_sm", 0, 16) in c8 and ("fused", "one_sm", 2, 16) in c8 and ("chunked", None, None, None) in c8
    assert ("chunked", None, None, None) not in cands(8, True, 512)
    c2 = cands(2, True, 8192)
    assert ("fused", "pair", 0, 8) in c2 and ("fused", "pair", 1, 8) in c2 and ("fused", "one_sm", 2, 16) not in c2
    assert all(c[2] == 0 for c in cands(4, False, 2048) if c[1] == "pair")


def test_wave_aligned_communication_ctas():
    from ooverlap_b200.ops.overlap import wave_aligned_comm_ctas as f
    assert f(4096, 8192) == 20          # 512 tiles: 64 pairs still need 8 waves, 63 would need 9
    assert f(8192, 8192) == 10          # 1024 tiles: 15 waves on 72 .. 69 pairs, 16 from 68 pairs down
    assert f(512, 8192) == 20           # 64 tiles fit one wave on 64 pairs
    assert f(256, 256) == 24            # one tile: every budget is free
    for M, N in ((4096, 8192), (2048, 8192), (4096, 28672)):
        c = f(M, N)
        tiles = (M // 256) * (N // 256)
        assert 4 <= c <= 24 and -(-tiles // ((148 - c) // 2)) == min(-(-tiles // ((148 - k) // 2)) for k in range(4, 25, 2))
