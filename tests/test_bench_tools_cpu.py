"""Host-only tooling: result aggregation over backend orders, plot series, tuning solutions."""
import json
import os

import pytest

from ooverlap_b200.bench import aggregate, plot
from ooverlap_b200.ops import solutions


def _write(path, rows):
    path.write_text("\n".join(json.dumps(r) for r in rows) + "\nnot json\n")
    return str(path)


def test_aggregate_over_orders(tmp_path):
    f1 = _write(tmp_path / "a.jsonl", [
        {"model": "m", "tp": 8, "batch": 1, "backend": "nccl", "output_tok_s": 10.0},
        {"model": "m", "tp": 8, "batch": 1, "backend": "ours", "output_tok_s": 20.0},
        {"model": "m", "tp": 8, "batch": 64, "backend": "nccl", "output_tok_s": 100.0}])
    f2 = _write(tmp_path / "b.jsonl", [
        {"model": "m", "tp": 8, "batch": 1, "backend": "ours", "output_tok_s": 24.0},
        {"model": "m", "tp": 8, "batch": 1, "backend": "nccl", "output_tok_s": 12.0},
        {"model": "m", "tp": 8, "batch": 1, "backend": "nccl"}])  # row without the metric is ignored
    out = aggregate.aggregate(aggregate.read_lines([f1, f2]), "output_tok_s", ["model", "tp", "batch"], "backend", "nccl")
    assert len(out) == 2
    b1 = out[0]
    assert b1["batch"] == 1 and b1["stats"]["nccl"]["n"] == 2 and b1["stats"]["nccl"]["median"] == 11.0
    assert b1["stats"]["ours"]["mean"] == 22.0
    assert abs(b1["speedup_vs_nccl"]["ours"] - 2.0) < 1e-9
    assert "ours" not in out[1]["stats"]
    # latency-like metrics: lower is better
    lat = aggregate.aggregate([{"g": 1, "impl": "a", "us": 10.0}, {"g": 1, "impl": "b", "us": 5.0}], "us", ["g"], "impl", "a",
                              higher_is_better=False)
    assert lat[0]["speedup_vs_a"]["b"] == 2.0
    assert aggregate.main([f1, "--metric", "output_tok_s"]) == 0


def test_plot_series(tmp_path, capsys):
    sweep = [{"collective": "all_reduce", "impl": "nccl", "algo": "nccl", "bytes": 1024, "bus_gbs": 1.0, "ctas": 0},
             {"collective": "all_reduce", "impl": "ours", "algo": "twoshot_nvls", "bytes": 1024, "bus_gbs": 2.0, "ctas": 8},
             {"collective": "all_reduce", "impl": "ours", "algo": "twoshot_nvls", "bytes": 1024, "bus_gbs": 3.0, "ctas": 32}]
    s = plot.sweep_series(sweep)
    assert s["all_reduce"]["twoshot_nvls"] == [(1024, 3.0)] and s["all_reduce"]["nccl"] == [(1024, 1.0)]
    ov = plot.overlap_series([{"op": "gemm_ar", "M": 512, "impl": "ours_fused", "nvls": 2, "us": 50.0},
                              {"op": "gemm_ar", "M": 512, "impl": "ours_fused", "nvls": 2, "us": 40.0},
                              {"op": "gemm_ar", "M": 512, "impl": "cublas+nccl", "us": 80.0}])
    assert ov[("gemm_ar", 512)] == {"ours_fused(nvls=2)": 40.0, "cublas+nccl": 80.0}
    f = _write(tmp_path / "s.jsonl", sweep)
    assert plot.main([f, "--kind", "sweep"]) == 0
    assert "twoshot_nvls" in capsys.readouterr().out


def test_solutions_roundtrip(tmp_path, monkeypatch):
    path = str(tmp_path / "sol.json")
    k = solutions.key("gemm_ar", 8192, 8192, 8192, 8, "fp16")
    assert k == "gemm_ar:8192x8192x8192:tp8:fp16"
    solutions.save(path, {k: {"strategy": "fused", "comm_ctas": 16, "use_nvls": 0, "us": 417.0}})
    assert solutions.lookup("gemm_ar", 8192, 8192, 8192, 8, "fp16", path)["comm_ctas"] == 16
    assert solutions.lookup("gemm_ar", 8192, 8192, 0, 8, "fp16", path)["strategy"] == "fused"  # any K
    assert solutions.lookup("gemm_ar", 512, 8192, 8192, 8, "fp16", path) is None
    monkeypatch.setenv("OOB_OVERLAP_SOLUTIONS", path)
    assert solutions.lookup("gemm_ar", 8192, 8192, 8192, 8, "fp16")["us"] == 417.0
    monkeypatch.setenv("OOB_OVERLAP_SOLUTIONS", "none")
    assert solutions.lookup("gemm_ar", 8192, 8192, 8192, 8, "fp16") is None
    monkeypatch.delenv("OOB_OVERLAP_SOLUTIONS")
    assert solutions.lookup("gemm_ar", 8192, 8192, 8192, 8, "fp16")["us"] != 417.0  # the packaged table
    assert solutions.lookup("gemm_ar", 1000, 8192, 8192, 8, "fp16") is None
    assert solutions.load(str(tmp_path / "missing.json")) == {}


def test_packaged_overlap_solutions_plan_to_runnable_configurations(monkeypatch):
    """Every entry of the packaged table is a measured winner for a headline shape and resolves, through the same
    planner that GemmAllReduce uses, to a configuration the kernels accept."""
    import json
    from ooverlap_b200.ops.overlap import plan_gemm_all_reduce
    monkeypatch.delenv("OOB_OVERLAP_SOLUTIONS", raising=False)
    table = json.load(open(solutions.PACKAGED))
    entries = {k: v for k, v in table.items() if k.startswith("gemm_ar:")}
    assert len(entries) == 9 and isinstance(table["_about"], str)
    for k, v in entries.items():
        _, shape, tp, dtype = k.split(":")
        M, N, K = (int(x) for x in shape.split("x"))
        world = int(tp[2:])
        assert solutions.lookup("gemm_ar", M, N, 0, world, dtype) == v
        assert v["us"] <= v["unfused_us"] and v["measured_by"]
        strategy, chunks, use_nvls, comm_ctas, kernel = plan_gemm_all_reduce(world, M, N, False, "auto", solution=v)
        assert strategy == v["strategy"]
        if strategy == "fused":
            assert kernel == v["kernel"] and comm_ctas == v["comm_ctas"] and use_nvls == v["use_nvls"]
            assert kernel in ("pair", "one_sm") and 1 <= comm_ctas <= 64 and use_nvls in (0, 1, 2)
            assert not (kernel == "pair" and use_nvls == 2)  # the two-SM kernel has one path through the switch
        # what the caller fixes is never overridden by the table
        assert plan_gemm_all_reduce(world, M, N, False, "unfused", solution=v)[0] == "unfused"


def test_gemm_solution_table_lookup_and_profiler_candidates(tmp_path, monkeypatch):
    from ooverlap_b200.bench.gemm_profile import candidates
    path = str(tmp_path / "gemm.json")
    solutions.save(path, {solutions.gemm_key(512, 8192, 8192, "bf16"): {"pair": 1, "splits": 1, "stream_k": 1, "us": 60.0}})
    monkeypatch.setenv("OOB_GEMM_SOLUTIONS", path)
    solutions.reset_gemm_lookup()
    assert solutions.lookup_gemm(512, 8192, 8192, "bf16")["stream_k"] == 1
    assert solutions.lookup_gemm(512, 8192, 8192, "fp16") is None
    monkeypatch.setenv("OOB_GEMM_SOLUTIONS", "none")
    solutions.reset_gemm_lookup()
    assert solutions.lookup_gemm(512, 8192, 8192, "bf16") is None
    monkeypatch.delenv("OOB_GEMM_SOLUTIONS")
    solutions.reset_gemm_lookup()
    names = [c["name"] for c in candidates(64, 8192, 3584)]
    assert "weight_streaming" in names and "pair" not in names and "one_sm/split8" in names and "one_sm/split16" not in names
    names = [c["name"] for c in candidates(2048, 8192, 8192)]
    assert names[:4] == ["rule", "pair", "pair+stream_k", "one_sm"] and "cuda_core" not in names
    assert "cuda_core" in [c["name"] for c in candidates(1, 7168, 8192)]


def test_vllm_bench_model_dir_env_and_commands(tmp_path):
    import json
    import subprocess
    import sys
    from ooverlap_b200.bench import vllm_bench
    d = vllm_bench.write_model_dir(str(tmp_path / "m"), "llama3-70b", layers=4, max_len=1200)
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["num_hidden_layers"] == 4 and cfg["hidden_size"] == 8192 and cfg["num_key_value_heads"] == 8
    from transformers import AutoConfig
    hf = AutoConfig.from_pretrained(d)
    assert hf.model_type == "llama" and hf.intermediate_size == 28672 and hf.vocab_size == 128256
    env = vllm_bench.child_env("ooverlap", "/some/repo", base={"PYTHONPATH": "/x"}, plugin_dir="/plug", stats_file="/s.jsonl")
    assert env["VLLM_FORCE_ALLREDUCE_BACKEND"] == "ooverlap"
    assert env["PYTHONPATH"].split(os.pathsep) == ["/plug", "/some/repo", "/x"] and env["VLLM_OOVERLAP_STATS_FILE"] == "/s.jsonl"
    env2 = vllm_bench.child_env("pynccl", "/some/repo", base={"VLLM_FORCE_ALLREDUCE_BACKEND": "ooverlap"})
    assert env2["VLLM_FORCE_ALLREDUCE_BACKEND"] == "pynccl" and env2["MASTER_ADDR"] == "127.0.0.1"
    env3 = vllm_bench.child_env("default", "/some/repo", base={"VLLM_FORCE_ALLREDUCE_BACKEND": "ooverlap"})
    assert "VLLM_FORCE_ALLREDUCE_BACKEND" not in env3
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "ooverlap_b200.bench.vllm_bench", "--dry-run", "--model", "tiny", "--tp", "2",
                          "--batches", "1,4", "--backends", "pynccl,ooverlap", "--orders", "all"], cwd=root,
                         capture_output=True, text=True, check=True).stdout
    recs = [json.loads(ln) for ln in out.splitlines()]
    assert len(recs) == 2 * 2  # orders x backends: one engine per backend runs every batch size
    assert {r["backend"] for r in recs} == {"pynccl", "ooverlap"} and all(r["batches"] == "1,4" for r in recs)
    assert all("--worker" in r["cmd"] and "--model-dir" in r["cmd"] for r in recs)
    out = subprocess.run([sys.executable, "-m", "ooverlap_b200.bench.vllm_bench", "--dry-run", "--model", "tiny", "--tp", "2",
                          "--batches", "1,4", "--backends", "default,ooverlap", "--per-batch-engines"], cwd=root,
                         capture_output=True, text=True, check=True).stdout
    assert len(out.splitlines()) == 2 * 2  # batches x backends
    # per-rank statistics written by the backend at shutdown are summed for the record
    sf = tmp_path / "stats.jsonl"
    sf.write_text('{"rank": 0, "world": 2, "served": 5, "served_in_pieces": 1, "declined": {"x": 1}}\n'
                  '{"rank": 1, "world": 2, "served": 5, "served_in_pieces": 1, "declined": {"x": 2}}\n')
    assert vllm_bench.read_stats(str(sf)) == {"ranks": 2, "served": 10, "served_in_pieces": 2, "declined": {"x": 3}}
    assert vllm_bench.read_stats(str(tmp_path / "none")) is None


def test_vllm_plugin_entry_point_is_discoverable_without_an_installation(tmp_path):
    """pyproject.toml declares the vllm.general_plugins entry point; for runs from the source tree the benchmark driver
    writes the same metadata into a scratch directory, and with that directory and the repository root on PYTHONPATH a
    fresh interpreter (as vLLM's engine and worker processes are) finds and loads the hook."""
    import subprocess
    import sys
    from ooverlap_b200.bench import vllm_bench
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "pyproject.toml")).read()
    assert '[project.entry-points."vllm.general_plugins"]' in text
    assert 'ooverlap_b200 = "ooverlap_b200.parallel.vllm_adapter:install"' in text
    plug = vllm_bench.write_plugin_metadata(str(tmp_path / "plug"))
    code = ("from importlib.metadata import entry_points\n"
            "eps = [e for e in entry_points(group='vllm.general_plugins') if e.name == 'ooverlap_b200']\n"
            "assert len(eps) == 1, eps\n"
            "f = eps[0].load()\n"
            "import os\n"
            "os.environ.pop('VLLM_FORCE_ALLREDUCE_BACKEND', None)\n"
            "assert f() is False  # not forced: the hook leaves vLLM alone\n"
            "print('ok')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([plug, root]))
    out = subprocess.run([sys.executable, "-c", code], cwd="/", env=env, capture_output=True, text=True)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-800:]


def test_stable_tile_waves_over_several_recorded_launches():
    from ooverlap_b200.ops import stable_tile_waves
    # 8 units, waves of 2; launch 2 swaps units inside waves (still stable) and launch 3 moves unit 5 across the
    # boundary between waves 2 and 3
    a = [0, 1, 2, 3, 4, 5, 6, 7]
    b = [1, 0, 3, 2, 5, 4, 7, 6]
    r = stable_tile_waves([a, b], wave=2)
    assert r["waves"] == [0, 0, 1, 1, 2, 2, 3, 3] and r["stable_fraction"] == 1.0 and r["min_group_waves"] == 1
    assert r["hint"] == a
    c = [0, 1, 2, 3, 4, 6, 5, 7]
    r = stable_tile_waves([a, b, c], wave=2)
    assert r["waves"] == [0, 0, 1, 1, 2, -1, -1, 3] and r["stable_fraction"] == 0.75
    assert r["min_group_waves"] == 2          # waves {0,1} and {2,3} hold in every launch
    assert r["hint"][:4] == [0, 1, 2, 3]
    # units that move between waves 1 and 2 break groups of two waves; groups of three ({0,1,2} and {3}) hold
    d = [0, 1, 2, 4, 3, 5, 6, 7]
    assert stable_tile_waves([a, d], wave=2)["min_group_waves"] == 3
    # the records of tile_order() are accepted as they are
    recs = [[dict(unit=u, t_us=float(i), pair=0, index=i) for i, u in enumerate(o)] for o in (a, b)]
    assert stable_tile_waves(recs, wave=2)["stable_fraction"] == 1.0
    assert stable_tile_waves([], wave=2)["hint"] == []
    with pytest.raises(ValueError):
        stable_tile_waves([a, [0, 1, 2]], wave=2)


def test_overlap_tuner_latency_model_orders_the_candidates():
    """The tuner measures candidates in the order its model predicts; the model must rank a fused kernel whose
    reduction hides behind the GEMM ahead of the unfused pair, charge peer traffic more than the switch path, and
    charge the GEMM for the SMs it gives up."""
    from ooverlap_b200.bench.tune_overlap import candidates, predict_us
    cands = candidates([8, 16], [0, 1, 2], ["pair", "one_sm"], 8192, 8)
    assert cands[0]["strategy"] == "unfused" and cands[-1]["strategy"] == "chunked"
    assert not any(c["kernel"] == "pair" and c["use_nvls"] == 2 for c in cands)  # one switch path in the two-SM kernel
    assert len([c for c in cands if c["strategy"] == "fused"]) == 2 * 2 + 2 * 3
    assert all(c["strategy"] != "chunked" for c in candidates([8], [0], ["pair"], 512, 8))
    assert all(c["strategy"] != "chunked" for c in candidates([8], [0], ["pair"], 8192, 2))
    t_ar = {8: 300.0, 16: 290.0}
    p = {(c["strategy"], c["kernel"], c["comm_ctas"], c["use_nvls"]): predict_us(dict(c, slabs=4), 140.0, t_ar, 148, 25.0)
         for c in cands}
    assert p[("unfused", "", 0, 0)] == 140.0 + 290.0
    assert p[("fused", "pair", 16, 1)] == 290.0 + 25.0              # communication-bound: the GEMM hides
    assert p[("fused", "pair", 16, 0)] > p[("fused", "pair", 16, 1)]  # peer stores move 1.75 x the bytes
    assert p[("fused", "pair", 16, 1)] < p[("unfused", "", 0, 0)]
    # compute-bound case: the GEMM pays for the SMs the communication CTAs take
    q8 = predict_us(dict(strategy="fused", kernel="pair", comm_ctas=8, use_nvls=1), 400.0, {8: 100.0}, 148, 10.0)
    q32 = predict_us(dict(strategy="fused", kernel="pair", comm_ctas=32, use_nvls=1), 400.0, {32: 100.0}, 148, 10.0)
    assert q8 == pytest.approx(400.0 * 148 / 140 + 10.0) and q32 > q8


def test_run_manifest_captures_versions_and_the_steering_environment(tmp_path):
    import subprocess
    import sys
    from ooverlap_b200.utils import manifest
    env = {"OOB_LOG_LEVEL": "info", "VLLM_FORCE_ALLREDUCE_BACKEND": "ooverlap", "NCCL_DEBUG": "WARN", "HOME": "/h",
           "CUDA_VISIBLE_DEVICES": "0,1", "VLLM_API_KEY": "abcdef", "VLLM_OOVERLAP_BROKER_KEY": "k1", "PATH": "/bin"}
    got = manifest.captured_env(env)
    assert got == {"CUDA_VISIBLE_DEVICES": "0,1", "NCCL_DEBUG": "WARN", "OOB_LOG_LEVEL": "info",
                   "VLLM_API_KEY": "<6 characters>", "VLLM_FORCE_ALLREDUCE_BACKEND": "ooverlap",
                   "VLLM_OOVERLAP_BROKER_KEY": "k1"}
    m = manifest.run_manifest(["prog", "--x"], {"bench": "b"}, env)
    assert m["argv"] == ["prog", "--x"] and m["bench"] == "b" and m["env"] == got
    assert m["torch"] and m["python"] and "ooverlap_b200" in m["library"] and m["time_utc"].endswith("Z")
    path = tmp_path / "m.json"
    assert manifest.write_manifest(str(path), ["p"])["argv"] == ["p"]
    assert json.load(open(path))["argv"] == ["p"]
    # the vLLM benchmark driver writes one beside its output file, also for a dry run
    out = tmp_path / "v.jsonl"
    res = subprocess.run([sys.executable, "-m", "ooverlap_b200.bench.vllm_bench", "--dry-run", "--model", "tiny", "--tp", "2",
                          "--backends", "pynccl,ooverlap", "--orders", "all", "--out", str(out)],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-800:]
    mf = json.load(open(str(out) + ".manifest.json"))
    assert mf["bench"] == "vllm_throughput" and mf["tp"] == 2 and mf["backends"] == ["pynccl", "ooverlap"]
    assert mf["orders"] == 2 and "--dry-run" in mf["argv"]


def test_plot_kinds_and_the_builtin_svg_writer(tmp_path, capsys):
    import xml.dom.minidom
    sweep = []
    for nbytes, nccl_us, ours_us in ((1024, 16.0, 8.0), (1 << 20, 24.0, 16.0), (64 << 20, 190.0, 160.0)):
        for coll in ("all_reduce", "all_gather"):
            sweep.append({"collective": coll, "impl": "nccl", "algo": "nccl", "bytes": nbytes, "us": nccl_us,
                          "bus_gbs": nbytes / nccl_us / 1e3, "ctas": 0})
            for ctas, f in ((8, 1.0), (32, 1.2)):
                sweep.append({"collective": coll, "impl": "ours", "algo": "twoshot_nvls", "bytes": nbytes, "us": ours_us * f,
                              "bus_gbs": nbytes / (ours_us * f) / 1e3, "ctas": ctas})
    sweep.append({"collective": "all_reduce", "bytes": 1024, "impl": "nccl", "stat": "latency_us", "p50": 17.0})  # no 'us'
    lat = plot.latency_series(sweep)
    assert lat["all_reduce"]["twoshot_nvls"] == [(1024, 8.0), (1 << 20, 16.0), (64 << 20, 160.0)]  # best CTA budget
    eff = plot.efficiency_series(sweep)
    assert [round(v, 3) for _, v in eff["all_reduce"]["nccl"]] == [0.5, 0.667, 0.842]
    assert all(v == 1.0 for _, v in eff["all_gather"]["twoshot_nvls"])
    f = _write(tmp_path / "s.jsonl", sweep)
    for kind in ("sweep", "latency", "efficiency"):
        out = tmp_path / f"{kind}.svg"
        assert plot.main([f, "--kind", kind, "--out", str(out)]) == 0
        doc = xml.dom.minidom.parse(str(out))
        assert len(doc.getElementsByTagName("polyline")) == 4           # two collectives x two labels
        assert len(doc.getElementsByTagName("circle")) == 12
        for c in doc.getElementsByTagName("circle"):
            assert 0 <= float(c.getAttribute("cx")) <= 1040 and 0 <= float(c.getAttribute("cy")) <= 340
        texts = [t.firstChild.data for t in doc.getElementsByTagName("text") if t.firstChild is not None]
        assert "all_reduce" in texts and "twoshot_nvls" in texts and "1Ki" in texts and "64Mi" in texts
    assert plot.main([f, "--kind", "latency"]) == 0
    assert "all_gather nccl 1024:16" in capsys.readouterr().out
    # serving: median over runs and backend orders, grouped bars; a non-.svg name falls back to .svg without matplotlib
    serving = [{"model": "m", "tp": 4, "batch": b, "backend": be, "output_tok_s": v}
               for b, be, v in ((1, "default", 95.0), (1, "ooverlap", 97.0), (1, "ooverlap", 99.0), (64, "default", 1347.0),
                                (64, "ooverlap", 1322.0))]
    assert plot.serving_series(serving)[("m", 4, 1)] == {"default": 95.0, "ooverlap": 98.0}
    g = _write(tmp_path / "v.jsonl", serving)
    try:
        import matplotlib  # noqa: F401
        target, written = tmp_path / "v.svg", tmp_path / "v.svg"
    except ImportError:
        target, written = tmp_path / "v.png", tmp_path / "v.svg"
    assert plot.main([g, "--kind", "serving", "--out", str(target)]) == 0
    doc = xml.dom.minidom.parse(str(written))
    bars = [r for r in doc.getElementsByTagName("rect") if r.getAttribute("fill").startswith("#") and r.getAttribute("height") != "10"]
    assert len(bars) == 4
    ov = _write(tmp_path / "o.jsonl", [{"op": "gemm_ar", "M": 512, "impl": "ours_fused", "nvls": 1, "us": 50.0},
                                       {"op": "gemm_ar", "M": 512, "impl": "cublas+nccl", "us": 80.0}])
    assert plot.main([ov, "--kind", "overlap", "--out", str(tmp_path / "o.svg")]) == 0
    assert "cublas+nccl" in open(tmp_path / "o.svg").read()
