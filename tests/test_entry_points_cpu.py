"""The parts of the benchmark and build contract that run without a GPU: the reference arm's one-line answer, the
refusal of a multi-GPU request outside a launcher, and the build entry point (a no-op when the stamp is current)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.pop("RANK", None)
    e.pop("WORLD_SIZE", None)
    if env:
        e.update(env)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, env=e,
                          cwd=ROOT, timeout=300)


def test_reference_arm_prints_one_json_line_and_exits_zero():
    res = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert res.returncode == 0, res.stderr[-500:]
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and "\n" not in rec["unavailable"] and len(rec["unavailable"]) > 20
    # launched as several ranks, only rank 0 answers
    res = _run("--impl", "reference", "--gpus", "2", env={"RANK": "1", "WORLD_SIZE": "2"})
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_bench_defaults_are_the_single_gpu_run():
    sys.path.insert(0, ROOT)
    try:
        import bench
        old = sys.argv
        sys.argv = ["bench.py"]
        try:
            a = bench.parse_args()
        finally:
            sys.argv = old
        assert a.gpus == 1 and a.impl == "ours" and a.warmup >= 3 and a.steps >= 1 and a.strategy == "autotune"
        assert bench.MS == (512, 2048, 8192) and bench.N_DIM == 8192 and bench.K_DIM == 8192
    finally:
        sys.path.remove(ROOT)


def test_build_entry_point_is_a_no_op_when_current():
    sys.path.insert(0, ROOT)
    try:
        import __graft_entry__ as entry
        entry.build()   # compiles when sources changed, else returns at once; either way the library then loads
        from ooverlap_b200 import _lib
        assert b"sm_100a" in _lib.lib().oob_version()
    finally:
        sys.path.remove(ROOT)


def test_multi_gpu_request_outside_a_launcher_is_refused_before_any_cuda_call():
    res = _run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert res.returncode == 2 and "torch.distributed.run" in res.stderr
