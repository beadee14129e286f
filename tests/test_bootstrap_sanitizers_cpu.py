"""The rendezvous code (host-only C++) under AddressSanitizer + UBSan and under ThreadSanitizer: ranks run as
threads of one process through every primitive for many rounds (tests/native/bootstrap_stress.cpp)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build_and_run(tmp_path, name, flags, env=None):
    exe = tmp_path / name
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread", *flags, os.path.join(ROOT, "tests", "native", "bootstrap_stress.cpp"),
           os.path.join(ROOT, "csrc", "runtime", "bootstrap.cpp"), "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True)
    if built.returncode != 0 and "sanitize" in (built.stderr or ""):
        pytest.skip("sanitizer runtime not available: " + built.stderr[-200:])
    assert built.returncode == 0, built.stderr[-2000:]
    run = subprocess.run([str(exe), "4", "12"], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, **(env or {})))
    assert run.returncode == 0 and "ok 4 ranks" in run.stdout, (run.stdout[-500:], run.stderr[-3000:])
    return run


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_bootstrap_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    _build_and_run(tmp_path, "stress_asan", ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"],
                   {"ASAN_OPTIONS": "detect_leaks=1:abort_on_error=0", "UBSAN_OPTIONS": "halt_on_error=1"})


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_bootstrap_under_thread_sanitizer(tmp_path):
    run = _build_and_run(tmp_path, "stress_tsan", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1"})
    assert "WARNING: ThreadSanitizer" not in run.stderr
