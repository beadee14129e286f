"""The tuning-policy parser and selector (host-only C++) under AddressSanitizer + UBSan, fed the packaged policy,
truncations of it and random mutations (tests/native/policy_fuzz.cpp): any verdict is fine, memory errors are not."""
import os
import random
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA_INC = "/usr/local/cuda/include"


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and the CUDA headers")
def test_policy_parser_under_sanitizers(tmp_path):
    exe = tmp_path / "policy_fuzz"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-I", CUDA_INC,
           os.path.join(ROOT, "tests", "native", "policy_fuzz.cpp"), os.path.join(ROOT, "csrc", "runtime", "policy.cpp"),
           os.path.join(ROOT, "csrc", "runtime", "log.cpp"),
           "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True)
    if built.returncode != 0 and "sanitize" in (built.stderr or ""):
        pytest.skip("sanitizer runtime not available")
    assert built.returncode == 0, built.stderr[-2000:]
    good = open(os.path.join(ROOT, "ooverlap_b200", "policy", "b200_nvswitch.json")).read()
    rng = random.Random(1234)
    files = []

    def emit(name, text):
        path = tmp_path / name
        path.write_bytes(text if isinstance(text, bytes) else text.encode("utf-8", "ignore"))
        files.append(str(path))

    emit("good.json", good)
    emit("empty.json", "")
    emit("not_json.json", "policy: yes\n")
    emit("deep.json", "[" * 5000)
    emit("huge_numbers.json", '{"points": [{"world_size": 99999999999999999999, "collective": "all_reduce", "bytes": 1e999, '
                              '"nvls": -1, "ranked": [["x", 1e30]]}]}')
    for i in range(40):
        emit(f"trunc_{i}.json", good[: rng.randrange(1, len(good))])
    alphabet = '{}[]":,0123456789.eE-+ \n\\ntruefalsnul'
    for i in range(60):
        chars = list(good)
        for _ in range(rng.randrange(1, 30)):
            pos = rng.randrange(len(chars))
            op = rng.randrange(3)
            if op == 0:
                chars[pos] = rng.choice(alphabet)
            elif op == 1:
                del chars[pos]
            else:
                chars.insert(pos, rng.choice(alphabet))
        emit(f"mut_{i}.json", "".join(chars))
    emit("binary.json", bytes(rng.randrange(256) for _ in range(4096)))
    files.append(str(tmp_path / "does_not_exist.json"))
    run = subprocess.run([str(exe), *files], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="halt_on_error=1"))
    assert run.returncode == 0 and run.stdout.startswith("ok loaded="), (run.stdout[-300:], run.stderr[-3000:])
    loaded = int(run.stdout.split("loaded=")[1].split()[0])
    assert loaded >= 1  # at least the packaged policy parses
