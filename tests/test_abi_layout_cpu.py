"""The ctypes structures of ``ooverlap_b200._lib`` must have the layout of the C structs in ``csrc/api``:
a host compiler prints sizeof / offsetof for every field and the numbers are compared with ctypes."""
import ctypes
import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

PAIRS = [("oob_comm_info_t", "CommInfo"), ("oob_device_status_t", "DeviceStatus"), ("oob_norm_args_t", "NormArgs"),
         ("oob_gemm_args_t", "GemmArgs"), ("oob_rope_args_t", "RopeArgs"), ("oob_attn_decode_args_t", "AttnDecodeArgs"),
         ("oob_gemm_epilogue_swiglu_t", "SwigluEpilogue")]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_ctypes_structures_match_the_c_headers(tmp_path):
    from ooverlap_b200 import _lib
    lines = ['#include <cstddef>', '#include <cstdio>', '#include "oob.h"', '#include "oob_model.h"', 'int main() {',
             '  printf("{");']
    first = True
    for c_name, py_name in PAIRS:
        st = getattr(_lib, py_name)
        lines.append(f'  printf("{"" if first else ","}\\"{c_name}\\": {{\\"sizeof\\": %zu", sizeof({c_name}));')
        first = False
        for fname, _ in st._fields_:
            lines.append(f'  printf(", \\"{fname}\\": %zu", offsetof({c_name}, {fname}));')
        lines.append('  printf("}");')
    lines += ['  printf("}\\n");', '  return 0;', '}']
    src = tmp_path / "layout.cpp"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "csrc", "api"), str(src), "-o", str(exe)], check=True)
    c_layout = json.loads(subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout)
    for c_name, py_name in PAIRS:
        st = getattr(_lib, py_name)
        assert ctypes.sizeof(st) == c_layout[c_name]["sizeof"], (c_name, ctypes.sizeof(st), c_layout[c_name]["sizeof"])
        for fname, _ in st._fields_:
            assert getattr(st, fname).offset == c_layout[c_name][fname], (c_name, fname)


def test_every_declared_entry_point_is_exported():
    """Each function declared in csrc/api/*.h must be a symbol of the built library (and so loadable by ctypes)."""
    import re
    from ooverlap_b200 import _lib
    lib = _lib.lib()
    names = set()
    for header in ("oob.h", "oob_model.h", "oob_noalloc.h"):
        text = open(os.path.join(ROOT, "csrc", "api", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(oob_[a-z0-9_]+)\s*\(", text))
    assert len(names) > 40
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing


def test_planning_helpers_on_cpu():
    """Host-side planning used by the GPU paths: split counts and chunking never produce empty or oversized work."""
    from ooverlap_b200 import _lib
    from ooverlap_b200.ops import gemm_plan_splits
    lib = _lib.lib()
    for M, N, K in [(1, 1280, 8192), (64, 7168, 8192), (256, 8192, 3584), (512, 8192, 8192), (8192, 8192, 8192), (1, 256, 64)]:
        s = gemm_plan_splits(M, N, K)
        num_kb = (K + 63) // 64
        assert 1 <= s <= max(1, num_kb)
        per = (num_kb + s - 1) // s
        assert (s - 1) * per < num_kb  # no split is empty
        assert gemm_plan_splits(M, N, K, splits=1) == 1
    assert gemm_plan_splits(8192, 8192, 8192) == 1 and gemm_plan_splits(1, 1280, 8192) > 1
    for B, KV, bound in [(1, 1, 1152), (64, 1, 1152), (256, 1, 1152), (1, 8, 128), (3, 2, 70000)]:
        s = lib.oob_attn_decode_auto_splits(B, KV, bound)
        assert 1 <= s <= 32 and s <= (bound + 127) // 128
        assert lib.oob_attn_decode_workspace_bytes(B, 8, s) == (0 if s == 1 else B * 8 * s * 130 * 4)
