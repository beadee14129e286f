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
