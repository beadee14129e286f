"""In-tree build of the native library with nvcc for sm_100a.

Every source under ``csrc/`` is compiled with
``-gencode arch=compute_100a,code=sm_100a`` into ``build/obj`` and linked into
``ooverlap_b200/lib/libooverlap_b200.so`` (plus the ``oob_topology`` CLI).  A
stamp file holding a hash of the sources and flags makes the step a no-op when
nothing changed, so a machine that receives the tree with the built library
does not rebuild it.

Capability parity: the reference builds with CMake (CMakeLists.txt:12-129,
src/CMakeLists.txt:169-683) for compute_90a only.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build" / "obj"
LIB_DIR = Path(__file__).resolve().parent / "lib"
LIB = LIB_DIR / "libooverlap_b200.so"
CLI = LIB_DIR / "oob_topology"
STAMP = LIB_DIR / "build.stamp"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
          "-DOOB_BUILDING=1", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put it on PATH)")


def _sources() -> list[Path]:
    srcs = sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cpp") and "cli" not in p.parts)
    return srcs


def _all_inputs() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cpp", ".h", ".cuh"))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + COMMON).encode())
    for p in _all_inputs():
        h.update(str(p.relative_to(ROOT)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    return LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == source_hash()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link; returns the path of the shared library."""
    if not force and is_current():
        return LIB
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    srcs = _sources()
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def compile_one(src: Path) -> Path:
        obj = OBJ / (str(src.relative_to(CSRC)).replace("/", "__") + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *COMMON, *extra, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, srcs))
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fPIC", "-lpthread", "-ldl"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    cli_src = CSRC / "cli" / "topology_cli.cpp"
    cli = [nvcc, "-O2", "-std=c++17", str(cli_src), "-o", str(CLI), f"-L{LIB_DIR}", "-looverlap_b200",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    res = subprocess.run(cli, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"CLI link failed:\n{res.stdout}\n{res.stderr}")
    STAMP.write_text(source_hash() + "\n")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(path)
