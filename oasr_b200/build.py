"""In-tree build of liboasr_b200.so (sm_100a only) with nvcc.

``python -m oasr_b200.build`` compiles every ``csrc/*.cu`` to an object file and
links one shared library next to the package (``oasr_b200/lib/``).  The library
has no Python or torch dependency: it links the CUDA runtime statically and
resolves the one driver entry point it needs (tensor-map encoding) at run time.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "liboasr_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
    "-I", str(INCLUDE_DIR),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the oasr_b200 library cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    h.update(path.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(INCLUDE_DIR.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, ptxas_info: bool) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    obj = OBJ_DIR / (src.stem + ".o")
    stamp = OBJ_DIR / (src.stem + ".sha")
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    want = _digest(src, " ".join(flags))
    if obj.exists() and stamp.exists() and stamp.read_text() == want and not ptxas_info:
        return obj
    cmd = [_nvcc(), *flags, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if ptxas_info or verbose:
        sys.stderr.write(res.stderr)
    stamp.write_text(want)
    return obj


def build(verbose: bool = False, ptxas_info: bool = False, jobs: int | None = None) -> Path:
    """Compile (if stale) and link the shared library; returns its path."""
    srcs = _sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    jobs = jobs or min(len(srcs), os.cpu_count() or 4)
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, ptxas_info), srcs))
    LIB_DIR.mkdir(exist_ok=True)
    newest = max(o.stat().st_mtime for o in objs)
    if LIB_PATH.exists() and LIB_PATH.stat().st_mtime >= newest:
        return LIB_PATH
    cmd = [_nvcc(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", str(LIB_PATH), *map(str, objs)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
