"""Recipe for ``oracle/_ref``: an importable copy of the reference's pure-Python package.
TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [<reference checkout>]        (default: $OASR_REFERENCE, else DEFAULT_CHECKOUT below)

The reference's implementation of this path is Python/PyTorch (``oasr/models``, ``oasr/layers``,
``oasr/functionals``, ``oasr/cache``); its CUDA kernels need a CUTLASS submodule that is absent, so
nothing is compiled.  The recipe copies the ``oasr`` package directory as it lies in the checkout
into ``oracle/_ref/oasr`` (git-ignored: the copy never enters history, it only travels with the
working tree to the machine that runs the GPU tests).  Two users:

* ``bench.py --impl reference`` times the reference's own ``ConformerModel.forward_offline_packed``
  on the host cores (torch backend, fp32) when the copy is present, else the CPU port;
* ``tests/test_gpu_install.py`` imports it, calls ``oasr_b200.install(oasr)`` and runs the
  reference's own model on the kernels of this repository.

``load()`` imports the copy with the settings the reference documents for its CPU/torch route
(``OASR_LAYERS_BACKEND``, ``OASR_FUSED_ADDNORM``); it never touches ``sys.path`` permanently.
"""
from __future__ import annotations

import importlib
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"


DEFAULT_CHECKOUT = "/root/reference"   # where the build container mounts the reference checkout

def available() -> bool:
    return (DEST / "oasr" / "__init__.py").exists()


def make(reference: str | None = None) -> Path | None:
    """Copy ``<reference>/oasr`` to ``oracle/_ref/oasr``; returns the destination, or None when the
    checkout is not on this machine (then an existing copy is left as it is)."""
    src = Path(reference or os.environ.get("OASR_REFERENCE") or DEFAULT_CHECKOUT) / "oasr"
    if not (src / "__init__.py").exists():
        return None
    dst = DEST / "oasr"
    if dst.exists():
        shutil.rmtree(dst)
    DEST.mkdir(exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so", "*.o"))
    return dst


def load(backend: str = "torch"):
    """Import the copied reference package.  ``backend="torch"`` selects its torch route (CPU oracle
    runs); ``backend="oasr"`` leaves its kernel route on, for a run with the operators rebound."""
    if not available():
        raise RuntimeError("oracle/_ref/oasr is missing: run `python oracle/make_ref.py` where the reference checkout is")
    if "oasr" in sys.modules:
        mod = sys.modules["oasr"]
        if Path(getattr(mod, "__file__", "")).resolve().parent != (DEST / "oasr").resolve():
            raise RuntimeError("another 'oasr' package is already imported")
        return mod
    os.environ["OASR_LAYERS_BACKEND"] = backend
    os.environ["OASR_FUSED_ADDNORM"] = "0" if backend == "torch" else os.environ.get("OASR_FUSED_ADDNORM", "1")
    sys.path.insert(0, str(DEST))
    try:
        return importlib.import_module("oasr")
    finally:
        sys.path.remove(str(DEST))


if __name__ == "__main__":
    out = make(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "reference checkout not found; nothing copied")
