"""Process-wide integer tunables of the native library (tile shapes etc.).

``gemm_bn``: 0 lets the heuristic choose the GEMM tile width, 64 / 128 / 256 force it.
``gemm_pairs``: 1 runs large dense GEMMs on CTA pairs (tcgen05 cta_group::2), 0 (default) on single-CTA tiles.
"""
from __future__ import annotations

from . import _lib


def set(name: str, value: int) -> None:  # noqa: A001 - mirrors the C entry point's name
    _lib.call("oasr_b200_set_tunable", name.encode(), int(value))
