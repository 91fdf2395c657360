"""Process-wide integer tunables of the native library (tile shapes etc.).

``gemm_bn``: 0 lets the heuristic choose the GEMM tile width, 64 / 128 / 256 force it.
"""
from __future__ import annotations

from . import _lib


def set(name: str, value: int) -> None:  # noqa: A001 - mirrors the C entry point's name
    _lib.call("oasr_b200_set_tunable", name.encode(), int(value))
