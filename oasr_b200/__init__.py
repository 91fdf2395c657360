"""oasr_b200 -- the Conformer/FastConformer encoder + CTC hot path of OASR on B200 (sm_100a).

The package exposes the reference's operator names (``oasr_b200.gemm``,
``oasr_b200.fmha_varlen``, ``oasr_b200.add_layer_norm_residual`` ...) backed by
hand-written CUDA kernels behind a C-ABI (``include/oasr_b200.h``,
``liboasr_b200.so``).  ``install(oasr)`` rebinds those names on an imported
reference package so its layers, models and engine run on these kernels.
"""
from __future__ import annotations

from . import _lib
from .attention import fmha, fmha_varlen, gather_paged_kv  # noqa: F401
from .cache import PagedKVCache, gather_rows, scatter_rows, write_kv_chunk  # noqa: F401
from .functional import (  # noqa: F401
    add_layer_norm,
    add_layer_norm_residual,
    add_rms_norm,
    add_rms_norm_residual,
    batch_norm_1d,
    batch_norm_activation,
    batch_norm_swish,
    bmm,
    causal_conv1d,
    depthwise_conv1d,
    depthwise_conv1d_silu,
    device_status,
    gemm,
    gemm_activation,
    gemm_glu,
    gemm_log_softmax,
    gemm_residual_f32,
    get_activation_type_id,
    glu,
    group_gemm,
    layer_norm,
    layer_norm_activation,
    rms_norm,
    rms_norm_activation,
    swish,
)

__version__ = "0.1.0"

# Names rebound by install(): exactly the reference's flat ``oasr.*`` operator
# namespace for this path (oasr/__init__.py:32-123 in the reference).
OPERATOR_NAMES = (
    "gemm", "gemm_activation", "gemm_log_softmax", "group_gemm", "bmm",
    "layer_norm", "rms_norm", "add_layer_norm", "add_layer_norm_residual",
    "add_rms_norm", "add_rms_norm_residual", "layer_norm_activation", "rms_norm_activation",
    "batch_norm_1d", "batch_norm_activation", "batch_norm_swish",
    "glu", "swish", "depthwise_conv1d", "depthwise_conv1d_silu", "causal_conv1d",
)


def install(oasr_module, lift_row_floor: bool = False) -> dict:
    """Rebind the hot-path operators on an imported reference ``oasr`` package.

    Layers and models of the reference look operators up as module attributes
    at call time (``oasr.gemm(...)``; ``from oasr.functionals.attention import
    fmha`` inside the call), so rebinding the attributes swaps the backend with
    no model or engine edit.  Returns the replaced attributes so a caller can
    restore them (``uninstall``).

    ``lift_row_floor``: the reference's layers send projections of fewer than
    ``GEMM_MIN_ROWS`` (128) rows to ``F.linear`` because its tiled kernel loses
    to cuBLAS there (oasr/layers/_backend.py:293-320); the kernels here take any
    row count, so the floor can be set to 0 (streaming chunks of a few streams
    then stay on this library too).
    """
    import sys

    _lib.load()  # fail here, loudly, if the library is missing
    this = sys.modules[__name__]
    saved = {}
    for name in OPERATOR_NAMES:
        if hasattr(this, name):
            saved[name] = getattr(oasr_module, name, None)
            setattr(oasr_module, name, getattr(this, name))
    attn = getattr(getattr(oasr_module, "functionals", None), "attention", None)
    for name in ("fmha", "fmha_varlen"):
        if hasattr(this, name):
            if attn is not None:
                saved["functionals.attention." + name] = getattr(attn, name, None)
                setattr(attn, name, getattr(this, name))
            saved[name] = getattr(oasr_module, name, None)
            setattr(oasr_module, name, getattr(this, name))
    if lift_row_floor:
        backend = getattr(getattr(oasr_module, "layers", None), "_backend", None)
        if backend is not None and hasattr(backend, "GEMM_MIN_ROWS"):
            saved["layers._backend.GEMM_MIN_ROWS"] = backend.GEMM_MIN_ROWS
            backend.GEMM_MIN_ROWS = 0
    return saved


def uninstall(oasr_module, saved: dict) -> None:
    """Put back what ``install`` replaced (``saved`` is its return value)."""
    attn = getattr(getattr(oasr_module, "functionals", None), "attention", None)
    for key, value in saved.items():
        if key == "layers._backend.GEMM_MIN_ROWS":
            oasr_module.layers._backend.GEMM_MIN_ROWS = value
            continue
        target, name = (attn, key.rsplit(".", 1)[1]) if key.startswith("functionals.attention.") else (oasr_module, key)
        if target is None:
            continue
        if value is None:
            if hasattr(target, name):
                delattr(target, name)
        else:
            setattr(target, name, value)
