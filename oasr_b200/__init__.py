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


def install(oasr_module) -> dict:
    """Rebind the hot-path operators on an imported reference ``oasr`` package.

    Layers and models of the reference look operators up as module attributes
    at call time (``oasr.gemm(...)``; ``from oasr.functionals.attention import
    fmha`` inside the call), so rebinding the attributes swaps the backend with
    no model or engine edit.  Returns the replaced attributes so a caller can
    restore them.
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
    return saved
