"""ctypes binding of liboasr_b200.so (the C-ABI declared in include/oasr_b200.h).

There is no fallback: if the shared library is missing or a symbol cannot be
resolved, importing an operator raises.  Nothing in this module touches a GPU;
loading the library and resolving symbols works on a machine without one.
"""
from __future__ import annotations

import ctypes
import functools
from ctypes import c_char_p, c_double, c_int, c_int64, c_void_p, POINTER, c_uint32
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "liboasr_b200.so"

# Status codes (include/oasr_b200.h: enum oasr_status)
OK = 0
ERR_INVALID = -1
ERR_DTYPE = -2
ERR_ALIGN = -3
ERR_CUDA = -4
ERR_UNSUPPORTED = -5
ERR_DEVICE_WAIT = -6

# dtype ids (enum oasr_dtype)
DT_F32, DT_F16, DT_BF16, DT_FP8_E4M3, DT_INT8 = 0, 1, 2, 3, 4

# activation ids (enum oasr_activation)
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_SWISH, ACT_GELU_ERF = -1, 0, 1, 2, 4

P = c_void_p
I = c_int64

# name -> argtypes (restype is int for all of these)
_SIGNATURES = {
    "oasr_b200_device_status": [POINTER(c_uint32), P],
    "oasr_b200_set_tunable": [c_char_p, c_int],
    "oasr_b200_selftest_bounded_wait": [I, P, P],
    "oasr_b200_layer_norm": [P, P, P, P, I, I, c_double, c_int, P],
    "oasr_b200_layer_norm_activation": [P, P, P, P, I, I, c_double, c_int, c_int, P],
    "oasr_b200_add_layer_norm": [P, P, P, P, P, I, I, c_double, c_double, c_int, P],
    "oasr_b200_add_layer_norm_residual": [P, P, P, P, P, P, I, I, c_double, c_double, c_int, P],
    "oasr_b200_rms_norm": [P, P, P, P, I, I, c_double, c_int, P],
    "oasr_b200_rms_norm_activation": [P, P, P, P, I, I, c_double, c_int, c_int, P],
    "oasr_b200_add_rms_norm": [P, P, P, P, P, I, I, c_double, c_double, c_int, P],
    "oasr_b200_add_rms_norm_residual": [P, P, P, P, P, P, I, I, c_double, c_double, c_int, P],
    "oasr_b200_batch_norm": [P, P, P, P, P, P, I, I, c_double, c_int, c_int, P],
    "oasr_b200_add_norm_f32": [P, P, P, P, c_double, c_int, P, P, P, P, I, I, c_double, c_int, c_int, P],
    "oasr_b200_gemm_dup_first": [P, P, P, P, I, I, I, I, c_int, P],
    "oasr_b200_add_norm_f32_q8": [P, P, P, P, c_double, c_int, P, P, P, P, I, I, c_double, c_int, P, P, c_int, c_int, P],
    "oasr_b200_gemm_add_norm_f32": [P, P, P, P, P, P, I, I, I, c_double, c_int, P, P, P, P, c_double, c_int, c_int, P],
    "oasr_b200_gemm_add_norm_supported": [I, I],
    "oasr_b200_gemm_dup_first_supported": [I, I, I],
    "oasr_b200_ctc_greedy_collapse": [P, P, P, P, P, I, I, I, P],
    "oasr_b200_fbank": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, c_double, c_double, P],
    "oasr_b200_trace_buffer": [P],
    "oasr_b200_depthwise_conv1d_packed": [P, P, P, P, P, P, P, P, P, I, I, I, I, c_int, c_int, P],
    "oasr_b200_fmha_varlen_relpos": [P, P, P, I, I, P, I, I, I, I, c_double, c_int, P],
    "oasr_b200_fmha_varlen_relpos_planned": [P, P, P, I, I, P, I, I, I, I, c_double, P, c_int, P],
    "oasr_b200_fmha_relpos_plan": [P, I, P, I, I, I, P],
    "oasr_b200_fmha_paged_relpos": [P, P, P, P, P, I, I, P, P, P, I, I, I, I, I, I, c_double, c_int, P],
    "oasr_b200_depthwise_conv1d_affine": [P, P, P, P, P, P, I, I, I, I, I, I, c_int, c_int, P],
    "oasr_b200_conv_state_concat": [P, P, I, P, P, I, I, I, I, c_int, P],
    "oasr_b200_glu": [P, P, I, I, c_int, P],
    "oasr_b200_swish": [P, P, I, c_int, P],
    "oasr_b200_depthwise_conv1d": [P, P, P, P, I, I, I, I, I, I, P, c_int, c_int, c_int, c_int, P],
    "oasr_b200_causal_conv1d": [P, P, P, P, P, I, I, I, I, c_int, P],
    "oasr_b200_fmha_paged_relpos_fp8": [P, P, P, P, P, P, P, I, I, P, P, P, I, I, I, I, I, I, c_double, c_int, P],
    "oasr_b200_paged_kv_write_fp8": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, c_int, P],
    "oasr_b200_gemm_q8": [P, P, P, P, P, P, I, I, I, c_int, c_int, c_int, c_int, P],
    "oasr_b200_quantize_rows": [P, P, P, I, I, c_int, c_int, P],
    "oasr_b200_subsample_conv1": [P, P, P, P, P, I, I, I, I, I, I, c_int, P],
    "oasr_b200_relshift_bias_stream": [P, P, P, P, I, I, I, I, I, I, I, c_double, I, I, c_double, c_int, P],
    "oasr_b200_relshift_bias": [P, P, P, I, I, I, I, I, I, I, c_double, I, I, c_double, c_int, P],
    "oasr_b200_depthwise_conv2d_k3s2": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, c_int, P],
    "oasr_b200_subsample_conv1_s2d": [P, P, P, P, P, I, I, I, I, c_int, P],
    "oasr_b200_subsample_conv2": [P, P, P, P, P, I, I, I, I, I, I, c_int, P],
    "oasr_b200_gemm": [P, P, P, P, I, I, I, c_int, c_int, P],
    "oasr_b200_gemm_residual_f32": [P, P, P, P, P, I, I, I, c_double, c_int, P],
    "oasr_b200_gemm_glu": [P, P, P, P, I, I, I, c_int, P],
    "oasr_b200_bmm": [P, P, P, I, I, I, I, c_int, P],
    "oasr_b200_group_gemm": [P, P, P, P, I, I, I, I, c_int, P],
    "oasr_b200_gemm_log_softmax": [P, P, P, P, I, I, I, c_int, c_int, P, P],
    "oasr_b200_fmha": [P, P, P, P, P, P, P, P, I, I, I, P, P, P, I, I, I, I, I, I, I, I, I, c_double, c_int, c_int, P],
    "oasr_b200_depthwise_conv1d_packed_causal": [P, P, P, P, P, I, I, I, I, c_int, c_int, P],
    "oasr_b200_relshift_bias_packed": [P, P, P, P, I, I, I, I, I, c_double, I, I, c_double, c_int, P],
    "oasr_b200_fmha_varlen_strided": [P, P, P, P, I, I, I, P, P, c_int, c_int, P, P, I, I, I, I, I, I, I, c_double, c_int, P],
    "oasr_b200_bmm_strided": [P, P, P, I, I, I, I, I, I, I, I, c_int, P],
    "oasr_b200_fmha_bthd": [P, P, P, P, P, P, P, P, I, I, I, P, P, P, I, I, I, I, I, I, I, I, I, c_double, c_int, c_int, P],
    "oasr_b200_fmha_varlen": [P, P, P, P, P, P, c_int, P, P, I, I, I, I, I, I, I, c_double, c_int, P],
    "oasr_b200_paged_kv_write": [P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, c_int, P],
    "oasr_b200_paged_kv_gather": [P, P, P, P, P, I, I, I, I, I, I, c_int, P],
    "oasr_b200_gather_rows": [P, P, P, I, I, I, P],
    "oasr_b200_scatter_rows": [P, P, P, I, I, I, P],
}



class ConformerLayer(ctypes.Structure):
    """struct oasr_b200_conformer_layer (include/oasr_b200.h)."""

    _fields_ = [(n, c_void_p) for n in (
        "norm_ff_macaron_w", "norm_ff_macaron_b", "ffm_w1", "ffm_b1", "ffm_w2", "ffm_b2", "norm_mha_w", "norm_mha_b",
        "qkv4_w", "qkv4_b", "out_w", "out_b", "norm_conv_scale", "norm_conv_shift", "pw1_w", "pw1_b", "dw_w", "dw_b",
        "conv_bn_scale", "conv_bn_shift", "glu_of_bias", "pw2_w", "pw2_b", "norm_ff_w", "norm_ff_b", "ff_w1", "ff_b1",
        "ff_w2", "ff_b2", "norm_final_w", "norm_final_b")] + [("q_w", c_void_p * 8), ("q_s", c_void_p * 8)]


class ConformerModel(ctypes.Structure):
    """struct oasr_b200_conformer_model (include/oasr_b200.h)."""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "d_model", "heads", "ffn", "kernel", "num_layers", "vocab_padded", "embed_in", "dtype")] + [
        ("eps", c_double), ("layers", POINTER(ConformerLayer)),
        ("embed_w", c_void_p), ("embed_b", c_void_p), ("embed_ln_w", c_void_p), ("embed_ln_b", c_void_p),
        ("pos_w_all", c_void_p), ("pe", c_void_p), ("pe_rows", c_int64),
        ("after_norm_w", c_void_p), ("after_norm_b", c_void_p), ("ctc_w", c_void_p), ("ctc_b", c_void_p),
        ("pos_proj", c_void_p), ("pos_proj_rows", c_int64), ("quant_kind", ctypes.c_int32)]


class FastConformerLayer(ctypes.Structure):
    """struct oasr_b200_fastconformer_layer (include/oasr_b200.h)."""

    _fields_ = [(n, c_void_p) for n in (
        "norm_ff1_w", "norm_ff1_b", "ff1_w1", "ff1_b1", "ff1_w2", "ff1_b2", "norm_att_w", "norm_att_b", "qkv4_w", "qkv4_b",
        "rel_w", "o_w", "o_b", "norm_conv_w", "norm_conv_b", "pw1_w", "pw1_b", "dw_w", "dw_b", "conv_norm_w", "conv_norm_b",
        "pw2_w", "pw2_b", "norm_ff2_w", "norm_ff2_b", "ff2_w1", "ff2_b1", "ff2_w2", "ff2_b2", "norm_out_w", "norm_out_b")] + [
        ("q_w", c_void_p * 8), ("q_s", c_void_p * 8)]


class FastConformerModel(ctypes.Structure):
    """struct oasr_b200_fastconformer_model (include/oasr_b200.h)."""

    _fields_ = [(n, ctypes.c_int32) for n in (
        "hidden", "heads", "ffn", "kernel", "num_layers", "dtype", "left_context", "right_context")] + [
        ("eps", c_double), ("mask_floor", c_double), ("layers", POINTER(FastConformerLayer)), ("quant_kind", ctypes.c_int32)]


_SIGNATURES["oasr_b200_fastconformer_layers_packed"] = [POINTER(FastConformerModel), P, c_int, P, P, I, P, P, I, I, I, I, P, I, P]
_SIGNATURES["oasr_b200_conformer_encode_packed"] = [POINTER(ConformerModel), P, P, P, I, I, I, P, I, P, P, P]

_SIGNATURES["oasr_b200_conformer_encode_packed_noalloc"] = [POINTER(ConformerModel), P, P, P, I, I, I, P, P, P]
_SIGNATURES["oasr_b200_conformer_chunk_paged"] = [POINTER(ConformerModel), P, I, I, POINTER(c_void_p), POINTER(c_void_p),
                                                 P, P, P, P, I, I, I, P, P, I, P, P, I, P, P, P]
_SIGNATURES["oasr_b200_profile_enable"] = [c_int]
_SIGNATURES["oasr_b200_profile_get"] = [c_int, POINTER(c_char_p), POINTER(c_double), POINTER(c_double)]

_STRING_FUNCS = ("oasr_b200_version", "oasr_b200_last_error")


class OasrB200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


@functools.cache
def load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m oasr_b200.build` "
            "(needs nvcc); there is no fallback path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name in _STRING_FUNCS:
        fn = getattr(lib, name)
        fn.restype = c_char_p
        fn.argtypes = []
    lib.oasr_b200_launch_count.restype = ctypes.c_ulonglong
    lib.oasr_b200_launch_count.argtypes = []
    lib.oasr_b200_conformer_noalloc_capacity_bytes.restype = c_int64
    lib.oasr_b200_conformer_noalloc_capacity_bytes.argtypes = []
    lib.oasr_b200_conformer_chunk_workspace_bytes.restype = c_int64
    lib.oasr_b200_conformer_chunk_workspace_bytes.argtypes = [POINTER(ConformerModel), I, I]
    lib.oasr_b200_profile_count.restype = c_int
    lib.oasr_b200_profile_count.argtypes = []
    lib.oasr_b200_conformer_workspace_bytes.restype = c_int64
    lib.oasr_b200_conformer_workspace_bytes.argtypes = [POINTER(ConformerModel), I, I]
    lib.oasr_b200_fmha_relpos_plan_bytes.restype = c_int64
    lib.oasr_b200_fmha_relpos_plan_bytes.argtypes = [I, I, I]
    lib.oasr_b200_fastconformer_workspace_bytes.restype = c_int64
    lib.oasr_b200_fastconformer_workspace_bytes.argtypes = [POINTER(FastConformerModel), I, I, I]
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:  # pragma: no cover - a broken build
            raise RuntimeError(f"{LIB_PATH} does not export {name}") from e
        fn.restype = c_int
        fn.argtypes = argtypes
    return lib


def exported_names() -> list[str]:
    return list(_STRING_FUNCS) + ["oasr_b200_launch_count", "oasr_b200_conformer_workspace_bytes", "oasr_b200_profile_count",
                                  "oasr_b200_conformer_noalloc_capacity_bytes", "oasr_b200_conformer_chunk_workspace_bytes",
                                  "oasr_b200_fastconformer_workspace_bytes", "oasr_b200_fmha_relpos_plan_bytes"] + list(_SIGNATURES)


def launch_count() -> int:
    """Kernels launched through the library by this process so far."""
    return int(load().oasr_b200_launch_count())


# Optional per-call observer used by bench.py to time kernels with CUDA events:
# called as hook(name, phase) with phase "begin" / "end" around every C-ABI call.
_call_hook = None


def set_call_hook(hook) -> None:
    global _call_hook
    _call_hook = hook


def last_error() -> str:
    return load().oasr_b200_last_error().decode()


def check(code: int) -> None:
    """Raise the reference-style exception for a failing status."""
    if code == OK:
        return
    msg = last_error()
    if code in (ERR_INVALID, ERR_ALIGN, ERR_DTYPE, ERR_UNSUPPORTED):
        # The reference reports launcher validation failures as RuntimeError
        # (TVM_FFI_ICHECK, csrc/tvm_ffi_utils.h:36-106).
        raise OasrB200Error(code, msg)
    raise OasrB200Error(code, msg)


def call(name: str, *args) -> None:
    if _call_hook is None:
        check(getattr(load(), name)(*args))
        return
    _call_hook(name, "begin", args)
    try:
        check(getattr(load(), name)(*args))
    finally:
        _call_hook(name, "end", args)


def profile_steps(run) -> list:
    """Run ``run()`` once with the native executor's per-step CUDA-event timing on; returns
    ``[(label, ms, flops), ...]`` in launch order."""
    lib = load()
    call("oasr_b200_profile_enable", 1)
    try:
        run()
        out = []
        for i in range(lib.oasr_b200_profile_count()):
            label, ms, fl = c_char_p(), c_double(), c_double()
            call("oasr_b200_profile_get", i, ctypes.byref(label), ctypes.byref(ms), ctypes.byref(fl))
            out.append((label.value.decode(), ms.value, fl.value))
        return out
    finally:
        call("oasr_b200_profile_enable", 0)


def version() -> str:
    return load().oasr_b200_version().decode()
