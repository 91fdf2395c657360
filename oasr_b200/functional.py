"""Operator API of the encoder hot path, with the reference's signatures.

Every function here has the name, argument meaning, default values and error
behaviour of the function of the same name in the reference's
``oasr/functionals/*.py`` (cited per function) and launches hand-written
sm_100a kernels through the C-ABI in ``include/oasr_b200.h``.  Tensors must be
CUDA tensors; there is no CPU path.  Outputs are allocated here (``out=`` is
honoured and returned), kernels run on the current CUDA stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple, Union

import torch

from . import _lib
from ._lib import ACT_NONE, ACT_SWISH, DT_BF16, DT_F16, DT_F32

_DTYPE_ID = {torch.float32: DT_F32, torch.float16: DT_F16, torch.bfloat16: DT_BF16}

# activation names accepted by the reference (oasr/functionals/activation.py:13-25)
ACTIVATION_IDS = {"relu": 0, "gelu": 1, "gelu_tanh": 1, "swish": 2, "silu": 2, "gelu_erf": 4}


def _dt(t: torch.Tensor, allowed=(torch.float32, torch.float16, torch.bfloat16)) -> int:
    if t.dtype not in allowed:
        raise RuntimeError(f"unsupported dtype {t.dtype}; expected one of {allowed}")
    return _DTYPE_ID[t.dtype]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    """The caller's current stream on the tensor's device.  The library launches on the CURRENT device (its SM count,
    status word and tensor maps are per current device), so a tensor that lives on another GPU is refused here rather
    than launched against the wrong context."""
    if t.device.index is not None and t.device.index != torch.cuda.current_device():
        raise RuntimeError(f"tensor on {t.device} but the current CUDA device is cuda:{torch.cuda.current_device()}: "
                           f"wrap the call in `with torch.cuda.device({t.device.index}):`")
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("Input must be a CUDA tensor (oasr_b200 has no CPU path)")


def _same_dtype(ref: torch.Tensor, **others) -> None:
    for name, t in others.items():
        if t is not None and t.dtype != ref.dtype:
            raise RuntimeError(f"{name} must have dtype {ref.dtype}, got {t.dtype}")


def _is_row_dense(x: torch.Tensor) -> bool:
    """Rows (trailing dim) tile storage without gaps or overlap
    (the reference's IsRowDense, csrc/tvm_ffi_utils.h:63-79)."""
    n = x.dim()
    if n < 1 or (x.size(-1) > 1 and x.stride(-1) != 1):
        return False
    span = 1
    for extent, stride in zip(x.shape, x.stride()):
        if extent > 1 and stride <= 0:
            return False
        span += (extent - 1) * stride
    return span == x.numel()


def _check_rows(x: torch.Tensor, *same_layout: Optional[torch.Tensor]) -> None:
    if not _is_row_dense(x):
        raise RuntimeError(
            "Tensor rows must tile memory exactly (trailing dim contiguous, no padded row stride); "
            "a row-wise kernel walks `base + row * row_len`"
        )
    for o in same_layout:
        if o is None:
            continue
        if o.shape != x.shape or (o.stride() != x.stride() and not (o.is_contiguous() and x.is_contiguous())):
            raise RuntimeError("Tensors must have identical shape and strides")


def _param_check(hidden: int, ref: torch.Tensor, **params) -> None:
    for name, t in params.items():
        if t is None:
            continue
        if t.numel() != hidden:
            raise RuntimeError(f"{name} must have {hidden} elements, got {t.numel()}")
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
        if t.dtype != ref.dtype:
            raise RuntimeError(f"{name} must have dtype {ref.dtype}, got {t.dtype}")


def _rows_hidden(x: torch.Tensor) -> Tuple[int, int]:
    hidden = x.size(-1)
    return (x.numel() // hidden if hidden else 0), hidden


# ---------------------------------------------------------------------------
# Norms (reference: oasr/functionals/norm.py)
# ---------------------------------------------------------------------------
def layer_norm(input, weight, bias=None, eps: float = 1e-5, out=None):
    """LayerNorm over the last dim (reference: functionals/norm.py:20-43)."""
    _need_cuda(input, weight, bias, out)
    if out is None:
        out = torch.empty_like(input)
    _check_rows(input, out)
    rows, hidden = _rows_hidden(input)
    _param_check(hidden, input, weight=weight, bias=bias)
    _lib.call("oasr_b200_layer_norm", _p(out), _p(input), _p(weight), _p(bias), rows, hidden, float(eps),
              _dt(input), _stream(input))
    return out


def rms_norm(input, weight, bias=None, eps: float = 1e-5, out=None):
    """RMSNorm over the last dim (reference: functionals/norm.py:46-68)."""
    _need_cuda(input, weight, bias, out)
    if out is None:
        out = torch.empty_like(input)
    _check_rows(input, out)
    rows, hidden = _rows_hidden(input)
    _param_check(hidden, input, weight=weight, bias=bias)
    _lib.call("oasr_b200_rms_norm", _p(out), _p(input), _p(weight), _p(bias), rows, hidden, float(eps),
              _dt(input), _stream(input))
    return out


def _add_norm(name, input, residual, weight, bias, eps, alpha, out, residual_out, want_residual):
    _need_cuda(input, residual, weight, bias, out, residual_out)
    if out is None:
        out = torch.empty_like(input)
    if want_residual and residual_out is None:
        residual_out = torch.empty_like(input)
    _check_rows(input, residual, out, residual_out)
    _same_dtype(input, residual=residual, out=out, residual_out=residual_out)
    rows, hidden = _rows_hidden(input)
    _param_check(hidden, input, weight=weight, bias=bias)
    if want_residual:
        _lib.call(name, _p(out), _p(residual_out), _p(input), _p(residual), _p(weight), _p(bias), rows, hidden,
                  float(eps), float(alpha), _dt(input), _stream(input))
        return out, residual_out
    _lib.call(name, _p(out), _p(input), _p(residual), _p(weight), _p(bias), rows, hidden, float(eps),
              float(alpha), _dt(input), _stream(input))
    return out


def add_layer_norm(input, residual, weight, bias, eps: float = 1e-5, out=None, alpha: float = 1.0):
    """``LayerNorm(residual + alpha*input)`` (reference: functionals/norm.py:206-232)."""
    return _add_norm("oasr_b200_add_layer_norm", input, residual, weight, bias, eps, alpha, out, None, False)


def add_layer_norm_residual(input, residual, weight, bias=None, eps: float = 1e-5, alpha: float = 1.0,
                            out=None, residual_out=None):
    """Fused add + LayerNorm returning ``(out, sum)``; the sum feeds the norm
    unrounded and is rounded once for ``residual_out``
    (reference: functionals/norm.py:235-282)."""
    return _add_norm("oasr_b200_add_layer_norm_residual", input, residual, weight, bias, eps, alpha, out,
                     residual_out, True)


def add_rms_norm(input, residual, weight, bias=None, eps: float = 1e-5, alpha: float = 1.0, out=None):
    """``RMSNorm(residual + alpha*input)`` (reference: functionals/norm.py:71-90)."""
    return _add_norm("oasr_b200_add_rms_norm", input, residual, weight, bias, eps, alpha, out, None, False)


def add_rms_norm_residual(input, residual, weight, bias=None, eps: float = 1e-5, alpha: float = 1.0,
                          out=None, residual_out=None):
    """(reference: functionals/norm.py:93-118)."""
    return _add_norm("oasr_b200_add_rms_norm_residual", input, residual, weight, bias, eps, alpha, out,
                     residual_out, True)


def layer_norm_activation(input, weight, bias=None, eps: float = 1e-5, activation_type: int = 2, out=None):
    """Fused LayerNorm + activation (reference: functionals/norm.py:285-298)."""
    _need_cuda(input, weight, bias, out)
    if out is None:
        out = torch.empty_like(input)
    _check_rows(input, out)
    rows, hidden = _rows_hidden(input)
    _param_check(hidden, input, weight=weight, bias=bias)
    _lib.call("oasr_b200_layer_norm_activation", _p(out), _p(input), _p(weight), _p(bias), rows, hidden,
              float(eps), int(activation_type), _dt(input), _stream(input))
    return out


def rms_norm_activation(input, weight, bias=None, eps: float = 1e-5, activation_type: int = 2, out=None):
    """Fused RMSNorm + activation (reference: functionals/norm.py:301-314)."""
    _need_cuda(input, weight, bias, out)
    if out is None:
        out = torch.empty_like(input)
    _check_rows(input, out)
    rows, hidden = _rows_hidden(input)
    _param_check(hidden, input, weight=weight, bias=bias)
    _lib.call("oasr_b200_rms_norm_activation", _p(out), _p(input), _p(weight), _p(bias), rows, hidden,
              float(eps), int(activation_type), _dt(input), _stream(input))
    return out


def _batch_norm(input, weight, bias, running_mean, running_var, eps, act, out):
    _need_cuda(input, weight, bias, running_mean, running_var, out)
    if out is None:
        out = torch.empty_like(input)
    _check_rows(input, out)
    rows, channels = _rows_hidden(input)
    _param_check(channels, input, weight=weight, bias=bias, running_mean=running_mean, running_var=running_var)
    _lib.call("oasr_b200_batch_norm", _p(out), _p(input), _p(weight), _p(bias), _p(running_mean),
              _p(running_var), rows, channels, float(eps), int(act), _dt(input), _stream(input))
    return out


def batch_norm_1d(input, weight, bias, running_mean, running_var, eps: float = 1e-5, out=None):
    """Inference BatchNorm over channels-last ``(B, T, C)`` (reference: functionals/norm.py:148-175)."""
    return _batch_norm(input, weight, bias, running_mean, running_var, eps, ACT_NONE, out)


def batch_norm_activation(input, weight, bias, running_mean, running_var, eps: float = 1e-5,
                          activation_type: int = 2, out=None):
    """(reference: functionals/norm.py:317-334)."""
    return _batch_norm(input, weight, bias, running_mean, running_var, eps, activation_type, out)


def batch_norm_swish(input, weight, bias, running_mean, running_var, eps: float = 1e-5, out=None):
    """(reference: functionals/norm.py:364-378)."""
    return _batch_norm(input, weight, bias, running_mean, running_var, eps, ACT_SWISH, out)


# ---------------------------------------------------------------------------
# Activations (reference: oasr/functionals/activation.py)
# ---------------------------------------------------------------------------
def get_activation_type_id(name: str) -> int:
    try:
        return ACTIVATION_IDS[name.lower()]
    except KeyError:
        raise ValueError(f"Unknown activation {name!r}; supported: {sorted(ACTIVATION_IDS)}") from None


def glu(input, out=None):
    """``input[..., :C] * sigmoid(input[..., C:])`` (reference: functionals/activation.py:40-60)."""
    _need_cuda(input, out)
    if input.size(-1) % 2:
        raise RuntimeError("glu needs an even trailing dimension")
    channels = input.size(-1) // 2
    if not input.is_contiguous():
        input = input.contiguous()
    if out is None:
        out = torch.empty(input.shape[:-1] + (channels,), device=input.device, dtype=input.dtype)
    elif not out.is_contiguous() or out.dtype != input.dtype or out.shape != input.shape[:-1] + (channels,):
        raise RuntimeError("glu: out must be contiguous with shape input.shape[:-1] + (C,) and input's dtype")
    rows = input.numel() // (2 * channels) if channels else 0
    _lib.call("oasr_b200_glu", _p(out), _p(input), rows, channels, _dt(input), _stream(input))
    return out


def swish(input, out=None):
    """``x * sigmoid(x)`` (reference: functionals/activation.py:63-77)."""
    _need_cuda(input, out)
    if not input.is_contiguous():
        input = input.contiguous()
    if out is None:
        out = torch.empty_like(input)
    elif not out.is_contiguous() or out.dtype != input.dtype or out.shape != input.shape:
        raise RuntimeError("swish: out must be contiguous and match input")
    _lib.call("oasr_b200_swish", _p(out), _p(input), input.numel(), _dt(input), _stream(input))
    return out


# ---------------------------------------------------------------------------
# Depthwise conv1d (reference: oasr/functionals/conv.py)
# ---------------------------------------------------------------------------
def _padding_pair(padding: Union[int, Tuple[int, int]]) -> Tuple[int, int]:
    if isinstance(padding, int):
        return padding, padding
    left, right = padding
    return int(left), int(right)


def _depthwise(input, weight, bias, padding, out, mask, add_input, act):
    _need_cuda(input, weight, bias, out, mask)
    if input.dim() != 3:
        raise RuntimeError(f"Expected 3D tensor, got {input.dim()}D")
    if weight.dim() == 3:
        if weight.size(1) != 1:
            raise RuntimeError("depthwise weight must be [kernel_size, channels] or [kernel_size, 1, channels]")
        weight = weight.reshape(weight.size(0), weight.size(2))
    if weight.dim() != 2 or weight.size(1) != input.size(2):
        raise RuntimeError("depthwise weight must be [kernel_size, channels] matching the input channels")
    if not input.is_contiguous():
        raise RuntimeError("Tensor must be contiguous (row-major, no padded strides)")
    weight = weight.contiguous()
    _same_dtype(input, weight=weight, bias=bias, out=out)
    pl, pr = _padding_pair(padding)
    B, T, C = input.shape
    K = weight.size(0)
    out_len = T + pl + pr - K + 1
    if out_len <= 0:
        raise ValueError(f"depthwise_conv1d has invalid output length {out_len}")
    if out is None:
        out = torch.empty(B, out_len, C, device=input.device, dtype=input.dtype)
    elif tuple(out.shape) != (B, out_len, C) or not out.is_contiguous():
        raise RuntimeError(f"out must be contiguous with shape {(B, out_len, C)}")
    mask_is_bool = 0
    if mask is not None:
        if mask.numel() != B * T:
            raise RuntimeError("mask must be [batch, seq_len, 1]")
        if mask.dtype == torch.bool:
            mask_is_bool = 1
        elif mask.dtype != input.dtype:
            raise RuntimeError("mask must be bool or have the input dtype")
        mask = mask.contiguous()
    _lib.call("oasr_b200_depthwise_conv1d", _p(out), _p(input), _p(weight), _p(bias), B, T, C, K, pl, pr,
              _p(mask), mask_is_bool, int(bool(add_input)), act, _dt(input), _stream(input))
    return out


def depthwise_conv1d(input, weight, bias=None, padding: Union[int, Tuple[int, int]] = 0, out=None, *,
                     mask=None, add_input: bool = False):
    """Depthwise conv over ``(B, T, C)`` (reference: functionals/conv.py:371-422)."""
    return _depthwise(input, weight, bias, padding, out, mask, add_input, ACT_NONE)


def depthwise_conv1d_silu(input, weight, bias=None, padding: Union[int, Tuple[int, int]] = 0, out=None):
    """Depthwise conv + SiLU (reference: functionals/conv.py, ``depthwise_conv1d_silu``)."""
    return _depthwise(input, weight, bias, padding, out, None, False, ACT_SWISH)


def causal_conv1d(input, state, weight, bias=None, out=None):
    """Streaming causal depthwise conv; ``state`` ``(B, K-1, C)`` is updated in
    place, ``weight`` is ``(C, 1, K)`` (reference: functionals/conv.py:592-603)."""
    _need_cuda(input, state, weight, bias, out)
    if input.dim() != 3 or state.dim() != 3:
        raise RuntimeError("causal_conv1d expects input (B, T, C) and state (B, K-1, C)")
    B, T, C = input.shape
    if weight.dim() == 3:
        weight = weight.reshape(weight.size(0), weight.size(2))
    K = weight.size(1)
    if weight.size(0) != C or tuple(state.shape) != (B, K - 1, C):
        raise RuntimeError("causal_conv1d: weight must be (C, 1, K) and state (B, K-1, C)")
    if not (input.is_contiguous() and state.is_contiguous()):
        raise RuntimeError("Tensor must be contiguous (row-major, no padded strides)")
    weight = weight.contiguous()
    _same_dtype(input, state=state, weight=weight, bias=bias, out=out)
    if out is None:
        out = torch.empty_like(input)
    _lib.call("oasr_b200_causal_conv1d", _p(out), _p(input), _p(state), _p(weight), _p(bias), B, T, C, K,
              _dt(input), _stream(input))
    return out


# ---------------------------------------------------------------------------
# GEMM family (reference: oasr/functionals/gemm.py)
# ---------------------------------------------------------------------------
_HALF = (torch.float16, torch.bfloat16)


def _gemm_io(A: torch.Tensor, N: int, out: Optional[torch.Tensor], out_dtype=None):
    """``(A, out)`` -> ``(A_contig, out, M)`` (reference: functionals/gemm.py:78-85)."""
    if not A.is_contiguous():
        A = A.contiguous()
    if out is None:
        out = torch.empty(*A.shape[:-1], N, device=A.device, dtype=out_dtype or A.dtype)
    elif not out.is_contiguous():
        raise RuntimeError("Tensor must be contiguous (row-major, no padded strides)")
    return A, out, (A.numel() // A.shape[-1] if A.shape[-1] else 0)


def _check_gemm(A, B, C, N, K):
    _need_cuda(A, B, C)
    if B.dim() != 2:
        raise RuntimeError(f"Expected 2D tensor, got {B.dim()}D")
    if B.size(1) != K:
        raise RuntimeError(f"B must be [N, K] with K={K}, got {tuple(B.shape)}")
    _same_dtype(A, B=B, C=C)
    if A.dtype not in _HALF:
        raise RuntimeError(f"gemm supports fp16/bf16, got {A.dtype}")
    if C is not None and C.numel() != N:
        raise RuntimeError(f"bias must have N={N} elements, got {C.numel()}")


def gemm(A, B, C=None, out=None):
    """``A @ B.T + C`` with ``B`` as ``[N, K]`` (reference: functionals/gemm.py:223-259)."""
    K, N = A.shape[-1], B.shape[0]
    _check_gemm(A, B, C, N, K)
    A, out, M = _gemm_io(A, N, out)
    B = B if B.is_contiguous() else B.contiguous()
    _lib.call("oasr_b200_gemm", _p(out), _p(A), _p(B), _p(C), M, N, K, ACT_NONE, _dt(A), _stream(A))
    return out


def gemm_activation(A, B, C=None, activation_type: int = 2, out=None):
    """``act(A @ B.T + C)`` (reference: functionals/gemm.py:345-384)."""
    K, N = A.shape[-1], B.shape[0]
    _check_gemm(A, B, C, N, K)
    A, out, M = _gemm_io(A, N, out)
    B = B if B.is_contiguous() else B.contiguous()
    _lib.call("oasr_b200_gemm", _p(out), _p(A), _p(B), _p(C), M, N, K, int(activation_type), _dt(A), _stream(A))
    return out


def gemm_glu(A, B, C=None, out=None):
    """``glu(A @ B.T + C)`` with ``B`` as ``[2N, K]``: pointwise_conv1 + GLU of the
    conformer conv module in one kernel (no reference operator; equals
    ``oasr.glu(oasr.gemm(A, B, C))``, oasr/models/conformer/model.py:191-192)."""
    K, N2 = A.shape[-1], B.shape[0]
    if N2 % 2:
        raise RuntimeError("gemm_glu needs an even number of weight rows")
    _check_gemm(A, B, C, N2, K)
    N = N2 // 2
    A, out, M = _gemm_io(A, N, out)
    B = B if B.is_contiguous() else B.contiguous()
    _lib.call("oasr_b200_gemm_glu", _p(out), _p(A), _p(B), _p(C), M, N, K, _dt(A), _stream(A))
    return out


def gemm_residual_f32(residual: torch.Tensor, A, B, C=None, alpha: float = 1.0, out=None):
    """``residual(fp32) + alpha * (A @ B.T + C)`` kept in fp32 (the residual stream
    of the fused encoder layer; no reference operator)."""
    K, N = A.shape[-1], B.shape[0]
    _check_gemm(A, B, C, N, K)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise RuntimeError("residual must be a contiguous fp32 tensor")
    A, _, M = _gemm_io(A, N, residual)
    if residual.numel() != M * N:
        raise RuntimeError("residual must have M*N elements")
    if out is None:
        out = torch.empty_like(residual)
    B = B if B.is_contiguous() else B.contiguous()
    _lib.call("oasr_b200_gemm_residual_f32", _p(out), _p(residual), _p(A), _p(B), _p(C), M, N, K, float(alpha),
              _dt(A), _stream(A))
    return out


def bmm(A, B, out=None):
    """``A[b] @ B[b].T`` (reference: functionals/gemm.py:262-299)."""
    _need_cuda(A, B, out)
    if A.dim() != 3 or B.dim() != 3 or A.size(0) != B.size(0) or A.size(2) != B.size(2):
        raise RuntimeError("bmm expects A [b, M, K] and B [b, N, K]")
    _same_dtype(A, B=B, out=out)
    if A.dtype not in _HALF:
        raise RuntimeError(f"bmm supports fp16/bf16, got {A.dtype}")
    batch, M, K = A.shape
    N = B.shape[1]
    A = A if A.is_contiguous() else A.contiguous()
    B = B if B.is_contiguous() else B.contiguous()
    if out is None:
        out = torch.empty(batch, M, N, device=A.device, dtype=A.dtype)
    _lib.call("oasr_b200_bmm", _p(out), _p(A), _p(B), batch, M, N, K, _dt(A), _stream(A))
    return out


def group_gemm(A, B, offset, out=None):
    """Grouped GEMM; ``offset`` holds cumulative END rows per group
    (reference: functionals/gemm.py:302-342).  The offsets are read on the
    device: no host synchronisation."""
    _need_cuda(A, B, offset, out)
    if A.dim() != 2 or B.dim() != 3 or A.size(1) != B.size(2):
        raise RuntimeError("group_gemm expects A [L, K] and B [G, N, K]")
    if offset.dim() != 1 or offset.numel() != B.size(0):
        raise RuntimeError("offset must be [G]")
    _same_dtype(A, B=B, out=out)
    if A.dtype not in _HALF:
        raise RuntimeError(f"group_gemm supports fp16/bf16, got {A.dtype}")
    if offset.dtype != torch.int32:
        offset = offset.to(torch.int32)
    L, K = A.shape
    G, N = B.shape[0], B.shape[1]
    A = A if A.is_contiguous() else A.contiguous()
    B = B if B.is_contiguous() else B.contiguous()
    if out is None:
        out = torch.empty(L, N, device=A.device, dtype=A.dtype)
    _lib.call("oasr_b200_group_gemm", _p(out), _p(A), _p(B), _p(offset.contiguous()), L, G, N, K, _dt(A),
              _stream(A))
    return out


def gemm_log_softmax(A, B, C=None, out=None, *, out_dtype: Optional[torch.dtype] = None,
                     return_argmax: bool = False):
    """``log_softmax(A @ B.T + C, -1)`` in one kernel; logits never reach HBM
    (reference: functionals/gemm.py:387-426).

    ``out_dtype=torch.float32`` (an extension; the reference returns A's dtype)
    writes fp32 log-probs, which the CTC decoders consume.  ``return_argmax``
    also returns the per-row index of the first maximum (int32)."""
    K, N = A.shape[-1], B.shape[0]
    _check_gemm(A, B, C, N, K)
    if out is not None:
        out_dtype = out.dtype
    out_dtype = out_dtype or A.dtype
    if out_dtype not in (A.dtype, torch.float32):
        raise RuntimeError("gemm_log_softmax output must be fp32 or A's dtype")
    A, out, M = _gemm_io(A, N, out, out_dtype)
    B = B if B.is_contiguous() else B.contiguous()
    arg = torch.empty(A.shape[:-1], device=A.device, dtype=torch.int32) if return_argmax else None
    _lib.call("oasr_b200_gemm_log_softmax", _p(out), _p(A), _p(B), _p(C), M, N, K, _dt(A), _DTYPE_ID[out_dtype],
              _p(arg), _stream(A))
    return (out, arg) if return_argmax else out


def device_status(device=None) -> int:
    """Raise if any kernel on ``device`` abandoned a bounded wait since the last call."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = ctypes.c_uint32(0)
    with torch.cuda.device(dev):
        _lib.call("oasr_b200_device_status", ctypes.byref(word),
                  ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    return word.value
