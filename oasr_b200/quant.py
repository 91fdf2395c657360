"""8-bit operand GEMMs (fp8 e4m3 and W8A8 int8) with per-token / per-output-channel scales.

No counterpart in the reference (its ``layers/linear.py:7`` only names a future quantised path); the
arithmetic is restated on the CPU in ``oracle/ops.py`` (``quantize_rows``, ``gemm_q8``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .functional import _DTYPE_ID, _need_cuda, _p, _stream

FP8_E4M3 = 1
INT8 = 2


def quantize_rows(x: torch.Tensor, kind: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x (rows, cols)`` 16-bit -> ``(q uint8 (rows, cols), scale fp32 (rows,))`` with ``x ~ q * scale``:
    ``scale = amax / 448`` and fp8 e4m3 codes, or ``amax / 127`` and int8 codes (two's complement bytes)."""
    _need_cuda(x)
    x = x.contiguous()
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    scale = torch.empty(rows, dtype=torch.float32, device=x.device)
    _lib.call("oasr_b200_quantize_rows", _p(q), _p(scale), _p(x), rows, cols, int(kind), _DTYPE_ID[x.dtype], _stream(x))
    return q, scale


def gemm_q8(a_q: torch.Tensor, a_scale: torch.Tensor, b_q: torch.Tensor, b_scale: torch.Tensor,
            bias: Optional[torch.Tensor] = None, *, kind: int, activation: int = -1, glu: bool = False,
            out_dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act((a_q . b_q^T) * a_scale[:, None] * b_scale[None, :] + bias)`` on the tensor cores' 8-bit kinds;
    with ``glu`` the weight has ``2N`` rows (value | gate) and the result is ``value * sigmoid(gate)``."""
    _need_cuda(a_q, a_scale, b_q, b_scale, bias)
    M, K = a_q.shape
    N = b_q.size(0) // (2 if glu else 1)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    _lib.call("oasr_b200_gemm_q8", _p(out), _p(a_q), _p(a_scale), _p(b_q), _p(b_scale), _p(bias), M, N, K,
              int(activation), int(bool(glu)), int(kind), _DTYPE_ID[out.dtype], _stream(a_q))
    return out
