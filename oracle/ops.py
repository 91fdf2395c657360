"""Operator-level CPU oracle (torch fp32 / numpy integer).  TEST INFRASTRUCTURE ONLY.

Each function restates, in fp32 on the CPU, what the reference computes for
one operator of the encoder hot path.  The reference's own tests use exactly
these torch expressions as their oracle (tests/test_norm.py, test_gemm.py,
test_gemm_log_softmax.py, test_fmha.py, test_fmha_varlen.py, test_conv.py,
test_activation.py); the reference file:line each one follows is cited.
Inputs of any float dtype are upcast to fp32; results are fp32 unless the
reference defines a rounding (``residual_out``).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

# Activation ids: include/oasr/common/types.h:49-56, oasr/functionals/activation.py:13-25.
ACT_NONE, ACT_RELU, ACT_GELU_TANH, ACT_SWISH, ACT_GELU_ERF = -1, 0, 1, 2, 4


def activation(x: torch.Tensor, act: int) -> torch.Tensor:
    """include/oasr/common/math.h:20-57 (fp32 activation functors)."""
    x = x.float()
    if act == ACT_NONE:
        return x
    if act == ACT_RELU:
        return F.relu(x)
    if act == ACT_GELU_TANH:
        return F.gelu(x, approximate="tanh")
    if act == ACT_SWISH:
        return F.silu(x)
    if act == ACT_GELU_ERF:
        return F.gelu(x)
    raise ValueError(f"unknown activation id {act}")


# ---- norms -----------------------------------------------------------------
def layer_norm(x, weight, bias=None, eps: float = 1e-5, act: int = ACT_NONE):
    """include/oasr/norm.cuh:28-93 (layerNormKernel), :641 (layerNormActKernel);
    torch spelling oasr/layers/norm.py (F.layer_norm)."""
    y = F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
    return activation(y, act)


def rms_norm(x, weight, bias=None, eps: float = 1e-5, act: int = ACT_NONE):
    """include/oasr/norm.cuh:99-147 (rmsNormKernel): x * rsqrt(mean(x^2) + eps) * w (+ b)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    if bias is not None:
        y = y + bias.float()
    return activation(y, act)


def add_layer_norm_residual(x, residual, weight, bias=None, eps: float = 1e-5, alpha: float = 1.0):
    """include/oasr/norm.cuh:396-484 (addLayerNormResidualKernel); torch spelling
    oasr/layers/norm.py:88-100 (_add_layer_norm_ref): s = residual + alpha*x in
    fp32, out = LN(s) on the unrounded sum, residual_out = cast(s) rounded once."""
    s = residual.float() + alpha * x.float()
    return layer_norm(s, weight, bias, eps), s.to(x.dtype)


def add_rms_norm_residual(x, residual, weight, bias=None, eps: float = 1e-5, alpha: float = 1.0):
    """include/oasr/norm.cuh:490- (addRmsNorm*Kernel)."""
    s = residual.float() + alpha * x.float()
    return rms_norm(s, weight, bias, eps), s.to(x.dtype)


def batch_norm(x, weight, bias, mean, var, eps: float = 1e-5, act: int = ACT_NONE):
    """include/oasr/norm.cuh:153-187,779-813: (x - mean) * rsqrt(var + eps) * w + b, then act."""
    y = (x.float() - mean.float()) * torch.rsqrt(var.float() + eps) * weight.float() + bias.float()
    return activation(y, act)


# ---- activations -------------------------------------------------------------
def glu(x):
    """include/oasr/activation.cuh:25-60: x[..., :C] * sigmoid(x[..., C:]) (= F.glu, oasr/layers/conv.py:676-689)."""
    return F.glu(x.float(), dim=-1)


def swish(x):
    """include/oasr/activation.cuh:66-87."""
    return F.silu(x.float())


# ---- depthwise conv ------------------------------------------------------------
def depthwise_conv1d(x, weight, bias=None, padding=(0, 0), mask=None, add_input: bool = False,
                     act: int = ACT_NONE):
    """include/oasr/conv/conv1d.cuh:23-113 (and :119-181 with SiLU).  x (B,T,C),
    weight (K,C) or (K,1,C); out[b,t,c] = sum_k x[b, t - pl + k, c] * w[k, c] + bias,
    zero outside [0,T).  With mask m (B,T[,1]): the input is multiplied by m, the
    optionally added input by m[t], and the output by m[t]."""
    xf = x.float()
    w = weight.float().reshape(weight.shape[0], -1)  # (K, C)
    pl, pr = (padding, padding) if isinstance(padding, int) else padding
    B, T, C = xf.shape
    m = None
    if mask is not None:
        m = mask.reshape(B, T, 1).float()
        xf = xf * m
    xin = F.pad(xf.transpose(1, 2), (pl, pr))  # (B, C, T+pl+pr)
    y = F.conv1d(xin, w.t().unsqueeze(1), None if bias is None else bias.float(), groups=C).transpose(1, 2)
    if add_input:
        y = y + xf
    if m is not None:
        y = y * m
    return activation(y, act)


def causal_conv1d(x, state, weight, bias=None):
    """include/oasr/conv/conv1d.cuh:187-269,450-473.  x (B,T,C), state (B,K-1,C),
    weight (C,K) or (C,1,K).  Returns (out, new_state)."""
    w = weight.float().reshape(weight.shape[0], -1)  # (C, K)
    C, K = w.shape
    cat = torch.cat([state.float(), x.float()], dim=1)  # (B, K-1+T, C)
    y = F.conv1d(cat.transpose(1, 2), w.unsqueeze(1), None if bias is None else bias.float(), groups=C)
    new_state = torch.cat([state, x], dim=1)[:, -(K - 1):, :].clone()
    return y.transpose(1, 2), new_state


# ---- GEMM family ---------------------------------------------------------------
def gemm(A, B, C=None, act: int = ACT_NONE):
    """csrc/gemm.cu:40-115, epilogue include/oasr/common/epilogue_functors.h:
    act(A . B^T + C) with fp32 accumulation (tests/test_gemm.py:33-55 use torch.matmul)."""
    y = A.float() @ B.float().t()
    if C is not None:
        y = y + C.float()
    return activation(y, act)


def bmm(A, B):
    """csrc/bmm.cu (tests/test_gemm.py): A[b] . B[b]^T."""
    return torch.bmm(A.float(), B.float().transpose(1, 2))


def group_gemm(A, B, offsets: Sequence[int]):
    """csrc/group_gemm.cu:44-72; offsets are cumulative END rows (tests/test_gemm.py:56-70)."""
    out = torch.zeros(A.shape[0], B.shape[1], dtype=torch.float32)
    start = 0
    for g, end in enumerate(int(o) for o in offsets):
        out[start:end] = A[start:end].float() @ B[g].float().t()
        start = end
    return out


def gemm_log_softmax(A, B, C=None):
    """oasr/functionals/gemm_torch.py:64-75: log_softmax(linear(A, B, C), -1) (fp32)."""
    return F.log_softmax(F.linear(A.float(), B.float(), None if C is None else C.float()), dim=-1)


def gemm_glu(A, B, C=None):
    """pointwise_conv1 followed by GLU, oasr/models/conformer/model.py:191-192."""
    return glu(gemm(A, B, C))


# ---- attention -------------------------------------------------------------------
def _attention_core(q, k, v, scale, bias, keep):
    """q (Tq,D), k/v (Tk,D) fp32, bias (Tq,Tk) or None, keep (Tq,Tk) bool.
    softmax(q.k^T*scale + bias) over kept keys; a row with no kept key gives zeros
    (oasr/kernels/cute/softmax.py:141-146,176-181)."""
    s = (q @ k.t()) * scale
    if bias is not None:
        s = s + bias
    s = s.masked_fill(~keep, float("-inf"))
    row_max = s.max(dim=-1, keepdim=True).values
    row_max = torch.where(torch.isinf(row_max), torch.zeros_like(row_max), row_max)
    p = torch.exp(s - row_max)
    denom = p.sum(-1, keepdim=True)
    p = torch.where(denom > 0, p / denom.clamp_min(1e-38), torch.zeros_like(p))
    # masked V rows must not contribute even if they hold non-finite stale data: the
    # reference documents finite V as a precondition; the oracle is defined with zeros there
    return p @ v


def fmha(q, k, v, scale: float, bias=None, seqlens=None, seqstarts=None, block_table=None, causal=False):
    """oasr/functionals/attention.py:369-551 (+ _sdpa_reference :223-279, mask rules
    oasr/kernels/cute/mask.py:102-117).  q (B,H,Tq,D); dense k/v (B,Hkv,Tk,D) or
    paged pools (num_blocks, bs, Hkv, D) with block_table (B, nblk).  Returns fp32 (B,H,Tq,D)."""
    if block_table is not None:
        k, v = gather_paged_kv(k, v, block_table)
    q, k, v = q.float(), k.float(), v.float()
    B, H, Tq, D = q.shape
    Hkv, Tk = k.shape[1], k.shape[2]
    rep = H // Hkv
    out = torch.zeros(B, H, Tq, D)
    cols = torch.arange(Tk)
    rows = torch.arange(Tq)
    for b in range(B):
        keep = torch.ones(Tq, Tk, dtype=torch.bool)
        if seqlens is not None:
            keep &= (cols < int(seqlens[b])).unsqueeze(0)
        if seqstarts is not None:
            keep &= (cols >= int(seqstarts[b])).unsqueeze(0)
        if causal:
            keep &= cols.unsqueeze(0) <= rows.unsqueeze(1)
        for h in range(H):
            bb = None if bias is None else bias[b, h, :Tq, :Tk].float()
            out[b, h] = _attention_core(q[b, h], k[b, h // rep], v[b, h // rep], scale, bb, keep)
    return out


def fmha_varlen(q, k, v, scale: float, cu_q, cu_k, bias=None, bias_offsets=None):
    """oasr/functionals/attention.py:181-220,592-693: per-segment attention over packed
    (total,H,D) rows; segment s of the flat bias is (H,Tq_s,Tk_s) at bias_offsets[s]."""
    q, k, v = q.float(), k.float(), v.float()
    H, Hkv = q.shape[1], k.shape[1]
    rep = H // Hkv
    out = torch.zeros_like(q)
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    for s in range(len(cu_q) - 1):
        qa, qb, ka, kb = cu_q[s], cu_q[s + 1], cu_k[s], cu_k[s + 1]
        if qb == qa:
            continue
        keep = torch.ones(qb - qa, kb - ka, dtype=torch.bool)
        for h in range(H):
            bb = None
            if bias is not None:
                o = int(bias_offsets[s])
                bb = bias[o:o + H * (qb - qa) * (kb - ka)].view(H, qb - qa, kb - ka)[h].float()
            out[qa:qb, h] = _attention_core(q[qa:qb, h], k[ka:kb, h // rep], v[ka:kb, h // rep], scale, bb, keep)
    return out


# ---- paged KV (integer / byte work: numpy, bit-exact) -------------------------------
def flat_write_index(block_table: np.ndarray, offsets: np.ndarray, t_new: int, block_size: int) -> np.ndarray:
    """oasr/cache/paged_kv.py:23-40."""
    time_pos = offsets.astype(np.int64)[:, None] + np.arange(t_new, dtype=np.int64)[None, :]
    logical = time_pos // block_size
    within = time_pos % block_size
    physical = np.take_along_axis(block_table.astype(np.int64), logical, axis=1)
    return (physical * block_size + within).reshape(-1)


def write_kv_chunk(k_pool, v_pool, new_k, new_v, block_table, offsets, block_size: int):
    """oasr/cache/paged_kv.py:63-137 (heterogeneous-offset scatter).  Pools
    (num_blocks, bs, Hkv, D) are modified in place; new_k/new_v are (B,Hkv,T,D)."""
    T = new_k.shape[2]
    Hkv, D = k_pool.shape[2], k_pool.shape[3]
    idx = torch.from_numpy(flat_write_index(block_table.cpu().numpy(), offsets.cpu().numpy(), T, block_size))
    k_pool.view(-1, Hkv, D)[idx] = new_k.permute(0, 2, 1, 3).reshape(-1, Hkv, D)
    v_pool.view(-1, Hkv, D)[idx] = new_v.permute(0, 2, 1, 3).reshape(-1, Hkv, D)


def gather_paged_kv(k_pool, v_pool, block_table):
    """oasr/functionals/attention.py:153-178."""
    B, nblk = block_table.shape
    bs, Hkv, D = k_pool.shape[1], k_pool.shape[2], k_pool.shape[3]
    ids = block_table.long()
    k = k_pool[ids].reshape(B, nblk * bs, Hkv, D).permute(0, 2, 1, 3)
    v = v_pool[ids].reshape(B, nblk * bs, Hkv, D).permute(0, 2, 1, 3)
    return k, v


def ctc_greedy(log_probs: torch.Tensor, length: int, blank: int = 0):
    """csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55: per-frame argmax (first
    maximum on ties), drop repeats, drop blanks."""
    ids = log_probs[:length].argmax(dim=-1).tolist()
    out, prev = [], None
    for i in ids:
        if i != prev and i != blank:
            out.append(i)
        prev = i
    return out


# ---------------------------------------------------------------------------
# 8-bit operand GEMMs (no reference counterpart: oasr/layers/linear.py:7 only
# names a future quantised path).  Restated here so that the CUDA kernels have
# a CPU statement of their arithmetic to be checked against.
# ---------------------------------------------------------------------------
def quantize_rows(x: torch.Tensor, kind: int):
    """Row-wise dynamic quantisation, the arithmetic of the CUDA kernel step by step in fp32:
    ``scale = amax / qmax``; ``inv = 1 / scale``; ``q = round(x * inv)`` (fp8 e4m3 round-to-nearest-even,
    or int8 round-half-even clipped to +-127).  kind 1 = fp8 e4m3 (qmax 448), 2 = int8 (qmax 127).
    Returns ``(codes uint8, scale fp32, dequantised fp32 values of the codes)``."""
    x = x.float()
    amax = x.abs().amax(dim=1)
    qmax = 448.0 if kind == 1 else 127.0
    scale = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    inv = 1.0 / scale
    y = x * inv[:, None]
    if kind == 1:
        q8 = y.to(torch.float8_e4m3fn)
        return q8.view(torch.uint8), scale, q8.float()
    qi = torch.clamp(torch.round(y), -127, 127).to(torch.int8)
    return qi.view(torch.uint8), scale, qi.float()


def gemm_q8(a_vals: torch.Tensor, a_scale: torch.Tensor, b_vals: torch.Tensor, b_scale: torch.Tensor, bias=None,
            activation: int = -1, glu: bool = False) -> torch.Tensor:
    """fp32 statement of the 8-bit GEMM on the dequantised code values: ``(A . B^T) * sa * sb + bias``."""
    y = (a_vals.double() @ b_vals.double().t()).float() * a_scale[:, None] * b_scale[None, :]
    if bias is not None:
        y = y + bias.float()
    if glu:
        n = y.size(1) // 2
        return y[:, :n] * torch.sigmoid(y[:, n:])
    return globals()["activation"](y, activation) if activation >= 0 else y


def quantize_kv_fp8(x: torch.Tensor, scale: torch.Tensor):
    """fp8 page codes of keys / values ``x (..., H, D)`` with per-head scales ``scale (H,)``, the arithmetic of
    the CUDA page write in fp32: ``code = e4m3(x * (1 / scale[h]))`` (round to nearest even; inputs are expected
    within +-448 * scale).  Returns ``(codes uint8, dequantised fp32 = value(code) * scale[h])``."""
    inv = (1.0 / scale.float())[:, None]
    y = (x.float() * inv).clamp(-448.0, 448.0)
    q = y.to(torch.float8_e4m3fn)
    return q.view(torch.uint8), q.float() * scale.float()[:, None]
