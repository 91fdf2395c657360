"""Attention operators with the reference's signatures (oasr/functionals/attention.py)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from .functional import _DTYPE_ID, _need_cuda, _p, _stream

_HALF = (torch.float16, torch.bfloat16)


def _strides3(t: torch.Tensor):
    """(batch, head, row) element strides of a (B, H, T, D) view as a host int64[3]; None if the
    view cannot be addressed by the kernel (unit stride along D, the rest multiples of 8)."""
    if t.stride(3) != 1 and t.size(3) > 1:
        return None
    st = [t.stride(0), t.stride(1), t.stride(2)]
    for extent, s in zip(t.shape[:3], st):
        if extent > 1 and (s <= 0 or s % 8):
            return None
    st = [s if e > 1 else 8 for e, s in zip(t.shape[:3], st)]
    return (ctypes.c_int64 * 3)(*st)


def _canon(t: torch.Tensor):
    st = _strides3(t)
    if st is None or t.data_ptr() % 16:
        t = t.contiguous()
        st = _strides3(t)
    return t, st


def gather_paged_kv(k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor):
    """Gather paged K/V into dense ``(B, H_kv, T_kv_logical, D)`` tensors
    (reference: functionals/attention.py:153-178).  Pure data movement: bit-exact."""
    _need_cuda(k_pool, v_pool, block_table)
    if k_pool.dim() != 4 or k_pool.shape != v_pool.shape or block_table.dim() != 2:
        raise ValueError("gather_paged_kv expects pools (num_blocks, block_size, H_kv, D) and a 2-D block table")
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    block_table = block_table.contiguous()
    k_pool, v_pool = k_pool.contiguous(), v_pool.contiguous()
    B, nblk = block_table.shape
    num_blocks, bs, Hkv, D = k_pool.shape
    k = torch.empty(B, Hkv, nblk * bs, D, device=k_pool.device, dtype=k_pool.dtype)
    v = torch.empty_like(k)
    _lib.call("oasr_b200_paged_kv_gather", _p(k), _p(v), _p(k_pool), _p(v_pool), _p(block_table), B, Hkv, D, nblk, bs,
              num_blocks, k_pool.element_size(), _stream(k_pool))
    return k, v


def fmha(q, k, v, *, softmax_scale: float, attn_bias: Optional[torch.Tensor] = None,
         cache_seqlens: Optional[torch.Tensor] = None, cache_seqstarts: Optional[torch.Tensor] = None,
         block_table: Optional[torch.Tensor] = None, causal: bool = False, out: Optional[torch.Tensor] = None,
         validate: bool = True, token_major: bool = False) -> torch.Tensor:
    """Fused multi-head attention (reference: functionals/attention.py:369-551).

    ``q`` ``(B, H, T_q, D)``; dense ``k``/``v`` ``(B, H_kv, T_k, D)`` or, with
    ``block_table`` ``(B, max_blocks_per_seq)``, page pools
    ``(num_blocks, block_size, H_kv, D)``.  ``attn_bias`` ``(B, H, >=T_q, >=T_k)`` is an
    additive post-scale logit; ``cache_seqlens`` / ``cache_seqstarts`` keep keys in
    ``[start, len)``; ``causal`` masks ``k_col > q_row``.  A fully masked row gives zeros.
    Unlike the reference wrapper no padding of the bias or widening of the block table
    is needed: the kernel predicates its bias reads and clamps page lookups.
    ``token_major=True`` (an extension) returns ``(B, T_q, H, D)``, the layout the output
    projection reads, instead of ``(B, H, T_q, D)``.
    """
    _need_cuda(q, k, v, attn_bias, cache_seqlens, cache_seqstarts, block_table, out)
    if q.dim() != 4:
        raise ValueError(f"q must be (B, H, T_q, D); got {tuple(q.shape)}")
    B, H, T_q, D = q.shape
    paged = block_table is not None
    if paged:
        if k.dim() != 4 or k.shape != v.shape:
            raise ValueError("paged k/v must be (num_blocks, block_size, H_kv, D)")
        num_blocks, block_size, H_kv = k.size(0), k.size(1), k.size(2)
        T_k = block_table.size(1) * block_size
    else:
        if k.dim() != 4 or k.shape != v.shape:
            raise ValueError(f"k and v must match: {tuple(k.shape)} vs {tuple(v.shape)}")
        num_blocks, block_size, H_kv, T_k = 0, 0, k.size(1), k.size(2)
    if validate:
        if q.dtype not in _HALF:
            raise ValueError(f"fmha supports fp16/bf16, got {q.dtype}")
        if k.dtype != q.dtype or v.dtype != q.dtype:
            raise ValueError("q, k, v must share a dtype")
        if k.size(3) != D:
            raise ValueError("q and k head_dim must match")
        if H % H_kv != 0:
            raise ValueError(f"H ({H}) must be divisible by H_kv ({H_kv})")
        if not paged and k.size(0) != B:
            raise ValueError("q and k batch must match")
        if attn_bias is not None:
            if attn_bias.dim() != 4 or attn_bias.size(0) != B or attn_bias.size(1) != H or \
                    attn_bias.size(2) < T_q or attn_bias.size(3) < (T_k if not paged else 1):
                raise ValueError(f"attn_bias must be (B, H, >=T_q, >=T_k); got {tuple(attn_bias.shape)}")
            if attn_bias.dtype != q.dtype:
                attn_bias = attn_bias.to(q.dtype)
        if cache_seqlens is not None:
            if cache_seqlens.dim() != 1 or cache_seqlens.size(0) != B:
                raise ValueError(f"cache_seqlens must be (B,) = ({B},); got {tuple(cache_seqlens.shape)}")
            if cache_seqlens.dtype != torch.int32:
                cache_seqlens = cache_seqlens.to(torch.int32)
        if cache_seqstarts is not None:
            if cache_seqlens is None:
                raise ValueError("cache_seqstarts requires cache_seqlens (it bounds the window)")
            if cache_seqstarts.dim() != 1 or cache_seqstarts.size(0) != B:
                raise ValueError(f"cache_seqstarts must be (B,) = ({B},); got {tuple(cache_seqstarts.shape)}")
            if cache_seqstarts.dtype != torch.int32:
                cache_seqstarts = cache_seqstarts.to(torch.int32)
        if block_table is not None:
            if block_table.dim() != 2 or block_table.size(0) != B:
                raise ValueError("block_table must be (B, max_blocks_per_seq)")
            if block_table.dtype != torch.int32:
                block_table = block_table.to(torch.int32)
        want = (B, T_q, H, D) if token_major else (B, H, T_q, D)
        if out is not None and (tuple(out.shape) != want or out.dtype != q.dtype or not out.is_contiguous()):
            raise ValueError(f"out must be contiguous {want} in q's dtype")
    if out is None:
        out = torch.empty((B, T_q, H, D) if token_major else (B, H, T_q, D), dtype=q.dtype, device=q.device)
    q, qs = _canon(q)
    if paged:
        k, v = k.contiguous(), v.contiguous()
        ks = vs = None
        block_table = block_table.contiguous()
        # a bias narrower than the table's key range is fine as long as it covers the valid keys:
        # the kernel reads bias[..., j] only for j < cache_seqlens[b]
        if attn_bias is not None and attn_bias.size(3) < T_k and cache_seqlens is None:
            raise ValueError("a bias narrower than the block table needs cache_seqlens")
    else:
        k, ks = _canon(k)
        v, vs = _canon(v)
    bsb = bsh = bsq = 0
    if attn_bias is not None:
        if attn_bias.stride(3) != 1 and attn_bias.size(3) > 1:
            attn_bias = attn_bias.contiguous()
        bsb, bsh, bsq = attn_bias.stride(0), attn_bias.stride(1), attn_bias.stride(2)
    _lib.call("oasr_b200_fmha_bthd" if token_major else "oasr_b200_fmha", _p(out), _p(q), _p(k), _p(v), qs, ks, vs,
              _p(attn_bias), bsb, bsh, bsq,
              _p(cache_seqlens), _p(cache_seqstarts), _p(block_table),
              block_table.size(1) if paged else 0, block_size, num_blocks, B, H, H_kv, T_q, T_k, D,
              float(softmax_scale), int(bool(causal)), _DTYPE_ID[q.dtype], _stream(q))
    return out


def fmha_varlen(q, k, v, *, softmax_scale: float, cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor,
                max_seqlen_q: int, max_seqlen_k: int, attn_bias: Optional[torch.Tensor] = None,
                bias_offsets: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                validate: bool = True) -> torch.Tensor:
    """Variable-length (sequence-packed) attention (reference: functionals/attention.py:592-693).

    ``q`` ``(total_q, H, D)``, ``k``/``v`` ``(total_k, H_kv, D)``; segment ``s`` spans
    ``[cu[s], cu[s+1])`` and attends only to itself; ``attn_bias`` is the flat packed
    block-diagonal bias whose segment block ``(H, T_q_s, T_k_s)`` starts at ``bias_offsets[s]``.
    No host synchronisation (the reference's sm_100 route loops over ``cu_seqlens.tolist()``).
    """
    _need_cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, attn_bias, bias_offsets, out)
    if validate:
        if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
            raise ValueError("varlen q/k/v must be packed 3-D (total, H, D); got "
                             f"{tuple(q.shape)} / {tuple(k.shape)} / {tuple(v.shape)}")
        if k.shape != v.shape:
            raise ValueError(f"k and v must match: {tuple(k.shape)} vs {tuple(v.shape)}")
        if q.size(2) != k.size(2):
            raise ValueError("q and k head_dim must match")
        if q.size(1) % k.size(1) != 0:
            raise ValueError(f"H ({q.size(1)}) must be divisible by H_kv ({k.size(1)})")
        for name, cu in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_k", cu_seqlens_k)):
            if cu.dim() != 1 or cu.numel() < 2:
                raise ValueError(f"{name} must be 1-D with >= 2 entries")
        if cu_seqlens_q.numel() != cu_seqlens_k.numel():
            raise ValueError("cu_seqlens_q and cu_seqlens_k must have equal length")
        if (attn_bias is None) != (bias_offsets is None):
            raise ValueError("attn_bias and bias_offsets must be provided together")
        if out is not None and (out.shape != q.shape or out.dtype != q.dtype):
            raise ValueError("out must match q in shape/dtype")
        if q.dtype not in _HALF or k.dtype != q.dtype or v.dtype != q.dtype:
            raise ValueError("fmha_varlen supports fp16/bf16 with one dtype for q, k, v")
        if attn_bias is not None and attn_bias.dtype != q.dtype:
            attn_bias = attn_bias.to(q.dtype)
        if cu_seqlens_q.dtype != torch.int32:
            cu_seqlens_q = cu_seqlens_q.to(torch.int32)
        if cu_seqlens_k.dtype != torch.int32:
            cu_seqlens_k = cu_seqlens_k.to(torch.int32)
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device, memory_format=torch.contiguous_format)
    elif not out.is_contiguous():
        raise ValueError("out must be contiguous")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    off_i64 = 0
    if bias_offsets is not None:
        if bias_offsets.dtype == torch.int64:
            off_i64 = 1
        elif bias_offsets.dtype != torch.int32:
            bias_offsets = bias_offsets.to(torch.int64)
            off_i64 = 1
        bias_offsets = bias_offsets.contiguous()
        attn_bias = attn_bias.contiguous()
    S = cu_seqlens_q.numel() - 1
    _lib.call("oasr_b200_fmha_varlen", _p(out), _p(q), _p(k), _p(v), _p(attn_bias), _p(bias_offsets), off_i64,
              _p(cu_seqlens_q.contiguous()), _p(cu_seqlens_k.contiguous()), S, q.size(0), k.size(0),
              int(max_seqlen_q), q.size(1), k.size(1), q.size(2), float(softmax_scale), _DTYPE_ID[q.dtype],
              _stream(q))
    return out
