"""Paged KV-cache data movement with the reference's layout (oasr/cache/paged_kv.py,
oasr/cache/block_pool.py:33-41): per-layer pools ``(num_blocks, block_size, H_kv, D)``,
``block_table (B, max_blocks_per_seq)`` int32, ``cache_seqlens (B,)`` int32."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Union

import torch

from . import _lib
from .attention import gather_paged_kv  # noqa: F401  (re-exported)
from .functional import _need_cuda, _p, _stream


def write_kv_chunk(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor, new_k: torch.Tensor,
                   new_v: torch.Tensor, offset: Union[int, torch.Tensor]) -> None:
    """Scatter ``new_k`` / ``new_v`` ``(B, H_kv, T, D)`` into the pools: frame ``t`` of stream ``b``
    lands at logical position ``offset[b] + t`` (reference: PagedKVCache.write_kv_chunk,
    oasr/cache/paged_kv.py:63-137; index rule flat_write_index :23-40).  One kernel, no
    frame-major staging copy; the head-first inputs may be strided views."""
    _need_cuda(k_cache, v_cache, block_table, new_k, new_v)
    if new_k.shape != new_v.shape or new_k.dim() != 4:
        raise ValueError("new_k / new_v must be (B, H_kv, T, D) and match")
    B, Hkv, T, D = new_k.shape
    num_blocks, bs = k_cache.size(0), k_cache.size(1)
    if k_cache.shape != v_cache.shape or k_cache.size(2) != Hkv or k_cache.size(3) != D:
        raise ValueError("pools must be (num_blocks, block_size, H_kv, D) matching the new chunk")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("pools must be contiguous")
    if new_k.dtype != k_cache.dtype or new_v.dtype != v_cache.dtype:
        raise ValueError("chunk and pool dtypes must match")
    if isinstance(offset, int):
        offset = torch.full((B,), offset, dtype=torch.int32, device=new_k.device)
    elif offset.dtype != torch.int32:
        offset = offset.to(torch.int32)
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    block_table = block_table.contiguous()
    if new_k.stride(3) != 1:
        new_k = new_k.contiguous()
    if new_v.stride() != new_k.stride():
        new_v = new_v.contiguous()
        new_k = new_k.contiguous()
    _lib.call("oasr_b200_paged_kv_write", _p(k_cache), _p(v_cache), _p(new_k), _p(new_v), _p(block_table),
              _p(offset.contiguous()), B, Hkv, T, D, new_k.stride(0), new_k.stride(1), new_k.stride(2),
              block_table.size(1), bs, num_blocks, k_cache.element_size(), _stream(new_k))


@dataclass
class PagedKVCache:
    """Per-layer pool views plus the shared per-batch paging state; same fields and
    methods as the reference descriptor (oasr/cache/paged_kv.py:43-180)."""

    k_cache: torch.Tensor
    v_cache: torch.Tensor
    block_table: torch.Tensor
    cache_seqlens: torch.Tensor
    block_size: int
    host_seqlen_max: int = 0

    def write_kv_chunk(self, new_k: torch.Tensor, new_v: torch.Tensor, *, offset: Union[int, torch.Tensor]) -> None:
        write_kv_chunk(self.k_cache, self.v_cache, self.block_table, new_k, new_v, offset)

    def gather_full_kv(self, max_total_kv: int):
        B = self.block_table.size(0)
        Hkv, D = self.k_cache.size(2), self.k_cache.size(3)
        if max_total_kv == 0:
            empty = torch.zeros(B, Hkv, 0, D, dtype=self.k_cache.dtype, device=self.k_cache.device)
            return empty, empty.clone()
        nblk = (max_total_kv + self.block_size - 1) // self.block_size
        k, v = gather_paged_kv(self.k_cache, self.v_cache, self.block_table[:, :nblk])
        return k[:, :, :max_total_kv], v[:, :, :max_total_kv]


def gather_rows(src: torch.Tensor, index: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """``out[i] = src[index[i]]`` over the leading dimension (an index outside ``[0, len(src))`` gives a zero row):
    ``pack_hidden`` / gapped-conv gather / ``SlotTensor.gather``
    (oasr/models/conformer/packing.py:222-225, oasr/cache/state.py:88-94)."""
    _need_cuda(src, index, out)
    src = src.contiguous()
    row_bytes = (src.numel() // src.size(0)) * src.element_size() if src.size(0) else 0
    want_shape = (index.numel(),) + tuple(src.shape[1:])
    if out is None:
        out = torch.empty(want_shape, device=src.device, dtype=src.dtype)
    elif tuple(out.shape) != want_shape or out.dtype != src.dtype or not out.is_contiguous() or out.device != src.device:
        raise ValueError(f"out must be a contiguous {src.dtype} tensor of shape {want_shape} on {src.device}")
    if index.dtype != torch.int64:
        index = index.to(torch.int64)
    if index.numel() and row_bytes:
        with torch.cuda.device(src.device):
            _lib.call("oasr_b200_gather_rows", _p(out), _p(src), _p(index.contiguous()), index.numel(), row_bytes,
                      src.size(0), _stream(src))
    return out


def scatter_rows(dst: torch.Tensor, index: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``dst[index[i]] = src[i]`` (``index_copy_`` along dim 0: unpack_hidden / gapped-conv scatter /
    ``SlotTensor.scatter``); an index outside ``[0, len(dst))`` is skipped."""
    _need_cuda(dst, index, src)
    if not dst.is_contiguous():
        raise ValueError("dst must be contiguous")
    src = src.contiguous()
    if src.dtype != dst.dtype or tuple(src.shape[1:]) != tuple(dst.shape[1:]) or src.size(0) != index.numel():
        raise ValueError("src must hold one row of dst's row shape and dtype per index")
    row_bytes = (src.numel() // src.size(0)) * src.element_size() if src.size(0) else 0
    if index.dtype != torch.int64:
        index = index.to(torch.int64)
    if index.numel() and row_bytes:
        with torch.cuda.device(src.device):
            _lib.call("oasr_b200_scatter_rows", _p(dst), _p(src), _p(index.contiguous()), index.numel(), row_bytes,
                      dst.size(0), _stream(src))
    return dst
