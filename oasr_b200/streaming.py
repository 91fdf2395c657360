"""Paged streaming state for chunked Conformer inference.

``StreamingCache`` owns what the reference's ``BlockPool`` / ``AttentionCacheManager`` /
``SlotStateCache`` own for this path (oasr/cache/block_pool.py:33-41, attention_cache.py:234-292,
387-465, cnn_cache.py:37-48), in the same layouts: per-layer K/V page pools
``(L, num_blocks, block_size, H, D)``, ``block_table (slots, max_blocks) int32``,
``cache_seqlens (slots,) int32`` and the conv left-context buffer ``(L, slots, K-1, d)``.  The
page bookkeeping (free list, per-stream logical block lists, eviction of the oldest block) is host
logic; nothing here synchronises with the device.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class StreamingCache:
    def __init__(self, num_layers: int, heads: int, head_dim: int, d_model: int, conv_kernel: int, max_streams: int,
                 max_past_frames: int, chunk_frames: int = 16, block_size: int = 16, device="cuda",
                 dtype=torch.bfloat16, seed: Optional[int] = 0, kv_scales: Optional[torch.Tensor] = None):
        if chunk_frames % block_size:
            raise ValueError("a chunk must be a whole number of pages")
        self.L, self.H, self.D, self.d, self.K = num_layers, heads, head_dim, d_model, conv_kernel
        self.max_streams, self.block_size, self.chunk = max_streams, block_size, chunk_frames
        self.max_past = max_past_frames
        self.blocks_per_chunk = chunk_frames // block_size
        self.max_blocks = (max_past_frames + block_size - 1) // block_size + self.blocks_per_chunk
        self.num_blocks = max_streams * self.max_blocks
        self.device = torch.device(device)
        # pools are zero-initialised: stale page contents must be finite (they are masked, not skipped)
        # kv_scales (layers, 2, heads) fp32: the pools hold fp8 e4m3 codes (one byte per element, code 0 = 0.0)
        self.kv_scales = None
        if kv_scales is not None:
            if tuple(kv_scales.shape) != (num_layers, 2, heads):
                raise ValueError("kv_scales must be (layers, 2, heads)")
            self.kv_scales = kv_scales.to(self.device, torch.float32).contiguous()
            dtype_pool = torch.uint8
        else:
            dtype_pool = dtype
        self.k_pool = torch.zeros(num_layers, self.num_blocks, block_size, heads, head_dim, device=self.device, dtype=dtype_pool)
        self.v_pool = torch.zeros_like(self.k_pool)
        self.cnn_state = torch.zeros(num_layers, max_streams, conv_kernel - 1, d_model, device=self.device, dtype=dtype)
        # further per-stream buffers a front end keeps (leading dimension = slot); zeroed with the stream
        self.extra_state: List[torch.Tensor] = []
        # physical pages are handed out in a random order (a seeded permutation)
        if seed is None:
            order = list(range(self.num_blocks))
        else:
            order = torch.randperm(self.num_blocks, generator=torch.Generator().manual_seed(seed)).tolist()
        self._free: List[int] = order[::-1]
        self._blocks: List[List[int]] = [[] for _ in range(max_streams)]   # logical -> physical, per slot
        self._frames: List[int] = [0] * max_streams                         # committed (cached) frames per slot
        self._offset: List[int] = [0] * max_streams                         # encoder frames emitted per slot

    # ---- host bookkeeping -------------------------------------------------------------------
    def reset_stream(self, slot: int) -> None:
        self._free.extend(self._blocks[slot])
        self._blocks[slot] = []
        self._frames[slot] = 0
        self._offset[slot] = 0
        self.cnn_state[:, slot].zero_()
        for t in self.extra_state:
            t[slot].zero_()

    def prepare(self, slots: Sequence[int]):
        """Evict the oldest pages of every stream over its history cap, then give each stream the
        pages of the coming chunk.  Returns the device tensors one chunk forward needs:
        ``(block_table (B, max_blocks) int32, cache_seqlens, total_seqlens, pos_start (B,) int32, slot_ids int64)``."""
        rows, cached, total, pos = [], [], [], []
        for s in slots:
            while self._frames[s] > self.max_past:
                self._free.append(self._blocks[s].pop(0))
                self._frames[s] -= self.block_size
            for _ in range(self.blocks_per_chunk):
                if not self._free:
                    raise RuntimeError("page pool exhausted")
                self._blocks[s].append(self._free.pop())
            row = self._blocks[s] + [self._blocks[s][-1]] * (self.max_blocks - len(self._blocks[s]))
            rows.append(row)
            cached.append(self._frames[s])
            total.append(self._frames[s] + self.chunk)
            pos.append(self._offset[s] - self._frames[s])
        dev = self.device
        i32 = dict(dtype=torch.int32)
        return (torch.tensor(rows, **i32).to(dev, non_blocking=True), torch.tensor(cached, **i32).to(dev, non_blocking=True),
                torch.tensor(total, **i32).to(dev, non_blocking=True), torch.tensor(pos, **i32).to(dev, non_blocking=True),
                torch.tensor(list(slots), dtype=torch.int64).to(dev, non_blocking=True))

    def commit(self, slots: Sequence[int]) -> None:
        for s in slots:
            self._frames[s] += self.chunk
            self._offset[s] += self.chunk

    def cached_frames(self, slot: int) -> int:
        return self._frames[slot]
