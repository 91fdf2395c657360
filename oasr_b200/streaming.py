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

import numpy as np
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
            order = np.arange(self.num_blocks, dtype=np.int32)
        else:
            order = torch.randperm(self.num_blocks, generator=torch.Generator().manual_seed(seed)).numpy().astype(np.int32)
        # Host bookkeeping as arrays, so that a step over hundreds of streams is a handful of vectorised operations:
        # a stack of free pages (the top is the next page handed out), per slot the logical -> physical page list
        # (row of _table, first _nblk entries valid), the committed (cached) frames and the encoder frames emitted.
        self._free_stack = order[::-1].copy()
        self._nfree = self.num_blocks
        self._table = np.zeros((max_streams, self.max_blocks), dtype=np.int32)
        self._nblk = np.zeros(max_streams, dtype=np.int64)
        self._frames = np.zeros(max_streams, dtype=np.int64)
        self._offset = np.zeros(max_streams, dtype=np.int64)
        self._cols = np.arange(self.max_blocks, dtype=np.int64)[None, :]

    # ---- host bookkeeping -------------------------------------------------------------------
    @property
    def _free(self) -> List[int]:
        """The free pages, next one handed out last (introspection)."""
        return self._free_stack[:self._nfree].tolist()

    @property
    def _blocks(self) -> List[List[int]]:
        """Per slot the physical pages in logical order (introspection)."""
        return [self._table[s, :self._nblk[s]].tolist() for s in range(self.max_streams)]

    def _push_free(self, pages: np.ndarray) -> None:
        n = pages.size
        self._free_stack[self._nfree:self._nfree + n] = pages
        self._nfree += n

    def reset_stream(self, slot: int) -> None:
        self._push_free(self._table[slot, :self._nblk[slot]].copy())
        self._nblk[slot] = 0
        self._frames[slot] = 0
        self._offset[slot] = 0
        self.cnn_state[:, slot].zero_()
        for t in self.extra_state:
            t[slot].zero_()

    def prepare(self, slots: Sequence[int]):
        """Evict the oldest pages of every stream over its history cap, then give each stream the
        pages of the coming chunk.  Returns the device tensors one chunk forward needs:
        ``(block_table (B, max_blocks) int32, cache_seqlens, total_seqlens, pos_start (B,) int32, slot_ids int64)``.
        ``slots`` names every stream at most once."""
        s = np.asarray(slots, dtype=np.int64)
        n = s.size
        while True:                                   # oldest whole pages of the streams over their cap
            over = s[self._frames[s] > self.max_past]
            if over.size == 0:
                break
            self._push_free(self._table[over, 0].copy())
            self._table[over, :-1] = self._table[over, 1:]
            self._nblk[over] -= 1
            self._frames[over] -= self.block_size
        need = n * self.blocks_per_chunk
        if need > self._nfree:
            raise RuntimeError("page pool exhausted")
        pages = self._free_stack[self._nfree - need:self._nfree][::-1].reshape(n, self.blocks_per_chunk)
        self._nfree -= need
        for j in range(self.blocks_per_chunk):
            self._table[s, self._nblk[s] + j] = pages[:, j]
        self._nblk[s] += self.blocks_per_chunk
        # one int32 staging array: the table rows (unused tail entries repeat the stream's last page), then the
        # cached / total frame counts and the position of the first key
        mb = self.max_blocks
        stage = np.empty(n * (mb + 3), dtype=np.int32)
        last = (self._nblk[s] - 1)[:, None]
        stage[:n * mb] = np.take_along_axis(self._table[s], np.minimum(self._cols, last), axis=1).reshape(-1)
        frames = self._frames[s]
        stage[n * mb:n * mb + n] = frames
        stage[n * mb + n:n * mb + 2 * n] = frames + self.chunk
        stage[n * mb + 2 * n:] = self._offset[s] - frames
        dev = self.device
        packed = torch.from_numpy(stage)
        slot_ids = torch.from_numpy(s)
        if dev.type == "cuda":
            packed = packed.pin_memory().to(dev, non_blocking=True)
            slot_ids = slot_ids.pin_memory().to(dev, non_blocking=True)
        return (packed[:n * mb].view(n, mb), packed[n * mb:n * mb + n], packed[n * mb + n:n * mb + 2 * n],
                packed[n * mb + 2 * n:], slot_ids)

    def commit(self, slots: Sequence[int]) -> None:
        s = np.asarray(slots, dtype=np.int64)
        self._frames[s] += self.chunk
        self._offset[s] += self.chunk

    def cached_frames(self, slot: int) -> int:
        return int(self._frames[slot])
