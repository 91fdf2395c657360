"""Host-side logic that needs no GPU: CTC collapse, streaming page bookkeeping."""
import numpy as np
import pytest

from oasr_b200.encoder import ConformerCTC


def _collapse_loop(ids, segs):
    out, pos = [], 0
    for n in segs:
        hyp, prev = [], None
        for t in ids[pos:pos + n]:
            if t != prev and t != 0:
                hyp.append(t)
            prev = t
        out.append(hyp)
        pos += n
    return out


def test_ctc_collapse_matches_the_frame_loop():
    rng = np.random.default_rng(0)
    for _ in range(500):
        segs = [int(x) for x in rng.integers(0, 9, size=rng.integers(1, 7))]
        ids = rng.integers(0, 4, size=sum(segs)).tolist()
        assert ConformerCTC._collapse(ids, segs) == _collapse_loop(ids, segs)
    assert ConformerCTC._collapse([], [0, 0]) == [[], []]


def test_streaming_cache_bookkeeping_on_cpu():
    """Eviction keeps at most max_past frames of history before each chunk, pages are never shared
    between streams and return to the free list when a stream is reset."""
    from oasr_b200.streaming import StreamingCache

    c = StreamingCache(num_layers=1, heads=2, head_dim=64, d_model=128, conv_kernel=15, max_streams=3, max_past_frames=32,
                       chunk_frames=16, block_size=16, device="cpu", dtype=__import__("torch").float32, seed=3)
    assert c.max_blocks == 3 and c.num_blocks == 9
    for step in range(6):
        table, cached, total, pos, slots = c.prepare([0, 2])
        assert cached.tolist() == [min(step * 16, 32)] * 2
        assert total.tolist() == [min(step * 16, 32) + 16] * 2
        assert pos.tolist() == [step * 16 - min(step * 16, 32)] * 2
        used = [set(c._blocks[s]) for s in (0, 2)]
        assert not (used[0] & used[1]) and all(len(u) == len(c._blocks[s]) for u, s in zip(used, (0, 2)))
        assert table.shape == (2, 3) and slots.tolist() == [0, 2]
        c.commit([0, 2])
    free_before = len(c._free)
    c.reset_stream(2)
    assert len(c._free) == free_before + 3 and c.cached_frames(2) == 0
    with pytest.raises(ValueError):
        StreamingCache(1, 2, 64, 128, 15, 1, 32, chunk_frames=24, block_size=16, device="cpu")


def test_streaming_cache_invariants_under_random_batches_on_cpu():
    """The vectorised page bookkeeping over random subsets of streams, two pages per chunk, resets in between: every
    physical page is held by exactly one stream or the free list, a stream holds the pages of its capped history plus
    the coming chunk in logical order, the returned rows repeat the last page in their unused tail, and an exhausted
    pool is refused before anything is handed out."""
    import numpy as np
    import torch

    from oasr_b200.streaming import StreamingCache

    rng = np.random.default_rng(5)
    S, bs, chunk, max_past = 12, 8, 16, 40
    c = StreamingCache(num_layers=1, heads=2, head_dim=64, d_model=128, conv_kernel=15, max_streams=S, max_past_frames=max_past,
                       chunk_frames=chunk, block_size=bs, device="cpu", dtype=torch.float32, seed=11)
    assert c.blocks_per_chunk == 2 and c.max_blocks == 5 + 2
    frames = [0] * S            # a plain-Python model of the committed history and the emitted frames
    emitted = [0] * S
    for step in range(200):
        if step % 17 == 5:
            s = int(rng.integers(S))
            c.reset_stream(s)
            frames[s] = emitted[s] = 0
        slots = sorted(rng.choice(S, size=int(rng.integers(1, S + 1)), replace=False).tolist())
        table, cached, total, pos, ids = c.prepare(slots)
        for s in slots:
            while frames[s] > max_past:
                frames[s] -= bs
        assert ids.tolist() == slots
        assert cached.tolist() == [frames[s] for s in slots]
        assert total.tolist() == [frames[s] + chunk for s in slots]
        assert pos.tolist() == [emitted[s] - frames[s] for s in slots]
        blocks, free = c._blocks, c._free
        held = [p for b in blocks for p in b]
        assert len(set(held)) == len(held) and not (set(held) & set(free)) and len(held) + len(free) == c.num_blocks
        for row, s in zip(table.tolist(), slots):
            n = len(blocks[s])
            assert n == (frames[s] + bs - 1) // bs + c.blocks_per_chunk
            assert row[:n] == blocks[s] and all(x == blocks[s][-1] for x in row[n:])
        c.commit(slots)
        for s in slots:
            frames[s] += chunk
            emitted[s] += chunk
    # exhaustion: a pool with too few pages refuses the step and keeps its state
    small = StreamingCache(1, 2, 64, 128, 15, 2, max_past, chunk_frames=chunk, block_size=bs, device="cpu", dtype=torch.float32)
    small._nfree = 3                      # fewer than the four pages two streams need
    before = (small._nfree, small._nblk.copy())
    with pytest.raises(RuntimeError, match="exhausted"):
        small.prepare([0, 1])
    assert small._nfree == before[0] and (small._nblk == before[1]).all()
