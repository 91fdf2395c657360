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
