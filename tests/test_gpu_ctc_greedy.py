"""GPU: greedy CTC collapse on the device against the host rule (drop repeats, then blanks, per utterance;
csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55), on ragged batches with empty and one-frame utterances."""
import numpy as np
import pytest
import torch

from oasr_b200 import fused

pytestmark = pytest.mark.gpu


def _host_rule(ids, lens, blank):
    out, times, pos = [], [], 0
    for n in lens:
        seg = ids[pos:pos + n]
        pos += n
        toks, tt, prev = [], [], None
        for t, v in enumerate(seg):
            if v != prev and v != blank:
                toks.append(int(v))
                tt.append(t)
            prev = v
        out.append(toks)
        times.append(tt)
    return out, times


@pytest.mark.parametrize("blank", [0, 3])
def test_collapse_matches_the_host_rule(blank):
    rng = np.random.default_rng(5 + blank)
    lens = [0, 1, 1, 7, 255, 256, 257, 700, 0, 1999, 33]
    total = sum(lens)
    # a small alphabet with long runs, so that repeats, blanks and boundaries between equal ids all occur
    ids = np.repeat(rng.integers(0, 6, size=total), rng.integers(1, 4, size=total))[:total].astype(np.int32)
    ids[1] = ids[0] = 5          # the two one-frame utterances carry the same id: a boundary, not a repeat
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    want, want_times = _host_rule(ids.tolist(), lens, blank)
    tokens, counts, times = fused.ctc_greedy_collapse(torch.from_numpy(ids).cuda(), torch.from_numpy(cu).cuda(), max(lens), blank,
                                                      want_times=True)
    tokens, counts, times = tokens.cpu().numpy(), counts.cpu().tolist(), times.cpu().numpy()
    assert counts == [len(w) for w in want]
    for b, w in enumerate(want):
        assert tokens[b, :len(w)].tolist() == w
        assert times[b, :len(w)].tolist() == want_times[b]
        assert (tokens[b, len(w):] == blank).all() and (times[b, len(w):] == -1).all()


def test_rows_longer_than_max_len_are_cut_and_counted_as_cut():
    ids = torch.arange(1, 41, dtype=torch.int32).cuda()          # 40 distinct non-blank ids: 40 tokens
    cu = torch.tensor([0, 40], dtype=torch.int32).cuda()
    tokens, counts, _ = fused.ctc_greedy_collapse(ids, cu, 16)
    assert counts.tolist() == [16] and tokens.cpu()[0].tolist() == list(range(1, 17))
    empty_tokens, empty_counts, _ = fused.ctc_greedy_collapse(ids[:0], torch.zeros(1, dtype=torch.int32).cuda(), 4)
    assert empty_tokens.shape == (0, 4) and empty_counts.numel() == 0
