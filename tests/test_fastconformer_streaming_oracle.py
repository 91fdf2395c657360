"""CPU: the streaming restatement of the FastConformer layer stack equals the offline one.

The reference trains and serves this encoder with a chunked-limited attention mask over ABSOLUTE frame positions and
a causal conv module, which is what makes "one forward pass equal to the concatenation of the streaming chunks"
(oasr/models/nemotron/encoder.py:124-149).  The offline oracle is pinned to the reference at 2e-6
(tests/golden/fastconformer_tiny.npz); this test pins the chunked oracle to the offline one, chunk sizes of one, two
and four trained attention chunks, with cached histories cut to the trained left context or kept longer."""
import pytest
import torch

from oracle import fastconformer as OFC


@pytest.mark.parametrize("step,keep", [(4, -1), (8, -1), (16, 16), (4, 40)])
def test_chunked_layer_stack_equals_offline(step, keep):
    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=2, kernel=9, sliding_window=9, lookahead=3, bias=True)
    P = OFC.init_params(cfg, 99)
    T = 48
    hidden = torch.randn(1, T, cfg.hidden, generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        want = OFC.layers_forward(P, cfg, hidden, [T])[0]
        state = OFC.FastStreamState(cfg)
        got = torch.cat([OFC.layers_forward_chunk(P, cfg, state, hidden[0, t:t + step], keep_frames=keep)
                         for t in range(0, T, step)])
    assert state.offset == T
    assert (got - want).abs().max().item() < 2e-5


@pytest.mark.parametrize("step", [8, 16, 64])
def test_chunked_subsampling_equals_offline(step):
    """The streaming front end (cached two frames per stage, no right pad, no masks) against the offline one on a
    whole utterance whose length is a multiple of the 8x factor: identical arithmetic on the first T / 8 frames, so
    equal to rounding.  The offline pass emits one more frame, the one that reads its right pad; in a stream those
    inputs arrive with the next chunk."""
    sub = OFC.SubsamplingConfig(mels=80, channels=32, stages=3)
    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=1, kernel=9, sliding_window=9, lookahead=3, bias=True)
    P = OFC.init_params(cfg, 5)
    P.update(OFC.init_subsampling_params(sub, cfg.hidden, 6))
    T = 192
    feats = torch.randn(1, T, sub.mels, generator=torch.Generator().manual_seed(8))
    with torch.no_grad():
        want, out_len = OFC.subsampling_forward(P, sub, feats, torch.tensor([T]))
        state = OFC.SubsamplingStreamState(sub)
        got = torch.cat([OFC.subsampling_forward_chunk(P, sub, state, feats[0, t:t + step]) for t in range(0, T, step)])
    assert int(out_len[0]) == T // 8 + 1 and got.shape[0] == T // 8
    assert (got - want[0, :T // 8]).abs().max().item() < 2e-5
