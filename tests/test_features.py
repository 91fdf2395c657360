"""FBANK front end: the CPU oracle against the fixture written from the reference (any machine), the CUDA kernel
against the oracle and the fixture (GPU)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import features as OFE
from tests.golden.make_features_golden import features_case

GOLD = Path(__file__).resolve().parent / "golden" / "features.npz"
CASES = {"povey80": {}, "hamming40": dict(window_type="hamming", num_mel_bins=40, low_freq=0.0, high_freq=-400.0)}


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_equals_the_reference_fixture(name):
    gold = np.load(GOLD)
    wave, lengths = features_case()
    got, glen = OFE.fbank(wave, lengths, OFE.FbankConfig(**CASES[name]))
    assert glen.tolist() == gold[name + "_len"].tolist()
    assert np.abs(got.numpy() - gold[name]).max() < 1e-4


def test_oracle_edge_cases():
    cfg = OFE.FbankConfig()
    short = torch.zeros(2, 300)
    out, n = OFE.fbank(short, torch.tensor([300, 100]), cfg)           # shorter than one frame
    assert out.shape == (2, 0, 80) and n.tolist() == [0, 0]
    out, n = OFE.fbank(torch.zeros(1, 400), torch.tensor([400]), cfg)  # exactly one frame of silence: the log floor
    assert out.shape == (1, 1, 80) and torch.isfinite(out).all() and out.max().item() < -80.0


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(CASES))
def test_kernel_matches_oracle_and_reference_fixture(name):
    import oasr_b200 as ob
    from oasr_b200 import features as F

    gold = np.load(GOLD)
    wave, lengths = features_case()
    cfg = F.FbankConfig(**CASES[name])
    got, glen = F.batched_fbank(wave.cuda(), lengths, cfg)
    torch.cuda.synchronize()
    assert ob.device_status() == 0
    assert glen.cpu().tolist() == gold[name + "_len"].tolist()
    want, _ = OFE.fbank(wave, lengths, OFE.FbankConfig(**CASES[name]))
    got = got.cpu()
    for b, n in enumerate(glen.cpu().tolist()):
        d = (got[b, :n] - want[b, :n]).abs()
        assert d.max().item() < 2e-3, (b, d.max().item())               # fp32 FFT and summation order
        assert np.abs(got[b, :n].numpy() - gold[name][b, :n]).max() < 2e-3
        assert torch.count_nonzero(got[b, n:]) == 0                     # frames outside the utterance are zeros
    print(f"fbank {name}: max-abs vs oracle {(got[0] - want[0]).abs().max().item():.2e}")


@pytest.mark.gpu
def test_kernel_cmvn_ragged_batch_and_too_short_input():
    import oasr_b200 as ob
    from oasr_b200 import features as F

    g = torch.Generator().manual_seed(5)
    lengths = torch.tensor([16000, 399, 400, 7777, 0], dtype=torch.int32)
    wave = torch.randn(5, 16000, generator=g) * 0.2
    mean, istd = torch.randn(80, generator=g), torch.rand(80, generator=g) + 0.5
    got, glen = F.batched_fbank(wave.cuda(), lengths, cmvn=(mean, istd))
    torch.cuda.synchronize()
    assert ob.device_status() == 0
    want, wlen = OFE.fbank(wave, lengths, cmvn=(mean, istd))
    assert glen.cpu().tolist() == wlen.tolist() == [98, 0, 1, 47, 0]
    got = got.cpu()
    for b, n in enumerate(wlen.tolist()):
        if n:
            assert (got[b, :n] - want[b, :n]).abs().max().item() < 3e-3
        assert torch.count_nonzero(got[b, n:]) == 0
    empty, elen = F.batched_fbank(torch.zeros(2, 100).cuda(), torch.tensor([100, 50]))
    assert empty.shape == (2, 0, 80) and elen.cpu().tolist() == [0, 0]


@pytest.mark.gpu
def test_audio_to_tokens_through_fbank_and_encoder():
    """The front end feeds the encoder directly on the device: waveform -> FBANK + CMVN -> Conformer + CTC tokens equals
    the same encoder on the oracle's features."""
    from oasr_b200 import features as F
    from oasr_b200.encoder import ConformerCTC, ConformerConfig
    from oasr_b200.weights import init_params

    cfg = ConformerConfig(d_model=128, heads=2, ffn=256, layers=2, vocab=90)
    model = ConformerCTC(cfg, init_params(cfg, 77), device="cuda", dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(9)
    lengths = torch.tensor([24000, 11111], dtype=torch.int32)
    wave = torch.randn(2, 24000, generator=g) * 0.1
    feats, flen = F.batched_fbank(wave.cuda(), lengths)
    lp_a, ol_a = model.forward_offline_packed(feats, flen.cpu().tolist())
    want, wlen = OFE.fbank(wave, lengths)
    lp_b, ol_b = model.forward_offline_packed(want.cuda(), wlen.tolist())
    assert torch.equal(ol_a, ol_b)
    valid = (torch.arange(lp_a.shape[1])[None, :] < ol_a.cpu()[:, None])
    assert (lp_a.cpu() - lp_b.cpu())[valid].abs().max().item() < 2e-2
