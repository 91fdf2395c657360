"""Write ``features.npz``: the reference's own batched FBANK output for seeded waveforms.

    OASR_REFERENCE=<path of the reference checkout> python tests/golden/make_features_golden.py

Imports the reference (CPU, torch route of oasr/features/batched.py), runs ``batched_fbank`` on the seeded waveforms
of ``features_case()`` below, checks the CPU oracle against it and stores the reference's features.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))


def features_case():
    """Two utterances of 0.83 s and 0.40 s at 16 kHz, iid N(0, 0.1) plus a DC offset and a slow sine (so that DC
    removal, pre-emphasis and the low mel bins all matter), the second one padded with noise past its length."""
    g = torch.Generator().manual_seed(23)
    T = 13333
    t = torch.arange(T, dtype=torch.float32) / 16000.0
    wave = torch.randn(2, T, generator=g) * 0.1 + 0.05 + 0.3 * torch.sin(2 * torch.pi * 220.0 * t)
    return wave, torch.tensor([T, 6407], dtype=torch.int32)


if __name__ == "__main__":
    ref = os.environ.get("OASR_REFERENCE")
    if not ref:
        raise SystemExit("set OASR_REFERENCE to the path of the reference checkout")
    os.environ["OASR_LAYERS_BACKEND"] = "torch"
    sys.path.insert(0, ref)
    from oasr.features.batched import batched_fbank  # noqa: E402  (the reference)
    from oasr.features.config import FeatureConfig  # noqa: E402

    from oracle import features as OFE  # noqa: E402

    wave, lengths = features_case()
    out = {}
    for name, kw in (("povey80", {}), ("hamming40", dict(window_type="hamming", num_mel_bins=40, low_freq=0.0, high_freq=-400.0))):
        cfg = FeatureConfig(**kw)
        feats, flen = batched_fbank(wave, lengths, cfg)
        ora, olen = OFE.fbank(wave, lengths, OFE.FbankConfig(**kw))
        assert torch.equal(flen.cpu().int(), olen)
        d = (feats - ora).abs().max().item()
        print(f"{name}: reference vs oracle max-abs {d:.3e}, frames {tuple(feats.shape)}, lengths {flen.tolist()}")
        assert d < 1e-4
        out[name] = feats.numpy()
        out[name + "_len"] = flen.numpy()
    np.savez_compressed(HERE / "features.npz", **out)
