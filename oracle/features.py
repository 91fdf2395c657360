"""CPU oracle of the batched Kaldi FBANK front end and global CMVN.  TEST INFRASTRUCTURE ONLY.

Restates, in fp32 torch, the reference's torch route of ``batched_fbank``:
  * framing (snip_edges), per-frame DC removal, pre-emphasis with the first sample replicated, analysis window,
    zero-padded power spectrum, mel filterbank, log with the float32-tiny floor
                                                           oasr/features/batched.py:209-268 (``_log_mel_torch``)
  * Kaldi triangular mel filterbank                         oasr/features/batched.py:48-92  (``_mel_banks``)
  * Povey / Hamming window                                  oasr/features/batched.py:95-110 (``_frame_window``)
  * frame counts                                            oasr/features/batched.py:283-292 (``_feat_lengths``)
  * GlobalCMVN ``(x - mean) * istd``                        oasr/layers/norm.py:571-584
Pinned by ``tests/golden/features.npz`` (written from the reference by ``tests/golden/make_features_golden.py``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class FbankConfig:
    sample_rate: int = 16000
    num_mel_bins: int = 80
    frame_length_ms: float = 25.0
    frame_shift_ms: float = 10.0
    preemphasis_coefficient: float = 0.97
    window_type: str = "povey"
    low_freq: float = 20.0
    high_freq: float = 0.0

    @property
    def frame_length(self) -> int:
        return int(self.sample_rate * self.frame_length_ms * 0.001)

    @property
    def frame_shift(self) -> int:
        return int(self.sample_rate * self.frame_shift_ms * 0.001)


def mel_banks(cfg: FbankConfig, n_fft: int) -> torch.Tensor:
    nyquist = 0.5 * cfg.sample_rate
    high = cfg.high_freq if cfg.high_freq > 0.0 else nyquist + cfg.high_freq

    def to_mel(f):
        return 1127.0 * torch.log(1.0 + f / 700.0)

    edges = torch.linspace(to_mel(torch.tensor(cfg.low_freq)).item(), to_mel(torch.tensor(high)).item(), cfg.num_mel_bins + 2)
    bin_mel = to_mel(torch.arange(n_fft // 2 + 1, dtype=torch.float32) * (cfg.sample_rate / n_fft)).unsqueeze(0)
    left, center, right = edges[:-2].unsqueeze(1), edges[1:-1].unsqueeze(1), edges[2:].unsqueeze(1)
    return torch.clamp(torch.minimum((bin_mel - left) / (center - left), (right - bin_mel) / (right - center)), min=0.0)


def window(cfg: FbankConfig) -> torch.Tensor:
    n = cfg.frame_length
    a = 2 * math.pi * torch.arange(n, dtype=torch.float32) / (n - 1)
    return (0.5 - 0.5 * torch.cos(a)).pow(0.85) if cfg.window_type == "povey" else 0.54 - 0.46 * torch.cos(a)


def fbank(waveforms: torch.Tensor, lengths: torch.Tensor, cfg: FbankConfig = FbankConfig(), cmvn=None):
    """``(B, T)`` fp32 waveforms -> ``(log_mel (B, num_frames, num_mel), feat_lengths (B,) int32)``."""
    L, hop = cfg.frame_length, cfg.frame_shift
    B, T = waveforms.shape
    feat_len = torch.clamp((lengths.long() - L) // hop + 1, min=0).to(torch.int32)
    if T < L:
        return torch.zeros(B, 0, cfg.num_mel_bins), feat_len
    frames = waveforms.float().unfold(-1, L, hop)
    frames = frames - frames.mean(dim=-1, keepdim=True)
    pre = torch.empty_like(frames)
    pre[..., 1:] = frames[..., 1:] - cfg.preemphasis_coefficient * frames[..., :-1]
    pre[..., 0] = frames[..., 0] - cfg.preemphasis_coefficient * frames[..., 0]
    windowed = pre * window(cfg)
    n_fft = 1 << (L - 1).bit_length()
    spectrum = torch.fft.rfft(torch.nn.functional.pad(windowed, (0, n_fft - L)), n=n_fft)
    power = spectrum.real.pow(2) + spectrum.imag.pow(2)
    mel = torch.matmul(power, mel_banks(cfg, n_fft).t())
    out = torch.log(mel.clamp_min(torch.finfo(torch.float32).tiny))
    if cmvn is not None:
        out = (out - cmvn[0]) * cmvn[1]
    return out, feat_len
