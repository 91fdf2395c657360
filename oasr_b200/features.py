"""Kaldi-compatible FBANK features (+ global CMVN) on the GPU, feeding the encoder's subsampling front end.

Mirrors the reference's batched feature entry point (oasr/features/batched.py:295-332 ``batched_fbank``: ``(B, T)``
float32 waveforms + per-utterance sample counts -> ``(B, num_frames, num_mel_bins)`` float32 log-mel features +
int32 frame counts) for the configuration its batched path supports (snip_edges, no dither, no energy term,
Povey or Hamming window, power spectrum, log), with ``GlobalCMVN`` (oasr/layers/norm.py:571-584) optionally fused
into the same kernel.  One kernel launch (``oasr_b200_fbank``); there is no CPU path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache
from typing import Optional, Tuple

import torch

from . import _lib
from .functional import _need_cuda, _p, _stream


@dataclass(frozen=True)
class FbankConfig:
    """The fields of the reference's FeatureConfig (oasr/features/config.py:60-72) that the batched FBANK path reads."""

    sample_rate: int = 16000
    num_mel_bins: int = 80
    frame_length_ms: float = 25.0
    frame_shift_ms: float = 10.0
    preemphasis_coefficient: float = 0.97
    window_type: str = "povey"
    low_freq: float = 20.0
    high_freq: float = 0.0          # <= 0: offset from Nyquist

    @property
    def frame_length_samples(self) -> int:
        return int(self.sample_rate * self.frame_length_ms * 0.001)

    @property
    def frame_shift_samples(self) -> int:
        return int(self.sample_rate * self.frame_shift_ms * 0.001)

    @property
    def n_fft(self) -> int:
        return 1 << (self.frame_length_samples - 1).bit_length()


def mel_banks(cfg: FbankConfig) -> torch.Tensor:
    """Kaldi triangular mel filterbank ``(num_mel_bins, n_fft/2 + 1)`` fp32 on the CPU
    (oasr/features/batched.py:48-92 ``_mel_banks``)."""
    nyquist = 0.5 * cfg.sample_rate
    high = cfg.high_freq if cfg.high_freq > 0.0 else nyquist + cfg.high_freq
    if not 0.0 <= cfg.low_freq < high <= nyquist:
        raise ValueError("need 0 <= low_freq < high_freq <= Nyquist")
    to_mel = lambda f: 1127.0 * torch.log(1.0 + f / 700.0)
    edges = torch.linspace(to_mel(torch.tensor(cfg.low_freq)).item(), to_mel(torch.tensor(high)).item(), cfg.num_mel_bins + 2)
    bin_mel = to_mel(torch.arange(cfg.n_fft // 2 + 1, dtype=torch.float32) * (cfg.sample_rate / cfg.n_fft)).unsqueeze(0)
    left, center, right = edges[:-2].unsqueeze(1), edges[1:-1].unsqueeze(1), edges[2:].unsqueeze(1)
    up = (bin_mel - left) / (center - left)
    down = (right - bin_mel) / (right - center)
    return torch.clamp(torch.minimum(up, down), min=0.0).float()


def frame_window(cfg: FbankConfig) -> torch.Tensor:
    """Kaldi analysis window (oasr/features/batched.py:95-110 ``_frame_window``)."""
    n = cfg.frame_length_samples
    a = 2 * math.pi * torch.arange(n, dtype=torch.float32) / (n - 1)
    if cfg.window_type == "povey":
        return (0.5 - 0.5 * torch.cos(a)).pow(0.85)
    if cfg.window_type == "hamming":
        return 0.54 - 0.46 * torch.cos(a)
    raise ValueError(f"unsupported window_type {cfg.window_type!r} (povey or hamming)")


@lru_cache(maxsize=16)
def _tables(cfg: FbankConfig, device: torch.device):
    mel = mel_banks(cfg)
    nz = mel > 0
    lo = torch.where(nz.any(1), nz.float().argmax(1), torch.zeros(mel.size(0), dtype=torch.long))
    hi = torch.where(nz.any(1), mel.size(1) - nz.flip(1).float().argmax(1), torch.zeros(mel.size(0), dtype=torch.long))
    return (frame_window(cfg).to(device), mel.contiguous().to(device), lo.to(torch.int32).to(device), hi.to(torch.int32).to(device))


def feature_lengths(lengths, cfg: FbankConfig) -> torch.Tensor:
    """Frames per utterance under snip_edges (oasr/features/batched.py:283-292), int32."""
    lengths = torch.as_tensor(lengths).long()
    return torch.clamp((lengths - cfg.frame_length_samples) // cfg.frame_shift_samples + 1, min=0).to(torch.int32)


def batched_fbank(waveforms: torch.Tensor, lengths: torch.Tensor, cfg: FbankConfig = FbankConfig(),
                  cmvn: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(B, T)`` float32 CUDA waveforms (already scaled as the model expects) + ``(B,)`` sample counts ->
    ``(features (B, num_frames, num_mel_bins) float32, feat_lengths (B,) int32)``.  Frames past an utterance's own
    frame count are zeros.  ``cmvn = (mean, istd)`` applies ``(x - mean) * istd`` per mel bin in the same kernel."""
    _need_cuda(waveforms)
    if waveforms.dim() != 2 or waveforms.dtype != torch.float32:
        raise RuntimeError("waveforms must be a (B, T) float32 tensor")
    waveforms = waveforms.contiguous()
    B, T = waveforms.shape
    dev = waveforms.device
    L, hop = cfg.frame_length_samples, cfg.frame_shift_samples
    num_frames = max(0, (T - L) // hop + 1)
    feat_len = feature_lengths(lengths.cpu() if isinstance(lengths, torch.Tensor) else lengths, cfg).to(dev, non_blocking=True)
    out = torch.empty(B, num_frames, cfg.num_mel_bins, device=dev, dtype=torch.float32)
    if B == 0 or num_frames == 0:
        return out, feat_len
    window, mel, lo, hi = _tables(cfg, dev)
    len_dev = torch.as_tensor(lengths).to(torch.int32).to(dev, non_blocking=True)
    mean = istd = None
    if cmvn is not None:
        mean, istd = (t.to(dev, torch.float32).contiguous() for t in cmvn)
    _lib.call("oasr_b200_fbank", _p(out), _p(waveforms), _p(len_dev), _p(window), _p(mel), _p(lo), _p(hi), _p(mean), _p(istd),
              B, T, num_frames, L, hop, cfg.n_fft, cfg.num_mel_bins, float(cfg.preemphasis_coefficient),
              float(torch.finfo(torch.float32).tiny), _stream(waveforms))
    return out, feat_len
