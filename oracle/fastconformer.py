"""CPU oracle (test infrastructure, never imported by the product path) for the FastConformer / Nemotron
encoder: fp32 torch restatement of the reference's 8x subsampling front end and layer composition.
Pinned against the reference itself by ``tests/golden/make_golden.py`` (fixture
``tests/golden/fastconformer_tiny.npz``).

Restated from the reference (paths inside its project):
  * ``rel_shift``                          oasr/models/nemotron/encoder.py:82-96
  * ``relative_position_embedding``        oasr/models/nemotron/encoder.py:99-121
  * ``chunked_limited_mask``               oasr/models/nemotron/encoder.py:124-149
  * conv module (pw1, GLU, causal depthwise, LayerNorm+SiLU, pw2)   encoder.py:150-214
  * layer (macaron FFNs, fused add+LayerNorm chain)                 encoder.py:217-267
  * attention with the Transformer-XL position bias, MASK_FLOOR     encoder.py:300-359
  * encoder loop: window mask & key padding, silent rows            encoder.py:542-583
  * 8x causal depthwise-separable subsampling                       oasr/models/nemotron/subsampling.py:26-131, 204-224
The RNN-T head is not restated here.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

MASK_FLOOR = -1.0e4


@dataclass
class FastConformerConfig:
    hidden: int = 256
    heads: int = 2
    ffn: int = 512
    layers: int = 2
    kernel: int = 9
    sliding_window: int = 9      # left context = sliding_window - 1 frames
    lookahead: int = 3           # right context in frames (chunk = lookahead + 1)
    bias: bool = True            # attention_bias and convolution_bias of the reference config
    eps: float = 1e-5

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


TINY = FastConformerConfig()


def param_spec(cfg: FastConformerConfig):
    """(name, shape, kind) in the reference's state-dict naming; kind: 'w' matrix, 'g' norm gain, 'b' bias."""
    C, Fd, K, H, D = cfg.hidden, cfg.ffn, cfg.kernel, cfg.heads, cfg.head_dim
    out = []
    for i in range(cfg.layers):
        p = f"layers.{i}."
        for ff in ("feed_forward1", "feed_forward2"):
            out += [(p + ff + ".linear1.weight", (Fd, C), "w"), (p + ff + ".linear2.weight", (C, Fd), "w")]
            if cfg.bias:
                out += [(p + ff + ".linear1.bias", (Fd,), "b"), (p + ff + ".linear2.bias", (C,), "b")]
        a = p + "self_attn."
        out += [(a + "bias_u", (H, D), "w"), (a + "bias_v", (H, D), "w")]
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            out.append((a + n + ".weight", (C, C), "w"))
            if cfg.bias:
                out.append((a + n + ".bias", (C,), "b"))
        out.append((a + "relative_k_proj.weight", (C, C), "w"))
        c = p + "conv."
        out += [(c + "pointwise_conv1.weight", (2 * C, C, 1), "w"), (c + "depthwise_conv.weight", (K, 1, C), "w"),
                (c + "norm.weight", (C,), "g"), (c + "norm.bias", (C,), "b"), (c + "pointwise_conv2.weight", (C, C, 1), "w")]
        if cfg.bias:
            out += [(c + "pointwise_conv1.bias", (2 * C,), "b"), (c + "depthwise_conv.bias", (C,), "b"),
                    (c + "pointwise_conv2.bias", (C,), "b")]
        for n in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
            out += [(p + n + ".weight", (C,), "g"), (p + n + ".bias", (C,), "b")]
    return out


def init_params(cfg: FastConformerConfig, seed: int, w_std: float = 0.06) -> Dict[str, torch.Tensor]:
    """Seeded synthetic weights: matrices ~ N(0, w_std), gains 1 + N(0, 0.1), biases N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    P = {}
    for name, shape, kind in param_spec(cfg):
        if kind == "w":
            P[name] = torch.randn(shape, generator=g) * w_std
        elif kind == "g":
            P[name] = 1.0 + torch.randn(shape, generator=g) * 0.1
        else:
            P[name] = torch.randn(shape, generator=g) * 0.1
    return P


def rel_shift(scores: torch.Tensor) -> torch.Tensor:
    b, h, t_q, p = scores.shape
    padded = F.pad(scores, (1, 0))
    return padded.view(b, h, -1, t_q)[:, :, 1:].view(b, h, t_q, p)


def relative_position_embedding(length: int, dim: int) -> torch.Tensor:
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    positions = torch.arange(length - 1, -length, -1, dtype=torch.float32)
    freqs = torch.outer(positions, inv_freq)
    return torch.stack([freqs.sin(), freqs.cos()], dim=-1).reshape(freqs.size(0), dim)   # (2L-1, dim)


def chunked_limited_mask(query_len: int, key_len: int, left_context: int, right_context: int) -> torch.Tensor:
    chunk = right_context + 1
    left_chunks = left_context // chunk if left_context >= 0 else key_len
    q_chunk = torch.arange(query_len).div(chunk, rounding_mode="trunc")
    k_chunk = torch.arange(key_len).div(chunk, rounding_mode="trunc")
    diff = q_chunk.unsqueeze(1) - k_chunk.unsqueeze(0)
    return (diff >= 0) & (diff <= left_chunks)   # (T_q, T_k) bool


def _lin(P, name, x):
    return F.linear(x, P[name + ".weight"], P.get(name + ".bias"))


def _ln(P, name, x, eps):
    return F.layer_norm(x, (x.size(-1),), P[name + ".weight"], P[name + ".bias"], eps)


def _ffn(P, p, x):
    return _lin(P, p + ".linear2", F.silu(_lin(P, p + ".linear1", x)))


def attention(P, a, cfg, x, pos_emb, attn_mask, silent):
    B, T, C = x.shape
    H, D = cfg.heads, cfg.head_dim
    split = lambda t: t.view(B, T, H, D).transpose(1, 2)      # (B, H, T, D)
    q, k, v = split(_lin(P, a + "q_proj", x)), split(_lin(P, a + "k_proj", x)), split(_lin(P, a + "v_proj", x))
    rel_k = F.linear(pos_emb, P[a + "relative_k_proj.weight"]).view(1, -1, H, D)
    scaling = D ** -0.5
    matrix_bd = (q + P[a + "bias_v"].unsqueeze(1)) @ rel_k.permute(0, 2, 3, 1)
    matrix_bd = rel_shift(matrix_bd)[..., :T] * scaling
    bias = matrix_bd.masked_fill(attn_mask.logical_not(), MASK_FLOOR)
    scores = ((q + P[a + "bias_u"].unsqueeze(1)) @ k.transpose(-1, -2)) * scaling + bias
    out = torch.softmax(scores, dim=-1) @ v
    if silent is not None:
        out = out.masked_fill(silent.transpose(1, 2).unsqueeze(-1), 0.0)
    return _lin(P, a + "o_proj", out.transpose(1, 2).reshape(B, T, C))


def conv_module(P, c, cfg, x, silent):
    x = F.glu(F.linear(x, P[c + "pointwise_conv1.weight"].squeeze(-1), P.get(c + "pointwise_conv1.bias")), dim=-1)
    if silent is not None:
        x = x.masked_fill(silent, 0.0)
    x = F.pad(x, (0, 0, cfg.kernel - 1, 0))
    w = P[c + "depthwise_conv.weight"].permute(2, 1, 0)       # (K,1,C) -> (C,1,K)
    x = F.conv1d(x.transpose(1, 2), w, P.get(c + "depthwise_conv.bias"), groups=cfg.hidden).transpose(1, 2)
    x = F.silu(_ln(P, c + "norm", x, 1e-5))
    return F.linear(x, P[c + "pointwise_conv2.weight"].squeeze(-1), P.get(c + "pointwise_conv2.bias"))


def layer_forward(P, i: int, cfg, x, pos_emb, attn_mask, silent):
    p = f"layers.{i}."
    residual = x
    h = _ln(P, p + "norm_feed_forward1", x, cfg.eps)
    residual = residual + 0.5 * _ffn(P, p + "feed_forward1", h)
    h = _ln(P, p + "norm_self_att", residual, cfg.eps)
    residual = residual + attention(P, p + "self_attn.", cfg, h, pos_emb, attn_mask, silent)
    h = _ln(P, p + "norm_conv", residual, cfg.eps)
    residual = residual + conv_module(P, p + "conv.", cfg, h, silent)
    h = _ln(P, p + "norm_feed_forward2", residual, cfg.eps)
    residual = residual + 0.5 * _ffn(P, p + "feed_forward2", h)
    return _ln(P, p + "norm_out", residual, cfg.eps)


def layers_forward(P: Dict[str, torch.Tensor], cfg: FastConformerConfig, hidden: torch.Tensor, lengths: List[int]):
    """Layer stack of NemotronEncoder.forward on post-subsampling ``hidden (B, T, C)`` with valid ``lengths``:
    returns ``(B, T, C)`` (rows past a length are whatever the masked computation yields, as in the reference)."""
    B, T, C = hidden.shape
    keep = torch.arange(T).unsqueeze(0) < torch.tensor(lengths).unsqueeze(1)
    window = chunked_limited_mask(T, T, cfg.sliding_window - 1, cfg.lookahead).view(1, 1, T, T)
    attn_mask = window & keep.view(B, 1, 1, T)
    silent: Optional[torch.Tensor] = attn_mask.logical_not().all(dim=-1).transpose(1, 2)   # (B, T, 1)
    if not bool(silent.any()):
        silent = None
    pos_emb = relative_position_embedding(T, C)
    x = hidden.float()
    for i in range(cfg.layers):
        x = layer_forward(P, i, cfg, x, pos_emb, attn_mask, silent)
    return x


# ---------------------------------------------------------------------------
# 8x causal depthwise-separable subsampling (oasr/models/nemotron/subsampling.py:26-131, 204-224) and the whole
# encoder forward (oasr/models/nemotron/encoder.py:542-583)
# ---------------------------------------------------------------------------
@dataclass
class SubsamplingConfig:
    mels: int = 32
    channels: int = 64
    stages: int = 3          # log2(subsampling factor 8)

    def bins(self) -> int:
        b = self.mels
        for _ in range(self.stages):
            b = (b + 3 - 3) // 2 + 1
        return b


TINY_SUB = SubsamplingConfig()


def subsampling_param_spec(sub: SubsamplingConfig, hidden: int):
    Cs = sub.channels
    out = [("subsampling.conv_in.weight", (Cs, 3, 3, 1), "w"), ("subsampling.conv_in.bias", (Cs,), "b")]
    for i in range(sub.stages - 1):
        p = f"subsampling.layers.{i}."
        out += [(p + "depthwise_conv.weight", (Cs, 3, 3, 1), "w"), (p + "depthwise_conv.bias", (Cs,), "b"),
                (p + "pointwise_conv.weight", (Cs, 1, 1, Cs), "w"), (p + "pointwise_conv.bias", (Cs,), "b")]
    out += [("subsampling.linear.weight", (hidden, Cs * sub.bins()), "w"), ("subsampling.linear.bias", (hidden,), "b")]
    return out


def init_subsampling_params(sub: SubsamplingConfig, hidden: int, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    P = {}
    for name, shape, kind in subsampling_param_spec(sub, hidden):
        P[name] = torch.randn(shape, generator=g) * (0.25 if kind == "w" else 0.1)
    return P


def _mask_time(x, lengths):        # x NCHW (B, C, T, F)
    keep = torch.arange(x.size(2)).unsqueeze(0) < lengths.unsqueeze(1)
    return x * keep[:, None, :, None]


def subsampling_forward(P, sub: SubsamplingConfig, feats: torch.Tensor, lengths: torch.Tensor):
    """``feats (B, T, mels)`` -> ``(embeddings (B, T', hidden), lengths')``; pad (2, 1) on time and frequency before
    every 3x3 / stride-2 convolution, frames at or past the valid length re-zeroed after every stage."""
    pad = lambda x: F.pad(x, (2, 1, 2, 1))       # NCHW: last dim = frequency, then time
    out_len = lambda l: (l + 2 + 1 - 3) // 2 + 1
    x = feats.float().unsqueeze(1)               # (B, 1, T, F)
    w = P["subsampling.conv_in.weight"].permute(0, 3, 1, 2)
    x = torch.relu(F.conv2d(pad(x), w, P["subsampling.conv_in.bias"], stride=2))
    lengths = out_len(lengths)
    x = _mask_time(x, lengths)
    for i in range(sub.stages - 1):
        p = f"subsampling.layers.{i}."
        x = F.conv2d(pad(x), P[p + "depthwise_conv.weight"].permute(0, 3, 1, 2), P[p + "depthwise_conv.bias"], stride=2,
                     groups=sub.channels)
        pw = P[p + "pointwise_conv.weight"][:, 0, 0, :]                      # (C_out, C_in)
        x = torch.relu(torch.einsum("bctf,oc->botf", x, pw) + P[p + "pointwise_conv.bias"][None, :, None, None])
        lengths = out_len(lengths)
        x = _mask_time(x, lengths)
    b, c, t, f = x.shape
    flat = x.permute(0, 2, 3, 1).reshape(b, t, f * c)                        # NHWC flatten: (frequency, channel)
    return F.linear(flat, P["subsampling.linear.weight"], P["subsampling.linear.bias"]), lengths


class SubsamplingStreamState:
    """Per-stream state of the streaming front end: every stage's last ``kernel - 1 = 2`` input frames, before
    frequency padding (NemotronSubsampling.state_specs, oasr/models/nemotron/subsampling.py:130-154); zeros at stream
    start, which is what the offline pass pads on the left."""

    def __init__(self, sub: SubsamplingConfig):
        bins, chans = sub.mels, 1
        self.tails = []
        for _ in range(sub.stages):
            self.tails.append(torch.zeros(chans, 2, bins))               # NCHW without the batch axis
            bins = (bins + 3 - 3) // 2 + 1
            chans = sub.channels


def subsampling_forward_chunk(P, sub: SubsamplingConfig, state: SubsamplingStreamState, feats: torch.Tensor):
    """NemotronSubsampling.forward_chunk (oasr/models/nemotron/subsampling.py:156-189) for one stream:
    ``feats (T, mels)``, ``T`` a multiple of 8 -> ``(T / 8, hidden)``.  Each stage prepends its cached two frames
    instead of zero padding on the left, stores the last two frames of that concatenation, pads the frequency axis
    (2, 1) only, and has neither a right pad nor a length mask."""
    assert feats.shape[0] % (1 << sub.stages) == 0

    def stage_input(x, i):                        # x (C, T, F)
        cat = torch.cat([state.tails[i], x], dim=1)
        state.tails[i] = cat[:, -2:].clone()
        return F.pad(cat, (2, 1)).unsqueeze(0)    # frequency only

    x = feats.float().unsqueeze(0)                # (1, T, F)
    w = P["subsampling.conv_in.weight"].permute(0, 3, 1, 2)
    x = torch.relu(F.conv2d(stage_input(x, 0), w, P["subsampling.conv_in.bias"], stride=2))[0]
    for i in range(sub.stages - 1):
        p = f"subsampling.layers.{i}."
        x = F.conv2d(stage_input(x, i + 1), P[p + "depthwise_conv.weight"].permute(0, 3, 1, 2), P[p + "depthwise_conv.bias"],
                     stride=2, groups=sub.channels)
        pw = P[p + "pointwise_conv.weight"][:, 0, 0, :]
        x = torch.relu(torch.einsum("bctf,oc->botf", x, pw) + P[p + "pointwise_conv.bias"][None, :, None, None])[0]
    c, t, f = x.shape
    flat = x.permute(1, 2, 0).reshape(t, f * c)
    return F.linear(flat, P["subsampling.linear.weight"], P["subsampling.linear.bias"])


def encoder_forward(P, cfg: FastConformerConfig, sub: SubsamplingConfig, feats: torch.Tensor, lengths: List[int]):
    """NemotronEncoder.forward with scale_input False: ``(hidden (B, T', C), out_lengths)``."""
    hidden, out_len = subsampling_forward(P, sub, feats, torch.tensor(lengths))
    return layers_forward(P, cfg, hidden, out_len.tolist()), out_len


def ctc_head(P, hidden: torch.Tensor) -> torch.Tensor:
    """CtcProjection.forward (oasr/layers/ctc.py:48-51): ``log_softmax(hidden @ W^T + b)`` over the padded vocabulary;
    its torch spelling is torch_gemm_log_softmax (oasr/functionals/gemm_torch.py:64-75)."""
    return torch.log_softmax(F.linear(hidden, P["ctc.ctc_lo.weight"], P["ctc.ctc_lo.bias"]), dim=-1)


# ---------------------------------------------------------------------------
# Streaming: the layer stack chunk by chunk with cached keys / values and conv tails
# ---------------------------------------------------------------------------
class FastStreamState:
    """Per-stream state of the streaming layer stack, kept densely: per layer the keys / values of the frames still
    inside the trained left context ``(H, cached, D)`` and the conv module's post-GLU tail ``(kernel-1, C)``
    (zero at stream start: what the offline pass zero-pads), plus the number of encoder frames emitted so far."""

    def __init__(self, cfg: FastConformerConfig):
        H, D, C = cfg.heads, cfg.head_dim, cfg.hidden
        self.k = [torch.zeros(H, 0, D) for _ in range(cfg.layers)]
        self.v = [torch.zeros(H, 0, D) for _ in range(cfg.layers)]
        self.conv = [torch.zeros(cfg.kernel - 1, C) for _ in range(cfg.layers)]
        self.offset = 0


def layers_forward_chunk(P, cfg: FastConformerConfig, state: FastStreamState, x: torch.Tensor, keep_frames: int = -1):
    """One chunk ``x (T_q, C)`` of one stream through the layer stack: NemotronEncoderLayer.forward_chunk
    (oasr/models/nemotron/encoder.py:269-298) for every layer with the streaming attention of
    NemotronRelPositionAttention.forward_chunk (:362-410), the mask of NemotronEncoder._streaming_mask (:680-720) and the
    cached conv of NemotronConvolutionModule.forward_chunk (:191-208).

    The reference keeps a prefilled window of exactly ``sliding_window - 1`` cached frames whose not-yet-existing
    leading columns are masked (``k_abs >= 0``); here only real frames are cached, which gives the same visible keys at
    the same relative distances.  ``keep_frames`` (default: the trained left context) is how many of the newest cached
    frames survive into the next chunk; any value >= the left context gives the same result (older keys are masked)."""
    T_q, C = x.shape
    H, D = cfg.heads, cfg.head_dim
    left, chunk = cfg.sliding_window - 1, cfg.lookahead + 1
    left_chunks = left // chunk
    keep_frames = left if keep_frames < 0 else keep_frames
    assert T_q % chunk == 0 and state.offset % chunk == 0, "a streaming step is a whole number of trained attention chunks"
    cached = state.k[0].shape[1]
    key_len = cached + T_q
    q_abs = state.offset + torch.arange(T_q)
    k_abs = state.offset - cached + torch.arange(key_len)
    diff = q_abs.div(chunk, rounding_mode="trunc").unsqueeze(1) - k_abs.div(chunk, rounding_mode="trunc").unsqueeze(0)
    mask = (k_abs >= 0).unsqueeze(0) & (diff >= 0) & (diff <= left_chunks)          # (T_q, key_len)
    pos_emb = relative_position_embedding(key_len, C)                               # (2*key_len - 1, C)
    scaling = D ** -0.5
    x = x.float()
    for i in range(cfg.layers):
        p = f"layers.{i}."
        a, c = p + "self_attn.", p + "conv."
        residual = x
        h = _ln(P, p + "norm_feed_forward1", x, cfg.eps)
        residual = residual + 0.5 * _ffn(P, p + "feed_forward1", h)
        h = _ln(P, p + "norm_self_att", residual, cfg.eps)
        # --- attention over [cache ; chunk] ---
        split = lambda t: t.view(T_q, H, D).transpose(0, 1)                        # (H, T_q, D)
        q, k, v = split(_lin(P, a + "q_proj", h)), split(_lin(P, a + "k_proj", h)), split(_lin(P, a + "v_proj", h))
        state.k[i] = torch.cat([state.k[i], k], dim=1)
        state.v[i] = torch.cat([state.v[i], v], dim=1)
        rel_k = F.linear(pos_emb, P[a + "relative_k_proj.weight"]).view(-1, H, D)   # (2L-1, H, D)
        bd = (q + P[a + "bias_v"].unsqueeze(1)) @ rel_k.permute(1, 2, 0)            # (H, T_q, 2L-1)
        bd = rel_shift(bd.unsqueeze(0))[0][..., :key_len] * scaling
        bias = bd.masked_fill(mask.logical_not().unsqueeze(0), MASK_FLOOR)
        scores = ((q + P[a + "bias_u"].unsqueeze(1)) @ state.k[i].transpose(-1, -2)) * scaling + bias
        out = torch.softmax(scores, dim=-1) @ state.v[i]                            # (H, T_q, D)
        residual = residual + _lin(P, a + "o_proj", out.transpose(0, 1).reshape(T_q, C))
        state.k[i] = state.k[i][:, -keep_frames:] if keep_frames > 0 else state.k[i][:, :0]
        state.v[i] = state.v[i][:, -keep_frames:] if keep_frames > 0 else state.v[i][:, :0]
        # --- conv module with the cached post-GLU tail ---
        h = _ln(P, p + "norm_conv", residual, cfg.eps)
        g = F.glu(F.linear(h, P[c + "pointwise_conv1.weight"].squeeze(-1), P.get(c + "pointwise_conv1.bias")), dim=-1)
        padded = torch.cat([state.conv[i], g], dim=0)                               # (kernel-1 + T_q, C)
        state.conv[i] = padded[-(cfg.kernel - 1):].clone()
        w = P[c + "depthwise_conv.weight"].permute(2, 1, 0)                         # (K,1,C) -> (C,1,K)
        y = F.conv1d(padded.t().unsqueeze(0), w, P.get(c + "depthwise_conv.bias"), groups=C)[0].t()
        y = F.silu(_ln(P, c + "norm", y, 1e-5))
        residual = residual + F.linear(y, P[c + "pointwise_conv2.weight"].squeeze(-1), P.get(c + "pointwise_conv2.bias"))
        h = _ln(P, p + "norm_feed_forward2", residual, cfg.eps)
        residual = residual + 0.5 * _ffn(P, p + "feed_forward2", h)
        x = _ln(P, p + "norm_out", residual, cfg.eps)
    state.offset += T_q
    return x
