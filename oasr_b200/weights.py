"""Seeded synthetic weights for the Conformer encoder + CTC head.

No checkpoint of the reference's benchmark models is available offline, so
benchmarks and tests use random-init weights of the right architecture:
tensors with ndim >= 2 ~ N(0, 0.02); norm gains 1, biases 0, BatchNorm running
mean 0 / var 1 (the module defaults); padding rows of the CTC projection get
zero weight and bias -1e4 (the reference's init_pad_rows,
oasr/models/base.py:181-197).  Keys are the reference's state-dict names.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .encoder import PAD_LOGIT, ConformerConfig


def param_spec(cfg: ConformerConfig) -> List[Tuple[str, Tuple[int, ...], str]]:
    """Ordered (name, shape, kind), kind in {matrix, gain, bias, mean, var}."""
    d, F_, K, H, dk = cfg.d_model, cfg.ffn, cfg.kernel, cfg.heads, cfg.head_dim
    f1 = (cfg.input_size - 3) // 2 + 1
    f2 = (f1 - 3) // 2 + 1
    spec: List[Tuple[str, Tuple[int, ...], str]] = []

    def norm(prefix: str, kind: str):
        spec.append((prefix + ".weight", (d,), "gain"))
        spec.append((prefix + ".bias", (d,), "bias"))
        if kind == "batch_norm":
            spec.append((prefix + ".running_mean", (d,), "mean"))
            spec.append((prefix + ".running_var", (d,), "var"))

    def linear(prefix: str, n: int, k: int, bias: bool = True):
        spec.append((prefix + ".weight", (n, k), "matrix"))
        if bias:
            spec.append((prefix + ".bias", (n,), "bias"))

    e = "encoder.embed."
    spec.append((e + "convs.0.weight", (d, 3, 3, 1), "matrix"))
    spec.append((e + "convs.0.bias", (d,), "bias"))
    spec.append((e + "convs.1.weight", (d, 3, 3, d), "matrix"))
    spec.append((e + "convs.1.bias", (d,), "bias"))
    linear(e + "out.0", d, f2 * d)
    if cfg.embed_layer_norm:
        spec.append((e + "out.1.weight", (d,), "gain"))
        spec.append((e + "out.1.bias", (d,), "bias"))
    for i in range(cfg.layers):
        p = f"encoder.encoders.{i}."
        norm(p + "norm_ff_macaron", "layer_norm")
        linear(p + "feed_forward_macaron.w_1", F_, d)
        linear(p + "feed_forward_macaron.w_2", d, F_)
        norm(p + "norm_mha", "layer_norm")
        linear(p + "self_attn.linear_qkv", 3 * d, d)
        linear(p + "self_attn.linear_pos", d, d, bias=False)
        spec.append((p + "self_attn.pos_bias_u", (H, dk), "matrix"))
        spec.append((p + "self_attn.pos_bias_v", (H, dk), "matrix"))
        linear(p + "self_attn.linear_out", d, d)
        norm(p + "norm_conv", cfg.cnn_module_norm)
        spec.append((p + "conv_module.pointwise_conv1.weight", (2 * d, d, 1), "matrix"))
        spec.append((p + "conv_module.pointwise_conv1.bias", (2 * d,), "bias"))
        spec.append((p + "conv_module.depthwise_conv.weight", (K, 1, d), "matrix"))
        spec.append((p + "conv_module.depthwise_conv.bias", (d,), "bias"))
        norm(p + "conv_module.norm_activation", cfg.cnn_module_norm)
        spec.append((p + "conv_module.pointwise_conv2.weight", (d, d, 1), "matrix"))
        spec.append((p + "conv_module.pointwise_conv2.bias", (d,), "bias"))
        norm(p + "norm_ff", "layer_norm")
        linear(p + "feed_forward.w_1", F_, d)
        linear(p + "feed_forward.w_2", d, F_)
        norm(p + "norm_final", "layer_norm")
    norm("encoder.after_norm", "layer_norm")
    linear("ctc.ctc_lo", cfg.vocab_padded, d)
    return spec


def init_params(cfg: ConformerConfig, seed: int = 1234) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape, kind in param_spec(cfg):
        if kind == "matrix":
            out[name] = torch.randn(shape, generator=g) * 0.02
        elif kind in ("gain", "var"):
            out[name] = torch.ones(shape)
        else:
            out[name] = torch.zeros(shape)
    out["ctc.ctc_lo.weight"][cfg.vocab:] = 0.0
    out["ctc.ctc_lo.bias"][cfg.vocab:] = PAD_LOGIT
    return out


def fastconformer_param_spec(hidden: int, heads: int, ffn: int, layers: int, kernel: int, bias: bool
                             ) -> List[Tuple[str, Tuple[int, ...], str]]:
    """Ordered (name, shape, kind) of the FastConformer / Nemotron layer stack in the reference's state-dict
    naming (oasr/models/nemotron/encoder.py:150-359); kind 'w' matrix, 'g' norm gain, 'b' bias."""
    C, D = hidden, hidden // heads
    spec: List[Tuple[str, Tuple[int, ...], str]] = []
    for i in range(layers):
        p = f"layers.{i}."
        for ff in ("feed_forward1", "feed_forward2"):
            spec += [(p + ff + ".linear1.weight", (ffn, C), "w"), (p + ff + ".linear2.weight", (C, ffn), "w")]
            if bias:
                spec += [(p + ff + ".linear1.bias", (ffn,), "b"), (p + ff + ".linear2.bias", (C,), "b")]
        a = p + "self_attn."
        spec += [(a + "bias_u", (heads, D), "w"), (a + "bias_v", (heads, D), "w")]
        for n in ("q_proj", "k_proj", "v_proj", "o_proj"):
            spec.append((a + n + ".weight", (C, C), "w"))
            if bias:
                spec.append((a + n + ".bias", (C,), "b"))
        spec.append((a + "relative_k_proj.weight", (C, C), "w"))
        c = p + "conv."
        spec += [(c + "pointwise_conv1.weight", (2 * C, C, 1), "w"), (c + "depthwise_conv.weight", (kernel, 1, C), "w"),
                 (c + "norm.weight", (C,), "g"), (c + "norm.bias", (C,), "b"), (c + "pointwise_conv2.weight", (C, C, 1), "w")]
        if bias:
            spec += [(c + "pointwise_conv1.bias", (2 * C,), "b"), (c + "depthwise_conv.bias", (C,), "b"),
                     (c + "pointwise_conv2.bias", (C,), "b")]
        for n in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
            spec += [(p + n + ".weight", (C,), "g"), (p + n + ".bias", (C,), "b")]
    return spec


def subsampled_bins(mels: int, stages: int = 3) -> int:
    """Frequency bins left after ``stages`` 3x3 / stride-2 convolutions padded (2, 1)
    (oasr/models/nemotron/subsampling.py:26-131)."""
    for _ in range(stages):
        mels = mels // 2 + 1
    return mels


def init_fastconformer_params(hidden: int, heads: int, ffn: int, layers: int, kernel: int, mels: int, channels: int,
                              seed: int = 1234, w_std: float = 0.02, bias: bool = False, stages: int = 3,
                              vocab: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded synthetic FastConformer encoder weights (layer stack from ``seed``, 8x subsampling front end from
    ``seed + 1``, optional CTC projection of ``vocab`` rows from ``seed + 2``): matrices ~ N(0, w_std), norm gains
    1 + N(0, 0.1), biases N(0, 0.1); front-end matrices ~ N(0, 0.25) so that activations keep unit scale through
    the three ReLU stages."""
    g = torch.Generator().manual_seed(seed)
    P: Dict[str, torch.Tensor] = {}
    for name, shape, kind in fastconformer_param_spec(hidden, heads, ffn, layers, kernel, bias):
        if kind == "w":
            P[name] = torch.randn(shape, generator=g) * w_std
        elif kind == "g":
            P[name] = 1.0 + torch.randn(shape, generator=g) * 0.1
        else:
            P[name] = torch.randn(shape, generator=g) * 0.1
    g = torch.Generator().manual_seed(seed + 1)
    s = "subsampling."
    front = [(s + "conv_in.weight", (channels, 3, 3, 1), "w"), (s + "conv_in.bias", (channels,), "b")]
    for i in range(stages - 1):
        p = f"{s}layers.{i}."
        front += [(p + "depthwise_conv.weight", (channels, 3, 3, 1), "w"), (p + "depthwise_conv.bias", (channels,), "b"),
                  (p + "pointwise_conv.weight", (channels, 1, 1, channels), "w"), (p + "pointwise_conv.bias", (channels,), "b")]
    front += [(s + "linear.weight", (hidden, channels * subsampled_bins(mels, stages)), "w"), (s + "linear.bias", (hidden,), "b")]
    for name, shape, kind in front:
        P[name] = torch.randn(shape, generator=g) * (0.25 if kind == "w" else 0.1)
    if vocab:
        g = torch.Generator().manual_seed(seed + 2)
        vp = (vocab + 7) // 8 * 8
        P["ctc.ctc_lo.weight"] = torch.randn(vp, hidden, generator=g) * w_std
        P["ctc.ctc_lo.bias"] = torch.zeros(vp)
        P["ctc.ctc_lo.weight"][vocab:] = 0.0
        P["ctc.ctc_lo.bias"][vocab:] = PAD_LOGIT
    return P
