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
