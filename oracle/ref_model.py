"""The reference's own Conformer model, built from the copy under ``oracle/_ref`` and loaded with the seeded
synthetic weights.  TEST INFRASTRUCTURE ONLY (used by ``bench.py --impl reference`` and the install test).

``build_conformer(cfg, params)`` constructs ``oasr.models.conformer.model.ConformerModel``
(oasr/models/conformer/model.py, config classes in oasr/models/conformer/config.py) for an
``oracle.conformer.ConformerConfig`` and copies every tensor of the flat parameter dict into it by its
state-dict name.  On the torch route two call sites of the reference have no torch spelling at the
operator boundary and are rebound to the spelling the reference itself documents as identical:
``oasr.glu`` -> ``F.glu`` (oasr/layers/conv.py:676-689) and ``oasr.gemm_log_softmax`` ->
``log_softmax(linear)`` (oasr/functionals/gemm_torch.py:64-75).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import make_ref


def load_torch_route():
    """The reference package on its torch backend (CPU / fp32 oracle runs)."""
    oasr = make_ref.load("torch")
    oasr.glu = lambda x, out=None: F.glu(x, dim=-1)
    oasr.gemm_log_softmax = lambda A, B, C=None, out=None: F.log_softmax(F.linear(A, B, C), dim=-1)
    return oasr


def build_conformer(cfg, params):
    """``ConformerModel`` of the reference in eval mode with ``params`` loaded (shapes checked)."""
    from oasr.models.conformer.config import ConformerEncoderConfig, ConformerModelConfig
    from oasr.models.conformer.model import ConformerModel

    enc = ConformerEncoderConfig(
        input_size=cfg.input_size, output_size=cfg.d_model, attention_heads=cfg.heads, linear_units=cfg.ffn,
        num_blocks=cfg.layers, cnn_module_kernel=cfg.kernel, cnn_module_norm=cfg.cnn_module_norm,
        embed_layer_norm=cfg.embed_layer_norm, causal=cfg.causal)
    model = ConformerModel(ConformerModelConfig(encoder=enc, vocab_size=cfg.vocab_padded)).eval()
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    with torch.no_grad():
        for name, value in params.items():
            if name not in own:
                raise KeyError(f"the reference model has no tensor {name}")
            if tuple(own[name].shape) != tuple(value.shape):
                raise ValueError(f"{name}: reference shape {tuple(own[name].shape)}, given {tuple(value.shape)}")
            own[name].data.copy_(value)
    return model
