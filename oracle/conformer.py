"""Model-level CPU oracle: WeNet-style Conformer encoder + CTC head in fp32 torch.
TEST INFRASTRUCTURE ONLY.

A restatement of the reference's fp32 torch path (``OASR_LAYERS_BACKEND=torch``)
for the three entry points the engine calls:

* ``forward_offline``         padded batch      (oasr/models/base.py:749-754,
                                                 oasr/models/conformer/model.py:813-828)
* ``forward_offline_packed``  sequence packing  (base.py:756-761, model.py:830-868)
* ``forward_chunk_paged``     streaming chunk   (model.py:913-1023)

Parameters are a flat ``dict`` keyed by the reference's own state-dict names
(``encoder.encoders.3.self_attn.linear_qkv.weight`` ...), produced from a seed
by :func:`init_params`.  ``tests/golden/make_golden.py`` loads the same dict
into the reference model, runs the reference, checks this file against it and
writes the committed fixtures; the oracle is pinned by those fixtures.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

PAD_LOGIT = -1e4  # oasr/models/base.py:167


@dataclass(frozen=True)
class ConformerConfig:
    input_size: int = 80
    d_model: int = 256
    heads: int = 4
    ffn: int = 2048
    layers: int = 12
    kernel: int = 15
    vocab: int = 5002            # raw vocabulary; the head is padded to a multiple of 8
    cnn_module_norm: str = "batch_norm"   # also the type of norm_conv (model.py:575-581)
    embed_layer_norm: bool = True         # oasr/models/conformer/config.py:56
    eps: float = 1e-5
    causal: bool = False                  # causal depthwise conv (lorder = kernel - 1), used for streaming

    @property
    def vocab_padded(self) -> int:       # align_out_features, oasr/models/base.py:170-178
        return (self.vocab + 7) // 8 * 8

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


CONFIG1 = ConformerConfig()                                             # CPU-runnable reference case
CONFIG2 = ConformerConfig(d_model=512, heads=8)                         # offline bf16 headline case
TINY = ConformerConfig(d_model=128, heads=2, ffn=256, layers=2, vocab=90)
TINY_STREAM = ConformerConfig(d_model=128, heads=2, ffn=256, layers=2, vocab=90, causal=True)
CONFIG3 = ConformerConfig(d_model=512, heads=8, causal=True)           # streaming chunked case


# ---------------------------------------------------------------------------
# Parameters
# ---------------------------------------------------------------------------
def param_spec(cfg: ConformerConfig) -> List[Tuple[str, Tuple[int, ...], str]]:
    """Ordered (name, shape, kind); kind in {matrix, gain, bias, mean, var}."""
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
    spec.append((e + "convs.0.weight", (d, 3, 3, 1), "matrix"))      # KRSC (NHWC conv), layers/conv.py:524-537
    spec.append((e + "convs.0.bias", (d,), "bias"))
    spec.append((e + "convs.1.weight", (d, 3, 3, d), "matrix"))
    spec.append((e + "convs.1.bias", (d,), "bias"))
    linear(e + "out.0", d, f2 * d)                                   # input flattened (f, c), model.py:446-449
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


def init_params(cfg: ConformerConfig, seed: int = 1234, perturb: float = 0.0) -> Dict[str, torch.Tensor]:
    """Seeded synthetic weights: tensors with ndim >= 2 ~ N(0, 0.02); norm gains
    1, biases 0, BatchNorm running mean 0 / var 1 (module defaults); padding rows
    of the CTC projection zero weight / bias -1e4 (init_pad_rows,
    oasr/models/base.py:181-197).  ``perturb`` > 0 additionally draws biases,
    gains and BatchNorm statistics away from their defaults (std ``perturb``) so
    that every bias / affine path is exercised."""
    g = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for name, shape, kind in param_spec(cfg):
        if kind == "matrix":
            t = torch.randn(shape, generator=g) * 0.02
        elif kind == "gain":
            t = torch.ones(shape)
            if perturb:
                t = t + torch.randn(shape, generator=g) * perturb
        elif kind in ("bias", "mean"):
            t = torch.zeros(shape)
            if perturb:
                t = torch.randn(shape, generator=g) * perturb
        else:  # var
            t = torch.ones(shape)
            if perturb:
                t = t + torch.rand(shape, generator=g) * perturb
        out[name] = t
    w, b = out["ctc.ctc_lo.weight"], out["ctc.ctc_lo.bias"]
    w[cfg.vocab:] = 0.0
    b[cfg.vocab:] = PAD_LOGIT
    return out


# ---------------------------------------------------------------------------
# Building blocks
# ---------------------------------------------------------------------------
def positional_table(max_len: int, d: int) -> torch.Tensor:
    """RelPositionalEncoding.pe, oasr/models/conformer/model.py:254-266."""
    pe = torch.zeros(max_len, d)
    position = torch.arange(0, max_len, dtype=torch.float32).unsqueeze(1)
    div_term = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * -(math.log(10000.0) / d))
    pe[:, 0::2] = torch.sin(position * div_term)
    pe[:, 1::2] = torch.cos(position * div_term)
    return pe


def subsampled_lengths(lengths: torch.Tensor) -> torch.Tensor:
    """Number of valid frames after the 4x Conv2d subsampling: the mask is sliced
    [2::2] twice (model.py:450-452), i.e. output frame t is valid iff 6 + 4t < L."""
    return torch.clamp((lengths - 3) // 4, min=0)


def subsampled_time(T: int) -> int:
    t1 = (T - 3) // 2 + 1
    return (t1 - 3) // 2 + 1


def _norm(P, prefix: str, x: torch.Tensor, kind: str, eps: float) -> torch.Tensor:
    if kind == "layer_norm":
        return F.layer_norm(x, (x.shape[-1],), P[prefix + ".weight"], P[prefix + ".bias"], eps)
    # inference BatchNorm over channels-last rows (oasr/layers/norm.py:64-74)
    return (x - P[prefix + ".running_mean"]) * torch.rsqrt(P[prefix + ".running_var"] + eps) * P[prefix + ".weight"] \
        + P[prefix + ".bias"]


def embed(P, cfg: ConformerConfig, feats: torch.Tensor, offset: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Conv2dSubsampling4 (model.py:300-453): two 3x3 stride-2 NHWC convs with ReLU,
    (f, c)-major flatten, Linear (+LayerNorm), times sqrt(d).  Returns (x (B,Tp,d),
    pos_emb (Tp,d) for positions offset..offset+Tp)."""
    x = feats.float().unsqueeze(1)                                   # (B,1,T,F)  NCHW
    for i in range(2):
        w = P[f"encoder.embed.convs.{i}.weight"].permute(0, 3, 1, 2)  # KRSC -> KCRS
        x = F.relu(F.conv2d(x, w, P[f"encoder.embed.convs.{i}.bias"], stride=2))
    b, c, t, f = x.shape
    x = x.permute(0, 2, 3, 1).reshape(b, t, f * c)                   # NHWC-natural (f, c) flatten
    x = F.linear(x, P["encoder.embed.out.0.weight"], P["encoder.embed.out.0.bias"])
    if cfg.embed_layer_norm:
        x = F.layer_norm(x, (cfg.d_model,), P["encoder.embed.out.1.weight"], P["encoder.embed.out.1.bias"], 1e-5)
    x = x * math.sqrt(cfg.d_model)                                   # model.py:271
    pe = positional_table(5000, cfg.d_model)
    return x, pe[offset:offset + t]


def _ffn(P, prefix: str, x: torch.Tensor) -> torch.Tensor:
    """PositionwiseFeedForward (model.py:70-93): Linear -> swish -> Linear."""
    h = F.silu(F.linear(x, P[prefix + ".w_1.weight"], P[prefix + ".w_1.bias"]))
    return F.linear(h, P[prefix + ".w_2.weight"], P[prefix + ".w_2.bias"])


def _rel_attention(P, cfg, prefix: str, x: torch.Tensor, pos_emb: torch.Tensor,
                   key_bias: Optional[torch.Tensor]) -> torch.Tensor:
    """RelPositionMultiHeadedAttention._forward_offline (oasr/layers/attention/attention.py:282-321).
    x (B,T,d); pos_emb (T,d); key_bias (B,1,1,T) additive (-1e10 on padded keys, added BEFORE
    scaling, model.py:46-52) or None.  No rel-shift: matrix_bd[i,j] = (q_i + v) . p_j."""
    B, T, d = x.shape
    H, dk = cfg.heads, cfg.head_dim
    qkv = F.linear(x, P[prefix + ".linear_qkv.weight"], P[prefix + ".linear_qkv.bias"])
    q, k, v = qkv.split(d, dim=-1)
    q = q.view(B, T, H, dk).transpose(1, 2)
    k = k.view(B, T, H, dk).transpose(1, 2)
    v = v.view(B, T, H, dk).transpose(1, 2)
    p = F.linear(pos_emb, P[prefix + ".linear_pos.weight"]).view(T, H, dk).permute(1, 2, 0)   # (H,dk,T)
    q_u = q + P[prefix + ".pos_bias_u"].unsqueeze(1)
    q_v = q + P[prefix + ".pos_bias_v"].unsqueeze(1)
    scale = 1.0 / math.sqrt(dk)
    matrix_bd = torch.matmul(q_v, p)                                  # (B,H,T,T)
    bias = (matrix_bd + key_bias) * scale if key_bias is not None else matrix_bd * scale
    s = torch.matmul(q_u, k.transpose(-1, -2)) * scale + bias
    out = torch.matmul(torch.softmax(s, dim=-1), v)                   # (B,H,T,dk)
    out = out.transpose(1, 2).reshape(B, T, d)
    return F.linear(out, P[prefix + ".linear_out.weight"], P[prefix + ".linear_out.bias"])


def _conv_module(P, cfg, prefix: str, x: torch.Tensor, mask: Optional[torch.Tensor]) -> torch.Tensor:
    """ConvolutionModule.forward, non-causal (model.py:168-198).  mask (B,T,1) bool or None:
    padded rows are zeroed BEFORE pointwise_conv1 and AFTER pointwise_conv2 only."""
    d, K = cfg.d_model, cfg.kernel
    if mask is not None:
        x = x.masked_fill(~mask, 0.0)
    x = F.linear(x, P[prefix + ".pointwise_conv1.weight"].squeeze(-1), P[prefix + ".pointwise_conv1.bias"])
    x = F.glu(x, dim=-1)
    w = P[prefix + ".depthwise_conv.weight"].reshape(K, d).t().unsqueeze(1)     # (d,1,K)
    x = F.conv1d(x.transpose(1, 2), w, P[prefix + ".depthwise_conv.bias"], padding=(K - 1) // 2, groups=d)
    x = x.transpose(1, 2)
    x = F.silu(_norm(P, prefix + ".norm_activation", x, cfg.cnn_module_norm, cfg.eps))
    x = F.linear(x, P[prefix + ".pointwise_conv2.weight"].squeeze(-1), P[prefix + ".pointwise_conv2.bias"])
    if mask is not None:
        x = x.masked_fill(~mask, 0.0)
    return x


def encoder_layer(P, cfg, i: int, x, pos_emb, key_bias, mask) -> torch.Tensor:
    """ConformerEncoderLayer.forward, pre-norm macaron + conv (model.py:665-707)."""
    p = f"encoder.encoders.{i}"
    x = x + 0.5 * _ffn(P, p + ".feed_forward_macaron", _norm(P, p + ".norm_ff_macaron", x, "layer_norm", cfg.eps))
    x = x + _rel_attention(P, cfg, p + ".self_attn", _norm(P, p + ".norm_mha", x, "layer_norm", cfg.eps), pos_emb,
                           key_bias)
    x = x + _conv_module(P, cfg, p + ".conv_module", _norm(P, p + ".norm_conv", x, cfg.cnn_module_norm, cfg.eps),
                         mask)
    x = x + 0.5 * _ffn(P, p + ".feed_forward", _norm(P, p + ".norm_ff", x, "layer_norm", cfg.eps))
    return _norm(P, p + ".norm_final", x, "layer_norm", cfg.eps)


def ctc_head(P, hidden: torch.Tensor) -> torch.Tensor:
    """CtcProjection (oasr/layers/ctc.py:48-51) = log_softmax(linear) (functionals/gemm_torch.py:64-75)."""
    return F.log_softmax(F.linear(hidden, P["ctc.ctc_lo.weight"], P["ctc.ctc_lo.bias"]), dim=-1)


# ---------------------------------------------------------------------------
# Entry points
# ---------------------------------------------------------------------------
def encode_offline(P, cfg: ConformerConfig, feats: torch.Tensor, lengths: torch.Tensor):
    """ConformerEncoder.forward (model.py:813-828) on a padded batch."""
    x, pos_emb = embed(P, cfg, feats)
    Tp = x.shape[1]
    out_len = subsampled_lengths(lengths)
    valid = torch.arange(Tp).unsqueeze(0) < out_len.unsqueeze(1)          # (B,Tp)
    key_bias = ((~valid).float() * -1.0e10).view(x.shape[0], 1, 1, Tp)    # mask_to_bias, model.py:46-52
    mask = valid.unsqueeze(-1)
    for i in range(cfg.layers):
        x = encoder_layer(P, cfg, i, x, pos_emb, key_bias, mask)
    x = _norm(P, "encoder.after_norm", x, "layer_norm", cfg.eps)
    return x, out_len


def forward_offline(P, cfg, feats, lengths):
    """(log_probs (B,Tp,Vpad), out_lengths (B,)), oasr/models/base.py:749-754."""
    hidden, out_len = encode_offline(P, cfg, feats, lengths)
    return ctc_head(P, hidden), out_len


def encode_offline_packed(P, cfg: ConformerConfig, feats: torch.Tensor, lengths: torch.Tensor):
    """ConformerEncoder.forward_packed (model.py:830-868).  The reference packs the
    valid frames of every utterance into one row, restricts attention to each
    cu_seqlens segment and isolates the depthwise conv with zero gap frames, which
    it documents as bit-exact to B=1 inference; restated here as exactly that:
    every utterance's valid frames run alone, with no mask.  The embed runs on the
    padded batch (model.py:852) -- valid output frames never see padding because
    frame t reads input frames 4t..4t+6 < L."""
    x, pos_emb_full = embed(P, cfg, feats)
    B, Tp, d = x.shape
    out_len = subsampled_lengths(lengths)
    hidden = torch.zeros(B, Tp, d)
    for b in range(B):
        n = int(out_len[b])
        if n == 0:
            continue
        xb = x[b:b + 1, :n]
        for i in range(cfg.layers):
            xb = encoder_layer(P, cfg, i, xb, pos_emb_full[:n], None, None)
        hidden[b, :n] = _norm(P, "encoder.after_norm", xb, "layer_norm", cfg.eps)[0]
    return hidden, out_len                                              # padding rows are zeros (packing.py:228-232)


def forward_offline_packed(P, cfg, feats, lengths):
    """(log_probs, out_lengths), oasr/models/base.py:756-761."""
    hidden, out_len = encode_offline_packed(P, cfg, feats, lengths)
    return ctc_head(P, hidden), out_len


def greedy_tokens(log_probs: torch.Tensor, out_len: torch.Tensor, vocab: int, blank: int = 0) -> List[List[int]]:
    """Greedy CTC search over valid frames and the raw vocabulary columns
    (csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55)."""
    res = []
    for b in range(log_probs.shape[0]):
        ids = log_probs[b, :int(out_len[b]), :vocab].argmax(-1).tolist()
        hyp, prev = [], None
        for i in ids:
            if i != prev and i != blank:
                hyp.append(i)
            prev = i
        res.append(hyp)
    return res


# ---------------------------------------------------------------------------
# Streaming: chunk-by-chunk forward with cached keys/values and conv left context
# ---------------------------------------------------------------------------
class StreamState:
    """Per-stream state of ConformerEncoder.forward_chunk_paged (model.py:913-1023) kept densely:
    per layer the cached keys / values (H, T_cached, dk) and the conv module's left context
    (kernel-1 frames of its input), plus the number of encoder frames emitted so far."""

    def __init__(self, cfg: ConformerConfig):
        H, dk, d = cfg.heads, cfg.head_dim, cfg.d_model
        self.k = [torch.zeros(H, 0, dk) for _ in range(cfg.layers)]
        self.v = [torch.zeros(H, 0, dk) for _ in range(cfg.layers)]
        self.cnn = [torch.zeros(cfg.kernel - 1, d) for _ in range(cfg.layers)]   # zero-initialised slot buffer
        self.offset = 0


def forward_chunk(P, cfg: ConformerConfig, state: StreamState, xs: torch.Tensor, max_past_frames: int,
                  block: int = 16) -> torch.Tensor:
    """One streaming chunk of one stream: xs (T_in, F) feature window -> log-probs (chunk, Vpad).

    Restates forward_chunk_paged with att/cnn caches (model.py:913-1023), the paged attention of
    RelPositionMultiHeadedAttention._forward_paged (oasr/layers/attention/attention.py:229-280) and the
    cached causal ConvolutionModule.forward (model.py:168-198).  The cache manager keeps whole blocks
    of ``block`` frames and drops the oldest ones so that at most ``max_past_frames`` cached frames are
    visible when a chunk starts (oasr/cache/attention_cache.py:387-398,427-465); key j of the cache has
    absolute position offset - cached + j (model.py:993-1001)."""
    assert cfg.causal
    d, H, dk, K = cfg.d_model, cfg.heads, cfg.head_dim, cfg.kernel
    x, _ = embed(P, cfg, xs.unsqueeze(0))                 # (1, chunk, d); positions are handled below
    x = x[0]
    chunk = x.shape[0]
    while state.k[0].shape[1] > max_past_frames:          # evict whole blocks, oldest first
        for i in range(cfg.layers):
            state.k[i] = state.k[i][:, block:]
            state.v[i] = state.v[i][:, block:]
    cached = state.k[0].shape[1]
    pe = positional_table(5000, d)
    pos_start = state.offset - cached
    pos_emb = pe[pos_start:pos_start + cached + chunk]    # (cached + chunk, d)
    scale = 1.0 / math.sqrt(dk)
    for i in range(cfg.layers):
        p = f"encoder.encoders.{i}"
        x = x + 0.5 * _ffn(P, p + ".feed_forward_macaron", _norm(P, p + ".norm_ff_macaron", x, "layer_norm", cfg.eps))
        # --- attention over [cache ; chunk] ---
        h = _norm(P, p + ".norm_mha", x, "layer_norm", cfg.eps)
        a = p + ".self_attn"
        qkv = F.linear(h, P[a + ".linear_qkv.weight"], P[a + ".linear_qkv.bias"])
        q, k, v = (t.view(chunk, H, dk).transpose(0, 1) for t in qkv.split(d, dim=-1))     # (H, chunk, dk)
        state.k[i] = torch.cat([state.k[i], k], dim=1)
        state.v[i] = torch.cat([state.v[i], v], dim=1)
        pp = F.linear(pos_emb, P[a + ".linear_pos.weight"]).view(-1, H, dk).permute(1, 2, 0)  # (H, dk, T_kv)
        q_u = q + P[a + ".pos_bias_u"].unsqueeze(1)
        q_v = q + P[a + ".pos_bias_v"].unsqueeze(1)
        s = torch.matmul(q_u, state.k[i].transpose(-1, -2)) * scale + torch.matmul(q_v, pp) * scale
        o = torch.matmul(torch.softmax(s, dim=-1), state.v[i])                                # (H, chunk, dk)
        o = o.transpose(0, 1).reshape(chunk, d)
        x = x + F.linear(o, P[a + ".linear_out.weight"], P[a + ".linear_out.bias"])
        # --- conv module with left context (causal, lorder = K-1) ---
        c = p + ".conv_module"
        h = _norm(P, p + ".norm_conv", x, cfg.cnn_module_norm, cfg.eps)
        cat = torch.cat([state.cnn[i], h], dim=0)                      # (K-1 + chunk, d)
        state.cnn[i] = cat[-(K - 1):].clone()
        y = F.linear(cat, P[c + ".pointwise_conv1.weight"].squeeze(-1), P[c + ".pointwise_conv1.bias"])
        y = F.glu(y, dim=-1)
        w = P[c + ".depthwise_conv.weight"].reshape(K, d).t().unsqueeze(1)
        y = F.conv1d(y.t().unsqueeze(0), w, P[c + ".depthwise_conv.bias"], groups=d)[0].t()   # (chunk, d)
        y = F.silu(_norm(P, c + ".norm_activation", y, cfg.cnn_module_norm, cfg.eps))
        y = F.linear(y, P[c + ".pointwise_conv2.weight"].squeeze(-1), P[c + ".pointwise_conv2.bias"])
        x = x + y
        x = x + 0.5 * _ffn(P, p + ".feed_forward", _norm(P, p + ".norm_ff", x, "layer_norm", cfg.eps))
        x = _norm(P, p + ".norm_final", x, "layer_norm", cfg.eps)
    x = _norm(P, "encoder.after_norm", x, "layer_norm", cfg.eps)
    state.offset += chunk
    return ctc_head(P, x)
