"""Conformer encoder + CTC head on B200, with the reference's entry points.

``ConformerCTC`` mirrors the reference model's engine-facing calls
(oasr/models/base.py:749-761): ``forward_offline(features, lengths)`` and
``forward_offline_packed(features, lengths)`` return ``(log_probs, out_lengths)``.
Parameters are a flat dict keyed by the reference's state-dict names.

Both offline entry points run the same sequence-packed pipeline over the valid
frames only (the padded entry point reproduces, through ``right_fill`` of the
depthwise conv, what padded rows contribute in the reference's padded path):

    embed (Conv2d subsampling, torch/cuDNN for now) -> gather valid rows -> embed Linear
    per layer, 13 launches, fp32 residual stream, 16-bit activations:
      add_norm_f32 .. gemm(swish) .. gemm .. add_norm_f32 .. gemm(qkv4) .. fmha_varlen_relpos ..
      gemm .. add_norm_f32 .. gemm_glu .. depthwise_conv1d_packed(BN+swish) .. gemm ..
      add_norm_f32 .. gemm(swish) .. gemm .. add_norm_f32(norm_final + next pre-norm)
    gemm_log_softmax (fused CTC head, fp32 log-probs + per-frame argmax)

There is no CPU path and no torch fallback for the layer stack.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import functional as OF
from . import fused
from .cache import gather_rows

PAD_LOGIT = -1e4


@dataclass(frozen=True)
class ConformerConfig:
    """Hyper-parameters (names follow oasr/models/conformer/config.py)."""

    input_size: int = 80
    d_model: int = 256
    heads: int = 4
    ffn: int = 2048
    layers: int = 12
    kernel: int = 15
    vocab: int = 5002
    cnn_module_norm: str = "batch_norm"
    embed_layer_norm: bool = True
    eps: float = 1e-5

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + 7) // 8 * 8

    @property
    def head_dim(self) -> int:
        return self.d_model // self.heads


def subsampled_lengths(lengths: torch.Tensor) -> torch.Tensor:
    """Valid frames after the 4x subsampling: frame t is valid iff 6 + 4t < L
    (the mask slicing of oasr/models/conformer/model.py:450-452)."""
    return torch.clamp((lengths - 3) // 4, min=0)


@dataclass
class PackedBatch:
    """Host-side description of one packed batch (oasr/models/conformer/packing.py:32-97)."""

    num_segs: int
    total: int
    max_seg: int
    padded_t: int
    seg_lengths: List[int]
    cu_seqlens: torch.Tensor      # (S+1,) int32, device
    pack_src_idx: torch.Tensor    # (total,) int64, device: b * Tp + t
    fill_frames: torch.Tensor     # (S,) int32, device: padded frames right of each segment, capped at (K-1)/2


def build_packed_batch(out_lengths: List[int], padded_t: int, conv_kernel: int, device) -> PackedBatch:
    """Index tensors from HOST lengths: no device synchronisation (the reference pulls
    ``seg_lengths.tolist()`` from the device, packing.py:143)."""
    cu = [0]
    for n in out_lengths:
        cu.append(cu[-1] + n)
    total = cu[-1]
    half = (conv_kernel - 1) // 2
    idx = torch.cat([torch.arange(n, dtype=torch.int64) + b * padded_t for b, n in enumerate(out_lengths)]) \
        if total else torch.zeros(0, dtype=torch.int64)
    fill = torch.tensor([min(half, padded_t - n) for n in out_lengths], dtype=torch.int32)
    return PackedBatch(
        num_segs=len(out_lengths), total=total, max_seg=max(out_lengths) if out_lengths else 0, padded_t=padded_t,
        seg_lengths=list(out_lengths),
        cu_seqlens=torch.tensor(cu, dtype=torch.int32).to(device, non_blocking=True),
        pack_src_idx=idx.to(device, non_blocking=True),
        fill_frames=fill.to(device, non_blocking=True),
    )


class ConformerCTC:
    """WeNet-style Conformer encoder + CTC head running on the sm_100a kernels."""

    def __init__(self, cfg: ConformerConfig, params: Dict[str, torch.Tensor], device="cuda",
                 dtype: torch.dtype = torch.bfloat16):
        if cfg.head_dim != 64:
            raise ValueError("the fused relative-position attention kernel needs head_dim 64")
        if cfg.d_model % 8 or cfg.ffn % 8:
            raise ValueError("d_model and ffn must be multiples of 8")
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self._prepare({k: v.detach().to(torch.float32) for k, v in params.items()})

    # ------------------------------------------------------------------ weights
    def _prepare(self, P: Dict[str, torch.Tensor]) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        d, H, dk, L = cfg.d_model, cfg.heads, cfg.head_dim, cfg.layers

        def w(t):  # 16-bit device copy
            return t.to(dt).to(dev).contiguous()

        def f(t):  # fp32 device copy
            return t.to(torch.float32).to(dev).contiguous()

        e = "encoder.embed."
        # Conv2d weights are stored KRSC (NHWC); torch wants KCRS.  channels_last keeps NHWC in memory.
        self.conv1_w = f(P[e + "convs.0.weight"].reshape(d, 3, 3))   # (C, 3, 3, 1) -> (C, 3, 3), fp32
        self.conv1_b = f(P[e + "convs.0.bias"])
        self.conv2_w = w(P[e + "convs.1.weight"].permute(0, 3, 1, 2)).contiguous(memory_format=torch.channels_last)
        self.conv2_b = w(P[e + "convs.1.bias"])
        xscale = math.sqrt(d)
        if cfg.embed_layer_norm:
            self.embed_w, self.embed_b = w(P[e + "out.0.weight"]), w(P[e + "out.0.bias"])
            # x * sqrt(d) folded into the embed LayerNorm's affine (model.py:271)
            self.embed_ln_w, self.embed_ln_b = w(P[e + "out.1.weight"] * xscale), w(P[e + "out.1.bias"] * xscale)
        else:
            self.embed_w, self.embed_b = w(P[e + "out.0.weight"] * xscale), w(P[e + "out.0.bias"] * xscale)
            self.embed_ln_w = self.embed_ln_b = None

        self.layers: List[dict] = []
        pos_w = []
        for i in range(L):
            p = f"encoder.encoders.{i}."
            a = p + "self_attn."
            wq, wk, wv = P[a + "linear_qkv.weight"].split(d, dim=0)
            bq, bk, bv = P[a + "linear_qkv.bias"].split(d, dim=0)
            u, v = P[a + "pos_bias_u"].reshape(-1), P[a + "pos_bias_v"].reshape(-1)
            lw = {}
            for nm in ("norm_ff_macaron", "norm_mha", "norm_ff", "norm_final"):
                lw[nm] = (w(P[p + nm + ".weight"]), w(P[p + nm + ".bias"]))
            lw["ffm"] = tuple(w(P[p + "feed_forward_macaron." + s]) for s in ("w_1.weight", "w_1.bias", "w_2.weight", "w_2.bias"))
            lw["ff"] = tuple(w(P[p + "feed_forward." + s]) for s in ("w_1.weight", "w_1.bias", "w_2.weight", "w_2.bias"))
            # fused projection with the query block duplicated and pos_bias_u / pos_bias_v folded into its bias:
            # rows [q+u | q+v | k | v] (attention.py:348-367 adds the biases to a rounded q instead)
            lw["qkv4"] = (w(torch.cat([wq, wq, wk, wv], 0)), w(torch.cat([bq + u, bq + v, bk, bv], 0)))
            lw["out"] = (w(P[a + "linear_out.weight"]), w(P[a + "linear_out.bias"]))
            pos_w.append(P[a + "linear_pos.weight"])
            c = p + "conv_module."
            lw["pw1"] = (w(P[c + "pointwise_conv1.weight"].squeeze(-1)), w(P[c + "pointwise_conv1.bias"]))
            lw["dw"] = (w(P[c + "depthwise_conv.weight"].reshape(cfg.kernel, d)), w(P[c + "depthwise_conv.bias"]))
            lw["pw2"] = (w(P[c + "pointwise_conv2.weight"].squeeze(-1)), w(P[c + "pointwise_conv2.bias"]))
            if cfg.cnn_module_norm == "batch_norm":
                lw["conv_bn"] = self._fold_bn(P, c + "norm_activation", f)
                lw["norm_conv_affine"] = self._fold_bn(P, p + "norm_conv", f)
            else:
                raise NotImplementedError("cnn_module_norm other than batch_norm is not wired yet")
            # what a padded (zeroed) row carries after pointwise_conv1 + GLU in the padded path: GLU(bias)
            b1 = lw["pw1"][1].float()
            lw["glu_of_bias"] = (b1[:d] * torch.sigmoid(b1[d:])).to(dt).float().contiguous()
            self.layers.append(lw)
        self.pos_w_all = w(torch.cat(pos_w, 0))                      # (L*d, d): every layer's linear_pos at once
        self.after_norm = (w(P["encoder.after_norm.weight"]), w(P["encoder.after_norm.bias"]))
        # CTC head at close to fp32 input precision: weight split into 16-bit hi + lo parts and laid out
        # [W_hi | W_lo | W_hi] against hidden rows [h_hi | h_hi | h_lo] (the lo.lo term is dropped)
        cw = P["ctc.ctc_lo.weight"]
        cw_hi = cw.to(dt).float()
        self.ctc_w = w(torch.cat([cw_hi, cw - cw_hi, cw_hi], dim=1))
        self.ctc_b = w(P["ctc.ctc_lo.bias"])
        self.pe = w(self._positional_table(5000, d))

    @staticmethod
    def _fold_bn(P, prefix, f):
        scale = P[prefix + ".weight"] * torch.rsqrt(P[prefix + ".running_var"] + 1e-5)
        shift = P[prefix + ".bias"] - P[prefix + ".running_mean"] * scale
        return f(scale), f(shift)

    @staticmethod
    def _positional_table(max_len: int, d: int) -> torch.Tensor:
        """RelPositionalEncoding.pe (oasr/models/conformer/model.py:254-266)."""
        pe = torch.zeros(max_len, d)
        position = torch.arange(0, max_len, dtype=torch.float32).unsqueeze(1)
        div_term = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * -(math.log(10000.0) / d))
        pe[:, 0::2] = torch.sin(position * div_term)
        pe[:, 1::2] = torch.cos(position * div_term)
        return pe

    # ------------------------------------------------------------------ front end
    def _subsample(self, feats: torch.Tensor) -> torch.Tensor:
        """Conv2dSubsampling4 convolutions (model.py:433-449): (B,T,F) -> (B, T', F'*d) rows in
        NHWC-natural (f, c) order.  The first conv (one input channel) is an own fp32-in kernel;
        the second still runs through torch/cuDNN in the 16-bit dtype on the NHWC tensor."""
        x = fused.subsample_conv1(feats.float(), self.conv1_w, self.conv1_b, self.dtype)   # (B,T1,F1,C) NHWC
        x = x.permute(0, 3, 1, 2)                       # logical NCHW, channels_last in memory
        x = F.relu(F.conv2d(x, self.conv2_w, self.conv2_b, stride=2))
        B, C, T2, F2 = x.shape
        return x.permute(0, 2, 3, 1).reshape(B, T2, F2 * C)  # a view when x is channels_last

    # ------------------------------------------------------------------ layer stack
    def _encode_packed(self, rows: torch.Tensor, pk: PackedBatch, padded_semantics: bool) -> torch.Tensor:
        """rows: (total, F'*d) gathered embed-conv outputs.  Returns after_norm(hidden) as
        (total, 3*d) 16-bit rows [hi | hi | lo]."""
        cfg, dt = self.cfg, self.dtype
        d, M = cfg.d_model, pk.total
        dev = rows.device
        scale = 1.0 / math.sqrt(cfg.head_dim)
        res = torch.empty(M, d, device=dev, dtype=torch.float32)
        h = torch.empty(M, d, device=dev, dtype=dt)
        y = torch.empty(M, d, device=dev, dtype=dt)
        a_ffn = torch.empty(M, cfg.ffn, device=dev, dtype=dt)
        qkv4 = torch.empty(M, 4 * d, device=dev, dtype=dt)
        att = torch.empty(M, d, device=dev, dtype=dt)
        g = torch.empty(M, d, device=dev, dtype=dt)
        cv = torch.empty(M, d, device=dev, dtype=dt)

        # embed Linear (+LayerNorm, x sqrt(d) folded) -> fp32 residual, and the first pre-norm
        OF.gemm(rows, self.embed_w, self.embed_b, out=y)
        first = self.layers[0]["norm_ff_macaron"]
        if cfg.embed_layer_norm:
            fused.add_norm_f32(h, res, None, y, 1.0, fused.ADD_NORM_LN_LN, self.embed_ln_w, self.embed_ln_b, *first,
                               eps=1e-5)
        else:
            fused.add_norm_f32(h, res, None, y, 1.0, fused.ADD_NORM_LN, *first, eps=cfg.eps)
        # linear_pos of every layer in one GEMM: (Tm, d) x (L*d, d)^T
        pos_all = OF.gemm(self.pe[:pk.max_seg], self.pos_w_all)

        for i, lw in enumerate(self.layers):
            # macaron FFN (model.py:709-721)
            OF.gemm_activation(h, lw["ffm"][0], lw["ffm"][1], 2, out=a_ffn)
            OF.gemm(a_ffn, lw["ffm"][2], lw["ffm"][3], out=y)
            fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN, *lw["norm_mha"], eps=cfg.eps)
            # relative-position self-attention (attention.py:323-386)
            OF.gemm(h, lw["qkv4"][0], lw["qkv4"][1], out=qkv4)
            fused.fmha_varlen_relpos(qkv4, pos_all[:, i * d:(i + 1) * d], pk.cu_seqlens, pk.max_seg, cfg.heads, scale,
                                     out=att)
            OF.gemm(att, lw["out"][0], lw["out"][1], out=y)
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_AFFINE, *lw["norm_conv_affine"], eps=cfg.eps)
            # convolution module (model.py:223-233)
            OF.gemm_glu(h, lw["pw1"][0], lw["pw1"][1], out=g)
            fused.depthwise_conv1d_packed(
                g, lw["dw"][0], lw["dw"][1], pk.cu_seqlens, pk.max_seg, post_scale=lw["conv_bn"][0],
                post_shift=lw["conv_bn"][1], right_fill=lw["glu_of_bias"] if padded_semantics else None,
                fill_frames=pk.fill_frames if padded_semantics else None, activation=2, out=cv)
            OF.gemm(cv, lw["pw2"][0], lw["pw2"][1], out=y)
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_LN, *lw["norm_ff"], eps=cfg.eps)
            # FFN, then norm_final and the next layer's first pre-norm (or after_norm) in one pass
            OF.gemm_activation(h, lw["ff"][0], lw["ff"][1], 2, out=a_ffn)
            OF.gemm(a_ffn, lw["ff"][2], lw["ff"][3], out=y)
            if i + 1 < len(self.layers):
                fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_final"],
                                   *self.layers[i + 1]["norm_ff_macaron"], eps=cfg.eps)
            else:  # after_norm, written as [hi | hi | lo] for the split-precision head
                h3 = torch.empty(M, 3 * d, device=dev, dtype=dt)
                fused.add_norm_f32(h3, res, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_final"], *self.after_norm,
                                   eps=cfg.eps, split_out=True)
                return h3
        return h

    # ------------------------------------------------------------------ entry points
    def _forward(self, features: torch.Tensor, lengths, padded_semantics: bool, padded_output: bool,
                 return_argmax: bool):
        if not features.is_cuda:
            raise RuntimeError("features must be a CUDA tensor (oasr_b200 has no CPU path)")
        lens_host = lengths.tolist() if isinstance(lengths, torch.Tensor) else [int(x) for x in lengths]
        out_lens = [max((n - 3) // 4, 0) for n in lens_host]
        conv_rows = self._subsample(features)                                  # (B, Tp, F'*d)
        B, Tp, W = conv_rows.shape
        pk = build_packed_batch(out_lens, Tp, self.cfg.kernel, features.device)
        out_lengths = torch.tensor(out_lens, dtype=torch.int64, device=features.device)
        V = self.cfg.vocab_padded
        if pk.total == 0:
            lp = torch.zeros(B, Tp, V, device=features.device) if padded_output else torch.zeros(0, V, device=features.device)
            return (lp, out_lengths, None, pk) if return_argmax else (lp, out_lengths, pk)
        rows = gather_rows(conv_rows.reshape(B * Tp, W), pk.pack_src_idx)      # pack_hidden, before the embed Linear
        hidden = self._encode_packed(rows, pk, padded_semantics)
        res = OF.gemm_log_softmax(hidden, self.ctc_w, self.ctc_b, out_dtype=torch.float32, return_argmax=True)
        log_probs, argmax = res
        if padded_output:
            # padded rows carry hidden = 0 in the reference (packing.py:228-232): log_softmax(bias)
            pad_row = torch.log_softmax(self.ctc_b.float(), dim=-1)
            full = pad_row.expand(B * Tp, V).contiguous()
            full.index_copy_(0, pk.pack_src_idx, log_probs)
            log_probs = full.view(B, Tp, V)
        if return_argmax:
            return log_probs, out_lengths, argmax, pk
        return log_probs, out_lengths, pk

    def forward_offline(self, features: torch.Tensor, lengths) -> Tuple[torch.Tensor, torch.Tensor]:
        """Padded-batch semantics (oasr/models/base.py:749-754): ``(log_probs (B,T',V) fp32, out_lengths)``."""
        lp, ol, _ = self._forward(features, lengths, True, True, False)
        return lp, ol

    def forward_offline_packed(self, features: torch.Tensor, lengths, padded_output: bool = True):
        """Sequence-packing semantics (oasr/models/base.py:756-761).  With ``padded_output=False``
        the log-probs stay packed ``(total, V)`` and the packed-batch description is returned too."""
        lp, ol, pk = self._forward(features, lengths, False, padded_output, False)
        return (lp, ol) if padded_output else (lp, ol, pk)

    def greedy_search(self, features: torch.Tensor, lengths, packed: bool = True) -> List[List[int]]:
        """Features -> greedy CTC token lists (argmax per frame in the head's epilogue, then drop
        repeats and blanks; rule of csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55)."""
        _, _, argmax, pk = self._forward(features, lengths, not packed, False, True)
        if argmax is None:
            return [[] for _ in pk.seg_lengths]
        ids = argmax.cpu().tolist()
        out, pos = [], 0
        for n in pk.seg_lengths:
            hyp, prev = [], None
            for t in ids[pos:pos + n]:
                if t != prev and t != 0:
                    hyp.append(t)
                prev = t
            out.append(hyp)
            pos += n
        return out
