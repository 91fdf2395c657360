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
    causal: bool = False   # causal depthwise conv (left context kernel-1): the streaming configuration

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
    import numpy as np

    lens = np.asarray(out_lengths, dtype=np.int64).reshape(-1)
    cu = np.zeros(lens.size + 1, dtype=np.int64)
    np.cumsum(lens, out=cu[1:])
    total = int(cu[-1])
    half = (conv_kernel - 1) // 2
    # packed row r of utterance b sits at padded row b * padded_t + (r - cu[b]): one vectorised pass, no per-utterance work
    idx = torch.from_numpy(np.arange(total, dtype=np.int64) +
                           np.repeat(np.arange(lens.size, dtype=np.int64) * padded_t - cu[:-1], lens))
    fill = torch.from_numpy(np.minimum(half, padded_t - lens).astype(np.int32))
    return PackedBatch(
        num_segs=int(lens.size), total=total, max_seg=int(lens.max()) if lens.size else 0, padded_t=padded_t,
        seg_lengths=list(out_lengths),
        cu_seqlens=torch.from_numpy(cu.astype(np.int32)).to(device, non_blocking=True),
        pack_src_idx=idx.to(device, non_blocking=True),
        fill_frames=fill.to(device, non_blocking=True),
    )


class ConformerCTC:
    """WeNet-style Conformer encoder + CTC head running on the sm_100a kernels."""

    last_d2h_bytes = 0    # bytes the latest greedy_search_batches step read back (token rows + lengths)

    def __init__(self, cfg: ConformerConfig, params: Dict[str, torch.Tensor], device="cuda",
                 dtype: torch.dtype = torch.bfloat16, quant: Optional[str] = None):
        """``quant``: None = 16-bit GEMMs; "fp8" / "int8" = the eight Linear GEMMs of every layer run on
        fp8-e4m3 / int8 operands (weights quantised per output channel here, activations per token on the
        fly); offline entry points only."""
        if quant not in (None, "fp8", "int8"):
            raise ValueError("quant must be None, 'fp8' or 'int8'")
        self.quant_kind = {None: 0, "fp8": 1, "int8": 2}[quant]
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
        # Conv2d weights are stored KRSC (NHWC): exactly the (N, 9*C) K-major operand of the implicit GEMM.
        self.conv1_w = f(P[e + "convs.0.weight"].reshape(d, 3, 3))   # (C, 3, 3, 1) -> (C, 3, 3), fp32
        self.conv1_b = f(P[e + "convs.0.bias"])
        self.conv2_b = w(P[e + "convs.1.bias"])
        self.conv2_krsc = w(P[e + "convs.1.weight"])                  # (C_out, 3, 3, C_in): taps outermost, channels innermost
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
        # CTC head with its INPUT at close to fp32 precision: hidden rows arrive as two 16-bit terms [h_hi | h_lo] and
        # meet the 16-bit weight twice, [W | W] (rounding the head's input to bf16 alone costs 4e-4 mean-abs of the
        # log-probs against the fp32 path, rounding its weight 1e-4: the weight keeps its one rounding)
        cw = P["ctc.ctc_lo.weight"]
        self.ctc_w = w(torch.cat([cw, cw], dim=1))
        self.ctc_b = w(P["ctc.ctc_lo.bias"])
        self.pe = w(self._positional_table(5000, d))
        self._build_native_model()

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
    def _subsample_packed(self, feats: torch.Tensor, out_lens: List[int], cu_frames: torch.Tensor, total: int,
                          t1_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Conv2dSubsampling4 convolutions (model.py:433-449) + pack_hidden (packing.py:204-216):
        ``(B, T, F)`` fp32 features -> ``(total, F' * d)`` packed rows in ``(f, c)`` order, valid frames only.
        First conv: fp32-in stencil kernel writing the parity-split layout; second conv: tcgen05 implicit GEMM."""
        B, T, Fd = feats.shape
        T1, F1 = (T - 3) // 2 + 1, (Fd - 3) // 2 + 1
        x1 = fused.subsample_conv1_s2d(feats.float(), self.conv1_w, self.conv1_b, self.dtype, t1_limit=t1_limit)
        return fused.subsample_conv2(x1, T1, F1, self.conv2_krsc, self.conv2_b, cu_frames, total)

    # ------------------------------------------------------------------ layer stack
    def _quantize_weights(self) -> None:
        """Per-output-channel 8-bit copies of the eight Linear weights of every layer, in the order of
        oasr_b200_conformer_layer::q_w (ffm_w1, ffm_w2, qkv4, out, pw1, pw2, ff_w1, ff_w2)."""
        from . import quant

        for lw in self.layers:
            ws = [lw["ffm"][0], lw["ffm"][2], lw["qkv4"][0], lw["out"][0], lw["pw1"][0], lw["pw2"][0], lw["ff"][0], lw["ff"][2]]
            lw["q8"] = [quant.quantize_rows(w, self.quant_kind) for w in ws]

    def _build_native_model(self) -> None:
        """Fill the C structs of the native executor with the prepared device pointers."""
        if self.quant_kind and "q8" not in self.layers[0]:
            self._quantize_weights()
        import ctypes

        from . import _lib
        from .functional import _DTYPE_ID

        def ptr(t):
            return None if t is None else ctypes.c_void_p(t.data_ptr())

        L = len(self.layers)
        arr = (_lib.ConformerLayer * L)()
        for i, lw in enumerate(self.layers):
            c = arr[i]
            c.norm_ff_macaron_w, c.norm_ff_macaron_b = map(ptr, lw["norm_ff_macaron"])
            c.ffm_w1, c.ffm_b1, c.ffm_w2, c.ffm_b2 = map(ptr, lw["ffm"])
            c.norm_mha_w, c.norm_mha_b = map(ptr, lw["norm_mha"])
            c.qkv4_w, c.qkv4_b = map(ptr, lw["qkv4"])
            c.out_w, c.out_b = map(ptr, lw["out"])
            c.norm_conv_scale, c.norm_conv_shift = map(ptr, lw["norm_conv_affine"])
            c.pw1_w, c.pw1_b = map(ptr, lw["pw1"])
            c.dw_w, c.dw_b = map(ptr, lw["dw"])
            c.conv_bn_scale, c.conv_bn_shift = map(ptr, lw["conv_bn"])
            c.glu_of_bias = ptr(lw["glu_of_bias"])
            c.pw2_w, c.pw2_b = map(ptr, lw["pw2"])
            c.norm_ff_w, c.norm_ff_b = map(ptr, lw["norm_ff"])
            c.ff_w1, c.ff_b1, c.ff_w2, c.ff_b2 = map(ptr, lw["ff"])
            c.norm_final_w, c.norm_final_b = map(ptr, lw["norm_final"])
            if self.quant_kind:
                for qi, (wq, ws) in enumerate(lw["q8"]):
                    c.q_w[qi], c.q_s[qi] = wq.data_ptr(), ws.data_ptr()
        cfg = self.cfg
        m = _lib.ConformerModel()
        m.d_model, m.heads, m.ffn, m.kernel, m.num_layers = cfg.d_model, cfg.heads, cfg.ffn, cfg.kernel, L
        m.vocab_padded, m.embed_in, m.dtype, m.eps = cfg.vocab_padded, self.embed_w.size(1), _DTYPE_ID[self.dtype], cfg.eps
        m.layers = arr
        m.embed_w, m.embed_b = ptr(self.embed_w), ptr(self.embed_b)
        m.embed_ln_w, m.embed_ln_b = ptr(self.embed_ln_w), ptr(self.embed_ln_b)
        m.pos_w_all, m.pe, m.pe_rows = ptr(self.pos_w_all), ptr(self.pe), self.pe.size(0)
        m.after_norm_w, m.after_norm_b = map(ptr, self.after_norm)
        m.ctc_w, m.ctc_b = ptr(self.ctc_w), ptr(self.ctc_b)
        m.pos_proj, m.pos_proj_rows = None, 0
        m.quant_kind = self.quant_kind
        self._native_layers, self._native_model = arr, m   # keep both alive
        self._workspace = None
        self._pos_proj = None

    def _encode_packed(self, rows: torch.Tensor, pk: PackedBatch, padded_semantics: bool, want_log_probs: bool = True):
        """rows: (total, F'*d) gathered embed-conv outputs -> (log_probs (total, V) fp32, argmax (total,) int32).
        One call into the native executor (oasr_b200_conformer_encode_packed).  ``want_log_probs=False`` is the
        token-only form: the head sweeps the vocabulary once, keeps the running first maximum per frame and
        writes nothing but the argmax (``log_probs`` comes back ``None``)."""
        import ctypes

        from . import _lib
        from .functional import _p

        lib = _lib.load()
        need = lib.oasr_b200_conformer_workspace_bytes(ctypes.byref(self._native_model), pk.total, pk.max_seg)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(int(need * 1.25) + 256, dtype=torch.uint8, device=rows.device)
        ws = self._workspace
        off = (-ws.data_ptr()) % 256
        log_probs = torch.empty(pk.total, self.cfg.vocab_padded, device=rows.device, dtype=torch.float32) \
            if want_log_probs else None
        argmax = torch.empty(pk.total, device=rows.device, dtype=torch.int32)
        _lib.call("oasr_b200_conformer_encode_packed", ctypes.byref(self._native_model), _p(rows), _p(pk.cu_seqlens),
                  _p(pk.fill_frames) if padded_semantics else None, pk.num_segs, pk.total, pk.max_seg,
                  ctypes.c_void_p(ws.data_ptr() + off), ws.numel() - off, _p(log_probs), _p(argmax),
                  ctypes.c_void_p(torch.cuda.current_stream(rows.device).cuda_stream))
        return log_probs, argmax

    def encode_rows_noalloc(self, rows: torch.Tensor, pk: PackedBatch, log_probs: torch.Tensor,
                            argmax: torch.Tensor, padded_semantics: bool = False) -> None:
        """The layer stack + head for callers that cannot allocate device memory (a host that gave all
        GPU memory to its own pool, an allocator hook, a thread that must not risk a device-wide stall):
        ``log_probs (total, V) fp32`` and ``argmax (total,) int32`` are the caller's, the scratch is the
        64 MiB array built into the library (oasr_b200_conformer_encode_packed_noalloc).  Raises if the
        batch needs more scratch than that.  Calls share the array: do not overlap two of them on the
        GPU.  The first call on a device resolves the array's address; make it outside stream capture."""
        import ctypes

        from . import _lib
        from .functional import _p

        _lib.call("oasr_b200_conformer_encode_packed_noalloc", ctypes.byref(self._native_model), _p(rows),
                  _p(pk.cu_seqlens), _p(pk.fill_frames) if padded_semantics else None, pk.num_segs, pk.total,
                  pk.max_seg, _p(log_probs), _p(argmax),
                  ctypes.c_void_p(torch.cuda.current_stream(rows.device).cuda_stream))

    # ------------------------------------------------------------------ entry points
    # ------------------------------------------------------------------ streaming
    def new_streaming_cache(self, max_streams: int, max_past_frames: int, chunk_frames: int = 16, block_size: int = 16,
                            seed: Optional[int] = 0, kv_scales: Optional[torch.Tensor] = None):
        """Page pools, block table and conv left-context buffers for ``max_streams`` concurrent streams.
        ``kv_scales`` ``(layers, 2, heads)`` fp32 (K then V, e.g. from ``calibrate_kv_scales``) switches the
        pools to fp8 e4m3 codes with those per-head scales."""
        from .streaming import StreamingCache

        c = self.cfg
        return StreamingCache(c.layers, c.heads, c.head_dim, c.d_model, c.kernel, max_streams, max_past_frames,
                              chunk_frames, block_size, self.device, self.dtype, seed, kv_scales)

    def calibrate_kv_scales(self, windows, chunk_frames: int = 16, margin: float = 1.0) -> torch.Tensor:
        """Per (layer, head) fp8 scales ``amax / 448`` of the keys and values seen while the feature windows
        ``windows`` (an iterable of ``(B, window, F)`` tensors, consecutive chunks of the same B streams) run through
        a 16-bit cache.  Returns ``(layers, 2, heads)`` fp32."""
        c = self.cfg
        windows = list(windows)
        B = windows[0].size(0)
        cache = self.new_streaming_cache(B, max_past_frames=chunk_frames * len(windows), chunk_frames=chunk_frames, seed=None)
        for xs in windows:
            self.forward_chunk_paged(xs.to(self.device), list(range(B)), cache)
        k = cache.k_pool.float().abs().amax(dim=(1, 2, 4))     # (L, H)
        v = cache.v_pool.float().abs().amax(dim=(1, 2, 4))
        scales = torch.stack([k, v], dim=1) * (margin / 448.0)
        return torch.clamp(scales, min=1e-8).contiguous()

    def _chunk_launch(self, xs: torch.Tensor, cache, table, cached, total, pos_start, slot_ids):
        """The device work of one streaming step on the current stream: subsampling convolutions + ONE native call
        (oasr_b200_conformer_chunk_paged).  No host synchronisation, no host-to-device copy: capturable."""
        import ctypes

        from . import _lib
        from .functional import _p

        B = xs.size(0)
        T = cache.chunk
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=xs.device)
        rows = self._subsample_packed(xs, [T] * B, cu, B * T)                  # (B * chunk, F'*d)
        lib = _lib.load()
        need = lib.oasr_b200_conformer_chunk_workspace_bytes(ctypes.byref(self._native_model), B, T)
        if self._workspace is None or self._workspace.numel() < need + 256:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the workspace must exist before a capture: run one eager step of this shape first")
            self._workspace = torch.empty(int(need * 1.25) + 256, dtype=torch.uint8, device=xs.device)
        ws = self._workspace
        off = (-ws.data_ptr()) % 256
        L = self.cfg.layers
        kp = (ctypes.c_void_p * L)(*[cache.k_pool[i].data_ptr() for i in range(L)])
        vp = (ctypes.c_void_p * L)(*[cache.v_pool[i].data_ptr() for i in range(L)])
        log_probs = torch.empty(B, T, self.cfg.vocab_padded, device=xs.device, dtype=torch.float32)
        argmax = torch.empty(B, T, device=xs.device, dtype=torch.int32)
        _lib.call("oasr_b200_conformer_chunk_paged", ctypes.byref(self._native_model), _p(rows), B, T, kp, vp, _p(table),
                  _p(cached), _p(total), _p(pos_start), table.size(1), cache.block_size, cache.num_blocks,
                  _p(cache.kv_scales), _p(cache.cnn_state), cache.max_streams, _p(slot_ids), ctypes.c_void_p(ws.data_ptr() + off),
                  ws.numel() - off, _p(log_probs), _p(argmax),
                  ctypes.c_void_p(torch.cuda.current_stream(xs.device).cuda_stream))
        return log_probs, argmax

    def graphed_chunk_forward(self, cache, batch: int, window: int):
        """A streaming step of fixed shape captured once into a CUDA graph (the reference's GraphedEncoderForward,
        oasr/engine/graph_cache.py:24-29): see :class:`GraphedChunkForward`."""
        return GraphedChunkForward(self, cache, batch, window)

    def forward_chunk_paged(self, xs: torch.Tensor, slots, cache, return_argmax: bool = False):
        """One streaming chunk for the streams in ``slots``: ``xs (B, window, F)`` feature windows ->
        ``log_probs (B, chunk, V)`` fp32 (ConformerEncoder.forward_chunk_paged + head,
        oasr/models/conformer/model.py:913-1023, oasr/models/base.py:763-777).  K/V pages and the conv
        left context in ``cache`` are updated in place; page allocation, eviction and the commit of
        ``cache_seqlens`` happen around the single native call."""
        import ctypes

        from . import _lib
        from .functional import _p

        if not self.cfg.causal:
            raise RuntimeError("streaming needs a causal conv module (cfg.causal=True)")
        if not xs.is_cuda:
            raise RuntimeError("xs must be a CUDA tensor (oasr_b200 has no CPU path)")
        if self._pos_proj is None:   # linear_pos of the whole positional table, every layer at once
            self._pos_proj = OF.gemm(self.pe, self.pos_w_all)
            self._native_model.pos_proj = ctypes.c_void_p(self._pos_proj.data_ptr())
            self._native_model.pos_proj_rows = self._pos_proj.size(0)
        slots = list(slots)
        B = xs.size(0)
        T = (((xs.size(1) - 3) // 2 + 1) - 3) // 2 + 1
        if T != cache.chunk:      # checked before any page is handed out: a refused call leaves the cache untouched
            raise RuntimeError(f"the feature window gives {T} encoder frames, the cache was built for {cache.chunk}")
        if len(slots) != B:
            raise RuntimeError(f"{B} feature windows for {len(slots)} slots")
        table, cached, total, pos_start, slot_ids = cache.prepare(slots)
        log_probs, argmax = self._chunk_launch(xs, cache, table, cached, total, pos_start, slot_ids)
        cache.commit(slots)
        return (log_probs, argmax) if return_argmax else log_probs

    def _forward(self, features: torch.Tensor, lengths, padded_semantics: bool, padded_output: bool,
                 return_argmax: bool, tokens_only: bool = False):
        if self.cfg.causal:
            raise NotImplementedError("offline forward with a causal conv module is not wired; use forward_chunk_paged")
        if not features.is_cuda:
            raise RuntimeError("features must be a CUDA tensor (oasr_b200 has no CPU path)")
        lens_host = lengths.tolist() if isinstance(lengths, torch.Tensor) else [int(x) for x in lengths]
        out_lens = [max((n - 3) // 4, 0) for n in lens_host]
        T = features.size(1)
        Tp = (((T - 3) // 2 + 1) - 3) // 2 + 1
        pk = build_packed_batch(out_lens, Tp, self.cfg.kernel, features.device)
        t1_limit = torch.tensor([2 * n + 1 for n in out_lens], dtype=torch.int32).to(features.device, non_blocking=True)
        B = features.size(0)
        out_lengths = torch.tensor(out_lens, dtype=torch.int64, device=features.device)
        V = self.cfg.vocab_padded
        if pk.total == 0:
            lp = torch.zeros(B, Tp, V, device=features.device) if padded_output else torch.zeros(0, V, device=features.device)
            return (lp, out_lengths, None, pk) if return_argmax else (lp, out_lengths, pk)
        rows = self._subsample_packed(features, out_lens, pk.cu_seqlens, pk.total, t1_limit)   # packed before the embed Linear
        log_probs, argmax = self._encode_packed(rows, pk, padded_semantics, want_log_probs=not tokens_only)
        if padded_output and log_probs is not None:
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

    @staticmethod
    def _collapse(ids, seg_lengths) -> List[List[int]]:
        """Per-frame argmax ids of packed segments -> token lists: drop repeats, then blanks (id 0), never
        across a segment boundary (rule of csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55)."""
        import numpy as np

        a = np.asarray(ids, dtype=np.int64)
        if a.size == 0:
            return [[] for _ in seg_lengths]
        lens = np.asarray(seg_lengths, dtype=np.int64)
        ends = np.cumsum(lens)
        starts = ends - lens
        prev = np.empty_like(a)
        prev[1:] = a[:-1]
        prev[starts[lens > 0]] = -1
        keep = (a != prev) & (a != 0)
        csum = np.concatenate([[0], np.cumsum(keep)])
        counts = csum[ends] - csum[starts]
        kept = a[keep]
        out, pos = [], 0
        for c in counts.tolist():
            out.append(kept[pos:pos + c].tolist())
            pos += c
        return out

    def greedy_search(self, features: torch.Tensor, lengths, packed: bool = True) -> List[List[int]]:
        """Features -> greedy CTC token lists: the head keeps the per-frame first maximum in its epilogue and writes
        no log-probs (the reference's greedy search reads fp32 log-probs back, oasr/functionals/ctc_decode.py:359);
        repeats and blanks are dropped on the device (``ctc_greedy_collapse``), the host only slices the rows."""
        _, _, argmax, pk = self._forward(features, lengths, not packed, False, True, tokens_only=True)
        if argmax is None:
            return [[] for _ in pk.seg_lengths]
        tokens, counts, _ = fused.ctc_greedy_collapse(argmax, pk.cu_seqlens, max(pk.seg_lengths))
        return self._rows_to_lists(tokens.cpu(), counts.cpu())

    @staticmethod
    def _rows_to_lists(tokens: torch.Tensor, counts: torch.Tensor) -> List[List[int]]:
        rows = tokens.numpy()
        return [rows[b, :n].tolist() for b, n in enumerate(counts.tolist())]

    def greedy_search_batches(self, batches, packed: bool = True):
        """Pipelined greedy search over an iterable of ``(host_features, lengths)`` batches (pinned host
        memory for the copies to overlap): the host-to-device copy of batch i+1 runs on a copy stream
        under the encoder of batch i, and the device-to-host read of batch i's collapsed token rows runs
        under the encoder of batch i+1.  Yields one list of token lists per batch, in order."""
        dev = self.device
        main = torch.cuda.current_stream(dev)
        copy_stream = torch.cuda.Stream(dev)
        pending = None
        staged = None

        def stage(item):
            feats_host, lengths = item
            with torch.cuda.stream(copy_stream):
                f = feats_host.to(dev, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return f, lengths, ev

        it = iter(batches)
        nxt = next(it, None)
        if nxt is not None:
            staged = stage(nxt)
        while staged is not None:
            f, lengths, ev = staged
            nxt = next(it, None)
            staged = stage(nxt) if nxt is not None else None      # next copy goes out before this batch's launches
            main.wait_event(ev)
            f.record_stream(main)
            _, _, argmax, pk = self._forward(f, lengths, not packed, False, True, tokens_only=True)
            if argmax is None:
                cur = (None, pk, None)
            else:
                tokens, counts, _ = fused.ctc_greedy_collapse(argmax, pk.cu_seqlens, max(pk.seg_lengths))
                host = (torch.empty(tokens.shape, dtype=tokens.dtype, pin_memory=True),
                        torch.empty(counts.shape, dtype=counts.dtype, pin_memory=True))
                host[0].copy_(tokens, non_blocking=True)
                host[1].copy_(counts, non_blocking=True)
                done = torch.cuda.Event()
                done.record(main)
                cur = (host, pk, done)
                self.last_d2h_bytes = tokens.numel() * 4 + counts.numel() * 4
            if pending is not None:
                yield self._finish(pending)
            pending = cur
        if pending is not None:
            yield self._finish(pending)

    def _finish(self, item) -> List[List[int]]:
        host, pk, done = item
        if host is None:
            return [[] for _ in pk.seg_lengths]
        done.synchronize()
        return self._rows_to_lists(host[0], host[1])


class GraphedChunkForward:
    """One streaming step of ``batch`` streams x ``window`` feature frames, captured once into a CUDA graph and
    replayed per chunk (the reference captures its streaming encoder the same way: ``GraphedEncoderForward``,
    oasr/engine/graph_cache.py:24-29).  The step is about 170 launches of a few microseconds each, so replaying one
    graph instead of enqueueing them takes the launch path off the host.  Everything that changes from chunk to chunk
    is data in fixed device buffers: the feature windows, the block-table rows, the cached / total lengths, the
    position starts and the slot ids; the page pools and conv states are the cache's own.  Outputs are the graph's
    static ``log_probs (batch, chunk, V)`` / ``argmax``: read (or copy) them before the next call."""

    def __init__(self, model: "ConformerCTC", cache, batch: int, window: int):
        if model._pos_proj is None or model._workspace is None:
            raise RuntimeError("run one eager forward_chunk_paged of this shape first (it sizes the workspace and builds "
                               "the positional projection)")
        self.model, self.cache, self.batch = model, cache, batch
        dev = model.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.xs = torch.zeros(batch, window, model.cfg.input_size, device=dev, dtype=torch.float32)
        self.table = torch.zeros(batch, cache.max_blocks, **i32)
        self.cached = torch.zeros(batch, **i32)
        self.total = torch.full((batch,), cache.chunk, **i32)
        self.pos_start = torch.zeros(batch, **i32)
        self.slot_ids = torch.full((batch,), -1, dtype=torch.int64, device=dev)
        from . import _lib

        self.graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(dev)
        before = _lib.launch_count()
        with torch.cuda.graph(self.graph):
            self.log_probs, self.argmax = model._chunk_launch(self.xs, cache, self.table, self.cached, self.total,
                                                              self.pos_start, self.slot_ids)
        self.launches_per_replay = _lib.launch_count() - before     # this library's kernels inside the graph

    def __call__(self, xs: torch.Tensor, slots):
        slots = list(slots)
        if len(slots) != self.batch or tuple(xs.shape) != tuple(self.xs.shape):
            raise RuntimeError(f"this graph was captured for {tuple(self.xs.shape)} windows of {self.batch} streams")
        table, cached, total, pos_start, slot_ids = self.cache.prepare(slots)
        self.xs.copy_(xs, non_blocking=True)
        self.table.copy_(table, non_blocking=True)
        self.cached.copy_(cached, non_blocking=True)
        self.total.copy_(total, non_blocking=True)
        self.pos_start.copy_(pos_start, non_blocking=True)
        self.slot_ids.copy_(slot_ids, non_blocking=True)
        self.graph.replay()
        self.cache.commit(slots)
        return self.log_probs, self.argmax
