"""FastConformer / Nemotron encoder (8x subsampling front end + layer stack) on the sm_100a operators (offline,
padded batch).

The composition the reference's ``NemotronEncoderLayer.forward`` serves
(oasr/models/nemotron/encoder.py:217-267): macaron FFNs with SiLU, Transformer-XL relative-position
attention with a ``rel_shift``-ed position bias and the chunked-limited window
(encoder.py:82-149, 300-359), conv module with a causal depthwise conv and LayerNorm+SiLU
(encoder.py:150-214), fused add+LayerNorm between the sub-layers, fp32 residual stream.
Every contraction, normalisation, activation, convolution and the attention run on this package's
kernels (head_dim 128 attention with an additive bias, ``layer_norm_activation``, causal
``depthwise_conv1d``); the position bias is one batched GEMM against the projected relative table
followed by one kernel that applies the Transformer-XL shift, the scale and the window / padding mask.
``FastConformerEncoder`` puts the 8x causal depthwise-separable subsampling front end in front of the stack
(oasr/models/nemotron/subsampling.py:26-131, 204-224): stem conv on the fp32 stencil kernel, two stages of
depthwise 3x3 / stride-2 conv (own NHWC kernel) + pointwise GEMM with a fused ReLU, projection GEMM.  The RNN-T
head is outside this module.
"""
from __future__ import annotations

import math
from typing import Dict, List

import numpy as np
import torch

from . import functional as OF
from . import fused
from .attention import fmha

MASK_FLOOR = -1.0e4   # finite additive floor of a masked key (encoder.py:80)
_SWISH = 2


class FastConformerLayers:
    def __init__(self, hidden: int, heads: int, ffn: int, layers: int, kernel: int, sliding_window: int, lookahead: int,
                 params: Dict[str, torch.Tensor], device="cuda", dtype: torch.dtype = torch.bfloat16, eps: float = 1e-5,
                 quant: str = None):
        """``quant`` "fp8" / "int8": the Linear GEMMs of every layer (FFNs, q/k/v, output, pointwise convs) run on
        8-bit operands with per-output-channel weight scales and per-token dynamic activation scales."""
        if hidden % heads or hidden // heads not in (64, 128):
            raise ValueError("head_dim must be 64 or 128")
        if quant not in (None, "fp8", "int8"):
            raise ValueError("quant must be None, 'fp8' or 'int8'")
        self.qkind = {None: 0, "fp8": 1, "int8": 2}[quant]
        self._q8 = {}
        self._tables = {}
        self._stream_tables = {}
        self.C, self.H, self.D, self.F, self.L, self.K = hidden, heads, hidden // heads, ffn, layers, kernel
        self.left, self.right, self.eps = sliding_window - 1, lookahead, eps
        self.device, self.dtype = torch.device(device), dtype
        w = lambda t: t.detach().to(torch.float32).to(dtype).to(self.device).contiguous()
        f = lambda t: t.detach().to(torch.float32).to(self.device).contiguous()
        opt = lambda k: w(params[k]) if k in params else None
        self.layers: List[dict] = []
        for i in range(layers):
            p = f"layers.{i}."
            a, c = p + "self_attn.", p + "conv."
            lw = {}
            for ff in ("feed_forward1", "feed_forward2"):
                lw[ff] = (w(params[p + ff + ".linear1.weight"]), opt(p + ff + ".linear1.bias"),
                          w(params[p + ff + ".linear2.weight"]), opt(p + ff + ".linear2.bias"))
            # q projected twice, once per global bias: [Wq; Wq; Wk; Wv] with [bq+u; bq+v; bk; bv] (the biases are
            # added in fp32 here, as the packed Conformer path does)
            wq, wk, wv = (params[a + n + ".weight"].float() for n in ("q_proj", "k_proj", "v_proj"))
            zero = torch.zeros(hidden)
            bq, bk, bv = (params.get(a + n + ".bias", zero).float() for n in ("q_proj", "k_proj", "v_proj"))
            u, v = params[a + "bias_u"].float().reshape(-1), params[a + "bias_v"].float().reshape(-1)
            lw["qkv4"] = (w(torch.cat([wq, wq, wk, wv], 0)), w(torch.cat([bq + u, bq + v, bk, bv], 0)))
            lw["o"] = (w(params[a + "o_proj.weight"]), opt(a + "o_proj.bias"))
            lw["rel"] = w(params[a + "relative_k_proj.weight"])
            lw["pw1"] = (w(params[c + "pointwise_conv1.weight"].squeeze(-1)), opt(c + "pointwise_conv1.bias"))
            lw["dw"] = (w(params[c + "depthwise_conv.weight"].reshape(kernel, hidden)), opt(c + "depthwise_conv.bias"))
            lw["conv_norm"] = (w(params[c + "norm.weight"]), w(params[c + "norm.bias"]))
            lw["pw2"] = (w(params[c + "pointwise_conv2.weight"].squeeze(-1)), opt(c + "pointwise_conv2.bias"))
            for n in ("norm_feed_forward1", "norm_self_att", "norm_conv", "norm_feed_forward2", "norm_out"):
                lw[n] = (w(params[p + n + ".weight"]), w(params[p + n + ".bias"]))
            self.layers.append(lw)
        self._workspace = None
        self.native = True                # packed batches run through the one-call native executor
        self._build_native_model()

    def set_quant(self, quant) -> None:
        """Switch the Linear GEMMs of the stack between 16-bit (``None``) and an 8-bit kind ("fp8" / "int8")."""
        if quant not in (None, "fp8", "int8"):
            raise ValueError("quant must be None, 'fp8' or 'int8'")
        self.qkind = {None: 0, "fp8": 1, "int8": 2}[quant]
        self._q8 = {}
        self._build_native_model()

    def _build_native_model(self) -> None:
        """The host-side description of the stack the native executor takes (struct oasr_b200_fastconformer_model):
        device pointers of the prepared weights, kept alive by ``self.layers``."""
        import ctypes

        from . import _lib
        from .functional import _DTYPE_ID

        ptr = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
        arr = (_lib.FastConformerLayer * self.L)()
        for i, lw in enumerate(self.layers):
            c = arr[i]
            for field, key in (("norm_ff1", "norm_feed_forward1"), ("norm_att", "norm_self_att"), ("norm_conv", "norm_conv"),
                               ("norm_ff2", "norm_feed_forward2"), ("norm_out", "norm_out"), ("conv_norm", "conv_norm")):
                setattr(c, field + "_w", ptr(lw[key][0]))
                setattr(c, field + "_b", ptr(lw[key][1]))
            for field, key in (("ff1", "feed_forward1"), ("ff2", "feed_forward2")):
                for n, t in zip(("_w1", "_b1", "_w2", "_b2"), lw[key]):
                    setattr(c, field + n, ptr(t))
            c.qkv4_w, c.qkv4_b, c.rel_w = ptr(lw["qkv4"][0]), ptr(lw["qkv4"][1]), ptr(lw["rel"])
            c.o_w, c.o_b = ptr(lw["o"][0]), ptr(lw["o"][1])
            c.pw1_w, c.pw1_b = ptr(lw["pw1"][0]), ptr(lw["pw1"][1])
            c.dw_w, c.dw_b = ptr(lw["dw"][0]), ptr(lw["dw"][1])
            c.pw2_w, c.pw2_b = ptr(lw["pw2"][0]), ptr(lw["pw2"][1])
            if self.qkind:
                # the eight Linear weights per output channel in 8 bits, in the order of the struct's q_w / q_s
                linears = (lw["feed_forward1"][0], lw["feed_forward1"][2], lw["qkv4"][0], lw["o"][0], lw["pw1"][0],
                           lw["pw2"][0], lw["feed_forward2"][0], lw["feed_forward2"][2])
                for j, wt in enumerate(linears):
                    wq, ws = self._weight_q8(wt)
                    c.q_w[j], c.q_s[j] = wq.data_ptr(), ws.data_ptr()
        m = _lib.FastConformerModel()
        m.hidden, m.heads, m.ffn, m.kernel, m.num_layers = self.C, self.H, self.F, self.K, self.L
        m.dtype = _DTYPE_ID[self.dtype]
        m.left_context, m.right_context = self.left, self.right
        m.eps, m.mask_floor = self.eps, MASK_FLOOR
        m.layers = ctypes.cast(arr, ctypes.POINTER(_lib.FastConformerLayer))
        m.quant_kind = self.qkind
        self._native_layers, self._native_model = arr, m      # keep both alive

    def _layers_native(self, rows: torch.Tensor, g) -> torch.Tensor:
        """The packed stack in ONE call into the native executor (oasr_b200_fastconformer_layers_packed): the same
        kernels in the same order as :meth:`_layers_composed`, enqueued from C++ on the current stream."""
        import ctypes

        from . import _lib
        from .functional import _p, _stream

        M, C = rows.shape
        res = rows
        table = self._position_table(g["T"])
        lib = _lib.load()
        need = lib.oasr_b200_fastconformer_workspace_bytes(ctypes.byref(self._native_model), M, table.size(0), g["bias_numel"])
        if self._workspace is None or self._workspace.numel() < need + 256:
            self._workspace = torch.empty(int(need * 1.25) + 256, dtype=torch.uint8, device=res.device)
        ws = self._workspace
        off = (-ws.data_ptr()) % 256
        out = torch.empty(M, C, device=res.device, dtype=torch.float32)
        _lib.call("oasr_b200_fastconformer_layers_packed", ctypes.byref(self._native_model), _p(rows),
                  1 if rows.dtype == torch.float32 else 0, _p(out), _p(table),
                  table.size(0), _p(g["cu"]), _p(g["offsets"]), g["bias_numel"], g["cu"].numel() - 1, M, g["T"],
                  ctypes.c_void_p(ws.data_ptr() + off), ws.numel() - off, _stream(res))
        return out

    def _weight_q8(self, w: torch.Tensor):
        """The 8-bit copy of a Linear weight (per output channel) and its scales, quantised once and kept."""
        from . import quant
        key = w.data_ptr()
        if key not in self._q8:
            self._q8[key] = quant.quantize_rows(w, self.qkind)
        return self._q8[key]

    def _linear(self, x: torch.Tensor, w: torch.Tensor, b, act: int = -1, glu: bool = False) -> torch.Tensor:
        """One Linear: 16-bit GEMM, or per-token quantisation + 8-bit GEMM against the cached 8-bit weight."""
        if not self.qkind:
            if glu:
                return OF.gemm_glu(x, w, b)
            return OF.gemm_activation(x, w, b, act) if act >= 0 else OF.gemm(x, w, b)
        from . import quant
        wq, ws = self._weight_q8(w)
        xq, xs = quant.quantize_rows(x, self.qkind)
        return quant.gemm_q8(xq, xs, wq, ws, b, kind=self.qkind, activation=act, glu=glu, out_dtype=self.dtype)

    # ---- host-side tables (lengths are host values: no device synchronisation) ----
    def _position_table(self, T: int) -> torch.Tensor:
        """Sinusoid rows for relative positions T-1 .. -(T-1), then zero rows up to a multiple of 8 (the column granule
        of the GEMM that multiplies them); built once per T and kept on the device."""
        hit = self._tables.get(T)
        if hit is not None:
            return hit
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, self.C, 2, dtype=torch.float32) / self.C))
        positions = torch.arange(T - 1, -T, -1, dtype=torch.float32)
        freqs = torch.outer(positions, inv_freq)
        table = torch.stack([freqs.sin(), freqs.cos()], dim=-1).reshape(freqs.size(0), self.C)
        P = table.size(0)
        table = torch.nn.functional.pad(table, (0, 0, 0, (P + 7) // 8 * 8 - P))
        out = table.to(self.dtype).to(self.device)             # (roundup8(2T-1), C)
        if len(self._tables) >= 16:
            self._tables.clear()
        self._tables[T] = out
        return out

    # ---- one layer; ``g`` is the geometry of the rows: padded (B, T, lens) or packed (cu, offsets) ----
    def _attention(self, lw, h: torch.Tensor, rel_table: torch.Tensor, g) -> torch.Tensor:
        C, H, D = self.C, self.H, self.D
        M = h.size(0)
        qkv4 = self._linear(h, *lw["qkv4"]).view(M, 4, H, D)                          # q+u | q+v | k | v of every row
        # projected positions; the table carries zero rows up to a multiple of 8 (the GEMM's column granule)
        Pp = rel_table.size(0)
        rel_k = OF.gemm(rel_table, lw["rel"])                                         # (Pp, H*D)
        # (q + v) against the projected table, one batched GEMM over heads with every row of the batch as a row; both
        # operands are read in place: head h of the projection is the column block h*D of its rows
        bd = fused.bmm_strided(qkv4[:, 1].permute(1, 0, 2), rel_k.view(Pp, H, D).permute(1, 0, 2))      # (H, M, Pp)
        chunk = self.right + 1
        left_chunks = self.left // chunk if self.left >= 0 else g["T"]
        # Transformer-XL shift, scale, chunked-limited window (and key padding) with a finite floor in one kernel
        if g["packed"]:
            bias = fused.relshift_bias_packed(bd, g["cu"], g["offsets"], g["bias_numel"], g["T"], D ** -0.5, chunk, left_chunks,
                                              MASK_FLOOR)
            out = fused.fmha_varlen_strided(qkv4[:, 0], qkv4[:, 2], qkv4[:, 3], g["cu"], g["T"], D ** -0.5, bias, g["offsets"])
        else:
            B, T = g["B"], g["T"]
            bias = fused.relshift_bias(bd.view(H, B, T, Pp).permute(1, 0, 2, 3), g["lens"], T, D ** -0.5, chunk, left_chunks,
                                       MASK_FLOOR)
            q5 = qkv4.view(B, T, 4, H, D)
            qu, k, v = (q5[:, :, i].permute(0, 2, 1, 3) for i in (0, 2, 3))           # (B, H, T, D) views
            # Keys at or past a stream's length carry the floor in the bias, whose softmax weight is exactly zero beside
            # any visible key, so bounding the key range by the length only skips work
            out = fmha(qu, k, v, softmax_scale=D ** -0.5, attn_bias=bias, cache_seqlens=g["lens"], token_major=True)
        return self._linear(out.view(M, C), *lw["o"])

    def _conv(self, lw, h: torch.Tensor, g) -> torch.Tensor:
        x = self._linear(h, *lw["pw1"], glu=True)                                     # pointwise_conv1 + GLU
        if g["packed"]:
            x = fused.depthwise_conv1d_packed_causal(x, lw["dw"][0], lw["dw"][1], g["cu"], g["T"])
        else:
            x = OF.depthwise_conv1d(x.view(g["B"], g["T"], self.C), lw["dw"][0], lw["dw"][1], padding=(self.K - 1, 0))
        x = OF.layer_norm_activation(x.view(-1, self.C), *lw["conv_norm"], eps=1e-5, activation_type=_SWISH)
        return self._linear(x, *lw["pw2"])

    def _layers(self, rows: torch.Tensor, g) -> torch.Tensor:
        """``rows (M, C)`` post-subsampling states (fp32 or the model's 16-bit type) -> ``(M, C)`` fp32 output of the stack."""
        if self.native and g["packed"] and rows.dtype in (torch.float32, self.dtype):
            return self._layers_native(rows.contiguous(), g)        # one call: 16-bit or 8-bit Linear GEMMs
        return self._layers_composed(rows.to(torch.float32, copy=True).contiguous(), g)   # own copy: updated in place

    def _layers_composed(self, res: torch.Tensor, g) -> torch.Tensor:
        """The stack operator by operator from Python: padded batches, and the check of the native executor (same
        kernels, same order, so bit-identical results, with 16-bit and with 8-bit Linear GEMMs)."""
        M, C = res.shape
        rel_table = self._position_table(g["T"])
        h = torch.empty(M, C, device=res.device, dtype=self.dtype)
        first = self.layers[0]["norm_feed_forward1"]
        fused.add_norm_f32(h, None, res, None, 0.0, fused.ADD_NORM_LN, *first, eps=self.eps)          # LN(x)
        out = None
        for i, lw in enumerate(self.layers):
            w1, b1, w2, b2 = lw["feed_forward1"]
            y = self._linear(self._linear(h, w1, b1, _SWISH), w2, b2)
            fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN, *lw["norm_self_att"], eps=self.eps)
            y = self._attention(lw, h, rel_table, g)
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_LN, *lw["norm_conv"], eps=self.eps)
            y = self._conv(lw, h, g)
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_LN, *lw["norm_feed_forward2"], eps=self.eps)
            w1, b1, w2, b2 = lw["feed_forward2"]
            y = self._linear(self._linear(h, w1, b1, _SWISH), w2, b2)
            if i + 1 < self.L:
                # norm_out of this layer is the next layer's input; its norm_feed_forward1 follows at once
                nxt = self.layers[i + 1]["norm_feed_forward1"]
                fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_out"], *nxt, eps=self.eps)
            else:
                out = torch.empty(M, C, device=res.device, dtype=torch.float32)
                fused.add_norm_f32(h, out, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_out"], *lw["norm_out"], eps=self.eps)
        return out

    # ---- streaming: one chunk of B streams over paged keys / values and cached conv tails ----
    def new_streaming_cache(self, max_streams: int, chunk_frames: int = 16, block_size: int = 16, seed=0):
        """Page pools, block table and conv-tail buffers for ``max_streams`` concurrent streams.  The cached history is
        capped at the trained left context rounded up to whole pages."""
        from .streaming import StreamingCache

        chunk = self.right + 1
        if chunk_frames % chunk:
            raise ValueError(f"a streaming step must be a whole number of trained attention chunks ({chunk} frames)")
        max_past = (max(self.left, 0) + block_size - 1) // block_size * block_size
        return StreamingCache(self.L, self.H, self.D, self.C, self.K, max_streams, max_past, chunk_frames, block_size,
                              self.device, self.dtype, seed)

    def _stream_rel_k(self, i: int, lmax: int) -> torch.Tensor:
        """``relative_k_proj`` of the sinusoid table for ``lmax`` key positions, layer ``i``: constant per cache geometry."""
        key = (i, lmax)
        hit = self._stream_tables.get(key)
        if hit is None:
            hit = OF.gemm(self._position_table(lmax), self.layers[i]["rel"])          # (roundup8(2*lmax-1), C)
            self._stream_tables[key] = hit
        return hit

    def forward_chunk(self, hidden: torch.Tensor, slots, cache) -> torch.Tensor:
        """One streaming step: ``hidden (B, T_q, C)`` post-subsampling states of the streams in ``slots`` ->
        ``(B, T_q, C)`` fp32, the layer stack of NemotronEncoder.forward_chunk_paged
        (oasr/models/nemotron/encoder.py:269-298, 362-410, 585-720).  Keys / values of the chunk are appended to the
        streams' pages, attention runs over cached frames + chunk with the Transformer-XL bias at the true
        distances and the chunked-limited window over absolute frame positions, and the conv module continues from
        each stream's post-GLU tail.  ``cache`` comes from :meth:`new_streaming_cache`; only real frames are cached
        (the reference's prefilled placeholders are masked keys, which contribute nothing)."""
        import ctypes

        from . import _lib
        from .cache import write_kv_chunk
        from .functional import _DTYPE_ID, _p, _stream

        if not hidden.is_cuda:
            raise RuntimeError("hidden must be a CUDA tensor (oasr_b200 has no CPU path)")
        B, Tq, C = hidden.shape
        slots = list(slots)
        if Tq != cache.chunk or len(slots) != B:
            raise RuntimeError(f"expected {len(slots)} streams x {cache.chunk} frames, got {B} x {Tq}")
        H, D, SL = self.H, self.D, self.K - 1
        table, cached, total, pos_start, slot_ids = cache.prepare(slots)
        offsets = pos_start + cached                                   # encoder frames emitted before this chunk
        lmax = cache.max_past + Tq
        tk = table.size(1) * cache.block_size
        chunk = self.right + 1
        left_chunks = self.left // chunk if self.left >= 0 else lmax
        M = B * Tq
        res = hidden.reshape(M, C).to(torch.float32, copy=True).contiguous()
        h = torch.empty(M, C, device=res.device, dtype=self.dtype)
        fused.add_norm_f32(h, None, res, None, 0.0, fused.ADD_NORM_LN, *self.layers[0]["norm_feed_forward1"], eps=self.eps)
        out = None
        for i, lw in enumerate(self.layers):
            w1, b1, w2, b2 = lw["feed_forward1"]
            y = self._linear(self._linear(h, w1, b1, _SWISH), w2, b2)
            fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN, *lw["norm_self_att"], eps=self.eps)
            # --- attention over [cached pages ; chunk] ---
            qkv4 = self._linear(h, *lw["qkv4"]).view(B, Tq, 4, H, D)
            write_kv_chunk(cache.k_pool[i], cache.v_pool[i], table, qkv4[:, :, 2].permute(0, 2, 1, 3),
                           qkv4[:, :, 3].permute(0, 2, 1, 3), cached)
            rel_k = self._stream_rel_k(i, lmax)
            Pp = rel_k.size(0)
            bd = fused.bmm_strided(qkv4.view(M, 4, H, D)[:, 1].permute(1, 0, 2), rel_k.view(Pp, H, D).permute(1, 0, 2))   # (H, M, Pp)
            bias = torch.empty(B, H, Tq, tk, device=res.device, dtype=self.dtype)
            _lib.call("oasr_b200_relshift_bias_stream", _p(bias), _p(bd), _p(cached), _p(offsets), B, H, Tq, Pp, tk, lmax,
                      bd.stride(0), D ** -0.5, chunk, left_chunks, MASK_FLOOR, _DTYPE_ID[self.dtype], _stream(bd))
            att = fmha(qkv4[:, :, 0].permute(0, 2, 1, 3), cache.k_pool[i], cache.v_pool[i], softmax_scale=D ** -0.5,
                       attn_bias=bias, cache_seqlens=total, block_table=table, token_major=True)
            y = self._linear(att.reshape(M, C), *lw["o"])
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_LN, *lw["norm_conv"], eps=self.eps)
            # --- conv module continuing from the stream's post-GLU tail ---
            g = self._linear(h, *lw["pw1"], glu=True)
            xcat = torch.empty(B, SL + Tq, C, device=res.device, dtype=self.dtype)
            _lib.call("oasr_b200_conv_state_concat", _p(xcat), ctypes.c_void_p(cache.cnn_state[i].data_ptr()), cache.max_streams,
                      _p(slot_ids), _p(g), B, SL, Tq, C, _DTYPE_ID[self.dtype], _stream(g))
            x = OF.depthwise_conv1d(xcat, lw["dw"][0], lw["dw"][1], padding=0)        # valid conv: (B, Tq, C)
            x = OF.layer_norm_activation(x.reshape(M, C), *lw["conv_norm"], eps=1e-5, activation_type=_SWISH)
            y = self._linear(x, *lw["pw2"])
            fused.add_norm_f32(h, res, res, y, 1.0, fused.ADD_NORM_LN, *lw["norm_feed_forward2"], eps=self.eps)
            w1, b1, w2, b2 = lw["feed_forward2"]
            y = self._linear(self._linear(h, w1, b1, _SWISH), w2, b2)
            if i + 1 < self.L:
                nxt = self.layers[i + 1]["norm_feed_forward1"]
                fused.add_norm_f32(h, res, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_out"], *nxt, eps=self.eps)
            else:
                out = torch.empty(M, C, device=res.device, dtype=torch.float32)
                fused.add_norm_f32(h, out, res, y, 0.5, fused.ADD_NORM_LN_LN, *lw["norm_out"], *lw["norm_out"], eps=self.eps)
        cache.commit(slots)
        return out.view(B, Tq, C)

    def forward(self, hidden: torch.Tensor, lengths: List[int], packed: bool = True) -> torch.Tensor:
        """``hidden (B, T, C)`` post-subsampling states, host ``lengths`` -> ``(B, T, C)`` fp32: the output of the
        layer stack of NemotronEncoder.forward (encoder.py:542-583) on frames ``t < lengths[b]``.

        ``packed`` (default) runs the stack on the valid frames only - the rows of all streams back to back, attention
        and the causal conv per segment - and returns zeros in the padding frames; ``packed=False`` runs the padded
        batch as the reference does.  Either way frames past a stream's length are unspecified relative to the
        reference: it zero-fills attention rows that see no key (encoder.py:343-348), which are always padding frames (a
        valid frame sees at least itself), and no valid frame reads a padding frame - attention masks them as keys,
        the convolution is causal, everything else is per frame."""
        if not hidden.is_cuda:
            raise RuntimeError("hidden must be a CUDA tensor (oasr_b200 has no CPU path)")
        B, T, C = hidden.shape
        lengths = [min(max(int(n), 0), T) for n in lengths]
        if len(lengths) != B:
            raise ValueError("one length per stream")
        dev = hidden.device
        if not packed:
            g = {"packed": False, "B": B, "T": T,
                 "lens": torch.tensor(lengths, dtype=torch.int32).to(dev, non_blocking=True)}
            res = hidden.reshape(B * T, C).to(torch.float32, copy=True).contiguous()   # own copy: updated in place
            return self._layers(res, g).view(B, T, C)
        out = torch.zeros(B * T, C, device=dev, dtype=torch.float32)
        rows, rows_dev = self.forward_rows(hidden, lengths)
        if rows is not None:
            from .cache import scatter_rows

            scatter_rows(out, rows_dev, rows)
        return out.view(B, T, C)

    def forward_rows(self, hidden: torch.Tensor, lengths: List[int]):
        """The stack on the valid frames only: ``(rows (total, C) fp32, row_index (total,) int64)`` with
        ``row_index[r] = b * T + t`` of packed row r; ``(None, None)`` for a batch without a valid frame."""
        B, T, C = hidden.shape
        dev = hidden.device
        lengths = [min(max(int(n), 0), T) for n in lengths]
        total = sum(lengths)
        if total == 0:
            return None, None
        lens = np.asarray(lengths, dtype=np.int64)
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(lens, out=cu[1:])
        # packed row r of stream b sits at padded row b*T + (r - cu[b])
        rows = np.arange(total, dtype=np.int64) + np.repeat(np.arange(B, dtype=np.int64) * T - cu[:-1], lens)
        # bias segment b: (H, len, roundup8(len)) elements, back to back
        offsets = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(self.H * lens * ((lens + 7) // 8 * 8), out=offsets[1:])
        g = {"packed": True, "T": int(lens.max()), "bias_numel": int(offsets[-1]),
             "cu": torch.from_numpy(cu.astype(np.int32)).to(dev, non_blocking=True),
             "offsets": torch.from_numpy(offsets).to(dev, non_blocking=True)}
        rows_dev = torch.from_numpy(rows).to(dev, non_blocking=True)
        from .cache import gather_rows

        rows = gather_rows(hidden.reshape(B * T, C), rows_dev)                          # (total, C), the input's dtype
        return self._layers(rows, g), rows_dev


class FastConformerEncoder:
    """``NemotronEncoder.forward`` (oasr/models/nemotron/encoder.py:542-583, ``scale_input`` False): mel features
    ``(B, T, mels)`` with host lengths -> ``(hidden (B, T', C) fp32, out_lengths)``.  Takes the reference's state-dict
    names (``subsampling.conv_in.weight``, ``subsampling.layers.N.depthwise_conv.weight``, ``layers.N...``)."""

    def __init__(self, hidden: int, heads: int, ffn: int, layers: int, kernel: int, sliding_window: int, lookahead: int,
                 mels: int, sub_channels: int, params: Dict[str, torch.Tensor], device="cuda",
                 dtype: torch.dtype = torch.bfloat16, stages: int = 3):
        self.stack = FastConformerLayers(hidden, heads, ffn, layers, kernel, sliding_window, lookahead, params, device, dtype)
        self.device, self.dtype, self.stages, self.Cs = torch.device(device), dtype, stages, sub_channels
        self.mels = mels
        w = lambda t: t.detach().to(torch.float32).to(dtype).to(self.device).contiguous()
        f = lambda t: t.detach().to(torch.float32).to(self.device).contiguous()
        s = "subsampling."
        self.conv_in = (f(params[s + "conv_in.weight"].reshape(sub_channels, 3, 3)), f(params[s + "conv_in.bias"]))
        self.sub_stages = []
        for i in range(stages - 1):
            p = f"{s}layers.{i}."
            self.sub_stages.append((w(params[p + "depthwise_conv.weight"].reshape(sub_channels, 3, 3)),
                                    w(params[p + "depthwise_conv.bias"]),
                                    w(params[p + "pointwise_conv.weight"].reshape(sub_channels, sub_channels)),
                                    w(params[p + "pointwise_conv.bias"])))
        self.proj = (w(params[s + "linear.weight"]), w(params[s + "linear.bias"]))
        # optional CTC projection (CtcProjection, oasr/layers/ctc.py:48-51) with its input at close to fp32 precision:
        # rows arrive as two 16-bit terms [h_hi | h_lo] and meet the 16-bit weight twice, [W | W]
        self.ctc = None
        if "ctc.ctc_lo.weight" in params:
            cw = params["ctc.ctc_lo.weight"].detach().float()
            self.ctc = (w(torch.cat([cw, cw], dim=1)), w(params["ctc.ctc_lo.bias"]))
            self._one, self._zero = f(torch.ones(hidden)), f(torch.zeros(hidden))

    def subsample(self, feats: torch.Tensor, lengths: List[int]):
        """Frames at or past a row's valid length are never zeroed in memory: every consumer reads them as zeros
        (``in_len`` of the depthwise conv) or ignores them, so valid frames equal the reference's, padded frames differ."""
        B = feats.size(0)
        nxt = lambda ls: [(n + 2 + 1 - 3) // 2 + 1 for n in ls]
        dev_i32 = lambda ls: torch.tensor(ls, dtype=torch.int32).to(self.device, non_blocking=True)
        # stem: one input channel, pad (2, 1) on time and frequency, 3x3 / stride 2, + bias + ReLU (fp32 in, 16-bit NHWC out)
        # (frames past a stream's length are not computed: the next stage reads them as zeros through its ``in_len``)
        lengths = nxt(lengths)
        x = fused.subsample_conv1(torch.nn.functional.pad(feats.float(), (2, 1, 2, 1)), *self.conv_in, self.dtype,
                                  t1_limit=dev_i32(lengths))
        for dw_w, dw_b, pw_w, pw_b in self.sub_stages:
            in_len, lengths = lengths, nxt(lengths)
            x = fused.depthwise_conv2d_k3s2(x, dw_w, dw_b, 2, 1, out_len=dev_i32(lengths), in_len=dev_i32(in_len))
            _, T, Fd, C = x.shape
            x = OF.gemm_activation(x.view(B * T * Fd, C), pw_w, pw_b, 0).view(B, T, Fd, C)   # pointwise conv + ReLU
        B, T, Fd, C = x.shape
        return OF.gemm(x.reshape(B * T, Fd * C), *self.proj).view(B, T, -1), lengths

    def forward(self, feats: torch.Tensor, lengths: List[int], packed: bool = True):
        if not feats.is_cuda:
            raise RuntimeError("feats must be a CUDA tensor (oasr_b200 has no CPU path)")
        hidden, out_len = self.subsample(feats, [int(n) for n in lengths])
        return self.stack.forward(hidden, out_len, packed=packed), out_len

    # ------------------------------------------------------------------ streaming
    def new_streaming_cache(self, max_streams: int, chunk_frames: int = 16, block_size: int = 16, seed=0):
        """The layer stack's cache plus, per subsampling stage, each stream's last two input frames (``kernel - 1``:
        NemotronSubsampling.state_specs, oasr/models/nemotron/subsampling.py:130-154): the stem keeps raw fp32 feature
        frames ``(2, mels)``, every later stage 16-bit NHWC frames ``(2, bins * channels)``, all before frequency padding."""
        cache = self.stack.new_streaming_cache(max_streams, chunk_frames, block_size, seed)
        bins = self.mels
        cache.extra_state.append(torch.zeros(max_streams, 2, bins, device=self.device, dtype=torch.float32))
        for _ in range(self.stages - 1):
            bins = (bins + 3 - 3) // 2 + 1
            cache.extra_state.append(torch.zeros(max_streams, 2, bins * self.Cs, device=self.device, dtype=self.dtype))
        return cache

    def _stage_input(self, x: torch.Tensor, state: torch.Tensor, slot_ids: torch.Tensor) -> torch.Tensor:
        """``[cached two frames ; x]`` per stream, and the stream's cache set to the last two frames of that
        concatenation (NemotronSubsampling._stage_input, subsampling.py:178-189): ``x (B, T, W)`` -> ``(B, T + 2, W)``."""
        import ctypes

        from . import _lib
        from .functional import _DTYPE_ID, _p, _stream

        B, T, W = x.shape
        xcat = torch.empty(B, T + 2, W, device=x.device, dtype=x.dtype)
        _lib.call("oasr_b200_conv_state_concat", _p(xcat), ctypes.c_void_p(state.data_ptr()), state.size(0), _p(slot_ids),
                  _p(x), B, 2, T, W, _DTYPE_ID[x.dtype], _stream(x))
        return xcat

    def subsample_chunk(self, feats: torch.Tensor, slot_ids: torch.Tensor, cache) -> torch.Tensor:
        """NemotronSubsampling.forward_chunk (subsampling.py:156-176): ``feats (B, T, mels)``, ``T`` a multiple of 8,
        of the streams in ``slot_ids`` -> ``(B, T / 8, hidden)``.  Every stage reads its cached two frames in place of
        the offline pass's zero padding on the left and has no padding on the right; no length masks (every frame of a
        streaming chunk is real audio)."""
        B, T, mels = feats.shape
        if T % (1 << self.stages) or mels != self.mels:
            raise RuntimeError(f"a streaming chunk is (B, multiple of {1 << self.stages}, {self.mels}) feature frames, got {tuple(feats.shape)}")
        x = self._stage_input(feats.float().contiguous(), cache.extra_state[0], slot_ids)          # (B, T + 2, mels) fp32
        x = fused.subsample_conv1(torch.nn.functional.pad(x, (2, 1)), *self.conv_in, self.dtype)    # (B, T / 2, F1, Cs)
        for i, (dw_w, dw_b, pw_w, pw_b) in enumerate(self.sub_stages, start=1):
            _, Ti, Fd, C = x.shape
            x = self._stage_input(x.view(B, Ti, Fd * C), cache.extra_state[i], slot_ids).view(B, Ti + 2, Fd, C)
            x = fused.depthwise_conv2d_k3s2(x, dw_w, dw_b, 2, 1, time_pad=(0, 0))
            _, To, Fo, C = x.shape
            x = OF.gemm_activation(x.view(B * To * Fo, C), pw_w, pw_b, 0).view(B, To, Fo, C)
        B, To, Fo, C = x.shape
        return OF.gemm(x.reshape(B * To, Fo * C), *self.proj).view(B, To, -1)

    def forward_chunk(self, feats: torch.Tensor, slots, cache) -> torch.Tensor:
        """One streaming step from feature frames: NemotronEncoder.forward_chunk_paged
        (oasr/models/nemotron/encoder.py:585-650, ``scale_input`` False).  ``feats (B, 8 * chunk, mels)`` of the streams
        in ``slots`` -> ``(B, chunk, hidden)`` fp32; ``cache`` from :meth:`new_streaming_cache`."""
        if not feats.is_cuda:
            raise RuntimeError("feats must be a CUDA tensor (oasr_b200 has no CPU path)")
        slots = list(slots)
        if feats.size(0) != len(slots) or feats.size(1) != cache.chunk << self.stages:
            raise RuntimeError(f"expected {len(slots)} streams x {cache.chunk << self.stages} feature frames, got {tuple(feats.shape[:2])}")
        slot_ids = torch.tensor(slots, dtype=torch.int64).to(self.device, non_blocking=True)
        return self.stack.forward_chunk(self.subsample_chunk(feats, slot_ids, cache), slots, cache)

    def forward_ctc(self, feats: torch.Tensor, lengths: List[int], padded_output: bool = True, return_argmax: bool = False):
        """Encoder + CTC head: ``(log_probs fp32, out_lengths[, argmax])``.  The head (fused GEMM + log-softmax with the
        per-frame argmax in its epilogue) runs on the valid frames only; with ``padded_output`` the log-probs come
        back ``(B, T', V)`` with padding frames holding ``log_softmax(bias)`` (a zero hidden row, as the reference's
        padded batch gives), else packed ``(total, V)``."""
        if self.ctc is None:
            raise RuntimeError("this encoder was built without a CTC projection (no 'ctc.ctc_lo.weight' in the parameters)")
        if not feats.is_cuda:
            raise RuntimeError("feats must be a CUDA tensor (oasr_b200 has no CPU path)")
        hidden, out_len = self.subsample(feats, [int(n) for n in lengths])
        B, T, C = hidden.shape
        V = self.ctc[0].size(0)
        rows, rows_dev = self.stack.forward_rows(hidden, out_len)
        if rows is None:
            lp = torch.zeros((B, T, V) if padded_output else (0, V), device=feats.device)
            return (lp, out_len, None) if return_argmax else (lp, out_len)
        h3 = torch.empty(rows.size(0), 2 * C, device=rows.device, dtype=self.dtype)
        fused.add_norm_f32(h3, None, rows, None, 0.0, fused.ADD_NORM_AFFINE, self._one, self._zero, eps=1e-5, split_out=True)
        lp, arg = OF.gemm_log_softmax(h3, self.ctc[0], self.ctc[1], out_dtype=torch.float32, return_argmax=True)
        if padded_output:
            full = torch.log_softmax(self.ctc[1].float(), dim=-1).expand(B * T, V).contiguous()
            from .cache import scatter_rows

            scatter_rows(full, rows_dev, lp)
            lp = full.view(B, T, V)
        return (lp, out_len, arg) if return_argmax else (lp, out_len)
