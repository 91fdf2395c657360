"""Fused building blocks of the encoder layer that have no single counterpart in the
reference's operator list: each one replaces a short chain of reference operators and torch
glue (cited per function) so that intermediates never reach HBM or are never rounded."""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .functional import _DTYPE_ID, _need_cuda, _p, _stream

ADD_NORM_LN, ADD_NORM_AFFINE, ADD_NORM_LN_LN = 0, 1, 2


def add_norm_f32(h_out: torch.Tensor, res_out: Optional[torch.Tensor], res_in: Optional[torch.Tensor],
                 y: Optional[torch.Tensor], alpha: float, mode: int, w_a, b_a, w_b=None, b_b=None,
                 eps: float = 1e-5, split_out: bool = False) -> None:
    """``s = res_in + alpha*y`` in fp32, then (mode 0) ``h = LN_a(s)``, (mode 1) ``h = s*w_a + b_a``
    with fp32 per-channel ``w_a/b_a``, or (mode 2) ``res_out = LN_a(s); h = LN_b(res_out)``.
    With ``split_out`` the rows of ``h_out`` are ``2*hidden`` wide: ``[hi | lo]``, ``h = hi + lo``.
    The ``x = residual + alpha*sub(x)`` / ``norm(x)`` pairs of ConformerEncoderLayer.forward_packed
    (oasr/models/conformer/model.py:722-751) with an fp32 residual stream."""
    _need_cuda(h_out, res_out, res_in, y)
    hidden = h_out.size(-1) // (2 if split_out else 1)
    rows = h_out.numel() // h_out.size(-1)
    _lib.call("oasr_b200_add_norm_f32", _p(h_out), _p(res_out), _p(res_in), _p(y), float(alpha), int(mode), _p(w_a),
              _p(b_a), _p(w_b), _p(b_b), rows, hidden, float(eps), int(bool(split_out)), _DTYPE_ID[h_out.dtype],
              _stream(h_out))


def add_norm_f32_q8(h_out: torch.Tensor, res_out: Optional[torch.Tensor], res_in: Optional[torch.Tensor],
                    y: Optional[torch.Tensor], alpha: float, mode: int, w_a, b_a, w_b=None, b_b=None,
                    eps: float = 1e-5, kind: int = 1):
    """:func:`add_norm_f32` that also returns the rows of ``h`` in 8 bits for a following 8-bit GEMM:
    ``(q uint8 (rows, hidden), scale fp32 (rows,))``, bit for bit what ``quant.quantize_rows(h_out, kind)`` gives
    (``kind`` 1 = fp8 e4m3, 2 = int8), without the separate quantisation launch."""
    _need_cuda(h_out, res_out, res_in, y)
    hidden = h_out.size(-1)
    rows = h_out.numel() // hidden
    q = torch.empty(rows, hidden, dtype=torch.uint8, device=h_out.device)
    scale = torch.empty(rows, dtype=torch.float32, device=h_out.device)
    _lib.call("oasr_b200_add_norm_f32_q8", _p(h_out), _p(res_out), _p(res_in), _p(y), float(alpha), int(mode), _p(w_a),
              _p(b_a), _p(w_b), _p(b_b), rows, hidden, float(eps), 0, _p(q), _p(scale), int(kind), _DTYPE_ID[h_out.dtype],
              _stream(h_out))
    return q, scale


def gemm_dup_first(A: torch.Tensor, B: torch.Tensor, bias: Optional[torch.Tensor], dup_cols: int,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``A (M, K) @ B (N, K).T`` with the first ``dup_cols`` output columns stored twice: the result is ``(M, N +
    dup_cols)``, columns ``[0, dup)`` and ``[dup, 2*dup)`` both hold the first block of the product, the rest follows;
    ``bias`` (``N + dup_cols`` entries) is added per OUTPUT column.  Equal, bit for bit, to ``gemm`` against ``B`` with
    its first ``dup_cols`` rows repeated -- the fused q/q/k/v projection of the relative-position attention
    (oasr/layers/attention/attention.py:323-386: q+u and q+v differ only in their bias) at 3/4 of the products."""
    _need_cuda(A, B, bias, out)
    M, K = A.shape
    N = B.size(0)
    if out is None:
        out = torch.empty(M, N + dup_cols, device=A.device, dtype=A.dtype)
    _lib.call("oasr_b200_gemm_dup_first", _p(out), _p(A), _p(B), _p(bias), M, N, K, int(dup_cols), _DTYPE_ID[A.dtype], _stream(A))
    return out


def gemm_add_norm_f32(h_out: torch.Tensor, res_out: Optional[torch.Tensor], res_in: Optional[torch.Tensor],
                      A: torch.Tensor, B: torch.Tensor, bias: Optional[torch.Tensor], alpha: float, mode: int, w_a, b_a,
                      w_b=None, b_b=None, eps: float = 1e-5, split_out: bool = False) -> None:
    """``add_norm_f32`` with the sub-layer's last Linear folded in: ``y = A @ B.T + bias`` stays fp32 in tensor
    memory, ``s = res_in + alpha*y``, then the norm of ``mode`` as in :func:`add_norm_f32`.  One kernel instead of
    ``gemm`` + ``add_layer_norm_residual`` (oasr/models/conformer/model.py:722-751); needs an output width of
    128, 256 or 512.  ``res_in`` / ``res_out`` are fp32 buffers in the kernel's blocked layout
    (:func:`residual_to_blocked`), ``roundup32(M) * N`` floats."""
    _need_cuda(h_out, res_out, res_in, A, B, bias)
    K, N = A.shape[-1], B.shape[0]
    M = A.numel() // K
    _lib.call("oasr_b200_gemm_add_norm_f32", _p(h_out), _p(res_out), _p(res_in), _p(A), _p(B), _p(bias), M, N, K,
              float(alpha), int(mode), _p(w_a), _p(b_a), _p(w_b), _p(b_b), float(eps), int(bool(split_out)),
              _DTYPE_ID[A.dtype], _stream(A))


def residual_to_blocked(res: torch.Tensor) -> torch.Tensor:
    """Row-major fp32 ``(M, N)`` -> the blocked residual layout of :func:`gemm_add_norm_f32`: rows padded to a
    multiple of 32, 32 x 32 blocks band-major, element (row l, column 4j+e) of a block at ``(j*32 + l)*4 + e``."""
    M, N = res.shape
    Mp = (M + 31) // 32 * 32
    padded = torch.zeros(Mp, N, device=res.device, dtype=torch.float32)
    padded[:M] = res
    return padded.view(Mp // 32, 32, N // 32, 8, 4).permute(0, 2, 3, 1, 4).contiguous().view(-1)


def residual_from_blocked(blocked: torch.Tensor, M: int, N: int) -> torch.Tensor:
    """Inverse of :func:`residual_to_blocked`: the first ``M`` rows as a row-major ``(M, N)`` tensor."""
    Mp = (M + 31) // 32 * 32
    return blocked.view(Mp // 32, N // 32, 8, 32, 4).permute(0, 3, 1, 2, 4).reshape(Mp, N)[:M].contiguous()


def depthwise_conv1d_packed(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                            cu_seqlens: torch.Tensor, max_seg_len: int, *, post_scale=None, post_shift=None,
                            right_fill=None, fill_frames=None, activation: int = -1, out=None) -> torch.Tensor:
    """Depthwise conv over packed ``(total, C)`` rows, every ``cu_seqlens`` segment alone, optional
    folded BatchNorm (``post_scale/post_shift`` fp32) and activation: the gapped scatter / conv /
    gather / BatchNorm+swish of ConvolutionModule._forward_packed_noncausal
    (oasr/models/conformer/model.py:223-233) in one kernel."""
    _need_cuda(x, weight, bias, cu_seqlens)
    if out is None:
        out = torch.empty_like(x)
    K = weight.size(0)
    _lib.call("oasr_b200_depthwise_conv1d_packed", _p(out), _p(x), _p(weight), _p(bias), _p(post_scale),
              _p(post_shift), _p(right_fill), _p(fill_frames), _p(cu_seqlens), cu_seqlens.numel() - 1,
              int(max_seg_len), x.size(-1), K, int(activation), _DTYPE_ID[x.dtype], _stream(x))
    return out


def depthwise_conv1d_packed_causal(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                                   cu_seqlens: torch.Tensor, max_seg_len: int, activation: int = -1) -> torch.Tensor:
    """Causal depthwise conv over packed ``(total, C)`` rows, ``weight (K, C)``: frame t of a segment reads frames
    ``t-K+1 .. t`` of the same segment (zeros before its start)."""
    _need_cuda(x, weight, bias, cu_seqlens)
    out = torch.empty_like(x)
    _lib.call("oasr_b200_depthwise_conv1d_packed_causal", _p(out), _p(x), _p(weight), _p(bias), _p(cu_seqlens),
              cu_seqlens.numel() - 1, int(max_seg_len), x.size(-1), weight.size(0), int(activation), _DTYPE_ID[x.dtype],
              _stream(x))
    return out


def fmha_relpos_plan(cu_seqlens: torch.Tensor, heads: int, total: int) -> torch.Tensor:
    """Work list for :func:`fmha_varlen_relpos` (``plan=``): the (segment, head, query tile) items of a packed batch,
    longest segments first, built on the device from ``cu_seqlens``; at most 1024 segments.  Build once per batch."""
    _need_cuda(cu_seqlens)
    S = cu_seqlens.numel() - 1
    nbytes = int(_lib.load().oasr_b200_fmha_relpos_plan_bytes(S, heads, int(total)))
    plan = torch.empty((nbytes + 15) // 16 * 4, device=cu_seqlens.device, dtype=torch.int32)
    _lib.call("oasr_b200_fmha_relpos_plan", _p(plan), plan.numel() * 4, _p(cu_seqlens), S, heads, int(total), _stream(cu_seqlens))
    return plan


def fmha_varlen_relpos(qkv4: torch.Tensor, pos: torch.Tensor, cu_seqlens: torch.Tensor, max_seg_len: int,
                       heads: int, scale: float, out=None, plan: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Conformer relative-position attention over packed rows
    (RelPositionMultiHeadedAttention._forward_packed, oasr/layers/attention/attention.py:323-386).
    ``qkv4`` ``(total, 4*d)`` = ``[q+u | q+v | k | v]``; ``pos`` = ``linear_pos(pe)[:>=max_seg_len]``
    as a ``(rows, d)`` view with unit inner stride; returns ``(total, d)``.  ``plan`` (from :func:`fmha_relpos_plan`)
    makes the persistent kernel walk the longest segments first; the result does not depend on it."""
    _need_cuda(qkv4, pos, cu_seqlens, plan)
    total, d4 = qkv4.shape
    d = d4 // 4
    if out is None:
        out = torch.empty(total, d, device=qkv4.device, dtype=qkv4.dtype)
    if pos.stride(1) != 1:
        raise ValueError("pos must have unit stride along the feature axis")
    _lib.call("oasr_b200_fmha_varlen_relpos_planned", _p(out), _p(qkv4), _p(pos), pos.size(0), pos.stride(0), _p(cu_seqlens),
              cu_seqlens.numel() - 1, int(max_seg_len), total, heads, float(scale), _p(plan), _DTYPE_ID[qkv4.dtype],
              _stream(qkv4))
    return out


def subsample_conv1(feats: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype,
                    kernel: int = 3, stride: int = 2, t1_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First Conv2d + ReLU of the subsampling stack: fp32 ``(B, T, F)`` features in, 16-bit NHWC
    ``(B, T1, F1, C)`` out; ``weight`` ``(C, k, k)`` and ``bias`` ``(C,)`` fp32
    (oasr/models/conformer/model.py:433-444)."""
    _need_cuda(feats, weight, bias, t1_limit)
    if feats.dtype != torch.float32 or weight.dtype != torch.float32 or bias.dtype != torch.float32:
        raise RuntimeError("subsample_conv1 takes fp32 features, weight and bias")
    feats = feats.contiguous()
    B, T, Fd = feats.shape
    C = weight.size(0)
    T1, F1 = (T - kernel) // stride + 1, (Fd - kernel) // stride + 1
    out = torch.empty(B, T1, F1, C, device=feats.device, dtype=out_dtype)
    _lib.call("oasr_b200_subsample_conv1", _p(out), _p(feats), _p(weight.contiguous()), _p(bias.contiguous()),
              _p(t1_limit), B, T, Fd, C, kernel, stride, _DTYPE_ID[out_dtype], _stream(feats))
    return out


def subsample_conv1_s2d(feats: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, out_dtype: torch.dtype,
                        t1_limit: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First Conv2d (3x3, stride 2) + ReLU written in the parity-split layout ``subsample_conv2`` reads:
    ``(B, ceil(T1/2), 4, ceil(F1/2), C)``, plane ``(t1 & 1) * 2 + (f1 & 1)``, rows ``(t1 // 2, f1 // 2)``.
    Positions that no frame below ``t1_limit[b]`` needs stay unwritten."""
    _need_cuda(feats, weight, bias, t1_limit)
    if feats.dtype != torch.float32 or weight.dtype != torch.float32 or bias.dtype != torch.float32:
        raise RuntimeError("subsample_conv1_s2d takes fp32 features, weight and bias")
    feats = feats.contiguous()
    B, T, Fd = feats.shape
    C = weight.size(0)
    T1, F1 = (T - 3) // 2 + 1, (Fd - 3) // 2 + 1
    out = torch.empty(B, (T1 + 1) // 2, 4, (F1 + 1) // 2, C, device=feats.device, dtype=out_dtype)
    _lib.call("oasr_b200_subsample_conv1_s2d", _p(out), _p(feats), _p(weight.contiguous()), _p(bias.contiguous()),
              _p(t1_limit), B, T, Fd, C, _DTYPE_ID[out_dtype], _stream(feats))
    return out


def subsample_conv2(x1: torch.Tensor, T1: int, F1: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                    cu_frames: torch.Tensor, total_frames: int) -> torch.Tensor:
    """Second Conv2d (3x3, stride 2) + bias + ReLU of the subsampling stack on the tensor cores, valid
    output frames only and already packed: ``x1`` from ``subsample_conv1_s2d``; ``weight (N, 3, 3, C)``
    (taps outermost, input channels innermost); ``cu_frames (B+1,) int32`` packed frame offsets.
    Returns ``(total_frames, F2 * N)`` rows in ``(f, c)`` order (oasr/models/conformer/model.py:445-449
    followed by pack_hidden, packing.py:204-216)."""
    _need_cuda(x1, weight, bias, cu_frames)
    B, C = x1.size(0), x1.size(-1)
    N = weight.size(0)
    F2 = (F1 - 3) // 2 + 1
    out = torch.empty(total_frames, F2 * N, device=x1.device, dtype=x1.dtype)
    _lib.call("oasr_b200_subsample_conv2", _p(out), _p(x1), _p(weight), _p(bias), _p(cu_frames), B, T1, F1, C, N,
              total_frames, _DTYPE_ID[x1.dtype], _stream(x1))
    return out


def fmha_paged_relpos(qkv4: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, pos: torch.Tensor,
                      pos_start: torch.Tensor, block_table: torch.Tensor, seqlens: torch.Tensor, heads: int,
                      scale: float, out=None) -> torch.Tensor:
    """Relative-position attention of the new frames of ``B`` streams over their paged history
    (RelPositionMultiHeadedAttention.forward_paged, oasr/layers/attention/attention.py:388-470).
    ``qkv4 (B, Tq, 4*d)`` = ``[q+u | q+v | k | v]`` of the new frames (their k/v already written to the
    pages); pools ``(num_blocks, block_size, H, 64)``; ``pos (rows, d)`` = ``linear_pos(pe)``;
    ``pos_start (B,)`` = table row of each stream's key 0; ``seqlens (B,)`` = visible keys including the
    new frames.  Returns ``(B, Tq, d)``."""
    _need_cuda(qkv4, k_pool, v_pool, pos, block_table, seqlens, pos_start)
    B, Tq, d4 = qkv4.shape
    d = d4 // 4
    if out is None:
        out = torch.empty(B, Tq, d, device=qkv4.device, dtype=qkv4.dtype)
    if not qkv4.is_contiguous() or pos.stride(1) != 1:
        raise ValueError("qkv4 must be contiguous and pos must have unit stride along the feature axis")
    _lib.call("oasr_b200_fmha_paged_relpos", _p(out), _p(qkv4), _p(k_pool), _p(v_pool), _p(pos), pos.size(0),
              pos.stride(0), _p(pos_start), _p(block_table), _p(seqlens), B, Tq, heads, block_table.size(1),
              k_pool.size(1), k_pool.size(0), float(scale), _DTYPE_ID[qkv4.dtype], _stream(qkv4))
    return out


def fmha_paged_relpos_fp8(qkv4: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, k_scale: torch.Tensor,
                          v_scale: torch.Tensor, pos: torch.Tensor, pos_start: torch.Tensor, block_table: torch.Tensor,
                          seqlens: torch.Tensor, heads: int, scale: float, out=None) -> torch.Tensor:
    """``fmha_paged_relpos`` over fp8 pages: uint8 pools of e4m3 codes and per-head fp32 scales ``(H,)``."""
    _need_cuda(qkv4, k_pool, v_pool, k_scale, v_scale, pos, block_table, seqlens, pos_start)
    B, Tq, d4 = qkv4.shape
    d = d4 // 4
    if out is None:
        out = torch.empty(B, Tq, d, device=qkv4.device, dtype=qkv4.dtype)
    _lib.call("oasr_b200_fmha_paged_relpos_fp8", _p(out), _p(qkv4), _p(k_pool), _p(v_pool), _p(k_scale), _p(v_scale),
              _p(pos), pos.size(0), pos.stride(0), _p(pos_start), _p(block_table), _p(seqlens), B, Tq, heads,
              block_table.size(1), k_pool.size(1), k_pool.size(0), float(scale), _DTYPE_ID[qkv4.dtype], _stream(qkv4))
    return out


def paged_kv_write_fp8(k_pool: torch.Tensor, v_pool: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                       k_scale: torch.Tensor, v_scale: torch.Tensor, block_table: torch.Tensor,
                       offsets: torch.Tensor) -> None:
    """Quantising page write: ``k_new / v_new (B, H, T, D)`` 16-bit views (unit stride along D) -> e4m3 codes
    ``x / scale[h]`` in uint8 pools ``(num_blocks, block_size, H, D)`` at logical positions ``offsets[b] + t``."""
    _need_cuda(k_pool, v_pool, k_new, v_new, k_scale, v_scale, block_table, offsets)
    B, H, T, D = k_new.shape
    if k_new.stride() != v_new.stride() or k_new.stride(3) != 1:
        raise ValueError("k_new and v_new must share strides and have unit stride along D")
    sb, sh, st, _ = k_new.stride()
    _lib.call("oasr_b200_paged_kv_write_fp8", _p(k_pool), _p(v_pool), _p(k_new), _p(v_new), _p(k_scale), _p(v_scale),
              _p(block_table), _p(offsets), B, H, T, D, sb, sh, st, block_table.size(1), k_pool.size(1), k_pool.size(0),
              _DTYPE_ID[k_new.dtype], _stream(k_new))


def depthwise_conv2d_k3s2(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], pad_lo: int, pad_hi: int,
                          out_len: Optional[torch.Tensor] = None, in_len: Optional[torch.Tensor] = None,
                          time_pad: Optional[tuple] = None) -> torch.Tensor:
    """Depthwise 3x3 / stride-2 Conv2d on NHWC ``x (B, T, F, C)`` with ``pad_lo`` zeros before and ``pad_hi`` after on
    both axes (``time_pad = (lo, hi)`` overrides the time axis: ``(0, 0)`` for a streaming chunk that carries its own
    left context); ``weight (C, 3, 3)``; frames ``>= out_len[b]`` come out as zeros and input frames ``>= in_len[b]``
    are read as zeros (the per-stage time masks of oasr/models/nemotron/subsampling.py:26-31, applied at the consumer)."""
    _need_cuda(x, weight, bias, out_len, in_len)
    x = x.contiguous()
    B, T, Fd, C = x.shape
    tlo, thi = (pad_lo, pad_hi) if time_pad is None else (int(time_pad[0]), int(time_pad[1]))
    To, Fo = (T + tlo + thi - 3) // 2 + 1, (Fd + pad_lo + pad_hi - 3) // 2 + 1
    out = torch.empty(B, To, Fo, C, device=x.device, dtype=x.dtype)
    _lib.call("oasr_b200_depthwise_conv2d_k3s2", _p(out), _p(x), _p(weight.contiguous()), _p(bias), _p(out_len), _p(in_len), B, T, Fd,
              C, int(pad_lo), int(pad_hi), tlo, thi, _DTYPE_ID[x.dtype], _stream(x))
    return out


def relshift_bias_packed(bd: torch.Tensor, cu_seqlens: torch.Tensor, bias_offsets: torch.Tensor, bias_numel: int, T: int,
                         scale: float, chunk: int, left_chunks: int, floor_value: float = -1.0e4) -> torch.Tensor:
    """Packed ``relshift_bias``: ``bd (H, total, ld >= 2T-1)`` scores of packed rows -> flat block-diagonal bias, segment
    ``s`` = ``(H, len_s, roundup8(len_s))`` at ``bias_offsets[s]`` (int64, multiples of 8), ``bias_numel`` elements in all."""
    _need_cuda(bd, cu_seqlens, bias_offsets)
    H, total, ld = bd.shape
    if not bd.is_contiguous() or bias_offsets.dtype != torch.int64 or cu_seqlens.dtype != torch.int32:
        raise ValueError("bd must be contiguous (H, total, ld); cu_seqlens int32, bias_offsets int64")
    out = torch.empty(int(bias_numel), device=bd.device, dtype=bd.dtype)
    _lib.call("oasr_b200_relshift_bias_packed", _p(out), _p(bd), _p(cu_seqlens), _p(bias_offsets), cu_seqlens.numel() - 1, H,
              total, T, ld, float(scale), int(chunk), int(left_chunks), float(floor_value), _DTYPE_ID[bd.dtype], _stream(bd))
    return out


def fmha_varlen_strided(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_seg_len: int,
                        softmax_scale: float, bias: Optional[torch.Tensor] = None,
                        bias_offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Self-attention over packed segments with ``q/k/v (total, H, D)`` views whose rows may be strided (slices of one
    fused projection) and an optional block-diagonal bias whose segment rows are ``roundup8(len_s)`` apart.  Returns
    ``(total, H, D)`` contiguous."""
    _need_cuda(q, k, v, cu_seqlens, bias, bias_offsets)
    total, H, D = q.shape
    for t in (q, k, v):
        if t.shape != q.shape or t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError("q/k/v must be (total, H, D) views with unit stride along D and heads D apart")
    out = torch.empty(total, H, D, device=q.device, dtype=q.dtype)
    _lib.call("oasr_b200_fmha_varlen_strided", _p(out), _p(q), _p(k), _p(v), q.stride(0), k.stride(0), v.stride(0), _p(bias),
              _p(bias_offsets), 1, 1, _p(cu_seqlens), _p(cu_seqlens), cu_seqlens.numel() - 1, total, total, int(max_seg_len),
              H, H, D, float(softmax_scale), _DTYPE_ID[q.dtype], _stream(q))
    return out


def bmm_strided(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``out[i] = a[i] @ b[i]^T`` for views ``a (batch, M, K)``, ``b (batch, N, K)`` with unit stride along ``K`` and row /
    batch strides that are multiples of 8 elements: the operands are read in place (``oasr.bmm``,
    oasr/functionals/gemm.py:262-299, takes packed operands only)."""
    _need_cuda(a, b)
    if a.dim() != 3 or b.dim() != 3 or a.size(0) != b.size(0) or a.size(2) != b.size(2) or a.dtype != b.dtype:
        raise ValueError(f"bmm_strided: need (batch, M, K) and (batch, N, K); got {tuple(a.shape)}, {tuple(b.shape)}")
    if a.stride(2) != 1 or b.stride(2) != 1:
        raise ValueError("bmm_strided: unit stride along K required")
    batch, M, K = a.shape
    N = b.size(1)
    out = torch.empty(batch, M, N, device=a.device, dtype=a.dtype)
    _lib.call("oasr_b200_bmm_strided", _p(out), _p(a), _p(b), batch, M, N, K, a.stride(1), a.stride(0), b.stride(1), b.stride(0),
              _DTYPE_ID[a.dtype], _stream(a))
    return out


def relshift_bias(bd: torch.Tensor, lengths: torch.Tensor, T: int, scale: float, chunk: int, left_chunks: int,
                  floor_value: float = -1.0e4) -> torch.Tensor:
    """``bd (B, H, T, ld >= 2T-1)`` position scores -> attention bias ``(B, H, T, T)`` (a view whose rows are padded to a multiple of 8 elements): Transformer-XL relative shift,
    scale, chunked-limited window and key-padding mask with a finite floor, in one kernel
    (oasr/models/nemotron/encoder.py:82-96, 124-149, 343-348)."""
    _need_cuda(bd, lengths)
    B, H, Tq, ld = bd.shape
    if Tq != T or bd.stride(3) != 1 or bd.stride(2) != ld:
        raise ValueError("bd must be (B, H, T, ld) with packed rows (batch and head strides are free)")
    ld_out = (T + 7) // 8 * 8          # rows start on 16-byte boundaries so the attention kernel reads them in 16-byte pieces
    out = torch.empty(B, H, T, ld_out, device=bd.device, dtype=bd.dtype)
    _lib.call("oasr_b200_relshift_bias", _p(out), _p(bd), _p(lengths), B, H, T, ld, ld_out, bd.stride(0), bd.stride(1),
              float(scale), int(chunk), int(left_chunks),
              float(floor_value), _DTYPE_ID[bd.dtype], _stream(bd))
    return out[..., :T]


def gemm_argmax(A: torch.Tensor, B: torch.Tensor, C: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-row index of the first maximum of ``A @ B.T + C`` (int32) without writing logits or log-probs: the
    token-only form of the CTC head.  What ``gemm_log_softmax`` followed by the per-frame argmax of a greedy search
    computes (oasr/layers/ctc.py:48-51, oasr/functionals/ctc_decode.py:359), in one vocabulary sweep."""
    _need_cuda(A, B, C)
    K, N = A.shape[-1], B.shape[0]
    A2 = A.reshape(-1, K)
    A2 = A2 if A2.is_contiguous() else A2.contiguous()
    B = B if B.is_contiguous() else B.contiguous()
    arg = torch.empty(A.shape[:-1], device=A.device, dtype=torch.int32)
    _lib.call("oasr_b200_gemm_log_softmax", None, _p(A2), _p(B), _p(C), A2.size(0), N, K, _DTYPE_ID[A.dtype],
              _DTYPE_ID[torch.float32], _p(arg), _stream(A))
    return arg


def ctc_greedy_collapse(ids: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int, blank: int = 0, want_times: bool = False):
    """Greedy CTC decoding on the device: packed per-frame argmax ``ids (total,) int32`` with utterance boundaries
    ``cu_seqlens (B + 1,) int32`` -> ``(tokens (B, max_len) int32, lengths (B,) int32, times or None)``; repeats are
    dropped, then blanks, never across an utterance boundary (csrc/decoder/ctc/cpu/ctc_greedy_search.cc:26-55); the beam-1
    form of the reference's GPU decoder result (oasr/functionals/ctc_decode.py:81-101)."""
    _need_cuda(ids, cu_seqlens)
    if ids.dtype != torch.int32 or cu_seqlens.dtype != torch.int32 or not ids.is_contiguous() or not cu_seqlens.is_contiguous():
        raise ValueError("ids and cu_seqlens must be contiguous int32 tensors")
    B = cu_seqlens.numel() - 1
    tokens = torch.empty(B, int(max_len), device=ids.device, dtype=torch.int32)
    lengths = torch.empty(B, device=ids.device, dtype=torch.int32)
    times = torch.empty(B, int(max_len), device=ids.device, dtype=torch.int32) if want_times else None
    _lib.call("oasr_b200_ctc_greedy_collapse", _p(tokens), _p(lengths), _p(times), _p(ids), _p(cu_seqlens), B, int(max_len),
              int(blank), _stream(ids))
    return tokens, lengths, times
