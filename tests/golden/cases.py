"""Seeded test cases shared by the fixture generator and the tests.

Inputs are regenerated from seeds; only reference OUTPUTS are stored in the
``.npz`` fixtures next to this file (written by ``make_golden.py``).
Shapes follow the reference's own test grids (tests/test_fmha.py:89-100,204-222,
tests/test_fmha_varlen.py, tests/test_packing_encoder.py) and BASELINE config 1.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from oracle import conformer as OC

MODEL_CASES = {
    # every bias / gain / BatchNorm statistic away from its default, all paths exercised
    "tiny": dict(cfg=OC.TINY, weight_seed=1234, perturb=0.1, feat_seed=7, lengths=[67, 123, 40, 11], store="full"),
    # BASELINE config 1: 12 layers, d 256, 4 heads, vocab 5002; 400/650/800/1000 frames
    "config1": dict(cfg=OC.CONFIG1, weight_seed=1234, perturb=0.0, feat_seed=7, lengths=[400, 650, 800, 1000],
                    store="compact"),
}


def make_features(case):
    """iid N(0,1) features (B, Tmax, F); the tail beyond each length is N(0,1) too."""
    g = torch.Generator().manual_seed(case["feat_seed"])
    lengths = torch.tensor(case["lengths"], dtype=torch.int64)
    feats = torch.randn(len(case["lengths"]), int(lengths.max()), case["cfg"].input_size, generator=g)
    return feats, lengths


def _g(seed):
    return torch.Generator().manual_seed(seed)


# name -> dense attention case
FMHA_CASES = {
    "basic": dict(B=2, H=4, Hkv=4, Tq=64, Tk=64, D=64, bias=True, lens=None, starts=None, causal=False, seed=1),
    "odd_tk": dict(B=2, H=4, Hkv=4, Tq=33, Tk=33, D=64, bias=True, lens=[33, 20], starts=None, causal=False, seed=2),
    "long_odd": dict(B=1, H=2, Hkv=2, Tq=249, Tk=249, D=64, bias=True, lens=[249], starts=None, causal=False, seed=3),
    "gqa": dict(B=2, H=8, Hkv=2, Tq=40, Tk=72, D=64, bias=False, lens=[72, 9], starts=None, causal=False, seed=4),
    "mqa_d128": dict(B=2, H=4, Hkv=1, Tq=20, Tk=150, D=128, bias=True, lens=[150, 100], starts=None, causal=False,
                     seed=5),
    "causal": dict(B=2, H=2, Hkv=2, Tq=70, Tk=70, D=64, bias=False, lens=[70, 31], starts=None, causal=True, seed=6),
    "starts": dict(B=3, H=2, Hkv=2, Tq=16, Tk=96, D=64, bias=True, lens=[96, 50, 40], starts=[0, 10, 40],
                   causal=False, seed=7),   # last stream: empty window -> zero rows
    "stream_chunk": dict(B=4, H=4, Hkv=4, Tq=16, Tk=272, D=64, bias=True, lens=[272, 16, 100, 33], starts=None,
                         causal=False, seed=8),
    "no_mask_nobias": dict(B=1, H=1, Hkv=1, Tq=130, Tk=300, D=64, bias=False, lens=None, starts=None, causal=False,
                           seed=9),
}


def make_fmha(c):
    g = _g(c["seed"])
    q = torch.randn(c["B"], c["H"], c["Tq"], c["D"], generator=g)
    k = torch.randn(c["B"], c["Hkv"], c["Tk"], c["D"], generator=g)
    v = torch.randn(c["B"], c["Hkv"], c["Tk"], c["D"], generator=g)
    c["scale"] = 1.0 / math.sqrt(c["D"])
    t = dict(q=q, k=k, v=v)
    if c["bias"]:
        t["bias"] = torch.randn(c["B"], c["H"], c["Tq"], c["Tk"], generator=g)
    if c["lens"] is not None:
        t["seqlens"] = torch.tensor(c["lens"], dtype=torch.int32)
    if c["starts"] is not None:
        t["seqstarts"] = torch.tensor(c["starts"], dtype=torch.int32)
    return t


PAGED_CASES = {
    "bs16": dict(B=4, H=4, Hkv=4, Tq=16, D=64, block_size=16, nblk=17, num_blocks=80, lens=[272, 16, 100, 33],
                 t_new=16, seed=21),
    "bs16_gqa": dict(B=3, H=8, Hkv=2, Tq=16, D=64, block_size=16, nblk=5, num_blocks=20, lens=[80, 17, 64], t_new=16,
                     seed=22),
    "bs32": dict(B=2, H=2, Hkv=2, Tq=8, D=64, block_size=32, nblk=3, num_blocks=9, lens=[70, 96], t_new=8, seed=23),
}


def make_paged(c):
    g = _g(c["seed"])
    q = torch.randn(c["B"], c["H"], c["Tq"], c["D"], generator=g)
    k_pool = torch.randn(c["num_blocks"], c["block_size"], c["Hkv"], c["D"], generator=g)
    v_pool = torch.randn(c["num_blocks"], c["block_size"], c["Hkv"], c["D"], generator=g)
    perm = torch.randperm(c["num_blocks"], generator=g)[: c["B"] * c["nblk"]]
    block_table = perm.view(c["B"], c["nblk"]).to(torch.int32)
    Tk = c["nblk"] * c["block_size"]
    bias = torch.randn(c["B"], c["H"], c["Tq"], Tk, generator=g)
    seqlens = torch.tensor(c["lens"], dtype=torch.int32)
    offsets = (seqlens - c["t_new"]).clamp(min=0).to(torch.int32)
    c["scale"] = 1.0 / math.sqrt(c["D"])
    return dict(q=q, k_pool=k_pool, v_pool=v_pool, block_table=block_table, bias=bias, seqlens=seqlens,
                offsets=offsets)


VARLEN_CASES = {
    "one": dict(lens=[33], H=4, Hkv=4, D=64, seed=31),
    "two_full": dict(lens=[64, 64], H=4, Hkv=4, D=64, seed=32),
    "ragged": dict(lens=[33, 249, 17], H=4, Hkv=4, D=64, seed=33),
    "many_small": dict(lens=[8] * 12, H=2, Hkv=2, D=64, seed=34),
    "gqa": dict(lens=[130, 5, 70], H=8, Hkv=2, D=64, seed=35),
}


def make_varlen(c):
    g = _g(c["seed"])
    total = sum(c["lens"])
    q = torch.randn(total, c["H"], c["D"], generator=g)
    k = torch.randn(total, c["Hkv"], c["D"], generator=g)
    v = torch.randn(total, c["Hkv"], c["D"], generator=g)
    cu = torch.tensor([0] + list(np.cumsum(c["lens"])), dtype=torch.int32)
    sizes = [c["H"] * t * t for t in c["lens"]]
    bias_offsets = torch.tensor([0] + list(np.cumsum(sizes)), dtype=torch.int64)
    bias = torch.randn(int(bias_offsets[-1]), generator=g)
    c["scale"] = 1.0 / math.sqrt(c["D"])
    return dict(q=q, k=k, v=v, cu=cu, bias=bias, bias_offsets=bias_offsets)


def packed_layout(lens, conv_kernel: int, num_heads: int):
    """Index tensors of the packed layout (integer restatement of
    oasr/models/conformer/packing.py:99-219) for a batch whose padded length is max(lens)."""
    lens = np.asarray(lens, dtype=np.int64)
    B, Tp = len(lens), int(lens.max())
    half = (conv_kernel - 1) // 2
    cu = np.zeros(B + 1, dtype=np.int32)
    cu[1:] = np.cumsum(lens)
    seg_id = np.repeat(np.arange(B, dtype=np.int64), lens)
    local = np.arange(int(lens.sum()), dtype=np.int64) - cu[:-1].astype(np.int64)[seg_id]
    return dict(
        cu_seqlens=cu,
        pack_src_idx=seg_id * Tp + local,
        conv_gather_idx=np.arange(int(lens.sum()), dtype=np.int64) + half * seg_id,
        bias_offsets=np.concatenate([[0], np.cumsum(num_heads * lens * lens)]).astype(np.int32),
    )


# Streaming: chunk = 16 encoder frames = windows of 67 feature frames stepped by 64
# (oasr/engine/streaming_backend/paged.py:83-104), two streams, seven chunks, a history cap
# of 2 chunks so that eviction (and the shifted position window) is exercised.
STREAM_CASE = dict(cfg=OC.TINY_STREAM, weight_seed=1234, perturb=0.1, feat_seed=17, streams=2, chunks=7,
                   window=67, step=64, num_left_chunks=2, chunk_size=16)


def make_stream_features(case):
    g = torch.Generator().manual_seed(case["feat_seed"])
    total = case["step"] * (case["chunks"] - 1) + case["window"]
    return torch.randn(case["streams"], total, case["cfg"].input_size, generator=g)


# FastConformer / Nemotron layer stack (after the subsampling front end): two layers, hidden 256 = 2 heads x 128,
# kernel 9, chunked-limited attention (left 8 frames, lookahead 3), ragged lengths so that key padding is exercised.
FASTCONFORMER_CASE = dict(weight_seed=99, hidden_seed=5, lengths=[37, 21, 30])


def make_fastconformer_hidden(case, cfg):
    g = torch.Generator().manual_seed(case["hidden_seed"])
    return torch.randn(len(case["lengths"]), max(case["lengths"]), cfg.hidden, generator=g)


# whole FastConformer encoder (8x subsampling + layer stack): 32 mel bins, 64 subsampling channels, ragged lengths
FASTCONFORMER_ENCODER_CASE = dict(weight_seed=99, sub_seed=100, feat_seed=6, lengths=[203, 120, 77])


def make_fastconformer_features(case, sub):
    g = torch.Generator().manual_seed(case["feat_seed"])
    return torch.randn(len(case["lengths"]), max(case["lengths"]), sub.mels, generator=g)
