"""GPU: the allocation-free entry point gives the same result as the workspace one.

Some embedders of this library cannot call cudaMalloc at all: a plugin inside a serving process
whose memory pool took the whole GPU at start-up, code that runs inside a framework's allocator
callbacks, or a latency-critical thread for which a device-wide stall is unacceptable.  For them
``oasr_b200_conformer_encode_packed_noalloc`` keeps its scratch in a fixed 64 MiB array inside the
library.  This file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

from oasr_b200 import _lib
from oasr_b200.encoder import ConformerCTC, ConformerConfig, build_packed_batch
from oasr_b200.weights import init_params

pytestmark = pytest.mark.gpu


def _setup():
    cfg = ConformerConfig(d_model=128, heads=2, ffn=256, layers=2, vocab=90)
    model = ConformerCTC(cfg, init_params(cfg, 4321), device="cuda", dtype=torch.bfloat16)
    lengths = [96, 151, 40]
    out_lens = [(n - 3) // 4 for n in lengths]
    feats = torch.randn(len(lengths), max(lengths), cfg.input_size, generator=torch.Generator().manual_seed(11)).cuda()
    T = feats.size(1)
    Tp = (((T - 3) // 2 + 1) - 3) // 2 + 1
    pk = build_packed_batch(out_lens, Tp, cfg.kernel, feats.device)
    rows = model._subsample_packed(feats, out_lens, pk.cu_seqlens, pk.total)
    return cfg, model, pk, rows


def test_noalloc_entry_point_matches_workspace_entry_point_twice():
    cfg, model, pk, rows = _setup()
    want_lp, want_arg = model._encode_packed(rows, pk, False)          # existing entry point, caller workspace
    lp = torch.empty(pk.total, cfg.vocab_padded, device="cuda", dtype=torch.float32)
    arg = torch.empty(pk.total, device="cuda", dtype=torch.int32)
    for _ in range(2):                                                  # two calls in a row share the scratch
        lp.fill_(float("nan"))
        arg.fill_(-1)
        model.encode_rows_noalloc(rows, pk, lp, arg)
        torch.cuda.synchronize()
        assert torch.isfinite(lp).all()
        torch.testing.assert_close(lp, want_lp, rtol=0, atol=2e-2)      # the tolerance of the model-level tests
        assert (lp - want_lp).abs().max().item() <= 1e-6                # same kernels, same order: identical
        assert torch.equal(arg, want_arg)


def test_noalloc_entry_point_refuses_oversized_batches():
    cfg, model, pk, rows = _setup()
    cap = _lib.load().oasr_b200_conformer_noalloc_capacity_bytes()
    assert cap == 64 << 20
    need = _lib.load().oasr_b200_conformer_workspace_bytes(ctypes.byref(model._native_model), 10 ** 6, 500)
    assert need > cap
    with pytest.raises(_lib.OasrB200Error, match="bytes of scratch"):
        # sizes only: the refusal happens before any pointer is used or any kernel is launched
        _lib.call("oasr_b200_conformer_encode_packed_noalloc", ctypes.byref(model._native_model), None, None, None,
                  3, 10 ** 6, 500, None, None, None)


def test_noalloc_padded_semantics_and_a_batch_just_under_the_capacity():
    """The padded-batch form (``fill_frames``) and the largest batch the built-in array can hold: both equal the
    workspace entry point, and one more row tile is refused."""
    cfg, model, pk, rows = _setup()
    want_lp, want_arg = model._encode_packed(rows, pk, True)                # padded semantics
    lp = torch.full((pk.total, cfg.vocab_padded), float("nan"), device="cuda")
    arg = torch.full((pk.total,), -1, device="cuda", dtype=torch.int32)
    model.encode_rows_noalloc(rows, pk, lp, arg, padded_semantics=True)
    torch.cuda.synchronize()
    torch.testing.assert_close(lp, want_lp, rtol=0, atol=2e-2)
    assert (lp - want_lp).abs().max().item() <= 1e-6 and torch.equal(arg, want_arg)
    # the largest number of 400-frame segments whose scratch still fits
    lib = _lib.load()
    cap = lib.oasr_b200_conformer_noalloc_capacity_bytes()
    seg = 400
    n = 1
    while lib.oasr_b200_conformer_workspace_bytes(ctypes.byref(model._native_model), (n + 1) * seg, seg) <= cap:
        n += 1
    total = n * seg
    assert lib.oasr_b200_conformer_workspace_bytes(ctypes.byref(model._native_model), total, seg) > 0.95 * cap
    big = build_packed_batch([seg] * n, seg, cfg.kernel, "cuda")
    g = torch.Generator(device="cuda").manual_seed(5)
    big_rows = (torch.randn(total, rows.size(1), device="cuda", generator=g) * 0.5).to(rows.dtype)
    want_lp, want_arg = model._encode_packed(big_rows, big, False)
    lp = torch.full((total, cfg.vocab_padded), float("nan"), device="cuda")
    arg = torch.full((total,), -1, device="cuda", dtype=torch.int32)
    model.encode_rows_noalloc(big_rows, big, lp, arg)
    torch.cuda.synchronize()
    assert torch.isfinite(lp).all()
    torch.testing.assert_close(lp, want_lp, rtol=0, atol=2e-2)
    assert (lp - want_lp).abs().max().item() <= 1e-6 and torch.equal(arg, want_arg)
    over = build_packed_batch([seg] * (n + 1), seg, cfg.kernel, "cuda")
    with pytest.raises(_lib.OasrB200Error, match="bytes of scratch"):
        model.encode_rows_noalloc(big_rows, over, lp, arg)
