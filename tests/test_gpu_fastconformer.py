"""GPU parity of the FastConformer / Nemotron layer stack composed from this package's operators against the fp32
oracle and the fixture written from the reference's own layers."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oasr_b200 as ob
from oasr_b200.fastconformer import FastConformerEncoder, FastConformerLayers
from oracle import fastconformer as OFC
from tests.golden import cases

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("packed", [True, False])
def test_layer_stack_matches_oracle_and_reference_fixture(packed):
    cfg, case = OFC.TINY, cases.FASTCONFORMER_CASE
    P = OFC.init_params(cfg, case["weight_seed"])
    hidden = cases.make_fastconformer_hidden(case, cfg)
    model = FastConformerLayers(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    got = model.forward(hidden.cuda(), case["lengths"], packed=packed).cpu()
    assert ob.device_status() == 0
    want = OFC.layers_forward(P, cfg, hidden, case["lengths"])
    gold = torch.from_numpy(np.load(GOLD / "fastconformer_tiny.npz")["hidden_out"])
    valid = torch.arange(hidden.size(1))[None, :] < torch.tensor(case["lengths"])[:, None]
    for ref in (want, gold):
        d = (got - ref).abs()[valid]
        # layer-normalised outputs of O(1): bf16 GEMM inputs / weights against the fp32 path
        assert d.max().item() < 6e-2 and d.mean().item() < 6e-3, (d.max().item(), d.mean().item())
    cos = torch.nn.functional.cosine_similarity(got[valid].flatten(), want[valid].flatten(), dim=0).item()
    print(f"fastconformer layer stack: max-abs {(got - want).abs()[valid].max().item():.3e}, cosine {cos:.6f}")
    assert cos > 0.9995


@pytest.mark.parametrize("packed", [True, False])
def test_config4_sized_layer_runs_and_is_isolated_per_utterance(packed):
    """One layer at the FastConformer width (hidden 1024, 8 heads of 128, FFN 4096, kernel 9): an utterance inside a
    padded batch equals the same utterance alone on its valid frames (key padding and silent rows do their job)."""
    torch.manual_seed(3)
    cfg = OFC.FastConformerConfig(hidden=1024, heads=8, ffn=4096, layers=1, kernel=9, sliding_window=57, lookahead=3, bias=False)
    P = OFC.init_params(cfg, 11)
    lengths = [96, 41]
    hidden = torch.randn(2, 96, 1024)
    model = FastConformerLayers(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    hidden_dev = hidden.cuda()
    both = model.forward(hidden_dev, lengths, packed=packed)
    assert torch.equal(hidden_dev.cpu(), hidden)                       # the fp32 input is not the residual buffer
    alone = model.forward(hidden[1:2, :41].contiguous().cuda(), [41], packed=packed)
    assert ob.device_status() == 0
    assert torch.isfinite(both).all()
    assert (both[1, :41] - alone[0]).abs().max().item() < 2e-2


def test_packed_and_padded_execution_agree_on_ragged_batch():
    """Valid frames only (packed rows, per-segment attention and causal conv) against the padded batch: same frames out,
    zeros in the padding, with an empty stream and lengths that are not multiples of 8 in the batch."""
    torch.manual_seed(8)
    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=2, kernel=9, sliding_window=25, lookahead=2, bias=True)
    P = OFC.init_params(cfg, 5)
    lengths = [150, 0, 67, 133, 1]
    hidden = torch.randn(5, 150, 256).cuda()
    model = FastConformerLayers(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    padded = model.forward(hidden, lengths, packed=False)
    packed = model.forward(hidden, lengths, packed=True)
    assert ob.device_status() == 0
    valid = (torch.arange(150)[None, :] < torch.tensor(lengths)[:, None]).cuda()
    assert (packed[valid] - padded[valid]).abs().max().item() < 2e-2
    assert torch.count_nonzero(packed[~valid]) == 0
    want = OFC.layers_forward(P, cfg, hidden.cpu(), lengths)
    d = (packed.cpu() - want).abs()[valid.cpu()]
    assert d.max().item() < 6e-2 and d.mean().item() < 6e-3, (d.max().item(), d.mean().item())


def test_whole_encoder_matches_oracle_and_reference_fixture():
    """8x subsampling front end + layer stack against the oracle and the reference's NemotronEncoder output."""
    from oasr_b200.fastconformer import FastConformerEncoder

    cfg, sub, case = OFC.TINY, OFC.TINY_SUB, cases.FASTCONFORMER_ENCODER_CASE
    P = dict(OFC.init_params(cfg, case["weight_seed"]))
    P.update(OFC.init_subsampling_params(sub, cfg.hidden, case["sub_seed"]))
    feats = cases.make_fastconformer_features(case, sub)
    enc = FastConformerEncoder(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead,
                               sub.mels, sub.channels, P)
    got, out_len = enc.forward(feats.cuda(), case["lengths"])
    assert ob.device_status() == 0
    gold = np.load(GOLD / "fastconformer_tiny.npz")
    assert out_len == gold["encoder_len"].tolist()
    want, _ = OFC.encoder_forward(P, cfg, sub, feats, case["lengths"])
    valid = torch.arange(got.size(1))[None, :] < torch.tensor(out_len)[:, None]
    got = got.cpu()
    for ref in (want, torch.from_numpy(gold["encoder_out"])):
        d = (got - ref).abs()[valid]
        assert d.max().item() < 8e-2 and d.mean().item() < 8e-3, (d.max().item(), d.mean().item())
    # the subsampling front end alone, tighter
    hid, _ = enc.subsample(feats.cuda(), case["lengths"])
    ref_hid, ref_len = OFC.subsampling_forward(P, sub, feats, torch.tensor(case["lengths"]))
    dh = (hid.float().cpu() - ref_hid).abs()[valid]
    assert dh.max().item() < 3e-2 * max(1.0, ref_hid.abs().max().item()), dh.max().item()
    print(f"fastconformer encoder: max-abs {(got - want).abs()[valid].max().item():.3e}; front end {dh.max().item():.3e} of {ref_hid.abs().max().item():.2f}")


@pytest.mark.parametrize("mode", ["fp8", "int8"])
def test_quantised_layer_stack_reaches_the_cosine_gate_against_the_16_bit_run(mode):
    """FastConformer width (hidden 1024, 8 heads of 128, FFN 4096), two layers: Linear GEMMs on 8-bit operands
    (per-output-channel weight scales, per-token dynamic activation scales) against the bf16 run: cosine >= 0.999."""
    cfg = OFC.FastConformerConfig(hidden=1024, heads=8, ffn=4096, layers=2, kernel=9, sliding_window=57, lookahead=3, bias=False)
    P = OFC.init_params(cfg, 13, w_std=0.02)     # BASELINE's N(0, 0.02) init: at 0.06 and width 1024 the attention is
    lengths = [120, 77]                          # near one-hot and any rounding flips it
    hidden = torch.randn(2, 120, 1024, generator=torch.Generator().manual_seed(2)).cuda()
    args = (cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    ref = FastConformerLayers(*args).forward(hidden, lengths)
    got = FastConformerLayers(*args, quant=mode).forward(hidden, lengths)
    assert ob.device_status() == 0
    valid = (torch.arange(120)[None, :] < torch.tensor(lengths)[:, None]).cuda()
    cos = torch.nn.functional.cosine_similarity(got[valid].flatten().double(), ref[valid].flatten().double(), dim=0).item()
    rel = ((got[valid] - ref[valid]).norm() / ref[valid].norm()).item()
    print(f"{mode} FastConformer layers vs bf16: cosine {cos:.6f}, relative error {rel:.4f}")
    assert cos >= 0.999, cos


def test_relshift_bias_equals_the_pad_view_identity():
    """One-kernel rel_shift + scale + window / padding mask against the reference's pad-and-reinterpret identity and
    its mask (oasr/models/nemotron/encoder.py:82-96, 124-149, 343-348), bit for bit."""
    from oasr_b200 import fused

    torch.manual_seed(4)
    B, H, T, chunk, left = 3, 4, 37, 4, 8
    P = 2 * T - 1
    ld = (P + 7) // 8 * 8
    bd = torch.randn(B, H, T, ld).bfloat16()
    lengths = [37, 21, 30]
    scale = 128 ** -0.5
    got = fused.relshift_bias(bd.cuda(), torch.tensor(lengths, dtype=torch.int32).cuda(), T, scale, chunk, left // chunk).cpu()
    shifted = OFC.rel_shift(bd[..., :P].float())[..., :T] * scale
    window = OFC.chunked_limited_mask(T, T, left, chunk - 1).view(1, 1, T, T)
    keep = (torch.arange(T)[None, :] < torch.tensor(lengths)[:, None]).view(B, 1, 1, T)
    want = shifted.masked_fill((window & keep).logical_not(), -1.0e4).bfloat16()
    assert torch.equal(got, want)


def test_relshift_bias_reads_head_major_scores():
    """The same bias from scores stored (H, B, T, ld) and passed as a permuted view: batch / head strides are honoured."""
    from oasr_b200 import fused

    torch.manual_seed(5)
    B, H, T, chunk = 2, 3, 19, 3
    ld = (2 * T - 1 + 7) // 8 * 8
    bd = torch.randn(B, H, T, ld).bfloat16().cuda()
    lens = torch.tensor([19, 11], dtype=torch.int32).cuda()
    want = fused.relshift_bias(bd, lens, T, 0.25, chunk, 2)
    head_major = bd.permute(1, 0, 2, 3).contiguous().permute(1, 0, 2, 3)
    assert not head_major.is_contiguous()
    assert torch.equal(fused.relshift_bias(head_major, lens, T, 0.25, chunk, 2), want)


def test_bmm_strided_reads_heads_in_place():
    """Per-head products straight from a (tokens, heads, head_dim) projection equal bmm on head-major copies, bit for bit."""
    from oasr_b200 import fused

    torch.manual_seed(6)
    M, H, D, N = 300, 4, 64, 136
    proj = torch.randn(M, 3, H, D).bfloat16().cuda()          # a head's rows sit 3*H*D apart
    table = torch.randn(N, H, D).bfloat16().cuda()
    a = proj[:, 1].permute(1, 0, 2)                            # (H, M, D) view
    b = table.permute(1, 0, 2)                                 # (H, N, D) view
    got = fused.bmm_strided(a, b)
    want = ob.bmm(a.contiguous(), b.contiguous())
    assert ob.device_status() == 0
    assert torch.equal(got, want)
    ref = torch.einsum("hmd,hnd->hmn", a.float(), b.float())
    assert (got.float() - ref).abs().max() < 0.08 * ref.abs().max().clamp(min=1.0)


def test_relshift_bias_packed_equals_padded_per_segment():
    """Block-diagonal bias of packed rows against the padded kernel, stream by stream, bit for bit; rows of a segment are
    roundup8(len) apart and the padding columns carry the floor."""
    from oasr_b200 import fused

    torch.manual_seed(12)
    H, T, chunk, left_chunks = 3, 29, 3, 4
    lens = [29, 5, 0, 18]
    ld = (2 * T - 1 + 7) // 8 * 8
    bd_pad = torch.randn(len(lens), H, T, ld).bfloat16().cuda()
    padded = fused.relshift_bias(bd_pad, torch.tensor(lens, dtype=torch.int32).cuda(), T, 0.3, chunk, left_chunks)
    cu = np.concatenate([[0], np.cumsum(lens)])
    total = int(cu[-1])
    bd = torch.cat([bd_pad[b, :, :n] for b, n in enumerate(lens)], dim=1).contiguous()          # (H, total, ld)
    ld8 = [(n + 7) // 8 * 8 for n in lens]
    offs = np.concatenate([[0], np.cumsum([H * n * l for n, l in zip(lens, ld8)])]).astype(np.int64)
    flat = fused.relshift_bias_packed(bd, torch.from_numpy(cu.astype(np.int32)).cuda(), torch.from_numpy(offs).cuda(),
                                      int(offs[-1]), T, 0.3, chunk, left_chunks)
    assert bd.size(1) == total
    for b, n in enumerate(lens):
        seg = flat[offs[b]:offs[b + 1]].view(H, n, ld8[b])
        assert torch.equal(seg[..., :n], padded[b, :, :n, :n])
        assert (seg[..., n:] == -1.0e4).all()


@pytest.mark.parametrize("width", ["tiny", "real"])
def test_streaming_chunks_match_the_oracle_and_the_offline_pass(width):
    """FastConformer layer stack chunk by chunk over paged keys / values and cached conv tails: every chunk against the
    fp32 streaming oracle (itself equal to the offline oracle, tests/test_fastconformer_streaming_oracle.py), streams
    in scattered slots with different starting times, history longer than the trained left context so that pages are
    evicted; and the concatenation of a stream's chunks against this package's own offline pass."""
    if width == "tiny":
        cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=2, kernel=9, sliding_window=25, lookahead=3, bias=True)
        w_std = 0.06
    else:
        cfg = OFC.FastConformerConfig(hidden=1024, heads=8, ffn=4096, layers=2, kernel=9, sliding_window=57, lookahead=3, bias=False)
        w_std = 0.02
    P = OFC.init_params(cfg, 21, w_std=w_std)
    model = FastConformerLayers(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    step, chunks, streams = 16, 8, 3
    cache = model.new_streaming_cache(max_streams=5, chunk_frames=step)
    assert cache.max_past >= cfg.sliding_window - 1
    g = torch.Generator().manual_seed(3)
    hidden = torch.randn(streams, step * chunks, cfg.hidden, generator=g)
    slots = [4, 1, 2]
    states = [OFC.FastStreamState(cfg) for _ in range(streams)]
    outs = [[] for _ in range(streams)]
    worst = 0.0
    for c in range(chunks + 2):
        # stream s starts s chunks late: the batch composition changes over time
        active = [s for s in range(streams) if 0 <= c - s < chunks]
        if not active:
            continue
        xs = torch.stack([hidden[s, (c - s) * step:(c - s + 1) * step] for s in active])
        got = model.forward_chunk(xs.cuda(), [slots[s] for s in active], cache).cpu()
        assert ob.device_status() == 0
        for n, s in enumerate(active):
            with torch.no_grad():
                want = OFC.layers_forward_chunk(P, cfg, states[s], hidden[s, (c - s) * step:(c - s + 1) * step], keep_frames=cache.max_past)
            d = (got[n] - want).abs()
            worst = max(worst, d.max().item())
            assert d.max().item() < 6e-2 and d.mean().item() < 6e-3, (c, s, d.max().item(), d.mean().item())
            outs[s].append(got[n])
    print(f"fastconformer streaming ({width}): worst chunk max-abs {worst:.3e}")
    offline = model.forward(hidden.cuda(), [step * chunks] * streams).cpu()
    for s in range(streams):
        d = (torch.cat(outs[s]) - offline[s]).abs()
        assert d.max().item() < 6e-2 and d.mean().item() < 6e-3, (s, d.max().item(), d.mean().item())


def test_streaming_from_feature_frames_matches_the_oracle():
    """NemotronEncoder.forward_chunk_paged from mel frames: streaming 8x subsampling (every stage continues from its
    cached two input frames) feeding the streaming layer stack, streams in scattered slots that start at different
    times, against the fp32 streaming oracle chunk by chunk; then a slot is reset and reused, which must give the
    same first chunk again."""
    sub = OFC.SubsamplingConfig(mels=80, channels=32, stages=3)
    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=2, kernel=9, sliding_window=25, lookahead=3, bias=True)
    P = OFC.init_params(cfg, 31)
    P.update(OFC.init_subsampling_params(sub, cfg.hidden, 32))
    enc = FastConformerEncoder(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead,
                               sub.mels, sub.channels, P, stages=sub.stages)
    step, chunks, streams = 16, 5, 3
    cache = enc.new_streaming_cache(max_streams=6, chunk_frames=step)
    feats = torch.randn(streams, step * 8 * chunks, sub.mels, generator=torch.Generator().manual_seed(9))
    slots = [5, 0, 3]
    front = [OFC.SubsamplingStreamState(sub) for _ in range(streams)]
    stack = [OFC.FastStreamState(cfg) for _ in range(streams)]
    first = None
    worst = worst_mean = 0.0
    for c in range(chunks + 2):
        active = [s for s in range(streams) if 0 <= c - s < chunks]
        if not active:
            continue
        win = lambda s: feats[s, (c - s) * step * 8:(c - s + 1) * step * 8]
        got = enc.forward_chunk(torch.stack([win(s) for s in active]).cuda(), [slots[s] for s in active], cache).cpu()
        assert ob.device_status() == 0
        for n, s in enumerate(active):
            with torch.no_grad():
                hid = OFC.subsampling_forward_chunk(P, sub, front[s], win(s))
                want = OFC.layers_forward_chunk(P, cfg, stack[s], hid, keep_frames=cache.max_past)
            d = (got[n] - want).abs()
            worst, worst_mean = max(worst, d.max().item()), max(worst_mean, d.mean().item())
            assert d.max().item() < 8e-2 and d.mean().item() < 8e-3, (c, s, d.max().item(), d.mean().item())
            if s == 0 and c == 0:
                first = got[n].clone()
    print(f"fastconformer streaming from features: worst chunk max-abs {worst:.3e}, mean-abs {worst_mean:.3e}")
    cache.reset_stream(slots[0])
    again = enc.forward_chunk(feats[0:1, :step * 8].cuda(), [slots[0]], cache).cpu()[0]
    assert torch.equal(again, first)


@pytest.mark.parametrize("quant", ["fp8", "int8"])
def test_native_executor_with_8bit_linears_equals_the_composed_stack(quant):
    """With an 8-bit kind the native executor quantises every Linear's input per token and runs the fp8 / int8 GEMM on
    the weight quantised once per output channel -- the same two kernels per Linear as the Python composition, so
    the results are bit-identical, and they stay within the 8-bit gate (cosine >= 0.999) of the 16-bit stack."""
    from oasr_b200 import _lib

    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=2, kernel=9, sliding_window=25, lookahead=3, bias=True)
    P = OFC.init_params(cfg, 78, w_std=0.02)     # the benchmark's N(0, 0.02) init, as in the gate test above
    args = (cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    model = FastConformerLayers(*args, quant=quant)
    assert model.native and model._native_model.quant_kind in (1, 2)
    lengths = [61, 17, 128, 1]
    hidden = torch.randn(len(lengths), 128, cfg.hidden, generator=torch.Generator().manual_seed(3)).cuda()
    before = _lib.launch_count()
    rows_native, index = model.forward_rows(hidden, lengths)
    launched = _lib.launch_count() - before
    model.native = False
    rows_composed, _ = model.forward_rows(hidden, lengths)
    model.native = True
    assert ob.device_status() == 0
    assert torch.equal(rows_native, rows_composed)
    assert launched >= 21 * cfg.layers          # 17 + 4 per-token quantisations per layer (the other four ride in add + norm)
    rows16, _ = FastConformerLayers(*args).forward_rows(hidden, lengths)
    cos = torch.nn.functional.cosine_similarity(rows_native.flatten(), rows16.flatten(), dim=0).item()
    print(f"{quant} native stack vs 16-bit stack: cosine {cos:.6f}")
    assert cos >= 0.999


def test_native_executor_equals_the_operator_by_operator_stack():
    """oasr_b200_fastconformer_layers_packed enqueues the same kernels in the same order as the Python composition of
    the packed stack, so the two agree bit for bit; it refuses a workspace that is too small before launching."""
    import ctypes

    from oasr_b200 import _lib

    cfg = OFC.FastConformerConfig(hidden=256, heads=2, ffn=512, layers=3, kernel=9, sliding_window=25, lookahead=3, bias=True)
    P = OFC.init_params(cfg, 77)
    model = FastConformerLayers(cfg.hidden, cfg.heads, cfg.ffn, cfg.layers, cfg.kernel, cfg.sliding_window, cfg.lookahead, P)
    assert model.native
    lengths = [61, 0, 17, 128, 1]
    hidden = torch.randn(len(lengths), 128, cfg.hidden, generator=torch.Generator().manual_seed(2)).cuda()
    before = _lib.launch_count()
    rows_native, index = model.forward_rows(hidden, lengths)
    launched = _lib.launch_count() - before
    model.native = False
    rows_composed, index2 = model.forward_rows(hidden, lengths)
    model.native = True
    assert ob.device_status() == 0
    assert torch.equal(index, index2) and torch.equal(rows_native, rows_composed)
    assert launched >= 17 * cfg.layers
    # 16-bit post-subsampling states (what the front end hands over): the same agreement
    hidden16 = hidden.bfloat16()
    native16, _ = model.forward_rows(hidden16, lengths)
    model.native = False
    composed16, _ = model.forward_rows(hidden16, lengths)
    model.native = True
    assert torch.equal(native16, composed16)
    # too small a workspace: refused with a message, nothing launched
    table = model._position_table(128)
    before = _lib.launch_count()
    with pytest.raises(_lib.OasrB200Error, match="workspace"):
        ws = torch.empty(4096, dtype=torch.uint8, device="cuda")
        res = torch.zeros(8, cfg.hidden, device="cuda")
        cu = torch.tensor([0, 8], dtype=torch.int32, device="cuda")
        offs = torch.tensor([0, cfg.heads * 8 * 8], dtype=torch.int64, device="cuda")
        out = torch.empty_like(res)
        _lib.call("oasr_b200_fastconformer_layers_packed", ctypes.byref(model._native_model), ctypes.c_void_p(res.data_ptr()), 1,
                  ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(table.data_ptr()), table.size(0), ctypes.c_void_p(cu.data_ptr()),
                  ctypes.c_void_p(offs.data_ptr()), cfg.heads * 64, 1, 8, 128, ctypes.c_void_p(ws.data_ptr() + (-ws.data_ptr()) % 256),
                  2048, None)
    assert _lib.launch_count() == before
