"""GPU parity: paged streaming chunks (config-3 style) vs the streaming oracle and the fixture written
from the reference's forward_chunk_paged + cache managers."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oasr_b200 as ob
from oasr_b200.encoder import ConformerCTC, ConformerConfig
from oracle import conformer as OC
from tests.golden import cases

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def _cfg(c):
    return ConformerConfig(**{f: getattr(c, f) for f in ConformerConfig.__dataclass_fields__})


def test_streaming_chunks_match_oracle_and_reference_fixture():
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    gold = np.load(GOLD / "stream_tiny.npz")
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    model = ConformerCTC(_cfg(cfg), P)
    cache = model.new_streaming_cache(max_streams=4, max_past_frames=max_past, chunk_frames=case["chunk_size"])
    slots = [2, 0]                                                  # the two streams live in non-adjacent slots
    states = [OC.StreamState(cfg) for _ in range(case["streams"])]
    worst = 0.0
    for c in range(case["chunks"]):
        xs = feats[:, c * case["step"]: c * case["step"] + case["window"]]
        lp = model.forward_chunk_paged(xs.cuda(), slots, cache).cpu()
        assert ob.device_status() == 0
        for s in range(case["streams"]):
            want = OC.forward_chunk(P, cfg, states[s], xs[s], max_past)
            d = (lp[s] - want)[:, :cfg.vocab].abs()
            worst = max(worst, d.max().item())
            assert d.max().item() < 2e-2 and d.mean().item() < 2e-3, (c, s, d.max().item(), d.mean().item())
            assert np.abs(lp[s].numpy() - gold[f"stream{s}_log_probs"][c])[:, :cfg.vocab].max() < 2e-2
        assert cache.cached_frames(slots[0]) <= max_past + case["chunk_size"]
    print(f"streaming log-prob max-abs over {case['chunks']} chunks: {worst:.3e}")


def test_streaming_is_independent_of_batch_composition():
    """A stream's outputs do not depend on which other streams share its batch or on the physical
    pages it was given (random page permutation): bit-identical."""
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case).cuda()
    model = ConformerCTC(_cfg(cfg), P)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    both = model.new_streaming_cache(4, max_past, seed=1)
    alone = model.new_streaming_cache(1, max_past, seed=None)
    for c in range(5):
        xs = feats[:, c * case["step"]: c * case["step"] + case["window"]]
        a = model.forward_chunk_paged(xs, [3, 1], both)
        b = model.forward_chunk_paged(xs[1:2], [0], alone)
        assert torch.equal(a[1], b[0])


def test_graph_replay_equals_the_eager_step():
    """The streaming step captured once into a CUDA graph and replayed per chunk (GraphedChunkForward) against the
    eager step on a second cache with the same page order: bit-identical log-probs and argmax on every chunk, with
    the streams moving between slots of the batch from chunk to chunk."""
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case).cuda()
    model = ConformerCTC(_cfg(cfg), P)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    eager = model.new_streaming_cache(4, max_past, chunk_frames=case["chunk_size"], seed=3)
    graphed = model.new_streaming_cache(4, max_past, chunk_frames=case["chunk_size"], seed=3)
    scratch = model.new_streaming_cache(2, case["chunk_size"], chunk_frames=case["chunk_size"], seed=None)
    model.forward_chunk_paged(feats[:, :case["window"]], [0, 1], scratch)          # sizes the workspace before the capture
    step = model.graphed_chunk_forward(graphed, batch=2, window=case["window"])
    assert step.launches_per_replay > 0
    for c in range(case["chunks"]):
        xs = feats[:, c * case["step"]: c * case["step"] + case["window"]]
        order = [0, 1] if c % 2 == 0 else [1, 0]                                   # row r of the batch is stream order[r]
        slots = [[2, 0][s] for s in order]
        want_lp, want_arg = model.forward_chunk_paged(xs[order], slots, eager, return_argmax=True)
        got_lp, got_arg = step(xs[order], slots)
        assert torch.equal(got_lp, want_lp) and torch.equal(got_arg, want_arg), c
    assert ob.device_status() == 0
    with pytest.raises(RuntimeError, match="captured for"):
        step(feats[:1, :case["window"]], [0])


def test_fp8_page_write_is_bit_exact_and_fp8_attention_matches_the_dequantised_reference():
    from oasr_b200 import fused
    from oracle import ops as O

    torch.manual_seed(31)
    B, H, D, Tq, bs, hist = 19, 8, 64, 16, 16, 272
    d = H * D
    bps = hist // bs + 1
    num_blocks = B * bps + 2
    dev = "cuda"
    k_scale = (torch.rand(H) * 0.01 + 0.005).to(dev)
    v_scale = (torch.rand(H) * 0.01 + 0.005).to(dev)
    table = torch.randperm(num_blocks, device=dev)[: B * bps].view(B, bps).int()
    seqlens = torch.randint(Tq, hist + 1, (B,), device=dev, dtype=torch.int32)
    k_pool = torch.zeros(num_blocks, bs, H, D, dtype=torch.uint8, device=dev)
    v_pool = torch.zeros_like(k_pool)
    # fill every stream's history through the quantising page write, 16 frames at a time
    hist_k = (torch.randn(B, hist + Tq, H, D) * 1.5).bfloat16().to(dev)
    hist_v = (torch.randn(B, hist + Tq, H, D) * 1.5).bfloat16().to(dev)
    for c in range(0, hist + Tq, Tq):
        off = torch.full((B,), c, dtype=torch.int32, device=dev)
        fused.paged_kv_write_fp8(k_pool, v_pool, hist_k[:, c:c + Tq].permute(0, 2, 1, 3), hist_v[:, c:c + Tq].permute(0, 2, 1, 3),
                                 k_scale, v_scale, table, off)
    want_k, deq_k = O.quantize_kv_fp8(hist_k.cpu(), k_scale.cpu())
    want_v, deq_v = O.quantize_kv_fp8(hist_v.cpu(), v_scale.cpu())
    for b in (0, B - 1):
        idx = (table[b].long()[:, None] * bs + torch.arange(bs, device=dev)[None]).reshape(-1)[: hist + Tq]
        assert torch.equal(k_pool.view(-1, H, D)[idx].cpu(), want_k[b])
        assert torch.equal(v_pool.view(-1, H, D)[idx].cpu(), want_v[b])
    pos_start = torch.randint(0, 3000, (B,), device=dev, dtype=torch.int32)
    pos = torch.randn(5000, d, device=dev).bfloat16()
    qkv4 = (torch.randn(B, Tq, 4 * d, device=dev) * 0.5).bfloat16()
    scale = D ** -0.5
    got = fused.fmha_paged_relpos_fp8(qkv4, k_pool, v_pool, k_scale, v_scale, pos, pos_start, table, seqlens, H, scale).float().cpu()
    assert ob.device_status() == 0
    for b in range(B):
        n = int(seqlens[b])
        pp = pos[int(pos_start[b]): int(pos_start[b]) + n].float().cpu().view(n, H, D)
        qu = qkv4[b, :, :d].float().cpu().view(Tq, H, D)
        qv = qkv4[b, :, d:2 * d].float().cpu().view(Tq, H, D)
        s = (torch.einsum("qhd,khd->hqk", qu, deq_k[b, :n]) + torch.einsum("qhd,khd->hqk", qv, pp)) * scale
        want = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), deq_v[b, :n]).reshape(Tq, d)
        err = (got[b] - want).abs().max().item()
        assert err < 3e-2 * max(1.0, want.abs().max().item()), (b, n, err)


def test_streaming_with_fp8_pages_reaches_the_cosine_gate_against_16_bit_pages():
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case).cuda()
    model = ConformerCTC(_cfg(cfg), P)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    windows = [feats[:, c * case["step"]: c * case["step"] + case["window"]] for c in range(case["chunks"])]
    scales = model.calibrate_kv_scales(windows[:4], case["chunk_size"], margin=1.5)   # first four chunks, 50 % headroom
    assert scales.shape == (cfg.layers, 2, cfg.heads) and (scales > 0).all()
    ref_cache = model.new_streaming_cache(2, max_past, seed=1)
    q_cache = model.new_streaming_cache(2, max_past, seed=2, kv_scales=scales)
    assert q_cache.k_pool.dtype == torch.uint8
    a, b = [], []
    for xs in windows:
        a.append(model.forward_chunk_paged(xs, [0, 1], ref_cache)[..., :cfg.vocab].float())
        b.append(model.forward_chunk_paged(xs, [1, 0], q_cache)[..., :cfg.vocab].float())
    assert ob.device_status() == 0
    a, b = torch.stack(a).flatten().double(), torch.stack(b).flatten().double()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
    print(f"fp8 pages vs 16-bit pages: cosine {cos:.6f}, max-abs {(a - b).abs().max().item():.3e}")
    assert cos >= 0.999, cos


@pytest.mark.parametrize("mode", ["fp8", "int8"])
def test_streaming_with_8bit_linears_reaches_the_cosine_gate_against_the_16_bit_run(mode):
    """The chunk executor with the eight Linear GEMMs of every layer on 8-bit operands (weights per output channel,
    activations per token, the pointwise_conv1 input over the chunk and its cached left context): cosine >= 0.999
    against the 16-bit run of the same chunks, through eviction, and the same result from a graph replay."""
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case).cuda()
    ref_model = ConformerCTC(_cfg(cfg), P)
    q_model = ConformerCTC(_cfg(cfg), P, quant=mode)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    windows = [feats[:, c * case["step"]: c * case["step"] + case["window"]] for c in range(case["chunks"])]
    ref_cache = ref_model.new_streaming_cache(2, max_past, seed=1)
    q_cache = q_model.new_streaming_cache(2, max_past, seed=2)
    a, b = [], []
    for xs in windows:
        a.append(ref_model.forward_chunk_paged(xs, [0, 1], ref_cache)[..., :cfg.vocab].float())
        b.append(q_model.forward_chunk_paged(xs, [0, 1], q_cache)[..., :cfg.vocab].float())
    assert ob.device_status() == 0
    a, b = torch.stack(a), torch.stack(b)
    assert torch.isfinite(b).all()
    cos = torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()
    agree = (a.argmax(-1) == b.argmax(-1)).float().mean().item()
    print(f"{mode} streaming Linears vs 16-bit: cosine {cos:.6f}, argmax agreement {agree:.4f}, max-abs {(a - b).abs().max().item():.3e}")
    assert cos >= 0.999, cos
