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
