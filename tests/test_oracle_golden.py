"""CPU: the oracle reproduces the fixtures written from the reference (tests/golden/make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import conformer as OC
from oracle import ops as O
from tests.golden import cases

GOLD = Path(__file__).resolve().parent / "golden"
OPS = np.load(GOLD / "operators.npz")


@pytest.mark.parametrize("name", list(cases.FMHA_CASES))
def test_fmha_oracle(name):
    c = cases.FMHA_CASES[name]
    t = cases.make_fmha(c)
    got = O.fmha(t["q"], t["k"], t["v"], c["scale"], t.get("bias"), t.get("seqlens"), t.get("seqstarts"), None,
                 c["causal"])
    assert np.abs(got.numpy() - OPS[f"fmha_{name}"]).max() < 2e-5


def test_fully_masked_rows_are_zero():
    c = cases.FMHA_CASES["starts"]
    t = cases.make_fmha(c)
    got = O.fmha(t["q"], t["k"], t["v"], c["scale"], t["bias"], t["seqlens"], t["seqstarts"])
    assert torch.count_nonzero(got[2]) == 0  # window [40, 40) is empty


@pytest.mark.parametrize("name", list(cases.PAGED_CASES))
def test_paged_oracle(name):
    c = cases.PAGED_CASES[name]
    t = cases.make_paged(c)
    idx = O.flat_write_index(t["block_table"].numpy(), t["offsets"].numpy(), c["t_new"], c["block_size"])
    assert np.array_equal(idx, OPS[f"paged_{name}_write_index"])
    got = O.fmha(t["q"], t["k_pool"], t["v_pool"], c["scale"], t["bias"], t["seqlens"], None, t["block_table"])
    assert np.abs(got.numpy() - OPS[f"paged_{name}_out"]).max() < 2e-5


@pytest.mark.parametrize("name", list(cases.VARLEN_CASES))
def test_varlen_oracle_and_layout(name):
    c = cases.VARLEN_CASES[name]
    t = cases.make_varlen(c)
    got = O.fmha_varlen(t["q"], t["k"], t["v"], c["scale"], t["cu"], t["cu"], t["bias"], t["bias_offsets"])
    assert np.abs(got.numpy() - OPS[f"varlen_{name}"]).max() < 2e-5
    lay = cases.packed_layout(c["lens"], 15, c["H"])
    for key in ("cu_seqlens", "pack_src_idx", "conv_gather_idx", "bias_offsets"):
        assert np.array_equal(lay[key], OPS[f"layout_{name}_{key}"])


def test_add_layer_norm_and_head_oracle():
    g = torch.Generator().manual_seed(11)
    x, r = torch.randn(5, 7, 64, generator=g), torch.randn(5, 7, 64, generator=g)
    w, b = torch.randn(64, generator=g), torch.randn(64, generator=g)
    o, s = O.add_layer_norm_residual(x, r, w, b, 1e-5, 0.5)
    assert np.abs(o.numpy() - OPS["add_layer_norm_out"]).max() < 1e-6
    assert np.array_equal(s.numpy(), OPS["add_layer_norm_sum"])
    A, B, C = torch.randn(9, 64, generator=g), torch.randn(40, 64, generator=g), torch.randn(40, generator=g)
    assert np.abs(O.gemm_log_softmax(A, B, C).numpy() - OPS["gemm_log_softmax"]).max() < 1e-6


def test_paged_write_then_gather_roundtrip():
    c = dict(cases.PAGED_CASES["bs16"])
    t = cases.make_paged(c)
    g = torch.Generator().manual_seed(5)
    new_k = torch.randn(c["B"], c["Hkv"], c["t_new"], c["D"], generator=g)
    new_v = torch.randn(c["B"], c["Hkv"], c["t_new"], c["D"], generator=g)
    O.write_kv_chunk(t["k_pool"], t["v_pool"], new_k, new_v, t["block_table"], t["offsets"], c["block_size"])
    kd, vd = O.gather_paged_kv(t["k_pool"], t["v_pool"], t["block_table"])
    for b in range(c["B"]):
        o = int(t["offsets"][b])
        assert torch.equal(kd[b, :, o:o + c["t_new"]], new_k[b]) and torch.equal(vd[b, :, o:o + c["t_new"]], new_v[b])


@pytest.mark.parametrize("name", ["tiny", "config1"])
def test_model_oracle_matches_reference_fixture(name):
    case = cases.MODEL_CASES[name]
    cfg = case["cfg"]
    gold = np.load(GOLD / f"model_{name}.npz")
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats, lengths = cases.make_features(case)
    for path, fn in (("padded", OC.forward_offline), ("packed", OC.forward_offline_packed)):
        lp, out_len = fn(P, cfg, feats, lengths)
        assert np.array_equal(out_len.numpy(), gold[f"{path}_out_len"])
        valid = (torch.arange(lp.shape[1])[None, :] < out_len[:, None]).numpy()
        if case["store"] == "full":
            d = np.abs(lp.numpy() - gold[f"{path}_log_probs"])[valid][:, :cfg.vocab].max()
        else:
            d = np.abs(lp[:, :, :64].numpy() - gold[f"{path}_log_probs_head"])[valid].max()
            mx = lp[:, :, :cfg.vocab].max(-1)
            d = max(d, np.abs(mx.values.numpy() - gold[f"{path}_frame_max"])[valid].max())
        assert d < 5e-5, d
        toks = OC.greedy_tokens(lp, out_len, cfg.vocab)
        flat = np.array([t for h in toks for t in h + [-1]], dtype=np.int32)
        assert np.array_equal(flat, gold[f"{path}_tokens"])


def test_package_weight_init_equals_oracle_init():
    """The product's seeded init and the oracle's are the same tensors, so GPU runs and the
    CPU baseline see identical weights."""
    from oasr_b200.encoder import ConformerConfig
    from oasr_b200.weights import init_params

    cfg = OC.TINY
    mine = init_params(ConformerConfig(**{f: getattr(cfg, f) for f in ConformerConfig.__dataclass_fields__}), 99)
    theirs = OC.init_params(cfg, 99, 0.0)
    assert list(mine) == list(theirs)
    assert all(torch.equal(mine[k], theirs[k]) for k in mine)


def test_streaming_oracle_matches_reference_fixture():
    """Chunk-by-chunk oracle (cached K/V, conv left context, block eviction) vs the fixture written
    from the reference's forward_chunk_paged driven by its own cache managers."""
    case = cases.STREAM_CASE
    cfg = case["cfg"]
    gold = np.load(GOLD / "stream_tiny.npz")
    P = OC.init_params(cfg, case["weight_seed"], case["perturb"])
    feats = cases.make_stream_features(case)
    max_past = case["num_left_chunks"] * case["chunk_size"]
    for s in range(case["streams"]):
        state = OC.StreamState(cfg)
        for c in range(case["chunks"]):
            xs = feats[s, c * case["step"]: c * case["step"] + case["window"]]
            lp = OC.forward_chunk(P, cfg, state, xs, max_past)
            assert lp.shape[0] == case["chunk_size"]
            d = np.abs(lp.numpy() - gold[f"stream{s}_log_probs"][c])[:, :cfg.vocab].max()
            assert d < 5e-5, (s, c, d)
        assert state.k[0].shape[1] <= max_past + case["chunk_size"]


def test_fastconformer_oracle_matches_reference_fixture():
    """The FastConformer / Nemotron layer-stack oracle against the output of the reference's own layers
    (fixture written by tests/golden/make_golden.py from NemotronEncoderLayer on the CPU)."""
    from oracle import fastconformer as OFC

    gold = np.load(GOLD / "fastconformer_tiny.npz")
    cfg, case = OFC.TINY, cases.FASTCONFORMER_CASE
    P = OFC.init_params(cfg, case["weight_seed"])
    hidden = cases.make_fastconformer_hidden(case, cfg)
    out = OFC.layers_forward(P, cfg, hidden, case["lengths"]).numpy()
    assert np.abs(out - gold["hidden_out"]).max() < 5e-5
    # the relative shift identity the reference pins in its own tests: row i, column j holds source column (L-1)+j-i
    L = 5
    src = torch.arange(2 * L - 1, dtype=torch.float32).expand(1, 1, L, 2 * L - 1).contiguous()
    sh = OFC.rel_shift(src)[0, 0, :, :L]
    want = torch.tensor([[(L - 1) + j - i for j in range(L)] for i in range(L)], dtype=torch.float32)
    assert torch.equal(sh, want)


def test_fastconformer_encoder_oracle_matches_reference_fixture():
    """Whole FastConformer encoder oracle (8x subsampling + layer stack) against the reference's NemotronEncoder output."""
    from oracle import fastconformer as OFC

    gold = np.load(GOLD / "fastconformer_tiny.npz")
    cfg, sub, case = OFC.TINY, OFC.TINY_SUB, cases.FASTCONFORMER_ENCODER_CASE
    P = dict(OFC.init_params(cfg, case["weight_seed"]))
    P.update(OFC.init_subsampling_params(sub, cfg.hidden, case["sub_seed"]))
    feats = cases.make_fastconformer_features(case, sub)
    out, out_len = OFC.encoder_forward(P, cfg, sub, feats, case["lengths"])
    assert out_len.tolist() == gold["encoder_len"].tolist()
    assert np.abs(out.numpy() - gold["encoder_out"]).max() < 1e-4


def test_unshifted_position_term_factorises_in_the_oracle():
    """The packed relative-position scores carry no relative shift (matrix_bd[i, j] = (q_i + v) . p_j), so
    (q_i + u) . k_j + (q_i + v) . p_j = q_i . (k_j + p_j) + (u . k_j + v . p_j): one product against k + p plus a
    per-key, per-head constant.  Checked on the oracle's own tensors in float64 -- the identity a leaner projection /
    attention pair could use (three output blocks instead of four, half the query bytes per tile)."""
    torch.manual_seed(0)
    H, dk, T = 4, 64, 37
    q, k, p = (torch.randn(H, T, dk, dtype=torch.float64) for _ in range(3))
    u, v = torch.randn(H, 1, dk, dtype=torch.float64), torch.randn(H, 1, dk, dtype=torch.float64)
    want = (q + u) @ k.transpose(-1, -2) + (q + v) @ p.transpose(-1, -2)          # the oracle's two terms (conformer.py:219-224)
    c = (u * k).sum(-1) + (v * p).sum(-1)                                          # (H, T): per key and head
    got = q @ (k + p).transpose(-1, -2) + c.unsqueeze(1)
    assert (got - want).abs().max().item() < 1e-10
