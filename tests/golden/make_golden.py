"""Generate the golden fixtures in this directory from the REFERENCE implementation.

Run where the reference checkout is available (it is not on the GPU box):

    OASR_REFERENCE=<path of the reference checkout> python tests/golden/make_golden.py

The script imports the reference package with its torch backend
(``OASR_LAYERS_BACKEND=torch OASR_FUSED_ADDNORM=0``), rebinds the two call
sites that have no torch route at the operator boundary (``oasr.glu`` ->
``F.glu``, ``oasr.gemm_log_softmax`` -> ``log_softmax(linear)``), loads the
seeded synthetic weights of ``oracle.conformer.init_params`` into the
reference model, runs the reference entry points on seeded inputs, checks the
CPU oracle against them and writes small ``.npz`` fixtures.  Inputs are never
stored: tests regenerate them from the same seeds.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))
REF = os.environ.get("OASR_REFERENCE")
if not REF:
    raise SystemExit("set OASR_REFERENCE to the path of the reference checkout")
os.environ["OASR_LAYERS_BACKEND"] = "torch"
os.environ["OASR_FUSED_ADDNORM"] = "0"
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

import oasr  # noqa: E402  (the reference)
from oasr.models.conformer.config import ConformerEncoderConfig, ConformerModelConfig  # noqa: E402
from oasr.models.conformer.model import ConformerModel  # noqa: E402

from oracle import conformer as OC  # noqa: E402
from oracle import ops as O  # noqa: E402
from tests.golden import cases  # noqa: E402

torch.set_grad_enabled(False)
oasr.glu = lambda x, out=None: F.glu(x, dim=-1)
oasr.gemm_log_softmax = lambda A, B, C=None, out=None: F.log_softmax(F.linear(A, B, C), dim=-1)


def build_reference_model(cfg: OC.ConformerConfig, params):
    enc = ConformerEncoderConfig(
        input_size=cfg.input_size, output_size=cfg.d_model, attention_heads=cfg.heads, linear_units=cfg.ffn,
        num_blocks=cfg.layers, cnn_module_kernel=cfg.kernel, cnn_module_norm=cfg.cnn_module_norm,
        embed_layer_norm=cfg.embed_layer_norm, causal=cfg.causal)
    model = ConformerModel(ConformerModelConfig(encoder=enc, vocab_size=cfg.vocab_padded)).eval()
    sd = model.state_dict()
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = [k for k in sd if k not in params and not k.endswith("pos_enc.pe") and "num_batches_tracked" not in k]
    assert not missing, f"oracle parameter spec misses reference tensors: {missing}"
    for name, value in params.items():
        assert name in own, f"reference model has no tensor {name}"
        assert tuple(own[name].shape) == tuple(value.shape), (name, own[name].shape, value.shape)
        own[name].data.copy_(value)
    return model


def model_case(name: str):
    case = cases.MODEL_CASES[name]
    cfg = case["cfg"]
    params = OC.init_params(cfg, seed=case["weight_seed"], perturb=case["perturb"])
    feats, lengths = cases.make_features(case)
    model = build_reference_model(cfg, params)
    out = {}
    for path, ref_fn, ora_fn in (
        ("padded", model.forward_offline, OC.forward_offline),
        ("packed", model.forward_offline_packed, OC.forward_offline_packed),
    ):
        ref_lp, ref_len = ref_fn(feats, lengths)
        ora_lp, ora_len = ora_fn(params, cfg, feats, lengths)
        assert torch.equal(ref_len.long().cpu(), ora_len.long()), (ref_len, ora_len)
        valid = torch.arange(ref_lp.shape[1])[None, :] < ora_len[:, None]
        # padding classes sit at about -1e4, where one fp32 ulp is 1e-3: compare the raw vocabulary only
        diff = (ref_lp - ora_lp)[valid][:, :cfg.vocab].abs().max().item()
        print(f"{name}/{path}: reference vs oracle max-abs over valid frames = {diff:.3e}")
        assert diff < 5e-5, "oracle does not restate the reference"
        ref_tok = OC.greedy_tokens(ref_lp, ora_len, cfg.vocab)
        assert ref_tok == OC.greedy_tokens(ora_lp, ora_len, cfg.vocab)
        out[f"{path}_out_len"] = ref_len.long().numpy()
        out[f"{path}_tokens"] = np.array([t for h in ref_tok for t in h + [-1]], dtype=np.int32)
        if case["store"] == "full":
            out[f"{path}_log_probs"] = ref_lp.numpy()
        else:  # compact: first 64 classes of every frame + per-frame (max, argmax) over the raw vocabulary
            out[f"{path}_log_probs_head"] = ref_lp[:, :, :64].numpy()
            mx = ref_lp[:, :, :cfg.vocab].max(-1)
            out[f"{path}_frame_max"] = mx.values.numpy()
            out[f"{path}_frame_argmax"] = mx.indices.numpy().astype(np.int32)
            top2 = ref_lp[:, :, :cfg.vocab].topk(2, -1).values
            out[f"{path}_frame_margin"] = (top2[..., 0] - top2[..., 1]).numpy()
    np.savez_compressed(HERE / f"model_{name}.npz", **out)


def operator_cases():
    """Operator-level outputs of the reference's own torch routes."""
    from oasr.cache.paged_kv import flat_write_index
    from oasr.functionals.attention import _sdpa_reference, _sdpa_varlen_reference, gather_paged_kv
    from oasr.functionals.gemm_torch import torch_gemm_log_softmax
    from oasr.layers.norm import _add_layer_norm_ref
    from oasr.models.conformer.packing import build_packed_layout

    out = {}
    # --- dense attention with bias, lengths, starts, causal, GQA -------------------------------
    for name, c in cases.FMHA_CASES.items():
        t = cases.make_fmha(c)
        ref = _sdpa_reference(t["q"], t["k"], t["v"], c["scale"], t.get("bias"), t.get("seqlens"), c["causal"],
                              t.get("seqstarts"))
        ora = O.fmha(t["q"], t["k"], t["v"], c["scale"], t.get("bias"), t.get("seqlens"), t.get("seqstarts"),
                     None, c["causal"])
        ref = torch.nan_to_num(ref, nan=0.0)  # SDPA gives NaN on a fully masked row; the kernel contract is 0
        d = (ref - ora).abs().max().item()
        print(f"fmha/{name}: reference vs oracle {d:.3e}")
        assert d < 2e-5
        out[f"fmha_{name}"] = ref.numpy()
    # --- paged gather + attention ----------------------------------------------------------------
    for name, c in cases.PAGED_CASES.items():
        t = cases.make_paged(c)
        kd, vd = gather_paged_kv(t["k_pool"], t["v_pool"], t["block_table"])
        ok, ov = O.gather_paged_kv(t["k_pool"], t["v_pool"], t["block_table"])
        assert torch.equal(kd, ok) and torch.equal(vd, ov)
        idx = flat_write_index(t["block_table"], t["offsets"], c["t_new"], c["block_size"])
        oidx = O.flat_write_index(t["block_table"].numpy(), t["offsets"].numpy(), c["t_new"], c["block_size"])
        assert np.array_equal(idx.numpy(), oidx)
        out[f"paged_{name}_write_index"] = idx.numpy()
        ref = _sdpa_reference(t["q"], kd, vd, c["scale"], t["bias"], t["seqlens"])
        ora = O.fmha(t["q"], t["k_pool"], t["v_pool"], c["scale"], t["bias"], t["seqlens"], None, t["block_table"])
        d = (torch.nan_to_num(ref, nan=0.0) - ora).abs().max().item()
        print(f"paged/{name}: reference vs oracle {d:.3e}")
        assert d < 2e-5
        out[f"paged_{name}_out"] = torch.nan_to_num(ref, nan=0.0).numpy()
    # --- varlen -----------------------------------------------------------------------------------
    for name, c in cases.VARLEN_CASES.items():
        t = cases.make_varlen(c)
        ref = torch.zeros_like(t["q"])
        _sdpa_varlen_reference(t["q"], t["k"], t["v"], c["scale"], t["cu"], t["cu"], t["bias"], t["bias_offsets"], ref)
        ora = O.fmha_varlen(t["q"], t["k"], t["v"], c["scale"], t["cu"], t["cu"], t["bias"], t["bias_offsets"])
        d = (ref - ora).abs().max().item()
        print(f"varlen/{name}: reference vs oracle {d:.3e}")
        assert d < 2e-5
        out[f"varlen_{name}"] = ref.numpy()
        # the packed layout index tensors (integer work, bit-exact)
        valid = torch.arange(max(c["lens"]))[None, :] < torch.tensor(c["lens"])[:, None]
        lay = build_packed_layout(valid, 15, num_heads=c["H"])
        mine = cases.packed_layout(c["lens"], 15, c["H"])
        for key in ("cu_seqlens", "pack_src_idx", "conv_gather_idx", "bias_offsets"):
            assert np.array_equal(getattr(lay, key).numpy(), mine[key]), key
            out[f"layout_{name}_{key}"] = getattr(lay, key).numpy()
    # --- add + LayerNorm and the CTC head ------------------------------------------------------------
    g = torch.Generator().manual_seed(11)
    x, r = torch.randn(5, 7, 64, generator=g), torch.randn(5, 7, 64, generator=g)
    w, b = torch.randn(64, generator=g), torch.randn(64, generator=g)
    ref_o, ref_s = _add_layer_norm_ref(x, r, w, b, 1e-5, 0.5)
    ora_o, ora_s = O.add_layer_norm_residual(x, r, w, b, 1e-5, 0.5)
    assert (ref_o - ora_o).abs().max() < 1e-6 and torch.equal(ref_s, ora_s)
    out["add_layer_norm_out"], out["add_layer_norm_sum"] = ref_o.numpy(), ref_s.numpy()
    A, B, C = torch.randn(9, 64, generator=g), torch.randn(40, 64, generator=g), torch.randn(40, generator=g)
    ref = torch.empty(9, 40)
    torch_gemm_log_softmax(ref, A, B, C, 1)
    assert (ref - O.gemm_log_softmax(A, B, C)).abs().max() < 1e-6
    out["gemm_log_softmax"] = ref.numpy()
    np.savez_compressed(HERE / "operators.npz", **out)


def stream_case():
    """Chunk-by-chunk streaming through the reference's own cache managers on the CPU
    (the per-stream driver of tests/test_pipeline.py:166-239)."""
    from oasr.cache import AttentionCacheManager, BlockPool, CacheConfig, CnnCacheManager, StreamContext

    case = cases.STREAM_CASE
    cfg = case["cfg"]
    params = OC.init_params(cfg, seed=case["weight_seed"], perturb=case["perturb"])
    model = build_reference_model(cfg, params)
    feats = cases.make_stream_features(case)
    ccfg = CacheConfig(num_layers=cfg.layers, n_kv_head=cfg.heads, head_dim=cfg.head_dim, hidden_dim=cfg.d_model,
                       kernel_size=cfg.kernel, chunk_size=case["chunk_size"], num_left_chunks=case["num_left_chunks"],
                       block_size_frames=case["chunk_size"], max_num_blocks=64, max_blocks_per_seq=16,
                       device=torch.device("cpu"), dtype=torch.float32)
    max_past = case["num_left_chunks"] * case["chunk_size"]   # commit-time eviction of the per-stream driver
    out = {}
    for sidx in range(case["streams"]):
        pool = BlockPool(ccfg)
        att_mgr, cnn_mgr = AttentionCacheManager(pool, ccfg), CnnCacheManager(ccfg)
        att_mgr.allocate_stream(sidx, slot_id=0)
        cnn_mgr.allocate_stream(sidx, slot_id=0)
        ctx = StreamContext(sidx, att_mgr, cnn_mgr)
        state = OC.StreamState(cfg)
        offset, ref_chunks, worst = 0, [], 0.0
        for c in range(case["chunks"]):
            xs = feats[sidx, c * case["step"]: c * case["step"] + case["window"]]
            ctx.prepare_chunk()
            probs = model.forward_chunk_paged(xs.unsqueeze(0), offset, ctx.get_att_caches(), ctx.get_cnn_cache(),
                                              cache_t1=int(att_mgr._cache_seqlens[0]))
            ctx.commit_chunk_paged(probs.size(1))
            offset += probs.size(1)
            mine = OC.forward_chunk(params, cfg, state, xs, max_past)
            worst = max(worst, (probs[0] - mine)[:, :cfg.vocab].abs().max().item())
            ref_chunks.append(probs[0])
        print(f"stream {sidx}: reference vs oracle max-abs over {case['chunks']} chunks = {worst:.3e}")
        assert worst < 5e-5, "streaming oracle does not restate the reference"
        out[f"stream{sidx}_log_probs"] = torch.stack(ref_chunks).numpy()
    np.savez_compressed(HERE / "stream_tiny.npz", **out)


def fastconformer_case():
    """Layer stack of the reference's NemotronEncoder (its own layers, masks and position table, random weights
    from the oracle's seeded initialiser) on a ragged batch of post-subsampling hidden states."""
    from oasr.models.nemotron.config import NemotronEncoderConfig
    from oasr.models.nemotron.encoder import (NemotronEncoderLayer, chunked_limited_mask,
                                              relative_position_embedding)
    from oracle import fastconformer as OF

    cfg = OF.TINY
    case = cases.FASTCONFORMER_CASE
    rc = NemotronEncoderConfig(hidden_size=cfg.hidden, num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                               num_key_value_heads=cfg.heads, intermediate_size=cfg.ffn, conv_kernel_size=cfg.kernel,
                               sliding_window=cfg.sliding_window, default_num_lookahead_tokens=cfg.lookahead,
                               attention_bias=cfg.bias, convolution_bias=cfg.bias)
    P = OF.init_params(cfg, case["weight_seed"])
    layers = torch.nn.ModuleList(NemotronEncoderLayer(rc) for _ in range(cfg.layers)).eval()
    missing, unexpected = layers.load_state_dict({k[len("layers."):]: v for k, v in P.items()}, strict=True)
    hidden = cases.make_fastconformer_hidden(case, cfg)
    lengths = torch.tensor(case["lengths"])
    t_out = hidden.size(1)
    with torch.no_grad():
        keep = torch.arange(t_out).unsqueeze(0) < lengths.unsqueeze(1)
        window = chunked_limited_mask(t_out, t_out, cfg.sliding_window - 1, cfg.lookahead, hidden.device)
        attn_mask = window & keep.view(-1, 1, 1, t_out)
        silent = attn_mask.logical_not().all(dim=-1).transpose(1, 2)
        if not bool(silent.any()):
            silent = None
        pos_emb = relative_position_embedding(t_out, cfg.hidden, hidden.device, hidden.dtype)
        x = hidden
        for layer in layers:
            x = layer(x, pos_emb, attn_mask, silent)
        mine = OF.layers_forward(P, cfg, hidden, case["lengths"])
    d = (x - mine).abs().max().item()
    print(f"fastconformer layer stack: reference vs oracle max-abs = {d:.3e} (silent rows: {silent is not None})")
    assert d < 5e-5, "FastConformer oracle does not restate the reference"
    # whole encoder: the reference's NemotronEncoder (subsampling + layers) on ragged mel features
    from oasr.models.nemotron.encoder import NemotronEncoder

    sub, ecase = OF.TINY_SUB, cases.FASTCONFORMER_ENCODER_CASE
    rc.num_mel_bins, rc.subsampling_conv_channels = sub.mels, sub.channels
    enc = NemotronEncoder(rc).eval()
    PE = dict(OF.init_params(cfg, ecase["weight_seed"]))
    PE.update(OF.init_subsampling_params(sub, cfg.hidden, ecase["sub_seed"]))
    enc.load_state_dict(PE, strict=True)
    feats = cases.make_fastconformer_features(ecase, sub)
    with torch.no_grad():
        ref_hidden, ref_mask = enc(feats, torch.tensor(ecase["lengths"]))
        mine_hidden, mine_len = OF.encoder_forward(PE, cfg, sub, feats, ecase["lengths"])
    ref_len = ref_mask.squeeze(1).sum(-1)
    assert torch.equal(ref_len, mine_len), (ref_len, mine_len)
    de = (ref_hidden - mine_hidden).abs().max().item()
    print(f"fastconformer encoder: reference vs oracle max-abs = {de:.3e}, out lengths {mine_len.tolist()}")
    assert de < 1e-4, "FastConformer encoder oracle does not restate the reference"
    np.savez_compressed(HERE / "fastconformer_tiny.npz", hidden_out=x.numpy(), encoder_out=ref_hidden.numpy(),
                        encoder_len=ref_len.numpy())


if __name__ == "__main__":
    if "--only-fastconformer" in sys.argv:
        fastconformer_case()
        sys.exit(0)
    fastconformer_case()
    stream_case()
    operator_cases()
    for name in cases.MODEL_CASES:
        model_case(name)
    print("fixtures written to", HERE)
