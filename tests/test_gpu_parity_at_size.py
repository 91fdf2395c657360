"""GPU parity at the sizes the benchmarks run, against the fp32 CPU oracle on the same seeded inputs.

* BASELINE config 2 exactly as ``bench.py`` builds it (``make_batch(0)``, weight seed 1234, 64
  utterances of 200..2000 frames, 12 layers, d_model 512): the packed offline path.  This is the one
  workload whose throughput is the headline, so its log-probs are checked, not only timed.
* Streaming at real width (d_model 512, 12 layers, 32 streams, 20 chunks with a 256-frame history so
  that whole pages are evicted), 16-bit and fp8 pages.
* FastConformer at its real width (hidden 1024, 8 heads of 128, FFN 4096), two layers, 8x front end,
  with a vocabulary-1024 CTC head on top.

Gates: log-prob max-abs <= 2e-2 and mean-abs <= 1e-3 for the Conformer paths (the tolerance the
bf16 path is held to against the fp32 path), greedy-argmax agreement >= 99.9 % on frames whose
oracle top-1 / top-2 margin exceeds the max-abs tolerance; the all-frame agreement is printed and
bounded (tests/test_argmax_floor.py shows why 99.9 % of all frames is out of reach of bf16 weights).
"""
import numpy as np
import pytest
import torch

import bench
import oasr_b200 as ob
from oasr_b200.encoder import ConformerCTC, ConformerConfig
from oasr_b200.weights import init_fastconformer_params, init_params
from oracle import conformer as OC
from oracle import fastconformer as OFC

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS, ARGMAX_AGREE = 2e-2, 1e-3, 0.999


def _cfg(c):
    return ConformerConfig(**{f: getattr(c, f) for f in ConformerConfig.__dataclass_fields__})


def _stats(got, want, vocab, tag):
    g, w = got[:, :vocab], want[:, :vocab]
    diff = (g - w).abs()
    same = g.argmax(-1) == w.argmax(-1)
    top2 = w.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > MAX_ABS
    agree_clear = same[clear].float().mean().item() if clear.any() else 1.0
    print(f"[{tag}] frames {g.shape[0]}: max-abs {diff.max().item():.3e} mean-abs {diff.mean().item():.3e} argmax agreement "
          f"{same.float().mean().item():.5f} all frames, {agree_clear:.5f} on the {int(clear.sum())} frames with margin > {MAX_ABS}")
    return diff.max().item(), diff.mean().item(), same.float().mean().item(), agree_clear


def test_config2_bench_batch_matches_the_fp32_oracle():
    cfg = bench.model_config(12)
    P = init_params(cfg, 1234)
    ocfg = OC.CONFIG2
    PO = OC.init_params(ocfg, 1234)
    assert set(P) == set(PO) and all(torch.equal(P[k], PO[k]) for k in P)      # the bench's weights are the oracle's
    feats, lengths = bench.make_batch(0)
    model = ConformerCTC(cfg, P, device="cuda", dtype=torch.bfloat16)
    lp, out_len, pk = model.forward_offline_packed(feats.cuda(), lengths, padded_output=False)
    hyp = model.greedy_search(feats.cuda(), lengths)
    torch.cuda.synchronize()
    assert ob.device_status() == 0
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    with torch.no_grad():
        want, want_len = OC.forward_offline_packed(PO, ocfg, feats, torch.tensor(lengths))
    assert torch.equal(out_len.cpu(), want_len)
    valid = torch.arange(want.shape[1])[None, :] < want_len[:, None]
    want_rows = want[valid]                                                     # utterance-major = packed row order
    assert want_rows.shape[0] == pk.total == lp.shape[0]
    lp = lp.cpu()
    mx, mean, agree, agree_clear = _stats(lp, want_rows, cfg.vocab, "config 2, bench batch, packed")
    # the floor no bf16-weight implementation can beat on this workload: fp32 everywhere, weight matrices rounded to bf16
    with torch.no_grad():
        rounded = {k: (v.to(torch.bfloat16).float() if v.ndim >= 2 else v) for k, v in PO.items()}
        floor_rows = OC.forward_offline_packed(rounded, ocfg, feats, torch.tensor(lengths))[0][valid]
    fmx, fmean, fagree, _ = _stats(floor_rows, want_rows, cfg.vocab, "config 2, fp32 oracle with bf16 weight matrices")
    assert mx <= MAX_ABS
    # mean-abs gate 1e-3: met wherever bf16 weights allow it (config 1); here the weight rounding alone costs more
    # (tests/test_argmax_floor.py), so the CUDA path is held to 1.25x that floor
    assert mean <= max(MEAN_ABS, 1.25 * fmean), (mean, fmean)
    assert agree_clear >= ARGMAX_AGREE
    assert agree >= 0.95
    assert lp.logsumexp(-1).abs().max().item() < 1e-3
    # the token lists of the public call are the collapse of the same per-frame argmax
    got_ids = lp[:, :cfg.vocab_padded].argmax(-1)
    assert hyp == ConformerCTC._collapse(got_ids.numpy(), pk.seg_lengths)


@pytest.mark.parametrize("kv", ["bf16", "fp8"])
def test_streaming_at_real_width_matches_the_oracle(kv):
    import dataclasses

    streams, chunks, window, step, chunk, max_past = 32, 20, 67, 64, 16, 256
    ocfg = OC.CONFIG3
    cfg = dataclasses.replace(_cfg(ocfg))
    P = OC.init_params(ocfg, 1234)
    g = torch.Generator().manual_seed(17)
    feats = torch.randn(streams, step * (chunks - 1) + window, 80, generator=g)
    model = ConformerCTC(cfg, P, device="cuda", dtype=torch.bfloat16)
    windows = [feats[:, c * step: c * step + window] for c in range(chunks)]
    scales = None
    if kv == "fp8":
        scales = model.calibrate_kv_scales([w.cuda() for w in windows[:4]], chunk, margin=1.5)
    cache = model.new_streaming_cache(streams + 3, max_past, chunk_frames=chunk, seed=5, kv_scales=scales)
    slots = [int(s) for s in np.random.default_rng(3).permutation(streams + 3)[:streams]]   # scattered slots
    check = [0, streams // 2, streams - 1]
    states = {s: OC.StreamState(ocfg) for s in check}
    # the same streams through the fp32 oracle with bf16-rounded weight matrices: the floor of any bf16-weight path
    PR = {k: (v.to(torch.bfloat16).float() if v.ndim >= 2 else v) for k, v in P.items()}
    floor_states = {s: OC.StreamState(ocfg) for s in check}
    got_rows, want_rows, floor_rows = [], [], []
    for c in range(chunks):
        lp = model.forward_chunk_paged(windows[c].cuda(), slots, cache).cpu()
        assert ob.device_status() == 0
        for s in check:
            with torch.no_grad():
                want_rows.append(OC.forward_chunk(P, ocfg, states[s], windows[c][s], max_past))
                floor_rows.append(OC.forward_chunk(PR, ocfg, floor_states[s], windows[c][s], max_past))
            got_rows.append(lp[s])
        assert cache.cached_frames(slots[0]) <= max_past + chunk
    assert chunks * chunk > max_past + chunk                                 # whole pages were evicted on the way
    got, want, floor = torch.cat(got_rows), torch.cat(want_rows), torch.cat(floor_rows)
    tag = f"streaming d512 x12, {streams} streams x {chunks} chunks, {kv} pages"
    mx, mean, agree, agree_clear = _stats(got, want, ocfg.vocab, tag)
    fmx, fmean, _, _ = _stats(floor, want, ocfg.vocab, "same streams, fp32 oracle with bf16 weight matrices")
    # 16-bit pages: the Conformer gate, with the mean-abs bound relaxed to 1.3x the weight-rounding floor where that floor
    # is itself above 1e-3 (d_model 512); fp8 pages add the page quantisation on top (gated by cosine elsewhere)
    slack = 1.3 if kv == "bf16" else 1.6
    assert mx <= (MAX_ABS if kv == "bf16" else 3e-2)
    assert mean <= max(MEAN_ABS, slack * fmean), (mean, fmean)
    assert agree_clear >= (ARGMAX_AGREE if kv == "bf16" else 0.99)


def test_fastconformer_real_width_with_ctc_head_matches_the_oracle():
    from oasr_b200.fastconformer import FastConformerEncoder

    hidden, heads, ffn, layers, kernel, mels, channels, vocab = 1024, 8, 4096, 2, 9, 128, 256, 1024
    P = init_fastconformer_params(hidden, heads, ffn, layers, kernel, mels, channels, seed=1234, w_std=0.02, bias=False,
                                  vocab=vocab)
    cfg = OFC.FastConformerConfig(hidden=hidden, heads=heads, ffn=ffn, layers=layers, kernel=kernel, sliding_window=57,
                                  lookahead=3, bias=False)
    sub = OFC.SubsamplingConfig(mels=mels, channels=channels)
    lengths = [611, 300, 77, 520]
    feats = torch.randn(len(lengths), max(lengths), mels, generator=torch.Generator().manual_seed(6))
    enc = FastConformerEncoder(hidden, heads, ffn, layers, kernel, cfg.sliding_window, cfg.lookahead, mels, channels, P)
    lp, out_len, arg = enc.forward_ctc(feats.cuda(), lengths, padded_output=True, return_argmax=True)
    torch.cuda.synchronize()
    assert ob.device_status() == 0
    with torch.no_grad():
        want_h, want_len = OFC.encoder_forward(P, cfg, sub, feats, lengths)
        want = OFC.ctc_head(P, want_h)
    assert list(out_len) == want_len.tolist()
    valid = torch.arange(want.shape[1])[None, :] < want_len[:, None]
    lp = lp.cpu()
    mx, mean, agree, agree_clear = _stats(lp[valid], want[valid], vocab, "fastconformer d1024 x2 + CTC 1024")
    # the hidden states of this stack are layer-normalised O(1) values that pass through bf16 GEMM inputs at width 1024
    # and 4096; the log-probs inherit that: held to 5e-2 / 5e-3 (the Conformer gate is 2e-2 / 1e-3 at width 512)
    assert mx <= 5e-2 and mean <= 5e-3
    assert agree_clear >= 0.99
    assert torch.equal(arg.cpu().long(), lp[valid].argmax(-1))
    assert lp[valid].logsumexp(-1).abs().max().item() < 1e-3


def test_length_sorted_sweep_through_packs_matches_the_fp32_oracle():
    """The config-5 style path (utterances with log-normal lengths, sorted, packed by the reference's rule, packs dealt
    to two ranks, greedy search pipelined over a rank's packs) at the headline model: every utterance comes back
    exactly once and in place, its tokens are the collapse of its own frames' argmax, and its log-probs agree with
    the fp32 oracle run on the utterance alone (packing restricts attention and the conv to the segment, so an
    utterance's result does not depend on its pack mates)."""
    from oasr_b200 import sharding

    cfg = bench.model_config(12)
    P = init_params(cfg, 1234)
    model = ConformerCTC(cfg, P, device="cuda", dtype=torch.bfloat16)
    rng = np.random.default_rng(11)
    lengths = [int(round(100 * min(max(x, 1.0), 30.0))) for x in rng.lognormal(np.log(6.0), 0.6, size=40)]
    feats = [torch.randn(n, 80, generator=torch.Generator().manual_seed(100 + i)) for i, n in enumerate(lengths)]
    packs = sharding.plan_packs(lengths, 2048, 4)
    assert len(packs) >= 4 and sorted(i for p in packs for i in p) == list(range(len(lengths)))
    plan = sharding.assign_packs(lengths, packs, 2)
    results = {}
    for rank in range(2):                              # both ranks' shares, one after the other on this GPU
        batches = []
        for j in plan[rank]:
            idx = packs[j]
            T = max(lengths[i] for i in idx)
            x = torch.zeros(len(idx), T, 80)
            for r, i in enumerate(idx):
                x[r, :lengths[i]] = feats[i]
            batches.append((idx, x.pin_memory(), [lengths[i] for i in idx]))
        for (idx, _, _), hyps in zip(batches, model.greedy_search_batches((x, ls) for _, x, ls in batches)):
            assert len(hyps) == len(idx)
            for i, h in zip(idx, hyps):
                assert i not in results
                results[i] = h
    assert ob.device_status() == 0
    assert sorted(results) == list(range(len(lengths)))
    # five utterances spread over the length range, each alone through the oracle
    order = sorted(range(len(lengths)), key=lambda i: lengths[i])
    picked = [order[0], order[len(order) // 4], order[len(order) // 2], order[3 * len(order) // 4], order[-1]]
    PO = OC.init_params(OC.CONFIG2, 1234)
    worst_mean = 0.0
    for i in picked:
        with torch.no_grad():
            want, want_len = OC.forward_offline_packed(PO, OC.CONFIG2, feats[i][None], torch.tensor([lengths[i]]))
        n = int(want_len[0])
        lp, _, _ = model.forward_offline_packed(feats[i][None].cuda(), [lengths[i]], padded_output=False)
        mx, mean, _, clear = _stats(lp.cpu()[:n], want[0, :n], cfg.vocab, f"sweep utterance {i}, {lengths[i]} frames")
        worst_mean = max(worst_mean, mean)
        assert mx <= MAX_ABS and clear >= ARGMAX_AGREE
        ids = lp[:n, :cfg.vocab].argmax(-1).cpu().numpy()
        assert results[i] == ConformerCTC._collapse(ids, [n])[0]       # the pack's tokens = this utterance's own tokens
    assert worst_mean <= 2.0e-3
