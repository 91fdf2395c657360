#!/usr/bin/env python
"""Headline benchmark: offline Conformer encoder + CTC throughput in audio-seconds / second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE config 2): 12-layer Conformer, d_model 512, 8 heads, FFN 2048, conv
kernel 15, 80-dim fbank, 4x Conv2d subsampling, CTC vocabulary 5002 (head padded to 5008),
bf16 compute, random-init weights from a seed; one step = one batch of 64 utterances with
lengths uniform in 200..2000 frames (10 ms hop), features iid N(0,1), sequence-packed.
Synthetic features stand in for real audio (no dataset is available offline).

One JSON line is printed by rank 0:
  value      features already in HBM, features -> packed fp32 log-probs + per-frame argmax,
             device-timed per step with CUDA events (L2 flushed between steps)
  e2e        the public call a user makes (ConformerCTC.greedy_search_batches): per step pinned
             host features -> H2D -> encoder + head -> D2H of the per-frame argmax -> token lists,
             the copies of neighbouring steps overlapped with compute on a copy stream
  roofline   the dominant kernel (the tcgen05 GEMM): algorithmic flops / CUDA-event time of
             its launches in an instrumented extra step, against the measured bf16 peak
  cpu_baseline  the fp32 CPU oracle (a port of the reference's torch path) on a bounded sample
Under torchrun every rank runs its own batch (utterance-sharded, no collective on the data
path); time is the max over ranks, value the sum of audio over ranks divided by it.

``--impl reference`` times the reference's own fp32 torch path on the host cores, the whole batch per
step: the reference's ``ConformerModel.forward_offline_packed`` from the copy under ``oracle/_ref``
(made by ``oracle/make_ref.py``; ``kind: "reference"``) when that copy is present, else the CPU port
``oracle.conformer`` (``kind: "port"``, pinned to the reference at 2e-6), and prints the same line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FRAME_S = 0.01
WORKLOAD = "conformer12_d512_h8_ffn2048_k15_vocab5002_b64_len200-2000_packed"
CPU_SAMPLE_UTTS = 8


def deal_lengths(rank: int, world: int, batch: int = 64):
    """The job's utterances are the ``world`` seeded draws of ``batch`` lengths (numpy default_rng(2024 + r)); one rank
    keeps its own draw, several ranks deal the pool so that every rank gets ``batch`` utterances of about equal total
    length (longest first, each to the lightest rank that still has room), as a length-aware loader shards a job: the
    step time is the slowest rank's."""
    draws = [[int(x) for x in np.random.default_rng(2024 + r).integers(200, 2001, size=batch)] for r in range(world)]
    if world == 1:
        return draws[0]
    pool = sorted((n for d in draws for n in d), reverse=True)
    load, mine = [0] * world, [[] for _ in range(world)]
    for n in pool:
        r = min((i for i in range(world) if len(mine[i]) < batch), key=lambda i: load[i])
        mine[r].append(n)
        load[r] += n
    order = np.random.default_rng(99 + rank).permutation(batch)          # no length order inside a rank's batch
    return [mine[rank][i] for i in order]


def make_batch(rank: int, batch: int = 64, world: int = 1):
    """Seeded lengths (``deal_lengths``) and features (torch seed 7 + rank)."""
    lengths = deal_lengths(rank, world, batch)
    g = torch.Generator().manual_seed(7 + rank)
    feats = torch.randn(batch, max(lengths), 80, generator=g)
    return feats, lengths


def model_config(layers: int = 12):
    from oasr_b200.encoder import ConformerConfig

    return ConformerConfig(input_size=80, d_model=512, heads=8, ffn=2048, layers=layers, kernel=15, vocab=5002)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def gemm_flops(name, args):
    """Algorithmic flops (2*M*N*K) of one GEMM-family C-ABI call from its integer arguments."""
    if name == "oasr_b200_gemm":
        M, N, K = args[4], args[5], args[6]
    elif name == "oasr_b200_gemm_glu":
        M, N, K = args[4], 2 * args[5], args[6]
    elif name == "oasr_b200_gemm_log_softmax":
        M, N, K = args[4], args[5], args[6]
    elif name == "oasr_b200_subsample_conv2":   # implicit GEMM: rows = frames x F2 positions, K = 9 taps x C
        F2 = (args[7] - 3) // 2 + 1
        M, N, K = args[10] * F2, args[9], 9 * args[8]
    elif name == "oasr_b200_gemm_residual_f32":
        M, N, K = args[5], args[6], args[7]
    else:
        return None
    return 2.0 * M * N * K


def instrumented_step(run_step):
    """One extra step with CUDA-event pairs on the launching stream: around every step of the
    native executor (its own event records) and around every other C-ABI call (Python hook)."""
    from oasr_b200 import _lib

    records, open_ev = [], {}

    def hook(name, phase, args):
        if name in ("oasr_b200_conformer_encode_packed", "oasr_b200_conformer_chunk_paged", "oasr_b200_profile_enable",
                    "oasr_b200_profile_get"):
            return
        if phase == "begin":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            open_ev[name] = ev
        else:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            records.append((name.replace("oasr_b200_", ""), open_ev.pop(name), end, gemm_flops(name, args)))

    _lib.set_call_hook(hook)
    try:
        native = _lib.profile_steps(run_step)
        torch.cuda.synchronize()
    finally:
        _lib.set_call_hook(None)
    per = {}

    def add(label, ms, fl):
        d = per.setdefault(label, {"launches": 0, "ms": 0.0, "flops": 0.0})
        d["launches"] += 1
        d["ms"] += ms
        d["flops"] += fl or 0.0

    for name, a, b, fl in records:
        add(name, a.elapsed_time(b), fl)
    for label, ms, fl in native:
        add(label, ms, fl)
    return per


_CPU_MODEL = {}


def _cpu_forward():
    """(kind, callable(feats, lengths) -> log_probs) of the CPU arm: the reference's own model from oracle/_ref when
    present, else the oracle port.  Built once per process."""
    if "fn" in _CPU_MODEL:
        return _CPU_MODEL["kind"], _CPU_MODEL["fn"]
    from oracle import conformer as OC
    from oracle import make_ref

    cfg = OC.CONFIG2
    P = OC.init_params(cfg, 1234)
    kind, fn = "port", (lambda f, lt: OC.forward_offline_packed(P, cfg, f, lt)[0])
    if make_ref.available():
        try:
            from oracle import ref_model

            ref_model.load_torch_route()
            model = ref_model.build_conformer(cfg, P)
            kind, fn = "reference", (lambda f, lt: model.forward_offline_packed(f, lt)[0])
        except Exception as e:   # an import problem of the copy must not take the bench down: fall back to the port
            print(f"[bench] oracle/_ref could not be used ({type(e).__name__}: {e}); timing the CPU port", file=sys.stderr)
    _CPU_MODEL.update(kind=kind, fn=fn)
    return kind, fn


def cpu_throughput(sample_utts: int, repeats: int = 1, threads=None):
    """audio-s/s of the fp32 CPU arm on the first `sample_utts` utterances of rank 0's batch:
    (value, audio_s, best_seconds, threads, kind)."""
    if threads:
        torch.set_num_threads(threads)
    kind, fn = _cpu_forward()
    feats, lengths = make_batch(0)
    lens = lengths[:sample_utts]
    f = feats[:sample_utts, :max(lens)].contiguous()
    lt = torch.tensor(lens, dtype=torch.int64)
    audio_s = sum(lens) * FRAME_S
    with torch.no_grad():
        best = None
        for _ in range(repeats):
            t0 = time.perf_counter()
            fn(f, lt)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    return audio_s / best, audio_s, best, torch.get_num_threads(), kind


def offline_config(batch: int, layers: int, world: int, audio_per_step: float):
    """The ``config`` object of the headline workload, shared by both arms."""
    workload = WORKLOAD if (batch, layers) == (64, 12) else \
        f"REDUCED profiling case: conformer{layers}_d512_h8_ffn2048_k15_vocab5002_b{batch}_len200-2000_packed"
    return {"workload": workload, "global_batch": batch * world,
            "parallelism": f"utterance-sharded x{world} (utterances dealt by length, {batch} per rank), no collective",
            "l2": "256 MiB flush write between steps; per-step working set (weights 240 MB + activations) > 126 MB L2",
            "output": "packed (total_frames, 5008) fp32 log-probs + per-frame argmax (padded_output=False: the (B, T', V) "
                      "re-padding of forward_offline_packed is not in the timed step)",
            "audio_seconds_per_step": audio_per_step}


REFERENCE_ARM_BUDGET_S = 150.0


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    for _ in range(max(args.warmup, 1)):
        v8, _, dt8, _, kind = cpu_throughput(4)
    # the whole 64-utterance batch per step when K steps of it fit the time budget, else the largest prefix that does
    feats, lengths = make_batch(0, args.batch, 1)
    full_audio = sum(lengths) * FRAME_S
    est_full = full_audio / v8
    n = args.batch
    if est_full * args.steps > REFERENCE_ARM_BUDGET_S:
        n = max(4, min(args.batch, int(args.batch * REFERENCE_ARM_BUDGET_S / (est_full * args.steps))))
    times, audio = [], 0.0
    for _ in range(args.steps):
        v, a, dt, thr, kind = cpu_throughput(n)
        times.append(dt)
        audio += a
    value = audio / sum(times)
    sample = (f"all {args.batch} utterances of the batch per step" if n == args.batch else
              f"first {n} of the {args.batch} utterances per step (the whole batch for {args.steps} steps would exceed "
              f"{REFERENCE_ARM_BUDGET_S:.0f} s)") + \
             (", the reference's ConformerModel.forward_offline_packed (torch backend, fp32) from oracle/_ref" if kind == "reference"
              else ", CPU port of the reference's fp32 packed path (oracle.conformer)")
    line = {
        "impl": "reference", "metric": "audio_seconds_per_second", "value": value, "unit": "audio-s/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": offline_config(args.batch, args.layers, world, full_audio * world),
        "cpu_baseline": {"value": value, "unit": "audio-s/s", "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": "audio-s/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def run_streaming(args):
    """Config-3 style measurement (``--workload streaming``): 256 concurrent streams, one step = one
    chunk (67-frame window, 16 encoder frames, 0.64 audio-s) for every stream through the paged chunk
    executor; history cap 256 frames in 16-frame pages handed out in a random order.  The cache is
    brought to its steady state (17 pages per stream) by the warm-up chunks."""
    import dataclasses

    import oasr_b200
    from oasr_b200 import _lib
    from oasr_b200.encoder import ConformerCTC
    from oasr_b200.weights import init_params

    torch.cuda.set_device(0)
    if args.pdl:
        from oasr_b200 import tunables
        tunables.set("pdl", 1)
    streams, window, chunk, max_past = args.batch if args.batch != 64 else 256, 67, 16, 256
    cfg = dataclasses.replace(model_config(args.layers), causal=True)
    model = ConformerCTC(cfg, init_params(cfg, 1234), device="cuda:0", dtype=torch.bfloat16,
                         quant=None if args.quant == "none" else args.quant)
    slots = list(range(streams))
    g = torch.Generator().manual_seed(7)
    host = [torch.randn(streams, window, 80, generator=g).pin_memory() for _ in range(8)]
    dev = [h.cuda() for h in host]
    kv_scales = model.calibrate_kv_scales([d[:16] for d in dev[:4]], chunk, margin=1.5) if args.kv == "fp8" else None
    cache = model.new_streaming_cache(streams, max_past, chunk_frames=chunk, seed=5, kv_scales=kv_scales)
    warm = max(args.warmup, max_past // chunk + 1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    for i in range(warm):
        model.forward_chunk_paged(dev[i % 8], slots, cache)
    torch.cuda.synchronize()
    assert oasr_b200.device_status() == 0
    time.sleep(1.0)
    sampler.rows.clear()
    # the step as one CUDA graph (the reference replays its streaming encoder the same way, oasr/engine/graph_cache.py)
    graphed = None if args.no_graph else model.graphed_chunk_forward(cache, streams, window)
    run_step = (lambda xs: graphed(xs, slots)) if graphed is not None else \
        (lambda xs: model.forward_chunk_paged(xs, slots, cache, return_argmax=True))
    for i in range(3):
        run_step(dev[i % 8])
    torch.cuda.synchronize()
    sampler.rows.clear()
    launches0 = _lib.launch_count()
    evs = []
    for i in range(args.steps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run_step(dev[i % 8])
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    launches = _lib.launch_count() - launches0
    if graphed is not None:
        launches = graphed.launches_per_replay * args.steps      # replayed launches do not pass through the library's counter
    total_ms = float(sum(a.elapsed_time(b) for a, b in evs))
    t0 = time.perf_counter()
    for i in range(args.steps):
        _, am = run_step(host[i % 8].cuda(non_blocking=True))
        toks = am.cpu()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    assert oasr_b200.device_status() == 0
    per = instrumented_step(lambda: model.forward_chunk_paged(dev[0], slots, cache))
    audio = streams * chunk * 4 * FRAME_S * args.steps
    kernels = {k: {"launches": v["launches"], "ms": round(v["ms"], 4),
                   **({"tflops": round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 1)} if v["flops"] and v["ms"] else {})}
               for k, v in sorted(per.items(), key=lambda kv: -kv[1]["ms"])}
    print(json.dumps({
        "metric": "audio_seconds_per_second", "value": audio / (total_ms * 1e-3), "unit": "audio-s/s", "n_gpus": 1,
        "steps": args.steps, "warmup": warm, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.quant == "none" else f"{args.quant} Linear GEMMs (per-token / per-channel scales), bf16 elsewhere",
        "data": "synthetic",
        "config": {"workload": f"streaming conformer{args.layers}_d512_h8_ffn2048_k15_vocab5002: {streams} streams x 1 chunk "
                               f"(window {window} frames -> {chunk} encoder frames), history {max_past} frames in 16-frame pages, "
                               f"random page order, {'fp8 e4m3 K/V pages with per-head scales' if args.kv == 'fp8' else 'bf16 K/V'}", "l2": "256 MiB flush write between steps",
                   "audio_seconds_per_step": audio / args.steps},
        "e2e": {"value": audio / e2e_s, "unit": "audio-s/s", "h2d_bytes_per_step": int(host[0].numel() * 4),
                "d2h_bytes_per_step": int(toks.numel() * 4),
                "api": ("GraphedChunkForward (CUDA-graph replay of the step)" if graphed is not None else "ConformerCTC.forward_chunk_paged")
                       + "(pinned host windows) -> per-frame argmax on the host"},
        "gpu_launches": int(launches), "clocks": clocks, "kernels_one_step": kernels}), flush=True)
    return 0


def run_sweep(args):
    """Config-5 style measurement (``--workload sweep``): 4096 utterances with log-normal lengths (median 6 s, clipped
    1-30 s) through the headline Conformer, sorted by length, packed to <= ``--pack-frames`` (8192) frames per pack
    (oasr_b200.sharding.plan_packs, the reference's packing rule) and dealt to the ranks by cost
    (assign_packs); no collective on the data path, token lists gathered on the host at the end.  One "step" = the
    whole sweep.  ``--quant int8|fp8`` runs the Linear GEMMs on 8-bit operands (bf16 is the control)."""
    import oasr_b200
    from oasr_b200 import _lib, sharding
    from oasr_b200.encoder import ConformerCTC
    from oasr_b200.weights import init_params

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    cfg = model_config(args.layers)
    model = ConformerCTC(cfg, init_params(cfg, 1234), device=f"cuda:{local_rank}", dtype=torch.bfloat16,
                         quant=None if args.quant == "none" else args.quant)
    n_utts = 4096 if args.batch == 64 else args.batch
    rng = np.random.default_rng(2024)
    lengths = [int(round(100 * min(max(x, 1.0), 30.0))) for x in rng.lognormal(np.log(6.0), 0.6, size=n_utts)]
    packs = sharding.plan_packs(lengths, args.pack_frames, 4)
    mine = sharding.assign_packs(lengths, packs, world)[rank]
    g = torch.Generator(device=f"cuda:{local_rank}").manual_seed(7 + rank)
    batches = []
    for j in mine:
        ls = [lengths[i] for i in packs[j]]
        batches.append((packs[j], torch.randn(len(ls), max(ls), 80, generator=g, device=f"cuda:{local_rank}"), ls))

    def sweep():
        out = {}   # pipelined: the D2H read and token collapse of pack i run under the encoder of pack i+1
        for (idx, _, _), hyps in zip(batches, model.greedy_search_batches((f, ls) for _, f, ls in batches)):
            out.update(zip(idx, hyps))
        return out

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for idx, feats, ls in batches[:3] + batches[-3:]:      # warm-up: smallest and largest shapes
        model._forward(feats, ls, False, False, True)
    barrier()
    sampler.rows.clear()
    launches0 = _lib.launch_count()
    barrier()
    t0 = time.perf_counter()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    local = sweep()
    b.record()
    torch.cuda.synchronize()
    wall_s = time.perf_counter() - t0
    dev_ms = a.elapsed_time(b)
    clocks = sampler.stop()
    assert oasr_b200.device_status() == 0
    merged = sharding.gather_results(local, n_utts) if dist is not None else [local[i] for i in range(n_utts)]
    t = torch.tensor([dev_ms, wall_s * 1e3], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        assert merged is not None and len(merged) == n_utts
        audio = sum(lengths) * FRAME_S
        print(json.dumps({
            "metric": "audio_seconds_per_second", "value": audio / (float(t[0]) * 1e-3), "unit": "audio-s/s", "n_gpus": world,
            "steps": 1, "warmup": 6, "ms_per_step": float(t[0]), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16" if args.quant == "none" else f"{args.quant} Linear GEMMs (per-token / per-channel scales), bf16 elsewhere",
            "data": "synthetic",
            "config": {"workload": f"sweep of {n_utts} utterances, log-normal lengths (median 6 s, 1-30 s), conformer{args.layers}_d512, "
                                   f"{len(packs)} packs of <= {args.pack_frames} frames, cost-balanced over {world} rank(s), no collective",
                       "audio_seconds": audio},
            "e2e": {"value": audio / (float(t[1]) * 1e-3), "unit": "audio-s/s",
                    "api": "ConformerCTC.greedy_search_batches over the packs (features resident on the device)"},
            "gpu_launches": int(_lib.launch_count() - launches0), "clocks": clocks}), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_fastconformer(args):
    """Config-4 style measurement (``--workload fastconformer``): FastConformer encoder (8x subsampling, 24 layers,
    hidden 1024, 8 heads of 128, FFN 4096, kernel 9, 128 mel bins), random-init weights, one step = one padded batch
    of 128 utterances with lengths uniform in 500..3000 frames (the layer stack runs on the valid frames, packed).  ``--quant fp8|int8`` runs the layers' Linear GEMMs on
    8-bit operands.  The 16-bit layer stack is one call into the native executor (oasr_b200_fastconformer_layers_packed);
    the subsampling front end and the head are separate operator calls."""
    import oasr_b200
    from oasr_b200 import _lib
    from oasr_b200.fastconformer import FastConformerEncoder
    from oasr_b200.weights import init_fastconformer_params

    torch.cuda.set_device(0)
    layers = 24 if args.layers == 12 else args.layers
    batch = 128 if args.batch == 64 else args.batch
    hidden, heads, ffn, kernel, mels, channels, vocab = 1024, 8, 4096, 9, 128, 256, 1024
    P = init_fastconformer_params(hidden, heads, ffn, layers, kernel, mels, channels, seed=1234, w_std=0.02, bias=False, vocab=vocab)
    enc = FastConformerEncoder(hidden, heads, ffn, layers, kernel, 57, 3, mels, channels, P)
    if args.quant != "none":
        enc.stack.set_quant(args.quant)
    rng = np.random.default_rng(2024)
    lengths = [int(x) for x in rng.integers(500, 3001, size=batch)]
    feats = torch.randn(batch, max(lengths), mels, generator=torch.Generator().manual_seed(7)).cuda()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        enc.forward_ctc(feats, lengths, padded_output=False, return_argmax=True)
    torch.cuda.synchronize()
    assert oasr_b200.device_status() == 0
    sampler.rows.clear()
    steps = min(args.steps, 10)
    launches0 = _lib.launch_count()
    evs = []
    for _ in range(steps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        enc.forward_ctc(feats, lengths, padded_output=False, return_argmax=True)   # encoder + vocabulary-1024 CTC head
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    total_ms = float(sum(a.elapsed_time(b) for a, b in evs))
    clocks = sampler.stop()
    audio = sum(lengths) * FRAME_S * steps
    print(json.dumps({
        "metric": "audio_seconds_per_second", "value": audio / (total_ms * 1e-3), "unit": "audio-s/s", "n_gpus": 1,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": total_ms / steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.quant == "none" else f"{args.quant} Linear GEMMs (per-token / per-channel scales), bf16 elsewhere",
        "data": "synthetic",
        "config": {"workload": f"fastconformer{layers}_d1024_h8_ffn4096_k9_mel128_sub8x_ctc1024_b{batch}_len500-3000_padded_in_packed_layers",
                   "audio_seconds_per_step": audio / steps, "l2": "256 MiB flush write between steps"},
        "gpu_launches": int(_lib.launch_count() - launches0), "clocks": clocks}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="offline", choices=["offline", "streaming", "fastconformer", "sweep"],
                    help="offline = the headline packed batch; streaming = 256 streams x one paged chunk per step; "
                         "fastconformer = a padded batch through the FastConformer encoder + CTC-1024 head")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the one-off check of this step's log-probs against the CPU oracle")
    ap.add_argument("--force-fused-addnorm", action="store_true",
                    help="profiling aid: run the fused Linear+add+norm kernel even when the batch does not fill the GPU (reduced cases)")
    ap.add_argument("--tunable", action="append", default=[], metavar="NAME=VALUE",
                    help="comparison runs: set a library tunable (oasr_b200.tunables) before the workload is built; repeatable")
    ap.add_argument("--unfused-addnorm", action="store_true",
                    help="comparison run: gemm + add_norm_f32 as two kernels instead of the fused Linear+add+norm kernel")
    ap.add_argument("--pdl", action="store_true", help="launch the hot kernels with programmatic stream serialisation (comparison run)")
    ap.add_argument("--no-graph", action="store_true",
                    help="streaming workload: enqueue every step's launches from the host instead of replaying the captured CUDA graph")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "fp8"],
                    help="streaming workload: K/V page format (fp8 = e4m3 codes with per-head scales calibrated on four chunks)")
    ap.add_argument("--pack-frames", type=int, default=8192,
                    help="sweep workload: post-subsampling frame budget of a pack (the reference's max_packed_frames default is 8192)")
    ap.add_argument("--quant", default="none", choices=["none", "fp8", "int8"],
                    help="run the eight Linear GEMMs of every layer on 8-bit operands (not the headline dtype)")
    ap.add_argument("--batch", type=int, default=64, help="utterances per step (64 = the headline workload)")
    ap.add_argument("--layers", type=int, default=12, help="encoder layers (12 = the headline workload); "
                    "smaller values with --batch give the reduced case used for ncu captures")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "streaming":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
        return run_streaming(args)
    if args.workload == "sweep":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
        return run_sweep(args)
    if args.workload == "fastconformer":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
        return run_fastconformer(args)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    # The CPU baseline runs FIRST, on rank 0, on every host core, before any process group exists: the other ranks
    # wait for it inside the rendezvous (a host wait), so no GPU spins in a collective while a CPU loop runs, and the
    # thread count is the same at every N (torchrun exports OMP_NUM_THREADS=1, which set_num_threads overrides).
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        threads_before = torch.get_num_threads()
        v, a, dt, thr, kind = cpu_throughput(args.batch, repeats=2, threads=os.cpu_count() or 1)
        torch.set_num_threads(threads_before)   # the GPU arm's small host ops must not wake every core
        cpu = {"value": v, "unit": "audio-s/s", "cores": thr, "kind": kind,
               "sample": f"all {args.batch} utterances of rank 0's batch ({a:.1f} audio-s), fp32 packed path, best of two runs ({dt:.1f} s)"}
    dist = None
    host_pg = None
    if world > 1:
        import datetime

        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(minutes=20))
        host_pg = dist_mod.new_group(backend="gloo")     # end-of-run wait on the host: no NCCL kernel spins on idle GPUs
        dist = dist_mod

    import oasr_b200
    from oasr_b200 import _lib
    from oasr_b200.encoder import ConformerCTC
    from oasr_b200.weights import init_params

    if args.pdl:
        from oasr_b200 import tunables
        tunables.set("pdl", 1)
    for item in args.tunable:
        from oasr_b200 import tunables
        name, _, value = item.partition("=")
        tunables.set(name, int(value))
    if args.unfused_addnorm or args.force_fused_addnorm:
        from oasr_b200 import tunables
        tunables.set("fused_addnorm", 0 if args.unfused_addnorm else 2)
    cfg = model_config(args.layers)
    model = ConformerCTC(cfg, init_params(cfg, 1234), device=f"cuda:{local_rank}", dtype=torch.bfloat16,
                         quant=None if args.quant == "none" else args.quant)
    feats_host, lengths = make_batch(rank, args.batch, world)
    feats_host = feats_host.pin_memory()
    feats_dev = feats_host.cuda(non_blocking=True)
    audio_s = sum(lengths) * FRAME_S
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def device_step():
        return model.forward_offline_packed(feats_dev, lengths, padded_output=False)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)   # started early: nvidia-smi needs ~1 s before its first sample
    sampler.start()
    for _ in range(args.warmup):
        device_step()
    barrier()
    assert oasr_b200.device_status() == 0
    time.sleep(1.0)
    sampler.rows.clear()                 # keep only samples taken from here on (timed regions)
    # ---------------- device-resident throughput ----------------
    launches0 = _lib.launch_count()
    evs = []
    barrier()
    for _ in range(args.steps):
        flush.fill_(1)                       # L2 flush, outside the per-step event pair
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        device_step()
        b.record()
        evs.append((a, b))
    barrier()
    launches = _lib.launch_count() - launches0
    step_ms = [a.elapsed_time(b) for a, b in evs]
    total_ms = float(sum(step_ms))
    # ---------------- end to end through the public call ----------------
    # greedy_search_batches pipelines the batches: H2D of batch i+1 and D2H + token collapse of batch
    # i-1 run under the encoder of batch i; every step's copies are inside the timed region.
    for _ in model.greedy_search_batches([(feats_host, lengths)] * 2):
        pass
    barrier()
    t0 = time.perf_counter()
    n_hyp = 0
    for hyp in model.greedy_search_batches((feats_host, lengths) for _ in range(args.steps)):
        n_hyp += len(hyp)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    assert n_hyp == args.steps * len(lengths)
    d2h = int(getattr(model, "last_d2h_bytes", 0))     # collapsed token rows (B, longest utterance) + their lengths
    clocks = sampler.stop()
    assert oasr_b200.device_status() == 0

    t = torch.tensor([total_ms, e2e_s * 1e3, audio_s * args.steps], dtype=torch.float64, device="cuda")
    if dist is not None:
        mx = t.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, audio_total = float(mx[0]), float(mx[1]), float(sm[2])
    else:
        total_ms, e2e_ms, audio_total = float(t[0]), float(t[1]), float(t[2])

    if rank == 0:
        per = instrumented_step(device_step)
        pk_rows = sum(max((n - 3) // 4, 0) for n in lengths)
        peaks = measured_peaks()
        gemm = {"launches": 0, "ms": 0.0, "flops": 0.0}
        for k, v in per.items():
            if k.startswith("gemm ") or k.startswith("gemm_glu") or k.startswith("gemm_q8") or k.startswith("gemm_addnorm"):
                for f in gemm:                      # every launch of the tcgen05 GEMM kernel in the layer stack (not the head)
                    gemm[f] += v[f]
        step_total = total_ms / args.steps if dist is None else float(np.mean(step_ms))
        achieved = gemm["flops"] / (gemm["ms"] * 1e-3) / 1e12 if gemm["ms"] else 0.0
        # flops the kernels issue beyond the algorithmic 2*M*N*K: with the 8-bit kinds (or the qkv_dup tunable off) the
        # query block of the fused projection is computed twice ([Wq; Wq; Wk; Wv], once per positional bias), 2*M*d*d
        # per layer; the 16-bit path computes it once and stores it twice (oasr_b200_gemm_dup_first)
        d_model, ffn = cfg.d_model, cfg.ffn
        dup_issued = args.quant != "none" or any(t.startswith("qkv_dup=0") for t in (args.tunable or [])) or d_model % 256 != 0
        issued = gemm["flops"] + (2.0 * pk_rows * d_model * d_model * cfg.layers if dup_issued else 0.0)
        # peak: the burst figure when the SM clock sampled during the timed region is in the burst regime (>= 0.9 of the
        # maximum), the sustained figure otherwise; both fractions are printed
        burst = bool(clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.9 * clocks["sm_max_mhz"])
        peak = peaks["bf16_burst"] if burst else peaks["bf16_sustained"]
        roofline = {
            "kernel": "gemm_tcgen05_kernel (all GEMM launches of one step of the layer stack, incl. the embed Linear)",
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak,
            "peak_source": f"{peaks['source']} ({'burst' if burst else 'sustained'} bf16: median SM clock {clocks.get('sm_mhz')} MHz "
                           f"of {clocks.get('sm_max_mhz')})",
            "frac_of_burst": achieved / peaks["bf16_burst"], "frac_of_sustained": achieved / peaks["bf16_sustained"],
            "flops": gemm["flops"], "flops_issued": issued, "achieved_issued": issued / (gemm["ms"] * 1e-3) / 1e12 if gemm["ms"] else 0.0,
            # algorithmic DRAM bytes of ONE FFN w_1 launch (M x ffn x d_model, the launch type with the largest share): every
            # operand byte once plus the output; the reduced-case ncu capture under profiles/ shows dram__bytes_read equal
            # to the operand bytes (its output stays in L2, so the write side cannot be captured at a size ncu may run)
            "traffic": int(2 * (pk_rows * d_model + ffn * d_model + pk_rows * ffn)),
            "traffic_of": "one FFN w_1 launch: operand + output bytes (formula; dram__bytes_read of the reduced ncu case matches the operand part)",
            "launches": gemm["launches"], "share_of_step": gemm["ms"] / step_total if step_total else None,
        }
        kernels = {k: {"launches": v["launches"], "ms": round(v["ms"], 4),
                       **({"tflops": round(v["flops"] / (v["ms"] * 1e-3) / 1e12, 1)} if v["flops"] and v["ms"] else {})}
                   for k, v in sorted(per.items(), key=lambda kv: -kv[1]["ms"])}
        # parity of what was timed: the first utterances of this step's own log-probs against the fp32 CPU oracle
        parity = None
        if not args.no_parity and args.quant == "none":
            from oracle import conformer as OC

            n_chk = min(4, len(lengths))
            lp, out_len, pk = device_step()
            rows = sum(pk.seg_lengths[:n_chk])
            got = lp[:rows].float().cpu()
            ocfg = OC.ConformerConfig(d_model=cfg.d_model, heads=cfg.heads, ffn=cfg.ffn, layers=cfg.layers, kernel=cfg.kernel,
                                      vocab=cfg.vocab)
            threads_before = torch.get_num_threads()
            torch.set_num_threads(os.cpu_count() or 1)
            with torch.no_grad():
                lens = lengths[:n_chk]
                want, wl = OC.forward_offline_packed(OC.init_params(ocfg, 1234), ocfg, feats_host[:n_chk, :max(lens)].contiguous(),
                                                     torch.tensor(lens))
            torch.set_num_threads(threads_before)
            want = want[torch.arange(want.shape[1])[None, :] < wl[:, None]]
            dlt = (got - want)[:, :cfg.vocab].abs()
            same = got[:, :cfg.vocab].argmax(-1) == want[:, :cfg.vocab].argmax(-1)
            top2 = want[:, :cfg.vocab].topk(2, -1).values
            clear = (top2[:, 0] - top2[:, 1]) > 2e-2
            parity = {"against": "fp32 CPU oracle (oracle.conformer.forward_offline_packed)", "utterances": n_chk, "frames": int(rows),
                      "max_abs": dlt.max().item(), "mean_abs": dlt.mean().item(), "argmax": same.float().mean().item(),
                      "argmax_margin_gt_2e-2": same[clear].float().mean().item() if clear.any() else None}
        line = {
            "metric": "audio_seconds_per_second", "value": audio_total / (total_ms * 1e-3), "unit": "audio-s/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if args.quant == "none" else f"{args.quant} Linear GEMMs (per-token / per-channel scales), bf16 elsewhere",
            "data": "synthetic",
            "config": offline_config(args.batch, args.layers, world, audio_total / args.steps),
            "e2e": {"value": audio_total / (e2e_ms * 1e-3), "unit": "audio-s/s",
                    "h2d_bytes_per_step": int(feats_host.numel() * 4), "d2h_bytes_per_step": int(d2h),
                    "api": "ConformerCTC.greedy_search_batches(pinned host features -> token lists), copies pipelined with compute"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "parity": parity,
            "kernels_one_step": kernels,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        torch.cuda.synchronize()
        dist.barrier(group=host_pg)          # ranks > 0 wait here on the host while rank 0 finishes its report
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
