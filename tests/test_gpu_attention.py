"""GPU parity: tcgen05 attention (dense / varlen / paged) and the paged-KV data movement.

Cases and tolerances follow the reference's tests/test_fmha.py (SDPA oracle, shape grid
with odd T_k, MQA/GQA, paged tables, fully-masked-row-is-zero, stale-data-inert with
atol=0) and tests/test_fmha_varlen.py (segment lists, tol 2e-2); outputs are also checked
against the fixtures written from the reference's own SDPA route.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import oasr_b200 as ob
from oracle import ops as O
from tests.golden import cases

pytestmark = pytest.mark.gpu
OPS = np.load(Path(__file__).resolve().parent / "golden" / "operators.npz")
DTYPES = [torch.bfloat16, torch.float16]
TOL = 2e-2


def _dev(t, dtype):
    out = {}
    for k, v in t.items():
        out[k] = (v.to(dtype) if v.is_floating_point() else v).cuda()
    return out


def _cpu(t, dtype):
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in t.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(cases.FMHA_CASES))
def test_fmha_dense(dtype, name):
    c = cases.FMHA_CASES[name]
    t = cases.make_fmha(c)
    g, h = _dev(t, dtype), _cpu(t, dtype)
    got = ob.fmha(g["q"], g["k"], g["v"], softmax_scale=c["scale"], attn_bias=g.get("bias"),
                  cache_seqlens=g.get("seqlens"), cache_seqstarts=g.get("seqstarts"), causal=c["causal"])
    want = O.fmha(h["q"], h["k"], h["v"], c["scale"], h.get("bias"), h.get("seqlens"), h.get("seqstarts"), None,
                  c["causal"])
    assert (got.float().cpu() - want).abs().max().item() < TOL
    # fixture from the reference's SDPA route on the unrounded fp32 inputs
    assert np.abs(got.float().cpu().numpy() - OPS[f"fmha_{name}"]).max() < 4e-2


def test_fmha_fully_masked_rows_are_exact_zero():
    c = cases.FMHA_CASES["starts"]
    g = _dev(cases.make_fmha(c), torch.bfloat16)
    got = ob.fmha(g["q"], g["k"], g["v"], softmax_scale=c["scale"], attn_bias=g["bias"],
                  cache_seqlens=g["seqlens"], cache_seqstarts=g["seqstarts"])
    assert torch.count_nonzero(got[2]) == 0
    assert torch.isfinite(got).all()


def test_fmha_strided_views_and_out():
    """q/k/v as (B,T,H,D)->transpose views, the layout the Conformer layer produces
    (oasr/layers/attention/attention.py:216-218)."""
    dtype = torch.bfloat16
    B, T, H, D = 2, 150, 4, 64
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(B, T, 3 * H * D, generator=g).to(dtype).cuda()
    q, k, v = (x.view(B, T, H, D).transpose(1, 2) for x in qkv.split(H * D, dim=-1))
    out = torch.empty(B, H, T, D, device="cuda", dtype=dtype)
    got = ob.fmha(q, k, v, softmax_scale=0.125, out=out)
    assert got is out
    want = O.fmha(q.cpu(), k.cpu(), v.cpu(), 0.125)
    assert (got.float().cpu() - want).abs().max().item() < TOL


def test_fmha_token_major_output_and_aligned_bias():
    """token_major=True writes (B, T, H, D) with the same bits as the head-major result; the bias rows are padded to a
    multiple of 8 elements, the form the kernel reads in 16-byte pieces, with ragged lengths and a tail group."""
    dtype = torch.bfloat16
    B, T, H, D = 2, 203, 2, 128
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(B, H, T, D, generator=g).to(dtype).cuda() for _ in range(3))
    ldb = (T + 7) // 8 * 8
    bias = torch.randn(B, H, T, ldb, generator=g).to(dtype).cuda()[..., :T]
    lens = torch.tensor([203, 77], dtype=torch.int32).cuda()
    head_major = ob.fmha(q, k, v, softmax_scale=0.1, attn_bias=bias, cache_seqlens=lens)
    packed_bias = ob.fmha(q, k, v, softmax_scale=0.1, attn_bias=bias.contiguous(), cache_seqlens=lens)
    token_major = ob.fmha(q, k, v, softmax_scale=0.1, attn_bias=bias, cache_seqlens=lens, token_major=True)
    assert ob.device_status() == 0
    assert token_major.shape == (B, T, H, D)
    assert torch.equal(token_major.transpose(1, 2), head_major)
    assert torch.equal(packed_bias, head_major)          # 16-byte and element-wise bias fetches agree bit for bit
    want = O.fmha(q.cpu(), k.cpu(), v.cpu(), 0.1, bias=bias.cpu(), seqlens=lens.cpu())
    assert (head_major.float().cpu() - want).abs().max().item() < TOL


def test_fmha_stale_keys_are_inert():
    """Finite stale data beyond cache_seqlens must not change the result at all (atol=0)."""
    dtype = torch.bfloat16
    c = dict(cases.FMHA_CASES["stream_chunk"])
    g = _dev(cases.make_fmha(c), dtype)
    a = ob.fmha(g["q"], g["k"], g["v"], softmax_scale=c["scale"], attn_bias=g["bias"], cache_seqlens=g["seqlens"])
    k2, v2 = g["k"].clone(), g["v"].clone()
    for b, n in enumerate(c["lens"]):
        k2[b, :, n:] = 1e4
        v2[b, :, n:] = -1e4
    b_ = ob.fmha(g["q"], k2, v2, softmax_scale=c["scale"], attn_bias=g["bias"], cache_seqlens=g["seqlens"])
    assert torch.equal(a, b_)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(cases.VARLEN_CASES))
@pytest.mark.parametrize("with_bias", [True, False])
def test_fmha_varlen(dtype, name, with_bias):
    c = cases.VARLEN_CASES[name]
    t = cases.make_varlen(c)
    g, h = _dev(t, dtype), _cpu(t, dtype)
    got = ob.fmha_varlen(g["q"], g["k"], g["v"], softmax_scale=c["scale"], cu_seqlens_q=g["cu"], cu_seqlens_k=g["cu"],
                         max_seqlen_q=max(c["lens"]), max_seqlen_k=max(c["lens"]),
                         attn_bias=g["bias"] if with_bias else None,
                         bias_offsets=g["bias_offsets"] if with_bias else None)
    want = O.fmha_varlen(h["q"], h["k"], h["v"], c["scale"], t["cu"], t["cu"], h["bias"] if with_bias else None,
                         t["bias_offsets"] if with_bias else None)
    assert (got.float().cpu() - want).abs().max().item() < TOL
    if with_bias:
        assert np.abs(got.float().cpu().numpy() - OPS[f"varlen_{name}"]).max() < 4e-2
        # int32 offsets (what the packed layout carries, oasr/models/conformer/packing.py:176-180)
        got2 = ob.fmha_varlen(g["q"], g["k"], g["v"], softmax_scale=c["scale"], cu_seqlens_q=g["cu"],
                              cu_seqlens_k=g["cu"], max_seqlen_q=max(c["lens"]), max_seqlen_k=max(c["lens"]),
                              attn_bias=g["bias"], bias_offsets=g["bias_offsets"].to(torch.int32))
        assert torch.equal(got, got2)


def test_fmha_varlen_config2_sized_is_deterministic_and_isolated():
    """64 segments of 49..499 tokens (BASELINE config 2): every segment equals the same
    segment run alone, bit for bit."""
    dtype = torch.bfloat16
    rng = np.random.default_rng(2024)
    lens = [int(x) for x in rng.integers(49, 500, size=64)]
    H, D = 8, 64
    total = sum(lens)
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(total, H, D, generator=g).to(dtype).cuda() for _ in range(3))
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    kw = dict(softmax_scale=0.125, max_seqlen_q=max(lens), max_seqlen_k=max(lens))
    full = ob.fmha_varlen(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, **kw)
    assert torch.equal(full, ob.fmha_varlen(q, k, v, cu_seqlens_q=cu, cu_seqlens_k=cu, **kw))
    for s in (0, 17, 63):
        a, b = int(cu[s]), int(cu[s + 1])
        one = torch.tensor([0, b - a], dtype=torch.int32).cuda()
        alone = ob.fmha_varlen(q[a:b].contiguous(), k[a:b].contiguous(), v[a:b].contiguous(), cu_seqlens_q=one,
                               cu_seqlens_k=one, softmax_scale=0.125, max_seqlen_q=b - a, max_seqlen_k=b - a)
        assert torch.equal(full[a:b], alone)
    want = O.fmha_varlen(q[:lens[0]].cpu(), k[:lens[0]].cpu(), v[:lens[0]].cpu(), 0.125, [0, lens[0]], [0, lens[0]])
    assert (full[:lens[0]].float().cpu() - want).abs().max().item() < TOL


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(cases.PAGED_CASES))
def test_fmha_paged_and_cache_movement(dtype, name):
    c = cases.PAGED_CASES[name]
    t = cases.make_paged(c)
    g, h = _dev(t, dtype), _cpu(t, dtype)
    # gather: bit-exact against the reference rule
    kd, vd = ob.gather_paged_kv(g["k_pool"], g["v_pool"], g["block_table"])
    ok, ov = O.gather_paged_kv(h["k_pool"], h["v_pool"], h["block_table"])
    assert torch.equal(kd.cpu(), ok) and torch.equal(vd.cpu(), ov)
    got = ob.fmha(g["q"], g["k_pool"], g["v_pool"], softmax_scale=c["scale"], attn_bias=g["bias"],
                  cache_seqlens=g["seqlens"], block_table=g["block_table"])
    want = O.fmha(h["q"], h["k_pool"], h["v_pool"], c["scale"], h["bias"], h["seqlens"], None, h["block_table"])
    assert (got.float().cpu() - want).abs().max().item() < TOL
    assert np.abs(got.float().cpu().numpy() - OPS[f"paged_{name}_out"]).max() < 4e-2
    # write: scatter a new chunk, compare pools bit for bit with the oracle's scatter
    gen = torch.Generator().manual_seed(77)
    new_k = torch.randn(c["B"], c["Hkv"], c["t_new"], c["D"], generator=gen).to(dtype)
    new_v = torch.randn(c["B"], c["Hkv"], c["t_new"], c["D"], generator=gen).to(dtype)
    kp, vp = h["k_pool"].clone(), h["v_pool"].clone()
    O.write_kv_chunk(kp, vp, new_k, new_v, h["block_table"], h["offsets"], c["block_size"])
    cache = ob.PagedKVCache(g["k_pool"], g["v_pool"], g["block_table"], g["offsets"], c["block_size"])
    # head-first strided view, as produced by .view(B,T,H,D).transpose(1,2) in the layer
    nk = new_k.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)
    nv = new_v.permute(0, 2, 1, 3).contiguous().cuda().permute(0, 2, 1, 3)
    cache.write_kv_chunk(nk, nv, offset=g["offsets"])
    assert torch.equal(g["k_pool"].cpu(), kp) and torch.equal(g["v_pool"].cpu(), vp)


def test_paged_kv_write_raw_bits_fp8_sized_and_int_offset():
    """1-byte payload (FP8 pages) and the homogeneous integer offset form."""
    B, Hkv, T, D, bs, nblk, num_blocks = 5, 4, 16, 64, 16, 4, 32
    gen = torch.Generator().manual_seed(5)
    pool_k = torch.randint(0, 255, (num_blocks, bs, Hkv, D), generator=gen, dtype=torch.uint8)
    pool_v = torch.randint(0, 255, (num_blocks, bs, Hkv, D), generator=gen, dtype=torch.uint8)
    table = torch.randperm(num_blocks, generator=gen)[: B * nblk].view(B, nblk).to(torch.int32)
    nk = torch.randint(0, 255, (B, Hkv, T, D), generator=gen, dtype=torch.uint8)
    nv = torch.randint(0, 255, (B, Hkv, T, D), generator=gen, dtype=torch.uint8)
    for offset in (24, torch.tensor([0, 5, 16, 33, 48], dtype=torch.int32)):
        kp, vp = pool_k.clone(), pool_v.clone()
        offs = torch.full((B,), offset, dtype=torch.int32) if isinstance(offset, int) else offset
        O.write_kv_chunk(kp, vp, nk, nv, table, offs, bs)
        gk, gv = pool_k.cuda(), pool_v.cuda()
        ob.write_kv_chunk(gk, gv, table.cuda(), nk.cuda(), nv.cuda(), offset if isinstance(offset, int) else offset.cuda())
        assert torch.equal(gk.cpu(), kp) and torch.equal(gv.cpu(), vp)


def test_gather_scatter_rows_roundtrip():
    gen = torch.Generator().manual_seed(6)
    src = torch.randn(50, 512, generator=gen).to(torch.bfloat16).cuda()
    idx = torch.randperm(50, generator=gen)[:37].cuda()
    got = ob.gather_rows(src, idx)
    assert torch.equal(got, src.index_select(0, idx))
    dst = torch.zeros(50, 512, device="cuda", dtype=torch.bfloat16)
    ob.scatter_rows(dst, idx, got)
    ref = torch.zeros_like(dst).index_copy_(0, idx, got)
    assert torch.equal(dst, ref)
    neg = torch.tensor([3, -1, 7], device="cuda")
    g2 = ob.gather_rows(src, neg)
    assert torch.count_nonzero(g2[1]) == 0 and torch.equal(g2[0], src[3])


@pytest.mark.parametrize("block_size,Tq,path", [(16, 16, 1), (16, 16, 0), (16, 5, 1), (32, 16, 1), (64, 9, 1)])
def test_fmha_paged_relpos_matches_fp32_reference(block_size, Tq, path):
    """Both kernels behind fmha_paged_relpos (warp-per-(stream, head) for <= 16 frames, 128-row tcgen05)
    against an fp32 torch restatement: random page permutation, ragged history lengths."""
    from oasr_b200 import fused, tunables

    torch.manual_seed(11)
    B, H, D, hist = 37, 8, 64, 272
    d = H * D
    bps = hist // block_size + 1
    num_blocks = B * bps + 3
    dt = torch.bfloat16
    dev = "cuda"
    k_pool = torch.randn(num_blocks, block_size, H, D, device=dev, dtype=dt)
    v_pool = torch.randn(num_blocks, block_size, H, D, device=dev, dtype=dt)
    table = torch.randperm(num_blocks, device=dev)[: B * bps].view(B, bps).int()
    seqlens = torch.randint(Tq, hist + 1, (B,), device=dev, dtype=torch.int32)
    seqlens[0], seqlens[1] = Tq, hist
    pos_start = torch.randint(0, 3000, (B,), device=dev, dtype=torch.int32)
    pos = torch.randn(5000, d, device=dev, dtype=dt)
    qkv4 = (torch.randn(B, Tq, 4 * d, device=dev) * 0.5).to(dt)
    scale = D ** -0.5
    tunables.set("fmha_chunk_path", path)
    try:
        got = fused.fmha_paged_relpos(qkv4, k_pool, v_pool, pos, pos_start, table, seqlens, H, scale).float()
    finally:
        tunables.set("fmha_chunk_path", 1)
    assert ob.device_status() == 0
    for b in range(B):
        n = int(seqlens[b])
        idx = (table[b].long()[:, None] * block_size + torch.arange(block_size, device=dev)[None]).reshape(-1)[:n]
        k = k_pool.view(-1, H, D)[idx].float()            # (n, H, D)
        v = v_pool.view(-1, H, D)[idx].float()
        pp = pos[int(pos_start[b]): int(pos_start[b]) + n].float().view(n, H, D)
        qu = qkv4[b, :, :d].float().view(Tq, H, D)
        qv = qkv4[b, :, d:2 * d].float().view(Tq, H, D)
        s = (torch.einsum("qhd,khd->hqk", qu, k) + torch.einsum("qhd,khd->hqk", qv, pp)) * scale
        want = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).reshape(Tq, d)
        assert (got[b] - want).abs().max().item() < 3e-2, (b, n, (got[b] - want).abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("path", [1, 0])
def test_fmha_varlen_relpos_matches_fp32_reference(dtype, path):
    """Packed relative-position attention, both kernels behind the entry point (two CTAs per SM with 64-key
    tiles; general 128-key kernel) against an fp32 torch restatement on ragged segments, incl. lengths that
    are not multiples of any tile size and a single-frame segment."""
    from oasr_b200 import fused, tunables

    torch.manual_seed(21)
    lens = [1, 49, 64, 65, 127, 128, 129, 300, 499, 31]
    H, D = 4, 64
    d = H * D
    total = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    qkv4 = (torch.randn(total, 4 * d) * 0.7).to(dtype).cuda()
    pos = torch.randn(600, d).to(dtype).cuda()
    scale = D ** -0.5
    tunables.set("fmha_relpos_path", path)
    try:
        got = fused.fmha_varlen_relpos(qkv4, pos, cu, max(lens), H, scale).float().cpu()
        again = fused.fmha_varlen_relpos(qkv4, pos, cu, max(lens), H, scale).float().cpu()
    finally:
        tunables.set("fmha_relpos_path", 1)
    assert ob.device_status() == 0
    assert torch.equal(got, again)
    x = qkv4.float().cpu()
    pp = pos.float().cpu()
    for s, n in enumerate(lens):
        a = int(cu[s])
        qu = x[a:a + n, :d].view(n, H, D)
        qv = x[a:a + n, d:2 * d].view(n, H, D)
        k = x[a:a + n, 2 * d:3 * d].view(n, H, D)
        v = x[a:a + n, 3 * d:].view(n, H, D)
        p = pp[:n].view(n, H, D)
        sc = (torch.einsum("qhd,khd->hqk", qu, k) + torch.einsum("qhd,khd->hqk", qv, p)) * scale
        want = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(n, d)
        err = (got[a:a + n] - want).abs().max().item()
        assert err < TOL, (s, n, err)


def test_planned_relpos_attention_equals_the_unplanned_order():
    """The persistent packed rel-pos kernel following a longest-first work list (oasr_b200_fmha_relpos_plan) against
    the same kernel walking (segment, head, tile) order: bit-identical output; the list holds every (segment, head,
    query tile) exactly once, longest segments first, and skips empty segments; many more items than resident CTAs."""
    from oasr_b200 import fused

    torch.manual_seed(4)
    rng = np.random.default_rng(0)
    lens = [0, 1, 130, 0, 500] + [int(x) for x in rng.integers(1, 400, size=90)]
    H, D = 8, 64
    d = H * D
    total = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    qkv4 = (torch.randn(total, 4 * d) * 0.7).bfloat16().cuda()
    pos = torch.randn(512, d).bfloat16().cuda()
    plan = fused.fmha_relpos_plan(cu, H, total)
    want = fused.fmha_varlen_relpos(qkv4, pos, cu, max(lens), H, D ** -0.5)
    got = fused.fmha_varlen_relpos(qkv4, pos, cu, max(lens), H, D ** -0.5, plan=plan)
    assert ob.device_status() == 0
    assert torch.equal(got, want)
    host = plan.cpu().numpy()
    n = int(host[0])
    items = host[4:4 + 2 * n].reshape(n, 2)
    seg, head, qt = items[:, 0], items[:, 1] >> 16, items[:, 1] & 0xffff
    expect = {(s, h, q) for s, L in enumerate(lens) for h in range(H) for q in range((L + 127) // 128)}
    assert n == len(expect) and set(zip(seg.tolist(), head.tolist(), qt.tolist())) == expect
    item_len = np.asarray(lens)[seg]
    assert (np.diff(item_len) <= 0).all()


def test_relpos_attention_over_many_single_tile_items():
    """A pack of short utterances (the sweep's shape): 700 segments of 1-60 frames, 8 heads, so every CTA of the
    persistent kernel walks about twenty work items of ONE key tile each and its K and V cursors cross item
    boundaries at every step.  Against the fp32 restatement, with and without the work list, twice (same bits), and
    the device status stays clean (no role gave up a wait)."""
    from oasr_b200 import fused

    torch.manual_seed(9)
    rng = np.random.default_rng(3)
    lens = [int(x) for x in rng.integers(1, 61, size=700)]
    H, D = 8, 64
    d = H * D
    total = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    qkv4 = (torch.randn(total, 4 * d) * 0.7).bfloat16().cuda()
    pos = torch.randn(64, d).bfloat16().cuda()
    scale = D ** -0.5
    plan = fused.fmha_relpos_plan(cu, H, total)
    outs = []
    for pl in (plan, None, plan, None):
        for _ in range(5):
            outs.append(fused.fmha_varlen_relpos(qkv4, pos, cu, max(lens), H, scale, plan=pl))
    assert ob.device_status() == 0
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    got = outs[0].float().cpu()
    x = qkv4.float().cpu()
    pp = pos.float().cpu()
    for s in list(range(0, 700, 37)) + [699]:
        n = lens[s]
        a = int(cu[s])
        qu = x[a:a + n, :d].view(n, H, D)
        qv = x[a:a + n, d:2 * d].view(n, H, D)
        k = x[a:a + n, 2 * d:3 * d].view(n, H, D)
        v = x[a:a + n, 3 * d:].view(n, H, D)
        p = pp[:n].view(n, H, D)
        sc = (torch.einsum("qhd,khd->hqk", qu, k) + torch.einsum("qhd,khd->hqk", qv, p)) * scale
        want = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(n, d)
        err = (got[a:a + n] - want).abs().max().item()
        assert err < TOL, (s, n, err)
