"""GPU parity: norm / activation / depthwise-conv kernels vs the CPU oracle.

Cases follow the reference's kernel unit tests (tests/test_norm.py,
tests/test_activation.py, tests/test_conv.py): same shapes families, same
tolerances or tighter, plus ragged / empty / non-vectorisable extents.
"""
import numpy as np
import pytest
import torch

import oasr_b200 as ob
from oracle import ops as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16, torch.float32]
TOL = {torch.bfloat16: 2e-2, torch.float16: 3e-3, torch.float32: 2e-5}


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _close(got, want, dtype, scale=1.0):
    got = got.float().cpu()
    want = want.float()
    # the oracle's fp32 result rounded to the kernel's output type is the target
    want_r = want.to(dtype).float()
    tol = TOL[dtype] * scale
    err = (got - want_r).abs().max().item() if got.numel() else 0.0
    assert err <= tol * max(1.0, want.abs().max().item() if want.numel() else 1.0), f"max err {err}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 250, 512), (3, 7, 256), (2, 5, 1024), (1, 1, 8), (2, 3, 80), (5, 333),
                                   (2, 4, 4096), (2, 4, 4104), (0, 16), (3, 5, 12)])
def test_layer_norm(dtype, shape):
    x = _rand(shape, dtype, 1, 2.0)
    H = shape[-1]
    w, b = _rand((H,), dtype, 2) + 1, _rand((H,), dtype, 3)
    got = ob.layer_norm(x.cuda(), w.cuda(), b.cuda(), 1e-5)
    _close(got, O.layer_norm(x, w, b, 1e-5), dtype)
    got = ob.layer_norm(x.cuda(), w.cuda(), None, 1e-5)
    _close(got, O.layer_norm(x, w, None, 1e-5), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", [0, 1, 2, 4])
def test_layer_norm_activation(dtype, act):
    x = _rand((3, 17, 512), dtype, 4)
    w, b = _rand((512,), dtype, 5) + 1, _rand((512,), dtype, 6)
    got = ob.layer_norm_activation(x.cuda(), w.cuda(), b.cuda(), 1e-5, act)
    _close(got, O.layer_norm(x, w, b, 1e-5, act), dtype)
    got = ob.rms_norm_activation(x.cuda(), w.cuda(), b.cuda(), 1e-5, act)
    _close(got, O.rms_norm(x, w, b, 1e-5, act), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 250, 512), (2, 3, 1000), (7, 24)])
def test_rms_norm(dtype, shape):
    x = _rand(shape, dtype, 7, 3.0)
    H = shape[-1]
    w, b = _rand((H,), dtype, 8) + 1, _rand((H,), dtype, 9)
    _close(ob.rms_norm(x.cuda(), w.cuda(), None, 1e-5), O.rms_norm(x, w, None, 1e-5), dtype)
    _close(ob.rms_norm(x.cuda(), w.cuda(), b.cuda(), 1e-6), O.rms_norm(x, w, b, 1e-6), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 250, 512), (2, 9, 256), (3, 5, 12)])
@pytest.mark.parametrize("alpha", [1.0, 0.5])
def test_add_layer_norm_residual(dtype, shape, alpha):
    x, r = _rand(shape, dtype, 10), _rand(shape, dtype, 11, 2.0)
    H = shape[-1]
    w, b = _rand((H,), dtype, 12) + 1, _rand((H,), dtype, 13)
    out, res = ob.add_layer_norm_residual(x.cuda(), r.cuda(), w.cuda(), b.cuda(), 1e-5, alpha)
    want_out, want_res = O.add_layer_norm_residual(x, r, w, b, 1e-5, alpha)
    _close(out, want_out, dtype)
    # the carried sum is the fp32 sum rounded ONCE: bit-exact (reference tests/test_norm.py:276-281)
    want_fma = torch.addcmul(r.float(), torch.tensor(alpha), x.float()).to(dtype)
    assert torch.equal(res.cpu(), want_res) or torch.equal(res.cpu(), want_fma)
    out2 = ob.add_layer_norm(x.cuda(), r.cuda(), w.cuda(), b.cuda(), 1e-5, alpha=alpha)
    assert torch.equal(out2, out)
    o3, r3 = ob.add_rms_norm_residual(x.cuda(), r.cuda(), w.cuda(), b.cuda(), 1e-5, alpha)
    w_o3, w_r3 = O.add_rms_norm_residual(x, r, w, b, 1e-5, alpha)
    _close(o3, w_o3, dtype)
    assert torch.equal(r3.cpu(), w_r3) or torch.equal(r3.cpu(), want_fma)
    assert torch.equal(ob.add_rms_norm(x.cuda(), r.cuda(), w.cuda(), b.cuda(), 1e-5, alpha), o3)


def test_norm_rejects_padded_rows_and_cpu():
    x = torch.randn(4, 8, 64, device="cuda", dtype=torch.bfloat16)[:, :, :32]
    w = torch.ones(32, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ob.layer_norm(x, w)
    with pytest.raises(RuntimeError):
        ob.layer_norm(torch.randn(2, 32), torch.ones(32))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 250, 512), (2, 7, 256), (3, 5, 20), (1, 3, 1024)])
@pytest.mark.parametrize("act", [-1, 2, 0])
def test_batch_norm(dtype, shape, act):
    x = _rand(shape, dtype, 14, 2.0)
    C = shape[-1]
    w, b = _rand((C,), dtype, 15) + 1, _rand((C,), dtype, 16)
    mean, var = _rand((C,), dtype, 17), _rand((C,), dtype, 18).abs() + 0.5
    want = O.batch_norm(x, w, b, mean, var, 1e-5, act)
    args = [t.cuda() for t in (x, w, b, mean, var)]
    if act == -1:
        got = ob.batch_norm_1d(*args, 1e-5)
    elif act == 2:
        got = ob.batch_norm_swish(*args, 1e-5)
    else:
        got = ob.batch_norm_activation(*args, 1e-5, act)
    _close(got, want, dtype, scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(4, 250, 1024), (2, 3, 16), (3, 5, 24), (1, 1, 2), (0, 4, 64)])
def test_glu_swish(dtype, shape):
    x = _rand(shape, dtype, 19, 2.0)
    _close(ob.glu(x.cuda()), O.glu(x), dtype)
    _close(ob.swish(x.cuda()), O.swish(x), dtype)
    out = torch.empty_like(x, device="cuda")
    assert ob.swish(x.cuda(), out=out) is out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B,T,C,K,pad", [(4, 250, 256, 15, 7), (2, 100, 512, 15, (14, 0)), (3, 33, 64, 9, (8, 0)),
                                          (1, 30, 512, 15, 0), (2, 17, 24, 3, 1), (2, 40, 10, 4, (2, 1)),
                                          (1, 5, 64, 15, 7), (2, 64, 128, 31, 15)])
def test_depthwise_conv1d(dtype, B, T, C, K, pad):
    x = _rand((B, T, C), dtype, 20)
    w = _rand((K, 1, C), dtype, 21, 0.3)
    b = _rand((C,), dtype, 22)
    got = ob.depthwise_conv1d(x.cuda(), w.cuda(), b.cuda(), pad)
    _close(got, O.depthwise_conv1d(x, w, b, pad), dtype, scale=2.0)
    got = ob.depthwise_conv1d(x.cuda(), w.cuda().reshape(K, C), None, pad)
    _close(got, O.depthwise_conv1d(x, w, None, pad), dtype, scale=2.0)
    got = ob.depthwise_conv1d_silu(x.cuda(), w.cuda(), b.cuda(), pad)
    _close(got, O.depthwise_conv1d(x, w, b, pad, act=2), dtype, scale=2.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bool_mask", [True, False])
def test_depthwise_conv1d_fsmn_mask(dtype, bool_mask):
    B, T, C, K = 3, 40, 64, 11
    x = _rand((B, T, C), dtype, 23)
    w = _rand((K, C), dtype, 24, 0.3)
    lens = torch.tensor([40, 25, 1])
    mask = (torch.arange(T)[None, :] < lens[:, None]).unsqueeze(-1)
    m = mask if bool_mask else mask.to(dtype)
    got = ob.depthwise_conv1d(x.cuda(), w.cuda(), None, (K - 1) // 2, mask=m.cuda(), add_input=True)
    _close(got, O.depthwise_conv1d(x, w, None, (K - 1) // 2, mask=mask, add_input=True), dtype, scale=2.0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("T", [16, 3, 1])
def test_causal_conv1d_state(dtype, T):
    B, C, K = 3, 64, 9
    w = _rand((C, 1, K), dtype, 25, 0.3)
    b = _rand((C,), dtype, 26)
    state = _rand((B, K - 1, C), dtype, 27)
    st_gpu = state.cuda().clone()
    for step in range(3):
        x = _rand((B, T, C), dtype, 28 + step)
        want, state = O.causal_conv1d(x, state, w, b)
        got = ob.causal_conv1d(x.cuda(), st_gpu, w.cuda(), b.cuda())
        _close(got, want, dtype, scale=2.0)
        assert torch.equal(st_gpu.cpu(), state)  # rolled state is a pure copy: bit-exact


@pytest.mark.parametrize("conv1_mma", [1, 0])
@pytest.mark.parametrize("C,lens", [(128, [96, 151, 40]), (512, [403, 67, 1000, 250]), (256, [67] * 5)])
def test_subsampling_front_end_matches_torch_conv2d(C, lens, conv1_mma):
    """conv1 (parity-split layout: split-bf16 GEMM on the tensor cores for 256 / 512 channels, else - or with the
    tunable off - the fp32 stencil) + conv2 (tcgen05 implicit GEMM, packed valid frames) against torch conv2d + ReLU
    in fp32 on the same 16-bit-rounded weights and intermediate."""
    from oasr_b200 import fused, tunables

    tunables.set("conv1_mma", conv1_mma)
    try:
        _front_end_case(C, lens, stencil=not (conv1_mma and C in (256, 512)))
    finally:
        tunables.set("conv1_mma", 1)


def _front_end_case(C, lens, stencil):
    from oasr_b200 import fused

    torch.manual_seed(5)
    B, T, F = len(lens), max(lens), 80
    feats = torch.randn(B, T, F, device="cuda")
    w1 = torch.randn(C, 3, 3, device="cuda") * 0.3
    b1 = torch.randn(C, device="cuda") * 0.1
    w2 = (torch.randn(C, 3, 3, C, device="cuda") * (9 * C) ** -0.5).bfloat16()
    b2 = (torch.randn(C, device="cuda") * 0.1).bfloat16()
    out_lens = [(n - 3) // 4 for n in lens]
    cu = torch.tensor([0] + list(np.cumsum(out_lens)), dtype=torch.int32, device="cuda")
    total = int(cu[-1])
    t1_limit = torch.tensor([2 * n + 1 for n in out_lens], dtype=torch.int32, device="cuda")
    T1, F1 = (T - 3) // 2 + 1, (F - 3) // 2 + 1
    x1 = fused.subsample_conv1_s2d(feats, w1, b1, torch.bfloat16, t1_limit=t1_limit)
    got = fused.subsample_conv2(x1, T1, F1, w2, b2, cu, total).float()
    assert ob.device_status() == 0
    # reference
    y1_f32 = torch.relu(torch.nn.functional.conv2d(feats[:, None], w1[:, None], b1, stride=2))                  # (B,C,T1,F1)
    y1 = y1_f32.bfloat16().float()
    # conv1 against the NHWC kernel and the parity-split layout
    nhwc = fused.subsample_conv1(feats, w1, b1, torch.bfloat16).float()
    assert (nhwc - y1.permute(0, 2, 3, 1)).abs().max().item() < 2e-2
    for b, n in enumerate(out_lens):
        lim = 2 * n + 1
        t1 = torch.arange(lim, device="cuda")
        f1 = torch.arange(F1, device="cuda")
        plane = (t1[:, None] & 1) * 2 + (f1[None] & 1)
        s2d = x1[b][t1[:, None] // 2, plane, f1[None] // 2].float()             # (lim, F1, C)
        if stencil:
            assert torch.equal(s2d, nhwc[b, :lim])
        else:
            # products of two-term bf16 operands (the lo x lo term dropped: 2^-16 of the summed magnitudes), one rounding
            # on store: within one 16-bit rounding step of the exact value plus that share of sum |x||w| + |b|
            # everywhere, and the same 16-bit value as the fp32 stencil almost everywhere
            exact = y1_f32[b, :, :lim].permute(1, 2, 0)
            mag = torch.nn.functional.conv2d(feats[b:b + 1, None].abs(), w1[:, None].abs(), b1.abs(), stride=2)[0, :, :lim].permute(1, 2, 0)
            assert ((s2d - exact).abs() <= exact.abs() * 2.0 ** -8 + mag * 2.0 ** -14 + 1e-6).all()
            assert (s2d != nhwc[b, :lim]).float().mean().item() < 2e-3
    y2 = torch.relu(torch.nn.functional.conv2d(y1, w2.float().permute(0, 3, 1, 2), b2.float(), stride=2))      # (B,C,T2,F2)
    want = torch.cat([y2[b, :, :n].permute(1, 2, 0).reshape(n, -1) for b, n in enumerate(out_lens)])
    err = (got - want).abs().max().item()
    assert err < 3e-2, err


@pytest.mark.parametrize("K,causal", [(15, False), (9, True)])
def test_packed_depthwise_conv_kernels_agree_with_each_other_and_with_fp32(K, causal):
    """The rolling register-window kernel (default for kernel sizes 9 / 15) against the run-at-once kernel
    (``dwconv_path`` 0) and an fp32 torch restatement, on ragged segments incl. ones shorter than the kernel, a run
    boundary inside a segment (60 frames), folded BatchNorm + swish (non-causal form) and the padded-semantics fill."""
    from oasr_b200 import fused, tunables

    torch.manual_seed(11)
    lens = [1, 7, 59, 60, 61, 120, 121, 333, 14, 15]
    C = 512
    total = sum(lens)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    x = torch.randn(total, C).bfloat16().cuda()
    w = (torch.randn(K, C) * 0.3).bfloat16().cuda()
    b = torch.randn(C).bfloat16().cuda()
    sc, sh = (torch.rand(C) + 0.5).cuda(), torch.randn(C).cuda()
    fill = torch.randn(C).cuda()
    fill_frames = torch.tensor([min((K - 1) // 2, 3 + i % 5) for i in range(len(lens))], dtype=torch.int32).cuda()

    def run():
        if causal:
            return fused.depthwise_conv1d_packed_causal(x, w, b, cu, max(lens), activation=-1).float()
        return fused.depthwise_conv1d_packed(x, w, b, cu, max(lens), post_scale=sc, post_shift=sh, right_fill=fill,
                                             fill_frames=fill_frames, activation=2).float()

    outs = {}
    for path in (2, 0):
        tunables.set("dwconv_path", path)
        try:
            outs[path] = run()
        finally:
            tunables.set("dwconv_path", 2)
    assert ob.device_status() == 0
    assert (outs[2] - outs[0]).abs().max().item() < 4e-2      # two roundings to bf16 of nearly equal fp32 values
    xf, wf = x.float().cpu(), w.float().cpu()
    for s, n in enumerate(lens):
        a = int(cu[s])
        seg = xf[a:a + n]
        if causal:
            padded = torch.cat([torch.zeros(K - 1, C), seg])
        else:
            nf = int(fill_frames[s])
            right = torch.cat([fill.cpu().bfloat16().float().expand(nf, C), torch.zeros((K - 1) // 2 - nf, C)])
            padded = torch.cat([torch.zeros((K - 1) // 2, C), seg, right])
        want = sum(padded[k:k + n] * wf[k] for k in range(K)) + b.float().cpu()
        if not causal:
            want = want * sc.cpu() + sh.cpu()
            want = want * torch.sigmoid(want)
        for path in (2, 0):
            err = (outs[path][a:a + n].cpu() - want).abs().max().item()
            assert err < 3e-2 * max(1.0, want.abs().max().item()), (path, s, n, err)
