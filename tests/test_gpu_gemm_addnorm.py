"""GPU parity: Linear + residual add + LayerNorm in one kernel (``oasr_b200_gemm_add_norm_f32``) against the fp32
composition it replaces: ``gemm`` (csrc/gemm_jit_binding.cu:9-12) then ``add_layer_norm_residual``
(include/oasr/norm.cuh:396-484) as ConformerEncoderLayer.forward_packed chains them
(oasr/models/conformer/model.py:722-751), with the residual stream kept in fp32."""
import pytest
import torch
import torch.nn.functional as F

import oasr_b200 as ob
from oasr_b200 import _lib, fused

pytestmark = pytest.mark.gpu


def test_blocked_residual_layout_round_trip_and_element_rule():
    M, N = 70, 128
    res = torch.arange(M * N, dtype=torch.float32, device="cuda").view(M, N)
    blk = fused.residual_to_blocked(res)
    assert blk.numel() == 96 * N
    assert torch.equal(fused.residual_from_blocked(blk, M, N), res)
    for row, col in [(0, 0), (33, 5), (69, 127), (31, 96)]:
        band, l, chunk, j, e = row // 32, row % 32, col // 32, (col % 32) // 4, col % 4
        off = (band * (N // 32) + chunk) * 1024 + (j * 32 + l) * 4 + e
        assert blk[off].item() == res[row, col].item()


def _case(M, N, K, dtype, seed, with_res=True):
    g = torch.Generator().manual_seed(seed)
    A = torch.randn(M, K, generator=g).to(dtype)
    B = (torch.randn(N, K, generator=g) * K ** -0.5).to(dtype)
    bias = (torch.randn(N, generator=g) * 0.3).to(dtype)
    res = torch.randn(M, N, generator=g) * 2.0 + 0.7 if with_res else None
    w1, b1 = (1.0 + 0.2 * torch.randn(N, generator=g)).to(dtype), (0.2 * torch.randn(N, generator=g)).to(dtype)
    w2, b2 = (1.0 + 0.2 * torch.randn(N, generator=g)).to(dtype), (0.2 * torch.randn(N, generator=g)).to(dtype)
    return A, B, bias, res, w1, b1, w2, b2


def _reference(A, B, bias, res, alpha, mode, w1, b1, w2, b2, eps):
    y = F.linear(A.float(), B.float(), None if bias is None else bias.float())
    s = alpha * y if res is None else res + alpha * y
    if mode == 0:
        return s, F.layer_norm(s, (s.size(-1),), w1.float(), b1.float(), eps)
    if mode == 1:
        return s, s * w1.float() + b1.float()
    r = F.layer_norm(s, (s.size(-1),), w1.float(), b1.float(), eps)
    return r, F.layer_norm(r, (r.size(-1),), w2.float(), b2.float(), eps)


def _run(A, B, bias, res, alpha, mode, w1, b1, w2, b2, eps, split=False, in_place=True):
    M, N = A.size(0), B.size(0)
    dev = "cuda"
    h = torch.full((M, N * (2 if split else 1)), float("nan"), device=dev, dtype=A.dtype)
    # the residual stream travels in the kernel's blocked layout
    res_in = None if res is None else fused.residual_to_blocked(res.to(dev))
    Mp = (M + 31) // 32 * 32
    res_out = res_in if (in_place and res_in is not None) else torch.full((Mp * N,), float("nan"), device=dev)
    wa, ba = (w1.float().to(dev), b1.float().to(dev)) if mode == 1 else (w1.to(dev), b1.to(dev))
    fused.gemm_add_norm_f32(h, res_out, res_in, A.to(dev), B.to(dev), None if bias is None else bias.to(dev), alpha, mode,
                            wa, ba, w2.to(dev) if mode == 2 else None, b2.to(dev) if mode == 2 else None, eps, split)
    torch.cuda.synchronize()
    assert ob.device_status() == 0
    return fused.residual_from_blocked(res_out, M, N).cpu(), h.float().cpu()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("M,N,K", [(300, 512, 512), (256, 512, 2048), (1, 512, 64), (1000, 256, 256), (130, 128, 256),
                                   (517, 512, 520), (129, 256, 1032)])
def test_gemm_add_norm_matches_the_fp32_composition(dtype, mode, M, N, K):
    A, B, bias, res, w1, b1, w2, b2 = _case(M, N, K, dtype, 100 + mode)
    alpha, eps = (0.5, 1e-5) if mode != 1 else (1.0, 1e-5)
    want_res, want_h = _reference(A, B, bias, res, alpha, mode, w1, b1, w2, b2, eps)
    got_res, got_h = _run(A, B, bias, res, alpha, mode, w1, b1, w2, b2, eps)
    # the residual stream is fp32 end to end: only the 16-bit GEMM operands were rounded (identically on both sides)
    torch.testing.assert_close(got_res, want_res, rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(got_h, want_h.to(dtype).float(), rtol=2e-2, atol=2e-2)


def test_without_residual_input_without_bias_and_out_of_place():
    dtype = torch.bfloat16
    A, B, bias, res, w1, b1, w2, b2 = _case(700, 512, 1216, dtype, 7, with_res=False)
    want_res, want_h = _reference(A, B, None, None, 1.0, 2, w1, b1, w2, b2, 1e-5)
    got_res, got_h = _run(A, B, None, None, 1.0, 2, w1, b1, w2, b2, 1e-5)
    torch.testing.assert_close(got_res, want_res, rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(got_h, want_h.to(dtype).float(), rtol=2e-2, atol=2e-2)
    A, B, bias, res, w1, b1, w2, b2 = _case(300, 256, 512, dtype, 8)
    want_res, want_h = _reference(A, B, bias, res, 0.5, 0, w1, b1, w2, b2, 1e-5)
    got_res, got_h = _run(A, B, bias, res, 0.5, 0, w1, b1, w2, b2, 1e-5, in_place=False)
    torch.testing.assert_close(got_res, want_res, rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(got_h, want_h.to(dtype).float(), rtol=2e-2, atol=2e-2)


def test_split_output_rows_are_hi_lo():
    dtype = torch.bfloat16
    M, N, K = 333, 512, 2048
    A, B, bias, res, w1, b1, w2, b2 = _case(M, N, K, dtype, 9)
    want_res, want_h = _reference(A, B, bias, res, 0.5, 2, w1, b1, w2, b2, 1e-5)
    got_res, got_h3 = _run(A, B, bias, res, 0.5, 2, w1, b1, w2, b2, 1e-5, split=True)
    hi, lo = got_h3[:, :N], got_h3[:, N:]
    assert hi.shape == lo.shape
    # hi + lo carries the fp32 value to ~16 mantissa bits (bf16 GEMM-operand rounding of A / B is common to both sides)
    torch.testing.assert_close(hi + lo, want_h, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(got_res, want_res, rtol=1e-4, atol=2e-4)


@pytest.mark.parametrize("N,K,mode", [(512, 512, 0), (512, 2048, 2), (512, 512, 1)])
def test_at_benchmark_size_equals_gemm_then_add_norm(N, K, mode):
    """M = the packed frames of the headline batch (66 CTA pairs, one tile each): the fused kernel against this
    library's own two-kernel composition; the only difference allowed is the 16-bit rounding of y the fusion removes."""
    dtype = torch.bfloat16
    M = 16722
    A, B, bias, res, w1, b1, w2, b2 = _case(M, N, K, dtype, 10)
    got_res, got_h = _run(A, B, bias, res, 0.5, mode, w1, b1, w2, b2, 1e-5)
    want_res, want_h = _reference(A, B, bias, res, 0.5, mode, w1, b1, w2, b2, 1e-5)
    torch.testing.assert_close(got_res, want_res, rtol=1e-4, atol=3e-4)
    torch.testing.assert_close(got_h, want_h.to(dtype).float(), rtol=2e-2, atol=2e-2)
    # the unfused composition on the same inputs
    dev = "cuda"
    y = ob.gemm(A.to(dev), B.to(dev), bias.to(dev))   # (this path keeps its residual row-major)
    h2 = torch.empty(M, N, device=dev, dtype=dtype)
    r2 = res.to(dev)
    wa, ba = (w1.float().to(dev), b1.float().to(dev)) if mode == 1 else (w1.to(dev), b1.to(dev))
    fused.add_norm_f32(h2, r2, r2, y, 0.5, mode, wa, ba, w2.to(dev) if mode == 2 else None, b2.to(dev) if mode == 2 else None)
    torch.testing.assert_close(h2.float().cpu(), got_h, rtol=2e-2, atol=2e-2)   # within a 16-bit rounding step of each other


def test_unsupported_width_is_refused():
    assert _lib.load().oasr_b200_gemm_add_norm_supported(512, 512) == 1
    assert _lib.load().oasr_b200_gemm_add_norm_supported(384, 512) == 0
    A, B, bias, res, w1, b1, w2, b2 = _case(64, 384, 128, torch.bfloat16, 3)
    with pytest.raises(_lib.OasrB200Error, match="tensor memory"):
        _run(A, B, bias, res, 1.0, 0, w1, b1, w2, b2, 1e-5)
