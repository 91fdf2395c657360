"""GPU parity of the 8-bit operand GEMM kinds (fp8 e4m3, W8A8 int8) against their CPU restatement, and the
cosine gate of the quantised result against the 16-bit GEMM on the unquantised operands."""
import pytest
import torch

import oasr_b200 as ob
from oasr_b200 import quant
from oracle import ops as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [quant.FP8_E4M3, quant.INT8])
@pytest.mark.parametrize("rows,cols", [(37, 512), (300, 2048), (5, 16), (0, 64)])
def test_quantize_rows_is_bit_exact_against_the_restatement(kind, rows, cols):
    torch.manual_seed(rows + cols)
    x = (torch.randn(rows, cols) * torch.rand(rows, 1) * 3).bfloat16()
    if rows > 2:
        x[1] = 0                                             # an all-zero row keeps scale 1 and codes 0
    q, s = quant.quantize_rows(x.cuda(), kind)
    want_q, want_s, _ = O.quantize_rows(x, kind)
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu(), want_q)


@pytest.mark.parametrize("kind", [quant.FP8_E4M3, quant.INT8])
@pytest.mark.parametrize("M,N,K,act,glu,bias", [
    (300, 512, 512, -1, False, True), (1000, 2048, 512, 2, False, True), (777, 512, 2048, -1, False, False),
    (129, 264, 80, 0, False, True), (513, 512, 512, -1, True, True), (64, 64, 16, -1, False, False)])
def test_gemm_q8_matches_the_restatement_and_the_cosine_gate(kind, M, N, K, act, glu, bias):
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K).bfloat16()
    B = (torch.randn(N * (2 if glu else 1), K) * 0.05).bfloat16()
    b = (torch.randn(N * (2 if glu else 1)) * 0.1).bfloat16() if bias else None
    aq, sa = quant.quantize_rows(A.cuda(), kind)
    bq, sb = quant.quantize_rows(B.cuda(), kind)
    got = quant.gemm_q8(aq, sa, bq, sb, b.cuda() if bias else None, kind=kind, activation=act, glu=glu).float().cpu()
    assert ob.device_status() == 0
    _, wsa, av = O.quantize_rows(A, kind)
    _, wsb, bv = O.quantize_rows(B, kind)
    want = O.gemm_q8(av, wsa, bv, wsb, b, act, glu)
    scale = want.abs().max().item() + 1e-6
    assert (got - want).abs().max().item() <= 1e-2 * scale, ((got - want).abs().max().item(), scale)
    # against the 16-bit GEMM of the unquantised operands: cosine >= 0.999
    y = A.float() @ B.float().t() + (b.float() if bias else 0)
    ref = y[:, :N] * torch.sigmoid(y[:, N:]) if glu else (O.activation(y, act) if act >= 0 else y)
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert cos >= 0.999, cos


@pytest.mark.parametrize("mode", ["fp8", "int8"])
def test_quantised_encoder_reaches_the_cosine_gate_against_the_16_bit_run(mode):
    """Model level: the eight Linear GEMMs of every layer on 8-bit operands (per-channel weight scales,
    per-token dynamic activation scales) against the bf16 run of the same model and batch: cosine >= 0.999
    on the valid frames' log-probs, and argmax agreement reported."""
    from oasr_b200.encoder import ConformerCTC, ConformerConfig
    from oasr_b200.weights import init_params

    cfg = ConformerConfig(d_model=256, heads=4, ffn=1024, layers=4, vocab=500)
    P = init_params(cfg, 77)
    lengths = [403, 250, 1000, 131]
    feats = torch.randn(len(lengths), max(lengths), cfg.input_size, generator=torch.Generator().manual_seed(3)).cuda()
    ref_model = ConformerCTC(cfg, P)
    q_model = ConformerCTC(cfg, P, quant=mode)
    ref, _, pk = ref_model.forward_offline_packed(feats, lengths, padded_output=False)
    got, _, _ = q_model.forward_offline_packed(feats, lengths, padded_output=False)
    assert ob.device_status() == 0
    assert torch.isfinite(got).all()
    a, b = got[:, :cfg.vocab].flatten().double(), ref[:, :cfg.vocab].flatten().double()
    cos = torch.nn.functional.cosine_similarity(a, b, dim=0).item()
    agree = (got[:, :cfg.vocab].argmax(-1) == ref[:, :cfg.vocab].argmax(-1)).float().mean().item()
    print(f"{mode}: cosine {cos:.6f}, argmax agreement with the bf16 run {agree:.4f}, max-abs {(got - ref)[:, :cfg.vocab].abs().max().item():.3e}")
    assert cos >= 0.999, cos


@pytest.mark.parametrize("kind", [1, 2])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_add_norm_with_8bit_output_equals_add_norm_then_quantize_rows(kind, mode):
    """oasr_b200_add_norm_f32_q8 writes, beside h, the row of h in 8 bits with its scale: the same bytes and scales
    as quantize_rows(h), and h / the residual stream exactly as oasr_b200_add_norm_f32 leaves them."""
    from oasr_b200 import fused, quant

    rows, hidden = 333, 512
    g = torch.Generator().manual_seed(5)
    res = torch.randn(rows, hidden, generator=g).cuda()
    y = torch.randn(rows, hidden, generator=g).cuda().bfloat16()
    if mode == 1:
        w_a, b_a = torch.rand(hidden, generator=g).cuda() + 0.5, torch.randn(hidden, generator=g).cuda()
    else:
        w_a, b_a = (torch.rand(hidden, generator=g).cuda() + 0.5).bfloat16(), torch.randn(hidden, generator=g).cuda().bfloat16()
    w_b, b_b = (torch.rand(hidden, generator=g).cuda() + 0.5).bfloat16(), torch.randn(hidden, generator=g).cuda().bfloat16()
    h1, r1 = torch.empty(rows, hidden, device="cuda", dtype=torch.bfloat16), torch.empty_like(res)
    h2, r2 = torch.empty_like(h1), torch.empty_like(res)
    fused.add_norm_f32(h1, r1, res, y, 0.5, mode, w_a, b_a, w_b if mode == 2 else None, b_b if mode == 2 else None)
    q, s = fused.add_norm_f32_q8(h2, r2, res, y, 0.5, mode, w_a, b_a, w_b if mode == 2 else None, b_b if mode == 2 else None, kind=kind)
    assert ob.device_status() == 0
    assert torch.equal(h1, h2) and torch.equal(r1, r2)
    q_ref, s_ref = quant.quantize_rows(h1, kind)
    assert torch.equal(s, s_ref) and torch.equal(q, q_ref)
