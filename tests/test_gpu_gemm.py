"""GPU parity: tcgen05 GEMM family vs the CPU oracle.

Shapes follow the reference's tests (tests/test_gemm.py:33-101 gemm / bmm /
group_gemm vs torch.matmul at rtol=atol=1e-2; tests/test_gemm_log_softmax.py:20-96
fp32 log_softmax(linear) oracle, row logsumexp ~ 0, out= aliasing) and the
GEMM shapes of the Conformer configs, plus ragged M/N/K tails.
"""
import pytest
import torch

import oasr_b200 as ob
from oracle import ops as O

pytestmark = pytest.mark.gpu

HALF = [torch.bfloat16, torch.float16]


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def _check(got, want, dtype, rtol=1e-2, atol=1e-2):
    got = got.float().cpu()
    torch.testing.assert_close(got, want.to(dtype).float(), rtol=rtol, atol=atol)


SHAPES = [
    (128, 128, 64), (128, 256, 128), (256, 512, 512), (1000, 1536, 512), (708, 2048, 256), (333, 264, 72),
    (1, 8, 16), (5, 5008, 256), (4096, 512, 2048), (129, 24, 200), (2000, 1024, 512), (64, 64, 64),
    (17, 776, 520), (300, 8, 8),
]


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm(dtype, M, N, K):
    A, B, C = _rand((M, K), dtype, 1), _rand((N, K), dtype, 2, K ** -0.5), _rand((N,), dtype, 3)
    _check(ob.gemm(A.cuda(), B.cuda(), C.cuda()), O.gemm(A, B, C), dtype)
    _check(ob.gemm(A.cuda(), B.cuda()), O.gemm(A, B), dtype)


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("M,N,K", [(1000, 1536, 512), (300, 520, 136), (128, 64, 64)])
def test_gemm_every_tile_width(bn, M, N, K):
    from oasr_b200 import tunables

    dtype = torch.bfloat16
    A, B, C = _rand((M, K), dtype, 1), _rand((N, K), dtype, 2, K ** -0.5), _rand((N,), dtype, 3)
    tunables.set("gemm_bn", bn)
    try:
        _check(ob.gemm(A.cuda(), B.cuda(), C.cuda()), O.gemm(A, B, C), dtype)
    finally:
        tunables.set("gemm_bn", 0)


def test_gemm_is_deterministic_and_leading_dims():
    dtype = torch.bfloat16
    A, B = _rand((3, 70, 512), dtype, 4), _rand((1024, 512), dtype, 5, 0.05)
    y1 = ob.gemm(A.cuda(), B.cuda())
    y2 = ob.gemm(A.cuda(), B.cuda())
    assert y1.shape == (3, 70, 1024) and torch.equal(y1, y2)
    out = torch.empty(3, 70, 1024, device="cuda", dtype=dtype)
    assert ob.gemm(A.cuda(), B.cuda(), out=out) is out and torch.equal(out, y1)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("act", [0, 1, 2, 4])
def test_gemm_activation(dtype, act):
    M, N, K = 700, 2048, 512
    A, B, C = _rand((M, K), dtype, 6), _rand((N, K), dtype, 7, K ** -0.5), _rand((N,), dtype, 8)
    _check(ob.gemm_activation(A.cuda(), B.cuda(), C.cuda(), act), O.gemm(A, B, C, act), dtype)


def test_gemm_rejects_bad_inputs():
    A = torch.randn(16, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):  # N not a multiple of 8 (reference CHECK_GEMM_ALIGNMENT)
        ob.gemm(A, torch.randn(5002, 64, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):  # dtype mismatch
        ob.gemm(A, torch.randn(8, 64, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError):  # fp32 is not a GEMM dtype
        ob.gemm(A.float(), torch.randn(8, 64, device="cuda"))
    with pytest.raises(RuntimeError):  # K mismatch
        ob.gemm(A, torch.randn(8, 32, device="cuda", dtype=torch.bfloat16))


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("M,N,K", [(1000, 512, 512), (333, 256, 256), (64, 1024, 1024), (130, 72, 264)])
def test_gemm_glu(dtype, M, N, K):
    A, B, C = _rand((M, K), dtype, 9), _rand((2 * N, K), dtype, 10, K ** -0.5), _rand((2 * N,), dtype, 11)
    _check(ob.gemm_glu(A.cuda(), B.cuda(), C.cuda()), O.gemm_glu(A, B, C), dtype)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("M,N,K,alpha", [(1000, 512, 2048, 0.5), (333, 256, 256, 1.0), (129, 1024, 520, 1.0)])
def test_gemm_residual_f32(dtype, M, N, K, alpha):
    A, B, C = _rand((M, K), dtype, 12), _rand((N, K), dtype, 13, K ** -0.5), _rand((N,), dtype, 14)
    R = _rand((M, N), torch.float32, 15)
    got = ob.gemm_residual_f32(R.cuda(), A.cuda(), B.cuda(), C.cuda(), alpha)
    want = R + alpha * O.gemm(A, B, C)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-4)
    Rg = R.cuda()
    assert ob.gemm_residual_f32(Rg, A.cuda(), B.cuda(), C.cuda(), alpha, out=Rg) is Rg  # in place
    torch.testing.assert_close(Rg.cpu(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("b,M,N,K", [(16, 200, 200, 64), (3, 130, 72, 136), (256, 16, 272, 64), (2, 1, 8, 16)])
def test_bmm(dtype, b, M, N, K):
    A, B = _rand((b, M, K), dtype, 16), _rand((b, N, K), dtype, 17, K ** -0.5)
    _check(ob.bmm(A.cuda(), B.cuda()), O.bmm(A, B), dtype)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("sizes", [[128, 128], [100, 0, 300, 7], [1], [513, 64, 255]])
def test_group_gemm(dtype, sizes):
    N, K = 264, 136
    L, G = sum(sizes), len(sizes)
    offs = torch.tensor(sizes).cumsum(0).to(torch.int32)
    A, B = _rand((L, K), dtype, 18), _rand((G, N, K), dtype, 19, K ** -0.5)
    _check(ob.group_gemm(A.cuda(), B.cuda(), offs.cuda()), O.group_gemm(A, B, offs.tolist()), dtype)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("M,N,K", [(708, 5008, 256), (300, 5008, 512), (64, 1024, 1024), (5, 8, 64), (130, 264, 72),
                                   (40, 9008, 64)])
@pytest.mark.parametrize("path", [1, 2])
def test_gemm_log_softmax(dtype, M, N, K, path):
    """path 1 = the fused two-sweep kernel, 2 = fp32 logits GEMM + in-place row log-softmax (fp32 output)."""
    from oasr_b200 import tunables

    A, B, C = _rand((M, K), dtype, 20), _rand((N, K), dtype, 21, K ** -0.5), _rand((N,), dtype, 22)
    want = O.gemm_log_softmax(A, B, C)
    tunables.set("lsm_path", path)
    try:
        got32, arg = ob.gemm_log_softmax(A.cuda(), B.cuda(), C.cuda(), out_dtype=torch.float32, return_argmax=True)
    finally:
        tunables.set("lsm_path", 0)
    assert ob.device_status() == 0
    torch.testing.assert_close(got32.cpu(), want, rtol=1e-4, atol=2e-4)
    # every row is a normalised distribution (reference tests/test_gemm_log_softmax.py: |logsumexp| < 5e-3)
    assert got32.logsumexp(-1).abs().max().item() < 1e-4
    got_arg = arg.cpu().long()
    want_arg = want.argmax(-1)
    same = got_arg == want_arg
    # a differing argmax is only acceptable on a numerical tie
    assert torch.all(same | ((want.gather(1, got_arg[:, None]) - want.gather(1, want_arg[:, None])).abs()[:, 0] < 1e-5))
    got16 = ob.gemm_log_softmax(A.cuda(), B.cuda(), C.cuda())
    assert got16.dtype == dtype
    torch.testing.assert_close(got16.float().cpu(), want, rtol=2e-2, atol=5e-2)


def test_gemm_log_softmax_padding_rows_are_inert():
    """Vocabulary padded 5002 -> 5008 with zero weight rows and bias -1e4
    (reference oasr/models/base.py:163-197): a padding class never wins and takes no mass."""
    dtype = torch.bfloat16
    M, N, K, raw = 200, 5008, 256, 5002
    A, B, C = _rand((M, K), dtype, 23), _rand((N, K), dtype, 24, 0.02), torch.zeros(N, dtype=dtype)
    B[raw:] = 0
    C[raw:] = -1e4
    got, arg = ob.gemm_log_softmax(A.cuda(), B.cuda(), C.cuda(), out_dtype=torch.float32, return_argmax=True)
    assert int(arg.max()) < raw
    want = O.gemm_log_softmax(A[:, :], B[:raw], C[:raw])
    torch.testing.assert_close(got[:, :raw].cpu(), want, rtol=1e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", HALF)
@pytest.mark.parametrize("M,N,K", [(1024, 256, 128), (1300, 520, 264), (4096, 2048, 512), (2049, 512, 2048),
                                   (17536, 512, 512)])
def test_gemm_cta_pairs_match_single_cta_tiles(dtype, M, N, K):
    """Large dense problems run on CTA pairs (cta_group::2); same products, same rounding as the
    single-CTA kernel and the oracle."""
    from oasr_b200 import tunables

    A, B, C = _rand((M, K), dtype, 31), _rand((N, K), dtype, 32, K ** -0.5), _rand((N,), dtype, 33)
    want = O.gemm(A, B, C, 2)
    got_single = ob.gemm_activation(A.cuda(), B.cuda(), C.cuda(), 2)
    tunables.set("gemm_pairs", 1)
    try:
        got_pair = ob.gemm_activation(A.cuda(), B.cuda(), C.cuda(), 2)
        if N % 2 == 0:
            Bg, Cg = _rand((2 * N, K), dtype, 34, K ** -0.5), _rand((2 * N,), dtype, 35)
            _check(ob.gemm_glu(A.cuda(), Bg.cuda(), Cg.cuda()), O.gemm_glu(A, Bg, Cg), dtype)
    finally:
        tunables.set("gemm_pairs", 0)
    _check(got_pair, want, dtype)
    _check(got_single, want, dtype)
    assert torch.equal(got_pair, got_single)   # fp32 accumulation order along K is the same
    if N % 2 == 0:
        Bg, Cg = _rand((2 * N, K), dtype, 34, K ** -0.5), _rand((2 * N,), dtype, 35)
        _check(ob.gemm_glu(A.cuda(), Bg.cuda(), Cg.cuda()), O.gemm_glu(A, Bg, Cg), dtype)


# ---- the regime the benchmark runs: M ~ 17k packed frames, ~1100 output tiles, ~7 tiles per persistent CTA, so the
# ---- accumulator double buffer and the operand ring wrap their phases many times inside one launch
BENCH_M = 16722          # packed frames of the headline batch (64 utterances, lengths seed 2024)


def _sample_rows(M, n=1536, seed=0):
    g = torch.Generator().manual_seed(seed)
    rows = torch.randperm(M, generator=g)[:n]
    edge = torch.arange(max(M - 200, 0), M)                   # the ragged last tile, entirely
    return torch.unique(torch.cat([rows, edge, torch.arange(0, min(M, 130))]))


@pytest.mark.parametrize("M,N,K,act", [(BENCH_M, 2048, 512, 2), (BENCH_M, 512, 2048, -1), (BENCH_M, 512, 512, -1),
                                       (BENCH_M, 1536, 512, -1), (BENCH_M, 2048, 512, -1), (17500, 512, 1520, -1)])
def test_gemm_at_benchmark_size_on_sampled_rows(M, N, K, act):
    dtype = torch.bfloat16
    A, B, C = _rand((M, K), dtype, 11), _rand((N, K), dtype, 12, K ** -0.5), _rand((N,), dtype, 13)
    got = (ob.gemm_activation(A.cuda(), B.cuda(), C.cuda(), act) if act >= 0 else ob.gemm(A.cuda(), B.cuda(), C.cuda()))
    rows = _sample_rows(M)
    want = O.gemm(A[rows], B, C, act) if act >= 0 else O.gemm(A[rows], B, C)
    _check(got[rows.cuda()], want, dtype)
    # every row, against the same product in fp32 on the device (cuBLAS used as a checker only)
    ref = torch.nn.functional.linear(A.cuda().float(), B.cuda().float(), C.cuda().float())
    if act >= 0:
        ref = O.activation(ref.cpu(), act).cuda()
    torch.testing.assert_close(got.float(), ref.to(dtype).float(), rtol=2e-2, atol=2e-2)
    assert ob.device_status() == 0


def test_gemm_glu_at_benchmark_size():
    dtype = torch.bfloat16
    M, N, K = BENCH_M, 512, 512
    A, B, C = _rand((M, K), dtype, 14), _rand((2 * N, K), dtype, 15, K ** -0.5), _rand((2 * N,), dtype, 16)
    got = ob.gemm_glu(A.cuda(), B.cuda(), C.cuda())
    rows = _sample_rows(M)
    _check(got[rows.cuda()], O.gemm_glu(A[rows], B, C), dtype)
    y = torch.nn.functional.linear(A.cuda().float(), B.cuda().float(), C.cuda().float())
    ref = y[:, :N] * torch.sigmoid(y[:, N:])
    torch.testing.assert_close(got.float(), ref.to(dtype).float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M", [BENCH_M, 12032])     # above and just above the row-tile count where the fused sweep form takes over
def test_gemm_log_softmax_default_path_at_benchmark_size(M):
    dtype = torch.bfloat16
    N, K = 5008, 512
    A, B, C = _rand((M, K), dtype, 17), _rand((N, K), dtype, 18, K ** -0.5), _rand((N,), dtype, 19, 0.1)
    out, arg = ob.gemm_log_softmax(A.cuda(), B.cuda(), C.cuda(), out_dtype=torch.float32, return_argmax=True)
    rows = _sample_rows(M, 1024)
    want = O.gemm_log_softmax(A[rows], B, C)
    got = out[rows.cuda()].cpu()
    assert (got - want).abs().max().item() < 2e-2
    assert out.logsumexp(-1).abs().max().item() < 1e-3
    assert torch.equal(arg.long(), out.argmax(-1))
    assert ob.device_status() == 0


@pytest.mark.parametrize("M", [1, 300, 4096, BENCH_M])
def test_token_only_head_equals_the_argmax_of_the_log_probs(M):
    """out == NULL: one vocabulary sweep, only the first-maximum index per row -- the same index the log-prob form
    reports, and the argmax of the oracle's log-probs wherever that is not a numerical tie."""
    from oasr_b200 import fused

    dtype = torch.bfloat16
    N, K = 5008, 512
    A, B, C = _rand((M, K), dtype, 21), _rand((N, K), dtype, 22, K ** -0.5), _rand((N,), dtype, 23, 0.1)
    got = fused.gemm_argmax(A.cuda(), B.cuda(), C.cuda())
    out, arg = ob.gemm_log_softmax(A.cuda(), B.cuda(), C.cuda(), out_dtype=torch.float32, return_argmax=True)
    assert got.dtype == torch.int32 and got.shape == (M,)
    if M > 93 * 128:                                           # both forms ran the same sweep kernel: identical
        assert torch.equal(got, arg)
    rows = _sample_rows(M, 512) if M > 2000 else torch.arange(M)
    want = O.gemm_log_softmax(A[rows], B, C)
    top2 = want.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2e-2
    assert torch.equal(got[rows.cuda()].cpu().long()[clear], want.argmax(-1)[clear])
    assert ob.device_status() == 0


@pytest.mark.parametrize("M", [1, 130, 4096, 16722])
def test_gemm_dup_first_equals_the_gemm_with_the_repeated_weight_block(M):
    """The fused q/q/k/v projection form: the first d columns of the product are stored twice, each copy with the bias
    of its output column -- bit for bit the plain GEMM against [Wq; Wq; Wk; Wv], the shape the layer stack runs."""
    from oasr_b200 import fused

    d = 512
    g = torch.Generator().manual_seed(M)
    A = torch.randn(M, d, generator=g).bfloat16().cuda()
    W3 = (torch.randn(3 * d, d, generator=g) * d ** -0.5).bfloat16().cuda()
    bias4 = torch.randn(4 * d, generator=g).bfloat16().cuda()
    W4 = torch.cat([W3[:d], W3], 0).contiguous()
    want = ob.gemm(A, W4, bias4)
    got = fused.gemm_dup_first(A, W3, bias4, d)
    # and reading [Wq; Wk; Wv] in place, as rows d.. of the repeated form
    got_view = fused.gemm_dup_first(A, W4[d:], bias4, d)
    assert ob.device_status() == 0
    assert got.shape == (M, 4 * d) and torch.equal(got, want) and torch.equal(got_view, want)
    with pytest.raises(Exception, match="multiples of 256"):
        fused.gemm_dup_first(A, W3[:3 * d - 8], bias4, d)
