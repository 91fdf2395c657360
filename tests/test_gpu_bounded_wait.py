"""GPU: a bounded device wait that runs out is reported to the host and leaves the context usable.

Every TMA / tcgen05 pipeline of the library polls its mbarriers a bounded number of times; past the limit the
waiter raises the CTA's abort flag, the other roles drain, a bit goes into the device status word and tensor memory
is released.  The self-test kernel takes exactly that path (a wait on a barrier nothing signals, limit of a few
thousand polls).  No fault, trap or endless loop is involved.
"""
import ctypes

import pytest
import torch

import oasr_b200 as ob
from oasr_b200 import _lib

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_sets_the_status_word_and_the_next_kernels_run():
    assert ob.device_status() == 0
    report = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.call("oasr_b200_selftest_bounded_wait", 4096, ctypes.c_void_p(report.data_ptr()), stream)
    torch.cuda.synchronize()
    assert int(report.item()) == 3                       # both roles gave up: the waiter and the one behind it
    with pytest.raises(_lib.OasrB200Error) as err:
        ob.device_status()
    assert err.value.code == _lib.ERR_DEVICE_WAIT and "0x00000100" in str(err.value)
    assert ob.device_status() == 0                       # reading cleared the word
    # the context is intact: a tensor-core GEMM (TMEM allocation, TMA, mbarriers) right after it is correct
    A = torch.randn(300, 256, device="cuda").bfloat16()
    B = torch.randn(512, 256, device="cuda").bfloat16()
    got = ob.gemm(A, B).float()
    torch.testing.assert_close(got, (A.float() @ B.float().t()).bfloat16().float(), rtol=2e-2, atol=2e-2)
    assert ob.device_status() == 0


def test_selftest_rejects_limits_outside_its_range():
    with pytest.raises(_lib.OasrB200Error):
        _lib.call("oasr_b200_selftest_bounded_wait", 8, None, None)
    with pytest.raises(_lib.OasrB200Error):
        _lib.call("oasr_b200_selftest_bounded_wait", 1 << 30, None, None)
