"""Failure detection on the device, without a fault: a bounded mbarrier wait that runs out makes
the kernel raise the per-device status word and return; the context stays usable."""
import ctypes as C

import pytest
import torch

import flash_attn_with_score_b200 as F
from flash_attn_with_score_b200 import _lib

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    lib = _lib.load()
    assert F.device_status() == 0
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.faws_selftest_wait_give_up(stream) == 0  # nobody arrives at the barrier: the wait runs out
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 100.0, "the give-up limit is about a millisecond"
    assert F.device_status(reset=False) == 1
    assert F.device_status(reset=True) == 1
    assert F.device_status() == 0
    # the context is intact: an operator runs and leaves the word clear
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, 2, 128, 64, generator=g).half().cuda()
    out = F.attention(q, q, q, True)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert F.device_status() == 0
