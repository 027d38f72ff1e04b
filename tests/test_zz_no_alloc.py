"""faws_attention_with_col_sum_noalloc, called through the C ABI.

This entry point exists for hosts that cannot give the library a workspace (their own pool
allocator owns the device, or cudaMalloc's device-wide synchronisation is not acceptable, or
the plugin interface passes tensor pointers only).  Its scratch is a fixed array inside the
library that every call shares and that keeps the previous call's contents, so the test makes
two different calls in a row and checks each against the ordinary entry point, which gets a
freshly allocated workspace.  The file sorts last so that a failure here cannot hide another
test's result in a run that stops at the first failure; it also passes when run alone.
"""
import ctypes as C

import pytest
import torch

import flash_attn_with_score_b200 as F
from flash_attn_with_score_b200 import _lib, api
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _noalloc_col_sum(q, k, v, causal, per_q_head=False):
    """Build the faws_problem exactly as the package does and call the C entry point."""
    call = api._Call(q, k, v, causal, None, 0.0)
    heads = call.H if per_q_head else call.Hk
    col = torch.full((call.B, heads, call.N), float("nan"), device=q.device, dtype=torch.float32)
    stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    torch.cuda.synchronize()
    held0 = torch.cuda.memory_allocated()
    rc = call.lib.faws_attention_with_col_sum_noalloc(C.byref(call.p), C.c_void_p(col.data_ptr()),
                                                      1 if per_q_head else 0, stream)
    torch.cuda.synchronize()
    # inputs and outputs were allocated above: the call itself asks the caller's allocator for nothing
    assert torch.cuda.memory_allocated() == held0
    return rc, call.out, col


def _inputs(shape, dtype, seed):
    B, Hq, Hk, S, D = shape
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g).to(dtype).cuda()
    k = torch.randn(B, Hk, S, D, generator=g).to(dtype).cuda()
    v = torch.randn(B, Hk, S, D, generator=g).to(dtype).cuda()
    return q, k, v


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # the third case fills half of the built-in array, the fourth is a small causal problem that runs over
    # whatever the third left there
    cases = [((1, 4, 2, 512, 128), torch.float16, True, False, 21),
             ((2, 6, 2, 320, 64), torch.bfloat16, False, True, 22),
             ((1, 16, 4, 2048, 64), torch.float16, False, False, 24),
             ((1, 2, 2, 192, 64), torch.float16, True, False, 25)]
    for shape, dtype, causal, per_q_head, seed in cases:
        q, k, v = _inputs(shape, dtype, seed)
        rc, out, col = _noalloc_col_sum(q, k, v, causal, per_q_head)
        assert rc == 0, _lib.load().faws_strerror(rc)
        ref_out, ref_col = F.attention_with_col_sum(q, k, v, causal, per_q_head=per_q_head)
        torch.cuda.synchronize()
        assert F.device_status() == 0
        assert col.shape == ref_col.shape
        ok, viol = orc.check_sum(col.cpu(), ref_col.cpu())
        assert ok, f"column sums differ from the workspace entry point: {viol}"
        assert torch.equal(col, ref_col), "same kernels, same order: results should be bit-identical"
        assert torch.equal(out, ref_out)
        # and against the CPU oracle, like the other parity tests
        o_ref, s_ref = orc.naive_attention_with_scores(q.cpu(), k.cpu(), v.cpu(), causal)
        want = orc.col_sum(s_ref) if per_q_head else orc.group_sum(orc.col_sum(s_ref), shape[2])
        ok, viol = orc.check_sum(col.cpu(), want)
        assert ok, viol


def test_rejects_problems_beyond_the_built_in_scratch():
    q, k, v = _inputs((1, 2, 2, 128, 64), torch.float16, 23)
    call = api._Call(q, k, v, True, None, 0.0)
    # claim a shape whose partial sums need 64 MiB; the size check comes before any launch
    call.p.Hq, call.p.Hk, call.p.M, call.p.N, call.p.m_end = 64, 64, 4096, 4096, 4096
    need = call.lib.faws_workspace_bytes(_lib.OP_COL_SUM, C.byref(call.p), 0)
    assert need > _lib.NOALLOC_SCRATCH_BYTES
    col = torch.empty(8, device="cuda")
    rc = call.lib.faws_attention_with_col_sum_noalloc(C.byref(call.p), C.c_void_p(col.data_ptr()), 0, None)
    assert rc == _lib.ETOOLARGE
    assert b"built-in" in call.lib.faws_strerror(rc)
    assert call.lib.faws_attention_with_col_sum_noalloc(None, None, 0, None) == -1
