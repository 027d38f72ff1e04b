"""Split-KV attention (few query rows, keys cut into ranges with a deterministic combine; the
reference's flash.py:68-70,97-134 and split_kv.py) against the CPU oracle and the unsplit kernel."""
import ctypes as C

import pytest
import torch

import flash_attn_with_score_b200 as F
from flash_attn_with_score_b200 import _lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, Hq, Hk, M, N, D
    (1, 4, 2, 1, 2048, 128),     # one-token decode
    (2, 8, 2, 16, 4096, 128),
    (1, 2, 1, 128, 1024, 64),
    (1, 2, 2, 200, 1000, 64),    # ragged M and N
    (1, 4, 4, 130, 2048, 128),   # two query tiles, the second nearly empty
]


def _inputs(shape, dtype, seed=0):
    B, Hq, Hk, M, N, D = shape
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    v = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_split_kv_matches_oracle_and_unsplit(shape, causal, dtype):
    B, Hq, Hk, M, N, D = shape
    q, k, v = _inputs(shape, dtype, seed=13)
    ref_out, ref_scores = orc.naive_attention_with_scores(q, k, v, causal, p_seq=N - M)
    slack = orc.bf16_out_slack(ref_scores, v, ref_out) if dtype == torch.bfloat16 else None
    Lref = orc.log_normalizer(ref_scores)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    one, L1, _, _, _ = F.attention(qd, kd, vd, causal, return_log_normalizer=True, kv_splits=1)
    for splits in (None, 2, 5, (N + 127) // 128):
        out, L, _, _, _ = F.attention(qd, kd, vd, causal, return_log_normalizer=True, kv_splits=splits)
        assert F.last_backend() == "tcgen05"
        ok, err = orc.check_out(out.cpu(), ref_out, slack)
        assert ok, (splits, err)
        fin = torch.isfinite(Lref)
        assert torch.equal(torch.isneginf(L.cpu()), ~fin)
        assert (L.cpu()[fin] - Lref[fin]).abs().max() < 2e-3
        # partial results are stored in 16 bits before the combine: one extra rounding against the unsplit kernel
        assert (out.float() - one.float()).abs().max() < (4e-3 if dtype == torch.float16 else 3e-2)
        again = F.attention(qd, kd, vd, causal, kv_splits=splits)
        assert torch.equal(again, out), "the combine must be deterministic"
    assert F.device_status() == 0


def test_split_plan_follows_the_occupancy_rule():
    lib = _lib.load()
    q, k, v = (t.cuda() for t in _inputs((1, 4, 2, 16, 16384, 128), torch.float16))
    out = torch.empty_like(q)

    def plan(qq, kk, vv, causal=False, dropout=0.0):
        p = _lib.Problem()
        p.B, p.Hq, p.M, p.D = qq.shape
        p.Hk, p.N = kk.shape[1], kk.shape[2]
        p.dtype, p.causal, p.sm_scale, p.m_end = _lib.FP16, int(causal), 0.088, qq.shape[2]
        t = lambda x: _lib.Tensor(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))  # noqa: E731
        p.q, p.k, p.v, p.out = t(qq), t(kk), t(vv), t(torch.empty_like(qq))
        p.dropout_p = dropout
        return lib.faws_split_kv_plan(C.byref(p))

    assert plan(q, k, v) > 1                      # 4 CTAs on 148 SMs: split
    assert plan(q, k, v, dropout=0.1) == 1        # never with dropout (flash.py:98)
    big = torch.empty(4, 32, 1024, 128, device="cuda", dtype=torch.float16)
    assert plan(big, big, big) == 1               # 1024 CTAs: enough work already
    del out
