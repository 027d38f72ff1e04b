"""attention() under autograd: dq, dk, dv through the C ABI (faws_attention_backward) against the CPU
oracle's torch-autograd gradients of the same fp32 formulas (the reference's FlashAttention.backward,
flash.py:172-261)."""
import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, Hq, Hk, M, N, D
    (1, 2, 2, 128, 128, 64),
    (2, 4, 2, 96, 96, 32),
    (1, 4, 1, 100, 100, 128),
    (1, 2, 1, 64, 160, 64),      # M < N
    (1, 2, 2, 160, 64, 16),      # M > N: causal rows without a visible key
    (1, 6, 2, 384, 384, 128),
    (1, 2, 1, 200, 328, 64),
    (2, 2, 2, 640, 640, 128),
]


def _inputs(shape, dtype, seed):
    B, Hq, Hk, M, N, D = shape
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    v = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    do = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    return q, k, v, do


def _run(q, k, v, do, causal, **kw):
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = F.attention(qd, kd, vd, causal, **kw)
    assert out.requires_grad and out.grad_fn is not None
    out.backward(do.cuda())
    return out.detach(), qd.grad, kd.grad, vd.grad


def _check(got, ref, what, bf16, slack):
    for name, x, r, sl in zip(("dq", "dk", "dv"), got, ref, slack):
        assert x.shape == r.shape and x.dtype in (torch.float16, torch.bfloat16), (what, name, x.shape, r.shape)
        ok, viol, err = orc.check_grad(x.cpu(), r, bf16, sl)
        assert ok, f"{what} {name}: violation {viol}, max abs err {err}"


@pytest.mark.parametrize("backend", ["generic", "auto", "tcgen05"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_backward_matches_autograd_oracle(shape, causal, dtype, backend):
    B, Hq, Hk, M, N, D = shape
    if backend == "tcgen05" and D not in (64, 128):
        pytest.skip("the tcgen05 kernels take head dims 64 and 128")  # forcing them elsewhere raises (tested below)
    q, k, v, do = _inputs(shape, dtype, seed=7)
    ref = orc.attention_backward(q, k, v, do, causal, p_seq=N - M)
    out, dq, dk, dv = _run(q, k, v, do, causal, backend=backend)
    ref_out, _ = orc.naive_attention_with_scores(q, k, v, causal, p_seq=N - M)
    assert (out.float().cpu() - ref_out).abs().max() < (2e-3 if dtype == torch.float16 else 3e-2)
    bf16 = dtype == torch.bfloat16
    _check((dq, dk, dv), ref, f"{shape} causal={causal} {backend}", bf16,
           orc.grad_slack(q, k, v, do, causal, p_seq=N - M, bf16=bf16))
    assert F.device_status() == 0


def test_backward_one_kv_group_of_cfg3():
    """cfg3's shape restricted to one kv head with its 7 query heads (bf16, S=4096, D=128, causal)."""
    shape = (1, 7, 1, 4096, 4096, 128)
    q, k, v, do = _inputs(shape, torch.bfloat16, seed=3)
    v = (v.float() * 0.5).to(torch.bfloat16)
    ref = orc.attention_backward(q, k, v, do, True)
    out, dq, dk, dv = _run(q, k, v, do, True, backend="tcgen05")
    _check((dq, dk, dv), ref, "cfg3 kv group", True, orc.grad_slack(q, k, v, do, True, bf16=True))
    assert F.device_status() == 0


def test_backward_with_dropout_matches_masked_oracle():
    shape = (1, 4, 2, 192, 192, 64)
    B, Hq, Hk, M, N, D = shape
    q, k, v, do = _inputs(shape, torch.float16, seed=5)
    seed, offset, p_drop = 1234, 64, 0.2
    keep = orc.dropout_keep_mask(seed, offset, B, Hq, M, N, p_drop)
    ref = orc.attention_backward(q, k, v, do, True, keep=keep, dropout_p=p_drop)
    out, dq, dk, dv = _run(q, k, v, do, True, dropout_p=p_drop, philox=(seed, offset))
    _, scores = orc.naive_attention_with_scores(q, k, v, True)
    assert (out.float().cpu() - orc.dropout_out(scores, v, keep, p_drop)).abs().max() < 4e-3
    sl = orc.grad_slack(q, k, v, do, True)
    _check((dq, dk, dv), ref, "dropout", False, tuple(x / (1.0 - p_drop) for x in sl))


def test_backward_is_deterministic_and_frees_the_caller_from_L():
    q, k, v, do = _inputs((1, 4, 2, 320, 320, 64), torch.float16, seed=9)
    a = _run(q, k, v, do, True)
    b = _run(q, k, v, do, True)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    # the 5-tuple form is differentiable in its first element too
    qd = q.cuda().requires_grad_(True)
    out, L, tot, _, _ = F.attention(qd, k.cuda(), v.cuda(), True, return_log_normalizer=True,
                                    return_total_attention=True)
    assert not L.requires_grad and not tot.requires_grad
    out.sum().backward()
    assert qd.grad is not None and torch.isfinite(qd.grad.float()).all()
    with pytest.raises(ValueError):
        F.attention(qd, k.cuda(), v.cuda(), True, q_rows=(0, 128))


def test_forcing_the_tcgen05_backward_on_an_unsupported_problem_raises():
    q, k, v, do = _inputs((1, 2, 2, 64, 64, 32), torch.float16, seed=1)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = F.attention(qd, kd, vd, True)  # forward on whichever family fits
    with pytest.raises(RuntimeError):
        torch.autograd.grad(F.attention(qd, kd, vd, True, backend="tcgen05"), (qd,), do.cuda())
    del out
