"""Randomised shapes: the tcgen05 kernels against the CUDA-core kernels on the device (both go
through the C ABI), plus the CPU oracle for the smaller draws.  Catches edge cases of ragged lengths,
query windows, splits and GQA that the fixed shape lists may miss."""
import random

import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _draw(rng):
    D = rng.choice([64, 128])
    Hk = rng.choice([1, 2, 3])
    G = rng.choice([1, 2, 4, 7])
    B = rng.choice([1, 2])
    M = rng.choice([rng.randrange(1, 40) * 8, rng.randrange(1, 12) * 128, rng.randrange(8, 900)])
    N = rng.choice([M, rng.randrange(1, 120) * 8, rng.randrange(1, 9) * 128])
    causal = rng.random() < 0.6
    dtype = rng.choice([torch.float16, torch.bfloat16])
    return B, Hk * G, Hk, M, N, D, causal, dtype


def _close(a, b, what, rel=2e-3):
    a, b = a.double().cpu(), b.double().cpu()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    scale = b.pow(2).mean().sqrt().item() + 1e-6
    err = (a - b).abs().max().item()
    assert err <= rel * (b.abs().max().item() + scale) + 1e-5, (what, err, scale)


@pytest.mark.parametrize("seed", range(24))
def test_tcgen05_matches_cuda_core_kernels(seed):
    rng = random.Random(1000 + seed)
    B, Hq, Hk, M, N, D, causal, dtype = _draw(rng)
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype).cuda()
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype).cuda()
    v = torch.randn(B, Hk, N, D, generator=g).to(dtype).cuda()
    tag = f"B{B} Hq{Hq} Hk{Hk} M{M} N{N} D{D} causal={causal} {dtype}"
    split = rng.randrange(1, N + 1)
    window = None
    if M > 256 and rng.random() < 0.5:
        b0 = rng.randrange(0, M // 128) * 128
        window = (b0, rng.randrange(b0 + 1, M + 1))

    def both(fn, *args, **kw):
        a = fn(q, k, v, *args, backend="auto", q_rows=window, **kw)
        used = F.last_backend()
        b = fn(q, k, v, *args, backend="generic", q_rows=window, **kw)
        return a, b, used

    rows = slice(*(window or (0, M)))
    (oa, sa), (ob, sb), used = both(F.attention_with_scores, causal)
    assert torch.equal(torch.isneginf(sa[:, :, rows]), torch.isneginf(sb[:, :, rows])), tag
    fin = torch.isfinite(sb[:, :, rows])
    assert (sa[:, :, rows][fin] - sb[:, :, rows][fin]).abs().max().item() < 2e-3, tag
    assert (oa[:, :, rows].float() - ob[:, :, rows].float()).abs().max().item() < 2e-2, tag
    for fn, args in [(F.attention_with_row_sum, ()), (F.attention_with_col_sum, ()),
                     (F.attention_with_col_sum_sequential, ()), (F.attention_with_softmax_col_sum, ()),
                     (F.attention_cross_token_qk_sum, (split,)), (F.attention_cross_token_softmax_sum, (split,)),
                     (F.attention_cross_token_softmax_sum_buffered, (split,))]:
        (o1, x1), (o2, x2), used = both(fn, *args, causal)
        if fn is F.attention_with_row_sum:
            x1, x2 = x1[:, :, rows], x2[:, :, rows]
        _close(x1, x2, f"{fn.__name__} [{used}] {tag} split={split} window={window}")
        assert (o1[:, :, rows].float() - o2[:, :, rows].float()).abs().max().item() < 2e-2, (fn.__name__, tag)
    assert F.device_status() == 0
    if M * N <= 400 * 400 and window is None:  # small enough for the CPU oracle
        ro, rs = orc.naive_attention_with_scores(q.cpu(), k.cpu(), v.cpu(), causal, p_seq=N - M)
        ok, viol, okm = orc.check_scores(sa.cpu(), rs)
        assert ok and okm, (tag, viol)
        _, xs = F.attention_cross_token_softmax_sum(q, k, v, split, causal, per_q_head=True)
        ok, viol = orc.check_sum(xs.cpu(), orc.cross_token_softmax_sum(rs, split))
        assert ok, (tag, split, viol)
