"""dropout_p > 0 on the GPU: the mask, where it applies and what is rescaled, against the reference
kernels' stored outputs (tests/golden/dropout_*.npz) and against the CPU oracle's Philox restatement."""
import glob
import os

import numpy as np
import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = sorted(f for f in glob.glob(os.path.join(GOLDEN, "dropout_*.npz")) if "philox_stream" not in f)

OPS = [
    ("attention", lambda q, k, v, c, s, **kw: (F.attention(q, k, v, c, **kw), None), True),
    ("scores", lambda q, k, v, c, s, **kw: F.attention_with_scores(q, k, v, c, **kw), True),
    ("row_sum", lambda q, k, v, c, s, **kw: F.attention_with_row_sum(q, k, v, c, **kw), False),
    ("col_sum", lambda q, k, v, c, s, **kw: F.attention_with_col_sum(q, k, v, c, **kw), False),
    ("col_sum_sequential", lambda q, k, v, c, s, **kw: F.attention_with_col_sum_sequential(q, k, v, c, **kw), False),
    ("softmax_col_sum", lambda q, k, v, c, s, **kw: F.attention_with_softmax_col_sum(q, k, v, c, **kw), False),
    ("cross_qk", lambda q, k, v, c, s, **kw: F.attention_cross_token_qk_sum(q, k, v, s, c, **kw), False),
    ("cross_softmax", lambda q, k, v, c, s, **kw: F.attention_cross_token_softmax_sum(q, k, v, s, c, **kw), False),
    ("cross_softmax_buffered",
     lambda q, k, v, c, s, **kw: F.attention_cross_token_softmax_sum_buffered(q, k, v, s, c, **kw), None),
]


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p) for p in FIXTURES])
def test_matches_reference_kernels_under_dropout(path):
    z = np.load(path)
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in "qkv")
    causal, split, p_drop = bool(z["causal"]), int(z["split"]), float(z["dropout_p"])
    philox = tuple(int(x) for x in z["philox"])
    for key, fn, _ in OPS:
        out, aux = fn(q, k, v, causal, split, dropout_p=p_drop, philox=philox)
        ref = torch.from_numpy(z[key + "_out"]).float()
        good = ~torch.isnan(ref).any(-1)  # NaN rows of the reference's reverse-order kernel
        assert key == "col_sum" or bool(good.all())
        err = (out.float().cpu() - ref)[good].abs().max().item()
        assert err < 4e-3, (key, err)
        if aux is not None:
            want = torch.from_numpy(z[key]).float()
            if key == "scores":
                got = torch.where(torch.isneginf(aux), torch.zeros_like(aux), aux).cpu()
                assert (got - want).abs().max() < 8e-3
            else:
                ok, viol = orc.check_sum(aux.cpu(), want)
                assert ok, (key, viol)


@pytest.mark.parametrize("backend", ["generic", "auto"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("shape,causal,p_drop,philox", [
    ((1, 4, 2, 200, 200, 64), True, 0.2, (99, 0)),
    ((2, 2, 2, 130, 77, 128), False, 0.5, ((3 << 32) | 5, 12344)),
    ((1, 3, 1, 64, 300, 32), True, 0.05, (2 ** 63 - 1, 2 ** 31 - 5000)),  # linear index passes 2**31
    ((1, 2, 1, 520, 392, 128), True, 0.25, (17, 2 ** 31 - 100000)),  # several tiles per row, M > N
], ids=["causal_gqa", "full_ragged_d128", "offset_wraps_int32", "multi_tile_d128"])
def test_matches_oracle_under_dropout(shape, causal, p_drop, philox, dtype, backend):
    B, Hq, Hk, M, N, D = shape
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    v = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    _, scores = orc.naive_attention_with_scores(q, k, v, causal, p_seq=N - M)
    keep = orc.dropout_keep_mask(philox[0], philox[1], B, Hq, M, N, p_drop)
    scaled = orc.dropout_out(scores, v, keep, p_drop)
    slack = orc.bf16_out_slack(scores, v, scaled) if dtype == torch.bfloat16 else None
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    split = max(1, N // 3)
    for key, fn, rescale in OPS:
        out, aux = fn(qd, kd, vd, causal, split, dropout_p=p_drop, philox=philox, backend=backend)
        if backend == "auto" and D >= 64 and rescale is not None and (key != "scores" or N % 4 == 0):
            assert F.last_backend() == "tcgen05", key  # the mask is drawn inside the tcgen05 kernel
        if rescale is None:
            ref = orc.naive_attention_with_scores(q, k, v, causal, p_seq=N - M)[0]
        else:
            ref = scaled if rescale else scaled * (1.0 - p_drop)
        ok, err = orc.check_out(out.float().cpu(), ref, slack)
        assert ok, (key, err)
        if key == "softmax_col_sum":
            ok, viol = orc.check_sum(aux.cpu(), orc.group_sum(orc.dropout_softmax_col_sum(scores, keep), Hk))
            assert ok, viol
        if key == "cross_softmax":
            ok, viol = orc.check_sum(aux.cpu(), orc.group_sum(orc.cross_token_softmax_sum(scores, split), Hk))
            assert ok, viol
        if key == "scores":
            ok, viol, okm = orc.check_scores(aux.cpu(), scores)
            assert ok and okm, viol


def test_generator_bookkeeping_and_replay():
    """Without `philox=` the pair comes from torch's CUDA generator and the offset advances by
    B*H*M*N rounded up to 4 (dropout.py:5-15); replaying the returned pair reproduces the bits."""
    torch.manual_seed(1234)
    B, H, M, N, D = 1, 2, 96, 80, 64
    q = torch.randn(B, H, M, D, device="cuda", dtype=torch.float16)
    k = torch.randn(B, H, N, D, device="cuda", dtype=torch.float16)
    v = torch.randn(B, H, N, D, device="cuda", dtype=torch.float16)
    o1, _, _, seed1, off1 = F.attention(q, k, v, True, dropout_p=0.3, return_seed_offset=True)
    o2, _, _, seed2, off2 = F.attention(q, k, v, True, dropout_p=0.3, return_seed_offset=True)
    assert seed1 == seed2 == 1234
    assert off2 - off1 == (B * H * M * N + 3) // 4 * 4
    assert not torch.equal(o1, o2)
    assert torch.equal(F.attention(q, k, v, True, dropout_p=0.3, philox=(seed1, off1)), o1)
    assert torch.equal(F.attention(q, k, v, True, dropout_p=0.3, philox=(seed2, off2)), o2)
    plain = F.attention(q, k, v, True, return_seed_offset=True)
    assert plain[3] is None and plain[4] is None


def test_dropout_rejections():
    q = torch.randn(1, 2, 128, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError):  # no dropout variant of the 16-bit-score hook on tcgen05
        F.attention_with_scores(q, q, q, True, dropout_p=0.1, philox=(1, 0), backend="tcgen05",
                                scores_dtype=torch.float16)
    with pytest.raises(NotImplementedError):
        F.attention(q, q, q, True, dropout_p=0.1, philox=(1, 2 ** 31))
