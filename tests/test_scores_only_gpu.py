"""compute_attention_scores (the reference's score-only operator, attention_scores.py:154-223) against
the CPU oracle's unmasked q.k^T * sm_scale."""
import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [(1, 2, 2, 128, 128, 64), (2, 4, 2, 96, 200, 32), (1, 4, 1, 100, 100, 128), (1, 2, 2, 160, 64, 16),
          (1, 6, 2, 640, 384, 128), (1, 2, 1, 1000, 1000, 64), (1, 3, 1, 300, 72, 128)]


@pytest.mark.parametrize("backend", ["generic", "auto"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_scores_only_matches_oracle(shape, dtype, backend):
    B, Hq, Hk, M, N, D = shape
    g = torch.Generator().manual_seed(21)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    _, ref = orc.naive_attention_with_scores(q, k, k, False)  # unmasked scaled scores
    qd, kd = q.cuda(), k.cuda()
    s32 = F.compute_attention_scores(qd, kd, scores_dtype=torch.float32, backend=backend)
    if backend == "auto" and D in (64, 128) and N % 4 == 0:
        assert F.last_backend() == "tcgen05"
    ok, viol, _ = orc.check_scores(s32.cpu(), ref)
    assert ok, viol
    s16 = F.compute_attention_scores(qd, kd, backend=backend)
    assert s16.dtype == dtype and s16.shape == (B, Hq, M, N)
    rel = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7  # rounding of the stored 16-bit value
    assert ((s16.float().cpu() - ref).abs() <= rel * ref.abs() + 1e-3 * ref.abs() + 1e-4).all()
    # `causal` is accepted and ignored, as in the reference (attention_scores.py:166,171)
    assert torch.equal(F.compute_attention_scores(qd, kd, True, backend=backend), s16)
    assert F.device_status() == 0
