"""One process driving two GPUs: kernel attributes, the compute-capability check and the status
word are per device, so the first tcgen05 launch on a second device must work like the first."""
import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_same_process_two_devices():
    g = torch.Generator().manual_seed(17)
    q = torch.randn(1, 4, 384, 128, generator=g).half()
    k = torch.randn(1, 2, 384, 128, generator=g).half()
    v = torch.randn(1, 2, 384, 128, generator=g).half()
    ref_out, ref_scores = orc.naive_attention_with_scores(q, k, v, True)
    want_col = orc.group_sum(orc.softmax_col_sum(ref_scores), 2)
    for dev in (0, 1, 0):
        d = torch.device("cuda", dev)
        qd, kd, vd = q.to(d), k.to(d), v.to(d)  # every operand lives on the device that computes
        out, scores = F.attention_with_scores(qd, kd, vd, True, backend="tcgen05")
        assert out.device == d and F.last_backend() == "tcgen05"
        ok, err = orc.check_out(out.cpu(), ref_out)
        assert ok, (dev, err)
        ok, viol, ok_mask = orc.check_scores(scores.cpu(), ref_scores)
        assert ok and ok_mask, (dev, viol)
        out, col = F.attention_with_softmax_col_sum(qd, kd, vd, True, backend="tcgen05")
        ok, viol = orc.check_sum(col.cpu(), want_col)
        assert ok, (dev, viol)
        with torch.cuda.device(d):
            assert F.device_status() == 0
