"""Persistent launches of the tcgen05 forward kernel (one CTA per SM walking a host-made work list)
against plain launches of the same kernel (one CTA per work item) and against a torch fp32 reference.

An item is computed by the same code in both kinds of launch, so the results must be bit-identical;
the plain launches are what every other parity test of the family covers.  FAWS_PERSISTENT=0 in the
environment keeps launches plain; it is read once per process, hence the child processes."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# name, B, Hq, Hk, M, N, D, dtype, causal, q_rows
CASES = [
    ("listed_causal", 2, 16, 4, 2048, 2048, 128, "float16", True, None),       # 256 items, per-CTA lists
    ("listed_window", 1, 24, 8, 2048, 2304, 128, "bfloat16", True, (256, 1920)),  # M != N, row window
    ("listed_full_d64", 2, 16, 16, 1536, 1280, 64, "float16", False, None),    # equal items, 192 of them
    ("rounds_full", 4, 32, 8, 4352, 512, 64, "bfloat16", False, None),         # 2176 items: dealt in rounds
    ("ragged_causal_d64", 2, 12, 4, 1900, 2100, 64, "bfloat16", True, None),   # M, N off the tile grid
    ("m_gt_n_causal", 1, 20, 4, 2304, 1800, 128, "float16", True, None),       # first row blocks see no key at all
    ("gqa_window_full", 1, 40, 8, 1100, 900, 128, "float16", False, (128, 1024)),
]

CHILD = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
import flash_attn_with_score_b200 as F
name, B, Hq, Hk, M, N, D, dtype, causal, q_rows = eval(sys.argv[2])
dtype = getattr(torch, dtype)
g = torch.Generator().manual_seed(7)
q = torch.randn(B, Hq, M, D, generator=g).to(dtype).cuda()
k = torch.randn(B, Hk, N, D, generator=g).to(dtype).cuda()
v = torch.randn(B, Hk, N, D, generator=g).to(dtype).cuda()
res = {}
out, L, *_ = F.attention(q, k, v, causal, return_log_normalizer=True, q_rows=q_rows)
res["attention.out"], res["attention.L"] = out, L
out, rs = F.attention_with_row_sum(q, k, v, causal, q_rows=q_rows)
res["row_sum.out"], res["row_sum"] = out, rs
out, cs = F.attention_with_col_sum(q, k, v, causal, q_rows=q_rows)
res["col_sum.out"], res["col_sum"] = out, cs
out, cs = F.attention_with_col_sum_sequential(q, k, v, causal, q_rows=q_rows)
res["col_seq.out"], res["col_seq"] = out, cs
out, cs = F.attention_with_softmax_col_sum(q, k, v, causal, q_rows=q_rows)
res["softmax_col_sum.out"], res["softmax_col_sum"] = out, cs
if M == N and q_rows is None:
    out, x = F.attention_cross_token_softmax_sum(q, k, v, N // 2, causal)
    res["cross_softmax.out"], res["cross_softmax"] = out, x
    out, x = F.attention_cross_token_qk_sum(q, k, v, N // 2, causal)
    res["cross_qk.out"], res["cross_qk"] = out, x
    out = F.attention(q, k, v, causal, dropout_p=0.25, philox=(1234, 77))
    res["dropout.out"] = out
torch.cuda.synchronize()
assert F.device_status() == 0
lo, hi = q_rows if q_rows is not None else (0, M)
rowwise = lambda n: n.endswith(".out") or n.endswith(".L") or n == "row_sum"  # rows outside the window are not written
torch.save({n: (t[:, :, lo:hi] if rowwise(n) else t).contiguous().cpu() for n, t in res.items()}, sys.argv[3])
"""


def _run(case, persistent, path):
    env = dict(os.environ, FAWS_PERSISTENT="1" if persistent else "0")
    res = subprocess.run([sys.executable, "-c", CHILD, ROOT, repr(case), path], env=env, capture_output=True,
                         text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    return torch.load(path)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_persistent_launch_equals_plain_launch(case, tmp_path):
    plain = _run(case, False, str(tmp_path / "plain.pt"))
    pers = _run(case, True, str(tmp_path / "persistent.pt"))
    assert plain.keys() == pers.keys()
    for name in plain:
        a, b = plain[name], pers[name]
        # bit patterns, so that equal NaNs and -inf compare equal and -0.0 != 0.0 is noticed
        same = torch.equal(a.view(torch.uint8), b.view(torch.uint8)) if a.dtype != torch.float32 else \
            torch.equal(a.view(torch.int32), b.view(torch.int32))
        assert same, f"{name}: persistent and plain launches differ"

    # and the persistent result itself against torch fp32 on one head of the last batch
    name, B, Hq, Hk, M, N, D, dtype, causal, q_rows = case
    dt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(7)
    q = torch.randn(B, Hq, M, D, generator=g).to(dt)
    k = torch.randn(B, Hk, N, D, generator=g).to(dt)
    v = torch.randn(B, Hk, N, D, generator=g).to(dt)
    h = Hq - 1
    hk = h // (Hq // Hk)
    s = (q[-1, h].float() @ k[-1, hk].float().T) * D ** -0.5
    if causal:
        i = torch.arange(M)[:, None]
        j = torch.arange(N)[None, :]
        s = s.masked_fill(j > i + (N - M), float("-inf"))
    seen = ~torch.isinf(s).all(-1)  # rows that see at least one key; the others are zero rows in the output
    ref = torch.softmax(s.masked_fill(~seen[:, None], 0.0), -1) @ v[-1, hk].float()
    ref[~seen] = 0.0
    lo, hi = q_rows if q_rows is not None else (0, M)
    got = pers["attention.out"][-1, h].float()  # (the saved tensors hold the window's rows only)
    tol = 2e-3 if dt == torch.float16 else 1.6e-2  # half a unit in the last place of the 16-bit output at |out| <= 4, doubled
    assert (got - ref[lo:hi]).abs().max().item() <= tol
    assert got[~seen[lo:hi]].abs().max().item() == 0.0 if (~seen[lo:hi]).any() else True
    want_rs = torch.where(torch.isinf(s), torch.zeros_like(s), s).sum(-1)
    rs = pers["row_sum"][-1, h]
    assert torch.allclose(rs, want_rs[lo:hi], rtol=2e-3, atol=2e-2)


def test_persistent_launch_replays_from_a_cuda_graph():
    """The work lists travel as a kernel parameter, so a captured persistent launch replays with them."""
    import flash_attn_with_score_b200 as F
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    q = torch.randn(2, 16, 2048, 128, device=dev, dtype=torch.float16, generator=g)  # 256 work items
    k = torch.randn(2, 4, 2048, 128, device=dev, dtype=torch.float16, generator=g)
    v = torch.randn(2, 4, 2048, 128, device=dev, dtype=torch.float16, generator=g)
    want_out, want_rs = F.attention_with_row_sum(q, k, v, True)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        got_out, got_rs = F.attention_with_row_sum(q, k, v, True)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        got_out.zero_()
        got_rs.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(got_out, want_out)
        assert torch.equal(got_rs, want_rs)
    assert F.device_status() == 0
