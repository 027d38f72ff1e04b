"""Parity of every entry point (through the C ABI) against the CPU oracle on seeded inputs."""
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
    (1, 2, 1, 64, 160, 64),
    (1, 2, 2, 160, 64, 16),
    (1, 7, 1, 256, 256, 128),
    (1, 2, 1, 384, 384, 128),
]


def _inputs(shape, dtype, seed=0):
    B, Hq, Hk, M, N, D = shape
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, M, D, generator=g).to(dtype)
    k = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    v = torch.randn(B, Hk, N, D, generator=g).to(dtype)
    return q, k, v


def _oracle(q, k, v, causal):
    M, N = q.shape[2], k.shape[2]
    return orc.naive_attention_with_scores(q, k, v, causal, p_seq=N - M)


def _check_out(o, ref, slack=None):
    ok, err = orc.check_out(o.cpu(), ref, slack if o.dtype == torch.bfloat16 else None)
    assert ok, f"out max abs err {err}"


def _check_sum(x, ref, what):
    assert x.shape == ref.shape, (what, x.shape, ref.shape)
    ok, viol = orc.check_sum(x.cpu(), ref)
    assert ok, f"{what}: violation {viol}"


@pytest.fixture(params=["generic", "auto"])
def backend(request):
    return request.param


@pytest.fixture(autouse=True)
def _no_wait_gave_up():
    yield
    assert F.device_status() == 0, "a bounded mbarrier wait gave up inside a tcgen05 kernel"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_all_entry_points(shape, causal, dtype, backend):
    B, Hq, Hk, M, N, D = shape
    q, k, v = _inputs(shape, dtype)
    ref_out, ref_scores = _oracle(q, k, v, causal)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    kw = dict(backend=backend)
    slack = orc.bf16_out_slack(ref_scores, v, ref_out) if dtype == torch.bfloat16 else None
    _check_out = lambda o, ref: globals()["_check_out"](o, ref, slack)  # noqa: E731

    o, L, tot, _, _ = F.attention(qd, kd, vd, causal, return_log_normalizer=True, return_total_attention=True, **kw)
    _check_out(o, ref_out)
    Lref = orc.log_normalizer(ref_scores)
    fin = torch.isfinite(Lref)
    assert torch.equal(torch.isneginf(L.cpu()), torch.isneginf(Lref))
    assert (L.cpu()[fin] - Lref[fin]).abs().max() < 2e-3
    _check_sum(tot, orc.softmax_col_sum(ref_scores), "total_attention")

    o, s = F.attention_with_scores(qd, kd, vd, causal, **kw)
    _check_out(o, ref_out)
    assert s.dtype == torch.float32
    ok, viol, ok_mask = orc.check_scores(s.cpu(), ref_scores)
    assert ok_mask, "masked entries differ from the oracle's -inf set"
    assert ok, f"scores violation {viol}"

    o, s0 = F.attention_with_scores(qd, kd, vd, causal, scores_dtype=dtype, masked_value=0.0, **kw)
    _check_out(o, ref_out)
    zref = torch.where(torch.isneginf(ref_scores), torch.zeros_like(ref_scores), ref_scores)
    tol = 4e-3 if dtype == torch.float16 else 3e-2
    assert s0.dtype == dtype and (s0.float().cpu() - zref).abs().max() < tol * max(1.0, zref.abs().max().item())
    assert bool((s0.cpu()[torch.isneginf(ref_scores)] == 0).all())

    o, rs = F.attention_with_row_sum(qd, kd, vd, causal, **kw)
    _check_out(o, ref_out)
    _check_sum(rs, orc.row_sum(ref_scores), "row_sum")

    col_ref = orc.col_sum(ref_scores)
    for fn in (F.attention_with_col_sum, F.attention_with_col_sum_sequential):
        o, cs = fn(qd, kd, vd, causal, **kw)
        _check_out(o, ref_out)
        _check_sum(cs, orc.group_sum(col_ref, Hk), fn.__name__)
        o, cs_h = fn(qd, kd, vd, causal, per_q_head=True, **kw)
        _check_sum(cs_h, col_ref, fn.__name__ + " per head")
    a = F.attention_with_col_sum(qd, kd, vd, causal, **kw)[1]
    b = F.attention_with_col_sum_sequential(qd, kd, vd, causal, **kw)[1]
    assert torch.equal(a, b), "tile order must not change the deterministic column sums"

    o, sc = F.attention_with_softmax_col_sum(qd, kd, vd, causal, **kw)
    _check_out(o, ref_out)
    _check_sum(sc, orc.group_sum(orc.softmax_col_sum(ref_scores), Hk), "softmax_col_sum")

    for split in sorted({1, min(N, M) // 2, max(1, min(N, M) - 1), N}):
        xq_ref = orc.cross_token_qk_sum(ref_scores, split)
        xs_ref = orc.cross_token_softmax_sum(ref_scores, split)
        o, xq = F.attention_cross_token_qk_sum(qd, kd, vd, split, causal, **kw)
        _check_out(o, ref_out)
        _check_sum(xq, orc.group_sum(xq_ref, Hk), f"cross_qk split={split}")
        o, xs = F.attention_cross_token_softmax_sum(qd, kd, vd, split, causal, **kw)
        _check_out(o, ref_out)
        _check_sum(xs, orc.group_sum(xs_ref, Hk), f"cross_softmax split={split}")
        o, xb = F.attention_cross_token_softmax_sum_buffered(qd, kd, vd, split, causal, **kw)
        _check_out(o, ref_out)
        _check_sum(xb, orc.group_sum(xs_ref, Hk), f"cross_softmax_buffered split={split}")
        _, xh = F.attention_cross_token_softmax_sum(qd, kd, vd, split, causal, per_q_head=True, **kw)
        _check_sum(xh, xs_ref, f"cross_softmax per head split={split}")


def test_determinism_and_buffers():
    q, k, v = (t.cuda() for t in _inputs((1, 4, 2, 320, 320, 64), torch.float16, seed=3))
    for fn, args in [(F.attention_with_col_sum, ()), (F.attention_with_softmax_col_sum, ()),
                     (F.attention_cross_token_qk_sum, (200,)), (F.attention_cross_token_softmax_sum, (200,)),
                     (F.attention_cross_token_softmax_sum_buffered, (200,))]:
        a = fn(q, k, v, *args, True)
        b = fn(q, k, v, *args, True)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), fn.__name__
    out = torch.empty_like(q)
    buf = torch.full((1, 2, 200), 7.0, device="cuda")
    o, x = F.attention_cross_token_qk_sum(q, k, v, 200, True, out=out, cross_token_qk_out=buf)
    assert o.data_ptr() == out.data_ptr() and x.data_ptr() == buf.data_ptr()
    ref = F.attention_cross_token_qk_sum(q, k, v, 200, True)[1]
    assert torch.equal(x, ref)
    with pytest.raises(AssertionError):
        F.attention_cross_token_qk_sum(q, k, v, 200, True, cross_token_qk_out=torch.empty(1, 2, 199, device="cuda"))


def test_strided_views_and_query_window():
    g = torch.Generator().manual_seed(5)
    big = torch.randn(1, 256, 3 * 4 * 64, generator=g).half().cuda()   # (B, S, 3*H*D) packed qkv
    qkv = big.view(1, 256, 3, 4, 64).permute(2, 0, 3, 1, 4)            # (3, B, H, S, D), non-contiguous
    q, k, v = qkv[0], qkv[1], qkv[2]
    ref_out, ref_scores = _oracle(q.cpu(), k.cpu(), v.cpu(), True)
    o, s = F.attention_with_scores(q, k, v, True)
    _check_out(o, ref_out)
    assert orc.check_scores(s.cpu(), ref_scores)[0]
    # query window: two halves of the rows give the full column sums after a rank reduce
    full = F.attention_with_col_sum(q, k, v, True)[1]
    a = F.attention_with_col_sum(q, k, v, True, q_rows=(0, 100))[1]
    b = F.attention_with_col_sum(q, k, v, True, q_rows=(100, 256))[1]
    _check_sum(a + b, orc.group_sum(orc.col_sum(ref_scores), 4), "windowed col_sum")
    assert (a + b - full).abs().max() < 1e-3
    xs = F.attention_cross_token_softmax_sum(q, k, v, 128, True, q_rows=(100, 256))[1]
    _check_sum(xs, orc.group_sum(orc.cross_token_softmax_sum(ref_scores, 128), 4), "windowed cross softmax")


def test_kernel_golden_fixtures(golden_dir):
    """The reference's own Triton-kernel outputs (fixtures) against the CUDA path."""
    import glob
    import os

    import numpy as np
    for path in sorted(glob.glob(os.path.join(golden_dir, "kernels_*.npz"))):
        z = np.load(path)
        q, k, v = (torch.from_numpy(z[n]).cuda() for n in "qkv")
        causal, split = bool(z["causal"]), int(z["split"])
        t = lambda n: torch.from_numpy(z[n]).float()
        o, s = F.attention_with_scores(q, k, v, causal, scores_dtype=q.dtype, masked_value=0.0)
        assert (o.float().cpu() - t("scores_out")).abs().max() < 4e-3
        assert (s.float().cpu() - t("scores")).abs().max() < 8e-3
        for fn, key, args in [
            (F.attention_with_row_sum, "row_sum", ()), (F.attention_with_col_sum, "col_sum", ()),
            (F.attention_with_col_sum_sequential, "col_sum_sequential", ()),
            (F.attention_with_softmax_col_sum, "softmax_col_sum", ()),
            (F.attention_cross_token_qk_sum, "cross_qk", (split,)),
            (F.attention_cross_token_softmax_sum, "cross_softmax", (split,)),
            (F.attention_cross_token_softmax_sum_buffered, "cross_softmax_buffered", (split,)),
        ]:
            o, x = fn(q, k, v, *args, causal)
            ok, viol = orc.check_sum(x.cpu(), t(key))
            assert ok, (os.path.basename(path), key, viol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
@pytest.mark.parametrize("shape", [(1, 2, 1, 256, 256, 128), (1, 2, 2, 200, 328, 64), (2, 6, 2, 640, 640, 128),
                                   (1, 1, 1, 128, 1000, 128), (1, 2, 2, 1000, 1000, 64), (1, 2, 1, 384, 128, 64),
                                   (1, 4, 4, 300, 72, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_tcgen05_family_is_used_and_matches(shape, causal, dtype):
    """Forces the tcgen05 kernels (an unsupported problem would raise) on aligned and ragged shapes."""
    B, Hq, Hk, M, N, D = shape
    q, k, v = _inputs(shape, dtype, seed=11)
    ref_out, ref_scores = _oracle(q, k, v, causal)
    slack = orc.bf16_out_slack(ref_scores, v, ref_out) if dtype == torch.bfloat16 else None
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    kw = dict(backend="tcgen05")
    o, s = F.attention_with_scores(qd, kd, vd, causal, **kw)
    assert F.last_backend() == "tcgen05"
    _check_out(o, ref_out, slack)
    ok, viol, ok_mask = orc.check_scores(s.cpu(), ref_scores)
    assert ok_mask and ok, viol
    if N % 8 == 0:  # the reference kernel's own output format: q.dtype scores, 0 at hidden entries
        o, s0 = F.attention_with_scores(qd, kd, vd, causal, scores_dtype=dtype, masked_value=0.0, **kw)
        assert F.last_backend() == "tcgen05"
        _check_out(o, ref_out, slack)
        zref = torch.where(torch.isneginf(ref_scores), torch.zeros_like(ref_scores), ref_scores)
        tol = 4e-3 if dtype == torch.float16 else 3e-2
        assert s0.dtype == dtype and (s0.float().cpu() - zref).abs().max() < tol * max(1.0, zref.abs().max().item())
        assert bool((s0.cpu()[torch.isneginf(ref_scores)] == 0).all())
        o, s1 = F.attention_with_scores(qd, kd, vd, causal, scores_dtype=dtype, **kw)
        assert torch.equal(torch.isneginf(s1.cpu()), torch.isneginf(ref_scores))
    o, L, _, _, _ = F.attention(qd, kd, vd, causal, return_log_normalizer=True, **kw)
    _check_out(o, ref_out, slack)
    Lref = orc.log_normalizer(ref_scores)
    fin = torch.isfinite(Lref)
    assert torch.equal(torch.isneginf(L.cpu()), ~fin) and (L.cpu()[fin] - Lref[fin]).abs().max() < 2e-3
    o, rs = F.attention_with_row_sum(qd, kd, vd, causal, **kw)
    _check_sum(rs, orc.row_sum(ref_scores), "row_sum")
    col_ref = orc.group_sum(orc.col_sum(ref_scores), Hk)
    o, cs = F.attention_with_col_sum(qd, kd, vd, causal, **kw)
    _check_out(o, ref_out, slack)
    _check_sum(cs, col_ref, "col_sum")
    o, cs2 = F.attention_with_col_sum_sequential(qd, kd, vd, causal, **kw)
    _check_out(o, ref_out, slack)
    assert torch.equal(cs, cs2)
    split = (min(M, N) // 2 // 32) * 32
    o, xq = F.attention_cross_token_qk_sum(qd, kd, vd, split, causal, **kw)
    _check_sum(xq, orc.group_sum(orc.cross_token_qk_sum(ref_scores, split), Hk), "cross_qk")
    # pass 1 on tcgen05 (out, L, score scratch), pass 2 on whichever family fits
    o, xs = F.attention_cross_token_softmax_sum(qd, kd, vd, split, causal)
    _check_out(o, ref_out, slack)
    xs_ref = orc.group_sum(orc.cross_token_softmax_sum(ref_scores, split), Hk)
    _check_sum(xs, xs_ref, "cross_softmax")
    o, xb = F.attention_cross_token_softmax_sum_buffered(qd, kd, vd, split, causal)
    _check_out(o, ref_out, slack)
    _check_sum(xb, xs_ref, "cross_softmax_buffered")
    o, sc = F.attention_with_softmax_col_sum(qd, kd, vd, causal)
    _check_sum(sc, orc.group_sum(orc.softmax_col_sum(ref_scores), Hk), "softmax_col_sum")


def _query_split_worker(rank, world, port, q, k, v, split, want_col, want_x):
    import os

    import torch.distributed as dist

    from flash_attn_with_score_b200 import shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        qd, kd, vd = q.cuda(rank), k.cuda(rank), v.cuda(rank)
        out, col, (b, e) = shard.query_split(F.attention_with_softmax_col_sum, qd, kd, vd, False)
        ok, viol = orc.check_sum(col.cpu(), want_col)
        assert ok, f"rank {rank}: query-split softmax col sum {viol}"
        out2, x, _ = shard.query_split(F.attention_cross_token_qk_sum, qd, kd, vd, split, True)
        ok, viol = orc.check_sum(x.cpu(), want_x)
        assert ok, f"rank {rank}: query-split cross-token qk sum {viol}"
        # every rank holds the same bits
        gathered = [torch.empty_like(col) for _ in range(world)]
        dist.all_gather(gathered, col)
        assert all(torch.equal(g, gathered[0]) for g in gathered)
        assert F.device_status() == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_query_split_two_gpus_nccl():
    """Query rows of every head split over 2 ranks; column-type sums all-gathered and reduced in rank order."""
    import socket

    import torch.multiprocessing as mp
    shape = (1, 4, 2, 512, 512, 128)
    q, k, v = _inputs(shape, torch.float16, seed=31)
    _, sc_full = _oracle(q, k, v, False)
    _, sc_causal = _oracle(q, k, v, True)
    want_col = orc.group_sum(orc.softmax_col_sum(sc_full), 2)
    want_x = orc.group_sum(orc.cross_token_qk_sum(sc_causal, 256), 2)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_query_split_worker, args=(2, port, q, k, v, 256, want_col, want_x), nprocs=2, join=True)


@pytest.mark.parametrize("env", [{"FAWS_SPLIT_KV": "0"}, {"FAWS_SPLIT_KV": "1"}], ids=["two_query_tiles", "split_kv"])
def test_every_cta_mode_of_the_forward_kernel(env):
    """The tcgen05 forward kernel has two CTA shapes (two query tiles per CTA, or one query tile whose
    key tiles are split over the two softmax warpgroups).  The library picks by launch size; here each
    is forced through FAWS_SPLIT_KV in a child process running the tcgen05 parity tests."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, **env)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_ops_gpu.py"), "-q", "-x",
                          "-m", "gpu", "-k", "tcgen05_family or determinism or strided"],
                         env=env, capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
