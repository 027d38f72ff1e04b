"""Host-side multi-rank logic on CPU: unit / row planners and the rank-order reduce over gloo (world 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_attn_with_score_b200 import shard


def test_plan_units_partitions():
    for n in (0, 1, 4, 16, 32, 33):
        for w in (1, 2, 3, 4, 8):
            blocks = shard.plan_units(n, w)
            assert len(blocks) == w
            flat = [u for b in blocks for u in b]
            assert flat == list(range(n))
            sizes = [len(b) for b in blocks]
            assert max(sizes) - min(sizes) <= 1
    assert shard.unit_to_bh(9, 8) == (1, 1)
    # cfg4: 16 units over 8 ranks -> 2 each; cfg5: 32 units -> 4 each
    assert [len(b) for b in shard.plan_units(16, 8)] == [2] * 8
    assert [len(b) for b in shard.plan_units(32, 8)] == [4] * 8


def test_plan_query_rows_cover_and_align():
    for M in (1, 100, 128, 1000, 4096, 16384):
        for w in (1, 2, 4, 8):
            wins = shard.plan_query_rows(M, w)
            assert wins[0][0] == 0 and wins[-1][1] == M
            for (b0, e0), (b1, e1) in zip(wins, wins[1:]):
                assert e0 == b1
            assert all(b % shard.ROW_ALIGN == 0 or b == M for b, _ in wins)
    assert shard.plan_query_rows(16384, 8)[3] == (6144, 8192)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fail_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        part = torch.randn(2, 3, 257, generator=g)
        total = shard.all_reduce_rank_order(part)
        # every rank rebuilds all partials and adds them in rank order: must match bit for bit
        want = torch.zeros_like(part)
        for r in range(world):
            want = want + torch.randn(2, 3, 257, generator=torch.Generator().manual_seed(100 + r))
        assert torch.equal(total, want)
        # windows of the ranks tile the rows; emulate "column sums of my window" and reduce them
        M, N = 1000, 64
        scores = torch.randn(M, N, generator=torch.Generator().manual_seed(7))
        b, e = shard.plan_query_rows(M, world)[rank]
        col = shard.all_reduce_rank_order(scores[b:e].sum(0))
        assert torch.allclose(col, scores.sum(0), atol=1e-4)
        # query_split over a stand-in operator (column sums of the window's rows), both exchange forms
        q = torch.randn(3, 2, 512, 8, generator=torch.Generator().manual_seed(11))
        kk = torch.randn(3, 1, 40, 8, generator=torch.Generator().manual_seed(12))

        def fake_op(q_, k_, v_, q_rows=None):
            lo, hi = q_rows
            sc = torch.einsum("bhmd,bknd->bhmn", q_, k_)
            return q_.clone(), sc[:, :, lo:hi].sum(2)

        want_sums = torch.einsum("bhmd,bknd->bhmn", q, kk)
        lo0, hi0 = shard.plan_query_rows(512, world)[0]
        want_sums = want_sums[:, :, lo0:hi0].sum(2) + want_sums[:, :, hi0:].sum(2)  # rank order, world 2
        for overlap in (False, True):
            out, sums, (lo, hi) = shard.query_split(fake_op, q, kk, kk, overlap=overlap)
            assert (lo, hi) == shard.plan_query_rows(512, world)[rank]
            assert torch.equal(sums, want_sums), overlap
            assert torch.equal(out[:, :, lo:hi], q[:, :, lo:hi])
        if fail_rank == rank:
            raise RuntimeError("injected host-side failure before the next exchange")
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_rank_order_reduce_gloo_world2():
    mp.spawn(_worker, args=(2, _free_port(), -1), nprocs=2, join=True)


def test_failed_rank_surfaces_as_error():
    """A rank that raises between steps ends the job with an error instead of a silent hang."""
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, _free_port(), 1), nprocs=2, join=True)


def test_sum_in_rank_order_is_left_to_right():
    # fp32: (1 + 1e8) - 1e8 = 0 left to right, but 1 + (1e8 - 1e8) = 1 right to left
    x = torch.tensor([[1.0], [1e8], [-1e8]], dtype=torch.float32)
    assert shard.sum_in_rank_order(x).item() == 0.0
