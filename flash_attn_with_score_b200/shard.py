"""Multi-GPU plumbing: one process per GPU over torch.distributed (NCCL on GPUs).

The hot path shards by *units* = (batch, kv head) with its G query heads: a unit's
out rows, score rows, row sums and complete column / cross-token vectors depend on
nothing outside the unit, so units are dealt to ranks in contiguous blocks and
nothing is exchanged (``plan_units``).

Only when one head's query rows are split across ranks (``query_split``) do the
column-type sums need one exchange: every rank computes the sums of its own row
window (``q_rows=``), the fp32 partial vectors are all-gathered into the rank's
own memory and added in rank order by the library's ``faws_reduce_ranks`` kernel,
so the result is bit-identical on every rank and from run to run.  No kernel
reads another GPU's memory.  The reference is single-GPU; this has no counterpart there.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib

ROW_ALIGN = 128  # windows start on a query-tile boundary so the tcgen05 kernels can take them


def plan_units(n_units: int, world: int) -> list[range]:
    """Contiguous, disjoint, covering blocks of unit ids, sizes differing by at most one."""
    assert n_units >= 0 and world >= 1
    base, extra = divmod(n_units, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def unit_to_bh(unit: int, Hk: int) -> tuple[int, int]:
    """unit id -> (batch index, kv head)."""
    return divmod(unit, Hk)


def plan_query_rows(M: int, world: int, align: int = ROW_ALIGN) -> list[tuple[int, int]]:
    """Contiguous row windows [begin, end), one per rank, begins on multiples of `align`."""
    assert M > 0 and world >= 1
    tiles = (M + align - 1) // align
    out = []
    for r in plan_units(tiles, world):
        out.append((min(r.start * align, M), min(r.stop * align, M)))
    return out


def sum_in_rank_order(gathered: torch.Tensor) -> torch.Tensor:
    """(world, ...) -> (...): parts[0] + parts[1] + ... in that order.

    CUDA tensors go through faws_reduce_ranks.  CPU tensors (the gloo tests of the
    exchange plumbing) are added by the same fixed-order loop on the host."""
    world = gathered.shape[0]
    if gathered.is_cuda:
        gathered = gathered.contiguous()
        out = torch.empty(gathered.shape[1:], device=gathered.device, dtype=torch.float32)
        lib = _lib.load()
        stream = C.c_void_p(torch.cuda.current_stream(gathered.device).cuda_stream)
        with torch.cuda.device(gathered.device):
            st = lib.faws_reduce_ranks(C.c_void_p(gathered.data_ptr()), world, out.numel(),
                                       C.c_void_p(out.data_ptr()), stream)
        _lib.check(st, "faws_reduce_ranks")
        return out
    out = torch.zeros_like(gathered[0])
    for r in range(world):
        out = out + gathered[r]
    return out


def all_reduce_rank_order(part: torch.Tensor, group=None) -> torch.Tensor:
    """Deterministic SUM of fp32 partial vectors over the ranks of `group`."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return part
    world = dist.get_world_size(group)
    part = part.contiguous()
    gathered = torch.empty((world,) + tuple(part.shape), device=part.device, dtype=part.dtype)
    # landing buffer = the reduce kernel's input; views keep every backend (nccl, gloo) happy
    dist.all_gather([gathered[r] for r in range(world)], part, group=group)
    return sum_in_rank_order(gathered)


def query_split(op, q, k, v, *args, group=None, overlap=False, **kwargs):
    """Run a column-type operator with this rank's window of query rows and reduce its sums.

    ``op`` is one of the package's column-type operators (col_sum, col_sum_sequential,
    softmax_col_sum, cross_token_*).  Every rank passes the same q, k, v.  Returns
    ``(out, sums, (begin, end))``: only rows [begin, end) of ``out`` are written on this rank;
    ``sums`` is complete and identical on every rank.

    ``overlap=True`` walks the batch one element at a time and starts the all-gather of an element's
    partial sums as soon as they exist, so the exchange of element b runs on NCCL's stream while
    the kernels of element b + 1 compute; the rank-order reduce follows at the end.  Deterministic like
    the whole-batch form; the two forms agree to rounding (a one-element call may use another launch
    shape, hence another fixed summation order inside a rank)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    begin, end = plan_query_rows(q.shape[2], world)[rank]
    if not overlap or world == 1 or q.shape[0] == 1:
        out, part = op(q, k, v, *args, q_rows=(begin, end), **kwargs)
        return out, all_reduce_rank_order(part, group), (begin, end)
    B = q.shape[0]
    out = torch.empty_like(q)
    landing, handles = [], []
    for b in range(B):
        o_b, part = op(q[b:b + 1], k[b:b + 1], v[b:b + 1], *args, q_rows=(begin, end), **kwargs)
        out[b:b + 1, :, begin:end] = o_b[:, :, begin:end]
        part = part.contiguous()
        flat = torch.empty((world * part.shape[0],) + tuple(part.shape[1:]), device=part.device, dtype=part.dtype)
        handles.append(dist.all_gather_into_tensor(flat, part, group=group, async_op=True))
        landing.append(flat.view((world,) + tuple(part.shape)))  # rank-major: the reduce kernel's input
    sums = []
    for h, gathered in zip(handles, landing):
        h.wait()
        sums.append(sum_in_rank_order(gathered))
    return out, torch.cat(sums, 0), (begin, end)
