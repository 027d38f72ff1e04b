"""Host-side mirror of the reference's operator interface (its __init__.py:29-39).

Same names, positional order, defaults and assertion behaviour as the
reference wrappers; the device work is done by libfaws.so through the C ABI of
include/faws.h.  PyTorch is used for device memory and the current stream only.

Deliberate differences, all keyword-only:
  * ``attention_with_scores(..., scores_dtype=torch.float32, masked_value=-inf)``:
    the default follows the reference *oracle* (fp32 values, -inf at hidden
    entries, reference_implementations.py:31-40); ``scores_dtype=q.dtype,
    masked_value=0.0`` reproduces the reference kernel (attention_with_scores.py:141-152,284).
  * column-type sums accept ``per_q_head=True`` to return (B,Hq,.) instead of the
    reference kernels' group-summed (B,Hk,.) (attention_with_col_sum.py:72,370).
  * ``q_rows=(begin, end)`` restricts the call to a window of query rows (the
    query-split multi-GPU variant); ``backend`` forces a kernel family.
  * ``dropout_p > 0`` draws the same mask as the reference kernels (Philox stream of
    ``tl.rand(seed, offset + linear index, n_rounds=6)``, flash.py:376-380,463-466) with seed and
    offset taken from, and advanced on, torch's CUDA generator exactly as dropout.py:5-15 does;
    ``philox=(seed, offset)`` pins them instead.
"""
from __future__ import annotations

import ctypes as C
import math
import struct

import torch

from . import _lib

_DTYPES = {torch.float16: _lib.FP16, torch.bfloat16: _lib.BF16}


def maybe_contiguous(x):
    # only the last dimension has to be contiguous (flash.py:23-26)
    return x.contiguous() if x.stride(-1) != 1 else x


def _tensor(t):
    return _lib.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def philox_cuda_seed_offset(increment, device=None):
    """(seed, offset) of the device's default CUDA generator; advances the offset by ``increment``
    rounded up to a multiple of 4 (the bookkeeping of dropout.py:5-15)."""
    device = torch.cuda.current_device() if device is None else torch.device(device).index
    gen = torch.cuda.default_generators[device]
    state = gen.get_state()
    words = state.view(torch.int64)
    seed, offset = int(words[0]), int(words[1])
    words[1] += (increment + 3) // 4 * 4
    gen.set_state(state)
    return seed, offset


class _Call:
    """Validated arguments + the faws_problem struct shared by every operator."""

    def __init__(self, q, k, v, causal, sm_scale, dropout_p, out=None, need_L=False, L=None,
                 q_rows=None, backend=None, msgs=None, philox=None, rescale=False):
        m = msgs or {}
        Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
        assert Dq == Dk == Dv, m.get("D", "feature size of q, k, v should be equal")
        assert Dk in {16, 32, 64, 128}, m.get("Dset", f"Unsupported head_dim: {Dk}")
        B, H, M, D = q.shape
        N = k.shape[2]
        Hk, Hv = k.shape[1], v.shape[1]
        assert Hk == Hv, m.get("Hkv", "num of heads in k and v should be equal")
        assert H % Hk == 0, m.get("G", "number of heads in q must be a multiple of that in k & v")
        assert k.shape[0] == B and v.shape[0] == B and v.shape[2] == N
        if not q.is_cuda:
            raise RuntimeError("flash_attn_with_score_b200 runs on CUDA tensors only (no CPU fallback)")
        if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
            raise TypeError(f"q, k, v must share dtype float16 or bfloat16, got {q.dtype}, {k.dtype}, {v.dtype}")
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        self.q, self.k, self.v = maybe_contiguous(q), maybe_contiguous(k), maybe_contiguous(v)
        self.B, self.H, self.Hk, self.M, self.N, self.D = B, H, Hk, M, N, D
        self.dev = q.device
        self.lib = _lib.load()
        if out is None:
            out = torch.empty_like(self.q)
        self.out = out
        if L is None and need_L:
            L = torch.empty((B, H, M), device=q.device, dtype=torch.float32)
        self.L = L
        m_begin, m_end = (0, M) if q_rows is None else q_rows
        assert 0 <= m_begin <= m_end <= M, f"q_rows must lie within [0, {M}]"
        if backend not in _lib.BACKENDS:
            raise ValueError(f"backend must be one of {sorted(k for k in _lib.BACKENDS if k)}")
        p = _lib.Problem()
        p.B, p.Hq, p.Hk, p.M, p.N, p.D = B, H, Hk, M, N, D
        p.dtype = _DTYPES[q.dtype]
        p.causal = 1 if causal else 0
        p.sm_scale = float(sm_scale)
        p.m_begin, p.m_end = m_begin, m_end
        p.q, p.k, p.v, p.out = _tensor(self.q), _tensor(self.k), _tensor(self.v), _tensor(self.out)
        p.log_normalizer = L.data_ptr() if L is not None else None
        p.backend = _lib.BACKENDS[backend]
        self.seed = self.offset = None
        if dropout_p and dropout_p > 0.0:
            assert dropout_p < 1.0, "dropout_p must be < 1"
            seed, offset = philox if philox is not None else philox_cuda_seed_offset(B * H * M * N, q.device)
            if not 0 <= offset < 2 ** 31:
                raise NotImplementedError("Philox offsets >= 2**31 select triton's 64-bit generator, "
                                          "which is not implemented")
            p.dropout_p = float(dropout_p)
            # attention and attention_with_scores rescale by 1/(1-p) (flash.py:488-491,
            # attention_with_scores.py:201-203); the reference's other operators only mask
            p.dropout_scale = 1.0 / (1.0 - float(dropout_p)) if rescale else 1.0
            p.philox_seed = seed & (2 ** 64 - 1)
            p.philox_offset = offset
            self.seed, self.offset = seed, offset
        self.p = p

    def workspace(self, op, split=0):
        n = self.lib.faws_workspace_bytes(op, C.byref(self.p), split)
        if n == 0:
            return None, 0
        ws = torch.empty(n, device=self.dev, dtype=torch.uint8)
        return ws, n

    def run(self, fn_name, *mid):
        with torch.cuda.device(self.dev):
            st = getattr(self.lib, fn_name)(C.byref(self.p), *mid, _stream(self.q))
        _lib.check(st, fn_name)


def _f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


def _attention_forward(q, k, v, causal, sm_scale, dropout_p, need_L, want_total, q_rows, backend, philox,
                       kv_splits=None):
    c = _Call(q, k, v, causal, sm_scale, dropout_p, need_L=need_L, q_rows=q_rows, backend=backend,
              philox=philox, rescale=True)
    # few query rows (decoding): split the keys over more CTAs, as flash.py:68-70,97-134 does
    n_splits = int(c.lib.faws_split_kv_plan(C.byref(c.p))) if kv_splits is None else int(kv_splits)
    if n_splits > 1:
        ws, n = c.workspace(_lib.OP_ATTENTION_SPLIT_KV, n_splits)
        c.run("faws_attention_split_kv", n_splits, C.c_void_p(ws.data_ptr()), n)
    else:
        c.run("faws_attention")
    tot = None
    if want_total:
        tot = torch.empty((c.B, c.H, c.N), device=c.dev, dtype=torch.float32)
        c.run("faws_total_attention", C.c_void_p(tot.data_ptr()))
    return c, tot


class _AttentionFunction(torch.autograd.Function):
    """attention() under autograd: the reference's FlashAttention (flash.py:32-261).  Saves
    (q, k, v, out, log-normaliser) like flash.py:152; backward runs faws_attention_backward."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, dropout_p, want_total, backend, philox, kv_splits):
        c, tot = _attention_forward(q, k, v, causal, sm_scale, dropout_p, True, want_total, None, backend, philox,
                                    kv_splits)
        ctx.save_for_backward(c.q, c.k, c.v, c.out, c.L)
        ctx.causal, ctx.sm_scale, ctx.dropout_p, ctx.backend = causal, float(c.p.sm_scale), dropout_p, backend
        ctx.philox = (c.seed, c.offset) if c.seed is not None else None
        ctx.mark_non_differentiable(*[t for t in (c.L, tot) if t is not None])
        return c.out, c.L, tot, c.seed, c.offset

    @staticmethod
    def backward(ctx, do, *ignored):
        q, k, v, o, L = ctx.saved_tensors
        do = maybe_contiguous(do)
        c = _Call(q, k, v, ctx.causal, ctx.sm_scale, ctx.dropout_p, out=o, L=L, backend=ctx.backend,
                  philox=ctx.philox, rescale=True)
        dq, dk, dv = torch.empty_like(c.q), torch.empty_like(c.k), torch.empty_like(c.v)
        g = _lib.Grads(_tensor(do), _tensor(dq), _tensor(dk), _tensor(dv))
        ws, n = c.workspace(_lib.OP_ATTENTION_BACKWARD)
        c.run("faws_attention_backward", C.byref(g), C.c_void_p(ws.data_ptr()), n)
        return dq, dk, dv, None, None, None, None, None, None, None


def attention(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
              return_log_normalizer=False, return_total_attention=False, return_seed_offset=False,
              *, q_rows=None, backend=None, philox=None, kv_splits=None):
    """FlashAttention; the reference's ``attention`` (flash.py:264-295), differentiable in q, k, v
    like the reference's autograd function (flash.py:32-261).  Problems with few query rows are run
    split-KV like there (flash.py:68-70); ``kv_splits`` pins the number of key ranges (1 = never).

    Returns ``out`` or, if any ``return_*`` flag is set, the reference's 5-tuple
    ``(out, log_normalizer|None, total_attention|None, seed|None, offset|None)``
    (flash.py:160-169)."""
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if needs_grad:
        if q_rows is not None:
            raise ValueError("q_rows (a window of query rows) is not differentiable; pass the whole problem")
        out, L, tot, seed, offset = _AttentionFunction.apply(q, k, v, causal, sm_scale, dropout_p,
                                                             return_total_attention, backend, philox, kv_splits)
    else:
        need_L = return_log_normalizer or return_total_attention
        c, tot = _attention_forward(q, k, v, causal, sm_scale, dropout_p, need_L, return_total_attention,
                                    q_rows, backend, philox, kv_splits)
        out, L, seed, offset = c.out, c.L, c.seed, c.offset
    if return_log_normalizer or return_total_attention or return_seed_offset:
        return (out, L if return_log_normalizer else None, tot,
                seed if return_seed_offset else None, offset if return_seed_offset else None)
    return out


def attention_with_scores(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
                          *, scores_dtype=torch.float32, masked_value=float("-inf"),
                          q_rows=None, backend=None, out=None, scores=None, philox=None):
    """``(out, scores)`` with q.k^T computed once (attention_with_scores.py:214-333).

    scores: (B,Hq,M,N), ``scores_dtype`` (fp32 or q.dtype), hidden entries = ``masked_value``."""
    c = _Call(q, k, v, causal, sm_scale, dropout_p, out=out, q_rows=q_rows, backend=backend,
              philox=philox, rescale=True)
    if scores_dtype not in (torch.float32, q.dtype):
        raise TypeError("scores_dtype must be torch.float32 or q.dtype")
    if scores is None:
        scores = torch.empty((c.B, c.H, c.M, c.N), device=c.dev, dtype=scores_dtype)
    else:
        assert scores.shape == (c.B, c.H, c.M, c.N) and scores.dtype == scores_dtype and scores.is_contiguous()
    sd = _lib.SCORES_F32 if scores_dtype == torch.float32 else _lib.SCORES_INPUT
    c.run("faws_attention_with_scores", C.c_void_p(scores.data_ptr()), sd, _f32_bits(masked_value))
    return c.out, scores


def compute_attention_scores(q, k, causal=False, sm_scale=None, *, scores_dtype=None, backend=None):
    """``q @ k^T * sm_scale`` as a (B,Hq,M,N) tensor in q.dtype, no softmax, no V: the reference's
    ``compute_attention_scores`` (attention_scores.py:154-223).  ``causal`` is accepted and ignored,
    exactly as there (:166,:171): no mask is applied.  ``scores_dtype=torch.float32`` keeps fp32."""
    Dq, Dk = q.shape[-1], k.shape[-1]
    assert Dq == Dk, "Q and K must have the same head_dim"
    assert Dk in {16, 32, 64, 128}, f"head_dim must be one of 16, 32, 64, 128, got {Dk}"
    assert q.shape[1] % k.shape[1] == 0, "num_heads_q must be a multiple of num_heads_k (GQA support)"
    c = _Call(q, k, k, False, sm_scale, 0.0, out=q, backend=backend)
    scores_dtype = q.dtype if scores_dtype is None else scores_dtype
    if scores_dtype not in (torch.float32, q.dtype):
        raise TypeError("scores_dtype must be torch.float32 or q.dtype")
    scores = torch.empty((c.B, c.H, c.M, c.N), device=c.dev, dtype=scores_dtype)
    sd = _lib.SCORES_F32 if scores_dtype == torch.float32 else _lib.SCORES_INPUT
    c.run("faws_compute_attention_scores", C.c_void_p(scores.data_ptr()), sd)
    return scores


def attention_with_row_sum(q, k, v, causal=False, sm_scale=None, dropout_p=0.0, *, q_rows=None, backend=None,
                           philox=None):
    """``(out, row_sum)``; row_sum (B,Hq,M) fp32 = sum over visible keys of the scaled
    score (attention_with_row_sum.py:204-326)."""
    c = _Call(q, k, v, causal, sm_scale, dropout_p, q_rows=q_rows, backend=backend, philox=philox)
    rs = torch.empty((c.B, c.H, c.M), device=c.dev, dtype=torch.float32)
    c.run("faws_attention_with_row_sum", C.c_void_p(rs.data_ptr()))
    return c.out, rs


def _col_like(fn_name, op, q, k, v, causal, sm_scale, dropout_p, per_q_head, q_rows, backend,
              split=None, out=None, sum_out=None, msgs=None, philox=None):
    c = _Call(q, k, v, causal, sm_scale, dropout_p, out=out, q_rows=q_rows, backend=backend, msgs=msgs,
              philox=philox)
    length = c.N if split is None else split
    heads = c.H if per_q_head else c.Hk
    if sum_out is None:
        sum_out = torch.empty((c.B, heads, length), device=c.dev, dtype=torch.float32)
    ws, n = c.workspace(op, 0 if split is None else split)
    args = [C.c_void_p(sum_out.data_ptr()), 1 if per_q_head else 0,
            C.c_void_p(ws.data_ptr() if ws is not None else None), n]
    if split is not None:
        args = [split] + args
    c.run(fn_name, *args)
    return c.out, sum_out


def attention_with_col_sum(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
                           *, per_q_head=False, q_rows=None, backend=None, philox=None):
    """``(out, col_sum)``; col_sum (B,Hk,N) fp32 = sum over visible queries (and the G query
    heads of the kv head) of the scaled score; reverse-order key tiles when causal
    (attention_with_col_sum.py:297-419).  Deterministic."""
    return _col_like("faws_attention_with_col_sum", _lib.OP_COL_SUM, q, k, v, causal, sm_scale,
                     dropout_p, per_q_head, q_rows, backend, philox=philox)


def attention_with_col_sum_sequential(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
                                      *, per_q_head=False, q_rows=None, backend=None, philox=None):
    """Same sums as ``attention_with_col_sum`` with round-robin key-tile order
    (attention_with_col_sum_sequential.py:214-341)."""
    return _col_like("faws_attention_with_col_sum_sequential", _lib.OP_COL_SUM_SEQUENTIAL, q, k, v,
                     causal, sm_scale, dropout_p, per_q_head, q_rows, backend, philox=philox)


def attention_with_softmax_col_sum(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
                                   *, per_q_head=False, q_rows=None, backend=None, philox=None):
    """``(out, col_sum)``; column sums of the softmax weights
    (attention_with_col_softmax_sum.py:274-401)."""
    return _col_like("faws_attention_with_softmax_col_sum", _lib.OP_SOFTMAX_COL_SUM, q, k, v, causal,
                     sm_scale, dropout_p, per_q_head, q_rows, backend, philox=philox)


_XMSG = {"D": "Feature dimensions of q, k, v must be equal", "Hkv": "Number of heads in k and v must be equal",
         "G": "Number of heads in q must be a multiple of that in k"}


def attention_cross_token_qk_sum(q, k, v, split, causal=False, sm_scale=None, dropout_p=0.0,
                                 *, out=None, cross_token_qk_out=None, reuse_buffers=False,
                                 per_q_head=False, q_rows=None, backend=None, philox=None):
    """``(out, cross_token_qk)``; cross_token_qk (B,Hk,split) fp32 = scaled-score sum from
    queries >= split into keys < split (attention_cross_token_qk_sum.py:255-408).
    ``out`` / ``cross_token_qk_out`` are optional caller-owned buffers (:341-357)."""
    N = k.shape[2]
    assert 0 < split <= N, f"Split position must be within valid range (0, {N}]"
    B, H = q.shape[0], q.shape[1]
    Hk = k.shape[1]
    if out is not None:
        assert out.shape == q.shape, f"out.shape must equal q.shape, current out={out.shape}, q={q.shape}"
        assert out.device == q.device, "out.device must match q.device"
        assert out.dtype == q.dtype, "out.dtype must match q.dtype"
        assert out.stride(-1) == 1
    if cross_token_qk_out is not None:
        want = (B, H if per_q_head else Hk, split)
        assert tuple(cross_token_qk_out.shape) == want, (
            f"cross_token_qk_out.shape must be {want}, current is {tuple(cross_token_qk_out.shape)}")
        assert cross_token_qk_out.device == q.device, "cross_token_qk_out.device must match q.device"
        assert cross_token_qk_out.dtype == torch.float32, "cross_token_qk_out.dtype must be torch.float32"
        assert cross_token_qk_out.is_contiguous()
    return _col_like("faws_attention_cross_token_qk_sum", _lib.OP_CROSS_QK_SUM, q, k, v, causal, sm_scale,
                     dropout_p, per_q_head, q_rows, backend, split=split, out=out,
                     sum_out=cross_token_qk_out, msgs=_XMSG, philox=philox)


def attention_cross_token_softmax_sum(q, k, v, split, causal=False, sm_scale=None, dropout_p=0.0,
                                      *, per_q_head=False, q_rows=None, backend=None, philox=None):
    """``(out, sums)``; sums (B,Hk,split) fp32 = softmax-weight sum from queries >= split into
    keys < split; second q.k^T over the cross region (attention_cross_token_softmax_sum.py:735-863)."""
    N = k.shape[2]
    assert 0 < split <= N, f"Split position must be in valid range (0, {N}]"
    return _col_like("faws_attention_cross_token_softmax_sum", _lib.OP_CROSS_SOFTMAX_SUM, q, k, v, causal,
                     sm_scale, dropout_p, per_q_head, q_rows, backend, split=split, philox=philox)


def attention_cross_token_softmax_sum_buffered(q, k, v, split, causal=False, sm_scale=None, dropout_p=0.0,
                                               *, per_q_head=False, q_rows=None, backend=None, philox=None):
    """Same sums as ``attention_cross_token_softmax_sum``; the first pass stores the cross
    region's scores and the second reads them back (attention_cross_token_softmax_sum.py:639-732).
    ``dropout_p`` is accepted and ignored, as in the reference (:646,713-730)."""
    N = k.shape[2]
    assert 0 < split <= N, f"Split position must be in valid range (0, {N}]"
    return _col_like("faws_attention_cross_token_softmax_sum_buffered", _lib.OP_CROSS_SOFTMAX_SUM_BUFFERED,
                     q, k, v, causal, sm_scale, 0.0, per_q_head, q_rows, backend, split=split)


def total_attention(q, k, log_normalizer, causal=False, sm_scale=None, *, backend=None):
    """Per-query-head softmax column sums (B,Hq,N) from a saved log-normaliser (total.py:9-47)."""
    c = _Call(q, k, k, causal, sm_scale, 0.0, L=log_normalizer.contiguous(), backend=backend, out=q)
    tot = torch.empty((c.B, c.H, c.N), device=c.dev, dtype=torch.float32)
    c.run("faws_total_attention", C.c_void_p(tot.data_ptr()))
    return tot


def last_backend() -> str:
    """Kernel family of this thread's last call: 'generic' or 'tcgen05'."""
    return {0: "none", 1: "generic", 2: "tcgen05"}[_lib.load().faws_last_backend()]


def launch_count() -> int:
    return int(_lib.load().faws_launch_count())


def device_status(reset: bool = True) -> int:
    """Synchronise and read the give-up flag of the tcgen05 kernels' bounded waits (0 = clean)."""
    return int(_lib.load().faws_device_status(1 if reset else 0))
