"""CPU oracle for the attention-with-scores family.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA kernels are compared against.  It is a
plain fp32 restatement (torch CPU ops, no custom kernels) of the reference's
own PyTorch oracle and of the derivations its verifier applies to that oracle:

* ``naive_attention_with_scores``   follows reference_implementations.py:11-52
* ``row_sum``                       follows benchmark.py:1528-1534
* ``col_sum``                       follows benchmark.py:1575-1581
* ``cross_token_qk_sum``            follows benchmark.py:1687-1693
* ``cross_token_softmax_sum``       follows benchmark.py:1627-1646 (true -inf
                                    instead of the -6e4 stand-in; identical in fp32)
* ``softmax_col_sum``               softmax(scores, -1).sum(-2); the reference
                                    verifier never checks this quantity
                                    (benchmark.py:1352 stores it, nothing reads it)
* ``log_normalizer``                flash.py:486  (L = m*sm_scale + log(l))
* ``attention_backward``            torch autograd through the formulas above: the gradients
                                    FlashAttention.backward (flash.py:172-261) computes
* ``group_sum``                     the (B,Hk,.) layout the reference kernels
                                    return because their output pointer is
                                    offset by the kv head (attention_with_col_sum.py:72)

Parity pin: ``tests/golden/*.npz`` were produced by importing the reference's
``reference_implementations.naive_attention_with_scores`` (see
``tests/golden/make_golden.py``) and ``tests/test_oracle.py`` checks this
restatement against them bit for bit.  Quantities the reference's own checks
never exercise (GQA group sums, softmax column sums, M != N, non-causal) are
"parity unpinned" by the reference; they are pinned here only through the
stored reference scores tensor and the formulas above.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
legs may import this module.  The product package never does.
"""
from __future__ import annotations

import math

import torch

NEG_INF_BITS = 0xFF800000


def _expand_kv(x: torch.Tensor, groups: int) -> torch.Tensor:
    return x if groups == 1 else torch.repeat_interleave(x, repeats=groups, dim=1)


def causal_mask(M: int, N: int, p_seq: int = 0) -> torch.Tensor:
    """True where key j is hidden from query i, i.e. j > i + p_seq.

    p_seq = 0 is the reference oracle's top-left mask
    (reference_implementations.py:36-40, torch.triu(diagonal=1)); p_seq = N - M
    is the kernels' bottom-right alignment (flash.py:451).  Equal when M == N.
    """
    i = torch.arange(M).unsqueeze(1)
    j = torch.arange(N).unsqueeze(0)
    return j > (i + p_seq)


def naive_attention_with_scores(q, k, v, causal, sm_scale=None, p_seq=0):
    """(out, scores) in fp32 from inputs upcast to fp32.

    scores = q @ k^T * sm_scale with -inf at masked entries; out =
    softmax(scores) @ v.  Rows with no visible key give out = 0 (the kernels'
    behaviour, flash.py:480-483) instead of NaN.
    """
    q = q.float()
    k = k.float()
    v = v.float()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    assert Hq % Hk == 0
    g = Hq // Hk
    k = _expand_kv(k, g)
    v = _expand_kv(v, g)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    scores = torch.matmul(q, k.transpose(-2, -1)) * sm_scale
    if causal:
        scores = scores.masked_fill(causal_mask(M, N, p_seq), float("-inf"))
    w = torch.softmax(scores, dim=-1)
    w = torch.nan_to_num(w, nan=0.0)
    out = torch.matmul(w, v)
    return out, scores


def _zero_masked(scores):
    return torch.where(torch.isneginf(scores), torch.zeros_like(scores), scores)


def row_sum(scores):
    """(B,Hq,M): sum over visible keys of the scaled raw score."""
    return _zero_masked(scores).sum(dim=-1)


def col_sum(scores):
    """(B,Hq,N): sum over visible queries of the scaled raw score."""
    return _zero_masked(scores).sum(dim=-2)


def softmax_weights(scores):
    return torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)


def softmax_col_sum(scores):
    """(B,Hq,N): column sums of the softmax weights."""
    return softmax_weights(scores).sum(dim=-2)


def cross_token_qk_sum(scores, split):
    """(B,Hq,split): raw-score sums of queries >= split into keys < split."""
    return _zero_masked(scores)[:, :, split:, :split].sum(dim=-2)


def cross_token_softmax_sum(scores, split):
    """(B,Hq,split): softmax-weight sums of queries >= split into keys < split."""
    return softmax_weights(scores)[:, :, split:, :split].sum(dim=-2)


def log_normalizer(scores):
    """(B,Hq,M): logsumexp of the scaled scores; -inf for empty rows."""
    return torch.logsumexp(scores, dim=-1)


def group_sum(x, Hk):
    """(B,Hq,L) -> (B,Hk,L): sum the G = Hq/Hk query heads sharing a kv head."""
    B, Hq, L = x.shape
    return x.view(B, Hk, Hq // Hk, L).sum(dim=2)


# ---------------------------------------------------------------------------
# O(S*D) known-answer identities for the raw sums (no S^2 tensor needed).
# With visible(i) = {j <= i + p_seq} (causal) or all j:
#   col_sum_j = sm_scale * k_j . sum_{i visible to j} q_i
#   row_sum_i = sm_scale * q_i . sum_{j visible to i} k_j
# ---------------------------------------------------------------------------

def linear_col_sum(q, k, causal, sm_scale=None, p_seq=0, i_begin=0, n_end=None):
    """fp64 (B,Hq,n_end) raw column sums over queries i >= i_begin."""
    q = q.double()
    k = k.double()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    n_end = N if n_end is None else n_end
    k = _expand_kv(k, Hq // Hk)[:, :, :n_end]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qz = q.clone()
    qz[:, :, :i_begin] = 0
    if causal:
        # suffix[i] = sum_{i' >= i} q_i'; key j sees queries i >= max(j - p_seq, 0)
        suffix = torch.flip(torch.cumsum(torch.flip(qz, dims=[2]), dim=2), dims=[2])
        suffix = torch.cat([suffix, torch.zeros_like(suffix[:, :, :1])], dim=2)
        first = (torch.arange(n_end, device=q.device) - p_seq).clamp(min=0, max=M)
        qs = suffix[:, :, first]
    else:
        qs = qz.sum(dim=2, keepdim=True).expand(B, Hq, n_end, D)
    return (k * qs).sum(-1) * sm_scale


def linear_row_sum(q, k, causal, sm_scale=None, p_seq=0):
    """fp64 (B,Hq,M) raw row sums."""
    q = q.double()
    k = k.double()
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    k = _expand_kv(k, Hq // Hk)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    if causal:
        prefix = torch.cumsum(k, dim=2)
        prefix = torch.cat([torch.zeros_like(prefix[:, :, :1]), prefix], dim=2)
        cnt = (torch.arange(M, device=q.device) + p_seq + 1).clamp(min=0, max=N)
        ks = prefix[:, :, cnt]
    else:
        ks = k.sum(dim=2, keepdim=True).expand(B, Hq, M, D)
    return (q * ks).sum(-1) * sm_scale

# -- dropout (dropout_p > 0) ---------------------------------------------------
# The reference kernels draw one uniform per (b, h, i, j) from Triton's Philox-4x32 with six
# rounds, `tl.rand(seed, offs, n_rounds=6)` (flash.py:465), at the linear offset
# offset + ((b*Hq + h)*M + i)*N + j computed in 32-bit arithmetic (flash.py:376-380), and keep an
# entry iff the uniform is > dropout_p.  The generator lives in the triton package (3.6.0:
# triton/language/random.py, `philox_impl`, `randint4x`, `uint_to_uniform_float`); it is restated
# below from its published definition and pinned by tests/golden/dropout_philox_stream.npz, which
# holds tl.rand outputs produced with that package.  Only the first of the four Philox outputs
# is used; the counter is (c0, 0, 0, 0) and the key is the 64-bit seed's two halves.

def philox_uniform(seed: int, offsets, n_rounds: int = 6):
    """tl.rand(seed, offsets, n_rounds) for 32-bit offsets; returns float32 numpy array."""
    import numpy as np

    ka, kb = 0x9E3779B9, 0xBB67AE85
    ra, rb = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    c0 = np.asarray(offsets).astype(np.uint32)
    c1 = np.zeros_like(c0)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(n_rounds):
        pb = rb * c2.astype(np.uint64)
        pa = ra * c0.astype(np.uint64)
        c0, c2, c1, c3 = ((pb >> np.uint64(32)).astype(np.uint32) ^ c1 ^ np.uint32(k0),
                          (pa >> np.uint64(32)).astype(np.uint32) ^ c3 ^ np.uint32(k1),
                          pb.astype(np.uint32), pa.astype(np.uint32))
        k0, k1 = (k0 + ka) & 0xFFFFFFFF, (k1 + kb) & 0xFFFFFFFF
    x = c0.view(np.int32)
    x = np.where(x < 0, -x - 1, x).astype(np.int32)
    return x.astype(np.float32) * np.float32(4.6566127342e-10)


def dropout_keep_mask(seed: int, offset: int, B: int, Hq: int, M: int, N: int, dropout_p: float):
    """(B,Hq,M,N) bool: entries the reference kernels keep (flash.py:376-380,463-466)."""
    import numpy as np

    assert 0 <= offset < 2 ** 31, "the 64-bit Philox variant Triton switches to is not restated"
    idx = (np.arange(B * Hq * M * N, dtype=np.uint64) + np.uint64(offset)).astype(np.uint32)
    u = philox_uniform(seed, idx)
    return torch.from_numpy(u > np.float32(dropout_p)).reshape(B, Hq, M, N)


def dropout_out(scores, v, keep, dropout_p):
    """out under dropout: (softmax(scores) * keep) @ v / (1 - p); the normaliser is taken before
    the mask (flash.py:459-466,488-491)."""
    Hq, Hk = scores.shape[1], v.shape[1]
    w = softmax_weights(scores) * keep.float()
    return torch.matmul(w, _expand_kv(v.float(), Hq // Hk)) * (1.0 / (1.0 - dropout_p))


def dropout_softmax_col_sum(scores, keep):
    """Softmax column sum of attention_with_softmax_col_sum under dropout: dropped weights are left
    out and nothing is rescaled (attention_with_col_softmax_sum.py:238-244)."""
    return (softmax_weights(scores) * keep.float()).sum(dim=-2)



# -- backward pass ---------------------------------------------------------------
def attention_backward(q, k, v, dout, causal, sm_scale=None, p_seq=0, keep=None, dropout_p=0.0):
    """(dq, dk, dv) of out = softmax(mask(q k^T * sm_scale)) v with respect to fp32 copies of the
    inputs, by torch autograd through the same formulas as naive_attention_with_scores (what
    FlashAttention.backward, flash.py:172-261, computes).  dk, dv come out in the (B,Hk,N,D) layout:
    autograd sums the G query heads of a kv head (flash.py:259-260).  ``keep`` (B,Hq,M,N) bool and
    ``dropout_p`` apply the forward pass's dropout mask (weights kept are rescaled by 1/(1-p))."""
    q = q.detach().float().requires_grad_(True)
    k = k.detach().float().requires_grad_(True)
    v = v.detach().float().requires_grad_(True)
    B, Hq, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    g = Hq // Hk
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    scores = torch.matmul(q, _expand_kv(k, g).transpose(-2, -1)) * sm_scale
    if causal:
        scores = scores.masked_fill(causal_mask(M, N, p_seq), float("-inf"))
    w = torch.nan_to_num(torch.softmax(scores, dim=-1), nan=0.0)
    if keep is not None:
        w = w * keep.float() * (1.0 / (1.0 - dropout_p))
    out = torch.matmul(w, _expand_kv(v, g))
    out.backward(dout.float())
    return q.grad, k.grad, v.grad


GRAD_ATOL = 2e-3


def grad_slack(q, k, v, dout, causal, sm_scale=None, p_seq=0, bf16=False):
    """Error a 16-bit pipeline cannot avoid in (dq, dk, dv), per element, from two roundings the
    reference's kernels perform as well: ``out`` is stored in 16 bits before delta_i = sum_d
    out_id * dout_id is taken from it (flash.py:202-213), which moves delta_i by at most
    e_i = eps * sum_d |out_id * dout_id| and hence dq_i by sm_scale * e_i * sum_j p_ij |k_j| and dk_j
    by sm_scale * sum_i p_ij e_i |q_i|; and P is rounded to 16 bits before P^T dO (flash.py:704),
    which moves dv_j by at most eps * sum_i p_ij |dout_i|.  eps = 2^-11 (fp16) or 2^-8 (bf16)."""
    eps = 2.0 ** -8 if bf16 else 2.0 ** -11
    q, k, v, dout = q.float(), k.float(), v.float(), dout.float()
    B, Hq, M, D = q.shape
    Hk = k.shape[1]
    g = Hq // Hk
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    out, scores = naive_attention_with_scores(q, k, v, causal, sm_scale, p_seq)
    p = softmax_weights(scores)
    e = eps * (out * dout).abs().sum(-1, keepdim=True)  # (B,Hq,M,1)
    s_dq = sm_scale * e * torch.matmul(p, _expand_kv(k.abs(), g))
    s_dk = sm_scale * torch.matmul(p.transpose(-2, -1), e * q.abs())
    s_dv = eps * torch.matmul(p.transpose(-2, -1), dout.abs())
    fold = lambda x: x.view(B, Hk, g, *x.shape[2:]).sum(2)  # noqa: E731
    return s_dq, fold(s_dk), fold(s_dv)


def check_grad(x, ref, bf16=False, slack=None):
    """|x - ref| <= 2e-3 * max(1, rms(ref)) + rel * |ref| (+ ``slack`` from grad_slack); rel = 2^-10
    (fp16 tensors) or 2^-7 (bf16): rounding of the stored 16-bit result."""
    x = x.double()
    ref = ref.double()
    rms = ref.pow(2).mean().sqrt().item()
    rel = 2.0 ** -7 if bf16 else 2.0 ** -10
    tol = GRAD_ATOL * max(1.0, rms) + rel * ref.abs()
    if slack is not None:
        tol = tol + slack.double()
    viol = (x - ref).abs() - tol
    return bool((viol <= 0).all()), viol.max().item(), (x - ref).abs().max().item()


# ---------------------------------------------------------------------------
# Tolerances (written once, used by every parity test).
#   out                      : max abs <= 2e-3 (+ bf16_out_slack when the tensors are bf16)
#   scores                   : |x-ref| <= 1e-3*|ref| + 1e-4, masked entries bit-exact
#   sums (fp32 accumulation) : |x-ref| <= 1e-3*|ref| + 1e-3*rms(ref)
# ---------------------------------------------------------------------------
OUT_ATOL = 2e-3
REL_TOL = 1e-3
SCORES_ATOL = 1e-4


def bf16_out_slack(scores, v, out):
    """Extra |out| error a bf16 pipeline cannot avoid, per element: the stored result is
    rounded to bf16 (<= 2^-8 |out|, bf16 keeps 8 significant bits) and the softmax weights
    are rounded to bf16 before the P.V product, as the reference kernel does
    (flash.py:470 ``p.to(input_dtype)``), which moves out by <= 2^-9 * sum_j w_ij |v_j|.
    fp16 (11 bits) stays inside the plain 2e-3 bound, so this is used for bf16 only."""
    Hq, Hk = scores.shape[1], v.shape[1]
    w = softmax_weights(scores)
    absv = _expand_kv(v.float().abs(), Hq // Hk)
    return out.float().abs() * 2.0 ** -8 + torch.matmul(w, absv) * 2.0 ** -9


def check_out(x, ref, slack=None):
    """max |x - ref| <= 2e-3 (+ ``slack`` from bf16_out_slack for bf16 tensors)."""
    diff = (x.float() - ref.float()).abs()
    tol = torch.full_like(diff, OUT_ATOL)
    if slack is not None:
        tol = tol + slack
    viol = (diff - tol).max().item()
    return viol <= 0, diff.max().item()


def check_sum(x, ref):
    x = x.double()
    ref = ref.double()
    atol = REL_TOL * ref.pow(2).mean().sqrt().item()
    viol = (x - ref).abs() - (REL_TOL * ref.abs() + atol)
    return bool((viol <= 0).all()), viol.max().item()


def check_scores(x, ref, masked_bits=NEG_INF_BITS):
    """Masked set identical and bit-exact fill; finite entries within tolerance."""
    x = x.float()
    ref = ref.float()
    hidden = torch.isneginf(ref)
    xb = x.contiguous().view(torch.int32)
    fill = masked_bits - (1 << 32) if masked_bits >= (1 << 31) else masked_bits
    ok_mask = bool((xb[hidden] == fill).all())
    if masked_bits == NEG_INF_BITS:
        ok_mask = ok_mask and bool((torch.isneginf(x) == hidden).all())
    xv, rv = x[~hidden], ref[~hidden]
    viol = (xv - rv).abs() - (REL_TOL * rv.abs() + SCORES_ATOL)
    ok_val = bool((viol <= 0).all()) if xv.numel() else True
    return ok_mask and ok_val, (viol.max().item() if xv.numel() else 0.0), ok_mask


# ---------------------------------------------------------------------------
# Seeded synthetic inputs with the shapes and value distributions of the five
# benchmark configurations (random tensors, as the reference's own benchmark
# uses: benchmark.py:281-283).
# ---------------------------------------------------------------------------
CONFIGS = {
    "cfg1": dict(B=1, Hq=8, Hk=8, S=512, D=64, dtype="float16", causal=True, v="normal", vscale=1.0, split=None),
    "cfg2": dict(B=1, Hq=32, Hk=32, S=1024, D=128, dtype="float16", causal=True, v="normal", vscale=1.0, split=None),
    "cfg3": dict(B=1, Hq=28, Hk=4, S=4096, D=128, dtype="bfloat16", causal=True, v="normal", vscale=0.5, split=None),
    "cfg4": dict(B=2, Hq=32, Hk=8, S=4096, D=128, dtype="float16", causal=True, v="normal", vscale=1.0, split=3072),
    "cfg5": dict(B=4, Hq=32, Hk=8, S=16384, D=128, dtype="bfloat16", causal=False, v="uniform", vscale=1.0, split=12288),
}


def make_unit_inputs(cfg: dict, unit: int, seed: int = 0, S: int | None = None):
    """q (1,G,S,D), k, v (1,1,S,D) of shard unit ``unit`` = b*Hk + hk.

    Drawn in fp32 on the CPU from ``seed + unit`` and cast to the config's
    dtype, so any rank (and the oracle) can rebuild any unit independently.
    """
    S = cfg["S"] if S is None else S
    G = cfg["Hq"] // cfg["Hk"]
    D = cfg["D"]
    dt = getattr(torch, cfg["dtype"])
    g = torch.Generator().manual_seed(seed + unit)
    q = torch.randn(1, G, S, D, generator=g)
    k = torch.randn(1, 1, S, D, generator=g)
    if cfg["v"] == "uniform":
        v = torch.rand(1, 1, S, D, generator=g) * 2 - 1
    else:
        v = torch.randn(1, 1, S, D, generator=g) * cfg["vscale"]
    return q.to(dt), k.to(dt), v.to(dt)


def make_inputs(cfg: dict, seed: int = 0, S: int | None = None, units=None):
    """Full (B,Hq,S,D)/(B,Hk,S,D) tensors assembled from per-unit draws."""
    B, Hk = cfg["B"], cfg["Hk"]
    G = cfg["Hq"] // Hk
    units = range(B * Hk) if units is None else units
    qs, ks, vs = [], [], []
    for u in units:
        q, k, v = make_unit_inputs(cfg, u, seed, S)
        qs.append(q)
        ks.append(k)
        vs.append(v)
    n = len(qs)
    if n == B * Hk:
        q = torch.cat(qs, 1).view(B, Hk * G, *qs[0].shape[2:])
        k = torch.cat(ks, 1).view(B, Hk, *ks[0].shape[2:])
        v = torch.cat(vs, 1).view(B, Hk, *vs[0].shape[2:])
    else:
        q = torch.cat(qs, 1)
        k = torch.cat(ks, 1)
        v = torch.cat(vs, 1)
    return q.contiguous(), k.contiguous(), v.contiguous()
