"""The benchmark configurations at their full sizes, checked through size-independent properties
(linear identities of the raw sums, mass conservation of the softmax sums, agreement of the two
cross-token softmax variants) and against the CPU oracle on sampled query rows."""
import math

import pytest
import torch

import flash_attn_with_score_b200 as F
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _device_inputs(cfg, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    dt = getattr(torch, cfg["dtype"])
    B, Hq, Hk, S, D = cfg["B"], cfg["Hq"], cfg["Hk"], cfg["S"], cfg["D"]
    q = torch.randn(B, Hq, S, D, device="cuda", generator=g).to(dt)
    k = torch.randn(B, Hk, S, D, device="cuda", generator=g).to(dt)
    if cfg["v"] == "uniform":
        v = (torch.rand(B, Hk, S, D, device="cuda", generator=g) * 2 - 1).to(dt)
    else:
        v = (torch.randn(B, Hk, S, D, device="cuda", generator=g) * cfg["vscale"]).to(dt)
    return q, k, v


def _sampled_rows_oracle(q, k, v, causal, rows, b, h):
    """Oracle out for a few query rows of one (b, h): fp32 on the CPU, full key range."""
    G = q.shape[1] // k.shape[1]
    qr = q[b, h, rows].float().cpu()
    kk = k[b, h // G].float().cpu()
    vv = v[b, h // G].float().cpu()
    s = qr @ kk.t() / math.sqrt(q.shape[-1])
    if causal:
        j = torch.arange(kk.shape[0]).unsqueeze(0)
        s = s.masked_fill(j > torch.tensor(rows).unsqueeze(1), float("-inf"))
    w = torch.softmax(s, -1)
    return w @ vv, s, w, vv


RAW_BF16_ERR = {}  # test label -> (largest raw |out - ref|, largest slack used), printed for the record


def _check_rows(out, q, k, v, causal, what):
    S = q.shape[2]
    rows = [0, 1, 127, 128, S // 2 - 1, S // 2, S - 2, S - 1]
    for b, h in [(0, 0), (q.shape[0] - 1, q.shape[1] - 1)]:
        ref, s, w, vv = _sampled_rows_oracle(q, k, v, causal, rows, b, h)
        got = out[b, h, rows].float().cpu()
        tol = torch.full_like(ref, orc.OUT_ATOL)
        err = (got - ref).abs()
        if out.dtype == torch.bfloat16:
            slack = ref.abs() * 2.0 ** -8 + (w @ vv.abs()) * 2.0 ** -9
            tol = tol + slack
            # on record: how far the raw bf16 error is from the plain 2e-3 bound, and how much of
            # the bf16 allowance the kernel actually uses
            old = RAW_BF16_ERR.get(what, (0.0, 0.0))
            RAW_BF16_ERR[what] = (max(old[0], err.max().item()), max(old[1], (err - orc.OUT_ATOL).clamp(min=0).max().item()))
            print(f"[bf16 out] {what} (b={b}, h={h}): raw max |out-ref| = {err.max().item():.3e} "
                  f"(plain bound {orc.OUT_ATOL:.0e}; bf16 half-ulp at max|ref|={ref.abs().max().item():.2f} is "
                  f"{ref.abs().max().item() * 2.0 ** -9:.3e}); allowance max {slack.max().item():.3e}")
        assert (err <= tol).all(), (what, b, h, err.max().item())


def _rel_rms_ok(x, ref, what):
    ok, viol = orc.check_sum(x.double().cpu(), ref.double().cpu())
    assert ok, (what, viol)


def test_cfg3_full_size_row_and_col_sums():
    cfg = orc.CONFIGS["cfg3"]
    q, k, v = _device_inputs(cfg)
    out, rs = F.attention_with_row_sum(q, k, v, True)
    assert F.last_backend() == "tcgen05"
    _check_rows(out, q, k, v, True, "cfg3 row_sum out")
    _rel_rms_ok(rs, orc.linear_row_sum(q, k, True), "cfg3 row_sum vs q_i . prefix(k)")
    out, cs = F.attention_with_col_sum(q, k, v, True, per_q_head=True)
    _check_rows(out, q, k, v, True, "cfg3 col_sum out")
    lin = orc.linear_col_sum(q, k, True)
    _rel_rms_ok(cs, lin, "cfg3 col_sum vs k_j . suffix(q)")
    _, cs_g = F.attention_with_col_sum_sequential(q, k, v, True)
    _rel_rms_ok(cs_g, orc.group_sum(lin.float(), cfg["Hk"]), "cfg3 group-summed col_sum")
    # softmax column sums conserve mass: every query row contributes exactly 1
    _, sc = F.attention_with_softmax_col_sum(q, k, v, True)
    G = cfg["Hq"] // cfg["Hk"]
    total = sc.double().sum(-1)
    assert (total - G * cfg["S"]).abs().max().item() < 1e-3 * G * cfg["S"]
    assert F.device_status() == 0


def test_cfg4_full_size_cross_token_sums():
    cfg = orc.CONFIGS["cfg4"]
    split = cfg["split"]
    q, k, v = _device_inputs(cfg)
    out, xq = F.attention_cross_token_qk_sum(q, k, v, split, True, per_q_head=True)
    assert F.last_backend() == "tcgen05"
    _check_rows(out, q, k, v, True, "cfg4 cross_qk out")
    assert xq.shape == (2, 32, 3072)
    _rel_rms_ok(xq, orc.linear_col_sum(q, k, True, i_begin=split, n_end=split), "cfg4 cross_qk identity")
    out, xs = F.attention_cross_token_softmax_sum(q, k, v, split, True)
    _check_rows(out, q, k, v, True, "cfg4 cross_softmax out")
    out_b, xb = F.attention_cross_token_softmax_sum_buffered(q, k, v, split, True)
    assert xs.shape == (2, 8, 3072)
    _rel_rms_ok(xb, xs, "buffered vs two-pass cross-token softmax sums")
    assert torch.equal(out, out_b) or (out.float() - out_b.float()).abs().max() < 2e-3
    # oracle for the queries of one head: weights of rows >= split on keys < split
    rows = list(range(split, cfg["S"]))
    G = cfg["Hq"] // cfg["Hk"]
    acc = torch.zeros(split)
    for h in range(G):  # the G query heads of kv head 0, batch 0
        _, _, w, _ = _sampled_rows_oracle(q, k, v, True, rows, 0, h)
        acc += w[:, :split].sum(0)
    _rel_rms_ok(xs[0, 0], acc, "cfg4 cross_softmax vs oracle, (b=0, kv head 0)")
    assert F.device_status() == 0


def test_cfg5_full_size_noncausal():
    cfg = orc.CONFIGS["cfg5"]
    split = cfg["split"]
    q, k, v = _device_inputs(cfg)
    S, G = cfg["S"], cfg["Hq"] // cfg["Hk"]
    out, sc = F.attention_with_softmax_col_sum(q, k, v, False)
    assert F.last_backend() == "tcgen05"
    assert sc.shape == (4, 8, S)
    _check_rows(out, q, k, v, False, "cfg5 softmax_col_sum out")
    total = sc.double().sum(-1)
    assert (total - G * S).abs().max().item() < 1e-3 * G * S
    out, xs = F.attention_cross_token_softmax_sum(q, k, v, split, False)
    assert xs.shape == (4, 8, split)
    # keys < split of rows >= split: bounded by the column sums over all rows
    assert bool((xs <= sc[:, :, :split] * (1 + 1e-3) + 1e-6).all())
    # oracle on one query head: rows >= split, all keys
    rows = list(range(split, S, 7))  # every 7th row keeps the CPU work small
    _, _, w, _ = _sampled_rows_oracle(q, k, v, False, rows, 3, 31)
    _, xh = F.attention_cross_token_softmax_sum(q, k, v, split, False, per_q_head=True, q_rows=None)
    rows_all = list(range(split, S))
    _, _, w_all, _ = _sampled_rows_oracle(q, k, v, False, rows_all, 3, 31)
    _rel_rms_ok(xh[3, 31], w_all[:, :split].sum(0), "cfg5 cross_softmax per head vs oracle")
    # raw sums via the linear identity (non-causal: every query sees every key)
    _, cs = F.attention_with_col_sum(q, k, v, False, per_q_head=True)
    _rel_rms_ok(cs[0, :4], orc.linear_col_sum(q[:1, :4], k[:1, :1], False), "cfg5 col_sum identity")
    assert F.device_status() == 0


# ------------------------------------------------------------------ the two score-materialising configurations
def _cfg_cpu_inputs(name):
    cfg = orc.CONFIGS[name]
    g = torch.Generator().manual_seed(0)
    B, Hq, Hk, S, D = cfg["B"], cfg["Hq"], cfg["Hk"], cfg["S"], cfg["D"]
    q = torch.randn(B, Hq, S, D, generator=g)  # fp32 draw, then the cast the GPU run receives
    k = torch.randn(B, Hk, S, D, generator=g)
    v = torch.randn(B, Hk, S, D, generator=g)
    return q.half(), k.half(), v.half()


def _check_scores_and_out(out, scores, ref_out, ref_scores, what):
    ok, err = orc.check_out(out.cpu(), ref_out)
    assert ok, f"{what}: out max abs err {err}"
    ok, viol, ok_mask = orc.check_scores(scores.cpu(), ref_scores)
    assert ok_mask, f"{what}: hidden entries are not exactly the oracle's -inf set"
    assert ok, f"{what}: scores violation {viol}"
    hidden = torch.isneginf(ref_scores)
    bits = scores.cpu().view(torch.int32)[hidden]
    assert bool((bits == orc.NEG_INF_BITS - (1 << 32)).all()), f"{what}: fill is not 0xFF800000"


@pytest.mark.parametrize("name", ["cfg1", "cfg2"])
def test_cfg1_cfg2_whole_tensor_against_oracle(name):
    """cfg1 (B1 H8 S512 D64) and cfg2 (B1 H32 S1024 D128), causal, fp16 inputs cast from an fp32
    draw with seed 0: the whole out and the whole fp32 score tensor against the CPU oracle."""
    cfg = orc.CONFIGS[name]
    q, k, v = _cfg_cpu_inputs(name)
    ref_out, ref_scores = orc.naive_attention_with_scores(q, k, v, True)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out, scores = F.attention_with_scores(qd, kd, vd, True)
    assert F.last_backend() == "tcgen05"
    assert scores.shape == (cfg["B"], cfg["Hq"], cfg["S"], cfg["S"]) and scores.dtype == torch.float32
    _check_scores_and_out(out, scores, ref_out, ref_scores, name)

    # caller-owned buffers (the call bench.py times), poisoned before every use
    out_b = torch.full_like(qd, float("nan"))
    sc_b = torch.full_like(scores, float("nan"))
    o2, s2 = F.attention_with_scores(qd, kd, vd, True, out=out_b, scores=sc_b)
    assert o2.data_ptr() == out_b.data_ptr() and s2.data_ptr() == sc_b.data_ptr()
    _check_scores_and_out(out_b, sc_b, ref_out, ref_scores, name + " out=/scores=")
    assert torch.equal(out_b, out) and torch.equal(sc_b.view(torch.int32), scores.view(torch.int32))

    # the same call captured in a CUDA graph and replayed onto poisoned buffers
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        F.attention_with_scores(qd, kd, vd, True, out=out_b, scores=sc_b)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        out_b.fill_(float("nan"))
        sc_b.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        _check_scores_and_out(out_b, sc_b, ref_out, ref_scores, name + " graph replay")
    assert F.device_status() == 0

    # every other score-free product of the same inputs, derived from the oracle's score tensor
    o, rs = F.attention_with_row_sum(qd, kd, vd, True)
    _rel_rms_ok(rs, orc.row_sum(ref_scores), name + " row_sum")
    o, cs = F.attention_with_col_sum(qd, kd, vd, True)
    _rel_rms_ok(cs, orc.group_sum(orc.col_sum(ref_scores), cfg["Hk"]), name + " col_sum")
    ok, err = orc.check_out(o.cpu(), ref_out)
    assert ok, err
    o, sc = F.attention_with_softmax_col_sum(qd, kd, vd, True)
    _rel_rms_ok(sc, orc.group_sum(orc.softmax_col_sum(ref_scores), cfg["Hk"]), name + " softmax_col_sum")
    assert F.device_status() == 0


def test_bf16_raw_error_report():
    """Runs after the cfg3 / cfg5 tests of this file: prints the raw bf16 errors they recorded."""
    for what, (raw, over) in sorted(RAW_BF16_ERR.items()):
        print(f"[bf16 out summary] {what}: raw max abs err {raw:.3e}, above the plain 2e-3 bound by {over:.3e}")
