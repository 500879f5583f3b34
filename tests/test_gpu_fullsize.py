"""GPU parity at the BASELINE.json sizes.

The oracle cannot redo these shapes whole in seconds, so each test combines
  * exact checks on a sample (query rows, q-blocks or one whole (batch, head)
    slice) against the fp64 oracle, with
  * size-independent properties over the full output (rows of scores sum to
    one, ranks sorted by average, ids unique and in range, merge / reverse
    index consistent with each other, untouched rows exactly zero).
"""

import numpy as np
import pytest
import torch

import cases
from oracle import ftk_oracle as orc

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def ftk():
    import flash_topk_attn_v2 as m
    return m


def _close(got, want, what, atol=ATOL, rtol=RTOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), f"{what}: finiteness differs"
    err = np.abs(got[fin] - want[fin])
    bad = err > atol + rtol * np.abs(want[fin])
    assert not bad.any(), f"{what}: {int(bad.sum())} bad, max err {float(err.max()):.3e}"


def _slice_head(t, b, h, D):
    """[B,N,H*D] torch tensor -> float64 numpy [1,N,D] of one (batch, head)."""
    return t[b:b + 1, :, h * D:(h + 1) * D].float().numpy().astype(np.float64)


def _oracle_rows(q1, k1, rows, bsz, pad):
    """fp64 block scores of selected query rows of one slice: [len(rows), M]."""
    n = k1.shape[1]
    m, starts, ends, valid = orc.block_geometry(n, bsz, pad)
    d = q1.shape[-1]
    s = (q1[0, rows] * d ** -0.5) @ k1[0].T
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return np.add.reduceat(p, starts, axis=1), valid


def _check_topk_properties(idx, raw, avg, M, K):
    idx, raw, avg = idx.cpu().numpy(), raw.cpu().numpy(), avg.cpu().numpy()
    assert idx.shape[-1] == min(K, M) if K > 0 else M
    valid = idx >= 0
    assert ((idx < M) | ~valid).all()
    # valid entries form a prefix, padding is (-1, 0, 0)
    assert (valid[..., :-1] | ~valid[..., 1:]).all()
    assert (raw[~valid] == 0).all() and (avg[~valid] == 0).all()
    # ranks sorted by average, descending
    a = np.where(valid, avg, -1.0)
    assert (a[..., :-1] >= a[..., 1:]).all()
    # ids unique per row
    srt = np.sort(np.where(valid, idx, -np.arange(1, idx.shape[-1] + 1)), axis=-1)
    assert (srt[..., 1:] != srt[..., :-1]).all()
    assert (raw.sum(-1) <= 1.0 + 1e-5).all() and (raw >= 0).all()
    return idx, raw, avg


def _check_sample_rows(idx, raw, q, k, H, D, bsz, pad, thr, K, samples, seed=0):
    """Selected rows against the fp64 oracle; returns the tie report."""
    rng = np.random.default_rng(seed)
    B, N = q.shape[0], q.shape[1]
    ties = hard = pos = 0
    for (b, h) in samples:
        rows = np.sort(rng.choice(N, size=48, replace=False))
        rows[0], rows[-1] = 0, N - 1              # include the padded edges
        q1, k1 = _slice_head(q, b, h, D), _slice_head(k, b, h, D)
        sc, valid = _oracle_rows(q1, k1, rows, bsz, pad)
        oi, oraw, _ = orc.topk_select(sc[None, None].astype(np.float32), thr, K, bsz, pad)
        rep = orc.classify_topk_mismatches(idx[b, h, rows], oi[0, 0], sc / valid, rel_band=1e-6)
        ties += rep["ties"]
        hard += rep["hard"]
        pos += rep["positions"]
        assert rep["hard"] == 0, rep
        same = idx[b, h, rows] == oi[0, 0]
        np.testing.assert_allclose(raw[b, h, rows][same], oraw[0, 0][same], rtol=2e-5, atol=1e-9)
    return {"positions": pos, "ties": ties, "hard": hard}


def test_config2_scoring(ftk):
    """B=1 N=32768 H=32 D=128 bf16, block 64, topk 32, threshold 0.9."""
    cfg = cases.BASELINE_CONFIGS[2]
    t = cases.make_inputs(dict(cfg, B=1))
    H, D, b, K, thr = cfg["H"], cfg["D"], cfg["score_block_size"], cfg["topk"], cfg["threshold"]
    q, k = t["q"], t["k"]
    idx, raw, avg = ftk.flash_topk_score(q.cuda(), k.cuda(), H, b, K, (0, 0), thr)
    ftk.check_errors()
    M = cfg["N"] // b
    idx, raw, avg = _check_topk_properties(idx, raw, avg, M, K)
    rep = _check_sample_rows(idx, raw, q, k, H, D, b, (0, 0), thr, K,
                             [(0, 0), (0, 13), (0, 31)])
    print("config2 sample:", rep)
    # a handful of full rows of the score matrix as well
    sc = ftk.flash_block_score(q[:, :, :2 * D].cuda(), k[:, :, :2 * D].cuda(), 2, b)
    np.testing.assert_allclose(sc.sum(-1).cpu().numpy(), 1.0, atol=3e-6)
    rows = np.array([0, 77, 4095, 20000, 32767])
    want, _ = _oracle_rows(_slice_head(q, 0, 1, D), _slice_head(k, 0, 1, D), rows, b, (0, 0))
    np.testing.assert_allclose(sc[0, 1, rows].cpu().numpy(), want, rtol=5e-6, atol=1e-10)


def test_config4_ragged_score_select_merge_attend(ftk):
    """B=2 N=30000 H=32 D=128 fp16, block 128, padding (40, 40), hot blocks,
    threshold 0.8, merge at q_block_size 128, then attention forward and
    backward at 128-row q / kv blocks (reduced to 2 x 8 heads to keep the
    host-side input generation short; shapes per slice are the config's)."""
    cfg = dict(cases.BASELINE_CONFIGS[4], H=8)
    t = cases.make_inputs(cfg)
    H, D, b, K, thr = cfg["H"], cfg["D"], cfg["score_block_size"], cfg["topk"], cfg["threshold"]
    pad = tuple(cfg["padding"])
    q, k = t["q"], t["k"]
    idx_t, raw_t, avg_t = ftk.flash_topk_score(q.cuda(), k.cuda(), H, b, K, pad, thr)
    ftk.check_errors()
    M = (pad[0] + cfg["N"] + pad[1]) // b
    assert M == 235
    idx, raw, avg = _check_topk_properties(idx_t, raw_t, avg_t, M, K)
    cut = (idx[..., -1] < 0).mean()
    print("config4: threshold cut before k on", float(cut), "of rows")
    assert cut > 0          # the skewed keys must exercise the threshold
    rep = _check_sample_rows(idx, raw, q, k, H, D, b, pad, thr, K, [(0, 0), (1, 5)], seed=4)
    print("config4 sample:", rep)

    # merge of the whole GPU top-k table, bit-exact against the oracle merge
    g = cfg["q_block_size"]
    qpad = tuple(cfg["q_padding"])
    merged, counts, W = ftk.build_qblock_topk_indices(idx_t, g, qpad, avg_t)
    ftk.check_errors()
    om, oc, oW, _ = orc.build_qblock_topk_indices(idx, g, qpad, avg, None)
    assert W == oW == g * K
    np.testing.assert_array_equal(merged.cpu().numpy(), om)
    np.testing.assert_array_equal(counts.cpu().numpy(), oc)

    # attention at 128-row q and kv blocks over those lists (beyond the
    # reference, which rejects q blocks above 64): forward and backward on the
    # GPU, one (batch, head) slice re-done by the fp64 oracle
    kvb = 128
    qg = q.cuda().requires_grad_(True)
    kg = k.cuda().requires_grad_(True)
    vg = t["v"].cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(qg, kg, vg, merged, counts, H, g, kvb,
                                 kv_padding=pad, q_padding=qpad)
    o.backward(t["do"].cuda())
    ftk.check_errors()
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    b_i, h_i = 1, 3
    x = {n: _slice_head(t[n], b_i, h_i, D) for n in ("q", "k", "v", "do")}
    m1 = om[b_i:b_i + 1, h_i:h_i + 1]
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], m1, 1, g, kvb, None, qpad, pad)
    go = o.detach()[b_i, :, h_i * D:(h_i + 1) * D].float().cpu().numpy()[None]
    _close(go, wo, "O")
    _close(lse[b_i, h_i].cpu().numpy(), wl[0, 0], "lse")
    wq, wk, wv = orc.sparse_attn_bwd(x["q"], x["k"], x["v"], go, wl, x["do"], m1, 1, g, kvb,
                                     None, qpad, pad)
    sl = (b_i, slice(None), slice(h_i * D, (h_i + 1) * D))
    _close(qg.grad[sl].float().cpu().numpy()[None], wq, "dQ")
    _close(kg.grad[sl].float().cpu().numpy()[None], wk, "dK")
    _close(vg.grad[sl].float().cpu().numpy()[None], wv, "dV")


def test_config3_train_step_one_slice_exact(ftk):
    """B=4 N=8192 H=16 D=128 bf16, topk 16, q/kv block 64, qblock_topk 256:
    whole forward + backward on the GPU; two (batch, head) slices re-done
    entirely by the fp64 oracle, the rest checked through properties."""
    cfg = cases.BASELINE_CONFIGS[3]
    t = cases.make_inputs(cfg)
    B, N, H, D = cfg["B"], cfg["N"], cfg["H"], cfg["D"]
    b, K, g, kvb, W = (cfg["score_block_size"], cfg["topk"], cfg["q_block_size"],
                       cfg["kv_block_size"], cfg["qblock_topk"])
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    idx, raw, avg = ftk.flash_topk_score(q.detach(), k.detach(), H, b, K)
    merged, counts, Wout = ftk.build_qblock_topk_indices(idx, g, topk_scores=avg, qblock_topk=W)
    assert Wout == W
    o, lse = ftk.flash_topk_attn(q, k, v, merged, counts, H, g, kvb)
    o.backward(t["do"].cuda())
    ftk.check_errors()
    M = N // b
    _check_topk_properties(idx, raw, avg, M, K)
    mg, cn = merged.cpu().numpy(), counts.cpu().numpy()
    assert ((mg >= 0).sum(-1) == cn).all() and (mg < M).all()
    assert np.isfinite(o.detach().float().cpu().numpy()).all()
    for b_i, h_i in ((0, 0), (3, 11)):
        x = {n: _slice_head(t[n], b_i, h_i, D) for n in ("q", "k", "v", "do")}
        m1 = mg[b_i:b_i + 1, h_i:h_i + 1]
        # merge itself: exact against the oracle fed with the GPU's top-k
        om, oc, _, _ = orc.build_qblock_topk_indices(
            idx[b_i:b_i + 1, h_i:h_i + 1].cpu().numpy(), g, (0, 0),
            avg[b_i:b_i + 1, h_i:h_i + 1].cpu().numpy(), W)
        np.testing.assert_array_equal(m1, om)
        wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], m1, 1, g, kvb)
        go = o.detach()[b_i, :, h_i * D:(h_i + 1) * D].float().cpu().numpy()[None]
        _close(go, wo, "O")
        _close(lse[b_i, h_i].cpu().numpy(), wl[0, 0], "lse")
        wq, wk, wv = orc.sparse_attn_bwd(x["q"], x["k"], x["v"], go, wl, x["do"], m1, 1, g, kvb)
        sl = (b_i, slice(None), slice(h_i * D, (h_i + 1) * D))
        _close(q.grad[sl].float().cpu().numpy()[None], wq, "dQ")
        _close(k.grad[sl].float().cpu().numpy()[None], wk, "dK")
        _close(v.grad[sl].float().cpu().numpy()[None], wv, "dV")


def test_config5_slice_of_long_context(ftk):
    """One batch element, 2 of the 64 heads of the N=65536 config (what one
    GPU sees of a chunk): M = QM = 1024, topk 64, default qblock_topk 4096."""
    cfg = dict(cases.BASELINE_CONFIGS[5], B=1, H=2)
    t = cases.make_inputs(cfg)
    N, H, D = cfg["N"], cfg["H"], cfg["D"]
    b, K, g, kvb = cfg["score_block_size"], cfg["topk"], cfg["q_block_size"], cfg["kv_block_size"]
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    idx_t, raw_t, avg_t = ftk.flash_topk_score(q.detach(), k.detach(), H, b, K)
    M = N // b
    idx, raw, avg = _check_topk_properties(idx_t, raw_t, avg_t, M, K)
    rep = _check_sample_rows(idx, raw, t["q"], t["k"], H, D, b, (0, 0), 1.0, K, [(0, 1)], seed=5)
    print("config5 sample:", rep)
    merged, counts, W = ftk.build_qblock_topk_indices(idx_t, g, topk_scores=avg_t)
    assert W == g * K == 4096 and merged.shape == (1, H, N // g, W)
    o, lse = ftk.flash_topk_attn(q, k, v, merged, counts, H, g, kvb)
    o.backward(t["do"].cuda())
    ftk.check_errors()
    mg = merged.cpu().numpy()
    # a few q-blocks and kv blocks of head 1 against the oracle
    x = {n: _slice_head(t[n], 0, 1, D) for n in ("q", "k", "v", "do")}
    pick = [0, 517, N // g - 1]
    m1 = np.full((1, 1, N // g, W), -1, dtype=np.int32)
    m1[0, 0, pick] = mg[0, 1, pick]
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], m1, 1, g, kvb)
    go = o.detach()[0, :, D:2 * D].float().cpu().numpy()[None]
    rows = np.concatenate([np.arange(m * g, (m + 1) * g) for m in pick])
    _close(go[:, rows], wo[:, rows], "O")
    _close(lse[0, 1].cpu().numpy()[rows], wl[0, 0, rows], "lse")
    wq, _, _ = orc.sparse_attn_bwd(x["q"], x["k"], x["v"], go, wl, x["do"], m1, 1, g, kvb)
    _close(q.grad[0, :, D:2 * D].float().cpu().numpy()[None][:, rows], wq[:, rows], "dQ")
    # dK / dV of two kv blocks: sum over every q-block that lists them, with
    # the GPU's own O and lse (both checked above on a sample)
    lse_g = lse[0, 1].cpu().numpy().astype(np.float64)
    delta = (go[0] * x["do"][0]).sum(-1)
    scale = D ** -0.5
    for j in (3, 800):
        tok = slice(j * kvb, (j + 1) * kvb)
        users = np.nonzero((mg[0, 1] == j).any(-1))[0]
        dk = np.zeros((kvb, D))
        dv = np.zeros((kvb, D))
        for m in users:
            r = slice(m * g, (m + 1) * g)
            s = (x["q"][0, r] * scale) @ x["k"][0, tok].T
            p = np.exp(s - lse_g[r, None])
            dp = x["do"][0, r] @ x["v"][0, tok].T
            ds = p * (dp - delta[r, None])
            dk += scale * ds.T @ x["q"][0, r]
            dv += p.T @ x["do"][0, r]
        _close(k.grad[0, tok, D:2 * D].float().cpu().numpy(), dk, f"dK block {j}")
        _close(v.grad[0, tok, D:2 * D].float().cpu().numpy(), dv, f"dV block {j}")


def test_config2_first_generation_union_and_attention(ftk):
    """The first-generation chain at B=1 N=32768 H=32 D=128 bf16: threshold-free
    scoring, exact union, attention over the union lists.  Whole-output
    properties (every rank filled, lists strictly ascending with a -1 tail of
    the right length, every picked block present in its q-block's list) plus
    sampled q-blocks against the oracle."""
    import flash_topk_attn as v1
    cfg = cases.BASELINE_CONFIGS[2]
    t = cases.make_inputs(dict(cfg, B=1))
    H, D, b, K, N = cfg["H"], cfg["D"], cfg["score_block_size"], cfg["topk"], cfg["N"]
    q, k, v = (t[n].cuda() for n in "qkv")
    idx, scores = v1.flash_topk_score(q, k, num_heads=H, score_block_size=b, topk=K,
                                      score_only=True)
    ftk.check_errors()
    M, g = N // b, 64
    assert idx.shape == (1, H, N, K) and int(idx.min()) >= 0 and int(idx.max()) < M
    assert bool((scores[..., :-1] >= scores[..., 1:]).all())
    merged, counts, width = v1.build_qblock_topk_indices(idx, g)
    ftk.check_errors()
    assert width == 2048 and merged.shape == (1, H, N // g, width)
    slot = torch.arange(width, device="cuda")
    valid = slot < counts.unsqueeze(-1)
    assert bool(((merged >= 0) == valid).all())
    asc = (merged[..., 1:] > merged[..., :-1]) | ~valid[..., 1:]
    assert bool(asc.all())
    # membership: the bitmap of each list equals the bitmap of the picks it came from
    want_bits = torch.zeros(1, H, N // g, M, dtype=torch.bool, device="cuda")
    want_bits.scatter_(3, idx.view(1, H, N // g, g * K).long(), True)
    got_bits = torch.zeros(1, H, N // g, M + 1, dtype=torch.bool, device="cuda")
    got_bits.scatter_(3, torch.where(valid, merged, torch.full_like(merged, M)).long(), True)
    assert torch.equal(got_bits[..., :M], want_bits)
    assert torch.equal(counts.long(), want_bits.sum(-1))

    o, lse = v1.flash_topk_attn(q, k, v, merged, counts, H, g, b)
    ftk.check_errors()
    mh, ch = merged.cpu().numpy(), counts.cpu().numpy()
    for h, m in ((0, 0), (13, 255), (31, 511)):
        rows = slice(m * g, (m + 1) * g)
        q1 = _slice_head(t["q"], 0, h, D)[:, rows]
        k1, v1_ = _slice_head(t["k"], 0, h, D), _slice_head(t["v"], 0, h, D)
        # one q-block on its own: pad the query side so that it is block 0 of a one-block problem
        toks = np.concatenate([np.arange(j * b, (j + 1) * b) for j in mh[0, h, m, :ch[0, h, m]]])
        s = (q1[0] * D ** -0.5) @ k1[0, toks].T
        mx = s.max(1, keepdims=True)
        p = np.exp(s - mx)
        want_o = (p / p.sum(1, keepdims=True)) @ v1_[0, toks]
        want_l = (mx + np.log(p.sum(1, keepdims=True)))[:, 0]
        _close(o[0, rows, h * D:(h + 1) * D].float().cpu().numpy(), want_o, f"o h{h} m{m}")
        _close(lse[0, h, rows].cpu().numpy(), want_l, f"lse h{h} m{m}")
