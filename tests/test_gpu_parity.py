"""GPU parity: the CUDA path (through the Python mirror -> C ABI) against the
CPU oracle and the golden vectors, on the same seeded inputs.

Bars: indices bit-exact except reported near-ties (two block scores closer
than 1e-6 relative in the fp64 arbiter); select / merge / reverse / sort
bit-exact when fed the same fp32 inputs; O, lse, dQ, dK, dV within 2e-3 abs /
1e-2 rel of the fp64 oracle.
"""

import os

import numpy as np
import pytest
import torch

import cases
import tolerance
from oracle import ftk_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def ftk():
    import flash_topk_attn_v2 as m
    return m


def _close(got, want, atol=ATOL, rtol=RTOL, what=""):
    """|got - want| <= atol + rtol |want| for every element."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), f"{what}: finiteness differs"
    assert (got[~fin] == want[~fin]).all(), what
    err = np.abs(got[fin] - want[fin])
    tol = atol + rtol * np.abs(want[fin])
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} bad, max err {float(err.max()):.3e}"


def _check_grads(x, merged, H, g, kvb, dtype, o, grads, qpad=(0, 0), kvpad=(0, 0), kx=None,
                 vx=None, fold=None):
    """dQ, dK, dV against the fp64 oracle.  fp16: the plain bound, every
    element.  bf16: the plain bound plus, per element, what the reference's own
    roundings of P and dS can contribute in the worst case, and a tensor-wide
    error no larger than that recipe's (tests/tolerance.py)."""
    og = o.detach().float().cpu().numpy()
    ora = tolerance.attention_oracles(orc, x, merged, H, g, kvb, "fp16" if dtype == "fp16" else "bf16",
                                      og, qpad, kvpad, kx, vx)
    for nm, t in zip(("dQ", "dK", "dV"), grads):
        got = t.float().cpu().numpy()
        ex, rd, env = (ora[part][nm] for part in ("exact", "rounded", "envelope"))
        if fold is not None and nm != "dQ":
            ex, rd, env = fold(ex), fold(rd), fold(env)
        if dtype == "fp16":
            _close(got, ex, what=nm)
        else:
            tolerance.check_rounded(got, ex, rd, env, nm)


def _inputs(cfg):
    t = cases.make_inputs(cfg)
    return t, {k: v.float().numpy() for k, v in t.items()}


def _gold(name):
    return dict(np.load(os.path.join(GOLD, f"{name}.npz")))


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_block_score_and_topk(ftk, name):
    cfg = cases.GOLDEN_CASES[name]
    t, x = _inputs(cfg)
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    q, k = t["q"].cuda(), t["k"].cuda()
    want = orc.block_score(x["q"], x["k"], H, b, pad, work=np.float64)

    got = ftk.flash_block_score(q, k, H, b, pad).cpu().numpy()
    ftk.check_errors()
    np.testing.assert_allclose(got.sum(-1), 1.0, atol=2e-6)
    np.testing.assert_allclose(got, want, rtol=3e-6, atol=1e-9)

    # [B,H,N,D] layout goes through the same kernels in place
    B, N = cfg["B"], cfg["N"]
    q4 = q.view(B, N, H, -1).permute(0, 2, 1, 3).contiguous()
    k4 = k.view(B, N, H, -1).permute(0, 2, 1, 3).contiguous()
    got4 = ftk.flash_block_score(q4, k4, H, b, pad).cpu().numpy()
    np.testing.assert_array_equal(got4, got)

    idx, raw, avg = ftk.flash_topk_score(q, k, H, b, cfg["topk"], pad, cfg["threshold"])
    ftk.check_errors()
    oi, oraw, oavg, _ = orc.flash_topk_score(
        x["q"], x["k"], H, b, cfg["topk"], pad, cfg["threshold"])
    _, _, _, valid = orc.block_geometry(cfg["N"], b, pad)
    rep = orc.classify_topk_mismatches(idx.cpu().numpy(), oi, want / valid, rel_band=1e-6)
    assert rep["hard"] == 0, rep
    same = idx.cpu().numpy() == oi
    np.testing.assert_allclose(raw.cpu().numpy()[same], oraw[same], rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(avg.cpu().numpy()[same], oavg[same], rtol=1e-5, atol=1e-10)
    assert idx.dtype == torch.int32 and raw.dtype == torch.float32
    assert tuple(idx.shape) == oi.shape


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_select_merge_reverse_exact(ftk, name):
    cfg = cases.GOLDEN_CASES[name]
    gold = _gold(name)
    b, pad = cfg["score_block_size"], tuple(cfg["padding"])
    if not cfg.get("drop_block_scores"):
        scores = torch.from_numpy(gold["block_scores"]).cuda()
        for thr, k in ((cfg["threshold"], cfg["topk"]), (1.0, 0), (0.3, 2)):
            gi, gr, ga = ftk.flash_topk_select(scores, thr, k, b, pad)
            oi, orw, oa = orc.topk_select(gold["block_scores"], thr, k, b, pad)
            np.testing.assert_array_equal(gi.cpu().numpy(), oi)
            np.testing.assert_array_equal(gr.cpu().numpy(), orw)
            np.testing.assert_array_equal(ga.cpu().numpy(), oa)

    # merge from the oracle's own per-query lists (bit-exact incl. scores)
    t, x = _inputs(cfg)
    H = cfg["H"]
    s32 = orc.block_score(x["q"], x["k"], H, b, pad, work=np.float32).astype(np.float32)
    ti, _, ta = orc.topk_select(s32, cfg["threshold"], cfg["topk"], b, pad)
    w = ta if cfg["score_weighted"] else None
    om, oc, W, oms = orc.build_qblock_topk_indices(
        ti, cfg["q_block_size"], tuple(cfg["q_padding"]), w, cfg["qblock_topk"])
    gm, gc, gW = ftk.build_qblock_topk_indices(
        torch.from_numpy(ti).cuda(), cfg["q_block_size"], tuple(cfg["q_padding"]),
        None if w is None else torch.from_numpy(w).cuda(), cfg["qblock_topk"])
    ftk.check_errors()
    assert gW == W and gm.dtype == torch.int32 and gc.dtype == torch.int32
    np.testing.assert_array_equal(gm.cpu().numpy(), om)
    np.testing.assert_array_equal(gc.cpu().numpy(), oc)

    M = (cfg["kv_padding"][0] + cfg["N"] + cfg["kv_padding"][1]) // cfg["kv_block_size"]
    rev, rc, skv = ftk.flash_build_reverse_indices_cuda(gm, gc, M)
    orev, orc_, oskv = orc.build_reverse_indices(om, oc, M)
    np.testing.assert_array_equal(rev.cpu().numpy(), orev)
    np.testing.assert_array_equal(rc.cpu().numpy(), orc_)
    np.testing.assert_array_equal(skv.cpu().numpy(), oskv)
    sc, ids = ftk.flash_sort_by_count_cuda(rc, H, M)
    osc, oids = orc.sort_by_count(orc_)
    np.testing.assert_array_equal(sc.cpu().numpy(), osc)
    np.testing.assert_array_equal(ids.cpu().numpy(), oids)


@pytest.mark.parametrize("M", [33, 40, 64, 100, 257, 512, 1000, 1024, 1500])
def test_select_paths_exact(ftk, M):
    """Every select path (filter-and-sort for up to 32 and up to 64 picks with 32 to
    256 candidates, the extraction loop behind it, the shared-memory kernel above
    M = 1024) against
    the oracle: smooth rows, rows with many exact ties, rows whose threshold
    cuts early, padded first/last blocks, flat rows (all candidates tie)."""
    rng = np.random.default_rng(1000 + M)
    rows = 96
    x = rng.random((1, 2, rows, M), dtype=np.float32) ** 4
    x[0, 0, :32] = np.round(x[0, 0, :32] * 8) / 8           # heavy ties
    x[0, 0, 32:40] = 0.25                                    # flat: everything ties
    x[0, 1, :16, :3] += 50.0                                 # early cut
    x[0, 1, 16:24, ::7] = 0.0
    x /= x.sum(-1, keepdims=True)
    scores = torch.from_numpy(x).cuda()
    for b, pad in ((64, (0, 0)), (48, (5, 47))):
        for thr, k in ((0.9, 32), (0.5, 8), (0.2, 1), (1.5, 17), (0.9, 0), (0.05, 40), (1.5, 64),
                       (0.6, 48), (1.5, 33)):
            gi, gr, ga = ftk.flash_topk_select(scores, thr, k, b, pad)
            oi, orw, oa = orc.topk_select(x, thr, k, b, pad)
            np.testing.assert_array_equal(gi.cpu().numpy(), oi, err_msg=f"{M} {b} {thr} {k}")
            np.testing.assert_array_equal(gr.cpu().numpy(), orw)
            np.testing.assert_array_equal(ga.cpu().numpy(), oa)
    ftk.check_errors()


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_attention_fwd_bwd(ftk, name):
    cfg = cases.GOLDEN_CASES[name]
    gold = _gold(name)
    t, x = _inputs(cfg)
    H, g, kvb = cfg["H"], cfg["q_block_size"], cfg["kv_block_size"]
    qpad, kvpad = tuple(cfg["q_padding"]), tuple(cfg["kv_padding"])
    merged = gold["merged"].astype(np.int32)
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    counts = torch.from_numpy((merged >= 0).sum(-1).astype(np.int32)).cuda()
    o, lse = ftk.flash_topk_attn(
        q, k, v, torch.from_numpy(merged).cuda(), counts, H, g, kvb,
        kv_padding=kvpad, q_padding=qpad)
    ftk.check_errors()
    assert o.dtype == q.dtype and lse.dtype == torch.float32
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    s = cfg.get("store_row_stride", 1)
    _close(o.detach().float().cpu().numpy()[:, ::s], gold["o_diff"], what="O vs golden")

    o.backward(t["do"].cuda())
    ftk.check_errors()
    o_rounded = o.detach().float().cpu().numpy()
    wq, wk, wv = orc.sparse_attn_bwd(
        x["q"], x["k"], x["v"], o_rounded, wl, x["do"], merged, H, g, kvb, None, qpad, kvpad)
    _close(q.grad.float().cpu().numpy(), wq, what="dQ")
    _close(k.grad.float().cpu().numpy(), wk, what="dK")
    _close(v.grad.float().cpu().numpy(), wv, what="dV")
    _close(q.grad.float().cpu().numpy()[:, ::s], gold["dq"], what="dQ vs golden")
    _close(k.grad.float().cpu().numpy()[:, ::s], gold["dk"], what="dK vs golden")
    _close(v.grad.float().cpu().numpy()[:, ::s], gold["dv"], what="dV vs golden")


@pytest.mark.parametrize("D", [64, 128])
def test_attention_empty_and_partial_lists(ftk, D):
    """q-blocks with no candidates give O = 0, lse = -inf and zero gradients;
    neighbours with different lists share a tile without leaking (head dim 128
    takes the dK/dV kernel that runs on pairs of SMs)."""
    cfg = dict(B=1, N=256, H=2, D=D, dtype="bf16", seed=3, do_seed=4)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    g, kvb, QM, M = 64, 64, 4, 4
    merged = np.full((1, 2, QM, 4), -1, dtype=np.int32)
    merged[0, 0, 0, :2] = [3, 0]
    merged[0, 0, 1, :1] = [1]          # same tile as q-block 0, different list
    merged[0, 0, 3, :4] = [2, 0, 1, 3]
    merged[0, 1, 2, :1] = [2]          # head 1: only q-block 2 attends
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, 2, g, kvb)
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, 2, g, kvb)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    assert torch.isinf(lse[0, 0, 128:192]).all() and (o[0, 128:192, :D] == 0).all()
    o.backward(t["do"].cuda())
    ftk.check_errors()
    wq, wk, wv = orc.sparse_attn_bwd(
        x["q"], x["k"], x["v"], o.detach().float().cpu().numpy(), wl, x["do"], merged, 2, g, kvb)
    _close(q.grad.float().cpu().numpy(), wq, what="dQ")
    _close(k.grad.float().cpu().numpy(), wk, what="dK")
    _close(v.grad.float().cpu().numpy(), wv, what="dV")


def _random_lists(rng, BH, QM, M, width, empty_every=5):
    merged = np.full((BH, QM, width), -1, dtype=np.int32)
    for i in range(BH):
        for m in range(QM):
            if (i + m) % empty_every == empty_every - 1:
                continue
            c = int(rng.integers(1, min(width, M) + 1))
            merged[i, m, :c] = rng.permutation(M)[:c]
    return merged


@pytest.mark.parametrize("g,D,N,qpad,kvpad,dtype", [
    (64, 128, 1000, (24, 0), (20, 4), "bf16"),
    (64, 128, 1024, (0, 0), (0, 0), "bf16"),
    (64, 64, 777, (0, 55), (0, 55), "bf16"),
    (64, 128, 1000, (24, 0), (20, 4), "fp16"),
    (64, 64, 777, (0, 55), (0, 55), "fp16"),
])
def test_fwd_pipelined_kernel(ftk, g, D, N, qpad, kvpad, dtype, monkeypatch):
    """64-row q and kv blocks take the pipelined forward kernel (fixed
    reference exponent, four tiles in flight; on pairs of SMs at head dim
    128).  Ragged lengths, virtual padding, empty and unequal neighbouring
    lists against the oracle, and against the exact kernel alone
    (FTK_FWD_PIPE=0)."""
    H, kvb = 3, 64
    cfg = dict(B=2, N=N, H=H, D=D, dtype=dtype, seed=11, do_seed=12)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    QM = (qpad[0] + N + qpad[1]) // g
    M = (kvpad[0] + N + kvpad[1]) // kvb
    merged = _random_lists(np.random.default_rng(5), 2 * H, QM, M, 12).reshape(2, H, QM, 12)
    args = (t["q"].cuda(), t["k"].cuda(), t["v"].cuda(), torch.from_numpy(merged).cuda(), None,
            H, g, kvb)
    o, lse = ftk.flash_topk_attn(*args, kv_padding=kvpad, q_padding=qpad)
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o.float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    monkeypatch.setenv("FTK_FWD_PIPE", "0")
    o2, lse2 = ftk.flash_topk_attn(*args, kv_padding=kvpad, q_padding=qpad)
    ftk.check_errors()
    _close(o.float().cpu().numpy(), o2.float().cpu().numpy(), what="O pipelined vs exact")
    _close(lse.cpu().numpy(), lse2.cpu().numpy(), atol=1e-4, rtol=1e-5, what="lse vs exact")


@pytest.mark.parametrize("g,kvb,D,dtype", [
    (16, 16, 64, "fp16"),
    (48, 48, 128, "fp16"),
    (32, 32, 32, "bf16"),     # head dim padded to 64 by the host layer
    (64, 64, 96, "bf16"),     # head dim padded to 128, pipelined forward
    (64, 64, 128, "fp32"),    # fp32 in, computed in bf16, fp32 out
    (32, 64, 128, "bf16"),    # four q-blocks per tile: exact forward kernel
])
def test_attention_block_shapes(ftk, g, kvb, D, dtype):
    """Block sizes other than 64, head dims that need padding and fp32 inputs,
    forward and backward against the oracle."""
    H, N = 2, 384
    cfg = dict(B=1, N=N, H=H, D=D, dtype="bf16" if dtype == "fp32" else dtype, seed=31, do_seed=32)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    if dtype == "fp32":
        t = {k: v.float() for k, v in t.items()}       # values already bf16-representable
    QM, M = N // g, N // kvb
    merged = _random_lists(np.random.default_rng(9), H, QM, M, 5, empty_every=7).reshape(1, H, QM, 5)
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, H, g, kvb)
    ftk.check_errors()
    assert o.dtype == q.dtype and o.shape == q.shape
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    o.backward(t["do"].cuda())
    ftk.check_errors()
    # with fp32 inputs the kernels saw bf16 O (o is the bf16 result widened back)
    _check_grads(x, merged, H, g, kvb, dtype, o, (q.grad, k.grad, v.grad))


@pytest.mark.parametrize("g,kvb,qpad,kvpad,dtype", [
    (128, 128, (70, 82), (100, 52), "bf16"),
    (128, 64, (10, 14), (8, 16), "fp16"),
    (64, 128, (24, 0), (0, 24), "bf16"),
    (96, 96, (20, 36), (50, 6), "fp16"),
])
def test_attention_blocks_up_to_128(ftk, g, kvb, qpad, kvpad, dtype):
    """q / kv blocks above 64 rows (the reference rejects q blocks above 64 and
    its dK/dV breaks for kv blocks above 64): forward and backward against the
    oracle, with pad heads on either side of half a block."""
    H, N, D = 2, 1000, 128
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=41, do_seed=42)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    QM, M = (qpad[0] + N + qpad[1]) // g, (kvpad[0] + N + kvpad[1]) // kvb
    merged = _random_lists(np.random.default_rng(13), H, QM, M, 4, empty_every=6).reshape(1, H, QM, 4)
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, H, g, kvb,
                                 kv_padding=kvpad, q_padding=qpad)
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    o.backward(t["do"].cuda())
    ftk.check_errors()
    _check_grads(x, merged, H, g, kvb, dtype, o, (q.grad, k.grad, v.grad), qpad, kvpad)


def test_pair_kernels_agree_with_one_cta_kernels(ftk, monkeypatch):
    """Head dim 128 with 64-row blocks runs on pairs of SMs (cta_group::2); the
    one-CTA kernels (FTK_FWD_2CTA / FTK_DQ_2CTA / FTK_DKV_2CTA = 0) serve every
    other shape.  Same inputs through both: the backward kernels do the same
    arithmetic per element, the forward differs only in rounding order."""
    H, N, D, g, kvb = 3, 1000, 128, 64, 64
    cfg = dict(B=2, N=N, H=H, D=D, dtype="bf16", seed=51, do_seed=52)
    t = cases.make_inputs(cfg)
    qpad, kvpad = (24, 0), (20, 4)
    QM, M = (qpad[0] + N) // g, (kvpad[0] + N + kvpad[1]) // kvb
    merged = _random_lists(np.random.default_rng(17), 2 * H, QM, M, 9).reshape(2, H, QM, 9)
    mg = torch.from_numpy(merged).cuda()

    def run():
        q = t["q"].cuda().requires_grad_(True)
        k = t["k"].cuda().requires_grad_(True)
        v = t["v"].cuda().requires_grad_(True)
        o, lse = ftk.flash_topk_attn(q, k, v, mg, None, H, g, kvb, kv_padding=kvpad,
                                     q_padding=qpad)
        o.backward(t["do"].cuda())
        ftk.check_errors()
        return [x.detach().float().cpu().numpy() for x in (o, lse, q.grad, k.grad, v.grad)]

    pair = run()
    for name in ("FTK_FWD_2CTA", "FTK_DQ_2CTA", "FTK_DKV_2CTA"):
        monkeypatch.setenv(name, "0")
    single = run()
    for a, b, what in zip(pair, single, ("O", "lse", "dQ", "dK", "dV")):
        _close(a, b, what=f"{what}: pair vs one-CTA kernel")


@pytest.mark.parametrize("D,g,dtype", [(128, 64, "bf16"), (64, 32, "fp16")])
def test_grouped_query_attention(ftk, D, g, dtype):
    """num_kv_heads < num_heads (the reference raises NotImplementedError):
    query head h reads kv head h // group.  The oracle sees K and V repeated
    per query head; its dK / dV are summed over each group."""
    H, Hkv, N, kvb = 4, 2, 512, 64
    grp = H // Hkv
    gen = torch.Generator().manual_seed(71)
    dt = torch.bfloat16 if dtype == "bf16" else torch.float16
    q = (torch.randn(1, N, H * D, generator=gen)).to(dt)
    k = (torch.randn(1, N, Hkv * D, generator=gen)).to(dt)
    v = (torch.randn(1, N, Hkv * D, generator=gen)).to(dt)
    do = (torch.randn(1, N, H * D, generator=gen)).to(dt)
    QM, M = N // g, N // kvb
    merged = _random_lists(np.random.default_rng(19), H, QM, M, 6, empty_every=9).reshape(1, H, QM, 6)
    qg = q.cuda().requires_grad_(True)
    kg = k.cuda().requires_grad_(True)
    vg = v.cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(qg, kg, vg, torch.from_numpy(merged).cuda(), None, H, g, kvb,
                                 num_kv_heads=Hkv)
    o.backward(do.cuda())
    ftk.check_errors()
    assert kg.grad.shape == k.shape and vg.grad.shape == v.shape

    def rep(t):   # [1, N, Hkv*D] -> [1, N, H*D], kv head of query head h = h // grp
        return t.float().view(1, N, Hkv, 1, D).expand(1, N, Hkv, grp, D).reshape(1, N, H * D).numpy()

    xq, xk, xv, xdo = q.float().numpy(), rep(k), rep(v), do.float().numpy()
    wo, wl = orc.sparse_attn_fwd(xq, xk, xv, merged, H, g, kvb)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    # each query head's dK / dV share is rounded to 16 bits before the group is added
    # up; the reference-rounded oracle does the same (it rounds per query head)
    fold = lambda a: a.reshape(1, N, Hkv, grp, D).sum(3).reshape(1, N, Hkv * D)
    _check_grads(dict(q=xq, do=xdo), merged, H, g, kvb, dtype, o, (qg.grad, kg.grad, vg.grad),
                 kx=xk, vx=xv, fold=fold)


@pytest.mark.parametrize("dtype,kscale", [("bf16", 30.0), ("fp16", 4.0)])
def test_fwd_pipelined_redo_on_exponent_range(ftk, monkeypatch, dtype, kscale):
    """Later blocks beat a row's first block by more than the format allows
    (2^80 for bf16, 2^15 for fp16): the pipelined kernel flags those tiles and
    the exact kernel redoes them, so the flagged tiles equal the exact
    kernel's output bit for bit."""
    H, g, kvb, N, D = 2, 64, 64, 512, 128
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=21, do_seed=22)
    t = cases.make_inputs(cfg)
    t["k"][:, 256:] *= kscale           # logits of blocks 4..7 leave the safe range
    t["q"] *= 2.0
    x = {k: v.float().numpy() for k, v in t.items()}
    QM = M = N // 64
    merged = np.tile(np.arange(M, dtype=np.int32), (1, H, QM, 1))
    merged[0, 1, :4, 4:] = -1           # head 1, first two tiles: only the tame blocks
    args = (t["q"].cuda(), t["k"].cuda(), t["v"].cuda(), torch.from_numpy(merged).cuda(), None,
            H, g, kvb)
    o, lse = ftk.flash_topk_attn(*args)
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb)
    assert np.abs(wl).max() > (100.0 if dtype == "bf16" else 20.0)
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    # one-hot softmax rows: the error is the bf16 rounding of two competing P
    _close(o.float().cpu().numpy(), wo, atol=2e-2, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    monkeypatch.setenv("FTK_FWD_PIPE", "0")
    o2, lse2 = ftk.flash_topk_attn(*args)
    wild = np.ones((H, N), dtype=bool)
    wild[1, :256] = False
    wild = torch.from_numpy(wild).cuda()
    o4, o24 = o.view(1, N, H, D).permute(0, 2, 1, 3)[0], o2.view(1, N, H, D).permute(0, 2, 1, 3)[0]
    assert torch.equal(o4[wild], o24[wild]) and torch.equal(lse[0][wild], lse2[0][wild])
    _close(o.float().cpu().numpy(), o2.float().cpu().numpy(), what="O vs exact")


def test_pair_kernels_with_empty_pairs(ftk):
    """Head dim 128, 64-row blocks, N = 512: eight q-blocks = two CTA pairs.
    Head 0: the second pair's q-blocks list nothing (forward / dQ pair with no
    work) and nobody lists kv blocks 4..7 (dK/dV pair with no work); head 1:
    only one q-block of each pair attends."""
    H, N, D, g, kvb = 2, 512, 128, 64, 64
    cfg = dict(B=1, N=N, H=H, D=D, dtype="bf16", seed=61, do_seed=62)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    QM = M = 8
    merged = np.full((1, H, QM, 8), -1, dtype=np.int32)
    merged[0, 0, :4, :4] = [[0, 1, 2, 3], [3, 1, 0, 2], [2, 0, 3, 1], [1, 3, 2, 0]]
    merged[0, 1, 1, :3] = [7, 0, 4]
    merged[0, 1, 6, :2] = [5, 2]
    q = t["q"].cuda().requires_grad_(True)
    k = t["k"].cuda().requires_grad_(True)
    v = t["v"].cuda().requires_grad_(True)
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, H, g, kvb)
    o.backward(t["do"].cuda())
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb)
    _close(o.detach().float().cpu().numpy(), wo, what="O")
    _close(lse.cpu().numpy(), wl, what="lse")
    assert torch.isinf(lse[0, 0, 256:]).all() and (o[0, 256:, :D] == 0).all()
    _check_grads(x, merged, H, g, kvb, "bf16", o, (q.grad, k.grad, v.grad))
    assert (k.grad[0, 256:, :D] == 0).all() and (v.grad[0, 256:, :D] == 0).all()


def test_score_overflow_fallback(ftk):
    """Logits far above the first key tile's maximum overflow the single-pass
    sums; the exact two-pass fallback must take over."""
    g = torch.Generator().manual_seed(7)
    B, N, H, D = 1, 512, 1, 64
    q = torch.randn(B, N, H * D, generator=g)
    k = torch.randn(B, N, H * D, generator=g)
    k[:, 300:] *= 40.0                  # later tiles dominate by hundreds of nats
    q *= 3.0
    qh, kh = q.half(), k.half()
    want = orc.block_score(qh.float().numpy(), kh.float().numpy(), H, 64, (0, 0))
    got = ftk.flash_block_score(qh.cuda(), kh.cuda(), H, 64).cpu().numpy()
    ftk.check_errors()
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=1e-7)


def test_error_codes_through_c_abi(ftk):
    """The C entry points validate before launching anything."""
    from flash_topk_attn_v2 import _lib
    lib = _lib.lib
    x = torch.zeros(1, 128, 64, dtype=torch.float16, device="cuda")
    ws = torch.empty(lib.ftk_block_score_workspace(1, 128), dtype=torch.uint8, device="cuda")
    out = torch.empty(1, 1, 128, 2, device="cuda")
    args = lambda bsz, D, wsz: (x.data_ptr(), x.data_ptr(), 0, 1, 1, 128, D, 128 * 64, 64, 64,
                                128 * 64, 64, 64, 0, 1, bsz, 0, 0, 0.125, out.data_ptr(),
                                ws.data_ptr(), wsz, 0, 0)
    assert lib.ftk_block_score(*args(64, 64, ws.numel())) == 0
    assert lib.ftk_block_score(*args(48, 64, ws.numel())) == -1      # 128 % 48 != 0
    assert lib.ftk_block_score(*args(8, 64, ws.numel())) == -2       # block size not /16
    assert lib.ftk_block_score(*args(64, 96, ws.numel())) == -2      # head dim
    assert lib.ftk_block_score(*args(64, 64, 16)) == -3              # workspace
    torch.cuda.synchronize()
    with pytest.raises(ValueError):
        ftk.flash_topk_score(x, x)                                   # num_heads missing
    with pytest.raises(ValueError):
        ftk.flash_topk_score(x, x, 1, 64, 16, (64, 0))
    with pytest.raises(ValueError, match="multiple of num_kv_heads"):
        ftk.flash_topk_attn(x, x, x, None, None, 1, 64, 64, num_kv_heads=2)
    with pytest.raises(ValueError):
        ftk.build_qblock_topk_indices(torch.zeros(1, 1, 100, 4, dtype=torch.int32).cuda(), 64)


def test_whole_chain_replays_from_a_cuda_graph(ftk):
    """score -> merge -> attention -> backward issues no host synchronisation
    and keeps no state between calls, so the chain can be captured once and
    replayed on new data: replayed results equal the eager ones bit for bit."""
    B, N, H, D, b, g = 1, 1024, 2, 128, 64, 64
    gen = torch.Generator().manual_seed(77)
    data = [[torch.randn(B, N, H * D, generator=gen).bfloat16() for _ in range(4)]
            for _ in range(2)]
    q, k, v = (x.cuda().requires_grad_(True) for x in data[0][:3])
    do = data[0][3].cuda()

    def chain():
        idx, raw, avg = ftk.flash_topk_score(q, k, H, b, 4, (0, 0), 0.9)
        merged, counts, _ = ftk.build_qblock_topk_indices(idx, g, topk_scores=avg)
        o, lse = ftk.flash_topk_attn(q, k, v, merged, counts, H, g, b)
        gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
        return idx, merged, o.detach(), lse, gq, gk, gv

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            chain()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = chain()
    for tensors in (data[1], data[0]):
        with torch.no_grad():
            for dst, src in zip((q, k, v, do), tensors):
                dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        replayed = [t.clone() for t in captured]
        eager = chain()
        ftk.check_errors()
        for name, a, e in zip(("idx", "merged", "o", "lse", "dq", "dk", "dv"), replayed, eager):
            assert torch.equal(a, e), name


def test_dkv_tiles_in_fan_in_order_equal_block_order(ftk, monkeypatch):
    """With short lists dK/dV runs one CTA per tile of kv blocks, heaviest tiles
    first (the order build_reverse sorted by fan-in; FTK_DKV_ORDER=0 issues them
    in block order instead).  The order decides when a tile runs, never what it
    computes: gradients are bit-identical.  Lists: a few hot kv blocks that every
    q-block names plus random ones, so fan-in is skewed."""
    H, N, D, g, kvb, W = 2, 2048, 128, 64, 64, 6
    t = cases.make_inputs(dict(B=1, N=N, H=H, D=D, dtype="bf16", seed=95, do_seed=96))
    rng = np.random.default_rng(23)
    QM = M = N // 64
    merged = np.full((1, H, QM, W), -1, dtype=np.int32)
    for h in range(H):
        hot = rng.permutation(M)[:2]
        for m in range(QM):
            rest = [j for j in rng.permutation(M)[:W] if j not in set(hot)][:W - 2]
            merged[0, h, m, :2] = hot
            merged[0, h, m, 2:2 + len(rest)] = rest
    mg = torch.from_numpy(merged).cuda()

    def run():
        q, k, v = (t[n].cuda().requires_grad_(True) for n in "qkv")
        o, _ = ftk.flash_topk_attn(q, k, v, mg, None, H, g, kvb)
        o.backward(t["do"].cuda())
        ftk.check_errors()
        return k.grad.clone(), v.grad.clone()

    by_fan_in = run()
    monkeypatch.setenv("FTK_DKV_ORDER", "0")
    by_block = run()
    assert torch.equal(by_fan_in[0], by_block[0]) and torch.equal(by_fan_in[1], by_block[1])
    x = {n: v.float().numpy() for n, v in t.items()}
    q, k, v = (t[n].cuda().requires_grad_(True) for n in "qkv")
    o, _ = ftk.flash_topk_attn(q, k, v, mg, None, H, g, kvb)
    o.backward(t["do"].cuda())
    _check_grads(x, merged, H, g, kvb, "bf16", o, (q.grad, k.grad, v.grad))


def test_scoring_in_chunks_of_slices_equals_one_call(ftk, monkeypatch):
    """When the block sums of all (batch, head) slices exceed the scratch budget
    (4 GiB by default: config 5 needs 17 GB per batch element) the host layer scores
    the slices in chunks.  Forced here with a tiny budget: three chunks, same bits."""
    from flash_topk_attn_v2 import ops
    cfg = dict(B=2, N=640, H=3, D=128, dtype="bf16", seed=97, do_seed=98)
    t = cases.make_inputs(cfg)
    q, k = t["q"].cuda(), t["k"].cuda()
    one = ftk.flash_topk_score(q, k, 3, 64, 4, (0, 0), 0.9)
    per_slice = ops.lib.ftk_score_topk_workspace(1, 640, 10)
    monkeypatch.setattr(ops, "_SCORE_SCRATCH_BYTES", 2 * per_slice + 64)
    calls = []
    real = ops._call

    def counting(name, fn, *a):
        calls.append(name)
        return real(name, fn, *a)

    monkeypatch.setattr(ops, "_call", counting)
    chunked = ftk.flash_topk_score(q, k, 3, 64, 4, (0, 0), 0.9)
    ftk.check_errors()
    assert calls.count("ftk_score_topk") == 3          # 6 slices, 2 per chunk
    for a, b in zip(one, chunked):
        assert torch.equal(a, b)
