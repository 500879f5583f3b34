"""The CPU restatement (oracle/) against outputs of the reference's own code.

The .npz files under tests/golden/ were produced by tests/golden/make_golden.py
from the reference's `_naive` PyTorch functions; inputs are rebuilt here from
the same seeds.  Integer results must match exactly (up to reported near-ties
of fp32-vs-fp64 block scores); floating-point results within 2e-3 abs /
1e-2 rel, the tolerance the path is specified to.
"""

import os

import numpy as np
import pytest
import torch

import cases
from oracle import ftk_oracle as orc

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL, RTOL = 2e-3, 1e-2


def _np_inputs(cfg):
    t = cases.make_inputs(cfg)
    return {k: v.float().numpy() for k, v in t.items()}


def _load(name):
    return dict(np.load(os.path.join(GOLD, f"{name}.npz")))


def _close(a, b, atol=ATOL, rtol=RTOL):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    fin = np.isfinite(b)
    assert (np.isfinite(a) == fin).all()
    assert (a[~fin] == b[~fin]).all()
    err = np.abs(a[fin] - b[fin])
    assert (err <= atol + rtol * np.abs(b[fin])).all(), float(err.max())


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_score_select_merge(name):
    cfg = cases.GOLDEN_CASES[name]
    gold = _load(name)
    x = _np_inputs(cfg)
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    scores = orc.block_score(x["q"], x["k"], H, b, pad, work=np.float64)
    np.testing.assert_allclose(scores.sum(-1), 1.0, atol=1e-12)
    stride = cfg.get("drop_block_scores") or 1
    np.testing.assert_allclose(
        scores[:, :, ::stride], gold["block_scores"], rtol=2e-5, atol=1e-7
    )

    # select: same fp32 scores in -> bit-exact out (ties: lower id first;
    # the golden came from torch.sort whose tie order is unspecified, so a
    # differing position must be an exact tie of the fp32 averages).
    if stride == 1:
        idx, raw, avg = orc.topk_select(
            gold["block_scores"], cfg["threshold"], cfg["topk"], b, pad
        )
        gi = gold["topk_idx"].astype(np.int32)
        diff = idx != gi
        if diff.any():
            np.testing.assert_array_equal(avg[diff], gold["topk_avg"][diff])
        np.testing.assert_array_equal(raw, gold["topk_raw"])
        np.testing.assert_array_equal(avg, gold["topk_avg"])

    # full chain from fp64 scores: indices equal up to near-ties.
    idx64, raw64, avg64, _ = orc.flash_topk_score(
        x["q"], x["k"], H, b, cfg["topk"], pad, cfg["threshold"]
    )
    _, _, _, valid = orc.block_geometry(cfg["N"], b, pad)
    rep = orc.classify_topk_mismatches(
        idx64, gold["topk_idx"].astype(np.int32), scores / valid, rel_band=1e-5
    )
    assert rep["hard"] == 0, rep

    # merge from the golden per-query lists -> bit-exact.
    weights = None
    if cfg["score_weighted"]:
        if stride != 1:
            # scores were stored on a stride; recompute them with the oracle
            _, _, weights = orc.topk_select(
                orc.block_score(x["q"], x["k"], H, b, pad, work=np.float32)
                .astype(np.float32), cfg["threshold"], cfg["topk"], b, pad)
            np.testing.assert_allclose(
                weights[:, :, ::stride], gold["topk_avg"], rtol=1e-4, atol=1e-9)
        else:
            weights = gold["topk_avg"]
    merged, counts, W, mscores = orc.build_qblock_topk_indices(
        gold["topk_idx"].astype(np.int32), cfg["q_block_size"],
        tuple(cfg["q_padding"]), weights, cfg["qblock_topk"],
    )
    gm = gold["merged"].astype(np.int32)
    assert W == gm.shape[-1]
    if stride == 1:
        diff = merged != gm
        if diff.any():  # only exact ties of the aggregated fp32 scores
            np.testing.assert_array_equal(
                mscores[diff], gold["merged_scores"][diff])
        np.testing.assert_array_equal(counts, gold["counts"])
        np.testing.assert_array_equal(mscores, gold["merged_scores"])
    else:
        np.testing.assert_array_equal(counts, gold["counts"])
        np.testing.assert_array_equal(np.sort(merged, -1), np.sort(gm, -1))


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_attention_fwd_bwd(name):
    cfg = cases.GOLDEN_CASES[name]
    gold = _load(name)
    x = _np_inputs(cfg)
    H, g, kvb = cfg["H"], cfg["q_block_size"], cfg["kv_block_size"]
    qpad, kvpad = tuple(cfg["q_padding"]), tuple(cfg["kv_padding"])
    merged = gold["merged"].astype(np.int32)
    s = cfg.get("store_row_stride", 1)
    o, lse = orc.sparse_attn_fwd(
        x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o[:, ::s], gold["o_diff"], atol=1e-5, rtol=1e-4)
    _close(o[:, ::s], gold["o"])          # stored in the I/O dtype
    _close(lse[:, :, ::s], gold["lse"], atol=1e-4, rtol=1e-5)
    dq, dk, dv = orc.sparse_attn_bwd(
        x["q"], x["k"], x["v"], o, lse, x["do"], merged, H, g, kvb, None,
        qpad, kvpad)
    _close(dq[:, ::s], gold["dq"], atol=2e-5, rtol=1e-4)
    _close(dk[:, ::s], gold["dk"], atol=2e-5, rtol=1e-4)
    _close(dv[:, ::s], gold["dv"], atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("name", list(cases.GOLDEN_CASES))
def test_reverse_and_sort(name):
    cfg = cases.GOLDEN_CASES[name]
    gold = _load(name)
    merged = gold["merged"].astype(np.int32)
    M = gold["reverse_counts"].shape[-1]
    rev, rc, order = orc.build_reverse_indices(merged, gold["counts"], M)
    np.testing.assert_array_equal(rc, gold["reverse_counts"])
    np.testing.assert_array_equal(rev, gold["reverse_indices"].astype(np.int32))
    sc, ids = orc.sort_by_count(rc)
    np.testing.assert_array_equal(sc, gold["sorted_counts"])
    assert (np.diff(sc) <= 0).all()
    np.testing.assert_array_equal(rc.reshape(-1)[ids], sc)
    # per-(b,h) order is descending by count, ascending id on ties
    cnt = np.take_along_axis(rc, order.astype(np.int64), -1)
    assert (np.diff(cnt, axis=-1) <= 0).all()


def test_select_edge_cases():
    # threshold reached exactly at a position (inclusive cut), topk = 0 => M
    s = np.array([[[[0.5, 0.25, 0.125, 0.125]]]], dtype=np.float32)
    idx, raw, avg = orc.topk_select(s, 0.75, 0, 64)
    assert idx.tolist() == [[[[0, 1, -1, -1]]]]
    assert raw.tolist() == [[[[0.5, 0.25, 0.0, 0.0]]]]
    # never reached -> keep everything up to the cap
    idx, _, _ = orc.topk_select(s, 2.0, 3, 64)
    assert idx.tolist() == [[[[0, 1, 2]]]]
    # ties keep the lower block id first
    idx, _, _ = orc.topk_select(s, 2.0, 4, 64)
    assert idx.tolist() == [[[[0, 1, 2, 3]]]]
    # head padding changes the averaging of block 0 only
    idx, raw, avg = orc.topk_select(s, 2.0, 1, 64, padding=(60, 0))
    assert idx.tolist() == [[[[0]]]] and avg[0, 0, 0, 0] == np.float32(0.5) / np.float32(4)
    with pytest.raises(ValueError):
        orc.topk_select(s, 1.0, -1, 64)
    with pytest.raises(ValueError):
        orc.topk_select(s, 1.0, 1, 64, padding=(64, 0))


def test_merge_edge_cases():
    idx = np.full((1, 1, 4, 2), -1, dtype=np.int32)
    merged, counts, W, _ = orc.build_qblock_topk_indices(idx, 2)
    assert W == 4 and (merged == -1).all() and (counts == 0).all()
    idx[0, 0, 0] = [3, 1]
    idx[0, 0, 1] = [1, -1]
    merged, counts, W, sc = orc.build_qblock_topk_indices(idx, 2, qblock_topk=6)
    assert merged[0, 0, 0].tolist() == [1, 3, -1, -1, -1, -1]
    assert sc[0, 0, 0, :2].tolist() == [2.0, 1.0]
    assert counts.tolist() == [[[2, 0]]]
    with pytest.raises(ValueError):
        orc.build_qblock_topk_indices(idx, 3)


V1_GOLDEN = ("tiny_fp16", "ragged_bf16")


@pytest.mark.parametrize("name", V1_GOLDEN)
def test_first_generation_operators(name):
    """oracle v1_* functions against the reference's first-generation dense
    twins (golden files v1_<case>.npz)."""
    cfg = cases.GOLDEN_CASES[name]
    gold = _load(f"v1_{name}")
    x = _np_inputs(cfg)
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    B, N = cfg["B"], cfg["N"]
    o, idx, scores, table = orc.v1_topk_score(
        x["q"], x["k"], x["v"], H, b, cfg["topk"], pad, score_only=False)
    # the dense twin returns o as [B, H, N, D] for [B, N, C] input, rounded to
    # the input dtype
    o_bhnd = o.reshape(B, N, H, -1).transpose(0, 2, 1, 3)
    _close(o_bhnd, gold["o_dense"], atol=4e-3)
    rep = orc.classify_topk_mismatches(idx, gold["topk_idx"].astype(np.int32), table)
    assert rep["hard"] == 0, rep
    _close(scores, gold["topk_scores"], atol=1e-6, rtol=2e-5)
    i2, s2, _ = orc.v1_topk_score(x["q"], x["k"], None, H, b, cfg["topk"], pad, score_only=True)
    assert (i2 == idx).all() and (s2 == scores).all()

    g, qpad = cfg["q_block_size"], tuple(cfg["q_padding"])
    kvb, kvpad = cfg["kv_block_size"], tuple(cfg["kv_padding"])
    merged, counts, width = orc.v1_qblock_union(gold["topk_idx"].astype(np.int32), g, qpad)
    assert width == gold["merged"].shape[-1]
    assert (merged == gold["merged"]).all() and (counts == gold["counts"]).all()
    ao, alse = orc.v1_topk_attn(x["q"], x["k"], x["v"], merged, counts, H, g, kvb, None,
                                kvpad, qpad)
    _close(ao, gold["attn_o"], atol=4e-3)
    _close(alse, gold["attn_lse"], atol=1e-4, rtol=1e-5)
    so, slse = orc.v1_topk_attn(x["q"], x["k"], x["v"], merged[:, :1],
                                np.maximum(counts[:, :1] - 1, 0), H, g, kvb, None, kvpad, qpad)
    _close(so, gold["shared_o"], atol=4e-3)
    _close(slse, gold["shared_lse"], atol=1e-4, rtol=1e-5)


def test_first_generation_union_edges():
    idx = np.full((1, 1, 8, 2), -1, dtype=np.int32)
    idx[0, 0, 0] = (5, 5)
    idx[0, 0, 1] = (3, 70000 % 4096)
    idx[0, 0, 5] = (0, -1)
    merged, counts, width = orc.v1_qblock_union(idx, 4, (2, 2))
    assert width == 8 and merged.shape == (1, 1, 3, 8)
    assert merged[0, 0, 0, :3].tolist() == [3, 5, 368] and counts[0, 0].tolist() == [3, 1, 0]
    assert merged[0, 0, 2].tolist() == [-1] * 8 and merged[0, 0, 1, :2].tolist() == [0, -1]


def test_round_to_dtype_matches_torch_casts():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(200000) * np.exp(rng.standard_normal(200000) * 6)).astype(np.float32)
    x[:4] = [0.0, -0.0, 65504.0, 1e-8]
    t = torch.from_numpy(x)
    np.testing.assert_array_equal(orc.round_to_dtype(x, "bf16"), t.bfloat16().float().numpy())
    small = np.clip(x, -6e4, 6e4)
    np.testing.assert_array_equal(orc.round_to_dtype(small, "fp16"),
                                  torch.from_numpy(small).half().float().numpy())
    assert orc.round_to_dtype(x.astype(np.float64), "bf16").dtype == np.float64


@pytest.mark.parametrize("name", ["tiny_fp16", "ragged_bf16", "hot_fp16"])
def test_reference_roundings_mode_and_envelope(name):
    """The oracle with the reference kernels' roundings (P, dS, delta from the
    rounded O, stored outputs) stays within the plain bound of the exact oracle
    on these cases, and within its own first-order worst-case envelope."""
    import tolerance
    cfg = cases.GOLDEN_CASES[name]
    gold = _load(name)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    H, g, kvb = cfg["H"], cfg["q_block_size"], cfg["kv_block_size"]
    qpad, kvpad = tuple(cfg["q_padding"]), tuple(cfg["kv_padding"])
    merged = gold["merged"]
    o_exact, _ = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    o_stored = orc.round_to_dtype(o_exact, cfg["dtype"])
    ora = tolerance.attention_oracles(orc, x, merged, H, g, kvb, cfg["dtype"], o_stored, qpad, kvpad)
    for nm in ("O", "dQ", "dK", "dV"):
        ex, rd, env = (ora[p][nm] for p in ("exact", "rounded", "envelope"))
        err = np.abs(rd - ex)
        assert (err <= ATOL + RTOL * np.abs(ex)).all(), nm
        # first order: second-order terms and the fp32 store of lse stay below half of it
        assert (err <= 1.5 * env + 1e-6).all(), (nm, float((err / (env + 1e-12)).max()))
        assert (env >= 0).all() and np.isfinite(env).all()
    with pytest.raises(ValueError):
        orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, roundings="reference")
    with pytest.raises(ValueError):
        orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, roundings="other",
                            io_dtype="bf16")
