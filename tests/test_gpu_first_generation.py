"""GPU parity of the first-generation operator names (package flash_topk_attn)
against the CPU oracle's v1_* functions and the golden vectors made from the
reference's first-generation dense twins (tests/golden/v1_<case>.npz).

Bars as for the second generation: indices bit-exact except reported
near-ties, the union lists bit-exact, O / lse / gradients within 2e-3 abs /
1e-2 rel of the fp64 oracle.
"""

import os

import numpy as np
import pytest
import torch

import cases
from oracle import ftk_oracle as orc

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ATOL, RTOL = 2e-3, 1e-2


@pytest.fixture(scope="module")
def v1():
    import flash_topk_attn as m
    return m


def _close(got, want, atol=ATOL, rtol=RTOL, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), f"{what}: finiteness differs"
    assert (got[~fin] == want[~fin]).all(), what
    err = np.abs(got[fin] - want[fin])
    assert (err <= atol + rtol * np.abs(want[fin])).all(), f"{what}: {float(err.max()):.3e}"


def _inputs(cfg):
    t = cases.make_inputs(cfg)
    return t, {k: v.float().numpy() for k, v in t.items()}


@pytest.mark.parametrize("name", ["tiny_fp16", "ragged_bf16", "hot_fp16"])
def test_score_union_attention_chain(v1, name):
    from flash_topk_attn_v2 import check_errors
    cfg = cases.GOLDEN_CASES[name]
    t, x = _inputs(cfg)
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    g, qpad = cfg["q_block_size"], tuple(cfg["q_padding"])
    kvb, kvpad = cfg["kv_block_size"], tuple(cfg["kv_padding"])
    q, k, v = (t[n].cuda() for n in "qkv")

    o, idx, scores = v1.flash_topk_score(q, k, v, H, b, cfg["topk"], pad)
    check_errors()
    wo, widx, wsc, table = orc.v1_topk_score(x["q"], x["k"], x["v"], H, b, cfg["topk"], pad)
    assert idx.dtype == torch.int32 and scores.dtype == torch.float32 and o.dtype == q.dtype
    rep = orc.classify_topk_mismatches(idx.cpu().numpy(), widx, table)
    assert rep["hard"] == 0, rep
    if rep["mismatched_positions"] == 0:
        np.testing.assert_allclose(scores.cpu().numpy(), wsc, rtol=1e-5, atol=1e-9)
    assert (idx >= 0).all()          # no threshold cut in this generation
    _close(o.float().cpu().numpy(), wo, what="dense o")
    i2, s2 = v1.flash_topk_score(q, k, num_heads=H, score_block_size=b, topk=cfg["topk"],
                                 padding=pad, score_only=True)
    assert torch.equal(i2, idx) and torch.equal(s2, scores)

    merged, counts, width = v1.build_qblock_topk_indices(idx, g, qpad)
    check_errors()
    wm, wc, ww = orc.v1_qblock_union(idx.cpu().numpy(), g, qpad)
    assert width == ww and merged.dtype == torch.int32 and counts.dtype == torch.int32
    np.testing.assert_array_equal(merged.cpu().numpy(), wm)
    np.testing.assert_array_equal(counts.cpu().numpy(), wc)

    ao, alse = v1.flash_topk_attn(q, k, v, merged, counts, H, g, kvb, None, None, kvpad, qpad)
    check_errors()
    wao, walse = orc.v1_topk_attn(x["q"], x["k"], x["v"], wm, wc, H, g, kvb, None, kvpad, qpad)
    _close(ao.float().cpu().numpy(), wao, what="o")
    _close(alse.cpu().numpy(), walse, what="lse")

    # one index head for all heads, counts hiding the last entry of each row
    sc = (counts[:, :1] - 1).clamp(min=0)
    so, slse = v1.flash_topk_attn(q, k, v, merged[:, :1], sc, H, g, kvb,
                                  kv_padding=kvpad, q_padding=qpad)
    wso, wslse = orc.v1_topk_attn(x["q"], x["k"], x["v"], wm[:, :1], np.maximum(wc[:, :1] - 1, 0),
                                  H, g, kvb, None, kvpad, qpad)
    _close(so.float().cpu().numpy(), wso, what="shared o")
    _close(slse.cpu().numpy(), wslse, what="shared lse")


@pytest.mark.parametrize("name", ["tiny_fp16", "ragged_bf16"])
def test_against_reference_vectors(v1, name):
    cfg = cases.GOLDEN_CASES[name]
    gold = dict(np.load(os.path.join(GOLD, f"v1_{name}.npz")))
    t, _ = _inputs(cfg)
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    B, N = cfg["B"], cfg["N"]
    q, k, v = (t[n].cuda() for n in "qkv")
    o, idx, scores = v1.flash_topk_score(q, k, v, H, b, cfg["topk"], pad)
    o_bhnd = o.float().view(B, N, H, -1).permute(0, 2, 1, 3).cpu().numpy()
    _close(o_bhnd, gold["o_dense"], atol=4e-3, what="dense o")
    same = idx.cpu().numpy() == gold["topk_idx"]
    assert same.mean() > 0.99
    np.testing.assert_allclose(scores.cpu().numpy()[same], gold["topk_scores"][same],
                               rtol=2e-5, atol=1e-7)
    gm = torch.from_numpy(gold["merged"].astype(np.int32)).cuda()
    gc = torch.from_numpy(gold["counts"]).cuda()
    m2, c2, _ = v1.build_qblock_topk_indices(
        torch.from_numpy(gold["topk_idx"].astype(np.int32)).cuda(), cfg["q_block_size"],
        tuple(cfg["q_padding"]))
    assert torch.equal(m2, gm) and torch.equal(c2, gc)
    ao, alse = v1.flash_topk_attn(q, k, v, gm, gc, H, cfg["q_block_size"], cfg["kv_block_size"],
                                  kv_padding=tuple(cfg["kv_padding"]),
                                  q_padding=tuple(cfg["q_padding"]))
    _close(ao.float().cpu().numpy(), gold["attn_o"], atol=4e-3, what="o")
    _close(alse.cpu().numpy(), gold["attn_lse"], what="lse")


def test_dense_output_gradients_and_4d_layout(v1):
    """score_only=False returns the dense attention output, differentiable in
    q, k, v (reference flash_topk_attn/scoring.py:1080-1211); N is not a
    multiple of the internal 64-row blocks."""
    B, N, H, D = 1, 208, 2, 64
    g = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(B, N, H * D, generator=g).half() for _ in range(4))
    qc, kc, vc = (x.cuda().requires_grad_(True) for x in (q, k, v))
    o, idx, scores = v1.flash_topk_score(qc, kc, vc, H, 16, 2)
    o.backward(do.cuda())
    qf, kf, vf = (x.double().requires_grad_(True) for x in (q, k, v))
    q4, k4, v4 = (x.view(B, N, H, D).transpose(1, 2) for x in (qf, kf, vf))
    p = torch.softmax(q4 @ k4.transpose(-1, -2) * D ** -0.5, dim=-1)
    want = (p @ v4).transpose(1, 2).reshape(B, N, H * D)
    want.backward(do.double())
    _close(o.detach().float().cpu().numpy(), want.detach().numpy(), what="o")
    for name, got, ref in (("dq", qc.grad, qf.grad), ("dk", kc.grad, kf.grad),
                           ("dv", vc.grad, vf.grad)):
        _close(got.float().cpu().numpy(), ref.numpy(), what=name)
    blocks = p.detach().view(B, H, N, 13, 16).sum(-1)
    rep = orc.classify_topk_mismatches(idx.cpu().numpy(),
                                       np.argsort(-blocks.numpy(), axis=-1, kind="stable")[..., :2],
                                       blocks.numpy())
    assert rep["hard"] == 0, rep

    # [B, H, N, D] in -> o comes back as [B, H, N, D]
    q4c, k4c, v4c = (x.view(B, N, H, D).transpose(1, 2).contiguous().cuda() for x in (q, k, v))
    o4, idx4, sc4 = v1.flash_topk_score(q4c, k4c, v4c, score_block_size=16, topk=2)
    assert o4.shape == (B, H, N, D)
    torch.testing.assert_close(o4.transpose(1, 2).reshape(B, N, H * D), o.detach(), rtol=0, atol=0)
    assert torch.equal(idx4, idx) and torch.equal(sc4, scores)


def test_union_of_wide_id_ranges(v1):
    """Ids up to 65535, repeats inside and across rows, empty rows, virtual
    padding rows; explicit narrower width cuts the row and reports it."""
    from flash_topk_attn_v2 import ops
    rng = np.random.default_rng(3)
    B, H, N, K, g = 2, 3, 500, 6, 32
    idx = rng.integers(0, 65536, size=(B, H, N, K)).astype(np.int32)
    idx[rng.random(idx.shape) < 0.3] = -1
    idx[:, :, 100:140] = -1
    idx[:, :, 200:232, :] = idx[:, :, 200:201, :1]        # one id repeated all over a block
    t = torch.from_numpy(idx).cuda()
    merged, counts, width = v1.build_qblock_topk_indices(t, g, (12, 0))
    ops.check_errors()
    wm, wc, ww = orc.v1_qblock_union(idx, g, (12, 0))
    assert width == ww == 256
    np.testing.assert_array_equal(merged.cpu().numpy(), wm)
    np.testing.assert_array_equal(counts.cpu().numpy(), wc)
    if ops._DEBUG:      # FTK_DEBUG=1: the cut is reported by the call itself
        with pytest.raises(RuntimeError):
            ops.flash_qblock_union(t, g, (12, 0), num_score_blocks=65536, width=8)
        return
    m2, c2 = ops.flash_qblock_union(t, g, (12, 0), num_score_blocks=65536, width=8)
    np.testing.assert_array_equal(m2.cpu().numpy(), wm[..., :8])
    np.testing.assert_array_equal(c2.cpu().numpy(), np.minimum(wc, 8))
    with pytest.raises(RuntimeError):
        ops.check_errors()


def test_reference_exceptions(v1):
    x = torch.zeros(1, 128, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="unsupported backend"):
        v1.flash_topk_score(x, x, x, 1, backend="cuda")
    with pytest.raises(ValueError, match="v is required"):
        v1.flash_topk_score(x, x, None, 1)
    with pytest.raises(ValueError, match="num_heads is required"):
        v1.flash_topk_score(x, x, x)
    with pytest.raises(ValueError, match="topk"):
        v1.flash_topk_score(x, x, x, 1, 64, 4)
    with pytest.raises(ValueError, match="divisible"):
        v1.flash_topk_score(x, x, x, 1, 48, 1)
    idx = torch.zeros(1, 1, 128, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="q_pad_head"):
        v1.build_qblock_topk_indices(idx, 32, (32, 0))
    with pytest.raises(AssertionError):
        v1.build_qblock_topk_indices(idx, 48)
    m, c, _ = v1.build_qblock_topk_indices(idx, 32)
    with pytest.raises(NotImplementedError):
        v1.flash_topk_attn(x, x, x, m, c, 2, 32, 64, num_kv_heads=1)
    with pytest.raises(ValueError, match="kv_pad_tail"):
        v1.flash_topk_attn(x, x, x, m, c, 1, 32, 64, kv_padding=(0, 64))
