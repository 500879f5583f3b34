"""Head dims 160 and 256 (the top of the reference's list,
flash_topk_attn_v2/block_score_cuda.py:16, sparse_attn.py:349-373): scoring,
select and the attention forward and backward against the fp64 oracle."""

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


def _close(got, want, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    fin = np.isfinite(want)
    assert (np.isfinite(got) == fin).all(), what
    err = np.abs(got[fin] - want[fin])
    assert (err <= ATOL + RTOL * np.abs(want[fin])).all(), f"{what}: {float(err.max()):.3e}"


@pytest.mark.parametrize("D,dtype,N,b,pad", [
    (256, "bf16", 1024, 64, (0, 0)),
    (256, "fp16", 600, 32, (20, 20)),      # ragged, virtual padding, three blocks per key tile
    (160, "bf16", 512, 128, (0, 0)),       # padded to 256 on the host; scale stays 1/sqrt(160)
    (256, "fp16", 768, 256, (0, 0)),       # score blocks spanning two key tiles
])
def test_scoring(ftk, D, dtype, N, b, pad):
    H = 2
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=41, do_seed=42, input_scale=0.7)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    q, k = t["q"].cuda(), t["k"].cuda()
    want = orc.block_score(x["q"], x["k"], H, b, pad, work=np.float64)
    got = ftk.flash_block_score(q, k, H, b, pad).cpu().numpy()
    ftk.check_errors()
    np.testing.assert_allclose(got, want, rtol=5e-6, atol=1e-9)
    topk = 3
    idx, raw, avg = ftk.flash_topk_score(q, k, H, b, topk, pad, 0.95)
    ftk.check_errors()
    oi, oraw, oavg, table = orc.flash_topk_score(x["q"], x["k"], H, b, topk, pad, 0.95)
    rep = orc.classify_topk_mismatches(idx.cpu().numpy(), oi, table)
    assert rep["hard"] == 0, rep
    if rep["mismatched_positions"] == 0:
        np.testing.assert_allclose(raw.cpu().numpy(), oraw, rtol=1e-5, atol=1e-9)
        np.testing.assert_allclose(avg.cpu().numpy(), oavg, rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("D,dtype,g,kvb,N,qpad,kvpad", [
    (256, "bf16", 64, 64, 512, (0, 0), (0, 0)),
    (256, "fp16", 32, 64, 300, (10, 10), (40, 44)),
    (160, "bf16", 64, 32, 384, (0, 0), (0, 0)),
    (256, "fp16", 128, 128, 512, (0, 0), (0, 0)),     # split into 64-row halves on the host
    (256, "bf16", 16, 16, 256, (0, 0), (0, 0)),
])
def test_attention_forward(ftk, D, dtype, g, kvb, N, qpad, kvpad):
    H = 2
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=43, do_seed=44)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    QM, M = (qpad[0] + N + qpad[1]) // g, (kvpad[0] + N + kvpad[1]) // kvb
    rng = np.random.default_rng(11)
    W = 5
    merged = np.full((1, H, QM, W), -1, dtype=np.int32)
    for h in range(H):
        for m in range(QM):
            c = 0 if m % 5 == 4 else int(rng.integers(1, min(W, M) + 1))
            merged[0, h, m, :c] = rng.permutation(M)[:c]
    q, k, v = (t[n].cuda() for n in "qkv")
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, H, g, kvb,
                                 kv_padding=kvpad, q_padding=qpad)
    ftk.check_errors()
    assert o.shape == q.shape and o.dtype == q.dtype
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o.float().cpu().numpy(), wo, "O")
    _close(lse.cpu().numpy(), wl, "lse")


@pytest.mark.parametrize("dtype", ["bf16", "fp16"])
def test_forward_rescales_shared_accumulator(ftk, dtype):
    """Later kv blocks carry much larger logits, so the running maximum grows
    several times and the one O accumulator is rescaled while the previous
    tile's P.V may still be in flight."""
    H, N, D, g, kvb = 2, 512, 256, 64, 64
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=47, do_seed=48)
    t = cases.make_inputs(cfg)
    boost = torch.tensor([1, 1, 5, 1, 9, 2, 14, 20], dtype=torch.float32)
    k = (t["k"].float().view(1, N // kvb, kvb, H * D) * boost.view(1, -1, 1, 1)).view(1, N, H * D)
    t["k"] = k.to(t["q"].dtype)
    x = {n: v.float().numpy() for n, v in t.items()}
    QM, M = N // g, N // kvb
    merged = np.tile(np.arange(M, dtype=np.int32), (1, H, QM, 1))
    merged[0, 1, 3, 5:] = -1
    q, kk, v = (t[n].cuda() for n in "qkv")
    o, lse = ftk.flash_topk_attn(q, kk, v, torch.from_numpy(merged).cuda(), None, H, g, kvb)
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb)
    # nearly one-hot rows: O is one bf16-rounded P times values of size 2..4, so the
    # bf16 bound is that of the output's own rounding (as for the other one-hot cases)
    got, want = o.float().cpu().numpy().astype(np.float64), np.asarray(wo, np.float64)
    atol = 2e-2 if dtype == "bf16" else ATOL
    assert (np.abs(got - want) <= atol + RTOL * np.abs(want)).all(), \
        float(np.abs(got - want).max())
    _close(lse.cpu().numpy(), wl, "lse")


@pytest.mark.parametrize("D,dtype,g,kvb,N,qpad,kvpad", [
    (256, "bf16", 64, 64, 512, (0, 0), (0, 0)),       # lists restated over 32-row blocks
    (256, "fp16", 32, 64, 300, (10, 10), (40, 44)),
    (160, "fp16", 64, 32, 384, (0, 0), (0, 0)),
    (256, "fp16", 128, 128, 512, (70, 58), (100, 28)),  # two rounds of halving
    (256, "fp16", 16, 16, 256, (0, 0), (0, 0)),
])
def test_attention_backward(ftk, D, dtype, g, kvb, N, qpad, kvpad):
    H = 2
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=45, do_seed=46)
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    QM, M = (qpad[0] + N + qpad[1]) // g, (kvpad[0] + N + kvpad[1]) // kvb
    rng = np.random.default_rng(12)
    W = 6
    merged = np.full((1, H, QM, W), -1, dtype=np.int32)
    for h in range(H):
        for m in range(QM):
            c = 0 if m % 5 == 4 else int(rng.integers(1, min(W, M) + 1))
            merged[0, h, m, :c] = rng.permutation(M)[:c]
    q, k, v = (t[n].cuda().requires_grad_(True) for n in "qkv")
    o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(merged).cuda(), None, H, g, kvb,
                                 kv_padding=kvpad, q_padding=qpad)
    o.backward(t["do"].cuda())
    ftk.check_errors()
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, g, kvb, None, qpad, kvpad)
    _close(o.detach().float().cpu().numpy(), wo, "O")
    wq, wk, wv = orc.sparse_attn_bwd(x["q"], x["k"], x["v"], o.detach().float().cpu().numpy(), wl,
                                     x["do"], merged, H, g, kvb, None, qpad, kvpad)
    frac = 0.0 if dtype == "fp16" else 1e-4
    for name, got, want in (("dQ", q.grad, wq), ("dK", k.grad, wk), ("dV", v.grad, wv)):
        got, want = got.float().cpu().numpy().astype(np.float64), np.asarray(want, np.float64)
        err = np.abs(got - want)
        tol = ATOL + RTOL * np.abs(want)
        assert (err > tol).sum() <= frac * err.size and not (err > 2 * tol).any(), \
            f"{name}: {int((err > tol).sum())} bad, max {float(err.max()):.3e}"


def test_backward_block_sizes_that_cannot_be_halved(ftk):
    """At head dim 256 the gradient kernels take 32-row blocks; 48 cannot be
    restated over them and must raise, not return something."""
    H, N, D = 1, 192, 256
    q, k, v = (torch.randn(1, N, H * D, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
               for _ in range(3))
    merged = torch.zeros(1, H, 4, 1, dtype=torch.int32, device="cuda")
    # inputs that want gradients: refused at the forward call already
    with pytest.raises(NotImplementedError, match="halves down"):
        ftk.flash_topk_attn(q, k, v, merged, None, H, 48, 48)
    # without gradients the forward itself takes 48-row blocks
    with torch.no_grad():
        o, _ = ftk.flash_topk_attn(q, k, v, merged, None, H, 48, 48)
    assert torch.isfinite(o).all()
