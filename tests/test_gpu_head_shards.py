"""Sharding one batch element by heads, on a GPU.

`shard.shard_heads` hands a rank a strided view [B, N, heads_of_rank * D] of the
full [B, N, H * D] tensors (no copy); the kernels address it in place through
their [b][n][h][d] strides.  Every kernel of the path works on one (batch,
head) slice at a time, so running the three API calls per shard, one shard after
the other on one GPU, and concatenating along the head axis must reproduce the
unsharded run bit for bit: indices, scores, merged lists, counts, O, lse, dQ,
dK, dV.
"""

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ftk():
    import flash_topk_attn_v2 as m
    return m


def _chain(ftk, q, k, v, do, H, b, topk, thr, g, kvb):
    q = q.detach().requires_grad_(True)
    k = k.detach().requires_grad_(True)
    v = v.detach().requires_grad_(True)
    idx, raw, avg = ftk.flash_topk_score(q.detach(), k.detach(), H, b, topk, (0, 0), thr)
    merged, counts, W = ftk.build_qblock_topk_indices(idx, g, topk_scores=avg)
    o, lse = ftk.flash_topk_attn(q, k, v, merged, counts, H, g, kvb)
    gq, gk, gv = torch.autograd.grad(o, (q, k, v), do)
    ftk.check_errors()
    return dict(idx=idx, raw=raw, avg=avg, merged=merged, counts=counts, o=o.detach(), lse=lse,
                dq=gq, dk=gk, dv=gv)


@pytest.mark.parametrize("D,dtype,g,world", [(128, "bf16", 64, 2), (128, "bf16", 64, 4),
                                             (64, "fp16", 32, 2)])
def test_head_shards_concatenate_to_the_unsharded_result(ftk, D, dtype, g, world):
    from flash_topk_attn_v2 import shard
    H, N, b, kvb, topk, thr = 4, 1024, 64, 64, 6, 0.9
    t = cases.make_inputs(dict(B=2, N=N, H=H, D=D, dtype=dtype, seed=91, do_seed=92))
    full = {n: x.cuda() for n, x in t.items()}
    want = _chain(ftk, full["q"], full["k"], full["v"], full["do"], H, b, topk, thr, g, kvb)
    parts = []
    for r in range(world):
        views = {}
        for n, x in full.items():
            views[n], per = shard.shard_heads(x, H, r, world)
            assert not views[n].is_contiguous() and views[n].data_ptr() == x.data_ptr() + \
                r * per * D * x.element_size()
        parts.append(_chain(ftk, views["q"], views["k"], views["v"], views["do"], per, b, topk,
                            thr, g, kvb))
    B = 2
    for name in ("idx", "raw", "avg", "merged", "counts", "lse"):      # [B, H, ...]: head axis 1
        got = torch.cat([p[name] for p in parts], dim=1)
        assert torch.equal(got, want[name]), name
    for name in ("o", "dq", "dk", "dv"):                               # [B, N, H*D]: heads inside C
        got = torch.cat([p[name].view(B, N, H // world, D) for p in parts], dim=2).view(B, N, H * D)
        assert torch.equal(got, want[name]), name
    lo, hi = shard.slice_range(B * H, 1, world)
    assert (lo, hi) == (B * H // world, 2 * B * H // world)
