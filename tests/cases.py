"""Seeded synthetic inputs shared by the tests, the golden generator and bench.

All tensors are drawn on the CPU with `torch.Generator().manual_seed(seed)` and
then cast, so the CPU checker and every GPU see identical bits.  The reference
project benchmarks on random tensors as well (its README usage section) and
names no dataset.
"""

from __future__ import annotations

import torch

_DT = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def make_inputs(cfg: dict) -> dict:
    """q, k, v (one generator, in that order) and dO (second generator).

    cfg keys: B, N, H, D, dtype ("fp16"|"bf16"), seed, do_seed, input_scale,
    optional "hot_blocks" = (count, boost, block_size, pad_head) which adds
    `boost * u` (u one shared random direction per head) to every key of
    `count` randomly chosen score blocks per (batch, head).
    """
    B, N, H, D = cfg["B"], cfg["N"], cfg["H"], cfg["D"]
    dt = _DT[cfg["dtype"]]
    g = torch.Generator().manual_seed(cfg.get("seed", 0))
    s = cfg.get("input_scale", 1.0)
    q = torch.randn(B, N, H * D, generator=g) * s
    k = torch.randn(B, N, H * D, generator=g) * s
    v = torch.randn(B, N, H * D, generator=g) * s
    hot = cfg.get("hot_blocks")
    if hot:
        count, boost, blk, ph = hot
        m = (ph + N + blk - 1) // blk
        k4 = k.view(B, N, H, D)
        u = torch.randn(D, generator=g)
        for b in range(B):
            for h in range(H):
                ids = torch.randperm(m, generator=g)[:count]
                for j in ids.tolist():
                    s0 = max(0, j * blk - ph)
                    s1 = min(N, (j + 1) * blk - ph)
                    k4[b, s0:s1, h] += boost * u
    g2 = torch.Generator().manual_seed(cfg.get("do_seed", 1))
    do = torch.randn(B, N, H * D, generator=g2)
    return {"q": q.to(dt), "k": k.to(dt), "v": v.to(dt), "do": do.to(dt)}


def _case(**kw):
    base = dict(
        seed=0, do_seed=1, input_scale=1.0, padding=(0, 0), q_padding=(0, 0),
        kv_padding=(0, 0), threshold=1.0, qblock_topk=None,
        score_weighted=True, attend=True,
    )
    base.update(kw)
    return base


# Cases whose reference outputs are stored under tests/golden/.
GOLDEN_CASES = {
    # small everything-on case, fp16, D=64
    "tiny_fp16": _case(
        B=1, N=256, H=2, D=64, dtype="fp16", score_block_size=64, topk=3,
        threshold=0.9, q_block_size=32, kv_block_size=64,
    ),
    # ragged length with virtual padding on scores, queries and keys, bf16
    "ragged_bf16": _case(
        B=1, N=200, H=2, D=128, dtype="bf16", score_block_size=64, topk=2,
        threshold=0.6, padding=(20, 36), q_block_size=32, q_padding=(24, 0),
        kv_block_size=64, kv_padding=(20, 36), score_weighted=False,
        qblock_topk=3,
    ),
    # skewed scores so the cumulative threshold cuts before k
    "hot_fp16": _case(
        B=1, N=512, H=2, D=64, dtype="fp16", score_block_size=32, topk=8,
        threshold=0.5, q_block_size=64, kv_block_size=32,
        hot_blocks=(2, 1.0, 32, 0),
    ),
    # BASELINE config 1 (the reference's CPU-runnable shape); dense outputs
    # are stored on a stride to keep the file small.
    "config1": _case(
        B=2, N=1024, H=8, D=64, dtype="fp16", score_block_size=64, topk=16,
        threshold=1.0, q_block_size=32, kv_block_size=64,
        store_row_stride=16, drop_block_scores=16,
    ),
}


# BASELINE.json configs (index = position in its "configs" list).
BASELINE_CONFIGS = {
    1: GOLDEN_CASES["config1"],
    2: _case(
        B=1, N=32768, H=32, D=128, dtype="bf16", input_scale=0.5,
        score_block_size=64, topk=32, threshold=0.9, q_block_size=64,
        kv_block_size=64,
    ),
    3: _case(
        B=4, N=8192, H=16, D=128, dtype="bf16", score_block_size=64, topk=16,
        q_block_size=64, kv_block_size=64, qblock_topk=256,
    ),
    4: _case(
        B=2, N=30000, H=32, D=128, dtype="fp16", score_block_size=128,
        topk=24, threshold=0.8, padding=(40, 40), q_block_size=128,
        q_padding=(40, 40), hot_blocks=(8, 2.0, 128, 40), attend=False,
    ),
    5: _case(
        B=8, N=65536, H=64, D=128, dtype="bf16", score_block_size=64, topk=64,
        q_block_size=64, kv_block_size=64,
    ),
}
