"""Generate the golden vectors in this folder from the reference's own code.

Run where the reference project is importable:

    python tests/golden/make_golden.py --reference /path/to/flash-topk-attention

It imports the reference's pure-PyTorch `_naive` twins (they run on CPU),
feeds them the seeded inputs built by tests/cases.py and stores their outputs
as compressed .npz files next to this script.  Inputs are NOT stored: the tests
rebuild them from the same seeds.  The reference ships no fixtures of its own,
so these files are the pin for the CPU restatement in oracle/ftk_oracle.py.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402  (tests/cases.py)


def run_case(name: str, ref) -> dict:
    cfg = cases.GOLDEN_CASES[name]
    t = cases.make_inputs(cfg)
    q, k, v, do = t["q"], t["k"], t["v"], t["do"]
    H = cfg["H"]
    b = cfg["score_block_size"]
    pad = tuple(cfg["padding"])

    scores = ref["block_score"](q, k, H, b, pad)
    idx, raw, avg = ref["select"](scores, cfg["threshold"], cfg["topk"], b, pad)

    # merge through the reference's public glue semantics (re-stated here with
    # the reference's naive merge because the glue itself requires CUDA).
    import torch.nn.functional as F

    g = cfg["q_block_size"]
    qpad = tuple(cfg["q_padding"])
    idx_p = F.pad(idx.to(torch.int32), (0, 0, qpad[0], qpad[1]), value=-1)
    valid = idx_p >= 0
    m_total = int(idx_p[valid].max().item()) + 1 if valid.any() else 1
    if cfg["score_weighted"]:
        scr_p = F.pad(avg.float(), (0, 0, qpad[0], qpad[1]), value=0.0)
    else:
        scr_p = valid.float()
    W = cfg["qblock_topk"] or g * idx.shape[-1]
    merged, mscores = ref["merge"](idx_p, scr_p, g, W, m_total)
    counts = (merged >= 0).sum(-1).int()

    out = {
        "block_scores": scores.numpy(),
        "topk_idx": idx.numpy().astype(np.int16),
        "topk_raw": raw.numpy(),
        "topk_avg": avg.numpy(),
        "merged": merged.numpy().astype(np.int16),
        "merged_scores": mscores.numpy(),
        "counts": counts.numpy().astype(np.int32),
    }

    if cfg.get("attend", True):
        kvb = cfg["kv_block_size"]
        kvpad = tuple(cfg["kv_padding"])
        o, lse = ref["attn"](
            q, k, v, merged, H, g, kvb, None, qpad, kvpad,
        )
        qf = q.float().requires_grad_(True)
        kf = k.float().requires_grad_(True)
        vf = v.float().requires_grad_(True)
        od = ref["attn_diff"](qf, kf, vf, merged, H, g, kvb, None, qpad, kvpad)
        od.backward(do.float())
        M = (kvpad[0] + cfg["N"] + kvpad[1]) // kvb
        rev, rc = ref["reverse"](merged, counts, M)
        sc, sid = ref["sort_by_count"](rc, H, M)
        stride = cfg.get("store_row_stride", 1)
        out.update(
            o=o.float().numpy()[:, ::stride],
            lse=lse.numpy()[:, :, ::stride],
            o_diff=od.detach().numpy()[:, ::stride],
            dq=qf.grad.numpy()[:, ::stride],
            dk=kf.grad.numpy()[:, ::stride],
            dv=vf.grad.numpy()[:, ::stride],
            reverse_counts=rc.numpy(),
            reverse_indices=rev.numpy().astype(np.int16),
            sorted_counts=sc.numpy(),
        )
    if cfg.get("drop_block_scores"):
        # keep the file small: a strided sample of the score matrix
        out["block_scores"] = out["block_scores"][:, :, :: cfg["drop_block_scores"]]
        out["topk_raw"] = out["topk_raw"][:, :, :: cfg["drop_block_scores"]]
        out["topk_avg"] = out["topk_avg"][:, :, :: cfg["drop_block_scores"]]
        out["merged_scores"] = out["merged_scores"].astype(np.float32)
    return out


V1_CASES = ("tiny_fp16", "ragged_bf16")


def run_case_v1(name: str, score_naive, attn_naive) -> dict:
    """Outputs of the first-generation package's dense twins
    (flash_topk_attn/scoring.py `_flash_topk_score_naive`,
    flash_topk_attn/attention.py `_flash_topk_attn_naive`) on the same seeded
    inputs.  The exact-union merge has no pure-PyTorch twin in the reference
    (only a Triton kernel), so the lists fed to the attention twin are built
    here with torch.unique, which is that kernel's definition."""
    cfg = cases.GOLDEN_CASES[name]
    t = cases.make_inputs(cfg)
    q, k, v = t["q"], t["k"], t["v"]
    H, b, pad = cfg["H"], cfg["score_block_size"], tuple(cfg["padding"])
    o, idx, scores = score_naive(q, k, v, num_heads=H, block_size=b, topk=cfg["topk"],
                                 padding=pad, score_only=False)
    g, qpad = cfg["q_block_size"], tuple(cfg["q_padding"])
    kvb, kvpad = cfg["kv_block_size"], tuple(cfg["kv_padding"])
    B, _, N, K = idx.shape
    QM = (qpad[0] + N + qpad[1]) // g
    width = 1 << (g * K - 1).bit_length()
    merged = torch.full((B, H, QM, width), -1, dtype=torch.int32)
    counts = torch.zeros(B, H, QM, dtype=torch.int32)
    for bi in range(B):
        for hi in range(H):
            for m in range(QM):
                r0, r1 = max(0, m * g - qpad[0]), min(N, (m + 1) * g - qpad[0])
                if r0 < r1:
                    ids = torch.unique(idx[bi, hi, r0:r1])
                    merged[bi, hi, m, : ids.numel()] = ids.int()
                    counts[bi, hi, m] = ids.numel()
    ao, alse = attn_naive(q, k, v, merged, counts, H, g, kvb, None, kvpad, qpad)
    # one index head shared by all heads, and a count that hides the last entry
    shared, shared_counts = merged[:, :1].contiguous(), (counts[:, :1] - 1).clamp(min=0)
    so, slse = attn_naive(q, k, v, shared, shared_counts, H, g, kvb, None, kvpad, qpad)
    return {
        "o_dense": o.float().numpy(),
        "topk_idx": idx.numpy().astype(np.int16),
        "topk_scores": scores.float().numpy(),
        "merged": merged.numpy().astype(np.int16),
        "counts": counts.numpy(),
        "attn_o": ao.float().numpy(),
        "attn_lse": alse.numpy(),
        "shared_o": so.float().numpy(),
        "shared_lse": slse.numpy(),
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True,
                    help="checkout of YouHuang67/flash-topk-attention (its pure-PyTorch "
                         "_naive functions are imported from it and run on the CPU)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.manual_seed(0)

    from flash_topk_attn_v2.block_score import _flash_block_score_naive
    from flash_topk_attn_v2.qblock_merge import _flash_qblock_merge_naive
    from flash_topk_attn_v2.sparse_attn import (
        _flash_sparse_attn_naive,
        _flash_sparse_attn_naive_differentiable,
    )
    from flash_topk_attn_v2.sparse_attn_bwd import (
        build_reverse_indices,
        sort_by_count,
    )
    from flash_topk_attn_v2.topk_select import _flash_topk_select_naive

    ref = {
        "block_score": _flash_block_score_naive,
        "select": _flash_topk_select_naive,
        "merge": _flash_qblock_merge_naive,
        "attn": _flash_sparse_attn_naive,
        "attn_diff": _flash_sparse_attn_naive_differentiable,
        "reverse": build_reverse_indices,
        "sort_by_count": sort_by_count,
    }
    for name in cases.GOLDEN_CASES:
        out = run_case(name, ref)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(name, {k: v.shape for k, v in out.items()},
              f"{os.path.getsize(path) / 1024:.0f} KiB")

    from flash_topk_attn.attention import _flash_topk_attn_naive
    from flash_topk_attn.scoring import _flash_topk_score_naive

    for name in V1_CASES:
        out = run_case_v1(name, _flash_topk_score_naive, _flash_topk_attn_naive)
        path = os.path.join(HERE, f"v1_{name}.npz")
        np.savez_compressed(path, **out)
        print("v1", name, {k: v.shape for k, v in out.items()},
              f"{os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
