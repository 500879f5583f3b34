"""First-generation operator names on the same sm_100a library.

Drop-in for the reference's older package `flash_topk_attn`
(flash_topk_attn/__init__.py:1-4): the same three names with its signatures,
defaults and return shapes, built on the entry points of libftk_sm100.so that
serve `flash_topk_attn_v2`.  Differences in meaning from the second
generation, kept here as the reference defines them:

* scoring has no cumulative-threshold cut: every query keeps exactly `topk`
  blocks, best first (flash_topk_attn/scoring.py:1289-1357, :1360-1469);
  returned scores are block sums without padding and per-token averages with
  padding (the two branches of the reference's dense formulation, :1448-1459);
* with `score_only=False` the dense attention output softmax(QK^T / sqrt(D)) V
  is returned as well and is differentiable in q, k, v (:1080-1211);
* the q-block merge is the exact union of the rows' picks in ascending block
  id, width next_pow2(q_block_size * K), no ranking and no cap
  (flash_topk_attn/attention.py:70-138);
* attention honours `counts` (only the first counts[b, h, m] entries of a row
  are read) and accepts one index head shared by all heads
  (flash_topk_attn/attention.py:423-568, :571-647).

Importing this package without the CUDA library raises ImportError; there is
no fallback path.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from flash_topk_attn_v2 import ops
from flash_topk_attn_v2.ops import flash_sparse_attn

Pair = Tuple[int, int]
Tensor = torch.Tensor

_NO_CUT = 2.0   # cumulative block mass never reaches 2: the threshold never fires
_DENSE_BLOCK = 64


def _to_bnc(x: Tensor) -> Tensor:
    B, H, N, D = x.shape
    return x.transpose(1, 2).reshape(B, N, H * D)


def _dense_attention(q, k, v, num_heads):
    """softmax(q k^T / sqrt(D)) v over all N keys, [B, N, C] in, [B, N, C] out:
    the gathered-KV kernels with every q-block listing every kv block."""
    B, N, C = q.shape
    blk = _DENSE_BLOCK
    tail = (-N) % blk
    blocks = (N + tail) // blk
    lists = torch.arange(blocks, dtype=torch.int32, device=q.device) \
        .expand(B, num_heads, blocks, blocks).contiguous()
    o, _ = flash_sparse_attn(
        q, k, v, lists, num_heads=num_heads, q_block_size=blk, kv_block_size=blk, scale=None,
        q_padding=(0, tail), kv_padding=(0, tail))
    return o


def flash_topk_score(q: Tensor, k: Tensor, v: Optional[Tensor] = None,
                     num_heads: Optional[int] = None, score_block_size: int = 64, topk: int = 16,
                     padding: Pair = (0, 0), score_only: bool = False, backend: str = "triton"):
    """(o, topk_indices, topk_scores), or (topk_indices, topk_scores) with
    `score_only=True` (reference flash_topk_attn/scoring.py:1289-1357).
    `backend` keeps the reference's only accepted value."""
    if backend != "triton":
        raise ValueError(f"unsupported backend: {backend!r}, must be 'triton'")
    if not score_only and v is None:
        raise ValueError("v is required when score_only=False")
    input_4d = q.ndim == 4
    if input_4d:
        B, H, N, D = q.shape
        if num_heads is not None and num_heads != H:
            raise ValueError(f"num_heads ({num_heads}) != q.shape[1] ({H})")
        num_heads = H
        if not score_only and v.shape != (B, H, N, D):
            raise ValueError("q, k, v must all be [B, H, N, D] for 4D input")
    else:
        if q.ndim != 3:
            raise ValueError("q must be 3D [B, N, C] or 4D [B, H, N, D]")
        if num_heads is None:
            raise ValueError("num_heads is required for 3D [B, N, C] input")
        N = q.shape[1]
    pad_head, pad_tail = padding
    if pad_head >= 0 and pad_tail >= 0 and score_block_size > 0 and \
            (pad_head + N + pad_tail) % score_block_size == 0:
        num_blocks = (pad_head + N + pad_tail) // score_block_size
        if topk > num_blocks:
            raise ValueError(f"topk ({topk}) > num_blocks ({num_blocks})")
    with torch.no_grad():
        idx, raw, avg = ops.flash_topk_score_fused(
            q, k, num_heads, score_block_size, topk, padding, _NO_CUT)
    scores = raw if (pad_head == 0 and pad_tail == 0) else avg
    if score_only:
        return idx, scores
    if input_4d:
        o = _dense_attention(_to_bnc(q), _to_bnc(k), _to_bnc(v), num_heads)
        B, N, C = o.shape
        o = o.view(B, N, num_heads, C // num_heads).transpose(1, 2).contiguous()
    else:
        o = _dense_attention(q, k, v, num_heads)
    return o, idx, scores


def build_qblock_topk_indices(topk_indices: Tensor, q_block_size: int,
                              q_padding: Pair = (0, 0)) -> Tuple[Tensor, Tensor, int]:
    """Sorted distinct block ids per q-block: (merged [B, H, QM, S_MAX] int32,
    counts [B, H, QM] int32, S_MAX = next_pow2(q_block_size * K))
    (reference flash_topk_attn/attention.py:70-138)."""
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, K]")
    q_pad_head, q_pad_tail = q_padding
    if q_pad_head >= q_block_size:
        raise ValueError(
            f"q_pad_head={q_pad_head} must be < q_block_size={q_block_size}; "
            "virtual padding should only complete partial blocks, not create new ones.")
    if q_pad_tail >= q_block_size:
        raise ValueError(
            f"q_pad_tail={q_pad_tail} must be < q_block_size={q_block_size}; "
            "virtual padding should only complete partial blocks, not create new ones.")
    padded = q_pad_head + topk_indices.shape[2] + q_pad_tail
    assert padded % q_block_size == 0, \
        f"N_Q_PADDED={padded} must be divisible by q_block_size={q_block_size}"
    merged, counts = ops.flash_qblock_union(
        topk_indices, q_block_size, (q_pad_head, q_pad_tail),
        num_score_blocks=getattr(topk_indices, "_ftk_num_score_blocks", None))
    return merged, counts, merged.shape[-1]


def flash_topk_attn(q: Tensor, k: Tensor, v: Tensor, merged_indices: Tensor, counts: Tensor,
                    num_heads: int, q_block_size: int, kv_block_size: int,
                    scale: Optional[float] = None, num_kv_heads: Optional[int] = None,
                    kv_padding: Pair = (0, 0), q_padding: Pair = (0, 0),
                    S_MAX: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """(o [B, N, C], lse [B, H, N] fp32): every query of a q-block attends
    over the tokens of the first counts[b, h, m] listed blocks (reference
    flash_topk_attn/attention.py:423-568).  Unlike the reference this call is
    also differentiable in q, k, v."""
    assert q.is_cuda and k.is_cuda and v.is_cuda
    assert q.dtype in (torch.float16, torch.bfloat16, torch.float32)
    H = num_heads
    if num_kv_heads is not None and num_kv_heads != H:
        raise NotImplementedError("GQA (num_kv_heads != num_heads) is not supported in v1")
    for name, pad, blk in (("kv_pad_head", kv_padding[0], kv_block_size),
                           ("kv_pad_tail", kv_padding[1], kv_block_size),
                           ("q_pad_head", q_padding[0], q_block_size),
                           ("q_pad_tail", q_padding[1], q_block_size)):
        if pad >= blk:
            which = "kv_block_size" if name.startswith("kv") else "q_block_size"
            raise ValueError(
                f"{name}={pad} must be < {which}={blk}; "
                "virtual padding should only complete partial blocks, not create new ones.")
    lists = merged_indices.to(torch.int32)
    if S_MAX is not None:
        lists = lists[..., :S_MAX]
    heads_in_lists = lists.shape[1]
    assert heads_in_lists == 1 or heads_in_lists == H
    if counts is not None:
        slot = torch.arange(lists.shape[-1], device=lists.device)
        lists = torch.where(slot < counts.to(lists.device).unsqueeze(-1), lists,
                            torch.full_like(lists, -1))
    if heads_in_lists != H:
        lists = lists.expand(-1, H, -1, -1)
    return flash_sparse_attn(
        q, k, v, lists.contiguous(), num_heads=H, q_block_size=q_block_size,
        kv_block_size=kv_block_size, scale=scale, q_padding=q_padding, kv_padding=kv_padding)


__all__ = ["flash_topk_score", "flash_topk_attn", "build_qblock_topk_indices"]
