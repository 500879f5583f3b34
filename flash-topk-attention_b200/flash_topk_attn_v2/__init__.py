"""Public API of flash_topk_attn_v2, B200-native.

Drop-in for the reference package of the same name: the three entry points
keep its signatures, defaults, return shapes and dtypes
(reference: flash_topk_attn_v2/__init__.py:16-176).  All compute runs in
libftk_sm100.so (hand-written sm_100a CUDA behind a C ABI); importing this
package without that library raises ImportError.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from .ops import (
    check_errors,
    flash_block_score,
    flash_build_reverse_indices_cuda,
    flash_qblock_merge,
    flash_sort_by_count_cuda,
    flash_sparse_attn,
    flash_topk_select,
)


def flash_topk_score(
    q: torch.Tensor,
    k: torch.Tensor,
    num_heads: Optional[int] = None,
    score_block_size: int = 64,
    topk: int = 16,
    padding: Tuple[int, int] = (0, 0),
    threshold: float = 1.0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Block-level top-k scoring: (topk_indices int32, topk_raw fp32, topk_avg
    fp32), each [B, H, N, min(topk, M)] (reference __init__.py:16-54)."""
    input_4d = q.ndim == 4
    if input_4d:
        _, head_count, _, _ = q.shape
        if num_heads is not None and num_heads != head_count:
            raise ValueError(f"num_heads ({num_heads}) != q.shape[1] ({head_count})")
        num_heads = head_count
    else:
        if q.ndim != 3:
            raise ValueError("q must be 3D [B, N, C] or 4D [B, H, N, D]")
        if num_heads is None:
            raise ValueError("num_heads is required for 3D [B, N, C] input")
    return ops.flash_topk_score_fused(
        q, k, num_heads, score_block_size, topk, padding, threshold)


def build_qblock_topk_indices(
    topk_indices: torch.Tensor,
    q_block_size: int,
    q_padding: Tuple[int, int] = (0, 0),
    topk_scores: Optional[torch.Tensor] = None,
    qblock_topk: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Per-q-block merged indices: (merged [B,H,QM,W] int32, counts [B,H,QM]
    int32, W) (reference __init__.py:57-133)."""
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, K]")
    _, _, sequence_length, topk_width = topk_indices.shape
    q_pad_head, q_pad_tail = q_padding
    if q_pad_head < 0 or q_pad_tail < 0:
        raise ValueError("q_padding must be non-negative")
    if q_pad_head >= q_block_size:
        raise ValueError(f"q_pad_head={q_pad_head} must be < q_block_size={q_block_size}")
    if q_pad_tail >= q_block_size:
        raise ValueError(f"q_pad_tail={q_pad_tail} must be < q_block_size={q_block_size}")
    padded = q_pad_head + sequence_length + q_pad_tail
    if padded % q_block_size != 0:
        raise ValueError(
            f"q_pad_head + N + q_pad_tail = {padded} must be divisible "
            f"by q_block_size ({q_block_size})"
        )
    if qblock_topk is None:
        qblock_topk = q_block_size * topk_width
    # size of the aggregation table: any bound >= max(valid id) + 1 gives the
    # same result.  Index tensors made by flash_topk_score carry the block
    # count; otherwise read the maximum back as the reference does.
    num_score_blocks = getattr(topk_indices, "_ftk_num_score_blocks", None)
    if num_score_blocks is None:
        mx = int(topk_indices.max().item()) if topk_indices.numel() else -1
        num_score_blocks = mx + 1 if mx >= 0 else 1
    merged, _scores, counts = flash_qblock_merge(
        topk_indices, topk_scores, q_block_size, qblock_topk, num_score_blocks,
        q_padding=(q_pad_head, q_pad_tail), return_counts=True,
    )
    return merged, counts, merged.shape[-1]


def flash_topk_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    merged_indices: torch.Tensor,
    counts: torch.Tensor,
    num_heads: int,
    q_block_size: int,
    kv_block_size: int,
    scale: Optional[float] = None,
    num_kv_heads: Optional[int] = None,
    kv_padding: Tuple[int, int] = (0, 0),
    q_padding: Tuple[int, int] = (0, 0),
    S_MAX: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse attention over merged KV block indices: (O [B,N,C], lse [B,H,N]);
    differentiable in q, k, v (reference __init__.py:136-169).  `counts` and
    `S_MAX` are ignored, as in the reference.  `num_kv_heads` different from
    `num_heads` (grouped-query attention) raises NotImplementedError in the
    reference (__init__.py:153-156) and is supported here: k and v are then
    [B, N, num_kv_heads * D]."""
    del counts, S_MAX
    return flash_sparse_attn(
        q, k, v, merged_indices,
        num_heads=num_heads, q_block_size=q_block_size, kv_block_size=kv_block_size,
        scale=scale, q_padding=q_padding, kv_padding=kv_padding, num_kv_heads=num_kv_heads,
    )


__all__ = [
    "flash_topk_score",
    "build_qblock_topk_indices",
    "flash_topk_attn",
]
