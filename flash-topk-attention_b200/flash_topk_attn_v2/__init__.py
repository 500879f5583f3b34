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


Pair = Tuple[int, int]
Tensor = torch.Tensor


def _head_count(q: Tensor, num_heads: Optional[int]) -> int:
    """Heads of a [B, N, C] (given) or [B, H, N, D] (read off the shape) input,
    with the reference's complaints (__init__.py:26-38)."""
    if q.ndim == 4:
        if num_heads not in (None, q.shape[1]):
            raise ValueError(f"num_heads ({num_heads}) != q.shape[1] ({q.shape[1]})")
        return q.shape[1]
    if q.ndim != 3:
        raise ValueError("q must be 3D [B, N, C] or 4D [B, H, N, D]")
    if num_heads is None:
        raise ValueError("num_heads is required for 3D [B, N, C] input")
    return num_heads


def _check_q_blocks(rows: int, q_block_size: int, q_padding: Pair) -> None:
    """Virtual q padding must complete partial blocks only (__init__.py:65-88)."""
    head, tail = q_padding
    if min(head, tail) < 0:
        raise ValueError("q_padding must be non-negative")
    for name, pad in (("q_pad_head", head), ("q_pad_tail", tail)):
        if pad >= q_block_size:
            raise ValueError(f"{name}={pad} must be < q_block_size={q_block_size}")
    if (head + rows + tail) % q_block_size:
        raise ValueError(f"q_pad_head + N + q_pad_tail = {head + rows + tail} must be divisible "
                         f"by q_block_size ({q_block_size})")


def flash_topk_score(q: Tensor, k: Tensor, num_heads: Optional[int] = None,
                     score_block_size: int = 64, topk: int = 16, padding: Pair = (0, 0),
                     threshold: float = 1.0) -> Tuple[Tensor, Tensor, Tensor]:
    """Block-level top-k scoring: (topk_indices int32, topk_raw fp32, topk_avg
    fp32), each [B, H, N, min(topk, M)] (reference __init__.py:16-54)."""
    return ops.flash_topk_score_fused(q, k, _head_count(q, num_heads), score_block_size, topk,
                                      padding, threshold)


def build_qblock_topk_indices(topk_indices: Tensor, q_block_size: int, q_padding: Pair = (0, 0),
                              topk_scores: Optional[Tensor] = None,
                              qblock_topk: Optional[int] = None,
                              num_score_blocks: Optional[int] = None) -> Tuple[Tensor, Tensor, int]:
    """Per-q-block merged indices: (merged [B,H,QM,W] int32, counts [B,H,QM]
    int32, W) (reference __init__.py:57-133).

    `num_score_blocks` (not in the reference) is an upper bound of the block
    ids, i.e. M of the scoring call; any bound >= max(valid id) + 1 gives the
    same result.  Without it the bound is taken from the index tensor when
    flash_topk_score of this package made it (the tensor carries M), and
    otherwise read back from the device as the reference does (one host
    synchronisation; under stream capture, where that is not allowed, the
    largest supported table, 4096 blocks, is used instead)."""
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, K]")
    rows, picks = topk_indices.shape[2:]
    _check_q_blocks(rows, q_block_size, q_padding)
    width = q_block_size * picks if qblock_topk is None else qblock_topk
    blocks = num_score_blocks
    if blocks is None:
        blocks = getattr(topk_indices, "_ftk_num_score_blocks", None)
    if blocks is None:
        if topk_indices.is_cuda and torch.cuda.is_current_stream_capturing():
            blocks = 4096
        else:
            blocks = ops.num_score_blocks_of(topk_indices)
    merged, _, counts = flash_qblock_merge(topk_indices, topk_scores, q_block_size, width, blocks,
                                           q_padding=tuple(q_padding), return_counts=True)
    return merged, counts, merged.shape[-1]


def flash_topk_attn(q: Tensor, k: Tensor, v: Tensor, merged_indices: Tensor, counts: Tensor,
                    num_heads: int, q_block_size: int, kv_block_size: int,
                    scale: Optional[float] = None, num_kv_heads: Optional[int] = None,
                    kv_padding: Pair = (0, 0), q_padding: Pair = (0, 0),
                    S_MAX: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """Sparse attention over merged KV block indices: (O [B,N,C], lse [B,H,N]);
    differentiable in q, k, v (reference __init__.py:136-169).  `counts` and
    `S_MAX` are ignored, as in the reference.  `num_kv_heads` different from
    `num_heads` (grouped-query attention) raises NotImplementedError in the
    reference (__init__.py:153-156) and is supported here: k and v are then
    [B, N, num_kv_heads * D]."""
    return flash_sparse_attn(q, k, v, merged_indices, num_heads, q_block_size, kv_block_size,
                             scale, q_padding, kv_padding, num_kv_heads)


__all__ = ["flash_topk_score", "build_qblock_topk_indices", "flash_topk_attn"]
