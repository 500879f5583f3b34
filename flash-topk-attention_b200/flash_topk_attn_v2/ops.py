"""Operators of the flash_topk_attn_v2 path on top of the C ABI.

Same names, arguments, checks and exceptions as the reference's operator layer
(flash_topk_attn_v2/block_score.py, topk_select.py, qblock_merge.py,
sparse_attn.py, build_reverse_indices_cuda.py, sort_by_count_cuda.py); the
work itself is done by libftk_sm100.so.  PyTorch is used for device memory and
streams only.
"""

from __future__ import annotations

import math
import os

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr

_SCORE_SCRATCH_BYTES = int(os.environ.get("FTK_SCORE_SCRATCH_BYTES", 4 << 30))
_DEBUG = os.environ.get("FTK_DEBUG", "0") not in ("", "0")
_status_words = {}
_launches = 0


def launch_count() -> int:
    """Kernels of libftk_sm100.so enqueued by this process so far."""
    return _launches


def _count(n: int) -> None:
    global _launches
    _launches += n


# Optional per-call CUDA-event timing (off by default; bench.py switches it on
# around its timed loop).  Every C-ABI call is bracketed by two events on the
# stream it launches on; `event_times()` returns milliseconds per entry point.
_events = None


def enable_event_timing(on: bool) -> None:
    global _events
    _events = [] if on else None


def _call(name, fn, *args) -> None:
    """Run one C-ABI entry point, map its return code, time it when asked."""
    if _events is None:
        check(fn(*args), name)
        return
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    rc = fn(*args)
    e1.record()
    _events.append((name, e0, e1))
    check(rc, name)


def event_times() -> dict:
    """Sum of device milliseconds and call count per entry point since
    enable_event_timing(True); synchronises."""
    out = {}
    if _events:
        torch.cuda.synchronize()
        for name, e0, e1 in _events:
            ms, n = out.get(name, (0.0, 0))
            out[name] = (ms + e0.elapsed_time(e1), n + 1)
    return out


def status_word(device) -> torch.Tensor:
    """Sticky per-device status word handed to every launch."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[key] = t
    return t


def check_errors(device=None) -> None:
    """Synchronise and raise if any launch since the last check reported a
    device-side failure (bounded wait ran out, block id out of range)."""
    for key, t in list(_status_words.items()):
        if device is not None and torch.device(device).index not in (None, key):
            continue
        code = int(t.item())
        snap = _snapshots.get(key)
        if snap is not None:
            snap[0][0] = 0
            snap[1] = None
        if code != 0:
            t.zero_()
            raise RuntimeError(
                f"flash_topk_attn_v2 device error: {_lib.error_text(code)} (status {code})"
            )


# A device-side failure (a bounded wait that ran out, a block id out of range)
# only sets the sticky status word.  So that a caller who never calls
# check_errors() still hears of it, every operator ends by copying the word to
# pinned host memory on its stream (4 bytes, no synchronisation) and begins by
# looking at the copy the previous operator left, if that copy has landed: the
# failure raises at the next call that finds it, usually one call late.
# FTK_DEBUG=1 checks synchronously after every operator instead.
_snapshots = {}
_deferred = True


def deferred_checks(on: bool) -> None:
    """Switch the look at the previous operator's status copy on or off (on by
    default).  Off, a device-side failure is only reported by check_errors()."""
    global _deferred
    _deferred = bool(on)


def _after(device) -> None:
    if _DEBUG:
        if not torch.cuda.is_current_stream_capturing():   # a capture cannot synchronise
            check_errors(device)
        return
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if not _deferred or torch.cuda.is_current_stream_capturing():
        return
    snap = _snapshots.get(key)
    if snap is None:
        snap = _snapshots[key] = [torch.zeros(1, dtype=torch.int32).pin_memory(), None]
    host, ev = snap
    if ev is not None:
        if not ev.query():
            return                       # previous copy still in flight: look next time
        code = int(host[0])
        if code != 0:
            host[0] = 0
            snap[1] = None
            status_word(dev).zero_()
            raise RuntimeError(
                f"flash_topk_attn_v2 device error in an earlier call: {_lib.error_text(code)} "
                f"(status {code})")
    host.copy_(status_word(dev), non_blocking=True)
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(dev))
    snap[1] = ev


def _next_pow2(x: int) -> int:
    return 1 if x <= 1 else 1 << (x - 1).bit_length()


# --------------------------------------------------------------------------
# layout helpers
# --------------------------------------------------------------------------
def _kernel_head_dim(d: int) -> int:
    if d <= 64:
        return 64
    if d <= 128:
        return 128
    if d <= 256:      # 160 and 256 of the reference's list (block_score_cuda.py:16) share one kernel
        return 256
    raise NotImplementedError(f"head dim {d} > 256 is not supported")


def _as_bnhd(x: torch.Tensor, input_4d: bool, H: int, D: int):
    """Return (tensor, sb, sn, sh) addressing x as [b][n][h][d] with d-stride 1,
    16-byte aligned base and strides that are multiples of 8 elements.
    Copies only when the layout cannot be addressed in place."""
    if input_4d:                       # [B, H, N, D]
        if x.stride(3) != 1:
            x = x.contiguous()
        sb, sh, sn = x.stride(0), x.stride(1), x.stride(2)
    else:                              # [B, N, H*D]
        if x.stride(2) != 1:
            x = x.contiguous()
        sb, sn, sh = x.stride(0), x.stride(1), D
    if x.data_ptr() % 16 or sb % 8 or sn % 8 or sh % 8:
        x = x.contiguous()
        if input_4d:
            sb, sh, sn = x.stride(0), x.stride(1), x.stride(2)
        else:
            sb, sn, sh = x.stride(0), x.stride(1), D
        if x.data_ptr() % 16 or sb % 8 or sn % 8 or sh % 8:
            raise ValueError("tensor cannot be aligned to 16 bytes (head dim must be a multiple of 8)")
    return x, sb, sn, sh


def _pad_head_dim(x: torch.Tensor, input_4d: bool, H: int, D: int, Dk: int) -> torch.Tensor:
    """Zero-pad the head dim to the kernel's, as the reference does
    (block_score_cuda.py:130-132, sparse_attn.py:358-373)."""
    if Dk == D:
        return x
    if input_4d:
        return torch.nn.functional.pad(x, (0, Dk - D))
    B, N, _ = x.shape
    return torch.nn.functional.pad(x.reshape(B, N, H, D), (0, Dk - D)).reshape(B, N, H * Dk)


# --------------------------------------------------------------------------
# scoring
# --------------------------------------------------------------------------
def _parse_block_score_args(q, k, num_heads, score_block_size, padding):
    """Argument checks of the reference (block_score.py:369-414)."""
    if q.device.type != "cuda":
        raise ValueError("flash_block_score requires CUDA tensors")
    input_4d = q.ndim == 4
    if input_4d:
        B, H, N, D = q.shape
        if num_heads != H:
            raise ValueError(f"num_heads ({num_heads}) != q.shape[1] ({H})")
        C = H * D
    else:
        if q.ndim != 3:
            raise ValueError("q must be 3D [B, N, C] or 4D [B, H, N, D]")
        B, N, C = q.shape
    H = num_heads
    D = C // H
    pad_head, pad_tail = padding
    if pad_head < 0 or pad_tail < 0:
        raise ValueError("padding must be non-negative (pad_head, pad_tail)")
    if pad_head >= score_block_size or pad_tail >= score_block_size:
        raise ValueError(
            f"padding ({pad_head}, {pad_tail}) must each be < score_block_size "
            f"({score_block_size})"
        )
    n_padded = pad_head + N + pad_tail
    if n_padded % score_block_size != 0:
        need = score_block_size - (n_padded % score_block_size)
        raise ValueError(
            f"pad_head + N + pad_tail = {n_padded} must be divisible by "
            f"score_block_size ({score_block_size}). Try padding=(0, {pad_tail + need})."
        )
    if input_4d:
        if k.shape != (B, H, N, D):
            raise ValueError(f"k shape {k.shape} != {(B, H, N, D)}")
    else:
        if k.shape != (B, N, C):
            raise ValueError(f"k shape {k.shape} != {(B, N, C)}")
    if C % H != 0:
        raise ValueError(f"C={C} not divisible by num_heads={H}")
    if q.dtype != k.dtype:
        raise ValueError(f"q.dtype ({q.dtype}) != k.dtype ({k.dtype})")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("q must be float16, bfloat16, or float32")
    return input_4d, B, H, N, D, n_padded // score_block_size, pad_head, pad_tail


def _prep_qk(q, k, input_4d, H, D):
    if q.dtype == torch.float32:       # block_score_cuda.py:115-118
        q, k = q.bfloat16(), k.bfloat16()
    Dk = _kernel_head_dim(D)
    q = _pad_head_dim(q, input_4d, H, D, Dk)
    k = _pad_head_dim(k, input_4d, H, D, Dk)
    q, *sq = _as_bnhd(q, input_4d, H, Dk)
    k, *sk = _as_bnhd(k, input_4d, H, Dk)
    return q, sq, k, sk, Dk


def flash_block_score(q, k, num_heads, score_block_size, padding=(0, 0)):
    """Softmax mass per (query, score block): [B, H, N, M] float32.

    Mirrors flash_block_score (flash_topk_attn_v2/block_score.py:417-452)."""
    input_4d, B, H, N, D, M, ph, pt = _parse_block_score_args(
        q, k, num_heads, score_block_size, padding)
    qq, sq, kk, sk, Dk = _prep_qk(q, k, input_4d, H, D)
    out = torch.empty(B, H, N, M, dtype=torch.float32, device=q.device)
    status = status_word(q.device)
    # slices are independent; chunk so that launches stay below the grid limit
    step = min(B * H, 32768)
    ws = torch.empty(lib.ftk_block_score_workspace(step, N), dtype=torch.uint8, device=q.device)
    flat = out.view(B * H, N, M)
    for b0 in range(0, B * H, step):
        cnt = min(step, B * H - b0)
        _call("ftk_block_score", lib.ftk_block_score, 
            ptr(qq), ptr(kk), _lib.dtype_code(qq), B, H, N, Dk, *sq, *sk, b0, cnt,
            score_block_size, ph, pt, float(D) ** -0.5, ptr(flat[b0]), ptr(ws), ws.numel(),
            ptr(status), stream_ptr(q.device))
        _count(4)
    _after(q.device)
    return out


def flash_topk_select(block_scores, threshold, max_topk, score_block_size, padding=(0, 0),
                      backend="auto"):
    """Top-k blocks per query with cumulative-threshold cut.

    Mirrors flash_topk_select (flash_topk_attn_v2/topk_select.py:185-311); the
    `backend` argument is accepted for compatibility and ignored (one native
    path, ties keep the lower block id)."""
    if block_scores.ndim != 4:
        raise ValueError("block_scores must be [B, H, N, M]")
    if block_scores.device.type != "cuda":
        raise ValueError("flash_topk_select requires CUDA tensor")
    if block_scores.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("block_scores must be float16/bfloat16/float32")
    B, H, N, M = block_scores.shape
    if M <= 0:
        raise ValueError("M must be positive")
    if score_block_size <= 0:
        raise ValueError("score_block_size must be positive")
    pad_head, pad_tail = padding
    if pad_head < 0 or pad_tail < 0:
        raise ValueError("padding must be non-negative (pad_head, pad_tail)")
    if pad_head >= score_block_size or pad_tail >= score_block_size:
        raise ValueError(
            f"padding ({pad_head}, {pad_tail}) must each be < score_block_size "
            f"({score_block_size})"
        )
    if max_topk < 0:
        raise ValueError("max_topk must be >= 0")
    if backend not in ("auto", "triton", "cuda"):
        raise ValueError(f"backend must be 'auto', 'triton', or 'cuda', got '{backend}'")
    if M > 4096:
        raise NotImplementedError(f"select requires M <= 4096, got M={M}")
    m_out = min(max_topk, M) if max_topk > 0 else M
    scores = block_scores.float().contiguous()
    dev = scores.device
    idx = torch.empty(B, H, N, m_out, dtype=torch.int32, device=dev)
    raw = torch.empty(B, H, N, m_out, dtype=torch.float32, device=dev)
    avg = torch.empty(B, H, N, m_out, dtype=torch.float32, device=dev)
    _call("ftk_topk_select", lib.ftk_topk_select, 
        ptr(scores), 0, B * H * N, M, max_topk, score_block_size, pad_head, pad_tail,
        float(threshold), ptr(idx), ptr(raw), ptr(avg), ptr(status_word(dev)), stream_ptr(dev))
    _count(1)
    _after(dev)
    return idx, raw, avg


def flash_topk_score_fused(q, k, num_heads, score_block_size, topk, padding, threshold):
    """block score + select without materialising [B,H,N,M] for the caller."""
    input_4d, B, H, N, D, M, ph, pt = _parse_block_score_args(
        q, k, num_heads, score_block_size, padding)
    if topk < 0:
        raise ValueError("max_topk must be >= 0")
    if M > 4096:
        raise NotImplementedError(f"select requires M <= 4096, got M={M}")
    qq, sq, kk, sk, Dk = _prep_qk(q, k, input_4d, H, D)
    dev = q.device
    m_out = min(topk, M) if topk > 0 else M
    idx = torch.empty(B, H, N, m_out, dtype=torch.int32, device=dev)
    raw = torch.empty(B, H, N, m_out, dtype=torch.float32, device=dev)
    avg = torch.empty(B, H, N, m_out, dtype=torch.float32, device=dev)
    per_slice = lib.ftk_score_topk_workspace(1, N, M)
    step = int(max(1, min(B * H, 32768, _SCORE_SCRATCH_BYTES // max(per_slice, 1))))
    ws = torch.empty(lib.ftk_score_topk_workspace(step, N, M), dtype=torch.uint8, device=dev)
    status = status_word(dev)
    fi, fr, fa = (t.view(B * H, N, m_out) for t in (idx, raw, avg))
    for b0 in range(0, B * H, step):
        cnt = min(step, B * H - b0)
        _call("ftk_score_topk", lib.ftk_score_topk, 
            ptr(qq), ptr(kk), _lib.dtype_code(qq), B, H, N, Dk, *sq, *sk, b0, cnt,
            score_block_size, ph, pt, float(D) ** -0.5, topk, float(threshold),
            ptr(fi[b0]), ptr(fr[b0]), ptr(fa[b0]), ptr(ws), ws.numel(), ptr(status),
            stream_ptr(dev))
        _count(4)
    _after(dev)
    # lets build_qblock_topk_indices size its table without a device round trip
    idx._ftk_num_score_blocks = M
    return idx, raw, avg


# --------------------------------------------------------------------------
# merge
# --------------------------------------------------------------------------
def num_score_blocks_of(topk_indices) -> int:
    """max(valid id) + 1 (at least 1) of an index tensor: one device reduction
    (ftk_max_index_plus1) and one four-byte read-back, where the reference
    masks, gathers and reduces with PyTorch (__init__.py:101-105)."""
    idx = topk_indices.to(torch.int32).contiguous()
    dev = idx.device
    out = torch.empty(1, dtype=torch.int32, device=dev)
    _call("ftk_max_index_plus1", lib.ftk_max_index_plus1, ptr(idx), idx.numel(), ptr(out),
          stream_ptr(dev))
    _count(2 if idx.numel() else 1)
    return int(out.item())


def flash_qblock_merge(topk_indices, topk_scores, q_block_size, qblock_topk, num_score_blocks,
                       q_padding=(0, 0), return_counts=False):
    """Per-q-block aggregation + ranking of (block, score) pairs.

    Mirrors flash_qblock_merge (flash_topk_attn_v2/qblock_merge.py:85-156).
    `q_padding` is an extension: the reference pads the index tensor on the
    host first (__init__.py:90-96); here the kernel skips the virtual rows."""
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, M_out]")
    if topk_scores is not None and topk_scores.ndim != 4:
        raise ValueError("topk_scores must be [B, H, N, M_out]")
    if topk_indices.device.type != "cuda":
        raise ValueError("flash_qblock_merge requires CUDA tensors")
    B, H, N, K = topk_indices.shape
    qh, qt = q_padding
    if (qh + N + qt) % q_block_size != 0:
        raise ValueError(f"N ({qh + N + qt}) must be divisible by q_block_size ({q_block_size})")
    if num_score_blocks <= 0:
        raise ValueError("num_score_blocks must be positive")
    if num_score_blocks > 4096:
        raise NotImplementedError(
            f"num_score_blocks={num_score_blocks} exceeds CUDA block sort limit 4096")
    if qblock_topk <= 0:
        raise ValueError("qblock_topk must be positive")
    QM = (qh + N + qt) // q_block_size
    dev = topk_indices.device
    idx = topk_indices.to(torch.int32).contiguous()
    scr = None if topk_scores is None else topk_scores.float().contiguous()
    merged = torch.empty(B, H, QM, qblock_topk, dtype=torch.int32, device=dev)
    mscores = torch.empty(B, H, QM, qblock_topk, dtype=torch.float32, device=dev)
    counts = torch.empty(B, H, QM, dtype=torch.int32, device=dev)
    _call("ftk_qblock_merge", lib.ftk_qblock_merge, 
        ptr(idx), ptr(scr), B * H, N, K, q_block_size, qh, qt, num_score_blocks, qblock_topk,
        ptr(merged), ptr(mscores), ptr(counts), ptr(status_word(dev)), stream_ptr(dev))
    _count(1)
    _after(dev)
    if return_counts:
        return merged, mscores, counts
    return merged, mscores


def flash_qblock_union(topk_indices, q_block_size, q_padding=(0, 0), num_score_blocks=None,
                       width=None):
    """Distinct block ids picked inside each q-block, ascending, -1 padded:
    (merged [B, H, QM, width] int32, counts [B, H, QM] int32).

    The exact-union merge of the first-generation operators
    (flash_topk_attn/attention.py:70-138).  `width` defaults to the
    reference's next_pow2(q_block_size * K); `num_score_blocks` bounds the ids
    (default: read back from the indices, one host round trip)."""
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, K]")
    if topk_indices.device.type != "cuda":
        raise ValueError("flash_qblock_union requires CUDA tensors")
    B, H, N, K = topk_indices.shape
    qh, qt = q_padding
    QM = (qh + N + qt) // q_block_size
    dev = topk_indices.device
    idx = topk_indices.to(torch.int32).contiguous()
    if num_score_blocks is None:
        num_score_blocks = max(int(idx.max().item()) + 1, 1)
    if num_score_blocks > 65536:
        raise NotImplementedError(f"num_score_blocks={num_score_blocks} exceeds 65536")
    if width is None:
        width = _next_pow2(q_block_size * K)
    merged = torch.empty(B, H, QM, width, dtype=torch.int32, device=dev)
    counts = torch.empty(B, H, QM, dtype=torch.int32, device=dev)
    _call("ftk_qblock_union", lib.ftk_qblock_union,
          ptr(idx), B * H, N, K, q_block_size, qh, qt, num_score_blocks, width, ptr(merged),
          ptr(counts), ptr(status_word(dev)), stream_ptr(dev))
    _count(1)
    _after(dev)
    return merged, counts


# --------------------------------------------------------------------------
# reverse index / count sort
# --------------------------------------------------------------------------
def flash_build_reverse_indices_cuda(merged_indices, counts, num_kv_blocks):
    """(reverse_indices [B,H,M,QM], reverse_counts [B,H,M], sorted_kv [B,H,M]).

    Mirrors flash_build_reverse_indices_cuda
    (flash_topk_attn_v2/build_reverse_indices_cuda.py:32-78)."""
    B, H, QM, W = merged_indices.shape
    M = num_kv_blocks
    dev = merged_indices.device
    merged = merged_indices.contiguous()
    cnt = None if counts is None else counts.to(torch.int32).contiguous()
    rev = torch.empty(B, H, M, QM, dtype=torch.int32, device=dev)
    rc = torch.empty(B, H, M, dtype=torch.int32, device=dev)
    skv = torch.empty(B, H, M, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.ftk_build_reverse_workspace(B * H, QM, M), dtype=torch.uint8, device=dev)
    _call("ftk_build_reverse", lib.ftk_build_reverse, 
        ptr(merged), ptr(cnt), B * H, QM, W, M, ptr(rev), ptr(rc), ptr(skv), ptr(ws), ws.numel(),
        ptr(status_word(dev)), stream_ptr(dev))
    _count(3)
    _after(dev)
    return rev, rc, skv


def flash_sort_by_count_cuda(reverse_counts, num_heads, num_kv_blocks):
    """Global descending sort of the reverse counts with flat ids.

    Mirrors flash_sort_by_count_cuda (flash_topk_attn_v2/sort_by_count_cuda.py:33-67),
    including its host read of the maximum count."""
    flat = reverse_counts.reshape(-1).to(torch.int32).contiguous()
    total = flat.numel()
    dev = flat.device
    max_val = int(flat.max().item()) if total else 0
    sc = torch.empty_like(flat)
    ids = torch.empty(total, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.ftk_sort_by_count_workspace(total, max_val), dtype=torch.uint8, device=dev)
    _call("ftk_sort_by_count", lib.ftk_sort_by_count, ptr(flat), total, max_val, ptr(sc), ptr(ids), ptr(ws), ws.numel(),
                                stream_ptr(dev))
    _count(3)
    return sc, ids


# --------------------------------------------------------------------------
# sparse attention
# --------------------------------------------------------------------------
def preprocess_delta(o, do, num_heads):
    """delta = rowsum(O * dO), [B, H, N] fp32 (sparse_attn_bwd.py:12-33).
    Host-side convenience; the backward computes it inside ftk_sparse_bwd_dq."""
    B, N, C = o.shape
    D = C // num_heads
    return (o.float().view(B, N, num_heads, D) * do.float().view(B, N, num_heads, D)).sum(-1) \
        .permute(0, 2, 1).contiguous()


class FlashSparseAttnFunc(torch.autograd.Function):
    """Forward and backward of the gathered-KV attention
    (reference: FlashSparseAttnFunc, flash_topk_attn_v2/sparse_attn.py:130-224)."""

    @staticmethod
    def forward(ctx, q, k, v, merged_indices, num_heads, q_block_size, kv_block_size, scale,
                q_pad_head, kv_pad_head, num_kv_blocks, num_kv_heads=None):
        B, N, C = q.shape
        H = num_heads
        Hkv = num_kv_heads or H
        D = C // H
        dev = q.device
        qq, sq_b, sq_n, sq_h = _as_bnhd(q, False, H, D)
        kk, sk_b, sk_n, sk_h = _as_bnhd(k, False, Hkv, D)
        vv, sv_b, sv_n, sv_h = _as_bnhd(v, False, Hkv, D)
        merged = merged_indices.contiguous()
        QM, W = merged.shape[2], merged.shape[3]
        o = torch.empty(B, N, C, dtype=q.dtype, device=dev)
        lse = torch.empty(B, H, N, dtype=torch.float32, device=dev)
        ws_bytes = int(lib.ftk_sparse_fwd_workspace(B, H, QM, q_block_size))
        ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
        _call("ftk_sparse_fwd", lib.ftk_sparse_fwd, 
            ptr(qq), ptr(kk), ptr(vv), _lib.dtype_code(qq), B, H, Hkv, N, D,
            sq_b, sq_n, sq_h, sk_b, sk_n, sk_h, sv_b, sv_n, sv_h,
            ptr(merged), QM, W, q_block_size, kv_block_size, q_pad_head, kv_pad_head,
            float(scale), ptr(o), N * C, C, D, ptr(lse), ptr(ws), ws_bytes,
            ptr(status_word(dev)), stream_ptr(dev))
        piped = (kv_block_size == 64 and q_block_size in (32, 64)
                 and os.environ.get("FTK_FWD_PIPE", "1")[:1] != "0")
        _count(2 if piped else 1)
        _after(dev)
        ctx.save_for_backward(qq, kk, vv, o, lse, merged)
        ctx.meta = (H, D, q_block_size, kv_block_size, float(scale), q_pad_head, kv_pad_head,
                    num_kv_blocks, Hkv)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, grad_o, _grad_lse):
        qq, kk, vv, o, lse, merged = ctx.saved_tensors
        H, D, g, kvb, scale, qph, kph, M, Hkv = ctx.meta
        B, N, C = qq.shape
        dev = qq.device
        _check_backward_blocks(D, g, kvb)
        if D > 128 and (g > 32 or kvb > 32):
            # head dim 256: the gradient kernels hold Q / dO (dQ) or K / V (dK, dV) of 256
            # columns in shared memory and have room for 32-row partner tiles only
            merged, g, kvb, qph, kph, M = _split_large_blocks(merged, N, g, kvb, qph, kph, 32)
        do, sdo_b, sdo_n, sdo_h = _as_bnhd(grad_o.to(qq.dtype), False, H, D)
        _, sq_b, sq_n, sq_h = _as_bnhd(qq, False, H, D)
        _, sk_b, sk_n, sk_h = _as_bnhd(kk, False, Hkv, D)
        _, sv_b, sv_n, sv_h = _as_bnhd(vv, False, Hkv, D)
        QM, W = merged.shape[2], merged.shape[3]
        status = status_word(dev)
        st = stream_ptr(dev)
        delta = torch.empty(B, H, N, dtype=torch.float32, device=dev)
        dq = torch.empty(B, N, C, dtype=qq.dtype, device=dev)
        dk = torch.empty(B, N, C, dtype=qq.dtype, device=dev)
        dv = torch.empty(B, N, C, dtype=qq.dtype, device=dev)
        dt = _lib.dtype_code(qq)
        _call("ftk_sparse_bwd_dq", lib.ftk_sparse_bwd_dq, 
            ptr(qq), ptr(kk), ptr(vv), ptr(o), ptr(do), dt, B, H, Hkv, N, D,
            sq_b, sq_n, sq_h, sk_b, sk_n, sk_h, sv_b, sv_n, sv_h, N * C, C, D,
            sdo_b, sdo_n, sdo_h, ptr(merged), QM, W, g, kvb, qph, kph, scale,
            ptr(lse), ptr(delta), ptr(dq), N * C, C, D, ptr(status), st)
        _count(2)
        rev, rc, skv = flash_build_reverse_indices_cuda(merged, None, M)
        _call("ftk_sparse_bwd_dkv", lib.ftk_sparse_bwd_dkv, 
            ptr(qq), ptr(kk), ptr(vv), ptr(do), dt, B, H, Hkv, N, D,
            sq_b, sq_n, sq_h, sk_b, sk_n, sk_h, sv_b, sv_n, sv_h, sdo_b, sdo_n, sdo_h,
            ptr(rev), ptr(rc), ptr(skv), QM, M, g, kvb, qph, kph, scale,
            ptr(lse), ptr(delta), ptr(dk), N * C, C, D, ptr(dv), N * C, C, D, W, ptr(status), st)
        _count(1)
        _after(dev)
        if Hkv != H:
            # the kernel wrote one dK / dV per query head: add up each group of
            # H / Hkv heads (fp32) to get the gradient of their shared kv head
            grp = H // Hkv
            dk = dk.view(B, N, Hkv, grp, D).float().sum(3).to(qq.dtype).view(B, N, Hkv * D)
            dv = dv.view(B, N, Hkv, grp, D).float().sum(3).to(qq.dtype).view(B, N, Hkv * D)
        return dq, dk, dv, None, None, None, None, None, None, None, None, None


def _check_backward_blocks(D, g, kvb):
    """Block sizes the gradient kernels take (the reference's take any q block of
    1..64 rows and any kv block): multiples of 16 rows, and at head dims above 128
    sizes that halve down to 16 or 32 rows."""
    if g % 16 != 0:
        raise NotImplementedError(
            f"the backward needs a q_block_size that is a multiple of 16, got {g}")
    if D > 128:
        for name, blk in (("q_block_size", g), ("kv_block_size", kvb)):
            part = blk
            while part > 32 and part % 2 == 0:
                part //= 2
            if part > 32 or part % 16 != 0:
                raise NotImplementedError(
                    f"backward at head dim > 128 needs a {name} that halves down to 16 or "
                    f"32 rows (16, 32, 64, 128), got {blk}")


def _split_large_blocks(merged, N, g, kvb, q_pad_head, kv_pad_head, limit=64):
    """Lists over blocks of more than `limit` rows (65..128 for the default),
    restated over half-size blocks, repeatedly if need be.

    The kernels work on q / kv blocks of at most 64 rows.  A block of `kvb` rows
    that starts at token j*kvb - pad is exactly the two half blocks
    2j - s, 2j - s + 1 of a grid with block kvb/2 and pad head pad - s*kvb/2,
    where s = 1 when the pad head covers the first half block; each listed id
    becomes those two ids (halves that lie before token 0 or at / after token N
    are dropped).  q-blocks split the same way: both halves of a q-block take
    its list.  Returns (merged', g', kvb', q_pad_head', kv_pad_head', M')."""
    while kvb > limit:
        half = kvb // 2
        s = 1 if kv_pad_head >= half else 0
        kv_pad_head -= s * half
        sub0 = 2 * merged - s
        sub = torch.stack([sub0, sub0 + 1], dim=-1)
        start = sub.to(torch.int64) * half - kv_pad_head
        keep = (merged >= 0).unsqueeze(-1) & (sub >= 0) & (start < N)
        merged = torch.where(keep, sub, torch.full_like(sub, -1)).flatten(-2)
        kvb = half
    while g > limit:
        half = g // 2
        s = 1 if q_pad_head >= half else 0
        q_pad_head -= s * half
        qm2 = 2 * merged.shape[2] - s
        parent = (torch.arange(qm2, device=merged.device) + s) // 2
        merged = merged.index_select(2, parent)
        g = half
    m_kv = (kv_pad_head + N + kvb - 1) // kvb
    return merged.contiguous(), g, kvb, q_pad_head, kv_pad_head, m_kv


def flash_sparse_attn(q, k, v, merged_indices, num_heads, q_block_size, kv_block_size,
                      scale=None, q_padding=(0, 0), kv_padding=(0, 0), num_kv_heads=None):
    """Block-sparse attention, differentiable in q, k, v: (O [B,N,C], lse [B,H,N]).

    Mirrors flash_sparse_attn (flash_topk_attn_v2/sparse_attn.py:227-392)
    including its argument checks, with one extension: q and kv blocks of up to
    128 rows (multiples of 32 above 64) are accepted for forward and backward;
    the reference rejects q blocks above 64 (sparse_attn.py:279) and its
    dK/dV kernel is only correct up to 64-row kv blocks.  `num_kv_heads`
    (grouped-query attention, also beyond the reference): k and v are
    [B, N, num_kv_heads * D] and query head h reads kv head
    h // (num_heads // num_kv_heads)."""
    if q.ndim != 3:
        raise ValueError("q must be [B, N, C]")
    if q.device.type != "cuda":
        raise ValueError("flash_sparse_attn requires CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("q must be float16, bfloat16, or float32")
    orig_dtype = q.dtype
    if orig_dtype == torch.float32:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    B, N, C = q.shape
    H = num_heads
    D = C // H
    if C != H * D:
        raise ValueError(f"C ({C}) must be divisible by num_heads ({H})")
    Hkv = H if num_kv_heads is None else int(num_kv_heads)
    if Hkv <= 0 or H % Hkv != 0:
        raise ValueError(f"num_heads ({H}) must be a multiple of num_kv_heads ({Hkv})")
    if k.shape != (B, N, Hkv * D) or v.shape != (B, N, Hkv * D):
        raise ValueError(f"k and v must be [B, N, num_kv_heads * D] = {(B, N, Hkv * D)}")
    if q_block_size <= 0 or q_block_size > 128:
        raise ValueError(f"q_block_size must be in (0, 128], got {q_block_size}")
    if kv_block_size <= 0:
        raise ValueError(f"kv_block_size must be positive, got {kv_block_size}")
    if kv_block_size > 128:
        raise NotImplementedError(f"kv_block_size must be <= 128, got {kv_block_size}")
    for name, blk in (("q_block_size", q_block_size), ("kv_block_size", kv_block_size)):
        if blk > 64 and blk % 32 != 0:
            raise NotImplementedError(f"{name} above 64 must be a multiple of 32, got {blk}")
    if merged_indices.ndim != 4:
        raise ValueError("merged_indices must be [B, H, QM, qblock_topk]")
    if merged_indices.dtype != torch.int32:
        raise ValueError("merged_indices must be int32")
    q_pad_head, q_pad_tail = q_padding
    kv_pad_head, kv_pad_tail = kv_padding
    if q_pad_head < 0 or q_pad_tail < 0:
        raise ValueError("q_padding values must be non-negative")
    if kv_pad_head < 0 or kv_pad_tail < 0:
        raise ValueError("kv_padding values must be non-negative")
    if q_pad_head >= q_block_size:
        raise ValueError(f"q_pad_head={q_pad_head} must be < q_block_size={q_block_size}")
    if q_pad_tail >= q_block_size:
        raise ValueError(f"q_pad_tail={q_pad_tail} must be < q_block_size={q_block_size}")
    if kv_pad_head >= kv_block_size:
        raise ValueError(f"kv_pad_head={kv_pad_head} must be < kv_block_size={kv_block_size}")
    if kv_pad_tail >= kv_block_size:
        raise ValueError(f"kv_pad_tail={kv_pad_tail} must be < kv_block_size={kv_block_size}")
    n_q = q_pad_head + N + q_pad_tail
    n_kv = kv_pad_head + N + kv_pad_tail
    if n_q % q_block_size != 0:
        raise ValueError(
            f"q_pad_head + N + q_pad_tail = {n_q} must be divisible by q_block_size={q_block_size}")
    if n_kv % kv_block_size != 0:
        raise ValueError(
            f"kv_pad_head + N + kv_pad_tail = {n_kv} must be divisible by "
            f"kv_block_size={kv_block_size}")
    QM = n_q // q_block_size
    if merged_indices.shape[2] != QM:
        raise ValueError(
            f"merged_indices dim 2 ({merged_indices.shape[2]}) must match "
            f"QM = (q_pad_head + N + q_pad_tail) // q_block_size = {QM}")
    if D <= 0 or D % 16 != 0:
        raise ValueError(f"D ({D}) must be a positive multiple of 16")
    if D > 256:
        raise ValueError(f"D ({D}) must be <= 256")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    Dk = _kernel_head_dim(D)
    if Dk != D:
        q = _pad_head_dim(q, False, H, D, Dk)
        k = _pad_head_dim(k, False, Hkv, D, Dk)
        v = _pad_head_dim(v, False, Hkv, D, Dk)
    num_kv_blocks = n_kv // kv_block_size
    if q_block_size > 64 or kv_block_size > 64:
        (merged_indices, q_block_size, kv_block_size, q_pad_head, kv_pad_head,
         num_kv_blocks) = _split_large_blocks(
            merged_indices, N, q_block_size, kv_block_size, q_pad_head, kv_pad_head)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        # say so now rather than inside backward()
        _check_backward_blocks(Dk, q_block_size, kv_block_size)
    o, lse = FlashSparseAttnFunc.apply(
        q, k, v, merged_indices, H, q_block_size, kv_block_size, scale, q_pad_head, kv_pad_head,
        num_kv_blocks, Hkv)
    if Dk != D:
        o = o.view(B, N, H, Dk)[..., :D].reshape(B, N, C)
    if orig_dtype == torch.float32:
        o = o.float()
    return o, lse
