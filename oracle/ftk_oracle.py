"""CPU restatement of the flash_topk_attn_v2 hot path (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only the test-suite, the smoke
entry point and the benchmark's CPU-baseline leg may import it.  The shipped
package never does and fails loudly when its CUDA library is missing.

Every function restates, in numpy, the algorithm of one reference operator and
names the reference lines it follows (paths inside the reference project).
Parity is pinned: the functions are checked against outputs of the reference's
own `_naive` PyTorch twins, stored under tests/golden/ by
tests/golden/make_golden.py (see tests/test_oracle_golden.py).

Conventions
  * q, k, v are float arrays of shape [B, N, H*D] whose values already carry
    the rounding of the dtype under test (fp16 / bf16 values stored exactly in
    fp32/fp64).  The reference casts fp32 inputs to bf16 the same way
    (flash_topk_attn_v2/block_score_cuda.py:115-118).
  * `work` selects the arithmetic of the dense parts: np.float64 for the
    arbiter used by the parity tests, np.float32 for the timed CPU baseline.
  * Ties: wherever the reference leaves the order of equal keys to a library
    sort, this file uses (key descending, lower block id first), the order the
    reference's CUB kernels produce (csrc/topk_select_kernel.cu:62,
    csrc/qblock_merge_kernel.cu:71).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np

__all__ = [
    "block_geometry",
    "block_score",
    "topk_select",
    "flash_topk_score",
    "qblock_merge",
    "build_qblock_topk_indices",
    "sparse_attn_fwd",
    "round_to_dtype",
    "UNIT_ROUNDOFF",
    "sparse_attn_bwd",
    "preprocess_delta",
    "build_reverse_indices",
    "sort_by_count",
    "classify_topk_mismatches",
    "v1_topk_score",
    "v1_qblock_union",
    "v1_topk_attn",
]


# --------------------------------------------------------------------------
# geometry helpers
# --------------------------------------------------------------------------
def block_geometry(n: int, block: int, padding: Tuple[int, int]):
    """Blocks of `block` virtual tokens over [-pad_head, n + pad_tail).

    Returns (M, starts, ends, valid) with block j covering the real tokens
    [starts[j], ends[j]) and valid[j] = ends[j] - starts[j].
    Follows flash_topk_attn_v2/block_score.py:340-365 (argument checks and the
    slice loop) and csrc/topk_select_kernel.cu:55-58 (valid counts).
    """
    ph, pt = padding
    if ph < 0 or pt < 0:
        raise ValueError("padding must be non-negative (pad_head, pad_tail)")
    if ph >= block or pt >= block:
        raise ValueError(
            f"padding ({ph}, {pt}) must each be < score_block_size ({block})"
        )
    total = ph + n + pt
    if total % block != 0:
        raise ValueError(
            f"pad_head + N + pad_tail = {total} must be divisible by "
            f"score_block_size ({block})"
        )
    m = total // block
    starts = np.maximum(np.arange(m) * block - ph, 0)
    ends = np.minimum((np.arange(m) + 1) * block - ph, n)
    valid = np.maximum(ends - starts, 0)
    return m, starts, ends, valid


def _split_heads(x: np.ndarray, h: int) -> np.ndarray:
    b, n, c = x.shape
    if c % h != 0:
        raise ValueError(f"C={c} not divisible by num_heads={h}")
    return x.reshape(b, n, h, c // h).transpose(0, 2, 1, 3)


# --------------------------------------------------------------------------
# a2  block score
# --------------------------------------------------------------------------
def block_score(
    q: np.ndarray,
    k: np.ndarray,
    num_heads: int,
    score_block_size: int,
    padding: Tuple[int, int] = (0, 0),
    work=np.float64,
    row_chunk: int = 2048,
) -> np.ndarray:
    """Softmax mass of every query over every score block, [B,H,N,M].

    s_t(j) = sum_{i in block j} softmax_i(q_t . k_i / sqrt(D)), softmax over
    all N real keys; blocks clipped to [0, N).  Restates
    `_flash_block_score_naive` (flash_topk_attn_v2/block_score.py:295-366).
    Rows are processed in chunks so the N x N matrix is never held whole.
    """
    b, n, c = q.shape
    if k.shape != (b, n, c):
        raise ValueError(f"k shape {k.shape} != {(b, n, c)}")
    m, starts, ends, _ = block_geometry(n, score_block_size, padding)
    d = c // num_heads
    scale = d ** -0.5
    qh = _split_heads(q, num_heads).astype(work)
    kh = _split_heads(k, num_heads).astype(work)
    out = np.zeros((b, num_heads, n, m), dtype=work)
    # cumulative-sum trick: block sums are differences of a running sum at
    # block boundaries; done with reduceat on the non-empty blocks instead so
    # that every block is an independent sum (as in the reference loop).
    nonempty = ends > starts
    ne_idx = np.nonzero(nonempty)[0]
    for bi in range(b):
        for hi in range(num_heads):
            kt = kh[bi, hi].T
            for r0 in range(0, n, row_chunk):
                r1 = min(n, r0 + row_chunk)
                s = (qh[bi, hi, r0:r1] * work(scale)) @ kt
                s -= s.max(axis=1, keepdims=True)
                np.exp(s, out=s)
                s /= s.sum(axis=1, keepdims=True)
                sums = np.add.reduceat(s, starts[ne_idx], axis=1)
                # reduceat runs each segment to the next start; the last one
                # to the end of the row, which is `ends[-1] == n` by
                # construction, so segments equal the blocks.
                out[bi, hi, r0:r1][:, ne_idx] = sums
    return out


# --------------------------------------------------------------------------
# a3  top-k select
# --------------------------------------------------------------------------
def topk_select(
    block_scores: np.ndarray,
    threshold: float,
    max_topk: int,
    score_block_size: int,
    padding: Tuple[int, int] = (0, 0),
) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Sort blocks by average score, cut at the cumulative-raw threshold.

    fp32 arithmetic throughout, exactly as `_flash_topk_select_naive`
    (flash_topk_attn_v2/topk_select.py:128-182): avg = raw / valid_count
    (IEEE division), descending sort by avg, raw gathered (not recomputed),
    sequential fp32 cumulative sum, first position whose running sum reaches
    `threshold` (inclusive) else the last, capped at M_OUT = min(max_topk, M)
    (max_topk == 0 means M).  Entries past the cut are (-1, 0, 0).
    Equal averages: lower block id first (csrc/topk_select_kernel.cu:62).
    """
    if block_scores.ndim != 4:
        raise ValueError("block_scores must be [B, H, N, M]")
    ph, pt = padding
    if ph < 0 or pt < 0:
        raise ValueError("padding must be non-negative (pad_head, pad_tail)")
    if ph >= score_block_size or pt >= score_block_size:
        raise ValueError(
            f"padding ({ph}, {pt}) must each be < score_block_size "
            f"({score_block_size})"
        )
    if max_topk < 0:
        raise ValueError("max_topk must be >= 0")
    m = block_scores.shape[-1]
    raw = block_scores.astype(np.float32)
    valid = np.full((m,), float(score_block_size), dtype=np.float32)
    if ph > 0:
        valid[0] = float(score_block_size - ph)
    if pt > 0:
        valid[-1] = float(score_block_size - pt)
    avg = (raw / valid).astype(np.float32)
    # stable argsort of the negated key = descending, lower id first on ties
    order = np.argsort(-avg, axis=-1, kind="stable")
    s_avg = np.take_along_axis(avg, order, axis=-1)
    s_raw = np.take_along_axis(raw, order, axis=-1)
    cs = np.cumsum(s_raw, axis=-1, dtype=np.float32)
    exceed = cs >= np.float32(threshold)
    has = exceed.any(axis=-1)
    first = np.where(has, exceed.argmax(axis=-1), m - 1)
    m_out = min(max_topk, m) if max_topk > 0 else m
    if m_out < m:
        first = np.minimum(first, m_out - 1)
    keep = (np.arange(m) <= first[..., None])[..., :m_out]
    idx = np.where(keep, order[..., :m_out], -1).astype(np.int32)
    o_raw = np.where(keep, s_raw[..., :m_out], 0.0).astype(np.float32)
    o_avg = np.where(keep, s_avg[..., :m_out], 0.0).astype(np.float32)
    return idx, o_raw, o_avg


def flash_topk_score(
    q, k, num_heads, score_block_size=64, topk=16, padding=(0, 0),
    threshold=1.0, work=np.float64,
):
    """block_score followed by topk_select (flash_topk_attn_v2/__init__.py:16-54).

    Returns (idx, raw, avg, scores) where `scores` is the [B,H,N,M] block-score
    matrix in `work` precision (kept for tie classification).
    """
    scores = block_score(q, k, num_heads, score_block_size, padding, work=work)
    idx, raw, avg = topk_select(
        scores.astype(np.float32), threshold, topk, score_block_size, padding
    )
    return idx, raw, avg, scores


# --------------------------------------------------------------------------
# a4/a5  q-block merge
# --------------------------------------------------------------------------
def qblock_merge(
    topk_indices: np.ndarray,
    topk_scores: np.ndarray,
    q_block_size: int,
    qblock_topk: int,
    num_score_blocks: int,
) -> Tuple[np.ndarray, np.ndarray]:
    """Aggregate per-query (block, score) pairs per q-block and rank them.

    agg[j] = sum of the scores of every entry of the q-block that names block
    j, summed in fp32 in row-major entry order (query row, then rank), which
    is the order `scatter_add_` applies on the host
    (flash_topk_attn_v2/qblock_merge.py:52-64).  Output: blocks with agg > 0
    by agg descending (ties: lower id first, csrc/qblock_merge_kernel.cu:71),
    cut to `qblock_topk`, padded with (-1, 0.0) to exactly that width
    (qblock_merge.py:66-80, csrc/qblock_merge_kernel.cu:75-88).
    """
    if topk_indices.ndim != 4 or topk_scores.ndim != 4:
        raise ValueError("topk_indices/topk_scores must be [B, H, N, M_out]")
    b, h, n, k = topk_indices.shape
    if n % q_block_size != 0:
        raise ValueError(
            f"N ({n}) must be divisible by q_block_size ({q_block_size})"
        )
    if num_score_blocks <= 0:
        raise ValueError("num_score_blocks must be positive")
    if qblock_topk <= 0:
        raise ValueError("qblock_topk must be positive")
    qm = n // q_block_size
    flat = q_block_size * k
    idx = topk_indices.reshape(b * h * qm, flat).astype(np.int64)
    scr = topk_scores.astype(np.float32).reshape(b * h * qm, flat)
    rows = idx.shape[0]
    agg = np.zeros((rows, num_score_blocks), dtype=np.float32)
    valid = idx >= 0
    # sequential fp32 accumulation in entry order: loop over the entry axis,
    # vectorised over q-blocks (entries of one column never collide).
    row_ids = np.arange(rows)
    for e in range(flat):
        v = valid[:, e]
        if v.any():
            r = row_ids[v]
            agg[r, idx[v, e]] += scr[v, e]
    order = np.argsort(-agg, axis=-1, kind="stable")
    s_agg = np.take_along_axis(agg, order, axis=-1)
    take = min(qblock_topk, num_score_blocks)
    order = order[:, :take]
    s_agg = s_agg[:, :take]
    bad = s_agg <= 0.0
    m_idx = np.where(bad, -1, order).astype(np.int32)
    m_scr = np.where(bad, 0.0, s_agg).astype(np.float32)
    if qblock_topk > take:
        pad = qblock_topk - take
        m_idx = np.pad(m_idx, ((0, 0), (0, pad)), constant_values=-1)
        m_scr = np.pad(m_scr, ((0, 0), (0, pad)), constant_values=0.0)
    return (
        m_idx.reshape(b, h, qm, qblock_topk),
        m_scr.reshape(b, h, qm, qblock_topk),
    )


def build_qblock_topk_indices(
    topk_indices: np.ndarray,
    q_block_size: int,
    q_padding: Tuple[int, int] = (0, 0),
    topk_scores: Optional[np.ndarray] = None,
    qblock_topk: Optional[int] = None,
):
    """Glue of flash_topk_attn_v2/__init__.py:57-133.

    Pads the query axis with all-(-1) rows for the virtual q padding, gives
    every valid entry the weight 1.0 when no scores are passed, sizes the
    aggregation table as max(valid id)+1 and returns
    (merged [B,H,QM,W] int32, counts [B,H,QM] int32, W, merged_scores).
    """
    if topk_indices.ndim != 4:
        raise ValueError("topk_indices must be [B, H, N, K]")
    _, _, n, kw = topk_indices.shape
    qh, qt = q_padding
    if qh < 0 or qt < 0:
        raise ValueError("q_padding must be non-negative")
    if qh >= q_block_size:
        raise ValueError(f"q_pad_head={qh} must be < q_block_size={q_block_size}")
    if qt >= q_block_size:
        raise ValueError(f"q_pad_tail={qt} must be < q_block_size={q_block_size}")
    if (qh + n + qt) % q_block_size != 0:
        raise ValueError(
            f"q_pad_head + N + q_pad_tail = {qh + n + qt} must be divisible "
            f"by q_block_size ({q_block_size})"
        )
    idx = topk_indices.astype(np.int32)
    pad = ((0, 0), (0, 0), (qh, qt), (0, 0))
    idx = np.pad(idx, pad, constant_values=-1)
    if qblock_topk is None:
        qblock_topk = q_block_size * kw
    valid = idx >= 0
    m_total = int(idx[valid].max()) + 1 if valid.any() else 1
    if topk_scores is not None:
        scr = np.pad(topk_scores.astype(np.float32), pad, constant_values=0.0)
    else:
        scr = valid.astype(np.float32)
    merged, mscores = qblock_merge(idx, scr, q_block_size, qblock_topk, m_total)
    counts = (merged >= 0).sum(axis=-1).astype(np.int32)
    return merged, counts, merged.shape[-1], mscores


# --------------------------------------------------------------------------
# a6  sparse attention forward
# --------------------------------------------------------------------------
def _kv_token_mask(blocks: np.ndarray, n: int, kvb: int, kv_pad_head: int):
    mask = np.zeros(n, dtype=bool)
    for j in blocks:
        s = max(0, int(j) * kvb - kv_pad_head)
        e = min(n, (int(j) + 1) * kvb - kv_pad_head)
        if s < e:
            mask[s:e] = True
    return mask


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Round to the nearest fp16 / bf16 value (ties to even), kept in x's dtype."""
    x = np.asarray(x)
    if dtype == "fp16":
        return x.astype(np.float16).astype(x.dtype)
    if dtype != "bf16":
        raise ValueError(dtype)
    f = np.ascontiguousarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = u.astype(np.uint32).view(np.float32).reshape(f.shape)
    return np.where(np.isfinite(f), out, f).astype(x.dtype)


# unit roundoff (half an ulp, relative) of the two 16-bit formats
UNIT_ROUNDOFF = {"fp16": 2.0 ** -12, "bf16": 2.0 ** -9}


def sparse_attn_fwd(
    q, k, v, merged_indices, num_heads, q_block_size, kv_block_size,
    scale=None, q_padding=(0, 0), kv_padding=(0, 0), work=np.float64,
    roundings=None, io_dtype=None, envelope=False,
):
    """Gathered-KV attention per q-block: returns (O [B,N,C], lse [B,H,N]).

    Every real query row of q-block m attends to the union of the tokens of
    its candidate KV blocks; an empty candidate set gives O = 0, lse = -inf.
    Restates `_flash_sparse_attn_naive`
    (flash_topk_attn_v2/sparse_attn.py:24-127); O is left unrounded.

    `roundings="reference"` (with `io_dtype` "fp16" | "bf16") applies the
    roundings of the reference's GPU kernel on top of exact arithmetic: the
    probabilities exp(s - rowmax) are rounded to the I/O dtype before P.V
    while the row sum uses the unrounded ones
    (csrc/sparse_attn_kernel.cu:282-309), and O is rounded to the I/O dtype
    when stored (:333-342).  The kernel rounds against its running maximum;
    here the final row maximum is used, which moves individual roundings but
    not their size.  `envelope=True` additionally returns a first-order
    worst-case bound on |O_rounded - O_exact| per element (u * sum_i P_i |v_i|
    / l for the rounding of P plus u |O| for the store), u the unit roundoff.
    """
    if roundings not in (None, "reference"):
        raise ValueError(f"roundings must be None or 'reference', got {roundings!r}")
    if (roundings or envelope) and io_dtype not in UNIT_ROUNDOFF:
        raise ValueError("io_dtype must be 'fp16' or 'bf16'")
    b, n, c = q.shape
    h = num_heads
    d = c // h
    qh_, qt_ = q_padding
    kh_, kt_ = kv_padding
    if (qh_ + n + qt_) % q_block_size != 0:
        raise ValueError("q padding does not tile")
    if (kh_ + n + kt_) % kv_block_size != 0:
        raise ValueError("kv padding does not tile")
    qm = (qh_ + n + qt_) // q_block_size
    if merged_indices.shape[:3] != (b, h, qm):
        raise ValueError("merged_indices shape mismatch")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    qq = _split_heads(q, h).astype(work)
    kk = _split_heads(k, h).astype(work)
    vv = _split_heads(v, h).astype(work)
    out = np.zeros((b, h, n, d), dtype=work)
    env = np.zeros((b, h, n, d), dtype=work) if envelope else None
    lse = np.full((b, h, n), -np.inf, dtype=work)
    u = UNIT_ROUNDOFF.get(io_dtype, 0.0)
    for bi in range(b):
        for hi in range(h):
            for m in range(qm):
                r0 = max(0, m * q_block_size - qh_)
                r1 = min(n, (m + 1) * q_block_size - qh_)
                if r0 >= r1:
                    continue
                row = merged_indices[bi, hi, m]
                blocks = row[row >= 0]
                if blocks.size == 0:
                    continue
                tok = np.nonzero(_kv_token_mask(blocks, n, kv_block_size, kh_))[0]
                if tok.size == 0:
                    continue
                s = (qq[bi, hi, r0:r1] * work(scale)) @ kk[bi, hi, tok].T
                mx = s.max(axis=1, keepdims=True)
                p = np.exp(s - mx)
                l = p.sum(axis=1, keepdims=True)
                if roundings:
                    out[bi, hi, r0:r1] = (round_to_dtype(p, io_dtype) @ vv[bi, hi, tok]) / l
                else:
                    out[bi, hi, r0:r1] = (p / l) @ vv[bi, hi, tok]
                if envelope:
                    env[bi, hi, r0:r1] = u * ((p / l) @ np.abs(vv[bi, hi, tok]))
                lse[bi, hi, r0:r1] = (mx + np.log(l))[:, 0]
    o = out.transpose(0, 2, 1, 3).reshape(b, n, c)
    if roundings:
        o = round_to_dtype(o, io_dtype)
    if envelope:
        e = env.transpose(0, 2, 1, 3).reshape(b, n, c) + u * np.abs(o)
        return o, lse, e
    return o, lse


# --------------------------------------------------------------------------
# a7-a10  backward
# --------------------------------------------------------------------------
def preprocess_delta(o: np.ndarray, do: np.ndarray, num_heads: int) -> np.ndarray:
    """delta[b,h,t] = sum_d O*dO (flash_topk_attn_v2/sparse_attn_bwd.py:12-33)."""
    oh = _split_heads(o, num_heads)
    dh = _split_heads(do, num_heads)
    return (oh * dh).sum(axis=-1)


def sparse_attn_bwd(
    q, k, v, o, lse, do, merged_indices, num_heads, q_block_size,
    kv_block_size, scale=None, q_padding=(0, 0), kv_padding=(0, 0),
    work=np.float64, roundings=None, io_dtype=None, envelope=False, o_envelope=None,
):
    """Closed-form gradients of sparse_attn_fwd: (dQ, dK, dV), each [B,N,C].

    P = exp(scale q.k - lse) on the candidate tokens, delta = rowsum(O*dO),
    dS = P*(dO.v - delta), dQ = scale dS K, dK = scale dS^T Q, dV = P^T dO.
    Restates `bwd_dq_naive` / `bwd_dkv_naive`
    (flash_topk_attn_v2/sparse_attn_bwd.py:111-199, 202-294).  `o` is the
    forward output as stored (rounded to the I/O dtype), as the reference
    computes delta from it (sparse_attn.py:163-175).

    `roundings="reference"` (with `io_dtype`) applies the roundings of the
    reference's GPU kernels on top of exact arithmetic: dS is rounded to the
    I/O dtype before dS.K (csrc/sparse_attn_bwd_dq_kernel.cu:355-358), P and dS
    before P^T.dO and dS^T.Q (csrc/sparse_attn_bwd_dkv_kernel.cu:314-317,
    353-356), lse is the stored fp32 value and the gradients are rounded to the
    I/O dtype when stored.  `envelope=True` additionally returns, per gradient,
    a first-order worst-case bound on what those roundings can move an element
    by (`o_envelope`, the forward's bound, carries the rounding of O into
    delta); the result is (dQ, dK, dV, (eQ, eK, eV)).
    """
    if roundings not in (None, "reference"):
        raise ValueError(f"roundings must be None or 'reference', got {roundings!r}")
    if (roundings or envelope) and io_dtype not in UNIT_ROUNDOFF:
        raise ValueError("io_dtype must be 'fp16' or 'bf16'")
    b, n, c = q.shape
    h = num_heads
    d = c // h
    qh_, _ = q_padding
    kh_, _ = kv_padding
    qm = merged_indices.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    qq = _split_heads(q, h).astype(work)
    kk = _split_heads(k, h).astype(work)
    vv = _split_heads(v, h).astype(work)
    dd = _split_heads(do, h).astype(work)
    delta = preprocess_delta(o.astype(work), do.astype(work), h)
    dq = np.zeros((b, h, n, d), dtype=work)
    dk = np.zeros((b, h, n, d), dtype=work)
    dv = np.zeros((b, h, n, d), dtype=work)
    u = UNIT_ROUNDOFF.get(io_dtype, 0.0)
    if envelope:
        eq, ek, ev = (np.zeros((b, h, n, d), dtype=work) for _ in range(3))
        # |error of delta| <= sum_d |error of O| |dO|
        oe = o_envelope if o_envelope is not None else u * np.abs(o)
        ddelta = (_split_heads(oe.astype(work), h) * np.abs(dd)).sum(axis=-1)
    if roundings:
        lse = np.asarray(lse, dtype=np.float32)
    for bi in range(b):
        for hi in range(h):
            for m in range(qm):
                r0 = max(0, m * q_block_size - qh_)
                r1 = min(n, (m + 1) * q_block_size - qh_)
                if r0 >= r1:
                    continue
                row = merged_indices[bi, hi, m]
                blocks = row[row >= 0]
                if blocks.size == 0:
                    continue
                tok = np.nonzero(_kv_token_mask(blocks, n, kv_block_size, kh_))[0]
                if tok.size == 0:
                    continue
                kt = kk[bi, hi, tok]
                vt = vv[bi, hi, tok]
                s = (qq[bi, hi, r0:r1] * work(scale)) @ kt.T
                p = np.exp(s - lse[bi, hi, r0:r1, None].astype(work))
                dp = dd[bi, hi, r0:r1] @ vt.T
                ds = p * (dp - delta[bi, hi, r0:r1, None])
                if envelope:
                    # rounding of dS (dQ, dK) and of P (dV), plus delta's error through P
                    ads = u * np.abs(ds) + p * ddelta[bi, hi, r0:r1, None]
                    qa = np.abs(qq[bi, hi, r0:r1])
                    eq[bi, hi, r0:r1] = work(scale) * (ads @ np.abs(kt))
                    ek[bi, hi, tok] += work(scale) * (ads.T @ qa)
                    ev[bi, hi, tok] += u * (p.T @ np.abs(dd[bi, hi, r0:r1]))
                if roundings:
                    ds = round_to_dtype(ds, io_dtype)
                    p = round_to_dtype(p, io_dtype)
                dq[bi, hi, r0:r1] = work(scale) * (ds @ kt)
                dk[bi, hi, tok] += work(scale) * (ds.T @ qq[bi, hi, r0:r1])
                dv[bi, hi, tok] += p.T @ dd[bi, hi, r0:r1]

    def merge(x):
        return x.transpose(0, 2, 1, 3).reshape(b, n, c)

    grads = [merge(dq), merge(dk), merge(dv)]
    if roundings:
        grads = [round_to_dtype(x, io_dtype) for x in grads]
    if envelope:
        envs = tuple(merge(e) + u * np.abs(x) for e, x in zip((eq, ek, ev), grads))
        return grads[0], grads[1], grads[2], envs
    return grads[0], grads[1], grads[2]


# --------------------------------------------------------------------------
# a8/a11  reverse index and count sort
# --------------------------------------------------------------------------
def build_reverse_indices(merged_indices, counts, num_kv_blocks):
    """Invert q-block -> kv-block lists.

    Returns (reverse_indices [B,H,M,QM] int32 (-1 padded), reverse_counts
    [B,H,M] int32, sorted_kv_indices [B,H,M] int32).  Slots are filled in
    ascending q-block order, the order of the reference's Python loop
    (flash_topk_attn_v2/sparse_attn_bwd.py:36-76); sorted_kv_indices is the
    stable descending argsort of the counts
    (csrc/build_reverse_indices_kernel.cu:29-62).
    """
    b, h, qm, _ = merged_indices.shape
    m = num_kv_blocks
    rev = np.full((b, h, m, qm), -1, dtype=np.int32)
    rc = np.zeros((b, h, m), dtype=np.int32)
    for bi in range(b):
        for hi in range(h):
            for t in range(qm):
                cnt = int(counts[bi, hi, t])
                for s in range(cnt):
                    j = int(merged_indices[bi, hi, t, s])
                    if j < 0:
                        continue
                    rev[bi, hi, j, rc[bi, hi, j]] = t
                    rc[bi, hi, j] += 1
    order = np.argsort(-rc, axis=-1, kind="stable").astype(np.int32)
    return rev, rc, order


def sort_by_count(reverse_counts):
    """Global descending sort of all counts with their flat ids.

    Stable, so equal counts keep ascending flat id, as an LSD radix sort does
    (flash_topk_attn_v2/sparse_attn_bwd.py:79-108,
    csrc/sort_by_count_kernel.cu:12-52).
    """
    flat = reverse_counts.reshape(-1)
    order = np.argsort(-flat.astype(np.int64), kind="stable")
    return flat[order].astype(np.int32), order.astype(np.int32)


# --------------------------------------------------------------------------
# tie classification for index parity
# --------------------------------------------------------------------------
def classify_topk_mismatches(
    got_idx: np.ndarray,
    want_idx: np.ndarray,
    avg_scores: np.ndarray,
    rel_band: float = 1e-6,
):
    """Compare two [..., K] index tables row by row.

    `avg_scores` [..., M] are the arbiter's (fp64) average block scores.  A
    position where the two tables name different blocks is a *tie* when the
    arbiter's scores of those two blocks differ by less than `rel_band`
    relative, else a *hard* mismatch; a -1 on one side only is judged by the
    same rule against the other side's block at the cut (or counted hard when
    there is nothing to compare with).  Returns a dict of counts.
    """
    g = got_idx.reshape(-1, got_idx.shape[-1])
    w = want_idx.reshape(-1, want_idx.shape[-1])
    a = avg_scores.reshape(-1, avg_scores.shape[-1])
    diff = g != w
    rows, cols = np.nonzero(diff)
    ties = hard = 0
    hard_examples = []
    for r, c in zip(rows.tolist(), cols.tolist()):
        gi, wi = int(g[r, c]), int(w[r, c])
        if gi < 0 or wi < 0:
            hard += 1
            if len(hard_examples) < 8:
                hard_examples.append((r, c, gi, wi, None))
            continue
        sg, sw = float(a[r, gi]), float(a[r, wi])
        rel = abs(sg - sw) / max(abs(sg), abs(sw), 1e-300)
        if rel < rel_band:
            ties += 1
        else:
            hard += 1
            if len(hard_examples) < 8:
                hard_examples.append((r, c, gi, wi, rel))
    return {
        "positions": int(g.size),
        "rows": int(g.shape[0]),
        "mismatched_positions": int(diff.sum()),
        "mismatched_rows": int(diff.any(axis=1).sum()),
        "ties": ties,
        "hard": hard,
        "hard_examples": hard_examples,
    }


# --------------------------------------------------------------------------
# first-generation operators (package flash_topk_attn of the reference)
# --------------------------------------------------------------------------
def v1_topk_score(
    q, k, v=None, num_heads=None, block_size=64, topk=16, padding=(0, 0),
    score_only=False, work=np.float64,
):
    """Top-k blocks per query without a threshold, plus the dense attention
    output unless `score_only`.

    Restates `_flash_topk_score_naive` (flash_topk_attn/scoring.py:1360-1469):
    block scores are softmax sums when there is no padding and sums divided by
    the block's real-token count when there is (:1448-1459); the k best are
    returned best first (ties: lower block id, where the reference's
    torch.topk leaves the order open).  Returns (idx int32, scores[, o]) with
    idx / scores [B,H,N,min(topk,M)] and o [B,N,C] unrounded; also the full
    score table as the last element for tie arbitration.
    """
    if not score_only and v is None:
        raise ValueError("v is required when score_only=False")
    b, n, c = q.shape
    h = num_heads
    m, starts, ends, valid = block_geometry(n, block_size, padding)
    if topk > m:
        raise ValueError(f"topk ({topk}) > num_blocks ({m})")
    sums = block_score(q, k, h, block_size, padding, work=work)
    if tuple(padding) == (0, 0):
        table = sums
    else:
        table = sums / np.maximum(valid, 1).astype(work)
        table[..., valid == 0] = 0
    kk = min(topk, m)
    order = np.argsort(-table, axis=-1, kind="stable")[..., :kk]
    scores = np.take_along_axis(table, order, axis=-1)
    idx = order.astype(np.int32)
    if score_only:
        return idx, scores, table
    d = c // h
    qq = _split_heads(q, h).astype(work)
    kh = _split_heads(k, h).astype(work)
    vv = _split_heads(v, h).astype(work)
    o = np.zeros((b, h, n, d), dtype=work)
    for bi in range(b):
        for hi in range(h):
            s = (qq[bi, hi] * work(d ** -0.5)) @ kh[bi, hi].T
            s -= s.max(axis=1, keepdims=True)
            np.exp(s, out=s)
            s /= s.sum(axis=1, keepdims=True)
            o[bi, hi] = s @ vv[bi, hi]
    return o.transpose(0, 2, 1, 3).reshape(b, n, c), idx, scores, table


def v1_qblock_union(topk_indices, q_block_size, q_padding=(0, 0)):
    """Distinct block ids of each q-block's rows, ascending, -1 padded to
    S_MAX = next_pow2(q_block_size * K): (merged [B,H,QM,S_MAX] int32, counts
    [B,H,QM] int32, S_MAX).  Restates build_qblock_topk_indices and its
    load / sort / drop-repeats / compact kernel
    (flash_topk_attn/attention.py:23-67, :70-138)."""
    b, h, n, kq = topk_indices.shape
    qh_, qt_ = q_padding
    if qh_ >= q_block_size or qt_ >= q_block_size:
        raise ValueError("q padding must be smaller than q_block_size")
    if (qh_ + n + qt_) % q_block_size != 0:
        raise ValueError("q padding does not tile")
    qm = (qh_ + n + qt_) // q_block_size
    raw = q_block_size * kq
    s_max = 1 if raw <= 1 else 1 << (raw - 1).bit_length()
    merged = np.full((b, h, qm, s_max), -1, dtype=np.int32)
    counts = np.zeros((b, h, qm), dtype=np.int32)
    for bi in range(b):
        for hi in range(h):
            for m in range(qm):
                r0 = max(0, m * q_block_size - qh_)
                r1 = min(n, (m + 1) * q_block_size - qh_)
                if r0 >= r1:
                    continue
                ids = np.unique(topk_indices[bi, hi, r0:r1])
                ids = ids[ids >= 0]
                merged[bi, hi, m, : ids.size] = ids
                counts[bi, hi, m] = ids.size
    return merged, counts, s_max


def v1_topk_attn(
    q, k, v, merged_indices, counts, num_heads, q_block_size, kv_block_size,
    scale=None, kv_padding=(0, 0), q_padding=(0, 0), work=np.float64,
):
    """Attention over the first counts[b,h,m] listed blocks of each q-block;
    the index tensor may carry one head shared by all heads.  Restates
    `_flash_topk_attn_naive` (flash_topk_attn/attention.py:571-647) on top of
    sparse_attn_fwd: (O [B,N,C] unrounded, lse [B,H,N])."""
    mi = np.array(merged_indices, dtype=np.int64, copy=True)
    slot = np.arange(mi.shape[-1])
    mi[slot >= np.asarray(counts)[..., None]] = -1
    if mi.shape[1] == 1 and num_heads > 1:
        mi = np.repeat(mi, num_heads, axis=1)
    return sparse_attn_fwd(q, k, v, mi, num_heads, q_block_size, kv_block_size, scale,
                           q_padding, kv_padding, work=work)
