"""CPU-side checks of the boundary: the shared library loads without a GPU,
exports every symbol include/ftk_api.h declares, and the Python mirror raises
the reference's exceptions before touching the device."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ftk_api.h")


@pytest.fixture(scope="module")
def ftk():
    import flash_topk_attn_v2 as m
    return m


def test_library_exports_every_declared_symbol(ftk):
    from flash_topk_attn_v2 import _lib
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b(ftk_\w+)\s*\(", text))
    assert len(declared) >= 15
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} declared in ftk_api.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_version_and_error_text(ftk):
    from flash_topk_attn_v2 import _lib
    assert _lib.lib.ftk_version() >= 100
    for code in (0, -1, -2, -3, -4, -5, 101, 105):
        assert _lib.error_text(code) != "unknown code"
    assert _lib.error_text(12345) == "unknown code"
    with pytest.raises(ValueError):
        _lib.check(-1, "x")
    with pytest.raises(NotImplementedError):
        _lib.check(-2, "x")
    with pytest.raises(RuntimeError):
        _lib.check(-4, "x")


def test_workspace_queries_need_no_gpu(ftk):
    from flash_topk_attn_v2 import _lib
    lib = _lib.lib
    a = lib.ftk_score_topk_workspace(2, 1024, 16)
    b = lib.ftk_block_score_workspace(2, 1024)
    assert a >= b + 2 * 1024 * 16 * 4 and b >= 2 * 2 * 1024 * 4
    assert lib.ftk_build_reverse_workspace(4, 64, 64) >= 4 * 64 * 2 * 4
    assert lib.ftk_sort_by_count_workspace(5000, 10) >= 11 * 3 * 4


def test_api_names_and_signatures(ftk):
    import inspect
    assert ftk.__all__ == ["flash_topk_score", "build_qblock_topk_indices", "flash_topk_attn"]
    s = inspect.signature(ftk.flash_topk_score)
    assert list(s.parameters) == ["q", "k", "num_heads", "score_block_size", "topk", "padding",
                                  "threshold"]
    assert s.parameters["score_block_size"].default == 64 and s.parameters["topk"].default == 16
    s = inspect.signature(ftk.build_qblock_topk_indices)
    # the reference's five parameters in its order, then this package's optional extension
    assert list(s.parameters) == ["topk_indices", "q_block_size", "q_padding", "topk_scores",
                                  "qblock_topk", "num_score_blocks"]
    assert s.parameters["num_score_blocks"].default is None
    s = inspect.signature(ftk.flash_topk_attn)
    assert list(s.parameters) == ["q", "k", "v", "merged_indices", "counts", "num_heads",
                                  "q_block_size", "kv_block_size", "scale", "num_kv_heads",
                                  "kv_padding", "q_padding", "S_MAX"]


def test_reference_exceptions_before_any_launch(ftk):
    x = torch.zeros(1, 128, 64)
    with pytest.raises(ValueError, match="requires CUDA"):
        ftk.flash_topk_score(x, x, num_heads=1)
    with pytest.raises(ValueError, match="num_heads is required"):
        ftk.flash_topk_score(x, x)
    with pytest.raises(ValueError, match="3D"):
        ftk.flash_topk_score(x[0], x[0], num_heads=1)
    x4 = torch.zeros(1, 2, 128, 32)
    with pytest.raises(ValueError, match="num_heads"):
        ftk.flash_topk_score(x4, x4, num_heads=3)
    idx = torch.zeros(1, 1, 100, 4, dtype=torch.int32)
    with pytest.raises(ValueError, match="divisible"):
        ftk.build_qblock_topk_indices(idx, 64)
    with pytest.raises(ValueError, match="q_pad_head"):
        ftk.build_qblock_topk_indices(idx, 64, q_padding=(64, 0))
    with pytest.raises(ValueError, match="non-negative"):
        ftk.build_qblock_topk_indices(idx, 64, q_padding=(-1, 0))
    with pytest.raises(ValueError, match=r"\[B, H, N, K\]"):
        ftk.build_qblock_topk_indices(idx[0], 64)
    with pytest.raises(ValueError, match="requires CUDA"):
        ftk.flash_topk_attn(x, x, x, idx, None, 1, 64, 64)


def test_no_fallback_when_library_missing(tmp_path, monkeypatch):
    """The package must refuse to import without its CUDA library."""
    from flash_topk_attn_v2 import _lib
    monkeypatch.setattr(os.path, "exists", lambda p, _e=os.path.exists: False
                        if p == _lib.LIB_PATH else _e(p))
    with pytest.raises(ImportError, match="no fallback"):
        _lib._load()


def test_large_block_lists_split_into_half_blocks():
    """q / kv blocks of 65..128 rows are restated over half-size blocks on the
    host: every query row must keep exactly the same set of key tokens."""
    import numpy as np
    import torch
    from flash_topk_attn_v2 import ops

    def token_sets(merged, N, g, kvb, qph, kph):
        qm = merged.shape[2]
        out = []
        for m in range(qm):
            toks = set()
            for j in merged[0, 0, m].tolist():
                if j >= 0:
                    toks.update(t for t in range(j * kvb - kph, (j + 1) * kvb - kph) if 0 <= t < N)
            for r in range(m * g - qph, (m + 1) * g - qph):
                if 0 <= r < N:
                    out.append((r, frozenset(toks)))
        return dict(out)

    rng = np.random.default_rng(0)
    for N, g, kvb, qpad, kpad in [(1000, 128, 128, (70, 82), (100, 52)),
                                  (1000, 128, 64, (10, 14), (8, 16)),
                                  (1000, 64, 128, (24, 0), (0, 24)),
                                  (1000, 96, 96, (20, 36), (50, 6)),
                                  (100, 128, 128, (14, 14), (27, 1))]:
        QM, M = (qpad[0] + N + qpad[1]) // g, (kpad[0] + N + kpad[1]) // kvb
        merged = np.full((1, 1, QM, 4), -1, dtype=np.int32)
        for m in range(QM):
            c = int(rng.integers(0, 5))
            merged[0, 0, m, :c] = rng.permutation(M)[:c]
        want = token_sets(merged, N, g, kvb, qpad[0], kpad[0])
        m2, g2, kvb2, qph2, kph2, mkv2 = ops._split_large_blocks(
            torch.from_numpy(merged), N, g, kvb, qpad[0], kpad[0])
        assert g2 <= 64 and kvb2 <= 64 and 0 <= qph2 < g2 and 0 <= kph2 < kvb2
        assert m2.shape[2] * g2 >= qph2 + N and int(m2.max()) < mkv2
        got = token_sets(m2.numpy(), N, g2, kvb2, qph2, kph2)
        assert got == want, (N, g, kvb)
        # down to 32-row blocks (gradient kernels at head dim 256), where halving allows
        if g % 64 == 0 and kvb % 64 == 0:
            m3, g3, kvb3, qph3, kph3, mkv3 = ops._split_large_blocks(
                torch.from_numpy(merged), N, g, kvb, qpad[0], kpad[0], limit=32)
            assert g3 == 32 and kvb3 == 32 and 0 <= qph3 < 32 and 0 <= kph3 < 32
            assert m3.shape[2] * g3 >= qph3 + N and int(m3.max()) < mkv3
            assert token_sets(m3.numpy(), N, g3, kvb3, qph3, kph3) == want, (N, g, kvb)


def test_first_generation_api_names_and_signatures():
    """The older package name keeps the reference's three signatures
    (flash_topk_attn/__init__.py:1-4, scoring.py:1289-1299, attention.py:70-74,
    :423-437) and refuses CPU tensors before any launch."""
    import inspect
    import flash_topk_attn as v1
    assert v1.__all__ == ["flash_topk_score", "flash_topk_attn", "build_qblock_topk_indices"]
    s = inspect.signature(v1.flash_topk_score)
    assert list(s.parameters) == ["q", "k", "v", "num_heads", "score_block_size", "topk",
                                  "padding", "score_only", "backend"]
    assert s.parameters["score_only"].default is False
    assert s.parameters["backend"].default == "triton"
    assert list(inspect.signature(v1.build_qblock_topk_indices).parameters) == [
        "topk_indices", "q_block_size", "q_padding"]
    assert list(inspect.signature(v1.flash_topk_attn).parameters) == [
        "q", "k", "v", "merged_indices", "counts", "num_heads", "q_block_size", "kv_block_size",
        "scale", "num_kv_heads", "kv_padding", "q_padding", "S_MAX"]
    x = torch.zeros(1, 128, 64)
    with pytest.raises(ValueError, match="requires CUDA"):
        v1.flash_topk_score(x, x, x, 1, topk=2)
    with pytest.raises(ValueError, match="topk"):
        v1.flash_topk_score(x, x, x, 1)
    with pytest.raises(ValueError, match="unsupported backend"):
        v1.flash_topk_score(x, x, x, 1, backend="cuda")
    with pytest.raises(ValueError, match="requires CUDA"):
        v1.build_qblock_topk_indices(torch.zeros(1, 1, 128, 2, dtype=torch.int32), 32)
    with pytest.raises(AssertionError):
        v1.flash_topk_attn(x, x, x, None, None, 1, 32, 64)
