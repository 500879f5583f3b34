"""ftk_build_reverse_noalloc against ftk_build_reverse, through the C ABI.

The no-allocation variant exists for callers that cannot allocate device
memory where they call the library (allocator callbacks, fixed-buffer plugins,
loops that must stay out of the allocator).  Its scratch is one array inside
the library, shared by all calls and never cleared between them except by the
call itself, so the check runs two different problems back to back: stale bits
from the first must not leak into the second.  Results are integers and must
be identical to the workspace-taking entry point's.  This file is named to be
collected last.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _random_merged(rng, BH, QM, W, M, fill):
    merged = np.full((BH, QM, W), -1, dtype=np.int32)
    for b in range(BH):
        for m in range(QM):
            n = int(rng.integers(0, min(W, M) + 1)) if fill is None else fill
            merged[b, m, :n] = rng.permutation(M)[:n]
    return merged


def _run(lib, fn_noalloc, merged, M):
    from flash_topk_attn_v2._lib import ptr
    BH, QM, W = merged.shape
    dev = torch.device("cuda", 0)
    mt = torch.from_numpy(merged).to(dev)
    cnt = (mt >= 0).sum(-1).to(torch.int32).contiguous()
    st = torch.cuda.current_stream(dev).cuda_stream
    out = []
    for noalloc in (False, True):
        rev = torch.full((BH, M, QM), 7, dtype=torch.int32, device=dev)
        rc = torch.full((BH, M), 7, dtype=torch.int32, device=dev)
        skv = torch.full((BH, M), 7, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        if noalloc:
            rcode = lib.ftk_build_reverse_noalloc(
                ptr(mt), ptr(cnt), BH, QM, W, M, ptr(rev), ptr(rc), ptr(skv), ptr(status), st)
        else:
            ws = torch.empty(lib.ftk_build_reverse_workspace(BH, QM, M), dtype=torch.uint8,
                             device=dev)
            rcode = lib.ftk_build_reverse(
                ptr(mt), ptr(cnt), BH, QM, W, M, ptr(rev), ptr(rc), ptr(skv), ptr(ws),
                ws.numel(), ptr(status), st)
        assert rcode == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        out.append((rev.cpu().numpy(), rc.cpu().numpy(), skv.cpu().numpy()))
    return out


def test_noalloc_matches_workspace_version_twice_in_a_row():
    from flash_topk_attn_v2 import _lib
    lib = _lib.lib
    rng = np.random.default_rng(11)
    # first a dense problem that sets many bits, then a sparse one of another
    # shape that reuses the same part of the array
    for BH, QM, W, M, fill in ((3, 70, 40, 40, 40), (4, 33, 16, 50, None)):
        merged = _random_merged(rng, BH, QM, W, M, fill)
        (rev_a, rc_a, skv_a), (rev_b, rc_b, skv_b) = _run(lib, True, merged, M)
        np.testing.assert_array_equal(rev_b, rev_a)
        np.testing.assert_array_equal(rc_b, rc_a)
        np.testing.assert_array_equal(skv_b, skv_a)
        # and both agree with a direct count
        want = np.zeros((BH, M), dtype=np.int32)
        for b in range(BH):
            ids, c = np.unique(merged[b][merged[b] >= 0], return_counts=True)
            want[b, ids] = c
        np.testing.assert_array_equal(rc_b, want)


def test_noalloc_rejects_problems_beyond_its_capacity():
    from flash_topk_attn_v2 import _lib
    lib = _lib.lib
    cap = lib.ftk_build_reverse_noalloc_capacity()
    assert cap == 4 << 20
    dev = torch.device("cuda", 0)
    x = torch.zeros(16, dtype=torch.int32, device=dev)
    BH, QM, M = 64, 4096, 4096          # 64 * 4096 * 128 words * 4 B = 128 MiB
    assert BH * M * ((QM + 31) // 32) * 4 > cap
    rcode = lib.ftk_build_reverse_noalloc(x.data_ptr(), 0, BH, QM, 1, M, x.data_ptr(),
                                          x.data_ptr(), 0, 0, 0)
    assert rcode == -6
    assert "fixed buffer" in _lib.error_text(rcode)
