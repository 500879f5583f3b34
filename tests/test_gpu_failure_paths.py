"""Failure detection on the device, proved without faulting, trapping or hanging a GPU.

1. A bounded wait that runs out.  tests/native/wait_probe.cu compiles the wait
   helpers of csrc/ftk_sm100.cuh with a limit of 200 000 clock ticks and waits
   on an mbarrier nobody arrives at (one CTA, no TMA and no tcgen05 in flight):
   the wait gives up, records its code, raises the abort flag, the kernel
   returns, and the context stays usable.  Also with a null status pointer,
   which the C ABI allows.
2. Block ids outside the table.  Every walk over a caller-supplied list drops
   an id >= the block count before any address is formed and records
   FTK_DEV_BAD_INDEX (105); the other entries are processed as usual.
3. ftk_max_index_plus1, the device-side reduction for sizing the merge table.
"""

import ctypes
import os

import numpy as np
import pytest
import torch

import cases
from oracle import ftk_oracle as orc

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
PROBE = os.path.join(HERE, "native", "libftk_wait_probe.so")


@pytest.fixture(scope="module")
def ftk():
    import flash_topk_attn_v2 as m
    from flash_topk_attn_v2 import ops
    if ops._DEBUG:
        pytest.skip("FTK_DEBUG=1 raises inside the failing call; these tests read the status "
                    "word themselves")
    return m


@pytest.fixture(scope="module")
def probe():
    if not os.path.exists(PROBE):
        pytest.fail(f"{PROBE} is missing: run __graft_entry__.build()")
    lib = ctypes.CDLL(PROBE)
    lib.ftk_wait_probe.restype = ctypes.c_int
    lib.ftk_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.ftk_wait_probe_cycles.restype = ctypes.c_longlong
    return lib


def _small_score_matches_oracle(ftk):
    cfg = cases.GOLDEN_CASES["tiny_fp16"]
    t = cases.make_inputs(cfg)
    got = ftk.flash_block_score(t["q"].cuda(), t["k"].cuda(), cfg["H"], cfg["score_block_size"])
    ftk.check_errors()
    want = orc.block_score(t["q"].float().numpy(), t["k"].float().numpy(), cfg["H"],
                           cfg["score_block_size"], (0, 0))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=3e-6, atol=1e-9)


@pytest.mark.parametrize("with_status", [True, False])
def test_bounded_wait_runs_out_and_the_kernel_returns(ftk, probe, with_status):
    assert probe.ftk_wait_probe_cycles() == 200000
    dev = torch.device("cuda", 0)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    trace = torch.full((8,), -7, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    rc = probe.ftk_wait_probe(status.data_ptr() if with_status else None, trace.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()          # returns: the launch completed
    tr = trace.cpu().tolist()
    assert tr[0] == 0 and tr[2] == 0, tr      # both waits gave up
    assert tr[1] == 1, tr                     # abort flag raised for the CTA
    assert tr[3] == 0, tr                     # mbar_wait_all with one dead barrier gives up too
    assert tr[4] == 1, tr                     # a completed barrier still answers at once
    assert 0 < tr[5] < 50_000_000, tr         # within the limit plus slack, not seconds
    code = int(status.item())
    if with_status:
        # first failure wins: the TMA-side code of warp 0 or the consumer code of warp 1
        assert code in (101, 103), code
        from flash_topk_attn_v2 import _lib
        assert "wait" in _lib.error_text(code).lower() or "timeout" in _lib.error_text(code).lower()
    else:
        assert code == 0
    # the context is intact: a normal launch afterwards still passes parity
    _small_score_matches_oracle(ftk)


def _lists_with_one_bad_id(H, QM, M, W, bad_at, bad_id):
    rng = np.random.default_rng(3)
    merged = np.full((1, H, QM, W), -1, dtype=np.int32)
    for h in range(H):
        for m in range(QM):
            merged[0, h, m, :W - 1] = rng.permutation(M)[:W - 1]
    h, m, e = bad_at
    merged[0, h, m, e] = bad_id
    clean = merged.copy()
    clean[0, h, m, e] = -1
    return merged, clean


@pytest.mark.parametrize("D,g,kvb,dtype", [(128, 64, 64, "bf16"), (64, 32, 64, "fp16")])
def test_out_of_range_block_id_in_attention_lists(ftk, D, g, kvb, dtype):
    """Forward and dQ walk merged_indices (pair kernels at D = 128 with 64-row
    blocks, one-CTA kernels otherwise); dK/dV walks the reverse index built from
    it.  The bad id is dropped, status 105 is raised, every output equals the
    run on the same lists with that entry removed."""
    H, N = 2, 512
    cfg = dict(B=1, N=N, H=H, D=D, dtype=dtype, seed=81, do_seed=82)
    t = cases.make_inputs(cfg)
    QM, M, W = N // g, N // kvb, 4
    merged, clean = _lists_with_one_bad_id(H, QM, M, W, (1, 3, 2), M + 5)

    def run(lists, expect_error):
        q, k, v = (t[n].cuda().requires_grad_(True) for n in "qkv")
        o, lse = ftk.flash_topk_attn(q, k, v, torch.from_numpy(lists).cuda(), None, H, g, kvb)
        if expect_error:
            with pytest.raises(RuntimeError, match="105"):
                ftk.check_errors()
        else:
            ftk.check_errors()
        # the operators inside backward() would report the failure themselves as soon as
        # they see it; switched off here so that the gradients of the bad run can be compared
        from flash_topk_attn_v2 import ops
        ops.deferred_checks(False)
        try:
            o.backward(t["do"].cuda())
        finally:
            ops.deferred_checks(True)
        if expect_error:
            with pytest.raises(RuntimeError, match="105"):
                ftk.check_errors()
        else:
            ftk.check_errors()
        return [x.detach().float().cpu().numpy() for x in (o, lse, q.grad, k.grad, v.grad)]

    bad = run(merged, True)
    good = run(clean, False)
    for a, b, what in zip(bad, good, ("O", "lse", "dQ", "dK", "dV")):
        np.testing.assert_array_equal(a, b, err_msg=what)
    x = {n: v.float().numpy() for n, v in t.items()}
    wo, wl = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], clean, H, g, kvb)
    np.testing.assert_allclose(bad[0], wo, atol=2e-3, rtol=1e-2)
    np.testing.assert_allclose(bad[1], wl, atol=2e-3, rtol=1e-2)


def test_out_of_range_block_id_in_merge_and_reverse(ftk):
    rng = np.random.default_rng(4)
    B, H, N, K, g, M = 1, 2, 256, 4, 32, 16
    idx = np.stack([rng.permutation(M)[:K] for _ in range(B * H * N)]).astype(np.int32)
    idx = idx.reshape(B, H, N, K)
    scr = rng.random((B, H, N, K), dtype=np.float32) + 0.1
    bad = idx.copy()
    bad[0, 1, 70, 2] = M + 9
    clean = bad.copy()
    clean[0, 1, 70, 2] = -1
    cs = scr.copy()
    cs[0, 1, 70, 2] = 0.0

    def merge(i, s):
        return ftk.flash_qblock_merge(torch.from_numpy(i).cuda(), torch.from_numpy(s).cuda(), g,
                                      g * K, M, return_counts=True)

    mb = merge(bad, scr)
    with pytest.raises(RuntimeError, match="105"):
        ftk.check_errors()
    mc = merge(clean, cs)
    ftk.check_errors()
    for a, b in zip(mb, mc):
        assert torch.equal(a, b)
    om, oc, _, oms = orc.build_qblock_topk_indices(clean, g, (0, 0), cs, g * K)
    np.testing.assert_array_equal(mc[0].cpu().numpy(), om)
    np.testing.assert_array_equal(mc[2].cpu().numpy(), oc)

    merged = mc[0].clone()
    merged[0, 0, 3, 1] = M + 1
    rb = ftk.flash_build_reverse_indices_cuda(merged, None, M)
    with pytest.raises(RuntimeError, match="105"):
        ftk.check_errors()
    merged[0, 0, 3, 1] = -1
    rg = ftk.flash_build_reverse_indices_cuda(merged, None, M)
    ftk.check_errors()
    for a, b in zip(rb, rg):
        assert torch.equal(a, b)
    mnp = merged.cpu().numpy()
    # the kernel read every row to its full width (counts = NULL), skipping -1
    orev, orc_, oskv = orc.build_reverse_indices(mnp, np.full(mnp.shape[:3], mnp.shape[3]), M)
    np.testing.assert_array_equal(rg[0].cpu().numpy(), orev)
    np.testing.assert_array_equal(rg[1].cpu().numpy(), orc_)


def test_device_error_surfaces_at_a_later_call_without_check_errors(ftk):
    """A caller that never calls check_errors(): every operator leaves a copy of
    the status word in pinned memory and looks at the previous copy, so the
    failure of one call raises at a following call."""
    rng = np.random.default_rng(5)
    M, K, g = 16, 4, 32
    idx = np.stack([rng.permutation(M)[:K] for _ in range(2 * 256)]).astype(np.int32)
    idx = idx.reshape(1, 2, 256, K)
    good = torch.from_numpy(idx).cuda()
    bad = good.clone()
    bad[0, 0, 5, 1] = M + 3
    ftk.check_errors()
    ftk.flash_qblock_merge(bad, None, g, g * K, M)          # sets status 105 on the device
    torch.cuda.synchronize()                                 # the 4-byte copy has landed
    with pytest.raises(RuntimeError, match="earlier call.*105"):
        for _ in range(3):
            ftk.flash_qblock_merge(good, None, g, g * K, M)
            torch.cuda.synchronize()
    ftk.flash_qblock_merge(good, None, g, g * K, M)          # cleared: works again
    torch.cuda.synchronize()
    ftk.check_errors()


def test_max_index_plus1(ftk):
    from flash_topk_attn_v2 import _lib
    lib, dev = _lib.lib, torch.device("cuda", 0)
    st = torch.cuda.current_stream(dev).cuda_stream
    out = torch.full((1,), -5, dtype=torch.int32, device=dev)
    rng = np.random.default_rng(8)
    for n, hi in ((1, 3), (1000, 17), (1 << 20, 4000), (3_000_001, 123456)):
        a = rng.integers(-1, hi, size=n).astype(np.int32)
        t = torch.from_numpy(a).to(dev)
        assert lib.ftk_max_index_plus1(t.data_ptr(), n, out.data_ptr(), st) == 0
        assert int(out.item()) == max(int(a.max()) + 1, 1)
    # nothing valid at all -> 1 (a table of one block), as the reference does
    t = torch.full((77,), -1, dtype=torch.int32, device=dev)
    assert lib.ftk_max_index_plus1(t.data_ptr(), 77, out.data_ptr(), st) == 0
    assert int(out.item()) == 1
    assert lib.ftk_max_index_plus1(t.data_ptr(), 0, out.data_ptr(), st) == 0
    assert int(out.item()) == 1
    assert lib.ftk_max_index_plus1(None, 5, out.data_ptr(), st) == -1
    # the API sizes its table from it when the index tensor carries no block count
    idx = torch.from_numpy(rng.integers(0, 40, size=(1, 2, 128, 4)).astype(np.int32)).to(dev)
    assert ops_num_blocks(ftk, idx) == int(idx.max().item()) + 1


def ops_num_blocks(ftk, idx):
    from flash_topk_attn_v2 import ops
    return ops.num_score_blocks_of(idx)
