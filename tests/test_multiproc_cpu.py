"""Multi-rank host logic on CPU (gloo, world size 2): sharding (batch x head)
slices across ranks reproduces the unsharded result with no data-path
collective.  The per-slice arithmetic here is the CPU oracle; the only
communication is the final gather a test needs to compare."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import ftk_oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _chain(x, H, cfg):
    idx, raw, avg, _ = orc.flash_topk_score(
        x["q"], x["k"], H, cfg["score_block_size"], cfg["topk"], (0, 0), cfg["threshold"])
    merged, counts, W, _ = orc.build_qblock_topk_indices(idx, cfg["q_block_size"], (0, 0), avg)
    o, lse = orc.sparse_attn_fwd(x["q"], x["k"], x["v"], merged, H, cfg["q_block_size"],
                                 cfg["kv_block_size"])
    dq, dk, dv = orc.sparse_attn_bwd(x["q"], x["k"], x["v"], o, lse, x["do"], merged, H,
                                     cfg["q_block_size"], cfg["kv_block_size"])
    return idx, merged, o, dq, dk, dv


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flash_topk_attn_v2.shard import shard_heads, slice_range
    cfg = cases.GOLDEN_CASES["tiny_fp16"]
    t = cases.make_inputs(cfg)
    H = cfg["H"]
    b0, b1 = slice_range(cfg["B"] * H, rank, world)
    assert (b0, b1) == (rank, rank + 1)
    x = {}
    for k, v in t.items():
        sh, per = shard_heads(v.float(), H, rank, world)
        x[k] = sh.numpy()
    res = _chain(x, per, cfg)
    # gather only what the test compares (O and dK), rank-major = head-major
    for name, arr in (("o", res[2]), ("dk", res[4])):
        mine = torch.from_numpy(np.ascontiguousarray(arr))
        bucket = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(bucket, mine)
        if rank == 0:
            np.save(os.path.join(out_dir, f"{name}.npy"),
                    np.concatenate([b.numpy() for b in bucket], axis=-1))
    if rank == 0:
        np.save(os.path.join(out_dir, "merged0.npy"), res[1])
    dist.barrier()
    dist.destroy_process_group()


def test_slice_range_partitions():
    from flash_topk_attn_v2.shard import slice_range
    for n in (1, 7, 32, 512):
        for world in (1, 2, 3, 8):
            spans = [slice_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        slice_range(4, 2, 2)


def test_two_ranks_match_unsharded(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    cfg = cases.GOLDEN_CASES["tiny_fp16"]
    t = cases.make_inputs(cfg)
    x = {k: v.float().numpy() for k, v in t.items()}
    idx, merged, o, dq, dk, dv = _chain(x, cfg["H"], cfg)
    np.testing.assert_array_equal(np.load(tmp_path / "merged0.npy"), merged[:, :1])
    np.testing.assert_allclose(np.load(tmp_path / "o.npy"), o, rtol=0, atol=1e-12)
    np.testing.assert_allclose(np.load(tmp_path / "dk.npy"), dk, rtol=0, atol=1e-12)
