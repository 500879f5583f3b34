"""Run the reference project's own flash_topk_attn_v2 GPU kernels on this GPU.

The reference package is installed, unmodified, under ``baseline/_ref`` (by
``pip install --target``; that folder is not part of this repository's
history).  Its CUDA extensions are compiled when first used, for sm_80/sm_86
only and against a CUTLASS checkout at a path of its author's machine
(flash_topk_attn_v2/block_score_cuda.py:14,28-40, sparse_attn_cuda.py:13,35-36,
sparse_attn_bwd_dq_cuda.py:13-15,37-38, sparse_attn_bwd_dkv_cuda.py:13-15,37-38).
Nothing of that source is edited or copied; two things are patched in the
running interpreter before the first kernel is built:

* every module's ``_CUTLASS_INCLUDE`` points at the CUTLASS headers that ship
  with flashinfer in this image;
* every module's ``load_inline`` global is a wrapper that rewrites the
  ``-gencode`` pairs to ``arch=compute_100,code=sm_100``, builds under
  ``baseline/_ref/_ext/<name>/`` and, once built, loads the finished ``.so``
  directly on later runs (a stamp file holds the hash of sources and flags).

The reference and this repository's package share the import name
``flash_topk_attn_v2``, so the reference always runs in a process of its own:

    python baseline/ref_v2_gpu.py prebuild            # no GPU needed (nvcc only)
    python baseline/ref_v2_gpu.py run  --case tiny_fp16 --out x.npz [--stages score,merge,attn,bwd] [--cfg JSON]
    python baseline/ref_v2_gpu.py time --shape headline --steps 5 --warmup 2

``run`` executes one stage at a time with a synchronize and an error check after
each (the reference checks no launch itself) and writes its outputs as .npz;
``time`` prints one JSON line of per-stage and whole-chain CUDA-event times.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")
EXT = os.path.join(REF, "_ext")
CUTLASS_CANDIDATES = (
    "flashinfer/data/cutlass/include",
    "tilelang/3rdparty/cutlass/include",
)
EXT_MODULES = (
    "block_score_cuda", "topk_select_cuda", "qblock_merge",
    "build_reverse_indices_cuda", "sort_by_count_cuda", "sparse_attn_cuda",
    "sparse_attn_bwd_dq_cuda", "sparse_attn_bwd_dkv_cuda",
)


def available() -> bool:
    return os.path.isdir(os.path.join(REF, "flash_topk_attn_v2", "csrc"))


def _cutlass_include() -> str:
    import site
    for sp in site.getsitepackages():
        for c in CUTLASS_CANDIDATES:
            p = os.path.join(sp, c)
            if os.path.isfile(os.path.join(p, "cute", "tensor.hpp")):
                return p
    raise RuntimeError("no CUTLASS/CuTe header tree found in site-packages")


def _rewrite_gencode(flags):
    out, skip = [], False
    seen = False
    for f in flags or []:
        if skip:
            skip = False
            continue
        if f == "-gencode":
            skip = True
            if not seen:
                out += ["-gencode", "arch=compute_100,code=sm_100"]
                seen = True
            continue
        out.append(f)
    if not seen:
        out += ["-gencode", "arch=compute_100,code=sm_100"]
    return out


def _wrap_load_inline(real):
    def load_inline(name, cpp_sources, cuda_sources=None, extra_cuda_cflags=None,
                    extra_include_paths=None, **kw):
        flags = _rewrite_gencode(extra_cuda_cflags)
        h = hashlib.sha256()
        for s in list(cpp_sources) + list(cuda_sources or []) + flags:
            h.update(s.encode())
        # headers the sources include from the reference's csrc folder
        csrc = os.path.join(REF, "flash_topk_attn_v2", "csrc")
        for f in sorted(os.listdir(csrc)):
            if f.endswith(".cuh"):
                h.update(open(os.path.join(csrc, f), "rb").read())
        digest = h.hexdigest()
        bdir = os.path.join(EXT, name)
        so, stamp = os.path.join(bdir, name + ".so"), os.path.join(bdir, "stamp")
        if (os.path.isfile(so) and os.path.isfile(stamp)
                and open(stamp).read().strip() == digest):
            import torch  # noqa: F401  (the extension links against libtorch)
            spec = importlib.util.spec_from_file_location(name, so)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            return mod
        os.makedirs(bdir, exist_ok=True)
        kw.pop("build_directory", None)
        mod = real(name=name, cpp_sources=cpp_sources, cuda_sources=cuda_sources,
                   extra_cuda_cflags=flags, extra_include_paths=extra_include_paths,
                   build_directory=bdir, **kw)
        with open(stamp, "w") as f:
            f.write(digest)
        return mod
    return load_inline


def load():
    """Import the reference package from baseline/_ref with the two patches."""
    if not available():
        raise RuntimeError("baseline/_ref is absent: install the reference there first")
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    sys.path[:] = [p for p in sys.path if "flash-topk-attention_b200" not in p]
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import flash_topk_attn_v2 as ref
    assert os.path.dirname(os.path.abspath(ref.__file__)).startswith(REF), ref.__file__
    cutlass = _cutlass_include()
    for name in EXT_MODULES:
        m = importlib.import_module("flash_topk_attn_v2." + name)
        if hasattr(m, "_CUTLASS_INCLUDE"):
            m._CUTLASS_INCLUDE = cutlass
        if not getattr(m.load_inline, "_ftk_patched", False):
            w = _wrap_load_inline(m.load_inline)
            w._ftk_patched = True
            m.load_inline = w
    return ref


def prebuild(only=None) -> dict:
    """Compile the extensions (works without a GPU; each is one long nvcc run, so
    separate processes with --only build them side by side); seconds per module."""
    load()
    out = {}
    for name in (only or EXT_MODULES):
        m = importlib.import_module("flash_topk_attn_v2." + name)
        t0 = time.time()
        m._get_ext()
        out[name] = round(time.time() - t0, 1)
        print(name, out[name], "s", flush=True)
    return out


# --------------------------------------------------------------------------------------
# running the chain


def _sync_check(torch, what):
    torch.cuda.synchronize()
    err = torch.cuda.current_stream().query()  # raises on a sticky error
    del err
    print("ok:", what, flush=True)


def _case(name):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import cases
    if name in cases.GOLDEN_CASES:
        return cases, dict(cases.GOLDEN_CASES[name])
    if name.startswith("config"):
        return cases, dict(cases.BASELINE_CONFIGS[int(name[6:])])
    raise KeyError(name)


def run_case(case, out, stages, cfg_json=None):
    import numpy as np
    import torch
    ref = load()
    if cfg_json:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import cases
        cfg = json.loads(cfg_json)
    else:
        cases, cfg = _case(case)
    t = cases.make_inputs(cfg)
    dev = torch.device("cuda", 0)
    H, b, g, kvb = cfg["H"], cfg["score_block_size"], cfg["q_block_size"], cfg["kv_block_size"]
    res = {}
    q = t["q"].to(dev)
    k = t["k"].to(dev)
    v = t["v"].to(dev)
    idx = avg = merged = None
    if "score" in stages:
        idx, raw, avg = ref.flash_topk_score(q, k, H, b, cfg["topk"], tuple(cfg["padding"]),
                                             cfg["threshold"])
        _sync_check(torch, "flash_topk_score")
        res.update(topk_idx=idx.cpu().numpy(), topk_raw=raw.cpu().numpy(),
                   topk_avg=avg.cpu().numpy())
    if "merge" in stages:
        merged, counts, W = ref.build_qblock_topk_indices(
            idx, g, tuple(cfg["q_padding"]),
            avg if cfg.get("score_weighted", True) else None, cfg.get("qblock_topk"))
        _sync_check(torch, "build_qblock_topk_indices")
        res.update(merged=merged.cpu().numpy(), counts=counts.cpu().numpy())
    if "attn" in stages and cfg.get("attend", True):
        q.requires_grad_(True)
        k.requires_grad_(True)
        v.requires_grad_(True)
        o, lse = ref.flash_topk_attn(q, k, v, merged, counts, H, g, kvb,
                                     kv_padding=tuple(cfg["kv_padding"]),
                                     q_padding=tuple(cfg["q_padding"]))
        _sync_check(torch, "flash_topk_attn forward")
        res.update(o=o.detach().float().cpu().numpy(), lse=lse.detach().cpu().numpy())
        if "bwd" in stages:
            o.backward(t["do"].to(dev))
            _sync_check(torch, "flash_topk_attn backward")
            res.update(dq=q.grad.float().cpu().numpy(), dk=k.grad.float().cpu().numpy(),
                       dv=v.grad.float().cpu().numpy())
    np.savez(out, **res)
    print("wrote", out, sorted(res))


SHAPES = {
    # the bench workload of this repository: B=1, N=32768, H=32, D=128, bf16
    "headline": dict(B=1, N=32768, H=32, D=128, dtype="bf16", input_scale=0.5,
                     score_block_size=64, topk=32, threshold=0.9, q_block_size=64,
                     kv_block_size=64),
    "small": dict(B=1, N=8192, H=8, D=128, dtype="bf16", input_scale=0.5,
                  score_block_size=64, topk=32, threshold=0.9, q_block_size=64,
                  kv_block_size=64),
}


def time_chain(shape, steps, warmup, heads=None, quiet=False, cfg=None):
    """Per-stage and whole-chain CUDA-event times of the reference on one GPU.
    `cfg` (keys as in SHAPES, optional qblock_topk) overrides the named shape."""
    import torch
    ref = load()
    cfg = dict(cfg) if cfg else dict(SHAPES[shape])
    if heads:
        cfg["H"] = heads
    dev = torch.device("cuda", 0)
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[cfg["dtype"]]
    B, N, H, D = cfg["B"], cfg["N"], cfg["H"], cfg["D"]
    gen = torch.Generator().manual_seed(0)
    mk = lambda: (torch.randn(B, N, H * D, generator=gen) * cfg["input_scale"]).to(dt).to(dev)
    q, k, v, do = mk(), mk(), mk(), mk()
    b, g, kvb = cfg["score_block_size"], cfg["q_block_size"], cfg["kv_block_size"]
    names = ("score", "merge", "fwd", "bwd")
    acc = {n: 0.0 for n in names}
    total = 0.0

    def step(timed):
        nonlocal total
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        qq, kk, vv = (x.detach().requires_grad_(True) for x in (q, k, v))
        ev[0].record()
        idx, raw, avg = ref.flash_topk_score(qq.detach(), kk.detach(), H, b, cfg["topk"], (0, 0),
                                             cfg["threshold"])
        ev[1].record()
        merged, counts, W = ref.build_qblock_topk_indices(idx, g, topk_scores=avg,
                                                          qblock_topk=cfg.get("qblock_topk"))
        ev[2].record()
        o, lse = ref.flash_topk_attn(qq, kk, vv, merged, counts, H, g, kvb)
        ev[3].record()
        o.backward(do)
        ev[4].record()
        torch.cuda.synchronize()
        if timed:
            for i, n in enumerate(names):
                acc[n] += ev[i].elapsed_time(ev[i + 1])
            total += ev[0].elapsed_time(ev[4])
        return int(counts.sum().item())

    for _ in range(warmup):
        pairs = step(False)
    for _ in range(steps):
        pairs = step(True)
    line = {"impl": "reference-v2-gpu", "shape": shape, "config": cfg, "steps": steps,
            "warmup": warmup, "ms_per_step": total / steps,
            "stage_ms": {n: acc[n] / steps for n in names},
            "tokens_per_s": B * N / (total / steps) * 1e3, "pairs": pairs,
            "gpu": torch.cuda.get_device_name(0)}
    if not quiet:
        print(json.dumps(line))
    return line


def main():
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    pb = sub.add_parser("prebuild")
    pb.add_argument("--only", default="")
    r = sub.add_parser("run")
    r.add_argument("--case", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--stages", default="score,merge,attn,bwd")
    r.add_argument("--cfg", default="", help="the whole case as JSON (keys as in tests/cases.py)")
    t = sub.add_parser("time")
    t.add_argument("--shape", default="headline")
    t.add_argument("--steps", type=int, default=5)
    t.add_argument("--warmup", type=int, default=2)
    t.add_argument("--heads", type=int, default=0)
    a = ap.parse_args()
    if a.cmd == "prebuild":
        prebuild([x for x in a.only.split(",") if x] or None)
    elif a.cmd == "run":
        run_case(a.case, a.out, a.stages.split(","), a.cfg or None)
    else:
        time_chain(a.shape, a.steps, a.warmup, a.heads or None)


if __name__ == "__main__":
    main()
