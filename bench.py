#!/usr/bin/env python
"""Benchmark of the flash_topk_attn_v2 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the path over one batch of synthetic input:
flash_topk_score -> build_qblock_topk_indices -> flash_topk_attn -> backward,
at B=1 (per GPU), N=32768, H=32, D=128, bf16, score block 64, topk 32,
threshold 0.9, q/kv block 64 (the shape the headline metric is quoted on).
Rank r draws its own batch element (seed r); ranks never exchange data, so
scaling is weak: `value` is the tokens all ranks processed per second of the
slowest rank's device time.

`--impl reference` times the CPU restatement of the reference's dense PyTorch
path (oracle/) on the host cores over a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "flash-topk-attention_b200"))
sys.path.insert(0, ROOT)

# The CPU legs use every host core whatever launched this process: torchrun
# exports OMP_NUM_THREADS=1, which the BLAS behind numpy reads when it loads.
HOST_CORES = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
if "reference" in sys.argv:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(HOST_CORES)

import numpy as np  # noqa: E402
import torch  # noqa: E402

WORKLOAD = dict(
    name="config2-e2e", B=1, N=32768, H=32, D=128, dtype="bf16", input_scale=0.5,
    score_block_size=64, topk=32, threshold=0.9, q_block_size=64, kv_block_size=64,
    qblock_topk=None,
)
# Side workloads (--workload): the other BASELINE.json shapes, per GPU.  The
# headline line always comes from WORKLOAD above.
WORKLOADS = {
    "config2-e2e": WORKLOAD,
    # configs[0]: the reference's CPU-runnable shape
    "config1": dict(name="config1", B=2, N=1024, H=8, D=64, dtype="fp16", input_scale=1.0,
                    score_block_size=64, topk=16, threshold=1.0, q_block_size=32,
                    kv_block_size=64, qblock_topk=None),
    # configs[2]: full training step, score-weighted merge to 256 blocks
    "config3": dict(name="config3", B=4, N=8192, H=16, D=128, dtype="bf16", input_scale=1.0,
                    score_block_size=64, topk=16, threshold=1.0, q_block_size=64,
                    kv_block_size=64, qblock_topk=256),
    # configs[3]: ragged length, virtual padding, hot key blocks, fp16; score + select +
    # merge only (q blocks of 128 rows: the reference's attention stops at 64)
    "config4": dict(name="config4", B=2, N=30000, H=32, D=128, dtype="fp16", input_scale=1.0,
                    score_block_size=128, topk=24, threshold=0.8, q_block_size=128,
                    kv_block_size=128, qblock_topk=None, padding=(40, 40), q_padding=(40, 40),
                    attend=False),
    # configs[4]: one batch element (64 of its 512 slices) per GPU
    "config5": dict(name="config5", B=1, N=65536, H=64, D=128, dtype="bf16", input_scale=1.0,
                    score_block_size=64, topk=64, threshold=1.0, q_block_size=64,
                    kv_block_size=64, qblock_topk=None),
}
METRIC = "score+sparse fwd+bwd tokens/s @N=32k,H=32,D=128 bf16"
UNIT = "tokens/s"


# DRAM bytes (read + written) per launch and per head, measured with ncu at B=1, N=32768, H=4
# (profiles/dram_traffic_n32768_h4.txt).  Every kernel works on (batch, head) slices
# independently, so a launch over B*H slices of this sequence length moves B*H times this.
DRAM_BYTES_PER_SLICE_N32768 = {
    "ftk_score_topk": (85.0e6 + 224.0e6 + 269.0e6 + 36.3e6) / 4,
    "ftk_qblock_merge": (33.7e6 + 33.6e6) / 4,
    "ftk_sparse_fwd": (118.1e6 + 19.5e6) / 4,
    "ftk_sparse_bwd_dq": (67.1e6 + 153.3e6 + 19.9e6) / 4,
    "ftk_sparse_bwd_dkv": (143.6e6 + 41.7e6) / 4,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sus=d["bf16_tflops_sustained"],
                    src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sus=1400.0, src="fallback")


# ---------------------------------------------------------------------------
# host placement
# ---------------------------------------------------------------------------
def bind_near_gpu(index):
    """Run this rank on the CPU cores next to its GPU (read from NVML), so the
    pinned host buffers it allocates afterwards land on that NUMA node and the
    end-to-end copies do not cross sockets.  Only the process's own CPU affinity
    changes; nothing about the GPU is set.  Returns the number of cores or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


# ---------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------
def make_host_inputs(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    shape = (cfg["B"], cfg["N"], cfg["H"] * cfg["D"])
    s = cfg["input_scale"]
    dt = torch.float16 if cfg.get("dtype") == "fp16" else torch.bfloat16
    out = {}
    for name in ("q", "k", "v"):
        out[name] = (torch.randn(shape, generator=g) * s).to(dt).pin_memory()
    g2 = torch.Generator().manual_seed(1000 + seed)
    out["do"] = torch.randn(shape, generator=g2).to(dt).pin_memory()
    return out


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def run_ours(args):
    import flash_topk_attn_v2 as ftk
    from flash_topk_attn_v2 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    near = bind_near_gpu(local) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    cfg = dict(WORKLOADS[args.workload])
    if args.small:
        cfg.update(N=8192, H=16, name="small")
    if args.seq or args.heads:
        cfg.update(N=args.seq or cfg["N"], H=args.heads or cfg["H"])
        cfg["name"] = f"{cfg['name']}-n{cfg['N']}-h{cfg['H']}"
    if args.head_dim and args.head_dim != cfg["D"]:
        cfg.update(D=args.head_dim, name=f"{cfg['name']}-d{args.head_dim}")
    H, D, N, B = cfg["H"], cfg["D"], cfg["N"], cfg["B"]
    b, K, thr = cfg["score_block_size"], cfg["topk"], cfg["threshold"]
    g, kvb = cfg["q_block_size"], cfg["kv_block_size"]
    host = make_host_inputs(cfg, seed=rank)
    devt = {k: torch.empty_like(v, device=dev) for k, v in host.items()}
    for k in devt:
        devt[k].copy_(host[k])
    host_out = {k: torch.empty_like(host["q"]).pin_memory() for k in ("o", "dq", "dk", "dv")}

    stage_ms = {"score_select": 0.0, "merge": 0.0, "sparse_fwd": 0.0, "sparse_bwd": 0.0}
    pairs = [0]

    def step(record, before_attn=None, after_fwd=None):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if record else None
        q = devt["q"].detach().requires_grad_(True)
        k = devt["k"].detach().requires_grad_(True)
        v = devt["v"].detach().requires_grad_(True)
        if record:
            evs[0].record()
        idx, raw, avg = ftk.flash_topk_score(q.detach(), k.detach(), H, b, K,
                                             tuple(cfg.get("padding", (0, 0))), thr)
        if record:
            evs[1].record()
        merged, counts, W = ftk.build_qblock_topk_indices(
            idx, g, tuple(cfg.get("q_padding", (0, 0))), avg, cfg["qblock_topk"])
        if record:
            evs[2].record()
        if not cfg.get("attend", True):
            # workloads that stop after the merge (configs[3])
            if record:
                evs[3].record()
                evs[4].record()
            return evs, (merged, None, None, None, counts)
        if before_attn is not None:
            before_attn()          # end-to-end leg: V and dO have arrived
        o, lse = ftk.flash_topk_attn(q, k, v, merged, counts, H, g, kvb)
        if record:
            evs[3].record()
        if after_fwd is not None:
            after_fwd(o)           # end-to-end leg: O goes home under the backward
        o.backward(devt["do"])
        if record:
            evs[4].record()
        return evs, (o, q.grad, k.grad, v.grad, counts)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        _, res = step(False)
    torch.cuda.synchronize()
    ftk.check_errors()
    pairs[0] = int(res[4].sum().item())

    # ---- device-resident timing -------------------------------------------
    sampler = ClockSampler(local)
    launches0 = ops.launch_count()
    barrier()
    ops.enable_event_timing(True)
    sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    all_evs = []
    t0.record()
    for _ in range(args.steps):
        evs, res = step(True)
        all_evs.append(evs)
    t1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    call_ms = {k: v[0] / args.steps for k, v in ops.event_times().items()}
    ops.enable_event_timing(False)
    launches = ops.launch_count() - launches0
    ms = t0.elapsed_time(t1)
    for evs in all_evs:
        for i, nm in enumerate(stage_ms):
            stage_ms[nm] += evs[i].elapsed_time(evs[i + 1]) / args.steps
    ftk.check_errors()

    # ---- end to end: host buffers in, host buffers out --------------------
    # Every step's four inputs come from pinned host memory and its four
    # results go back to pinned host memory, all inside the timed region.  The
    # copies run on two side streams (PCIe is full duplex) over double-buffered
    # device inputs, so step i+1's upload and step i-1's download overlap step
    # i's kernels; scoring starts as soon as Q and K are there (V and dO follow
    # under it) and O leaves under the backward.  Dependencies are CUDA events.
    cur = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    bufs = [devt, {k: torch.empty_like(v) for k, v in devt.items()}]
    ev_qk = [torch.cuda.Event(), torch.cuda.Event()]
    ev_in = [torch.cuda.Event(), torch.cuda.Event()]
    ev_done = [torch.cuda.Event(), torch.cuda.Event()]

    def upload(i):
        with torch.cuda.stream(s_in):
            for k in ("q", "k"):
                bufs[i % 2][k].copy_(host[k], non_blocking=True)
            ev_qk[i % 2].record(s_in)
            for k in ("v", "do"):
                bufs[i % 2][k].copy_(host[k], non_blocking=True)
            ev_in[i % 2].record(s_in)

    def download(names, tensors):
        ev = torch.cuda.Event()
        ev.record(cur)
        s_out.wait_event(ev)
        with torch.cuda.stream(s_out):
            for nm, t in zip(names, tensors):
                if t is None:      # workload without attention: nothing to send home
                    continue
                host_out[nm].copy_(t, non_blocking=True)
                t.record_stream(s_out)

    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    upload(0)
    keep = []
    for i in range(args.steps):
        devt = bufs[i % 2]
        cur.wait_event(ev_qk[i % 2])
        _, res = step(False, before_attn=lambda i=i: cur.wait_event(ev_in[i % 2]),
                      after_fwd=lambda o: download(("o",), (o.detach(),)))
        ev_done[i % 2].record(cur)
        if i + 1 < args.steps:
            if i >= 1:
                # buffer (i+1)%2 was last read by step i-1: the copy stream
                # must not overwrite it before that step's kernels finished
                s_in.wait_event(ev_done[(i + 1) % 2])
            upload(i + 1)
        download(("dq", "dk", "dv"), res[1:4])
        keep.append(res)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    devt = bufs[0]
    del keep
    ftk.check_errors()

    # the same copies with no kernels: what the host <-> device path alone takes per step
    barrier()
    c0 = torch.cuda.Event(enable_timing=True)
    c1 = torch.cuda.Event(enable_timing=True)
    copy_steps = min(args.steps, 3)
    c0.record()
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    for i in range(copy_steps):
        with torch.cuda.stream(s_in):
            for k in ("q", "k", "v", "do"):
                bufs[i % 2][k].copy_(host[k], non_blocking=True)
        with torch.cuda.stream(s_out):
            for nm, src in zip(("o", "dq", "dk", "dv"), ("q", "k", "v", "do")):
                host_out[nm].copy_(bufs[(i + 1) % 2][src], non_blocking=True)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
    c1.record()
    torch.cuda.synchronize()
    copy_ms = c0.elapsed_time(c1) / copy_steps
    for k in devt:
        devt[k].copy_(host[k])
    torch.cuda.synchronize()

    if dist is not None:
        tt = torch.tensor([ms, e2e_ms, copy_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_ms, copy_ms = float(tt[0]), float(tt[1]), float(tt[2])
    tokens_per_step = world * B * N
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    bytes_in = sum(v.numel() * v.element_size() for v in host.values())
    bytes_out = sum(v.numel() * v.element_size() for v in host_out.values())

    if rank == 0:
        peaks = measured_peaks()
        P = pairs[0]
        unit_flops = D * g * kvb * P           # one GEMM over every (q-block, kv-block) pair
        # algorithmic flops per C-ABI call (recomputation inside a kernel is not counted):
        #   scoring  one Q.K^T                      2 B H N^2 D
        #   forward  S and P.V                      4 per pair unit
        #   dQ call  S, dP, dQ                      6 per pair unit
        #   dK/dV    dK, dV (it also recomputes S^T and dP^T: 8 executed)  4 per pair unit
        kern = {
            "ftk_score_topk": dict(flops=2.0 * B * H * N * N * D),
            "ftk_sparse_fwd": dict(flops=4.0 * unit_flops),
            "ftk_sparse_bwd_dq": dict(flops=6.0 * unit_flops),
            "ftk_sparse_bwd_dkv": dict(flops=4.0 * unit_flops, executed_flops=8.0 * unit_flops),
        }
        for name, d in kern.items():
            d["ms"] = call_ms.get(name, 0.0)
            d["tflops"] = d["flops"] / (d["ms"] * 1e-3) / 1e12 if d["ms"] > 0 else 0.0
            d["frac"] = d["tflops"] / peaks["tf_sus"]
            if "executed_flops" in d:
                d["executed_tflops"] = d.pop("executed_flops") / (d["ms"] * 1e-3) / 1e12 \
                    if d["ms"] > 0 else 0.0
        dom = max(kern, key=lambda n: kern[n]["ms"])
        line = {
            "metric": METRIC.replace("D=128", f"D={D}").replace("N=32k", f"N={N // 1024}k")
            .replace("H=32", f"H={H}"),
            "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": cfg.get("dtype", "bf16"), "data": "synthetic",
            "config": {"workload": cfg["name"], "B_per_gpu": B, "N": N, "H": H, "D": D,
                       "score_block_size": b, "topk": K, "threshold": thr, "q_block_size": g,
                       "kv_block_size": kvb, "sharding": "batch x head slices, no collective",
                       "host_cores_near_gpu": near,
                       "l2": f"inputs larger than L2 (4 x {B * N * H * D * 2 // 1000000} MB per step)",
                       "candidate_pairs_per_step": P},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": bytes_in,
                    "d2h_bytes_per_step": bytes_out, "ms_per_step": e2e_ms / args.steps,
                    "host_copy_only_ms": copy_ms,
                    "host_copy_only_note": "the step's uploads and downloads alone, no kernels, "
                                           "both directions at once, max over ranks"},
            "gpu_launches": launches,
            "stage_ms": stage_ms,
            "call_ms": call_ms,
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": kern[dom]["tflops"],
                         "peak": peaks["tf_sus"], "unit": "TFLOP/s",
                         "frac": kern[dom]["frac"],
                         "traffic": (DRAM_BYTES_PER_SLICE_N32768[dom] * B * H
                                     if N == 32768 and D == 128 else None),
                         "traffic_unit": "bytes per launch (DRAM read + written)",
                         "traffic_note": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one "
                                         "launch at B=1, N=32768, H=4, times B*H/4: slices are "
                                         "independent, traffic is proportional to their number "
                                         "(profiles/dram_traffic_n32768_h4.txt)",
                         "traffic_all": ({n: v * B * H for n, v in
                                          DRAM_BYTES_PER_SLICE_N32768.items()}
                                         if N == 32768 and D == 128 else None),
                         "peak_source": peaks["src"] + " bf16, sustained (kernel timed inside a "
                                        "100 ms step)",
                         "score_frac_of_burst_peak": kern["ftk_score_topk"]["tflops"] / peaks["tf"],
                         "all": {n: {k2: v2 for k2, v2 in d.items() if k2 != "flops"}
                                 for n, d in kern.items()}},
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(cfg, seconds=args.cpu_seconds)
        if world == 1 and not args.no_reference_gpu and cfg["name"] == WORKLOAD["name"]:
            # the reference's own V2 CUDA kernels on this GPU, same shape, in a child process
            # (both packages are called flash_topk_attn_v2)
            line["reference_v2_gpu"] = reference_gpu_leg(ms / args.steps)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# CPU arm (the oracle port, reported baseline only)
# ---------------------------------------------------------------------------
def cpu_sample_step(cfg, x, rows):
    """One bounded sample: `rows` query rows of one (batch, head) slice through
    score -> select -> merge -> sparse fwd -> bwd, fp32 numpy on all cores."""
    from oracle import ftk_oracle as orc
    b, K, thr = cfg["score_block_size"], cfg["topk"], cfg["threshold"]
    g, kvb, N = cfg["q_block_size"], cfg["kv_block_size"], cfg["N"]
    q, k, v, do = x
    M = N // b
    scale = np.float32(cfg["D"] ** -0.5)
    s = (q[:rows] * scale) @ k.T
    s -= s.max(axis=1, keepdims=True)
    np.exp(s, out=s)
    s /= s.sum(axis=1, keepdims=True)
    scores = s.reshape(rows, M, b).sum(-1)[None, None]
    idx, raw, avg = orc.topk_select(scores, thr, K, b)
    merged, counts, W, _ = orc.build_qblock_topk_indices(idx, g, (0, 0), avg, None)
    # attention over the sampled q-blocks only; keys/values are the full slice
    qm = rows // g
    pad_rows = np.zeros((N - rows, q.shape[1]), dtype=np.float32)
    qfull = np.concatenate([q[:rows], pad_rows])[None]
    dofull = np.concatenate([do[:rows], pad_rows])[None]
    mfull = np.full((1, 1, N // g, W), -1, dtype=np.int32)
    mfull[0, 0, :qm] = merged[0, 0]
    o, lse = orc.sparse_attn_fwd(qfull, k[None], v[None], mfull, 1, g, kvb, work=np.float32)
    orc.sparse_attn_bwd(qfull, k[None], v[None], o, lse, dofull, mfull, 1, g, kvb,
                        work=np.float32)
    return rows


def cpu_baseline(cfg, seconds=15.0, rows=512):
    cores = use_all_host_cores()
    N, H, D = cfg["N"], cfg["H"], cfg["D"]
    g = torch.Generator().manual_seed(0)
    x = [(torch.randn(N, D, generator=g) * cfg["input_scale"]).to(torch.bfloat16).float().numpy()
         for _ in range(4)]
    rows = min(rows, N)
    cpu_sample_step(cfg, x, min(rows, 128))  # warm
    t0 = time.perf_counter()
    done = 0
    while True:
        done += cpu_sample_step(cfg, x, rows)
        el = time.perf_counter() - t0
        if el > seconds or done >= N:
            break
    # `done` rows of ONE head took `el` seconds; a token needs all H heads
    return {"value": done / H / el, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{done} query rows of one (batch, head) slice, full key length {N}, "
                      f"score+select+merge+sparse fwd+bwd in fp32 numpy ({el:.1f} s); "
                      f"extrapolated to {H} heads"}


def use_all_host_cores() -> int:
    """numpy's BLAS and torch on every core this process may run on; returns the count."""
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=HOST_CORES)
    except Exception:
        pass
    torch.set_num_threads(HOST_CORES)
    return HOST_CORES


def reference_gpu_leg(our_ms_per_step, steps=3, warmup=2):
    """Run `bench.py --impl reference-gpu` as a child and return its line plus the ratio."""
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flash_topk_attn_v2")):
        return {"unavailable": "baseline/_ref (the reference install) is absent"}
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu",
                            "--steps", str(steps), "--warmup", str(warmup)],
                           capture_output=True, text=True, timeout=1500, env=env, cwd=ROOT)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        out = json.loads(lines[-1]) if lines else {"unavailable": (r.stderr or "no output")[-400:]}
    except Exception as e:  # noqa: BLE001
        out = {"unavailable": f"{type(e).__name__}: {e}"[:400]}
    if "ms_per_step" in out:
        out["speedup_device_timed"] = out["ms_per_step"] / our_ms_per_step
    return out


def run_reference_gpu(args):
    """The reference's own flash_topk_attn_v2 CUDA path on this GPU, same workload,
    CUDA-event timed, inputs resident (its extensions rebuilt for sm_100 at run time by
    baseline/ref_v2_gpu.py; nothing of this repository's kernels is on that path)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import ref_v2_gpu
        if not ref_v2_gpu.available():
            raise RuntimeError("baseline/_ref (the reference install) is absent")
        wl = {k: v for k, v in WORKLOADS[args.workload].items() if k != "name"}
        if args.head_dim and args.head_dim != wl["D"]:
            wl["D"] = args.head_dim
        line = ref_v2_gpu.time_chain(args.workload, args.steps, max(args.warmup, 1), quiet=True,
                                     cfg=wl)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"{type(e).__name__}: {e}"[:600]}),
              flush=True)
        return
    cfg = line.pop("config")
    out = {
        "impl": "reference-gpu", "metric": METRIC, "value": line["tokens_per_s"], "unit": UNIT,
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 1),
        "ms_per_step": line["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": cfg.get("dtype", "bf16"), "data": "synthetic",
        "config": {"workload": args.workload, "B_per_gpu": cfg["B"], "N": cfg["N"],
                   "H": cfg["H"], "D": cfg["D"], "score_block_size": cfg["score_block_size"],
                   "topk": cfg["topk"], "threshold": cfg["threshold"],
                   "q_block_size": cfg["q_block_size"], "kv_block_size": cfg["kv_block_size"]},
        "stage_ms": line["stage_ms"], "candidate_pairs_per_step": line["pairs"],
        "gpu": line["gpu"],
        "how": "reference package from baseline/_ref, its CUDA extensions compiled for sm_100 "
               "with the image's CUTLASS headers (run-time patch, no source edits), CUDA events "
               "around flash_topk_score -> build_qblock_topk_indices -> flash_topk_attn -> backward",
    }
    print(json.dumps(out), flush=True)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = use_all_host_cores()
    cfg = dict(WORKLOAD)
    N, H, D = cfg["N"], cfg["H"], cfg["D"]
    g = torch.Generator().manual_seed(0)
    x = [(torch.randn(N, D, generator=g) * cfg["input_scale"]).to(torch.bfloat16).float().numpy()
         for _ in range(4)]
    rows = 256
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_sample_step(cfg, x, 128)
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        done += cpu_sample_step(cfg, x, rows)
    el = time.perf_counter() - t0
    value = done / H / el
    sample = (f"each step = {rows} query rows of one (batch, head) slice against all {N} keys, "
              f"extrapolated to {H} heads")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": cfg["name"], "B_per_gpu": cfg["B"], "N": N, "H": H, "D": D,
                   "score_block_size": cfg["score_block_size"], "topk": cfg["topk"],
                   "threshold": cfg["threshold"], "q_block_size": cfg["q_block_size"],
                   "kv_block_size": cfg["kv_block_size"],
                   "reference_arm": "one process on rank 0's host cores whatever --gpus is: "
                                    "its value does not grow with N"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="reference = the reference's dense CPU formulation on the host cores; "
                         "reference-gpu = the reference's own V2 CUDA kernels on this GPU "
                         "(needs baseline/_ref)")
    ap.add_argument("--workload", default="config2-e2e", choices=sorted(WORKLOADS),
                    help="side workloads: the other BASELINE.json shapes (per GPU)")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip the reference-V2-on-this-GPU leg of the default run")
    ap.add_argument("--small", action="store_true", help="N=8192, H=16 (profiling-sized case)")
    ap.add_argument("--head-dim", type=int, default=0,
                    help="head dim other than the headline 128 (profiling / side measurements; "
                         "the workload name says so)")
    ap.add_argument("--seq", type=int, default=0, help="sequence length override (profiling)")
    ap.add_argument("--heads", type=int, default=0, help="head count override (profiling)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "reference-gpu":
        run_reference_gpu(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
