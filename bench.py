#!/usr/bin/env python
"""Benchmark of the HiLS attention hot path (forward + backward of one attention layer's op chain).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "c2"): B=8, T=8192, 16 heads (MHA), head_dim 64, chunk 64 (128 chunks),
top-k 32, window 512, causal, bf16; q, v ~ N(0,1), k ~ N(0,1) + a per-(batch, chunk, head) offset
~ N(0, 0.5), dO ~ N(0,1), landmark query = q; all seeded.  A step is: sliding-window branch ->
chunk pooling (k', b') -> chunk selection -> inter-chunk softmax -> sparse chunk attention ->
combine, and the backward of all of it.  With N > 1 every rank runs the same shape on its own
batch (the path shards by batch/head with no collective): weak scaling, value = total tokens/s.

Prints ONE JSON line.  `value` is timed with inputs resident in HBM; `e2e` times the same step
through the public API with pinned HOST buffers (q, k, v, dO copied in; o, dq, dk, dv copied out
every step, copies of neighbouring steps overlapped with compute by hils_attention_b200.host_pipeline).
`roofline` is for the dominant kernel, timed alone with CUDA events on the launch stream.
`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the host
cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, T, h_q, h_kv, D, S, K, W
    "c2": dict(B=8, T=8192, h_q=16, h_kv=16, D=64, S=64, K=32, W=512),
    "c2_small": dict(B=1, T=8192, h_q=16, h_kv=16, D=64, S=64, K=32, W=512),
    # same tokens with the head grouping of the reference's 345M model (2 kv heads, groups of 8 query heads)
    "c2_gqa": dict(B=8, T=8192, h_q=16, h_kv=2, D=64, S=64, K=32, W=512),
    "c3": dict(B=1, T=65536, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    # decode: 32 sequences, one new token each, against a 131072-token KV store
    "c4": dict(B=32, T=131072, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    "c4_small": dict(B=4, T=16384, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
}
CPU_SAMPLE = dict(B=1, T=2048, h_q=16, h_kv=16, D=64, S=64, K=8, W=512)   # the reference's CPU-runnable case


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def make_inputs(w, seed, device, dtype):
    g = torch.Generator().manual_seed(seed)
    B, T, hq, hk, D, S = w["B"], w["T"], w["h_q"], w["h_kv"], w["D"], w["S"]
    q = torch.randn(B, T, hq, D, generator=g)
    k = torch.randn(B, T, hk, D, generator=g)
    off = torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5
    k[:, :(T // S) * S] += off.expand(-1, -1, S, -1, -1).reshape(B, (T // S) * S, hk, D)
    v = torch.randn(B, T, hk, D, generator=g)
    do = torch.randn(B, T, hq, D, generator=g)
    return [t.to(dtype).pin_memory() if device != "cpu" else t.to(dtype) for t in (q, k, v, do)]


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for n, val in zip(names, r[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_chain_tokens_per_s(steps=1):
    """The oracle's fp32 chain (fwd + bwd) on the host cores, at CPU_SAMPLE."""
    from oracle import hils_oracle as orc
    w = CPU_SAMPLE
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1)
    B, T, H, D = w["B"], w["T"], w["h_q"], w["D"]
    q, k, v = (torch.randn(B, T, H, D, generator=g) / math.sqrt(D) for _ in range(3))
    do = torch.randn(B, T, H, D, generator=g)
    best = None
    for _ in range(steps):
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        t0 = time.perf_counter()
        o = orc.hils_attention_chain(qq, kk, vv, qq, chunk_size=w["S"], window_size=w["W"], topk=w["K"])
        o.backward(do)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return B * T / best, cores, best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    times = []
    for i in range(args.warmup + args.steps):
        tps, cores, dt = cpu_chain_tokens_per_s(1)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = CPU_SAMPLE["B"] * CPU_SAMPLE["T"] / (ms / 1e3)
    sample = ("CPU restatement of the reference's PyTorch chain, fp32, fwd+bwd, on B=1 T=2048 H=16 D=64 "
              "S=64 K=8 W=512 (the reference's CPU-runnable configuration)")
    print(json.dumps({
        "impl": "reference", "metric": "hils_attn_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, **w, "sample": "B=1,T=2048,K=8 (bounded CPU sample)"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_decode(args):
    """Decode against a cached HiLS KV store: one new token per sequence and step through the whole
    chain (store append, sliding-window branch, selection over the pooled chunk keys, inter-chunk
    softmax, sparse chunk attention, combine).  The batch is sharded over the ranks (no collective)."""
    import torch.distributed as dist
    from hils_attention_b200 import _lib
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.cache import HiLSCache
    import hils_attention_b200 as hb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    Bt, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    B = max(1, Bt // world)
    dtype = torch.bfloat16
    n_e2e = 16
    n_steps = args.warmup + args.steps + n_e2e + 3
    cap = T + n_steps + 8
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    kbuf = torch.empty((cap, B, hk, D), dtype=dtype, device=dev)
    vbuf = torch.empty((cap, B, hk, D), dtype=dtype, device=dev)
    for t0 in range(0, T, 4096):                                   # fill in slices: no second copy of the store
        n = min(4096, T - t0)
        off = torch.randn((n // S + 1, 1, B, hk, D), generator=g, device=dev) * 0.5
        off = off.expand(-1, S, -1, -1, -1).reshape(-1, B, hk, D)[:n]
        kbuf[t0:t0 + n] = (torch.randn((n, B, hk, D), generator=g, device=dev) + off).to(dtype)
        vbuf[t0:t0 + n] = torch.randn((n, B, hk, D), generator=g, device=dev).to(dtype)
    cache = HiLSCache()
    layer = cache.layer(1)
    layer.adopt(kbuf, vbuf, T)
    N = T // S
    with torch.no_grad():                                          # pooled chunk keys of the cached prefix
        kf, _ = layer.folded()
        mu = torch.randn((1, N, B * hq, D), generator=g, device=dev).to(dtype)
        lmk_k, prior_b = hb.chunk_attn_pool(mu, kf[:, :N * S].unflatten(1, (N, S)))
    cache._hils_prior_cache[0] = {"lmk_k": lmk_k, "prior_b": prior_b}
    core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).eval()
    host = [torch.randn((B, 1, h, D), generator=torch.Generator().manual_seed(9 + i)).to(dtype).pin_memory()
            for i, h in enumerate((hq, hk, hk))]
    qn, kn, vn = (t.to(dev) for t in host)
    out_host = torch.empty((B, 1, hq, D), dtype=dtype).pin_memory()

    def step(q1, k1, v1):
        with torch.no_grad():
            return core(q1, k1, v1, q1, past_key_values=cache, use_cache=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(qn, kn, vn)
    barrier()
    c0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step(qn, kn, vn)
        e1.record()
        barrier()
    launches = _lib.launch_count() - c0
    ms = e0.elapsed_time(e1)
    # end to end: the new token's q, k, v come from pinned host memory, the output row goes back
    dq_, dk_, dv_ = (torch.empty_like(t) for t in (qn, kn, vn))

    def e2e_step():
        for d_, h_ in zip((dq_, dk_, dv_), host):
            d_.copy_(h_, non_blocking=True)
        out_host.copy_(step(dq_, dk_, dv_), non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    us_step = 1e3 * ms / args.steps
    pk = peaks()
    # bytes a step must touch: pooled keys + bias, the K selected K/V chunks, the sliding window
    alg = B * hk * (N * D * 2 + N * 4 * (hq // hk) + K * S * D * 2 * 2 + (W + S) * D * 2 * 2)
    achieved = alg / (us_step * 1e-6) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": "hils_decode_us_per_step", "value": us_step, "unit": "us/step", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": us_step / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, **w, "sequences_per_gpu": B,
                       "parallelism": f"batch-sharded x{world}, no collective", "l2": "kv_store_larger_than_L2"},
            "e2e": {"value": 1e3 * ms_e2e, "unit": "us/step",
                    "h2d_bytes_per_step": sum(h.numel() * 2 for h in host), "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": launches, "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "traffic": None, "kernel": "decode step (all kernels)",
                         "algorithmic_bytes_per_step": alg, "peak_source": pk["source"]},
            "cpu_baseline": None,
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return run_reference(args)
    if args.workload.startswith("c4"):
        return run_decode(args)

    import torch.distributed as dist
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOADS[args.workload]
    B, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    dtype = torch.bfloat16
    host = make_inputs(w, 2 + rank, "cuda", dtype)
    q, k, v, do = (t.to(dev, non_blocking=True) for t in host)
    torch.cuda.synchronize()
    core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).train()

    def step(qi, ki, vi, doi):
        qi, ki, vi = (t.detach().requires_grad_(True) for t in (qi, ki, vi))
        o = core(qi, ki, vi, qi)
        o.backward(doi)
        return o, qi.grad, ki.grad, vi.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step(q, k, v, do)
    barrier()
    c0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step(q, k, v, do)
        e1.record()
        barrier()
    launches = _lib.launch_count() - c0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    value = world * B * T / (ms_step / 1e3)

    # ---- end to end through the public API with pinned host buffers ----------------------------
    # every step copies q, k, v, dO in and o, dq, dk, dv out; the package's HostPipeline runs the copies
    # of neighbouring steps on their own streams so that they overlap this step's kernels
    from hils_attention_b200.host_pipeline import HostPipeline
    out_host = [torch.empty_like(h).pin_memory() for h in (host[0], host[0], host[1], host[2])]
    pipe = HostPipeline(step, host, dev, depth=2)
    for _ in range(2):
        pipe.submit(host, out_host)
    pipe.drain()
    barrier()
    n_e2e = max(4, min(args.steps, 8))
    e0.record()
    for _ in range(n_e2e):
        pipe.submit(host, out_host)
    pipe.join_stream()
    e1.record()
    pipe.drain()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    e2e_val = world * B * T / (ms_e2e / n_e2e / 1e3)
    h2d = sum(h.numel() * h.element_size() for h in host)
    d2h = sum(h.numel() * h.element_size() for h in out_host)

    # ---- dominant kernel, timed alone: sparse chunk attention forward and backward ---------------
    pk = peaks()
    with torch.no_grad():
        _, aux = core(q, k, v, q, return_aux=True)
    idx, wts = aux["indices"], aux["weights"].contiguous()
    valid_slots = int((idx >= 0).sum().item()) * (hq // hk)
    f_fwd = 4.0 * valid_slots * S * D
    f_bwd = 10.0 * valid_slots * S * D

    def time_op(fn, n=5):
        fn(); torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record(); torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    qg, kg, vg, wg = (t.detach().requires_grad_(True) for t in (q, k, v, wts))
    t_fwd = time_op(lambda: hb.HiLS_block_M_head(q, k, v, wts, idx, block_size=S, is_training=False))
    o_t = hb.HiLS_block_M_head(qg, kg, vg, wg, idx, block_size=S)
    t_bwd = time_op(lambda: torch.autograd.grad(o_t, (qg, kg, vg, wg), do, retain_graph=True), n=3)
    dom = "sparse_attn_bwd" if t_bwd > t_fwd else "sparse_attn_fwd"
    f_dom, t_dom = (f_bwd, t_bwd) if t_bwd > t_fwd else (f_fwd, t_fwd)
    achieved = f_dom / (t_dom / 1e3) / 1e12
    # DRAM bytes per launch of the dominant kernel, from an ncu capture of this workload whose summary is kept
    # under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum; the backward is the dq pass plus the dkv
    # pass); captured at c2 only
    traffic = {"sparse_attn_bwd": (724 + 301 + 622 + 246) * 1e6, "sparse_attn_fwd": (586 + 123) * 1e6}[dom] \
        if args.workload == "c2" else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
                "frac": achieved / pk["tflops"], "traffic": traffic, "kernel": dom,
                "kernel_ms": t_dom, "peak_source": pk["source"],
                "sparse_attn_fwd_ms": t_fwd, "sparse_attn_bwd_ms": t_bwd,
                "algorithmic_flops_fwd": f_fwd, "algorithmic_flops_bwd": f_bwd}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            tps, cores, dt = cpu_chain_tokens_per_s(1)
            cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                   "sample": "oracle fp32 chain fwd+bwd, B=1 T=2048 H=16 D=64 S=64 K=8 W=512, one pass "
                             f"({dt:.1f} s)"}
        print(json.dumps({
            "metric": "hils_attn_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, **w, "global_batch": B * world,
                       "parallelism": f"batch-sharded x{world}, no collective", "l2": "inputs_larger_than_L2"},
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches, "clocks": clk.summary(), "roofline": roofline, "cpu_baseline": cpu,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
