#!/usr/bin/env python
"""Benchmark of the HiLS attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3] [--only]

Headline workload (config.workload = "c3", the metric's 64K context): B=1, T=65536, 32 heads (MHA),
head_dim 128, chunk 64 (1024 chunks), top-k 32, window 512, causal, bf16, forward + backward of one
attention layer's op chain: sliding-window branch -> chunk pooling (k', b') -> chunk selection ->
inter-chunk softmax -> sparse chunk attention -> combine, and the backward of all of it.
q, v ~ N(0,1), k ~ N(0,1) + a per-(chunk, head) offset ~ N(0, 0.5), dO ~ N(0,1), landmark query = q; seeded.

With N > 1 the heads are split over the ranks (32/N heads each; every stage of the path is independent
per kv head, so there is no data-path collective): strong scaling, value = T / slowest rank's step time.

Prints ONE JSON line.  `value` is timed with inputs resident in HBM; `e2e` times the same step through the
public API with pinned HOST buffers (q, k, v, dO copied in; o, dq, dk, dv copied out every step, copies of
neighbouring steps overlapped with compute).  `roofline` is for sparse chunk attention forward + backward,
each timed alone with CUDA events, and carries a per-kernel list for the other stages.  `secondary` holds
the same measurements for workload c2 (B=8, T=8192, 16 heads, D=64: the 345M model's attention shape) and
c4 (decode: 32 sequences x one new token against a 131072-token KV store, batch split over the ranks),
c4_paged / c4_paged_ragged (the same decode through the paged store, pages scattered over the pool; sequence
lengths from 64K to 128K tokens in one batch), c5 (forward at 1,048,576 tokens, sequence-sharded for N > 1), and
the sparse op alone on index sets with the reference's own overlap generator.
`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the host cores
at its CPU-runnable configuration c1 (B=1, T=2048, 16 heads, D=64, top-k 8, fp32).
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
    "c1": dict(B=1, T=2048, h_q=16, h_kv=16, D=64, S=64, K=8, W=512, dtype="f32"),
    "c2": dict(B=8, T=8192, h_q=16, h_kv=16, D=64, S=64, K=32, W=512),
    "c2_small": dict(B=1, T=8192, h_q=16, h_kv=16, D=64, S=64, K=32, W=512),
    # same tokens with the head grouping of the reference's 345M model (2 kv heads, groups of 8 query heads)
    "c2_gqa": dict(B=8, T=8192, h_q=16, h_kv=2, D=64, S=64, K=32, W=512),
    "c3": dict(B=1, T=65536, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    "c3_small": dict(B=1, T=16384, h_q=8, h_kv=8, D=128, S=64, K=32, W=512),
    # the 64K-token shape with 4 of its 32 heads: every kernel takes the path it takes at c3, a few hundred MB on the device
    "c3_4h": dict(B=1, T=65536, h_q=4, h_kv=4, D=128, S=64, K=32, W=512),
    # decode: 32 sequences, one new token each, against a 131072-token KV store
    "c4": dict(B=32, T=131072, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    "c4_small": dict(B=4, T=16384, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    # the same decode through the paged store (page = chunk, pages of the sequences interleaved in the pool);
    # "ragged": sequence lengths spread evenly from T/2 to T in one batch
    "c4_paged": dict(B=32, T=131072, h_q=32, h_kv=32, D=128, S=64, K=32, W=512, ragged=False),
    "c4_paged_ragged": dict(B=32, T=131072, h_q=32, h_kv=32, D=128, S=64, K=32, W=512, ragged=True),
    "c4_paged_small": dict(B=4, T=16384, h_q=32, h_kv=32, D=128, S=64, K=32, W=512, ragged=True),
    # ultra-long context, forward only, the sequence sharded over the ranks
    "c5": dict(B=1, T=1048576, h_q=32, h_kv=32, D=128, S=64, K=32, W=512),
    "c5_small": dict(B=1, T=131072, h_q=4, h_kv=4, D=128, S=64, K=32, W=512),
}
CPU_SAMPLE = WORKLOADS["c1"]   # the reference's CPU-runnable case


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def dram_traffic(workload, kernel):
    """DRAM bytes per launch of `kernel` at `workload` as captured by ncu, from the table that is regenerated
    together with the ncu summaries; None when there is no entry."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        return json.load(open(p)).get(workload, {}).get(kernel)
    except Exception:
        return None


def make_inputs(w, seed, dtype, heads=None, pin=True):
    """Seeded host tensors q, k, v, dO of workload `w`; `heads` = (first kv head, count) keeps a head slice."""
    g = torch.Generator().manual_seed(seed)
    B, T, hq, hk, D, S = w["B"], w["T"], w["h_q"], w["h_kv"], w["D"], w["S"]
    q = torch.randn(B, T, hq, D, generator=g)
    k = torch.randn(B, T, hk, D, generator=g)
    off = torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5
    k[:, :(T // S) * S] += off.expand(-1, -1, S, -1, -1).reshape(B, (T // S) * S, hk, D)
    v = torch.randn(B, T, hk, D, generator=g)
    do = torch.randn(B, T, hq, D, generator=g)
    if w.get("dtype") == "f32":   # the CPU-runnable configuration scales q, k, v by 1/sqrt(D)
        q, k, v = (t / math.sqrt(D) for t in (q, k, v))
    if heads is not None:
        G = hq // hk
        h0, n = heads
        q, do = (t[:, :, h0 * G:(h0 + n) * G] for t in (q, do))
        k, v = (t[:, :, h0:h0 + n] for t in (k, v))
    out = [t.to(dtype).contiguous() for t in (q, k, v, do)]
    return [t.pin_memory() for t in out] if pin else out


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU every 50 ms.  The sampler is started BEFORE the warm-up
    steps (nvidia-smi needs a few hundred ms to deliver its first line) and the summary keeps the samples that arrived
    between `start()` and `stop()`, i.e. inside the timed region; if the region was shorter than a sampling period the
    nearest samples (within 0.5 s, the GPU still busy with the neighbouring steps) are used and the summary says so."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thr = threading.Thread(target=self._read, daemon=True)
            self.thr.start()
        except Exception:
            self.proc = None
        self.t0 = time.monotonic()          # until start() is called the whole `with` body counts
        return self

    def start(self):
        self.t0 = time.monotonic()

    def stop(self):
        self.t1 = time.monotonic()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [x.strip() for x in line.split(",")]))

    def __exit__(self, *a):
        if self.t1 is None:
            self.t1 = time.monotonic()
        if self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [r for t, r in self.rows if self.t0 <= t <= self.t1]
        window = "timed_region"
        if not inside:
            inside = [r for t, r in self.rows if self.t0 - 0.5 <= t <= self.t1 + 0.5]
            window = "nearest_within_0.5s"
        sm, mx, reasons = [], [], set()
        for r in inside:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
                for n, val in zip(names, r[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


# -------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's fp32 chain on the host cores
# -------------------------------------------------------------------------------------------------
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


CPU_SAMPLE_TEXT = ("CPU restatement of the reference's PyTorch chain, fp32, fwd+bwd, at workload c1: B=1 T=2048 H=16 "
                   "D=64 S=64 K=8 W=512 (the reference's CPU-runnable configuration)")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    for i in range(args.warmup + args.steps):
        _, cores, dt = cpu_chain_tokens_per_s(1)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = CPU_SAMPLE["B"] * CPU_SAMPLE["T"] / (ms / 1e3)
    w = {k: v for k, v in CPU_SAMPLE.items() if k != "dtype"}
    print(json.dumps({
        "impl": "reference", "metric": "hils_attn_fwd_bwd_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # what this arm really times: the CPU-runnable configuration, not the GPU arm's 64K-context shape
        "config": {"workload": "c1", **w, "same_config_as_gpu_arm": False,
                   "note": "the GPU arm's line carries secondary.c1 = the same configuration on the GPU"},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                         "sample": CPU_SAMPLE_TEXT},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# -------------------------------------------------------------------------------------------------
# helpers
# -------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max(self, *vals):
        if self.world == 1:
            return [float(v) for v in vals]
        import torch.distributed as dist
        t = torch.tensor(list(vals), dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def require_clean_status(where):
    """A tensor-core kernel whose bounded wait expired returns early with partial output: such a run must
    not produce a record."""
    from hils_attention_b200 import _lib
    st = int(_lib.load().hils_take_device_status())
    if st != 0:
        raise RuntimeError(f"device status {st} after {where}: a bounded wait expired, the timing is void")


def time_op(fn, n=3):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def overlap_indices(B, L, H, K, S, N, overlap_ratio, block_M, device, seed):
    """Chunk ids with the neighbour overlap of the reference's own stand-in for trained selections
    (ops/hils_fwd_bwd_head.py:96-187, `build_block_indices_block_M`): the first token of every run of
    `block_M` tokens draws K random causal chunks; each following token keeps a random `overlap_ratio` of its
    predecessor's chunks and redraws the rest.  Vectorised over (batch, head, run); ascending ids, -1 padded."""
    g = torch.Generator(device=device).manual_seed(seed)
    nrun = (L + block_M - 1) // block_M
    out = torch.full((B, nrun * block_M, H, K), -1, dtype=torch.int32, device=device)
    t0 = torch.arange(nrun, device=device) * block_M
    cand = torch.arange(N, device=device)
    prev = None
    for j in range(block_M):
        t = t0 + j                                                   # (nrun,)
        nmax = torch.clamp(t // S + 1, max=N)                        # causal candidates of each run's token
        allowed = (cand[None, :] < nmax[:, None])[None, :, None, :]  # (1, nrun, 1, N)
        nsel = torch.clamp(nmax, max=K)[None, :, None]               # (1, nrun, 1)
        r = torch.rand((B, nrun, H, N), generator=g, device=device)
        if prev is None:
            score = torch.where(allowed, r, torch.full_like(r, -1.0))
        else:
            n_keep = (overlap_ratio * nsel.float()).long()
            keep_rank = torch.where(prev, r, torch.full_like(r, -1.0)).argsort(-1, descending=True).argsort(-1)
            kept = prev & (keep_rank < n_keep[..., None])
            r2 = torch.rand((B, nrun, H, N), generator=g, device=device)
            score = torch.where(kept, r2 + 2.0, torch.where(allowed & ~kept, r2, torch.full_like(r2, -1.0)))
        order = score.argsort(-1, descending=True)
        rank = order.argsort(-1)
        sel = (rank < nsel[..., None]) & (score >= 0)
        ids = torch.where(sel, cand.expand_as(sel), torch.full_like(rank, N + 1)).sort(-1).values[..., :K]
        ids = torch.where(ids > N, torch.full_like(ids, -1), ids).to(torch.int32)
        out[:, j::block_M][:, :nrun, :, :ids.shape[-1]] = ids
        prev = sel
    return out[:, :L].contiguous()


def swa_keys_total(T, S, W):
    """Sum over query positions of the keys the sliding-window branch sees (chunk-snapped left edge, the
    landmark key of every chunk dropped)."""
    t = torch.arange(T, dtype=torch.int64)
    start = torch.clamp(((t - W + 1) // S) * S, min=0)
    n = t - start + 1
    lmk = (t + 1) // S - start // S      # landmark columns inside [start, t]
    return int((n - lmk).sum())


# -------------------------------------------------------------------------------------------------
# training / prefill workloads: forward + backward of the chain
# -------------------------------------------------------------------------------------------------
def run_train(args, name, ds, steps, warmup, with_e2e=True, with_kernels=True, with_overlap=True):
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.host_pipeline import HostPipeline

    w = WORKLOADS[name]
    B, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    dtype = torch.float32 if w.get("dtype") == "f32" else torch.bfloat16
    G = hq // hk
    world, rank, dev = ds.world, ds.rank, ds.dev
    if hk % world != 0:
        raise SystemExit(f"workload {name}: {hk} kv heads do not split over {world} ranks")
    hk_r = hk // world
    hq_r = hk_r * G
    host = make_inputs(w, 2 if name.startswith("c2") else 3, dtype, heads=(rank * hk_r, hk_r) if world > 1 else None)
    q, k, v, do = (t.to(dev, non_blocking=True) for t in host)
    torch.cuda.synchronize()
    core = HiLSAttentionCore(HiLSAttentionConfig(hq_r, hk_r, K, S, W)).train()

    def step(qi, ki, vi, doi):
        qi, ki, vi = (t.detach().requires_grad_(True) for t in (qi, ki, vi))
        o = core(qi, ki, vi, qi)
        o.backward(doi)
        return o, qi.grad, ki.grad, vi.grad

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(ds.local) as clk:
        for _ in range(warmup):
            step(q, k, v, do)
        ds.barrier()
        c0 = _lib.launch_count()
        clk.start()
        e0.record()
        for _ in range(steps):
            step(q, k, v, do)
        e1.record()
        ds.barrier()
        clk.stop()
    launches = _lib.launch_count() - c0
    require_clean_status(f"the timed steps of {name}")
    (ms,) = ds.max(e0.elapsed_time(e1))
    ms_step = ms / steps
    out = {
        "metric": "hils_attn_fwd_bwd_tokens_per_s", "value": B * T / (ms_step / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "bf16",
        "data": "synthetic",
        "config": {"workload": name, **{x: w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W")},
                   "heads_per_gpu": hq_r, "parallelism": f"head-sharded x{world}, no collective",
                   "l2": "inputs_larger_than_L2" if sum(t.numel() * t.element_size() for t in host) > 126e6
                   else "inputs_smaller_than_L2_outputs_rewritten"},
        "gpu_launches": launches, "clocks": clk.summary(),
    }

    if with_e2e:
        # every step copies q, k, v, dO in and o, dq, dk, dv out; the copies of neighbouring steps run on their
        # own streams so that they overlap this step's kernels
        out_host = [torch.empty_like(h).pin_memory() for h in (host[0], host[0], host[1], host[2])]
        pipe = HostPipeline(step, host, dev, depth=2)
        for _ in range(2):
            pipe.submit(host, out_host)
        pipe.drain()
        ds.barrier()
        n_e2e = max(4, min(steps, 8))
        e0.record()
        for _ in range(n_e2e):
            pipe.submit(host, out_host)
        pipe.join_stream()
        e1.record()
        pipe.drain()
        ds.barrier()
        require_clean_status(f"the end-to-end steps of {name}")
        (ms_e2e,) = ds.max(e0.elapsed_time(e1))
        h2d = sum(h.numel() * h.element_size() for h in host)
        d2h = sum(h.numel() * h.element_size() for h in out_host)
        sec = ms_e2e / n_e2e / 1e3
        out["e2e"] = {"value": B * T / sec, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "ms_per_step": 1e3 * sec,
                      # a step cannot be faster than its copies: these rates show when the host link is the limit
                      "h2d_gbs_if_copy_bound": h2d / sec / 1e9, "d2h_gbs_if_copy_bound": d2h / sec / 1e9}
        del pipe, out_host

    if with_kernels and dtype == torch.bfloat16:
        out["roofline"] = kernel_rooflines(name, core, q, k, v, do, w, hq_r, hk_r, with_overlap)
    del q, k, v, do, host
    torch.cuda.empty_cache()
    return out


def kernel_rooflines(name, core, q, k, v, do, w, hq, hk, with_overlap):
    """Every stage of the chain timed alone (CUDA events on the launch stream) against the roofline that bounds it.
    The headline entry is sparse chunk attention forward + backward together."""
    import hils_attention_b200 as hb
    B, T, D, S, K, W = (w[x] for x in ("B", "T", "D", "S", "K", "W"))
    G = hq // hk
    pk = peaks()
    N = T // S
    with torch.no_grad():
        _, aux = core(q, k, v, q, return_aux=True)
    idx, wts, lse = aux["indices"], aux["weights"].contiguous(), aux["lse_swa"]
    lmk_k, prior_b, scores = aux["lmk_k"], aux["prior_b"], aux["scores"]
    valid_slots = int((idx >= 0).sum().item()) * G
    kernels = []

    def add(kname, ms, flops=None, nbytes=None):
        e = {"kernel": kname, "ms": ms}
        if flops is not None:
            e.update(bound="tensor", achieved=flops / (ms / 1e3) / 1e12, unit="TFLOP/s", algorithmic_flops=flops)
            e["frac"] = e["achieved"] / pk["tflops"]
        else:
            e.update(bound="hbm", achieved=nbytes / (ms / 1e3) / 1e9, unit="GB/s", algorithmic_bytes=nbytes)
            e["frac"] = e["achieved"] / pk["hbm_gbs"]
        kernels.append(e)
        return e

    def fwd_bwd(make, grads_of, gouts, n=3):
        """(forward ms, backward ms) of a differentiable op."""
        t_f = time_op(lambda: make(False), n)
        outs = make(True)
        outs = outs if isinstance(outs, tuple) else (outs,)
        t_b = time_op(lambda: torch.autograd.grad(outs, grads_of, gouts, retain_graph=True), n)
        return t_f, t_b

    es = q.element_size()
    # ---- sparse chunk attention --------------------------------------------------------------------
    qg, kg, vg, wg = (t.detach().requires_grad_(True) for t in (q, k, v, wts))
    t_f, t_b = fwd_bwd(lambda tr: hb.HiLS_block_M_head(qg if tr else q, kg if tr else k, vg if tr else v,
                                                       wg if tr else wts, idx, block_size=S, is_training=tr),
                       (qg, kg, vg, wg), (do,))
    f_f, f_b = 4.0 * valid_slots * S * D, 10.0 * valid_slots * S * D
    add("sparse_attn_fwd", t_f, flops=f_f)
    add("sparse_attn_bwd", t_b, flops=f_b)
    # ---- sliding-window branch ---------------------------------------------------------------------
    nk = swa_keys_total(T, S, W) * B * hq
    t_f2, t_b2 = fwd_bwd(lambda tr: hb.flex_attn_tl(qg if tr else q, kg if tr else k, vg if tr else v, W, S,
                                                    training=True),
                         (qg, kg, vg), (do, torch.zeros_like(lse, dtype=torch.float32)))
    add("swa_fwd", t_f2, flops=4.0 * nk * D)
    add("swa_bwd", t_b2, flops=10.0 * nk * D)
    # ---- chunk selection ---------------------------------------------------------------------------
    t = torch.arange(T)
    nvalid = torch.clamp((t - W + 1) // S, min=0, max=N)
    f_sel = 2.0 * float(nvalid.sum()) * D * hq * B
    lg, kg2 = q.detach().requires_grad_(True), lmk_k.detach().requires_grad_(True)
    t_f3, t_b3 = fwd_bwd(lambda tr: hb.online_softmax_topk_head(lg if tr else q, kg2 if tr else lmk_k, lse, K, S, W,
                                                                G=lmk_k.shape[2] // hk, bias=prior_b)[1],
                         (lg, kg2), (torch.randn_like(scores),))
    add("selection_fwd", t_f3, flops=f_sel)
    add("selection_bwd", t_b3, flops=4.0 * valid_slots * D)
    # ---- pooling, inter-chunk softmax ----------------------------------------------------------------
    kc = k[:, :N * S].unflatten(1, (N, S))
    mu = q[:, S - 1::S][:, :N]
    mg, kcg = mu.detach().requires_grad_(True), kc.detach().requires_grad_(True)
    t_f4, t_b4 = fwd_bwd(lambda tr: hb.chunk_attn_pool(mg if tr else mu, kcg if tr else kc),
                         (mg, kcg), (torch.randn_like(lmk_k), torch.randn_like(prior_b)))
    pool_bytes = float(B * N * S * hk * D * es)
    add("pool_fwd", t_f4, nbytes=pool_bytes)
    add("pool_bwd", t_b4, nbytes=2 * pool_bytes)
    sg = scores.detach().requires_grad_(True)
    t_f5, t_b5 = fwd_bwd(lambda tr: hb.inter_chunk_softmax(sg if tr else scores, idx, lse, prior_b),
                         (sg,), (torch.randn_like(wts),))
    row_bytes = float(B * T * hq) * (K * es + K * 4 / G + (K + 1) * es)
    add("chunk_weights_fwd", t_f5, nbytes=row_bytes)
    add("chunk_weights_bwd", t_b5, nbytes=row_bytes + float(B * T * hq) * (K + 1) * es)
    # ---- exact per-chunk log Z (the NaiveBSA scoring op; not a stage of the HiLS step) ---------------
    if S == 64:
        f_lz = 2.0 * float(nvalid.sum()) * S * D * hq * B
        t_lz = time_op(lambda: hb.exact_chunk_log_z_tl(q, k, chunk_size=S, window_size=W))
        e = add("exact_chunk_log_z_fwd", t_lz, flops=f_lz)
        e["output_gbs"] = float(B * T * hq) * N * 4 / (t_lz / 1e3) / 1e9
        # backward: S recomputed in both passes, dQ = dS K, dK = dS^T Q (the upstream gradient is zero where log Z is -inf)
        qz, kz = q.detach().requires_grad_(True), k.detach().requires_grad_(True)
        lz = hb.exact_chunk_log_z_tl(qz, kz, chunk_size=S, window_size=W)
        gz = torch.randn_like(lz).masked_fill_(~torch.isfinite(lz), 0.0)
        t_lzb = time_op(lambda: torch.autograd.grad(lz, (qz, kz), gz, retain_graph=True))
        add("exact_chunk_log_z_bwd", t_lzb, flops=2.0 * f_lz)
        del lz, gz, qz, kz
    require_clean_status(f"the per-kernel timings of {name}")

    t_sp, f_sp = t_f + t_b, f_f + f_b
    achieved = f_sp / (t_sp / 1e3) / 1e12
    roof = {"bound": "tensor", "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s",
            "frac": achieved / pk["tflops"], "traffic": dram_traffic(name, "sparse_attn_fwd+bwd"),
            "kernel": "sparse_attn_fwd+bwd", "kernel_ms": t_sp, "peak_source": pk["source"],
            "algorithmic_flops": f_sp, "valid_slots": valid_slots, "kernels": kernels,
            "hbm_peak": pk["hbm_gbs"]}
    if with_overlap:
        # the sparse op alone on the reference's stand-in for a trained model's overlapping selections
        idx_o = overlap_indices(B, T, hk, K, S, N, 0.8, 32, q.device, 11)
        vs = int((idx_o >= 0).sum().item()) * G
        t_fo, t_bo = fwd_bwd(lambda tr: hb.HiLS_block_M_head(qg if tr else q, kg if tr else k, vg if tr else v,
                                                             wg if tr else wts, idx_o, block_size=S, is_training=tr),
                             (qg, kg, vg, wg), (do,))
        fo = 14.0 * vs * S * D
        roof["overlap_0.8_indices"] = {"sparse_attn_fwd_ms": t_fo, "sparse_attn_bwd_ms": t_bo, "valid_slots": vs,
                                       "achieved": fo / ((t_fo + t_bo) / 1e3) / 1e12,
                                       "frac": fo / ((t_fo + t_bo) / 1e3) / 1e12 / pk["tflops"],
                                       "generator": "overlap_ratio=0.8, runs of 32 tokens, causal candidates"}
        require_clean_status(f"the overlap-index timings of {name}")
    return roof


# -------------------------------------------------------------------------------------------------
# decode workload
# -------------------------------------------------------------------------------------------------
def run_decode(args, name, ds, steps, warmup):
    """Decode against a cached HiLS KV store: one new token per sequence and step through the whole
    chain (store append, sliding-window branch, selection over the pooled chunk keys, inter-chunk
    softmax, sparse chunk attention, combine).  The batch is sharded over the ranks (no collective)."""
    from hils_attention_b200 import _lib
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.cache import HiLSCache
    import hils_attention_b200 as hb

    world, rank, dev = ds.world, ds.rank, ds.dev
    w = WORKLOADS[name]
    Bt, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    B = max(1, Bt // world)
    dtype = torch.bfloat16
    n_e2e = 16
    n_steps = warmup + steps + n_e2e + 3
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

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(ds.local) as clk:
        for _ in range(warmup):
            step(qn, kn, vn)
        ds.barrier()
        c0 = _lib.launch_count()
        clk.start()
        e0.record()
        for _ in range(steps):
            step(qn, kn, vn)
        e1.record()
        ds.barrier()
        clk.stop()
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
    ds.barrier()
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    ds.barrier()
    require_clean_status(f"the decode steps of {name}")
    ms, ms_e2e = ds.max(ms, e0.elapsed_time(e1) / n_e2e)
    us_step = 1e3 * ms / steps
    pk = peaks()
    # bytes a step must touch: pooled keys + bias, the K selected K/V chunks, the sliding window
    alg = B * hk * (N * D * 2 + N * 4 * (hq // hk) + K * S * D * 2 * 2 + (W + S) * D * 2 * 2)
    achieved = alg / (us_step * 1e-6) / 1e9
    out = {
        "metric": "hils_decode_us_per_step", "value": us_step, "unit": "us/step", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": us_step / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, **w, "sequences_per_gpu": B,
                   "parallelism": f"batch-sharded x{world}, no collective", "l2": "kv_store_larger_than_L2"},
        "e2e": {"value": 1e3 * ms_e2e, "unit": "us/step",
                "h2d_bytes_per_step": sum(h.numel() * 2 for h in host), "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": launches, "clocks": clk.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": dram_traffic(name, "decode_step"),
                     "kernel": "decode step (all kernels)", "algorithmic_bytes_per_step": alg,
                     "peak_source": pk["source"]},
    }
    del kbuf, vbuf, cache, layer, core, lmk_k, prior_b
    torch.cuda.empty_cache()
    return out

def run_decode_paged(args, name, ds, steps, warmup):
    """The decode step of run_decode through the paged store: K/V in a pool of 64-token pages, the pages of the
    sequences interleaved at random in the pool, page tables and lengths read on the device; optionally with
    sequences of different lengths in the batch.  Sharded over the ranks by sequence (no collective)."""
    from hils_attention_b200 import _lib
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.kv_store import PagedKVStore
    import hils_attention_b200 as hb

    world, rank, dev = ds.world, ds.rank, ds.dev
    w = WORKLOADS[name]
    Bt, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    B = max(1, Bt // world)
    dtype = torch.bfloat16
    n_e2e = 16
    lens0 = [T - (T // 2) * b // max(1, B - 1) if w["ragged"] else T for b in range(B)]
    lens0 = [t - t % S + 7 for t in lens0]       # with the default step counts nobody completes a chunk while timed
    max_pages = T // S + 2
    store = PagedKVStore(B * max_pages + 1, B, max_pages, hk, D, hq, dtype=dtype, device=dev)
    store.pool.shuffle(11 + rank)                                   # a sequence's pages lie scattered over the pool
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    P = store.k_pages.shape[1]
    for p0 in range(0, P, 1024):                                    # fill in slices: no second copy of the pool
        n = min(1024, P - p0)
        off = torch.randn((n, hk, 1, D), generator=g, device=dev) * 0.5
        store.k_pages[0, p0:p0 + n] = (torch.randn((n, hk, S, D), generator=g, device=dev) + off).to(dtype)
        store.v_pages[0, p0:p0 + n] = torch.randn((n, hk, S, D), generator=g, device=dev).to(dtype)
    with torch.no_grad():
        for b in range(B):
            slot = store.allocate(lens0[b])
            N = lens0[b] // S                                        # pooled chunk keys of the cached prefix
            ids = torch.tensor(store.pages_of(slot)[:N], dtype=torch.long, device=dev)
            mu = torch.randn((1, N, hq, D), generator=g, device=dev).to(dtype)
            lk, pb = hb.chunk_attn_pool(mu, store.k_pages[0].index_select(0, ids).transpose(1, 2).unsqueeze(0).contiguous())
            store.lmk_k[0, slot, :N].copy_(lk[0])
            store.prior_b[0, slot, :N].copy_(pb[0])
            del ids, mu, lk, pb
    core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).eval()
    host = [torch.randn((B, 1, h, D), generator=torch.Generator().manual_seed(9 + i)).to(dtype).pin_memory()
            for i, h in enumerate((hq, hk, hk))]
    qn, kn, vn = (t.to(dev) for t in host)
    out_host = torch.empty((B, 1, hq, D), dtype=dtype).pin_memory()

    def step(q1, k1, v1):
        with torch.no_grad():
            store.begin_step()
            o = core.decode_paged(q1, k1, v1, q1, store)
            store.end_step()
            return o

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(ds.local) as clk:
        for _ in range(warmup):
            step(qn, kn, vn)
        ds.barrier()
        c0 = _lib.launch_count()
        clk.start()
        e0.record()
        for _ in range(steps):
            step(qn, kn, vn)
        e1.record()
        ds.barrier()
        clk.stop()
    launches = _lib.launch_count() - c0
    ms = e0.elapsed_time(e1)
    dq_, dk_, dv_ = (torch.empty_like(t) for t in (qn, kn, vn))

    def e2e_step():
        for d_, h_ in zip((dq_, dk_, dv_), host):
            d_.copy_(h_, non_blocking=True)
        out_host.copy_(step(dq_, dk_, dv_), non_blocking=True)

    for _ in range(3):
        e2e_step()
    ds.barrier()
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    ds.barrier()
    require_clean_status(f"the decode steps of {name}")
    ms, ms_e2e = ds.max(ms, e0.elapsed_time(e1) / n_e2e)
    us_step = 1e3 * ms / steps
    pk = peaks()
    # bytes a step must touch: pooled keys + bias of each sequence's chunks, the K selected pages, the sliding window
    alg = sum(hk * ((t // S) * D * 2 + (t // S) * 4 * (hq // hk) + K * S * D * 2 * 2 + (W + S) * D * 2 * 2) for t in lens0)
    achieved = alg / (us_step * 1e-6) / 1e9
    out = {
        "metric": "hils_decode_us_per_step", "value": us_step, "unit": "us/step", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": us_step / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, **w, "sequences_per_gpu": B, "lengths": [min(lens0), max(lens0)],
                   "store": f"paged, {P} pages of {S} tokens, {store.bytes_held() / 2**30:.1f} GiB",
                   "parallelism": f"batch-sharded x{world}, no collective", "l2": "kv_store_larger_than_L2"},
        "e2e": {"value": 1e3 * ms_e2e, "unit": "us/step",
                "h2d_bytes_per_step": sum(h.numel() * 2 for h in host), "d2h_bytes_per_step": out_host.numel() * 2},
        "gpu_launches": launches, "clocks": clk.summary(),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": None,
                     "kernel": "paged decode step (all kernels)", "algorithmic_bytes_per_step": alg,
                     "peak_source": pk["source"]},
    }
    del store, core
    torch.cuda.empty_cache()
    return out


# -------------------------------------------------------------------------------------------------
# ultra-long context: forward of the chain with the sequence sharded over the ranks
# -------------------------------------------------------------------------------------------------
def run_context_parallel(args, name, ds, steps, warmup):
    """Forward of the chain over one sequence of T tokens: on one GPU the plain chain, on N >= 2 GPUs the
    context-parallel chain (zig-zag blocks; the pooled chunk keys all-gathered, the selected K/V tiles fetched per
    kv head).  Strong scaling: T is fixed, value = T / slowest rank's step.  Inputs are generated on the device
    block by block from per-block seeds, so the sequence is the same at every N."""
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.parallel import SeqPartition, context_parallel_forward
    from hils_attention_b200 import _lib

    w = WORKLOADS[name]
    B, T, hq, hk, D, S, K, W = (w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W"))
    world, rank, dev = ds.world, ds.rank, ds.dev
    part = SeqPartition(world, "zigzag")
    nblk = 16                                   # generation blocks: a multiple of 2 * world for world <= 8
    tb = T // nblk

    def gen_block(j):
        g = torch.Generator(device=dev).manual_seed(5000 + j)
        qb = torch.randn((B, tb, hq, D), generator=g, device=dev, dtype=torch.bfloat16)
        kb = torch.randn((B, tb, hk, D), generator=g, device=dev, dtype=torch.bfloat16)
        off = torch.randn((B, tb // S, 1, hk, D), generator=g, device=dev, dtype=torch.bfloat16) * 0.5
        kb = (kb.unflatten(1, (tb // S, S)) + off).flatten(1, 2)
        vb = torch.randn((B, tb, hk, D), generator=g, device=dev, dtype=torch.bfloat16)
        return qb, kb, vb

    per = nblk // part.n_blocks if world > 1 else nblk
    mine = [b * per + i for b in (part.blocks(rank) if world > 1 else [0]) for i in range(per)]
    parts = [gen_block(j) for j in mine]
    q, k, v = (torch.cat([p[i] for p in parts], 1) for i in range(3))
    del parts
    core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).eval()

    def step(timings=None, aux=False):
        with torch.no_grad():
            if world == 1:
                return core(q, k, v, q)
            return context_parallel_forward(q, k, v, q, h_kv=hk, topk=K, chunk_size=S, window_size=W,
                                            partition="zigzag", return_aux=aux, timings=timings)

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(ds.local) as clk:
        for _ in range(warmup):
            step()
        ds.barrier()
        c0 = _lib.launch_count()
        clk.start()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        ds.barrier()
        clk.stop()
    launches = _lib.launch_count() - c0
    require_clean_status(f"the timed steps of {name}")
    (ms,) = ds.max(e0.elapsed_time(e1))
    ms_step = ms / steps
    out = {"metric": "hils_attn_fwd_tokens_per_s", "value": B * T / (ms_step / 1e3), "unit": "tokens/s",
           "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
           "scaling": "strong", "dtype": "bf16", "data": "synthetic",
           "config": {"workload": name, **{x: w[x] for x in ("B", "T", "h_q", "h_kv", "D", "S", "K", "W")},
                      "tokens_per_gpu": T // world,
                      "parallelism": "single GPU" if world == 1 else f"context-parallel x{world}, zig-zag blocks",
                      "l2": "inputs_larger_than_L2"},
           "gpu_launches": launches, "clocks": clk.summary()}
    if world > 1:
        tm = {}
        _, aux = step(timings=tm, aux=True)
        stage_max = ds.max(*[tm[x] for x in sorted(tm)])
        out["stages_ms_max_over_ranks"] = dict(zip(sorted(tm), stage_max))
        fetch_b, ag_b, halo_b = ds.max(aux["fetch_bytes"], aux["allgather_bytes"], aux["halo_bytes"])
        t_f = out["stages_ms_max_over_ranks"].get("fetch", 0.0)
        t_a = out["stages_ms_max_over_ranks"].get("pool+allgather", 0.0)
        out["exchange"] = {"fetch_bytes_received_per_gpu": fetch_b, "allgather_bytes_received_per_gpu": ag_b,
                           "halo_bytes_received_per_gpu": halo_b,
                           "fetch_gbs": fetch_b / (t_f / 1e3) / 1e9 if t_f else None,
                           "remote_tiles_of_all": aux["remote_tiles"] / float(B * hk * (T // S) * (world - 1) / world),
                           "fetch_mode": aux["fetch_mode"], "wanted_fraction_of_group": aux["wanted_fraction"],
                           "collectives": "all_gather (pooled keys), all_to_all (request bitmaps, K/V tiles), "
                                          "send/recv (halo)",
                           "allgather_ms": t_a}
        require_clean_status(f"the staged run of {name}")
    del q, k, v
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--only", action="store_true", help="the named workload alone, no secondary entries")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    ds = Dist()
    decode = args.workload.startswith("c4")
    if args.workload.startswith("c5"):
        line = run_context_parallel(args, args.workload, ds, args.steps, args.warmup)
    elif args.workload.startswith("c4_paged"):
        line = run_decode_paged(args, args.workload, ds, args.steps, args.warmup)
    elif decode:
        line = run_decode(args, args.workload, ds, args.steps, args.warmup)
    else:
        line = run_train(args, args.workload, ds, args.steps, args.warmup)
    secondary = {}
    if not args.only and args.workload == "c3":
        def attempt(name, fn):
            # a secondary workload that fails must not take the headline record with it; the failure is reported
            try:
                secondary[name] = fn()
            except Exception as e:  # noqa: BLE001
                secondary[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()
        attempt("c2", lambda: run_train(args, "c2", ds, max(args.steps, 10), 3, with_e2e=True))
        attempt("c4", lambda: run_decode(args, "c4", ds, max(2 * args.steps, 20), 5))
        attempt("c4_paged", lambda: run_decode_paged(args, "c4_paged", ds, max(2 * args.steps, 20), 5))
        attempt("c4_paged_ragged", lambda: run_decode_paged(args, "c4_paged_ragged", ds, max(2 * args.steps, 20), 5))
        attempt("c5", lambda: run_context_parallel(args, "c5", ds, 2, 1))
        if ds.world == 1:
            # the reference arm's configuration on the GPU (fp32 kernels), for a like-for-like CPU/GPU ratio
            attempt("c1", lambda: run_train(args, "c1", ds, 10, 3, with_e2e=False, with_kernels=False))
    if ds.rank == 0:
        line["cpu_baseline"] = None
        if ds.world == 1 and not args.no_cpu_baseline and not decode and not args.workload.startswith("c5"):
            tps, cores, dt = cpu_chain_tokens_per_s(1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"{CPU_SAMPLE_TEXT}, one pass ({dt:.1f} s)"}
        if secondary:
            line["secondary"] = secondary
        print(json.dumps(line))
    ds.close()


if __name__ == "__main__":
    main()
